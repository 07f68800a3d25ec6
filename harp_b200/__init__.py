"""harp_b200: a B200-native execution backend for eclat (uthree/harp).

The product is ``libeb200.so`` (hand-written sm_100a kernels behind the C ABI of
``include/eb200.h``) plus a host-side mirror of the reference's backend plugin
surface (``harp_b200.backend``).  There is no CPU execution path: everything
that computes goes through the CUDA library and fails loudly when it is absent.
"""
__version__ = "0.1.0"
