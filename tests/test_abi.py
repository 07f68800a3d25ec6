"""The C-ABI library loads and exports every symbol include/eb200.h declares;
struct layouts agree between the header, the library and the ctypes mirror.
No compute calls: runs without a GPU."""
import ctypes as C
import os
import re

from harp_b200 import capi
from harp_b200 import desc as D

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "eb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(eb200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    lib = capi.load()
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/eb200.h but not exported"


def test_binding_covers_every_declared_symbol():
    bound = set(capi.SIGNATURES) | {"eb200_abi_version", "eb200_last_error"}
    assert set(declared_symbols()) <= bound


def test_abi_version_and_struct_sizes():
    lib = capi.load()
    assert lib.eb200_abi_version() == 2
    a, b, c, d = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t()
    capi.call("eb200_abi_sizes", C.byref(a), C.byref(b), C.byref(c), C.byref(d))
    assert a.value == C.sizeof(D.CKernelDesc)
    assert b.value == C.sizeof(D.COperand)
    assert c.value == C.sizeof(D.CDeviceProps)
    assert d.value == C.sizeof(D.CKernelInfo)


def test_header_constants_match_python():
    text = open(os.path.join(ROOT, "include", "eb200.h")).read()
    for name, val in [("EB200_MAX_DIMS", D.MAX_DIMS), ("EB200_MAX_INPUTS", D.MAX_INPUTS),
                      ("EB200_MAX_BOUNDS", D.MAX_BOUNDS), ("EB200_MAX_INSNS", D.MAX_INSNS)]:
        m = re.search(rf"#define {name} (\d+)", text)
        assert m and int(m.group(1)) == val
    for name, val in [("EB200_OP_FMA", D.OP_FMA), ("EB200_OP_SELECT", D.OP_SELECT), ("EB200_K_SGD", D.K_SGD),
                      ("EB200_R_PROD", D.R_PROD), ("EB200_OP_EXP2", D.OP_EXP2)]:
        m = re.search(rf"{name} = (\d+)", text)
        assert m and int(m.group(1)) == val, name


def test_no_device_is_an_error_not_a_fallback():
    """Without a GPU the library reports NO_DEVICE; nothing computes on the CPU."""
    n = C.c_int(-1)
    st = capi.load().eb200_device_count(C.byref(n))
    if st == capi.OK and n.value > 0:
        return  # running on a GPU box
    h = C.c_void_p()
    st = capi.load().eb200_device_open(0, C.byref(h))
    assert st == capi.ERR_NO_DEVICE
    assert capi.load().eb200_last_error()
