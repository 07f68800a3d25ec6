"""Program executor over the CPU oracle (test infrastructure only): the same
kernel lists the front end lowers for the GPU run through the emitted-C oracle,
so whole graphs -- forward, gradients, parameter update -- can be compared."""
import numpy as np

from . import c_emit as O


class _OracleKernel:
    def __init__(self, d, openmp):
        self.k = O.OracleKernel(d, openmp=openmp)

    def execute(self, ins, outs):
        self.k([b for b in ins], outs[0])


class OracleExecutor:
    def __init__(self, openmp=False):
        self.openmp = openmp

    def alloc(self, numel):
        return np.zeros(int(numel), np.float32)

    def alloc_counter(self):
        return np.zeros(1, np.int32)

    def free(self, buf):
        pass

    def upload(self, buf, data):
        buf[...] = np.asarray(data, np.float32).reshape(-1)

    def download(self, buf, numel):
        return buf.copy()

    def compile(self, d):
        return _OracleKernel(d, self.openmp)

    def synchronize(self):
        pass
