"""tests/golden/kernels.json: {lowered-kernel descriptor <-> the C the reference's
C backend is expected to emit}.  On the CPU: the committed file is what the
generator produces today, every descriptor survives the JSON round trip, and the
planner serves every one of them.  On the GPU: every golden kernel runs through
the C ABI and is compared with its own C compiled by gcc."""
import ctypes as C
import importlib.util
import json
import os

import numpy as np
import pytest

from harp_b200 import capi
from harp_b200 import desc as D

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "kernels.json")


def _items():
    with open(GOLDEN) as f:
        return json.load(f)


def test_golden_file_is_current():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    built = json.loads(json.dumps(mod.build()))
    assert built == _items(), "tests/golden/kernels.json is stale: run python tests/golden/make_golden.py"


def test_descriptors_round_trip_and_are_served():
    from oracle import c_emit as O
    items = _items()
    assert len(items) >= 30
    classes = set()
    for it in items:
        d = D.KernelDesc.from_json(it["desc"])
        assert d.to_json() == it["desc"], it["name"]
        assert O.emit_kernel_c(d, "kernel") == it["c"], it["name"]
        info = D.CKernelInfo()
        cd = d.to_c()
        capi.call("eb200_kernel_query", C.byref(cd), 148, C.byref(info))
        classes.add(d.kclass)
    assert {D.K_ELEMENTWISE, D.K_REDUCE, D.K_COPY, D.K_SCATTER, D.K_SCAN} <= classes


def test_reference_vectors_through_the_golden_c():
    """The reference's own known-answer vectors (crates/backend-c/src/lib.rs:181-295) through the
    golden C text itself."""
    from oracle import c_emit as O
    by_name = {it["name"]: it for it in _items()}
    for name, a, b, want in (("add_1d", [1, 2, 3, 4], [5, 6, 7, 8], [6, 8, 10, 12]),
                             ("mul_1d", [1, 2, 3, 4], [2, 3, 4, 5], [2, 6, 12, 20])):
        lib = C.CDLL(O.compile_c(by_name[name]["c"]))
        x, y, out = (np.array(v, np.float32) for v in (a, b, [0] * 4))
        lib.kernel(x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p))
        assert out.tolist() == want


@pytest.mark.gpu
def test_golden_kernels_on_the_gpu(dev):
    from oracle import c_emit as O
    from util import run_gpu
    rng = np.random.default_rng(11)
    for it in _items():
        d = D.KernelDesc.from_json(it["desc"])
        ins = [rng.uniform(0.5, 1.5, int(o.numel)).astype(np.float32) for o in d.inputs]
        ins = [D.bf16_bits(a) if o.dtype == D.BF16 else a.astype(np.float16) if o.dtype == D.F16 else a for a, o in zip(ins, d.inputs)]
        got, kern = run_gpu(dev, d, ins)
        ref = O.run(d, ins)
        if d.kclass == D.K_COPY or d.reduce_op in (D.R_MAX, D.R_MIN):
            assert got.tobytes() == ref.tobytes(), it["name"]
        elif d.output.dtype in (D.F16, D.BF16):      # one unit in the last place of the stored type
            g = (D.bf16_value(got) if d.output.dtype == D.BF16 else got).astype(np.float64)
            r = (D.bf16_value(ref) if d.output.dtype == D.BF16 else ref).astype(np.float64)
            assert (np.abs(g - r) <= 2.0 ** (-7 if d.output.dtype == D.BF16 else -10) * np.abs(r)).all(), it["name"]
        else:
            assert np.allclose(got, ref, rtol=2e-5, atol=1e-6), (it["name"], kern.impl, float(np.abs(got - ref).max()))
