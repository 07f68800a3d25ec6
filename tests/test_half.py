"""f16 / bf16 storage (EB200_F16, EB200_BF16): elements widen to f32 when loaded, arithmetic and
accumulators are f32, stores round to nearest even.  CPU part: the oracle's `_Float16` / `__bf16`
kernels (the types the reference renders, crates/backend-c/src/renderer.rs:129-130) against numpy,
and the planner's choice of the 64-bit path.  The GPU runs are in test_gpu_half.py."""
import ctypes as C

import numpy as np

from harp_b200 import capi
from harp_b200 import desc as D
from harp_b200.desc import Ast
from oracle import c_emit as O

w = Ast.w


def half_inputs(shape, dtype, seed):
    x = np.random.default_rng(seed).standard_normal(shape).astype(np.float32)
    if dtype == D.F16:
        return x.astype(np.float16)
    if dtype == D.BF16:
        return D.bf16_bits(x)
    return x


def as_f32(a, dtype):
    return D.bf16_value(a) if dtype == D.BF16 else np.asarray(a, np.float32)


def ulp(dtype):
    return {D.F16: 2.0 ** -10, D.BF16: 2.0 ** -7, D.F32: 2.0 ** -23}[dtype]


def test_bf16_helpers_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 1e-40], np.float32)   # 1 + 2^-8 is a tie: rounds to even (1.0)
    b = D.bf16_bits(x)
    assert b[0] == 0x3F80 and b[1] == 0x3F80 and b[2] == 0x3F82 and b[3] == 0xC020
    assert (D.bf16_value(D.bf16_bits(D.bf16_value(b))) == D.bf16_value(b)).all()


def test_oracle_16_bit_kernels_match_numpy():
    for dt in (D.F16, D.BF16):
        a, b = half_inputs((64, 48), dt, 1), half_inputs((64, 48), dt, 2)
        k = D.KernelDesc(D.K_ELEMENTWISE, [64, 48], [D.contiguous([64, 48], dt)] * 2, D.contiguous([64, 48], dt), w(0) + w(1))
        got = as_f32(O.run(k, [a, b]), dt).reshape(64, 48)
        exact = as_f32(a, dt).astype(np.float64) + as_f32(b, dt)
        assert (np.abs(got - exact) <= ulp(dt) * np.abs(exact) + 1e-30).all()
        # f32 accumulator over 16-bit elements (the reference's `float acc`)
        k = D.reduce([64, 48], [D.contiguous([64, 48], dt)], w(0), D.R_SUM, 1)
        got = O.run(k, [a])
        np.testing.assert_allclose(got, as_f32(a, dt).astype(np.float64).sum(1), rtol=1e-5, atol=1e-5)


def test_planner_moves_16_bit_operands_four_at_a_time():
    def query(k):
        info = D.CKernelInfo()
        cd = k.to_c()
        capi.call("eb200_kernel_query", C.byref(cd), 148, C.byref(info))
        return info
    k = D.KernelDesc(D.K_ELEMENTWISE, [512, 1024], [D.contiguous([512, 1024], D.BF16), D.contiguous([512, 1024], D.F32)],
                     D.contiguous([512, 1024], D.F16), w(0) * w(1))
    i = query(k)
    assert i.impl.decode() == "ew_chain_v4" and i.algo_bytes == 512 * 1024 * (2 + 4 + 2)
    k = D.KernelDesc(D.K_ELEMENTWISE, [511, 1023], [D.contiguous([511, 1023], D.F16)], D.contiguous([511, 1023], D.F16), w(0) * 2.0)
    assert query(k).impl.decode() == "ew_chain_v1"
    k = D.reduce([300, 1000], [D.contiguous([300, 1000], D.BF16)], w(0), D.R_SUM, 1)
    assert query(k).impl.decode().startswith("reduce_inner")


def half_matmul_desc(m, n, k, dt, out_dt=D.F32, batch=1):
    """C[b][m][n] = sum_k A[b][m][k] * B[b][n][k] with 16-bit A and B, both contiguous along k (x @ W^T)."""
    if batch > 1:
        shape = [batch, m, n, k]
        a = D.Operand([m * k, k, 0, 1], 0, dt, batch * m * k)
        b = D.Operand([n * k, 0, k, 1], 0, dt, batch * n * k)
        out = D.Operand([m * n, n, 1, 0], 0, out_dt, batch * m * n)
        return D.reduce(shape, [a, b], w(0) * w(1), D.R_SUM, 3, out=out)
    a = D.Operand([k, 0, 1], 0, dt, m * k)
    b = D.Operand([0, k, 1], 0, dt, n * k)
    return D.reduce([m, n, k], [a, b], w(0) * w(1), D.R_SUM, 2, out=D.Operand([n, 1, 0], 0, out_dt, m * n))


def test_planner_sends_16_bit_contractions_to_the_tensor_cores():
    def query(k):
        info = D.CKernelInfo()
        cd = k.to_c()
        capi.call("eb200_kernel_query", C.byref(cd), 148, C.byref(info))
        return info
    i = query(half_matmul_desc(1024, 512, 4096, D.BF16))
    assert i.impl.decode() == "gemm_tcgen05_bf16_kk" and i.launches == 1 and i.scratch_bytes == 0
    assert i.algo_flops == 2 * 1024 * 512 * 4096
    assert query(half_matmul_desc(300, 200, 72, D.F16, D.F16, batch=3)).impl.decode() == "gemm_tcgen05_f16_kk"
    # rows that are not 16-byte aligned (k = 100 elements of 2 bytes is fine, k = 99 is not) stay a plain reduce
    assert query(half_matmul_desc(256, 256, 99, D.F16)).impl.decode().startswith("reduce_")
    # B contiguous along n (the matmul_demo form) is not staged for 16-bit operands: plain reduce
    a = D.Operand([64, 0, 1], 0, D.F16, 128 * 64)
    b = D.Operand([0, 1, 256], 0, D.F16, 64 * 256)
    k = D.reduce([128, 256, 64], [a, b], w(0) * w(1), D.R_SUM, 2, out=D.Operand([256, 1, 0], 0, D.F32, 128 * 256))
    assert query(k).impl.decode().startswith("reduce_")
    # mixed operand types are not a GEMM
    k = half_matmul_desc(256, 256, 128, D.F16)
    k.inputs[1].dtype = D.BF16
    assert query(k).impl.decode().startswith("reduce_")
