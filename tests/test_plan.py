"""Kernel-class dispatch (descriptor -> hand-written kernel) checked on the CPU
through eb200_kernel_query: classification, validation errors, collapsing."""
import ctypes as C

import pytest

from harp_b200 import capi
from harp_b200 import desc as D
from harp_b200 import workloads as W
from harp_b200.desc import Ast

w = Ast.w


def query(k: D.KernelDesc, sms: int = 148):
    info = D.CKernelInfo()
    cd = k.to_c()
    capi.call("eb200_kernel_query", C.byref(cd), sms, C.byref(info))
    return info


def test_cfg2_row_sum_is_vectorised_warp_per_row_and_compiled():
    i = query(W.cfg2_y())
    assert i.impl.decode() == "reduce_inner_t32_v4"
    assert i.specialised == 1 and i.launches == 1 and i.scratch_bytes == 0
    assert i.algo_bytes == 4 * 8192 * 8192 + 4 * 8192 + 8   # x once, y once, two scalars


def test_cfg2_col_max_splits_rows_into_scratch():
    i = query(W.cfg2_z())
    assert i.impl.decode() == "reduce_outer_v4_split"
    assert i.launches == 2 and i.scratch_bytes > 0 and i.scratch_bytes % (8192 * 4) == 0
    assert i.algo_bytes == 4 * 8192 * 8192 + 4 * 8192


def test_cfg2_permute_is_a_transpose():
    i = query(W.cfg2_t())
    assert i.impl.decode() == "transpose_copy"
    assert i.algo_bytes == 8 * 8192 * 8192


def test_contiguous_elementwise_collapses_to_one_vector_dim():
    k = D.elementwise([8, 16, 32], [D.contiguous([8, 16, 32])] * 2, w(0) + w(1))
    assert query(k).impl.decode() == "ew_chain_v4"
    k = D.elementwise([7, 3], [D.contiguous([7, 3])] * 2, w(0) + w(1))
    assert query(k).impl.decode() == "ew_chain_v1"   # 21 elements: not a multiple of 4


def test_unknown_expression_runs_on_the_interpreter():
    e = (w(0).sin() * w(1).sqrt() + w(0)).floor()
    k = D.elementwise([64], [D.contiguous([64])] * 2, e)
    i = query(k)
    assert i.impl.decode() == "ew_chain_v4" and i.specialised == 0


def test_matmul_spelled_as_broadcast_mul_sum_is_a_gemm():
    for k in (W.matmul_desc(512, 512, 512), W.linear_desc(64, 32, 16), W.matmul_desc(64, 32, 48, batch=4)):
        i = query(k)
        assert i.impl.decode().startswith("gemm"), i.impl
    i = query(W.matmul_desc(512, 512, 512))
    assert i.algo_flops == 2 * 512 ** 3
    # 512^3 is 85 flop per operand byte: hi / lo are split inside the kernel, scratch holds split-K partials only
    assert i.impl.decode().startswith("gemm_tcgen05_3xtf32_kn") and i.scratch_bytes < 4 * 4 * 512 * 512
    big = query(W.matmul_desc(8192, 8192, 8192))
    assert big.impl.decode() == "gemm_tcgen05_3xtf32_kn" and big.scratch_bytes >= 4 * 4 * 8192 * 8192 and big.launches == 3
    assert query(W.matmul_desc(512, 512, 512, mode=D.GEMM_TF32)).impl.decode().startswith("gemm_tcgen05_tf32_kn")
    assert query(W.matmul_desc(8192, 8192, 8192, mode=D.GEMM_TF32)).impl.decode() == "gemm_tcgen05_tf32_kn"
    assert query(W.linear_desc(4096, 256, 256)).impl.decode() == "gemm_tcgen05_3xtf32_kk"
    assert query(W.matmul_desc(64, 30, 64)).impl.decode() == "gemm_simt_f32"     # lda not 16-byte aligned
    k = W.matmul_desc(512, 512, 512); k.flags = 8
    assert query(k).impl.decode().startswith("gemm_simt_f32")


def test_weight_gradient_contractions_split_k():
    # dW[o,i] = sum_b dy[b,o] x[b,i]: A is M-major, K = batch is long, M x N is small
    a = D.Operand([256, 1, 0], 0, D.F32, 65536 * 256)
    b = D.Operand([256, 0, 1], 0, D.F32, 65536 * 256)
    k = D.reduce([65536, 256, 256], [a, b], w(0) * w(1), D.R_SUM, 0)
    i = query(k)
    assert i.impl.decode() == "gemm_tcgen05_3xtf32_mn_splitk" and i.launches == 2      # kernel (hi / lo split inside) + partial sum
    # conv1 weight gradient: ldb = 9 floats cannot be a TMA stride -> f32 kernels, still split:
    # the one-tile tall form for long reductions, the tiled one when asked (flag 16) or short
    a = D.Operand([32, 1, 0], 0, D.F32, 346112 * 32)
    b = D.Operand([9, 0, 1], 0, D.F32, 346112 * 9)
    k = D.reduce([346112, 32, 9], [a, b], w(0) * w(1), D.R_SUM, 0)
    i = query(k)
    assert i.impl.decode() == "gemm_tall_f32_splitk" and i.scratch_bytes > 0
    a = D.Operand([32, 1, 0], 0, D.F32, 8000 * 32)
    b = D.Operand([9, 0, 1], 0, D.F32, 8000 * 9)
    i = query(D.reduce([8000, 32, 9], [a, b], w(0) * w(1), D.R_SUM, 0))
    assert i.impl.decode() == "gemm_simt_f32_splitk" and i.scratch_bytes > 0


def test_small_rows_use_thread_or_warp_per_row():
    k = D.reduce([1000, 10], [D.contiguous([1000, 10])], w(0), D.R_MAX, 1)
    assert query(k).impl.decode() == "reduce_inner_t1_v1"
    k = D.reduce([1000, 1024], [D.contiguous([1000, 1024])], w(0), D.R_SUM, 1)
    assert query(k).impl.decode() == "reduce_inner_t32_v4"
    # many short rows: eight lanes per row (few such rows stay on a warp per row)
    k = D.reduce([65536, 256], [D.contiguous([65536, 256])], w(0), D.R_SUM, 1)
    assert query(k).impl.decode() == "reduce_inner_t8_v4"
    k = D.reduce([1000, 256], [D.contiguous([1000, 256])], w(0), D.R_SUM, 1)
    assert query(k).impl.decode() == "reduce_inner_t32_v4"


def test_long_single_row_is_split():
    n = 1 << 24
    k = D.reduce([1, n], [D.contiguous([1, n])], w(0), D.R_SUM, 1)
    i = query(k)
    assert i.impl.decode() == "reduce_inner_t256_v4_split" and i.launches == 2 and i.scratch_bytes > 0


def test_out_of_range_store_is_rejected_not_faulted():
    # a sliced/offset store view that would index past the allocation
    out = D.Operand([1], 8, D.F32, 16)
    k = D.elementwise([16], [D.contiguous([16])], w(0), out=out)
    with pytest.raises(capi.Eb200Error) as e:
        query(k)
    assert e.value.status == capi.ERR_BOUNDS


def test_out_of_range_load_is_rejected():
    src = D.Operand([2], 0, D.F32, 16)
    k = D.elementwise([16], [src], w(0))
    with pytest.raises(capi.Eb200Error) as e:
        query(k)
    assert e.value.status == capi.ERR_BOUNDS


def test_malformed_program_is_invalid():
    k = D.elementwise([16], [D.contiguous([16])], w(0) + w(1))   # loads input 1 of 1
    with pytest.raises(capi.Eb200Error) as e:
        query(k)
    assert e.value.status == capi.ERR_INVALID


def test_trivially_true_bounds_are_dropped():
    # conv2d always pads, even with padding 0 (crates/nn/src/functional/conv.rs:142):
    # the mask is kept by View::padded but can never fail
    op = D.Operand([1], 0, D.F32, 64, [D.Bound([1], 0, 0, 64)], 0.0)
    k = D.elementwise([64], [op], w(0) * D.Ast.const(2.0))
    assert query(k).impl.decode() == "ew_chain_v4"
    op = D.Operand([1], -1, D.F32, 64, [D.Bound([1], 0, 1, 65)], 0.0)
    k = D.elementwise([66], [op], w(0) * D.Ast.const(2.0))
    assert query(k).impl.decode() == "ew_chain_v1"


def test_broadcast_operand_keeps_vector_path():
    bias = D.Operand([0, 1], 0, D.F32, 32)
    k = D.elementwise([128, 32], [D.contiguous([128, 32]), bias], w(0) + w(1))
    assert query(k).impl.decode() == "ew_chain_v4"


def test_i64_is_unsupported_not_miscomputed():
    k = D.elementwise([16], [D.contiguous([16], D.I64)], w(0), out_dtype=D.I64)
    with pytest.raises(capi.Eb200Error) as e:
        query(k)
    assert e.value.status == capi.ERR_UNSUPPORTED


def test_conv2d_is_one_implicit_gemm_with_weight_scratch():
    i = query(D.conv2d(64, 32, 28, 28, 64, 3, 3, pad=1, relu=True))
    assert i.impl.decode() == "conv2d_igemm_3xtf32"
    assert i.launches == 2                                   # weight split/pad + the implicit GEMM
    assert i.scratch_bytes == 2 * 64 * 288 * 4               # hi and lo weights, K = 288 already a multiple of 32
    assert i.algo_flops == 2 * 64 * 28 * 28 * 64 * 288
    k = D.conv2d(8, 1, 28, 28, 32, 3, 3, pad=0, mode=D.GEMM_TF32)
    i = query(k)
    assert i.impl.decode() == "conv2d_direct_f32" and i.launches == 1 and i.scratch_bytes == 0     # K = 9: streaming f32 kernel
    k.flags |= D.FLAG_TENSOR_CORE
    i = query(k)
    assert i.impl.decode() == "conv2d_igemm_tf32" and i.scratch_bytes == 2 * 32 * 32 * 4     # K = 9 padded to 32


def test_conv2d_rejects_what_the_kernel_does_not_serve():
    with pytest.raises(capi.Eb200Error) as e:
        query(D.conv2d(1, 250, 8, 8, 16, 3, 3))              # K = 2250 > 2048 and the channels are not a multiple of 32
    assert e.value.status == capi.ERR_UNSUPPORTED
    assert query(D.conv2d(1, 256, 8, 8, 16, 3, 3)).impl.decode() == "conv2d_igemm_3xtf32"     # K = 2304, channel-blocked: no table
    with pytest.raises(capi.Eb200Error):
        query(D.conv2d(1, 1, 2, 2, 4, 3, 3))                 # window larger than the padded image
    k = D.conv2d(2, 3, 8, 8, 4, 3, 3)
    k.inputs[1].numel -= 1                                   # weight buffer one element short
    with pytest.raises(capi.Eb200Error) as e:
        query(k)
    assert e.value.status == capi.ERR_BOUNDS


def test_narrow_column_reduce_uses_row_lanes():
    k = D.reduce([2768896, 32], [D.contiguous([2768896, 32])], w(0), D.R_SUM, 0)     # conv1 bias gradient of config 4
    i = query(k)
    assert i.impl.decode() == "reduce_outer_narrow_v4_split" and i.launches == 2
    k.flags = 16
    assert query(k).impl.decode() == "reduce_outer_v4_split"
    assert query(W.cfg2_z()).impl.decode() == "reduce_outer_v4_split"            # wide outputs keep a thread per vector


def test_conv1_weight_gradient_is_the_tall_kernel():
    a = D.Operand([32, 1, 0], 0, D.F32, 2768896 * 32)
    b = D.Operand([9, 0, 1], 0, D.F32, 2768896 * 9)
    i = query(D.reduce([2768896, 32, 9], [a, b], w(0) * w(1), D.R_SUM, 0))
    assert i.impl.decode() == "gemm_tall_f32_splitk" and i.launches == 2
    assert i.scratch_bytes == 2 * 148 * 32 * 9 * 4


def test_conv2d_gradient_forms():
    i = query(D.conv2d(64, 64, 11, 11, 32, 3, 3, pad=2, bias=False, flip=True))
    assert i.impl.decode() == "conv2d_igemm_3xtf32_dgrad"
    i = query(D.conv2d_wgrad(4096, 32, 13, 13, 64, 3, 3))
    assert i.impl.decode() == "conv2d_igemm_3xtf32_wgrad" and i.launches == 2
    assert i.scratch_bytes == (148 // 3) * 288 * 64 * 4          # one partial per image stream, three row tiles of k
    with pytest.raises(capi.Eb200Error) as e:
        query(D.conv2d_wgrad(8, 64, 56, 56, 64, 3, 3, pad=1))   # image planes (802 KB) do not fit shared memory
    assert e.value.status == capi.ERR_UNSUPPORTED


def test_groups_of_four_when_an_operand_is_laid_out_like_the_output():
    # max-pool gradient: the input (laid out like the output) against broadcast pooled value and gradient
    full = [4096, 32, 13, 2, 13, 2]
    x6 = D.contiguous(full)
    bc = D.Operand([5408, 169, 13, 0, 1, 0], 0, D.F32, 4096 * 32 * 169)
    k = D.KernelDesc(D.K_ELEMENTWISE, full, [bc, x6, bc], D.contiguous(full), Ast.select(w(1).lt(w(2)), 0.0, w(0)))
    assert query(k).impl.decode() == "ew_chain_g4"
    # every operand strided (max-pool forward as four taps): the plain scalar kernel is faster
    taps = [D.Operand([5408 * 4, 676, 52, 2], off, D.F32, 4096 * 32 * 676) for off in (0, 1, 26, 27)]
    k = D.KernelDesc(D.K_ELEMENTWISE, [4096, 32, 13, 13], taps, D.contiguous([4096, 32, 13, 13]),
                     w(0).maximum(w(1)).maximum(w(2)).maximum(w(3)))
    assert query(k).impl.decode() == "ew_chain_v1"
    assert query(W.cfg2_t()).impl.decode() == "transpose_copy"


def _padded_conv_window_operand(offset_error=0):
    """x [2, 3, 6, 6] padded by 1 and unfolded 3x3: iteration [2, 3, 6, 6, 3, 3], the load
    sits at n*108 + c*36 + (oh+kh-1)*6 + (ow+kw-1) and is masked where the window leaves
    the image (View::padded then unfold, src/graph/shape/view.rs:980-1054,1162-1381)."""
    st = [108, 36, 6, 1, 6, 1]
    bounds = [D.Bound([0, 0, 1, 0, 1, 0], -1, 0, 6), D.Bound([0, 0, 0, 1, 0, 1], -1, 0, 6)]
    return D.Operand(st, -7 + offset_error, D.F32, 2 * 3 * 36, bounds)


def test_masked_operand_addresses_are_validated_at_create():
    shape = [2, 3, 6, 6, 3, 3]
    ok = D.KernelDesc(D.K_COPY, shape, [_padded_conv_window_operand()], D.contiguous(shape), None)
    assert query(ok).impl.decode().startswith("ew_chain")
    # the same view with a wrong offset would read past the end wherever the mask holds
    bad = D.KernelDesc(D.K_COPY, shape, [_padded_conv_window_operand(+40)], D.contiguous(shape), None)
    with pytest.raises(capi.Eb200Error) as e:
        query(bad)
    assert e.value.status == capi.ERR_BOUNDS
    bad = D.KernelDesc(D.K_COPY, shape, [_padded_conv_window_operand(-1)], D.contiguous(shape), None)
    with pytest.raises(capi.Eb200Error) as e:
        query(bad)
    assert e.value.status == capi.ERR_BOUNDS
    # a mask that never holds loads nothing: any addressing is acceptable
    never = D.Operand([1], 10 ** 9, D.F32, 4, [D.Bound([1], 100, 0, 4)])
    assert query(D.KernelDesc(D.K_COPY, [4], [never], D.contiguous([4]), None)).impl.decode().startswith("ew_chain")
    # strides that do not follow the bound's coefficients: validated by enumeration
    odd = D.Operand([3, 1], 0, D.F32, 12, [D.Bound([1, 1], 0, 0, 4)])
    assert query(D.KernelDesc(D.K_COPY, [4, 4], [odd], D.contiguous([4, 4]), None)).impl.decode().startswith("ew_chain")
    odd_bad = D.Operand([3, 1], 0, D.F32, 6, [D.Bound([1, 1], 0, 0, 4)])       # (3, 0) -> 9 is past 6
    with pytest.raises(capi.Eb200Error) as e:
        query(D.KernelDesc(D.K_COPY, [4, 4], [odd_bad], D.contiguous([4, 4]), None))
    assert e.value.status == capi.ERR_BOUNDS


def test_contraction_beyond_the_gemm_grids_stays_a_reduce():
    # 100 000 batches of 8x8x8: no GEMM kernel's grid.z holds the batch; the generic reduce serves it
    i = query(W.matmul_desc(8, 8, 8, batch=100000))
    assert i.impl.decode().startswith("reduce_"), i.impl
    assert query(W.matmul_desc(8, 8, 8, batch=60000)).impl.decode().startswith("gemm")
