// ew_chain: fused elementwise chains (kernel class E_, src/lowerer/lower.rs:504-522)
// and strided gathers (class C_, lower.rs:448-501) that are not transposes.
//
// The reference renders a scalar nested loop per arithmetic node.  Here one
// launch evaluates a whole composed chain: each thread owns 4 consecutive
// elements along the innermost collapsed dim and moves them with 128-bit
// loads/stores; broadcast operands (stride 0) are read once per vector.
// HBM-bound: algorithmic bytes = 4 B x (elements read + elements written).
#include "expr.cuh"
#include "index.cuh"

namespace eb200 {

template <class F>
__device__ __forceinline__ void load_vec4(const KParams& p, long long e, float (*in)[4]) {
    long long idx[KMAX_DIMS];
    decompose(p, e, idx);
    const int inner = p.ndim - 1;
    const int n = F::nin(p);
#pragma unroll
    for (int i = 0; i < (F::kCompiled ? n : KMAX_IN); ++i) {
        if (i >= n) break;
        const KOperand& o = p.in[i];
        long long a = operand_index(p, o, idx);
        const float* src = reinterpret_cast<const float*>(o.ptr) + a;
        if (o.strides[inner] == 1) {
            float4 t = __ldg(reinterpret_cast<const float4*>(src));
            in[i][0] = t.x; in[i][1] = t.y; in[i][2] = t.z; in[i][3] = t.w;
        } else {
            float t = __ldg(src);
            in[i][0] = t; in[i][1] = t; in[i][2] = t; in[i][3] = t;
        }
    }
}

__device__ __forceinline__ void store_vec4(const KParams& p, long long e, const float* v) {
    long long idx[KMAX_DIMS];
    decompose(p, e, idx);
    long long a = operand_index(p, p.out, idx);
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out.ptr) + a) = make_float4(v[0], v[1], v[2], v[3]);
}

template <class F>
__global__ void __launch_bounds__(256) ew_kernel(const __grid_constant__ KParams p) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (p.vec == 4) {
        const long long nvec = p.total >> 2;
        for (long long v0 = tid; v0 < nvec; v0 += 2 * stride) {
            const long long v1 = v0 + stride;
            const bool has1 = v1 < nvec;
            float in0[KMAX_IN][4], in1[KMAX_IN][4];
            float r0[4], r1[4];
            load_vec4<F>(p, v0 << 2, in0);
            if (has1) load_vec4<F>(p, v1 << 2, in1);
            F::template eval<4>(p, in0, r0);
            store_vec4(p, v0 << 2, r0);
            if (has1) {
                F::template eval<4>(p, in1, r1);
                store_vec4(p, v1 << 2, r1);
            }
        }
    } else {
        const int n = F::nin(p);
        for (long long e = tid; e < p.total; e += stride) {
            long long idx[KMAX_DIMS];
            decompose(p, e, idx);
            float in[KMAX_IN][1];
#pragma unroll
            for (int i = 0; i < (F::kCompiled ? n : KMAX_IN); ++i) {
                if (i >= n) break;
                const KOperand& o = p.in[i];
                if (o.n_bounds && !bounds_ok(p, o, idx)) in[i][0] = o.pad;
                else in[i][0] = load_elem(o, operand_index(p, o, idx));
            }
            float r[1];
            F::template eval<1>(p, in, r);
            store_elem(p.out, operand_index(p, p.out, idx), r[0]);
        }
    }
}

template <class F>
static int launch_one(Device* dev, const KParams& p) {
    long long work = p.vec == 4 ? (p.total >> 2) : p.total;
    if (work <= 0) return EB200_OK;
    long long per_block = 256LL * (p.vec == 4 ? 2 : 1);
    long long blocks = (work + per_block - 1) / per_block;
    long long cap = (long long)dev->prop.multiProcessorCount * 16;
    if (blocks > cap) blocks = cap;
    ew_kernel<F><<<(unsigned)blocks, 256, 0, dev->stream>>>(p);
    count_launch();
    EB_CHECK_CUDA(cudaGetLastError());
    return EB200_OK;
}

int launch_ew(Device* dev, const Plan& plan, const KParams& p) {
    switch (plan.chain) {
#define X(i) case i: return launch_one<Compiled<Chain##i>>(dev, p);
        EB_FOR_EACH_CHAIN(X)
#undef X
        default: return launch_one<Interp>(dev, p);
    }
}

}  // namespace eb200
