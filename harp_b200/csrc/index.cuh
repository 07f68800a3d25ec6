// Index arithmetic shared by the generic kernels: linear work index ->
// multi-index over the collapsed iteration dims -> operand element address
// (the role of src/lowerer/index_gen.rs:45-63 in the reference).
//
// ND > 0 is a compile-time rank with 32-bit division (the launcher only picks
// it when the iteration space has fewer than 2^31 elements); ND == 0 is the
// any-rank 64-bit form, unrolled over the maximum rank with uniform predicates
// so the multi-index stays in registers.
#pragma once

#include "common.h"

namespace eb200 {

// Multi-index of linear element `e`; dim `skip` (if >= 0) is left out of the
// decomposition and gets index 0.
template <int ND = 0>
__device__ __forceinline__ void decompose(const KParams& p, long long e, long long* idx, int skip = -1) {
    if (ND > 0) {
        unsigned r = (unsigned)e;
#pragma unroll
        for (int d = ND - 1; d >= 0; --d) {
            if (d == skip) { idx[d] = 0; continue; }
            if (d == 0 && skip != 0) { idx[0] = r; break; }
            const unsigned s = (unsigned)p.shape[d];
            const unsigned q = (unsigned)(((unsigned long long)r * p.dmul[d]) >> p.dshr[d]);     // r / s, exact for r < 2^31
            idx[d] = r - q * s;
            r = q;
        }
    } else if (p.total < (1LL << 31)) {
        unsigned r = (unsigned)e;
#pragma unroll
        for (int d = KMAX_DIMS - 1; d >= 0; --d) {
            if (d >= p.ndim || d == skip) { idx[d] = 0; continue; }
            const unsigned s = (unsigned)p.shape[d];
            const unsigned q = (unsigned)(((unsigned long long)r * p.dmul[d]) >> p.dshr[d]);
            idx[d] = r - q * s;
            r = q;
        }
    } else {
        long long r = e;
#pragma unroll
        for (int d = KMAX_DIMS - 1; d >= 0; --d) {
            if (d >= p.ndim || d == skip) { idx[d] = 0; continue; }
            const long long s = p.shape[d];
            const long long q = r / s;
            idx[d] = r - q * s;
            r = q;
        }
    }
}

template <int ND = 0>
__device__ __forceinline__ long long operand_index(const KParams& p, const KOperand& o, const long long* idx) {
    long long a = o.offset;
    if (ND > 0) {
#pragma unroll
        for (int d = 0; d < ND; ++d) a += o.strides[d] * idx[d];
    } else {
#pragma unroll
        for (int d = 0; d < KMAX_DIMS; ++d)
            if (d < p.ndim) a += o.strides[d] * idx[d];
    }
    return a;
}

}  // namespace eb200
