// Index arithmetic shared by the generic kernels: linear work index ->
// multi-index over the collapsed iteration dims -> operand element address
// (the role of src/lowerer/index_gen.rs:45-63 in the reference).
// Loops are unrolled over the maximum rank with uniform predicates so the
// multi-index stays in registers.
#pragma once

#include "common.h"

namespace eb200 {

// Multi-index of linear element `e` over all dims; `skip` (if >= 0) is left
// out of the decomposition and gets index 0.
__device__ __forceinline__ void decompose(const KParams& p, long long e, long long* idx, int skip = -1) {
    if (p.total < (1LL << 31)) {
        unsigned r = (unsigned)e;
#pragma unroll
        for (int d = KMAX_DIMS - 1; d >= 0; --d) {
            if (d >= p.ndim || d == skip) { idx[d] = 0; continue; }
            unsigned s = (unsigned)p.shape[d];
            unsigned q = r / s;
            idx[d] = r - q * s;
            r = q;
        }
    } else {
        long long r = e;
#pragma unroll
        for (int d = KMAX_DIMS - 1; d >= 0; --d) {
            if (d >= p.ndim || d == skip) { idx[d] = 0; continue; }
            long long s = p.shape[d];
            long long q = r / s;
            idx[d] = r - q * s;
            r = q;
        }
    }
}

__device__ __forceinline__ long long operand_index(const KParams& p, const KOperand& o, const long long* idx) {
    long long a = o.offset;
#pragma unroll
    for (int d = 0; d < KMAX_DIMS; ++d)
        if (d < p.ndim) a += o.strides[d] * idx[d];
    return a;
}

}  // namespace eb200
