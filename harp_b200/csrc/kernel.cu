// Kernel objects of the C ABI: create (classify + select), launch, release.
//
// eb200_kernel_create stands where the reference's backends render source and
// run a compiler (crates/backend-c/src/lib.rs:91-110 -> Pipeline::compile_ast,
// src/backend/pipeline.rs:135-216); eb200_kernel_launch stands where they call
// the loaded symbol (crates/backend-c/src/kernel.rs:114-168) or launch the PTX
// (crates/backend-cuda/src/kernel.rs:148-233).  Launches are asynchronous on the
// device stream; the reference synchronises after every launch.
#include <string.h>

#define EB_CHAIN_TABLE
#include "expr.cuh"

namespace eb200 {

int chain_count() { return EB_CHAIN_COUNT; }
const char* chain_name(int chain) { return chain >= 0 && chain < EB_CHAIN_COUNT ? chain_table[chain].name : "interpreter"; }

int find_chain(const KInsn* prog, int n_insns) {
    for (int c = 0; c < EB_CHAIN_COUNT; ++c) {
        const ChainEntry& e = chain_table[c];
        if (e.n != n_insns) continue;
        bool same = true;
        for (int i = 0; i < n_insns && same; ++i) {
            // operator, operand number, and for constants the slot (equal constants share one)
            if (e.prog[i].op != prog[i].op || e.prog[i].arg != prog[i].arg) same = false;
        }
        if (same) return c;
    }
    return -1;
}

static int dtype_bytes(int dt) { return dt == EB200_BOOL ? 1 : dt == EB200_I64 ? 8 : (dt == EB200_F16 || dt == EB200_BF16) ? 2 : 4; }

}  // namespace eb200

using namespace eb200;

extern "C" {

int eb200_kernel_create(eb200_device* dev, const eb200_kernel_desc* desc, eb200_kernel** out) {
    EB_REQUIRE(dev && desc && out, EB200_ERR_INVALID, "null argument");
    auto k = new eb200_kernel();
    k->dev = dev;
    int st = build_plan(desc, dev->prop.multiProcessorCount, &k->plan);
    if (st) { delete k; return st; }
    if (k->plan.scratch_bytes > 0) {
        cudaSetDevice(dev->index);
        st = storage_alloc(dev, (size_t)k->plan.scratch_bytes, k->plan.scratch_zero, &k->scratch);
        if (st) { delete k; return st; }
    }
    *out = k;
    return EB200_OK;
}

static void fill_info(const Plan& plan, eb200_kernel_info* info) {
    memset(info, 0, sizeof(*info));
    strncpy(info->impl, plan.name, sizeof(info->impl) - 1);
    info->launches = plan.launches;
    info->specialised = plan.chain >= 0 || plan.impl == IMPL_TRANSPOSE || plan.impl == IMPL_SCATTER || plan.impl == IMPL_FOLD_GATHER ||
                        plan.impl == IMPL_SGD || plan.impl == IMPL_SGD_MOMENTUM || plan.impl == IMPL_ADAM || plan.impl == IMPL_SOFTMAX_XENT || plan.impl == IMPL_MAXPOOL || plan.impl == IMPL_GEMM_SIMT || plan.impl == IMPL_GEMM_TC || plan.impl == IMPL_CONV2D || plan.impl == IMPL_GEMM_TALL || plan.impl == IMPL_CONV2D_WGRAD || plan.impl == IMPL_CONV2D_DIRECT || plan.impl == IMPL_CONV2D_DIRECT_WGRAD;
    info->scratch_bytes = plan.scratch_bytes;
    info->algo_bytes = plan.algo_bytes;
    info->algo_flops = plan.algo_flops;
}

int eb200_kernel_get_info(eb200_kernel* k, eb200_kernel_info* info) {
    EB_REQUIRE(k && info, EB200_ERR_INVALID, "null argument");
    fill_info(k->plan, info);
    return EB200_OK;
}

int eb200_kernel_query(const eb200_kernel_desc* desc, int sm_count, eb200_kernel_info* info) {
    EB_REQUIRE(desc && info, EB200_ERR_INVALID, "null argument");
    Plan plan;
    int st = build_plan(desc, sm_count > 0 ? sm_count : 148, &plan);
    if (st) return st;
    fill_info(plan, info);
    return EB200_OK;
}

int eb200_kernel_launch(eb200_kernel* k, eb200_buffer* const* inputs, int n_inputs,
                        eb200_buffer* const* outputs, int n_outputs) {
    EB_REQUIRE(k && (inputs || !n_inputs) && outputs, EB200_ERR_INVALID, "null argument");
    const Plan& plan = k->plan;
    EB_REQUIRE(n_inputs == plan.n_inputs, EB200_ERR_INVALID, "kernel takes %d inputs, got %d", plan.n_inputs, n_inputs);
    EB_REQUIRE(n_outputs == 1, EB200_ERR_INVALID, "kernel writes 1 output, got %d", n_outputs);
    Device* dev = k->dev;
    for (int i = 0; i < n_inputs; ++i) {
        EB_REQUIRE(inputs[i] && inputs[i]->dev == dev, EB200_ERR_INVALID, "input %d is null or lives on another device", i);
        size_t need = (size_t)plan.in_numel[i] * dtype_bytes(plan.in_dtype[i]);
        EB_REQUIRE(inputs[i]->bytes >= need, EB200_ERR_BOUNDS, "input %d holds %zu bytes, kernel addresses %zu", i, inputs[i]->bytes, need);
    }
    eb200_buffer* ob = outputs[0];
    EB_REQUIRE(ob && ob->dev == dev, EB200_ERR_INVALID, "output is null or lives on another device");
    {
        size_t need = (size_t)plan.out_numel * dtype_bytes(plan.out_dtype);
        EB_REQUIRE(ob->bytes >= need, EB200_ERR_BOUNDS, "output holds %zu bytes, kernel addresses %zu", ob->bytes, need);
    }
    EB_CHECK_CUDA(cudaSetDevice(dev->index));
    // the output may share storage with a clone: give it its own, keeping the
    // bytes the kernel does not overwrite
    int st = buffer_unshare(ob, true);
    if (st) return st;
    const bool optimizer = plan.impl == IMPL_SGD || plan.impl == IMPL_SGD_MOMENTUM || plan.impl == IMPL_ADAM;
    for (int i = 0; i < n_inputs; ++i)
        EB_REQUIRE(inputs[i]->storage->ptr != ob->storage->ptr || (optimizer && i == 0), EB200_ERR_INVALID,
                   "input %d aliases the output", i);
    // optimizer state (velocity, moments, step counter) is updated in place: give it its own storage first
    if (plan.impl == IMPL_SGD_MOMENTUM || plan.impl == IMPL_ADAM)
        for (int i = 2; i < n_inputs; ++i)
            if ((st = buffer_unshare(inputs[i], true))) return st;

    KParams p = plan.p;
    for (int c = 0; c < p.n_in; ++c) p.in[c].ptr = reinterpret_cast<char*>(inputs[plan.perm[c]]->storage->ptr);
    for (int j = 0; j < p.n_consts; ++j)
        p.cptr[j] = plan.dyn_input[j] >= 0
                        ? reinterpret_cast<const float*>(inputs[plan.dyn_input[j]]->storage->ptr) + plan.dyn_offset[j]
                        : nullptr;
    p.out.ptr = reinterpret_cast<char*>(ob->storage->ptr);
    p.error_flag = dev->error_flag_dev;
    void* scratch = k->scratch ? k->scratch->ptr : nullptr;
    switch (plan.impl) {
        case IMPL_EW: return launch_ew(dev, plan, p);
        case IMPL_REDUCE_INNER:
        case IMPL_REDUCE_OUTER: {
            if (!k->comm) return launch_reduce(dev, plan, p, scratch);
            // sharded reduce: this rank's result is combined with the peers' as part of the launch
            float* out = reinterpret_cast<float*>(p.out.ptr) + p.out.offset;
            if (p.splits > 1 && comm_can_fuse(k->comm, p.kept)) {
                if ((st = launch_reduce(dev, plan, p, scratch, false))) return st;
                return comm_reduce_finish_allreduce(k->comm, reinterpret_cast<const float*>(scratch), p.splits, p.kept, p.rop, out);
            }
            if ((st = launch_reduce(dev, plan, p, scratch))) return st;
            return comm_allreduce_buffer(k->comm, out, p.kept, p.rop);
        }
        case IMPL_TRANSPOSE: return launch_transpose(dev, plan, p.in[0].ptr, p.out.ptr);
        case IMPL_SCATTER: return launch_scatter(dev, plan, p);
        case IMPL_FOLD_GATHER: return launch_fold_gather(dev, plan, p);
        case IMPL_SGD:
            return launch_sgd(dev, plan, reinterpret_cast<const float*>(p.in[0].ptr) + p.in[0].offset,
                              reinterpret_cast<const float*>(p.in[1].ptr) + p.in[1].offset,
                              reinterpret_cast<float*>(p.out.ptr) + p.out.offset, p.total);
        case IMPL_SGD_MOMENTUM:
            return launch_sgd_momentum(dev, plan, reinterpret_cast<const float*>(p.in[0].ptr) + p.in[0].offset,
                                       reinterpret_cast<const float*>(p.in[1].ptr) + p.in[1].offset,
                                       reinterpret_cast<float*>(p.in[2].ptr) + p.in[2].offset,
                                       reinterpret_cast<float*>(p.out.ptr) + p.out.offset, p.total);
        case IMPL_ADAM:
            return launch_adam(dev, plan, reinterpret_cast<const float*>(p.in[0].ptr) + p.in[0].offset,
                               reinterpret_cast<const float*>(p.in[1].ptr) + p.in[1].offset,
                               reinterpret_cast<float*>(p.in[2].ptr) + p.in[2].offset,
                               reinterpret_cast<float*>(p.in[3].ptr) + p.in[3].offset,
                               reinterpret_cast<int*>(p.in[4].ptr) + p.in[4].offset,
                               reinterpret_cast<float*>(p.out.ptr) + p.out.offset, p.total, scratch);
        case IMPL_SCAN: return launch_scan(dev, plan, p, scratch);
        case IMPL_SIBLINGS:
            return launch_siblings(dev, plan, p, reinterpret_cast<const float*>(p.in[0].ptr) + p.in[0].offset,
                                   reinterpret_cast<float*>(p.out.ptr) + p.out.offset, scratch);
        case IMPL_MAXPOOL:
            return launch_maxpool(dev, plan, reinterpret_cast<const float*>(p.in[0].ptr) + p.in[0].offset,
                                  p.n_in > 1 ? reinterpret_cast<const float*>(p.in[1].ptr) + p.in[1].offset : nullptr,
                                  p.n_in > 2 ? reinterpret_cast<const float*>(p.in[2].ptr) + p.in[2].offset : nullptr,
                                  reinterpret_cast<float*>(p.out.ptr) + p.out.offset);
        case IMPL_SOFTMAX_XENT:
            return launch_softmax_xent(dev, plan, reinterpret_cast<const float*>(p.in[0].ptr) + p.in[0].offset,
                                       reinterpret_cast<const float*>(p.in[1].ptr) + p.in[1].offset,
                                       reinterpret_cast<float*>(p.out.ptr) + p.out.offset, scratch);
        case IMPL_GEMM_SIMT:
            return launch_gemm_simt(dev, plan, reinterpret_cast<const float*>(p.in[plan.gemm.a_input].ptr),
                                    reinterpret_cast<const float*>(p.in[plan.gemm.b_input].ptr),
                                    reinterpret_cast<float*>(p.out.ptr), scratch);
        case IMPL_GEMM_TC:
            return launch_gemm_tc(dev, plan, reinterpret_cast<const float*>(p.in[plan.gemm.a_input].ptr),
                                  reinterpret_cast<const float*>(p.in[plan.gemm.b_input].ptr),
                                  reinterpret_cast<float*>(p.out.ptr), scratch);
        case IMPL_CONV2D_DIRECT:
            return launch_conv2d_direct(dev, plan, reinterpret_cast<const float*>(p.in[0].ptr) + p.in[0].offset,
                                        reinterpret_cast<const float*>(p.in[1].ptr) + p.in[1].offset,
                                        plan.n_inputs == 3 ? reinterpret_cast<const float*>(p.in[2].ptr) + p.in[2].offset : nullptr,
                                        reinterpret_cast<float*>(p.out.ptr) + p.out.offset);
        case IMPL_CONV2D_DIRECT_WGRAD:
            return launch_conv2d_direct_wgrad(dev, plan, reinterpret_cast<const float*>(p.in[0].ptr) + p.in[0].offset,
                                              reinterpret_cast<const float*>(p.in[1].ptr) + p.in[1].offset,
                                              reinterpret_cast<float*>(p.out.ptr) + p.out.offset, scratch);
        case IMPL_CONV2D_WGRAD:
            return launch_conv2d_wgrad(dev, plan, reinterpret_cast<const float*>(p.in[0].ptr) + p.in[0].offset,
                                       reinterpret_cast<const float*>(p.in[1].ptr) + p.in[1].offset,
                                       reinterpret_cast<float*>(p.out.ptr) + p.out.offset, scratch);
        case IMPL_GEMM_TALL:
            return launch_gemm_tall(dev, plan, reinterpret_cast<const float*>(p.in[plan.gemm.a_input].ptr),
                                    reinterpret_cast<const float*>(p.in[plan.gemm.b_input].ptr),
                                    reinterpret_cast<float*>(p.out.ptr), scratch);
        case IMPL_CONV2D:
            return launch_conv2d(dev, plan, reinterpret_cast<const float*>(p.in[0].ptr) + p.in[0].offset,
                                 reinterpret_cast<const float*>(p.in[1].ptr) + p.in[1].offset,
                                 plan.n_inputs == 3 ? reinterpret_cast<const float*>(p.in[2].ptr) + p.in[2].offset : nullptr,
                                 reinterpret_cast<float*>(p.out.ptr) + p.out.offset, scratch);
        default: return set_error(EB200_ERR_UNSUPPORTED, "kernel implementation %d is not built", (int)plan.impl);
    }
}

int eb200_kernel_set_allreduce(eb200_kernel* k, eb200_comm* comm) {
    EB_REQUIRE(k, EB200_ERR_INVALID, "kernel is null");
    if (!comm) { k->comm = nullptr; return EB200_OK; }
    const Plan& plan = k->plan;
    EB_REQUIRE(plan.impl == IMPL_REDUCE_INNER || plan.impl == IMPL_REDUCE_OUTER, EB200_ERR_UNSUPPORTED,
               "only reduce kernels take an attached all-reduce (%s)", plan.name);
    const KParams& p = plan.p;
    EB_REQUIRE(p.out.dtype == EB200_F32, EB200_ERR_UNSUPPORTED, "all-reduce of a non-f32 output");
    // the kept elements must sit at out.offset + k: contiguous strides over the dims that are not reduced
    long long acc = 1;
    for (int d = p.ndim - 1; d >= 0; --d) {
        if (d == p.raxis) continue;
        EB_REQUIRE(p.shape[d] == 1 || p.out.strides[d] == acc, EB200_ERR_UNSUPPORTED, "the reduce output is not a contiguous range");
        acc *= p.shape[d];
    }
    k->comm = comm;
    return EB200_OK;
}

int eb200_kernel_release(eb200_kernel* k) {
    if (!k) return EB200_OK;
    if (k->refs.fetch_sub(1) == 1) {
        cudaSetDevice(k->dev->index);
        delete k;
    }
    return EB200_OK;
}

}  // extern "C"
