// Dispatch plans and the single-process communicator of the device runtime.
//
// A plan is the CUDA counterpart of the reference's compiled dispatch list: every op names an ahead-of-time kernel of this
// library (the analogue of a KernelSpec), where each of its buffers comes from (function input, function output, an
// offset of the plan's arena, an offset of its constant pool — BufferBinding / BufferSource,
// Sources/MetalHLOCore/Compiler/KernelTypes.swift:77-143) and its extents, scalars and launch knobs (DispatchConfig,
// :12-62). mhlo_cuda_plan_execute binds and enqueues the ops in order on one stream, as IntegratedExecutor.execute does
// with a command buffer (Runtime/IntegratedExecutor.swift:150-270), without per-call allocation or zero-filling.
//
// The communicator covers the one exchange of the hot path, an all-gather of equal shards over the GPUs of one process:
// every device pushes its shard into every peer's buffer with its own kernel over NVLink peer memory.
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"

namespace mhlo {
namespace {

struct Plan {
    std::vector<mhlo_cuda_plan_op> ops;
    void* arena = nullptr;
    void* constants = nullptr;
    int64_t arena_bytes = 0, constant_bytes = 0;
    int32_t n_inputs = 0, n_outputs = 0;
    int device = 0;
};

struct KernelInfo { const char* name; int32_t id; int32_t n_args; };
const KernelInfo kKernels[] = {
    {"fused_layer_norm", MHLO_CUDA_KERNEL_LAYER_NORM, 4},
    {"fused_rms_norm", MHLO_CUDA_KERNEL_RMS_NORM, 3},
    {"fused_softmax", MHLO_CUDA_KERNEL_SOFTMAX, 2},
    {"dot_general", MHLO_CUDA_KERNEL_GEMM, 4},
    {"fused_matmul_bias_activation", MHLO_CUDA_KERNEL_GEMM, 4},
    {"fused_scaled_dot_product_attention", MHLO_CUDA_KERNEL_ATTENTION, 5},
    {"fused_gelu", MHLO_CUDA_KERNEL_GELU, 2},
    {"fused_silu", MHLO_CUDA_KERNEL_SILU, 2},
};

int args_of(int32_t kernel) {
    for (const KernelInfo& k : kKernels)
        if (k.id == kernel) return k.n_args;
    return -1;
}

const void* resolve(const Plan& p, const mhlo_cuda_binding& b, const void* const* inputs, void* const* outputs) {
    switch (b.source) {
        case MHLO_CUDA_SRC_INPUT: return static_cast<const char*>(inputs[b.index]) + b.offset;
        case MHLO_CUDA_SRC_OUTPUT: return static_cast<const char*>(outputs[b.index]) + b.offset;
        case MHLO_CUDA_SRC_UNIFIED: return static_cast<const char*>(p.arena) + b.offset;
        case MHLO_CUDA_SRC_CONSTANT: return static_cast<const char*>(p.constants) + b.offset;
        default: return nullptr;
    }
}

int run_op(const Plan& p, const mhlo_cuda_plan_op& op, const void* const* inputs, void* const* outputs, mhlo_cuda_stream_t stream) {
    const void* a[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    for (int i = 0; i < 6; ++i) a[i] = resolve(p, op.args[i], inputs, outputs);
    auto out = [&](int i) { return const_cast<void*>(a[i]); };
    mhlo_cuda_row_tuning row{op.tuning[0], op.tuning[1], op.tuning[2]};
    const mhlo_cuda_row_tuning* rowp = (op.tuning[0] || op.tuning[1] || op.tuning[2]) ? &row : nullptr;
    switch (op.kernel) {
        case MHLO_CUDA_KERNEL_LAYER_NORM:
            return mhlo_cuda_layer_norm(op.dtype, a[0], a[1], a[2], out(3), op.dims[0], op.dims[1], op.scalars[0], rowp, stream);
        case MHLO_CUDA_KERNEL_RMS_NORM:
            return mhlo_cuda_rms_norm(op.dtype, a[0], a[1], out(2), op.dims[0], op.dims[1], op.scalars[0], rowp, stream);
        case MHLO_CUDA_KERNEL_SOFTMAX:
            return mhlo_cuda_softmax(op.dtype, a[0], out(1), op.dims[0], op.dims[1], op.dims[2], rowp, stream);
        case MHLO_CUDA_KERNEL_GEMM: {
            mhlo_cuda_gemm_tuning t{op.tuning[0], op.tuning[1], op.tuning[2], 0};
            const bool tuned = op.tuning[0] || op.tuning[1] || op.tuning[2];
            return mhlo_cuda_gemm_tuned(op.dtype, op.out_dtype, a[0], op.strides, a[1], op.strides + 4, out(3), op.dims[0], op.dims[1], op.dims[2],
                                        op.dims[3], op.dims[4], a[2], op.flags[0], tuned ? &t : nullptr, stream);
        }
        case MHLO_CUDA_KERNEL_ATTENTION: {
            mhlo_cuda_attention_tuning t{op.tuning[0], {0, 0, 0}};
            return mhlo_cuda_attention_tuned(op.dtype, a[0], op.strides, a[1], op.strides + 3, a[2], op.strides + 6, a[3], out(4), op.strides + 9,
                                             op.dims[0], op.dims[1], op.dims[2], op.dims[3], op.dims[4], op.scalars[0], op.flags[0],
                                             op.tuning[0] ? &t : nullptr, stream);
        }
        case MHLO_CUDA_KERNEL_GELU:
        case MHLO_CUDA_KERNEL_SILU: {
            mhlo_cuda_view in;
            std::memset(&in, 0, sizeof in);
            in.base = a[0]; in.dtype = op.dtype; in.rank = 1; in.shape[0] = op.dims[0]; in.stride[0] = 1;
            mhlo_cuda_ew_inst prog{op.kernel == MHLO_CUDA_KERNEL_GELU ? MHLO_EW_GELU_TANH : MHLO_EW_SILU, 0, 0, 0, 0.0};
            return mhlo_cuda_elementwise(&in, 1, &prog, 1, out(1), op.out_dtype ? op.out_dtype : op.dtype, op.dims, 1, stream);
        }
        default:
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "plan: unknown kernel %d", op.kernel);
    }
}

// ---- all-gather over peer memory ----
struct Comm {
    int n = 0;
    std::vector<cudaStream_t> streams;
};

// Device `rank` copies its shard (16-byte words [rank * words, (rank + 1) * words) of its own buffer) to the same place in
// every peer's buffer: plain 16-byte stores through peer addresses, all peers in one pass over the shard.
__global__ void all_gather_push_kernel(const uint4* __restrict__ own, uint4* const* __restrict__ peers, int n_peers, int64_t first, int64_t words) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < words; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const uint4 v = own[first + i];
        for (int d = 0; d < n_peers; ++d) peers[d][first + i] = v;
    }
}

}  // namespace
}  // namespace mhlo

using namespace mhlo;

extern "C" {

int mhlo_cuda_kernel_lookup(const char* fused_op_kind, int32_t dtype, int32_t* out_kernel) {
    if (!fused_op_kind || !out_kernel) return fail(MHLO_CUDA_INVALID_ARGUMENT, "kernel_lookup: null argument");
    *out_kernel = 0;
    if (mhlo_cuda_dtype_size(dtype) == 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "kernel_lookup: unknown dtype %d", dtype);
    for (const KernelInfo& k : kKernels) {
        if (std::strcmp(k.name, fused_op_kind) != 0) continue;
        if (dtype != MHLO_DT_F32 && dtype != MHLO_DT_F16 && dtype != MHLO_DT_BF16)
            return fail(MHLO_CUDA_UNSUPPORTED, "kernel_lookup: %s has no kernel for dtype %d", fused_op_kind, dtype);
        *out_kernel = k.id;
        return MHLO_CUDA_OK;
    }
    return fail(MHLO_CUDA_UNSUPPORTED, "kernel_lookup: no kernel named '%s'", fused_op_kind);
}

int mhlo_cuda_plan_create(const mhlo_cuda_plan_op* ops, int32_t n_ops, int32_t n_inputs, int32_t n_outputs, int64_t arena_bytes,
                          const void* constants_host, int64_t constant_bytes, mhlo_cuda_plan_t* out_plan) {
    if (!out_plan) return fail(MHLO_CUDA_INVALID_ARGUMENT, "plan_create: null output");
    *out_plan = nullptr;
    if (n_ops < 0 || (n_ops > 0 && !ops) || n_inputs < 0 || n_outputs < 0 || arena_bytes < 0 || constant_bytes < 0 || (constant_bytes > 0 && !constants_host))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "plan_create: bad argument");
    for (int32_t i = 0; i < n_ops; ++i) {
        const int want = args_of(ops[i].kernel);
        if (want < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "plan_create: op %d names unknown kernel %d", i, ops[i].kernel);
        for (int j = 0; j < 6; ++j) {
            const mhlo_cuda_binding& b = ops[i].args[j];
            const int64_t limit = b.source == MHLO_CUDA_SRC_UNIFIED ? arena_bytes : b.source == MHLO_CUDA_SRC_CONSTANT ? constant_bytes : -1;
            if (b.source < MHLO_CUDA_SRC_NONE || b.source > MHLO_CUDA_SRC_CONSTANT || b.offset < 0 || (limit >= 0 && b.offset >= limit) ||
                (b.source == MHLO_CUDA_SRC_INPUT && (b.index < 0 || b.index >= n_inputs)) ||
                (b.source == MHLO_CUDA_SRC_OUTPUT && (b.index < 0 || b.index >= n_outputs)))
                return fail(MHLO_CUDA_INVALID_ARGUMENT, "plan_create: op %d, argument %d: binding {source %d, index %d, offset %lld} is out of range", i, j,
                            b.source, b.index, static_cast<long long>(b.offset));
        }
    }
    Plan* p = new Plan();
    p->ops.assign(ops, ops + n_ops);
    p->arena_bytes = arena_bytes;
    p->constant_bytes = constant_bytes;
    p->n_inputs = n_inputs;
    p->n_outputs = n_outputs;
    cudaGetDevice(&p->device);
    int st = MHLO_CUDA_OK;
    if (arena_bytes > 0) st = mhlo_cuda_alloc(static_cast<size_t>(arena_bytes), &p->arena);
    if (st == MHLO_CUDA_OK && constant_bytes > 0) st = mhlo_cuda_alloc(static_cast<size_t>(constant_bytes), &p->constants);
    if (st == MHLO_CUDA_OK && constant_bytes > 0) st = mhlo_cuda_upload(p->constants, constants_host, static_cast<size_t>(constant_bytes), nullptr);
    if (st == MHLO_CUDA_OK && constant_bytes > 0) st = mhlo_cuda_stream_sync(nullptr);
    if (st != MHLO_CUDA_OK) {
        mhlo_cuda_free(p->arena);
        mhlo_cuda_free(p->constants);
        delete p;
        return st;
    }
    *out_plan = p;
    return MHLO_CUDA_OK;
}

int mhlo_cuda_plan_destroy(mhlo_cuda_plan_t plan) {
    Plan* p = static_cast<Plan*>(plan);
    if (!p) return MHLO_CUDA_OK;
    mhlo_cuda_free(p->arena);
    mhlo_cuda_free(p->constants);
    delete p;
    return MHLO_CUDA_OK;
}

int mhlo_cuda_plan_execute(mhlo_cuda_plan_t plan, const void* const* inputs, int32_t n_inputs, void* const* outputs, int32_t n_outputs,
                           mhlo_cuda_stream_t stream) {
    Plan* p = static_cast<Plan*>(plan);
    if (!p) return fail(MHLO_CUDA_INVALID_ARGUMENT, "plan_execute: null plan");
    if (n_inputs != p->n_inputs || n_outputs != p->n_outputs)
        return fail(MHLO_CUDA_INPUT_MISMATCH, "plan_execute: the plan takes %d inputs and %d outputs, got %d and %d", p->n_inputs, p->n_outputs, n_inputs, n_outputs);
    for (int32_t i = 0; i < n_inputs; ++i)
        if (!inputs || !inputs[i]) return fail(MHLO_CUDA_INVALID_ARGUMENT, "plan_execute: input %d is null", i);
    for (int32_t i = 0; i < n_outputs; ++i)
        if (!outputs || !outputs[i]) return fail(MHLO_CUDA_INVALID_ARGUMENT, "plan_execute: output %d is null", i);
    for (size_t i = 0; i < p->ops.size(); ++i) {
        const int st = run_op(*p, p->ops[i], inputs, outputs, stream);
        if (st != MHLO_CUDA_OK) return st;
    }
    return MHLO_CUDA_OK;
}

int mhlo_cuda_tuner_measure(mhlo_cuda_plan_t plan, const void* const* inputs, int32_t n_inputs, void* const* outputs, int32_t n_outputs,
                            int32_t warmup, int32_t iterations, float* out_median_ms) {
    if (!out_median_ms || iterations < 1 || warmup < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "tuner_measure: bad argument");
    void *e0 = nullptr, *e1 = nullptr;
    int st = mhlo_cuda_event_create(&e0);
    if (st == MHLO_CUDA_OK) st = mhlo_cuda_event_create(&e1);
    std::vector<float> ms(static_cast<size_t>(iterations), 0.f);
    for (int i = 0; i < warmup && st == MHLO_CUDA_OK; ++i) st = mhlo_cuda_plan_execute(plan, inputs, n_inputs, outputs, n_outputs, nullptr);
    for (int i = 0; i < iterations && st == MHLO_CUDA_OK; ++i) {
        st = mhlo_cuda_event_record(e0, nullptr);
        if (st == MHLO_CUDA_OK) st = mhlo_cuda_plan_execute(plan, inputs, n_inputs, outputs, n_outputs, nullptr);
        if (st == MHLO_CUDA_OK) st = mhlo_cuda_event_record(e1, nullptr);
        if (st == MHLO_CUDA_OK) st = mhlo_cuda_event_elapsed_ms(e0, e1, &ms[static_cast<size_t>(i)]);
    }
    if (e0) mhlo_cuda_event_destroy(e0);
    if (e1) mhlo_cuda_event_destroy(e1);
    if (st != MHLO_CUDA_OK) return st;
    std::sort(ms.begin(), ms.end());
    *out_median_ms = iterations % 2 ? ms[static_cast<size_t>(iterations / 2)] : 0.5f * (ms[static_cast<size_t>(iterations / 2 - 1)] + ms[static_cast<size_t>(iterations / 2)]);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_comm_init(int32_t n_devices, mhlo_cuda_comm_t* out_comm) {
    if (!out_comm) return fail(MHLO_CUDA_INVALID_ARGUMENT, "comm_init: null output");
    *out_comm = nullptr;
    int visible = 0;
    MHLO_CUDA_TRY(cudaGetDeviceCount(&visible), MHLO_CUDA_NO_DEVICE);
    if (n_devices < 1 || n_devices > visible || n_devices > 8)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "comm_init: %d devices asked, %d visible (1 to 8 supported)", n_devices, visible);
    int before = 0;
    cudaGetDevice(&before);
    Comm* c = new Comm();
    c->n = n_devices;
    c->streams.resize(static_cast<size_t>(n_devices), nullptr);
    for (int d = 0; d < n_devices; ++d) {
        cudaSetDevice(d);
        for (int e = 0; e < n_devices; ++e) {
            if (e == d) continue;
            int can = 0;
            cudaDeviceCanAccessPeer(&can, d, e);
            if (!can) {
                cudaSetDevice(before);
                delete c;
                return fail(MHLO_CUDA_UNSUPPORTED, "comm_init: device %d cannot address device %d's memory", d, e);
            }
            const cudaError_t en = cudaDeviceEnablePeerAccess(e, 0);
            if (en != cudaSuccess && en != cudaErrorPeerAccessAlreadyEnabled) {
                cudaSetDevice(before);
                delete c;
                return fail(MHLO_CUDA_EXECUTION_FAILED, "comm_init: cudaDeviceEnablePeerAccess(%d -> %d): %s", d, e, cudaGetErrorString(en));
            }
            cudaGetLastError();
        }
        if (cudaStreamCreateWithFlags(&c->streams[static_cast<size_t>(d)], cudaStreamNonBlocking) != cudaSuccess) {
            cudaSetDevice(before);
            delete c;
            return fail(MHLO_CUDA_EXECUTION_FAILED, "comm_init: stream on device %d: %s", d, cudaGetErrorString(cudaGetLastError()));
        }
    }
    cudaSetDevice(before);
    *out_comm = c;
    return MHLO_CUDA_OK;
}

int mhlo_cuda_comm_size(mhlo_cuda_comm_t comm) { return comm ? static_cast<Comm*>(comm)->n : 0; }

int mhlo_cuda_comm_destroy(mhlo_cuda_comm_t comm) {
    Comm* c = static_cast<Comm*>(comm);
    if (!c) return MHLO_CUDA_OK;
    int before = 0;
    cudaGetDevice(&before);
    for (int d = 0; d < c->n; ++d) {
        cudaSetDevice(d);
        if (c->streams[static_cast<size_t>(d)]) cudaStreamDestroy(c->streams[static_cast<size_t>(d)]);
    }
    cudaSetDevice(before);
    delete c;
    return MHLO_CUDA_OK;
}

int mhlo_cuda_all_gather(mhlo_cuda_comm_t comm, void* const* buffers, int64_t shard_bytes) {
    Comm* c = static_cast<Comm*>(comm);
    if (!c || !buffers) return fail(MHLO_CUDA_INVALID_ARGUMENT, "all_gather: null argument");
    if (shard_bytes < 0 || shard_bytes % 16 != 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "all_gather: the shard size must be a multiple of 16 bytes");
    for (int d = 0; d < c->n; ++d)
        if (!buffers[d] || !aligned16(buffers[d])) return fail(MHLO_CUDA_INVALID_ARGUMENT, "all_gather: buffer %d is null or not 16-byte aligned", d);
    if (shard_bytes == 0 || c->n == 1) return MHLO_CUDA_OK;
    int before = 0;
    cudaGetDevice(&before);
    const int64_t words = shard_bytes / 16;
    int st = MHLO_CUDA_OK;
    std::vector<void*> tables(static_cast<size_t>(c->n), nullptr);
    for (int d = 0; d < c->n && st == MHLO_CUDA_OK; ++d) {
        cudaSetDevice(d);
        std::vector<uint4*> peers;
        for (int e = 0; e < c->n; ++e)
            if (e != d) peers.push_back(static_cast<uint4*>(buffers[e]));
        const size_t table_bytes = peers.size() * sizeof(uint4*);
        cudaStream_t s = c->streams[static_cast<size_t>(d)];
        if (cudaMallocAsync(&tables[static_cast<size_t>(d)], table_bytes, s) != cudaSuccess ||
            cudaMemcpyAsync(tables[static_cast<size_t>(d)], peers.data(), table_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess ||
            cudaStreamSynchronize(s) != cudaSuccess) {  // the host table goes out of scope after this iteration
            st = fail(MHLO_CUDA_EXECUTION_FAILED, "all_gather: peer table on device %d: %s", d, cudaGetErrorString(cudaGetLastError()));
            break;
        }
        const int blocks = static_cast<int>(std::min<int64_t>((words + 255) / 256, 4 * kNumSMs));
        all_gather_push_kernel<<<blocks, 256, 0, s>>>(static_cast<const uint4*>(buffers[d]), static_cast<uint4* const*>(tables[static_cast<size_t>(d)]),
                                                     c->n - 1, static_cast<int64_t>(d) * words, words);
        if (cudaGetLastError() != cudaSuccess) st = fail(MHLO_CUDA_EXECUTION_FAILED, "all_gather: launch on device %d failed", d);
    }
    for (int d = 0; d < c->n; ++d) {
        cudaSetDevice(d);
        cudaStream_t s = c->streams[static_cast<size_t>(d)];
        if (cudaStreamSynchronize(s) != cudaSuccess && st == MHLO_CUDA_OK)
            st = fail(MHLO_CUDA_EXECUTION_FAILED, "all_gather: device %d: %s", d, cudaGetErrorString(cudaGetLastError()));
        if (tables[static_cast<size_t>(d)]) cudaFreeAsync(tables[static_cast<size_t>(d)], s);
    }
    cudaSetDevice(before);
    return st;
}

}  // extern "C"
