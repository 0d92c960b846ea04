/*
 * mhlo_cuda.h — C ABI of libmhlo_cuda.so, the sm_100a device runtime that stands where
 * MetalHLO's Metal objects stand on the compile/execute hot path.
 *
 * What each group replaces in the reference (paths relative to the MetalHLO project root):
 *   - device / memory calls     MTLDevice + MTLBuffer use in
 *                               Sources/MetalHLOCore/Runtime/IntegratedExecutor.swift:106-141,182-190
 *   - fused kernel entry points the KernelSpec pipelines built by
 *                               Sources/MetalHLOCore/Compiler/MetalHLOCompiler.swift:329-401 from
 *                               Sources/MetalHLOCore/Compiler/CodeGenerator.swift, and the hand-written
 *                               registry in Sources/MetalHLOCore/Metal/Kernels/
 *   - plan create / execute     the bind+dispatch loop of IntegratedExecutor.execute,
 *                               Sources/MetalHLOCore/Runtime/IntegratedExecutor.swift:150-270,390-615
 *
 * Conventions
 *   - Every function returns an int status: 0 on success, otherwise one of the MHLO status codes
 *     (3 parse, 4 unsupported op, 6 buffer, 7 input mismatch, 8 execution failed, 9 transfer, 10 invalid
 *     argument). mhlo_cuda_last_error() returns a thread-local message for the last non-zero status.
 *   - Pointers named *_dev are device pointers on the CUDA device that is current on the calling thread;
 *     `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream). Kernels are enqueued,
 *     not synchronised: the caller synchronises the stream.
 *   - No function aborts, traps or spins without a bound. There is no CPU fallback: without a CUDA device
 *     the kernel entry points return status 1 (no device).
 *   - dtype arguments use the MHLOElementType numbering (F16=0 F32=1 F64=2 BF16=3 I1=4 I8=5 I16=6 I32=7
 *     I64=8 UI8=9 UI16=10 UI32=11 UI64=12).
 */
#ifndef MHLO_CUDA_H
#define MHLO_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* mhlo_cuda_stream_t;

enum {
    MHLO_CUDA_OK = 0,
    MHLO_CUDA_NO_DEVICE = 1,
    MHLO_CUDA_UNSUPPORTED = 4,
    MHLO_CUDA_BUFFER_FAILED = 6,
    MHLO_CUDA_INPUT_MISMATCH = 7,
    MHLO_CUDA_EXECUTION_FAILED = 8,
    MHLO_CUDA_TRANSFER_FAILED = 9,
    MHLO_CUDA_INVALID_ARGUMENT = 10
};

enum {
    MHLO_DT_F16 = 0, MHLO_DT_F32 = 1, MHLO_DT_F64 = 2, MHLO_DT_BF16 = 3, MHLO_DT_I1 = 4, MHLO_DT_I8 = 5,
    MHLO_DT_I16 = 6, MHLO_DT_I32 = 7, MHLO_DT_I64 = 8, MHLO_DT_UI8 = 9, MHLO_DT_UI16 = 10,
    MHLO_DT_UI32 = 11, MHLO_DT_UI64 = 12
};

/* ---- library / error ------------------------------------------------------------------------------ */

/* Static version string of the runtime ("mhlo-cuda x.y.z sm_100a"). */
const char* mhlo_cuda_version(void);
/* Message of the last failing call on this thread; "" when none. Owned by the library. */
const char* mhlo_cuda_last_error(void);
/* Bytes per element of a dtype code; I1 is stored as one byte per element; 0 for an unknown code. */
size_t mhlo_cuda_dtype_size(int dtype);

/* ---- device and memory (replaces MTLDevice/MTLBuffer, IntegratedExecutor.swift:106-141) ------------ */

int mhlo_cuda_device_count(int* out_count);
/* Makes `ordinal` current on the calling thread. */
int mhlo_cuda_device_set(int ordinal);
/* Ordinal of the device that is current on the calling thread. */
int mhlo_cuda_device_current(int* out_ordinal);
/* Writes the device name into out_name (NUL-terminated, truncated to cap). */
int mhlo_cuda_device_name(int ordinal, char* out_name, size_t cap);
int mhlo_cuda_stream_create(mhlo_cuda_stream_t* out_stream);
int mhlo_cuda_stream_destroy(mhlo_cuda_stream_t stream);
int mhlo_cuda_stream_sync(mhlo_cuda_stream_t stream);
int mhlo_cuda_alloc(size_t bytes, void** out_dev);
int mhlo_cuda_free(void* dev);
/* Pinned host staging memory for mhlo_cuda_upload/download at full PCIe rate. */
int mhlo_cuda_host_alloc(size_t bytes, void** out_host);
int mhlo_cuda_host_free(void* host);
/* Asynchronous on `stream`; the host range must stay valid until the stream is synchronised. */
int mhlo_cuda_upload(void* dst_dev, const void* src_host, size_t bytes, mhlo_cuda_stream_t stream);
int mhlo_cuda_download(void* dst_host, const void* src_dev, size_t bytes, mhlo_cuda_stream_t stream);
int mhlo_cuda_copy(void* dst_dev, const void* src_dev, size_t bytes, mhlo_cuda_stream_t stream);
int mhlo_cuda_memset(void* dst_dev, int byte_value, size_t bytes, mhlo_cuda_stream_t stream);

/*
 * CUDA graphs: record everything the calling thread enqueues on `stream` between begin and end into an executable
 * graph, then replay it with one launch (replaces the per-dispatch encoder loop of IntegratedExecutor.swift:150-270
 * for programs that run repeatedly on the same buffers). `stream` must not be the default stream. Nothing runs
 * during capture. end returns the instantiated graph in *out_graph (NULL when the recorded work could not be
 * instantiated); a capture that failed half-way is ended and reported as MHLO_CUDA_UNSUPPORTED.
 */
int mhlo_cuda_graph_capture_begin(mhlo_cuda_stream_t stream);
int mhlo_cuda_graph_capture_end(mhlo_cuda_stream_t stream, void** out_graph);
int mhlo_cuda_graph_launch(void* graph, mhlo_cuda_stream_t stream);
int mhlo_cuda_graph_destroy(void* graph);

/*
 * Sharing one allocation between the processes of a multi-GPU job (one process per GPU on one node): the owner
 * exports a 64-byte handle of memory it got from mhlo_cuda_alloc, the others open it and receive an address that is
 * valid in their own process and reaches the owner's GPU over NVLink (peer access is enabled on first use). Close
 * before the owner frees. No counterpart in the reference, which runs on one device.
 */
int mhlo_cuda_ipc_export(const void* dev_ptr, unsigned char out_handle[64]);
int mhlo_cuda_ipc_open(const unsigned char handle[64], void** out_dev_ptr);
int mhlo_cuda_ipc_close(void* dev_ptr);

/* Device-side timing (replaces MTLCommandBuffer GPUStartTime/GPUEndTime, Executable.swift:164). */
int mhlo_cuda_event_create(void** out_event);
int mhlo_cuda_event_destroy(void* event);
int mhlo_cuda_event_record(void* event, mhlo_cuda_stream_t stream);
/* Blocks the host until the event's latest record has been reached (cudaEventSynchronize). */
int mhlo_cuda_event_sync(void* event);
/* Work queued on `stream` after this call waits for the event's latest record (cudaStreamWaitEvent). */
int mhlo_cuda_stream_wait_event(mhlo_cuda_stream_t stream, void* event);
/* fn(user) runs on a driver thread once everything queued on `stream` before it has finished (cudaLaunchHostFunc): how an
 * asynchronous transfer reports its completion. fn must not call into this library or CUDA. */
int mhlo_cuda_stream_host_callback(mhlo_cuda_stream_t stream, void (*fn)(void*), void* user);
/* Synchronises on `stop`, then writes the elapsed milliseconds between the two events. */
int mhlo_cuda_event_elapsed_ms(void* start, void* stop, float* out_ms);

/* ---- row kernels: LayerNorm / RMSNorm / softmax ----------------------------------------------------- */

/*
 * Tuning knobs of the row kernels (the CUDA counterpart of TuningConfig,
 * Sources/MetalHLOCore/Compiler/KernelTypes.swift:212-257). Zero in a field = let the library choose.
 *   threads        threads per CTA (multiple of 32, <= 1024); one CTA works on one row at a time
 *   vecs_per_thread  16-byte vectors each thread keeps in registers (1, 2, 4 or 8)
 *   ctas_per_sm    CTAs per SM of the persistent grid; 0 = as many as fit (occupancy query), -1 = one CTA per row
 */
typedef struct {
    int32_t threads;
    int32_t vecs_per_thread;
    int32_t ctas_per_sm;
} mhlo_cuda_row_tuning;

/*
 * y[r,:] = (x[r,:] - mean_r) / sqrt(var_r + eps) * gamma + beta, biased variance, statistics in fp32.
 * x, y: [rows, hidden] row-major of `dtype` (F32, F16 or BF16); gamma/beta: [hidden] of the same dtype,
 * either may be NULL (treated as 1 / 0). Replaces kernel_layer_norm
 * (Sources/MetalHLOCore/Compiler/CodeGenerator.swift:4610-4650), layer_norm_kernel(_half/_no_affine)
 * (Sources/MetalHLOCore/Metal/Kernels/LayerNormKernel.swift:41-351) with the semantics of
 * FusedLayerNormHandler (Sources/MetalHLOCore/Compiler/CustomCallHandlers.swift:285-342).
 */
int mhlo_cuda_layer_norm(int dtype, const void* x_dev, const void* gamma_dev, const void* beta_dev,
                         void* y_dev, int64_t rows, int64_t hidden, float eps,
                         const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream);

/*
 * y[r,:] = x[r,:] / sqrt(mean(x[r,:]^2) + eps) * gamma. gamma may be NULL. Replaces kernel_rms_norm
 * (CodeGenerator.swift:4652-4686), rms_norm_kernel(_half/_no_gamma) (LayerNormKernel.swift:427-677),
 * semantics of FusedRMSNormHandler (CustomCallHandlers.swift:349-394).
 */
int mhlo_cuda_rms_norm(int dtype, const void* x_dev, const void* gamma_dev, void* y_dev, int64_t rows,
                       int64_t hidden, float eps, const mhlo_cuda_row_tuning* tuning,
                       mhlo_cuda_stream_t stream);

/*
 * Residual add fused into the norm: sum = x + residual (rounded to `dtype`, exactly what a separate add writes),
 * y = LayerNorm(sum) or RMSNorm(sum). sum_dev receives the sum (the residual stream later layers read); x, residual,
 * sum, y: [rows, hidden]. One pass over x and residual instead of an add kernel plus a re-read by the norm. No
 * counterpart in the reference (its "residual-chain-fusion" pass is registered without an implementation,
 * Compiler/PassManager.swift:214-221).
 */
int mhlo_cuda_add_layer_norm(int dtype, const void* x_dev, const void* residual_dev, const void* gamma_dev,
                             const void* beta_dev, void* sum_dev, void* y_dev, int64_t rows, int64_t hidden,
                             float eps, const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream);
int mhlo_cuda_add_rms_norm(int dtype, const void* x_dev, const void* residual_dev, const void* gamma_dev,
                           void* sum_dev, void* y_dev, int64_t rows, int64_t hidden, float eps,
                           const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream);
/*
 * The same with a residual of residual_rows rows that repeats down the tensor (rows a multiple of residual_rows): row r
 * adds residual row r mod residual_rows. The position table added to the token embeddings before the first norm of a
 * transformer is this form: [sequence, hidden] repeated over the batch.
 */
int mhlo_cuda_add_layer_norm_rows(int dtype, const void* x_dev, const void* residual_dev, int64_t residual_rows,
                                  const void* gamma_dev, const void* beta_dev, void* sum_dev, void* y_dev, int64_t rows,
                                  int64_t hidden, float eps, const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream);
int mhlo_cuda_add_rms_norm_rows(int dtype, const void* x_dev, const void* residual_dev, int64_t residual_rows,
                                const void* gamma_dev, void* sum_dev, void* y_dev, int64_t rows, int64_t hidden, float eps,
                                const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream);

/*
 * Softmax along one axis of a tensor viewed as [outer, axis_len, inner] (inner = 1 for the last axis):
 * y = exp(x - max) / sum(exp(x - max)). Replaces kernel_softmax (CodeGenerator.swift:4690-4794) and
 * softmax_kernel(_half) (Sources/MetalHLOCore/Metal/Kernels/SoftmaxKernel.swift:23-167), semantics of
 * FusedSoftmaxHandler (CustomCallHandlers.swift:644-672).
 */
int mhlo_cuda_softmax(int dtype, const void* x_dev, void* y_dev, int64_t outer, int64_t axis_len,
                      int64_t inner, const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream);


/* ---- generic tensor kernels (strided views) --------------------------------------------------------- */

#define MHLO_CUDA_MAX_RANK 8
#define MHLO_CUDA_EW_MAX_INPUTS 8
#define MHLO_CUDA_EW_MAX_INSTS 32

/*
 * A strided view of device memory: element (i0..i{rank-1}) lives at base + sum(i_d * stride[d]) elements.
 * stride 0 broadcasts a dimension, a negative stride reverses it. This is what a reshape / transpose /
 * broadcast_in_dim / slice / reverse result is until a kernel needs it contiguous - the counterpart of
 * StridedTensorView (Sources/MetalHLOCore/Runtime/StridedTensorView.swift) and of the zero-copy reshape
 * views in CodeGenerator.swift:183-245.
 */
typedef struct {
    const void* base;
    int32_t dtype;
    int32_t rank;
    int64_t shape[MHLO_CUDA_MAX_RANK];
    int64_t stride[MHLO_CUDA_MAX_RANK];
} mhlo_cuda_view;

/* Opcodes of the elementwise program (one StableHLO elementwise op each, plus the fused activations). */
enum {
    MHLO_EW_COPY = 0,  /* r = a (also convert: the store rounds to the output dtype) */
    MHLO_EW_IMM,       /* r = imm */
    MHLO_EW_IOTA,      /* r = index along output dimension (int)imm */
    MHLO_EW_ADD, MHLO_EW_SUB, MHLO_EW_MUL, MHLO_EW_DIV, MHLO_EW_REM, MHLO_EW_MAX, MHLO_EW_MIN, MHLO_EW_POW,
    MHLO_EW_ATAN2, MHLO_EW_AND, MHLO_EW_OR, MHLO_EW_XOR, MHLO_EW_SHL, MHLO_EW_SHR_A, MHLO_EW_SHR_L,
    MHLO_EW_NEG, MHLO_EW_ABS, MHLO_EW_EXP, MHLO_EW_EXPM1, MHLO_EW_LOG, MHLO_EW_LOG1P, MHLO_EW_SQRT,
    MHLO_EW_RSQRT, MHLO_EW_CBRT, MHLO_EW_TANH, MHLO_EW_LOGISTIC, MHLO_EW_SIN, MHLO_EW_COS, MHLO_EW_TAN,
    MHLO_EW_FLOOR, MHLO_EW_CEIL, MHLO_EW_ROUND_AFZ, MHLO_EW_ROUND_EVEN, MHLO_EW_SIGN, MHLO_EW_NOT,
    MHLO_EW_IS_FINITE, MHLO_EW_POPCNT, MHLO_EW_CLZ,
    MHLO_EW_CMP_EQ, MHLO_EW_CMP_NE, MHLO_EW_CMP_LT, MHLO_EW_CMP_LE, MHLO_EW_CMP_GT, MHLO_EW_CMP_GE,
    MHLO_EW_SELECT,    /* r = a ? b : c */
    MHLO_EW_CLAMP,     /* r = min(max(b, a), c) with a = lower bound, c = upper bound */
    MHLO_EW_GELU_TANH, MHLO_EW_GELU_ERF, MHLO_EW_SILU, MHLO_EW_RELU,
    MHLO_EW_ROUND_TO,  /* r = a rounded to the float dtype (int)imm and widened again: keeps the unfused rounding
                          points of a fused chain */
    MHLO_EW_ERF,       /* chlo.erf */
    MHLO_EW_REDUCE_PRECISION, /* r = a rounded (to nearest even) to a float format with imm / 64 exponent bits and imm % 64
                                 mantissa bits, then widened again: overflow gives infinity, underflow zero, NaN stays NaN
                                 (infinity when the format has no mantissa bits) */
    MHLO_EW_OP_COUNT
};

/* One instruction: register a/b/c are indices into [inputs..., results of earlier instructions...]. */
typedef struct {
    int32_t op;
    int32_t a, b, c;
    double imm;
} mhlo_cuda_ew_inst;

/*
 * Runs `prog` once per output element. Registers 0..n_inputs-1 hold the element of each input view (all views
 * have the output's rank and shape; use stride 0 to broadcast); instruction k writes register n_inputs+k; the
 * last instruction's result is stored to out (contiguous, row-major) rounded/wrapped to out_dtype.
 * Arithmetic runs in fp64 when any operand or the output is f64, else in fp32 when any is a float type, else
 * in 64-bit integers (ui64 operands select unsigned division/shift/compare). Replaces the generated unary /
 * binary / compare / select / clamp / convert / iota / broadcast / transpose / slice / reverse kernels
 * (Sources/MetalHLOCore/Compiler/CodeGenerator.swift:851-1122,1558-2048,2840-3151) and kernel_elementwise_chain,
 * kernel_gelu, kernel_silu (:4853-4981).
 */
int mhlo_cuda_elementwise(const mhlo_cuda_view* inputs, int32_t n_inputs, const mhlo_cuda_ew_inst* prog,
                          int32_t n_insts, void* out_dev, int32_t out_dtype, const int64_t* out_shape,
                          int32_t out_rank, mhlo_cuda_stream_t stream);

/*
 * Same as mhlo_cuda_elementwise, but the result is written through a strided destination view (`out`, whose
 * dtype/rank/shape define the iteration space). With a one-instruction COPY program this is the strided copy
 * that materialises transposes, concatenate operands and pad interiors.
 */
int mhlo_cuda_elementwise_to_view(const mhlo_cuda_view* inputs, int32_t n_inputs, const mhlo_cuda_ew_inst* prog,
                                  int32_t n_insts, const mhlo_cuda_view* out, mhlo_cuda_stream_t stream);

enum {
    MHLO_REDUCE_SUM = 0, MHLO_REDUCE_MAX, MHLO_REDUCE_MIN, MHLO_REDUCE_PROD, MHLO_REDUCE_AND, MHLO_REDUCE_OR,
    MHLO_REDUCE_XOR, MHLO_REDUCE_ARGMAX, MHLO_REDUCE_ARGMIN
};

/*
 * Reduces the trailing (rank - n_kept) dimensions of `in` (the caller permutes the view so the kept dimensions
 * come first). out_dev is contiguous over the kept dimensions in the input dtype. init_dev (device scalar of the
 * input dtype, may be NULL) is folded in as one more element. Float types accumulate in fp32 (f64 in fp64),
 * integers in int64. ARGMAX/ARGMIN additionally need index_out_dev (dtype index_dtype, I32 or I64): the
 * flattened position of the first extremum along the reduced dimensions; NaN counts as the extremum.
 * Replaces kernel_reduce (CodeGenerator.swift:4071-4496) and MPSGraphCompiler.compileReduce
 * (Sources/MetalHLOCore/Compiler/MPSGraphCompiler.swift:1070-1144).
 */
int mhlo_cuda_reduce(const mhlo_cuda_view* in, int32_t n_kept, int32_t op, const void* init_dev, void* out_dev,
                     void* index_out_dev, int32_t index_dtype, mhlo_cuda_stream_t stream);

/*
 * Many independent dense dtype conversions in one launch (per 96 jobs): dst[i] = convert(src[i]) for i < count, with
 * the rounding of MHLO_EW_COPY (round to nearest even). Pairs supported: F32 <-> F16, F32 <-> BF16, and same-type
 * copies of those three. A model whose parameters arrive as fp32 and compute in 16 bit converts every weight at the
 * start of each forward pass; done one tensor per launch, the small ones cost a launch latency each. No counterpart
 * in the reference, which dispatches one kernel per convert (CodeGenerator.swift:1012-1075).
 */
typedef struct {
    const void* src;
    void* dst;
    int64_t count;
    int32_t src_dtype, dst_dtype;
} mhlo_cuda_convert_job;
int mhlo_cuda_convert_many(const mhlo_cuda_convert_job* jobs, int32_t n_jobs, mhlo_cuda_stream_t stream);

/*
 * mhlo_cuda_reduce for callers that cannot let the library allocate. No counterpart in the reference (its reduce
 * kernels use no scratch memory; this entry point exists because the split reduce above does).
 *
 * mhlo_cuda_reduce takes the partial accumulators of a split reduce from the stream-ordered allocator. A host that
 * has given all free device memory to its own pool and treats any later allocation as an error, or that is inside
 * a stream capture on a device without a configured memory pool, cannot accept that. This entry point always runs
 * the split algorithm and keeps the partials in an array that is part of the library image:
 *   - it allocates and frees nothing, on the device or on the host;
 *   - the array holds 65536 bytes per device = 4096 partial accumulators (16 bytes each); a call needs
 *     (number of outputs) x (segments per output) of them and is refused with MHLO_CUDA_UNSUPPORTED and a message
 *     naming both numbers when that is more. At most 65535 outputs; the reduced range must not be empty;
 *   - `splits` = segments per output; 0 picks the same count mhlo_cuda_reduce would use, which makes the results of
 *     the two entry points identical bit for bit whenever mhlo_cuda_reduce takes its split path;
 *   - nothing in the array has to be cleared beforehand, every partial that is read has been written by the same call;
 *   - there is one array per device: calls that overlap in time on one device (other streams, other threads) race
 *     on it and give wrong results. Calls on one stream are ordered and safe;
 *   - the first call on each device looks the array's address up (with that device current). If that first call is
 *     to happen around a stream capture, make one call on that device before the capture begins.
 * All other arguments as for mhlo_cuda_reduce.
 */
int mhlo_cuda_reduce_static_scratch(const mhlo_cuda_view* in, int32_t n_kept, int32_t op, const void* init_dev,
                                    void* out_dev, void* index_out_dev, int32_t index_dtype, int32_t splits,
                                    mhlo_cuda_stream_t stream);

/* Dimension numbers of stablehlo.gather; counts say how many entries of each array are used. */
typedef struct {
    int32_t n_offset_dims, n_collapsed, n_operand_batching, n_start_index_map;
    int32_t offset_dims[MHLO_CUDA_MAX_RANK];
    int32_t collapsed_slice_dims[MHLO_CUDA_MAX_RANK];
    int32_t operand_batching_dims[MHLO_CUDA_MAX_RANK];
    int32_t start_indices_batching_dims[MHLO_CUDA_MAX_RANK];
    int32_t start_index_map[MHLO_CUDA_MAX_RANK];
    int32_t index_vector_dim;
    int64_t slice_sizes[MHLO_CUDA_MAX_RANK];
} mhlo_cuda_gather_dims;

/*
 * stablehlo.gather with the full dimension-number semantics; start indices are clamped so that every slice
 * stays inside the operand (CodeGenerator.swift:1133-1292, clamp at :1252-1254). operand and indices are
 * contiguous; elem_size is the operand's bytes per element (values are moved, never interpreted).
 */
int mhlo_cuda_gather(const void* operand_dev, int32_t elem_size, const int64_t* operand_shape, int32_t operand_rank,
                     const void* indices_dev, int32_t index_dtype, const int64_t* indices_shape,
                     int32_t indices_rank, const mhlo_cuda_gather_dims* dims, void* out_dev,
                     const int64_t* out_shape, int32_t out_rank, mhlo_cuda_stream_t stream);

/*
 * dynamic_slice / dynamic_update_slice: start indices are read on the device from n_idx scalar tensors
 * (index_dtype I32 or I64) and clamped to keep the window inside `operand`
 * (CodeGenerator.swift:1640-1790). For the update form, out must already hold the operand.
 */
int mhlo_cuda_dynamic_slice(const void* operand_dev, int32_t elem_size, const int64_t* operand_shape, int32_t rank,
                            const void* const* index_devs, int32_t index_dtype, const int64_t* slice_sizes,
                            void* out_dev, mhlo_cuda_stream_t stream);
int mhlo_cuda_dynamic_update_slice(void* operand_inout_dev, int32_t elem_size, const int64_t* operand_shape,
                                   int32_t rank, const void* update_dev, const int64_t* update_shape,
                                   const void* const* index_devs, int32_t index_dtype, mhlo_cuda_stream_t stream);

/* Window of stablehlo.reduce_window / select_and_scatter over a rank-`rank` operand. */
typedef struct {
    int32_t rank;
    int64_t size[MHLO_CUDA_MAX_RANK];             /* window_dimensions */
    int64_t stride[MHLO_CUDA_MAX_RANK];           /* window_strides */
    int64_t base_dilation[MHLO_CUDA_MAX_RANK];
    int64_t window_dilation[MHLO_CUDA_MAX_RANK];
    int64_t pad_low[MHLO_CUDA_MAX_RANK];          /* may be negative; the high padding is implied by out_shape */
} mhlo_cuda_window;

/*
 * stablehlo.reduce_window with the full attribute set: out[o] = op over the window positions w of
 * padded(dilated(in))[o * stride + w * window_dilation], where positions that fall into the padding or between
 * dilated elements hold the init value. `in` may be any strided view; out_dev is contiguous in in->dtype and
 * init_dev is a device scalar of that dtype. op is one of MHLO_REDUCE_SUM/MAX/MIN/PROD/AND/OR/XOR; floats
 * accumulate in fp32 (f64 in fp64), integers in int64, in row-major window order. The reference covers the 2-D
 * NHWC pooling subset through MPSGraph pooling (Sources/MetalHLOCore/Compiler/MPSGraphCompiler.swift:3056-3200).
 */
int mhlo_cuda_reduce_window(const mhlo_cuda_view* in, const mhlo_cuda_window* window, int32_t op, const void* init_dev,
                            void* out_dev, const int64_t* out_shape, mhlo_cuda_stream_t stream);

/*
 * stablehlo.select_and_scatter (the gradient of a pooling): for every element of `source` the matching window of
 * the operand (padded with the init value; dilations are not part of this op) is scanned in row-major order keeping
 * the element e for which select(kept, e) fails, select(a, b) = a <cmp> b with cmp one of MHLO_EW_CMP_GE/GT/LE/LT;
 * the source element is then combined (scatter_mode: MHLO_SCATTER_ADD/MUL/MAX/MIN, atomically) into the result at the
 * kept element's position unless that lies in the padding. result_inout_dev (contiguous, operand's shape and dtype)
 * must already be filled with the init value. The reference covers the 2-D NHWC max-pool gradient through
 * maxPooling2DGradient (MPSGraphCompiler.swift:4203-4245).
 */
int mhlo_cuda_select_and_scatter(const mhlo_cuda_view* operand, const void* source_dev, const int64_t* source_shape,
                                 const void* init_dev, const mhlo_cuda_window* window, int32_t select_cmp,
                                 int32_t scatter_mode, void* result_inout_dev, mhlo_cuda_stream_t stream);

typedef struct {
    int32_t n_update_window_dims, n_inserted_window_dims, n_input_batching, n_scatter_dims_to_operand;
    int32_t update_window_dims[MHLO_CUDA_MAX_RANK];
    int32_t inserted_window_dims[MHLO_CUDA_MAX_RANK];
    int32_t input_batching_dims[MHLO_CUDA_MAX_RANK];
    int32_t scatter_indices_batching_dims[MHLO_CUDA_MAX_RANK];
    int32_t scatter_dims_to_operand_dims[MHLO_CUDA_MAX_RANK];
    int32_t index_vector_dim;
} mhlo_cuda_scatter_dims;

enum { MHLO_SCATTER_SET = 0, MHLO_SCATTER_ADD, MHLO_SCATTER_MUL, MHLO_SCATTER_MAX, MHLO_SCATTER_MIN };

/*
 * stablehlo.scatter with the full dimension numbers, applied in place: result_inout_dev must already hold the
 * operand (contiguous, `dtype`). Every element of `updates` (contiguous) is combined into the element it addresses
 * with an atomic read-modify-write (mode = the update computation); updates whose target lies outside the operand
 * are skipped. Colliding updates are applied in an unspecified order: SET keeps one of them, and floating-point ADD
 * / MUL may differ from a sequential sum in the last bits. Modes match the reference's scatter modes
 * (MPSGraphCompiler.swift:1639-1690).
 */
int mhlo_cuda_scatter(void* result_inout_dev, int32_t dtype, const int64_t* operand_shape, int32_t operand_rank,
                      const void* indices_dev, int32_t index_dtype, const int64_t* indices_shape, int32_t indices_rank,
                      const void* updates_dev, const int64_t* updates_shape, int32_t updates_rank,
                      const mhlo_cuda_scatter_dims* dims, int32_t mode, mhlo_cuda_stream_t stream);

/*
 * stablehlo.sort along one dimension by the first operand, the other operands carried along (argsort passes an
 * iota as the second operand). All n_operands tensors share `shape` (contiguous); operand i has dtypes[i] and is
 * written sorted to outs_dev[i] (must not alias the inputs). Ascending or descending order of the key under the
 * total order -NaN < -inf < .. < -0 < +0 < .. < +inf < +NaN; the sort is always stable. `descending` is a set of
 * flags: bit 0 = descending; bit 1 = -0 and +0 compare equal and keep the order they came in (a comparator that
 * compares with FLOAT semantics instead of TOTALORDER). Slices of up to
 * MHLO_CUDA_SORT_SMEM_MAX keys are sorted in shared memory by one CTA each; longer ones use `scratch_dev`
 * (mhlo_cuda_sort_scratch_bytes() bytes) for a bitonic network over global memory. Replaces argSort +
 * gatherAlongAxis (MPSGraphCompiler.swift:3599-3613).
 */
#define MHLO_CUDA_SORT_SMEM_MAX 8192
#define MHLO_CUDA_SORT_MAX_OPERANDS 8
int64_t mhlo_cuda_sort_scratch_bytes(const int64_t* shape, int32_t rank, int32_t dimension);
int mhlo_cuda_sort(const void* const* operands_dev, void* const* outs_dev, const int32_t* dtypes, int32_t n_operands,
                   const int64_t* shape, int32_t rank, int32_t dimension, int32_t descending, void* scratch_dev,
                   int64_t scratch_bytes, mhlo_cuda_stream_t stream);

/*
 * Geometry of stablehlo.convolution in canonical order: input [batch, spatial.., feature], kernel [spatial..,
 * input feature, output feature], output [batch, spatial.., feature]. The three tensors are addressed through
 * element strides, so any dimension_numbers layout (NHWC, NCHW, HWIO, OIHW, ..) is a choice of strides.
 */
#define MHLO_CUDA_CONV_MAX_SPATIAL 6
typedef struct {
    int32_t n_spatial;
    int32_t reverse[MHLO_CUDA_CONV_MAX_SPATIAL];       /* window_reversal */
    int64_t batch, in_features, out_features;           /* of the input, the input, the kernel */
    int64_t feature_group_count, batch_group_count;
    int64_t in_size[MHLO_CUDA_CONV_MAX_SPATIAL], kernel_size[MHLO_CUDA_CONV_MAX_SPATIAL], out_size[MHLO_CUDA_CONV_MAX_SPATIAL];
    int64_t stride[MHLO_CUDA_CONV_MAX_SPATIAL], pad_low[MHLO_CUDA_CONV_MAX_SPATIAL];
    int64_t lhs_dilation[MHLO_CUDA_CONV_MAX_SPATIAL], rhs_dilation[MHLO_CUDA_CONV_MAX_SPATIAL];
    int64_t in_batch_stride, in_feature_stride, in_spatial_stride[MHLO_CUDA_CONV_MAX_SPATIAL];
    int64_t kernel_in_stride, kernel_out_stride, kernel_spatial_stride[MHLO_CUDA_CONV_MAX_SPATIAL];
    int64_t out_batch_stride, out_feature_stride, out_spatial_stride[MHLO_CUDA_CONV_MAX_SPATIAL];
} mhlo_cuda_conv;

/*
 * 2-D convolution on the tensor cores without a patch matrix: dense NHWC input [images, in_h, in_w, channels], dense HWIO
 * filter [filter_h, filter_w, channels, features], dense NHWC result [images, out_h, out_w, features]; stride 1, one
 * feature group, zero padding pad_top / pad_left in front (whatever the result's extent needs behind), filter dilation.
 * out[n, y, x, f] = act(sum over (dy, dx, c) of in[n, y + dy * dilation_h - pad_top, x + dx * dilation_w - pad_left, c]
 * * filter[dy, dx, c, f] + bias[f]). The product's A tile for one filter tap and 64 channels is an 8 x 16 patch of input
 * pixels fetched by one bulk tensor copy (pixels outside the image arrive as zeros), so the input is read from HBM
 * once instead of being expanded to a patch matrix first (mhlo_cuda_im2col + mhlo_cuda_gemm: 9 times the bytes for a 3 x 3
 * filter). f16 / bf16 tensors, channels a multiple of 64, features a multiple of 8; anything else returns
 * MHLO_CUDA_UNSUPPORTED and the caller takes the patch-matrix route. bias_dev (of the result's type) may be NULL.
 * Stands where the reference lowers convolution to MPSGraph convolution2D (Compiler/MPSGraphCompiler.swift) and
 * FusedConvBiasActHandler (Compiler/CustomCallHandlers.swift:563-640).
 */
int mhlo_cuda_conv2d_nhwc(int32_t dtype, int32_t out_dtype, const void* x_dev, const void* filter_dev, void* out_dev,
                          int64_t images, int64_t in_h, int64_t in_w, int64_t channels, int64_t filter_h, int64_t filter_w,
                          int64_t features, int64_t out_h, int64_t out_w, int64_t pad_top, int64_t pad_left,
                          int64_t dilation_h, int64_t dilation_w, const void* bias_dev, int32_t epilogue,
                          mhlo_cuda_stream_t stream);
/* The same with window strides of 1 to 8: the patch of a tap is then every stride-th input pixel, which the bulk tensor
 * copy takes through its traversal strides, in[n, y * stride_h + dy * dilation_h - pad_top, x * stride_w + dx * dilation_w -
 * pad_left, c]. */
int mhlo_cuda_conv2d_nhwc_strided(int32_t dtype, int32_t out_dtype, const void* x_dev, const void* filter_dev, void* out_dev,
                                  int64_t images, int64_t in_h, int64_t in_w, int64_t channels, int64_t filter_h, int64_t filter_w,
                                  int64_t features, int64_t out_h, int64_t out_w, int64_t pad_top, int64_t pad_left,
                                  int64_t dilation_h, int64_t dilation_w, int64_t stride_h, int64_t stride_w, const void* bias_dev,
                                  int32_t epilogue, mhlo_cuda_stream_t stream);

/*
 * Direct convolution, one thread per output element, every attribute of the op honoured (strides, padding, both
 * dilations, window reversal, feature and batch groups). Floats accumulate in fp32 (f64 in fp64), integers in
 * int64. The general path; the reference lowers convolution to MPSGraph convolution2D
 * (Sources/MetalHLOCore/Compiler/MPSGraphCompiler.swift:2695-3050).
 */
int mhlo_cuda_convolution(int32_t dtype, const void* in_dev, const void* kernel_dev, void* out_dev, const mhlo_cuda_conv* conv,
                          mhlo_cuda_stream_t stream);

/*
 * The patch matrix of a convolution with batch_group_count 1: cols[g][m][k] for feature group g, output position
 * m = (batch, output spatial..) row-major and k = (kernel spatial.., input feature within the group) row-major,
 * rows padded with zeros to `row_pitch` elements (>= kernel volume x features per group). Positions that fall into
 * the padding or between dilated input elements are zero. The convolution is then one (batched over groups) GEMM
 * of cols with the kernel viewed as [k, output feature], which runs on the tcgen05 kernel of mhlo_cuda_gemm.
 */
int mhlo_cuda_im2col(int32_t dtype, const void* in_dev, void* cols_dev, int64_t row_pitch, const mhlo_cuda_conv* conv,
                     mhlo_cuda_stream_t stream);

/*
 * C[b0,b1,m,n] = sum_k A(b0,b1,m,k) * B(b0,b1,k,n) for arbitrary element strides (a_strides / b_strides =
 * {batch0, batch1, row, col} strides in elements; C is contiguous). Any dtype: floats accumulate in fp32
 * (f64 in fp64), integers in int64. This is the general-layout path of dot_general - strict fp32 as the
 * reference defaults to (Sources/MetalHLOCore/Compiler/TF32Transform.swift:20 is opt-in) - and the fallback
 * for shapes the tensor-core kernels do not take. Replaces kernel_matmul basic/tiled and kernel_gemv
 * (CodeGenerator.swift:3344-3454,3891-4068).
 */
int mhlo_cuda_dot_strided(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[4],
                          const void* b_dev, const int64_t b_strides[4], void* c_dev, int64_t batch0,
                          int64_t batch1, int64_t m, int64_t n, int64_t k, mhlo_cuda_stream_t stream);

/* ---- contractions ------------------------------------------------------------------------------------ */

enum {
    MHLO_EPILOGUE_NONE = 0, MHLO_EPILOGUE_RELU, MHLO_EPILOGUE_GELU_TANH, MHLO_EPILOGUE_GELU_ERF,
    MHLO_EPILOGUE_SILU, MHLO_EPILOGUE_TANH, MHLO_EPILOGUE_SIGMOID
};

/*
 * dot_general in canonical form with a fused epilogue:
 *   C[b0,b1,m,n] = act( sum_k A(b0,b1,m,k) * B(b0,b1,k,n) + bias[n] ),  C dense row-major, fp32 accumulation.
 * a_strides / b_strides = {batch0, batch1, row, col} element strides, so transposed and batch-interleaved
 * operands need no copy. bias_dev ([n], dtype = out_dtype) may be NULL. BF16/F16 operands whose rows or columns
 * are contiguous and 16-byte aligned run on the tcgen05 tensor-core kernel (TMA-fed, TMEM accumulators);
 * everything else takes the general-layout kernel behind mhlo_cuda_dot_strided. Replaces kernel_matmul (MPP and
 * simdgroup variants, Sources/MetalHLOCore/Compiler/CodeGenerator.swift:3463-3886), kernel_matmul_bias_act
 * (:4797-4850) and the semantics of FusedMatMulBiasActivationHandler
 * (Sources/MetalHLOCore/Compiler/CustomCallHandlers.swift:927-1073).
 */
int mhlo_cuda_gemm(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[4],
                   const void* b_dev, const int64_t b_strides[4], void* c_dev, int64_t batch0, int64_t batch1,
                   int64_t m, int64_t n, int64_t k, const void* bias_dev, int32_t epilogue,
                   mhlo_cuda_stream_t stream);

/*
 * Launch knobs of the tensor-core GEMM (the CUDA counterpart of the tile fields of TuningConfig,
 * Sources/MetalHLOCore/Tuning/AutoTuner.swift:31-103). 0 leaves a knob to the library's heuristic.
 *   tile_n     columns of C per tile: 128 or 256 (rows are 128 per CTA)
 *   stages     depth of the TMA operand ring, 2 .. the kernel's maximum (4 for 128x256 tiles, 6 otherwise)
 *   cta_group  1: one CTA per 128-row tile; 2: a pair of CTAs on neighbouring SMs per 256 x 256 tile, each staging
 *              its own rows of A and its own half of B (tcgen05 cta_group::2; no load is multicast)
 * mhlo_cuda_gemm_tuned is mhlo_cuda_gemm with these knobs; tuning == NULL is mhlo_cuda_gemm. Problems outside the
 * tensor-core path ignore the knobs.
 */
typedef struct {
    int32_t tile_n;
    int32_t stages;
    int32_t cta_group;
    int32_t reserved;
} mhlo_cuda_gemm_tuning;

int mhlo_cuda_gemm_tuned(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[4],
                         const void* b_dev, const int64_t b_strides[4], void* c_dev, int64_t batch0, int64_t batch1,
                         int64_t m, int64_t n, int64_t k, const void* bias_dev, int32_t epilogue,
                         const mhlo_cuda_gemm_tuning* tuning, mhlo_cuda_stream_t stream);

/*
 * C = A . B + bias + R: the product with a residual matrix R of C's shape and type (dense, [batch0, batch1, m, n]) added
 * before the one rounding to the output type - the residual connection behind a projection, which would otherwise cost
 * a pass of its own over C. On the tensor-core path (16-bit operands and result, rows of C on the 16-byte grid) the
 * epilogue reads R tile by tile, under the tile's MMAs; other products run as mhlo_cuda_gemm_tuned followed by an elementwise sum. R may be C itself only on
 * that second path; pass distinct buffers. residual_dev NULL makes this mhlo_cuda_gemm_tuned without activation.
 * Stands where the reference's FusedOpType matmul is followed by an add of the residual stream (the reference has no
 * fused form: Compiler/PassManager.swift registers residual-chain-fusion without an implementation).
 */
int mhlo_cuda_gemm_residual(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[4],
                            const void* b_dev, const int64_t b_strides[4], void* c_dev, int64_t batch0, int64_t batch1,
                            int64_t m, int64_t n, int64_t k, const void* bias_dev, const void* residual_dev,
                            const mhlo_cuda_gemm_tuning* tuning, mhlo_cuda_stream_t stream);

/*
 * C = A . B for a B (and C) split by columns over n_ranks GPUs, with the all-gather of C fused into the epilogue:
 * this rank computes columns [rank * n_local, (rank + 1) * n_local) of the [m, n_local * n_ranks] row-major result
 * and every tile is stored, straight from the epilogue, into that column range of all n_ranks copies of C
 * (c_devs[r] = base of rank r's copy: c_devs[rank] is local memory, the others are peer addresses from
 * mhlo_cuda_ipc_open). Transfers over NVLink therefore overlap the tensor-core work tile by tile, and no separate
 * gather or interleave pass runs. A: [m, k], B: [k, n_local] (this rank's columns), strides {row, col} in elements.
 * When every rank's kernel has finished (a barrier across the ranks after a stream sync), every copy of C is complete.
 * bf16 / f16 operands on the tensor-core path only; n_ranks <= 8. The reference has no multi-device path; this
 * is the exchange step of the column-split GEMM.
 */
int mhlo_cuda_gemm_all_gather(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[2],
                              const void* b_dev, const int64_t b_strides[2], void* const* c_devs, int32_t n_ranks,
                              int32_t rank, int64_t m, int64_t n_local, int64_t k, const void* bias_dev,
                              int32_t epilogue, mhlo_cuda_stream_t stream);

/*
 * The same product with its launch knobs set by the caller. tuning: tile width and TMA ring depth as in
 * mhlo_cuda_gemm_tuned; NULL leaves them to the library.
 * copy_stores: 0 or 1 = every lane stores 16 bytes into each copy, 2 = one bulk tensor store (TMA, 32 rows x 128 bytes)
 * per copy from the staged tile (products without an activation; with one, the copies keep the lane stores). The
 * results are bit-identical in every setting.
 */
int mhlo_cuda_gemm_all_gather_tuned(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[2],
                                    const void* b_dev, const int64_t b_strides[2], void* const* c_devs, int32_t n_ranks,
                                    int32_t rank, int64_t m, int64_t n_local, int64_t k, const void* bias_dev,
                                    int32_t epilogue, const mhlo_cuda_gemm_tuning* tuning, int32_t copy_stores,
                                    mhlo_cuda_stream_t stream);

/*
 * Completion barrier between the ranks of such an exchange, on the device: flag_devs[r] = eight 64-bit words in rank
 * r's memory (flag_devs[rank] local, the others peer addresses), zero before the first use. In stream order after the
 * kernels whose stores it covers, one small kernel stores `epoch` into word `rank` of every other rank's array
 * (system-scope release) and waits until every word of its own array has reached `epoch`; work queued behind it on the
 * stream therefore sees every rank's stores. Epochs must grow from call to call. The wait gives up after limit_ns
 * (at most 2 s) and records code 95 in the word mhlo_cuda_device_error reads, leaving the context usable. Every rank
 * must run on its own GPU: kernels that wait on one another are not launched on one device. The reference has no
 * counterpart (single device).
 */
int mhlo_cuda_peer_barrier(void* const* flag_devs, int32_t n_ranks, int32_t rank, uint64_t epoch, uint64_t limit_ns,
                           mhlo_cuda_stream_t stream);

/*
 * Every wait inside the tensor-core kernels (mbarrier phases fed by TMA and tcgen05.commit) is bounded; a kernel
 * whose wait expires records a non-zero word and drains instead of spinning. This call synchronises the device,
 * reads and clears that word: *out_code = 0 when no kernel gave up since the last call.
 */
int mhlo_cuda_device_error(int32_t* out_code);

/*
 * The same check without a device-wide synchronisation, for the execution path: _fetch enqueues, on `stream`, copies
 * of the error words into pinned host memory of the current device; after the caller has synchronised that stream,
 * _take reads them, clears the device words when one is set and returns MHLO_CUDA_EXECUTION_FAILED with the code in
 * *out_code and in the error string. The reference's executor has no counterpart (a Metal command buffer reports its
 * own status, IntegratedExecutor.swift:262-268); mhlo_execute turns a non-zero code into MHLO_ERROR_EXECUTION_FAILED.
 */
int mhlo_cuda_device_error_fetch(mhlo_cuda_stream_t stream);
int mhlo_cuda_device_error_take(int32_t* out_code);

/*
 * Test hooks for that path; neither faults, traps or hangs the device. _store_device_error writes `code` into the
 * error word of the GEMM kernel (which = 0) or the attention kernel (which = 1) from the host. _wait_expiry_probe
 * launches one CTA that waits on an mbarrier nobody arrives at for at most limit_ns (<= 1 s) and then records code 90
 * exactly as the contraction kernels record an expired wait.
 */
int mhlo_cuda_debug_store_device_error(int32_t which, int32_t code);
/* Test hook of the allocator's failure path: the next `count` mhlo_cuda_alloc calls return MHLO_CUDA_BUFFER_FAILED
 * without reaching the driver (0 switches it off). */
int mhlo_cuda_debug_refuse_allocs(int32_t count);
int mhlo_cuda_debug_wait_expiry_probe(uint64_t limit_ns, mhlo_cuda_stream_t stream);

/*
 * Fused scaled dot-product attention, O = softmax(scale * Q K^T [+ mask] [causal]) V with fp32 softmax and
 * accumulation. Q [B,H,Sq,D], K/V [B,H,Sk,D], O [B,H,Sq,D] logically; *_strides = {batch, head, sequence}
 * element strides (the head dimension D is contiguous), so [B,S,H,D] tensors are read and written in place.
 * causal: key j is visible to query i iff j <= i, also when Sq != Sk (the `kv_pos > q_pos` cut of
 * FlashAttentionKernel.swift:545,578). mask_dev: optional additive [Sq,Sk] mask of the
 * operand dtype shared by every batch and head. Replaces kernel_attention (CodeGenerator.swift:4527-4595) and
 * flash_attention_tiled_kernel (Sources/MetalHLOCore/Metal/Kernels/FlashAttentionKernel.swift:469-670) with the
 * semantics of FusedScaledDotProductAttentionHandler (CustomCallHandlers.swift:179-278).
 */
int mhlo_cuda_attention(int32_t dtype, const void* q_dev, const int64_t q_strides[3], const void* k_dev,
                        const int64_t k_strides[3], const void* v_dev, const int64_t v_strides[3],
                        const void* mask_dev, void* o_dev, const int64_t o_strides[3], int64_t batch,
                        int64_t heads, int64_t seq_q, int64_t seq_k, int64_t head_dim, float scale,
                        int32_t causal, mhlo_cuda_stream_t stream);

/*
 * stablehlo.rng: `count` values of `dtype` between the scalars *a_dev and *b_dev. distribution 0 = UNIFORM (floats in
 * [a, b), integers in [a, b)), 1 = NORMAL (mean a, standard deviation b; floats only). state_dev: two 64-bit words
 * {key, counter} in device memory that the caller keeps for this operator; the draw reads the Threefry-2x32-20 stream
 * at the counter and a one-thread kernel queued behind it advances the counter, so every execution - a replayed graph
 * included - continues the stream. The operator has no state operand: its stream is implementation-defined, and the
 * reference draws from MPSGraph's generator (Compiler/MPSGraphCompiler.swift, compileRng).
 */
int mhlo_cuda_rng(int32_t dtype, int32_t distribution, void* state_dev, const void* a_dev, const void* b_dev, void* out_dev,
                  int64_t count, mhlo_cuda_stream_t stream);

/*
 * stablehlo.rng_bit_generator: `count` elements of elem_bytes (1, 2, 4 or 8) of random bits and the advanced state.
 * state_dev / new_state_dev: two 64-bit words {key, counter}. Word pair b of the stream is Threefry-2x32-20 of the key
 * (low word k0, high word k1) at counter + b (low word x0, high word x1); elements of up to 32 bits take the low bits of
 * one word each, 64-bit elements a whole pair (first word low); the new counter is counter + pairs used. One generator
 * serves every `algorithm` attribute: the bit streams of this operator are implementation-defined, and the reference
 * draws from MPSGraph's own generator without reading the state (Compiler/MPSGraphCompiler.swift:4250-4263).
 */
int mhlo_cuda_rng_bit_generator(const void* state_dev, void* new_state_dev, void* out_dev, int64_t count,
                                int32_t elem_bytes, mhlo_cuda_stream_t stream);

/* ---- dense factorisations and solves (jax.numpy.linalg) -----------------------------------------------------------
 * stablehlo.cholesky: a_dev holds `batch` symmetric positive-definite n x n matrices; out_dev receives the factor L
 * (lower != 0: A = L L^T, L lower triangular) or U (A = U^T U), the other triangle set to zero. A matrix that is not
 * positive definite gives NaN. out_dev must not alias a_dev.
 * stablehlo.triangular_solve: solves op(a) X = b (left_side != 0; b and X are [batch, m, n]) or X op(a) = b (b and X are
 * [batch, n, m]) for the m x m triangular matrices a (`lower` says which triangle is read; the other is ignored),
 * op = identity, or transpose when transpose_a != 0; unit_diagonal != 0 takes the diagonal as ones.
 * f32 / f16 / bf16 compute in fp32, f64 in fp64. Correctness kernels, O(n^3) on one CTA per matrix; the reference lowers
 * both operators through MPSGraph (Sources/MetalHLOCore/Compiler/MPSGraphCompiler.swift). */
int mhlo_cuda_cholesky(int32_t dtype, const void* a_dev, void* out_dev, int64_t batch, int64_t n, int32_t lower,
                       mhlo_cuda_stream_t stream);
int mhlo_cuda_triangular_solve(int32_t dtype, const void* a_dev, const void* b_dev, void* out_dev, int64_t batch, int64_t m,
                               int64_t n, int32_t left_side, int32_t lower, int32_t unit_diagonal, int32_t transpose_a,
                               mhlo_cuda_stream_t stream);

/* ---- stablehlo.fft -------------------------------------------------------------------------------------------------
 * One pass of a discrete Fourier transform along one axis. Complex tensors are (re, im) pairs of f32 or f64 (dtype is the
 * part type), the layout the reference's FFT kernels read and write on float tensors
 * (Sources/MetalHLOCore/Compiler/CodeGenerator.swift:2701-2830). kind 0 = forward and 1 = inverse (scaled by 1/n) between
 * complex tensors [outer, n, inner]; these may run in place (out_dev == in_dev). kind 2 = real [outer, n] to the
 * n/2 + 1 leading bins [outer, n/2 + 1]; kind 3 = those bins back to the real line, scaled by 1/n (inner must be 1 for
 * both; not in place). A transform over several axes is one call per axis. n is bounded by the shared memory a line
 * needs (status MHLO_CUDA_UNSUPPORTED beyond it): powers of two up to 8192 points in f32 take a radix-2 Stockham FFT, every
 * other length up to 14 000 the direct sum the reference uses for all lengths; half of either in f64. */
int mhlo_cuda_fft_axis(int32_t dtype, int32_t kind, const void* in_dev, void* out_dev, int64_t outer, int64_t n, int64_t inner,
                       mhlo_cuda_stream_t stream);
/* Lines longer than that, powers of two up to 2^24 points: the same passes, one launch each, between two scratch buffers
 * in global memory. mhlo_cuda_fft_axis_scratch_bytes gives the scratch a call needs (0: the line fits shared memory, or its
 * length is not a power of two); mhlo_cuda_fft_axis_long takes it and is mhlo_cuda_fft_axis where none is needed. In place
 * (out_dev == in_dev) is allowed for kinds 0 and 1. */
int64_t mhlo_cuda_fft_axis_scratch_bytes(int32_t dtype, int64_t outer, int64_t n, int64_t inner);
int mhlo_cuda_fft_axis_long(int32_t dtype, int32_t kind, const void* in_dev, void* out_dev, void* scratch_dev, int64_t outer, int64_t n,
                            int64_t inner, mhlo_cuda_stream_t stream);

/* ---- dispatch plans ----------------------------------------------------------------------------------------------
 * The surface a host-side executor binds instead of MTLComputePipelineState / MTLBuffer / compute encoders
 * (MetalHLOCompiler.compileKernel, Sources/MetalHLOCore/Compiler/MetalHLOCompiler.swift:329-401; IntegratedExecutor,
 * Runtime/IntegratedExecutor.swift:106-270,390-615). A plan is a list of ops; each names an ahead-of-time kernel of this
 * library and says where its buffers come from - BufferBinding / BufferSource (Compiler/KernelTypes.swift:77-143) - and
 * its extents, scalars and launch knobs - the role of DispatchConfig (:12-62).
 */
enum { MHLO_CUDA_SRC_NONE = 0, MHLO_CUDA_SRC_INPUT = 1, MHLO_CUDA_SRC_OUTPUT = 2, MHLO_CUDA_SRC_UNIFIED = 3, MHLO_CUDA_SRC_CONSTANT = 4 };
typedef struct {
    int32_t source; /* MHLO_CUDA_SRC_*: function input / output number `index`, or `offset` bytes into the plan's arena
                       (UNIFIED) or constant pool (CONSTANT); NONE = the kernel's optional argument is absent */
    int32_t index;
    int64_t offset; /* bytes, added to the input / output pointer as well */
} mhlo_cuda_binding;

enum {
    MHLO_CUDA_KERNEL_LAYER_NORM = 1, /* args x, gamma, beta, y; dims rows, hidden; scalars eps; tuning threads, vectors, ctas */
    MHLO_CUDA_KERNEL_RMS_NORM = 2,   /* args x, gamma, y; dims rows, hidden; scalars eps */
    MHLO_CUDA_KERNEL_SOFTMAX = 3,    /* args x, y; dims outer, axis_len, inner */
    MHLO_CUDA_KERNEL_GEMM = 4,       /* args a, b, bias, c; dims batch0, batch1, m, n, k; strides a[4], b[4]; flags epilogue;
                                        tuning tile_n, stages, cta_group */
    MHLO_CUDA_KERNEL_ATTENTION = 5,  /* args q, k, v, mask, o; dims batch, heads, seq_q, seq_k, head_dim; strides q[3], k[3],
                                        v[3], o[3]; scalars scale; flags causal; tuning tile_order */
    MHLO_CUDA_KERNEL_GELU = 6,       /* args x, y; dims count (tanh approximation) */
    MHLO_CUDA_KERNEL_SILU = 7        /* args x, y; dims count */
};
typedef struct {
    int32_t kernel; /* MHLO_CUDA_KERNEL_*, e.g. from mhlo_cuda_kernel_lookup */
    int32_t dtype, out_dtype;
    mhlo_cuda_binding args[6];
    int64_t dims[6];
    int64_t strides[16];
    float scalars[2];
    int32_t flags[2];
    int32_t tuning[4];
} mhlo_cuda_plan_op;
typedef void* mhlo_cuda_plan_t;

/* Kernel of a fused-op name as the pass pipeline emits it ("fused_layer_norm", "fused_rms_norm", "fused_softmax",
 * "fused_gelu", "fused_silu", "fused_matmul_bias_activation", "dot_general", "fused_scaled_dot_product_attention"):
 * FusedOp.fusedOpTypeFromCustomCall (Compiler/IntegrationTypes.swift:471-600) on the CUDA side. MHLO_CUDA_UNSUPPORTED
 * when the library has no such kernel for the dtype. */
int mhlo_cuda_kernel_lookup(const char* fused_op_kind, int32_t dtype, int32_t* out_kernel);
/* Validates the ops, allocates the arena and uploads the constant pool (either may be empty). The caller owns the plan. */
int mhlo_cuda_plan_create(const mhlo_cuda_plan_op* ops, int32_t n_ops, int32_t n_inputs, int32_t n_outputs, int64_t arena_bytes,
                          const void* constants_host, int64_t constant_bytes, mhlo_cuda_plan_t* out_plan);
/* Enqueues every op in order on `stream`; inputs / outputs are device pointers. No allocation, no synchronisation. */
int mhlo_cuda_plan_execute(mhlo_cuda_plan_t plan, const void* const* inputs, int32_t n_inputs, void* const* outputs, int32_t n_outputs,
                           mhlo_cuda_stream_t stream);
int mhlo_cuda_plan_destroy(mhlo_cuda_plan_t plan);
/* Median device time of one execution of the plan on the default stream (warmup untimed + iterations timed launches, CUDA
 * events): the measurement step of the tuner (Tuning/AutoTuner.swift:479-513) for a caller that builds its own candidates. */
int mhlo_cuda_tuner_measure(mhlo_cuda_plan_t plan, const void* const* inputs, int32_t n_inputs, void* const* outputs, int32_t n_outputs,
                            int32_t warmup, int32_t iterations, float* out_median_ms);

/* ---- communicator over the GPUs of one process -----------------------------------------------------------------------
 * The reference has no multi-device path. mhlo_cuda_comm_init(n) joins devices 0 .. n-1 (peer access both ways, one
 * stream each); mhlo_cuda_all_gather exchanges equal shards: buffers[d] is device d's buffer of n * shard_bytes bytes
 * whose d-th shard is filled, and on return every buffer holds all n shards. Every device pushes its shard into its
 * peers' buffers with one kernel of its own over NVLink peer memory (plain 16-byte stores; no library collective). The
 * call returns when all devices have finished. */
typedef void* mhlo_cuda_comm_t;
int mhlo_cuda_comm_init(int32_t n_devices, mhlo_cuda_comm_t* out_comm);
int mhlo_cuda_comm_size(mhlo_cuda_comm_t comm);
int mhlo_cuda_all_gather(mhlo_cuda_comm_t comm, void* const* buffers, int64_t shard_bytes);
int mhlo_cuda_comm_destroy(mhlo_cuda_comm_t comm);

/*
 * Launch knobs of the tensor-core attention kernel (the attention block options of the reference's tuner,
 * Sources/MetalHLOCore/Tuning/AutoTuner.swift:81-103). 0 leaves a knob to the library.
 *   tile_order  order in which the persistent CTAs take the 256-query-row tiles: 1 = long and short tiles of one
 *               (batch, head) in pairs, neighbouring CTAs on neighbouring heads (K and V are read from HBM once);
 *               2 = longest tiles first, dealt to the CTAs forwards and backwards (balances a causal mask best, costs
 *               re-reads when K and V of all heads do not fit L2)
 * mhlo_cuda_attention_tuned is mhlo_cuda_attention with these knobs; tuning == NULL is mhlo_cuda_attention.
 */
typedef struct {
    int32_t tile_order;
    int32_t reserved[3];
} mhlo_cuda_attention_tuning;

int mhlo_cuda_attention_tuned(int32_t dtype, const void* q_dev, const int64_t q_strides[3], const void* k_dev,
                              const int64_t k_strides[3], const void* v_dev, const int64_t v_strides[3],
                              const void* mask_dev, void* o_dev, const int64_t o_strides[3], int64_t batch,
                              int64_t heads, int64_t seq_q, int64_t seq_k, int64_t head_dim, float scale,
                              int32_t causal, const mhlo_cuda_attention_tuning* tuning, mhlo_cuda_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MHLO_CUDA_H */
