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

/* Device-side timing (replaces MTLCommandBuffer GPUStartTime/GPUEndTime, Executable.swift:164). */
int mhlo_cuda_event_create(void** out_event);
int mhlo_cuda_event_destroy(void* event);
int mhlo_cuda_event_record(void* event, mhlo_cuda_stream_t stream);
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
 * Softmax along one axis of a tensor viewed as [outer, axis_len, inner] (inner = 1 for the last axis):
 * y = exp(x - max) / sum(exp(x - max)). Replaces kernel_softmax (CodeGenerator.swift:4690-4794) and
 * softmax_kernel(_half) (Sources/MetalHLOCore/Metal/Kernels/SoftmaxKernel.swift:23-167), semantics of
 * FusedSoftmaxHandler (CustomCallHandlers.swift:644-672).
 */
int mhlo_cuda_softmax(int dtype, const void* x_dev, void* y_dev, int64_t outer, int64_t axis_len,
                      int64_t inner, const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MHLO_CUDA_H */
