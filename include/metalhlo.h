/*
 * metalhlo.h — the MetalHLO C API as served by the B200 backend (libCMetalHLO.so).
 *
 * Every name, enum value, struct layout and calling convention below is that of the reference's C API
 * (Sources/CMetalHLO/include/metalhlo.h:23-397, implemented in Sources/CMetalHLO/CInterface.swift:202-1010),
 * so a C or C++ host written against MetalHLO links against this library unchanged. What differs is what runs
 * underneath: StableHLO text is compiled by the C++ compiler core and executed by hand-written sm_100a CUDA
 * kernels. There is no CPU fallback; without a CUDA device mhlo_client_create returns MHLO_ERROR_NO_DEVICE.
 *
 * Ownership: handles are opaque pointers. Whoever receives a handle from *_create, mhlo_compile* or
 * mhlo_execute* destroys it with the matching *_destroy. Strings from mhlo_client_device_name are heap copies
 * released with mhlo_free_string; mhlo_version and mhlo_get_last_error return library-owned storage.
 * Errors: functions return an MHLOStatusCode; the message of the most recent failure (process-global, as in the
 * reference, CInterface.swift:116-126) is read with mhlo_get_last_error. Calls are synchronous. A handle must
 * not be used from two threads at once.
 */
#ifndef METALHLO_H
#define METALHLO_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* MHLOClientRef;
typedef void* MHLOExecutableRef;
typedef void* MHLOBufferRef;

/* reference: metalhlo.h:37-49 */
typedef enum {
    MHLO_OK = 0,
    MHLO_ERROR_NO_DEVICE = 1,
    MHLO_ERROR_UNSUPPORTED_DEVICE = 2,
    MHLO_ERROR_PARSE_FAILED = 3,
    MHLO_ERROR_UNSUPPORTED_OP = 4,
    MHLO_ERROR_COMPILATION_FAILED = 5,
    MHLO_ERROR_BUFFER_FAILED = 6,
    MHLO_ERROR_INPUT_MISMATCH = 7,
    MHLO_ERROR_EXECUTION_FAILED = 8,
    MHLO_ERROR_TRANSFER_FAILED = 9,
    MHLO_ERROR_INVALID_ARGUMENT = 10,
} MHLOStatusCode;

/* reference: metalhlo.h:61-75 */
typedef enum {
    MHLO_F16 = 0, MHLO_F32 = 1, MHLO_F64 = 2, MHLO_BF16 = 3, MHLO_I1 = 4, MHLO_I8 = 5, MHLO_I16 = 6,
    MHLO_I32 = 7, MHLO_I64 = 8, MHLO_UI8 = 9, MHLO_UI16 = 10, MHLO_UI32 = 11, MHLO_UI64 = 12,
} MHLOElementType;

/* reference: metalhlo.h:102-107 */
typedef enum { MHLO_OPT_O0 = 0, MHLO_OPT_O1 = 1, MHLO_OPT_O2 = 2, MHLO_OPT_O3 = 3 } MHLOOptimizationLevel;

/* reference: metalhlo.h:110-116. Accepted for compatibility; every policy runs on the CUDA device. */
typedef enum {
    MHLO_DEVICE_GPU_ONLY = 0, MHLO_DEVICE_ANE_ONLY = 1, MHLO_DEVICE_AUTO = 2, MHLO_DEVICE_PREFER_ANE = 3,
    MHLO_DEVICE_PREFER_GPU = 4,
} MHLODevicePolicy;

/* reference: metalhlo.h:119-128 */
typedef struct {
    MHLOOptimizationLevel optimization_level; /* default MHLO_OPT_O2 */
    bool enable_caching;                      /* default true: identical text + config reuses the compiled program */
    bool enable_debug_info;                   /* default false */
    MHLODevicePolicy device_policy;           /* default MHLO_DEVICE_GPU_ONLY */
} MHLOCompileConfig;

/* reference: metalhlo.h:221-230 */
typedef struct {
    int64_t execution_count;
    double total_execution_time_ms;
    double last_execution_time_ms;
    double average_execution_time_ms;
} MHLOExecutionStats;

/* reference: metalhlo.h:351-368. The ANE fields are always zero / false here. */
typedef struct {
    int32_t partition_count;
    int32_t gpu_partition_count;
    int32_t ane_partition_count;
    double gpu_time_ms;
    double ane_time_ms;
    double transfer_time_ms;
    double total_time_ms;
    bool used_ane;
} MHLOExecutionProfile;

/* ---- library (reference: metalhlo.h:23, 53-56, 78, 397) ---- */
const char* mhlo_version(void);
const char* mhlo_get_last_error(void);
void mhlo_clear_error(void);
size_t mhlo_element_type_size(MHLOElementType type); /* 0 for I1, as in the reference */
void mhlo_free_string(const char* str);

/* ---- client (reference: metalhlo.h:87-95) ---- */
MHLOStatusCode mhlo_client_create(MHLOClientRef* out_client);
void mhlo_client_destroy(MHLOClientRef client);
char* mhlo_client_device_name(MHLOClientRef client);

/* ---- compilation (reference: metalhlo.h:132-177) ---- */
void mhlo_compile_config_init(MHLOCompileConfig* out_config);
bool mhlo_ane_available(void); /* always false on this backend */
MHLOStatusCode mhlo_compile(MHLOClientRef client, const char* mlir_text, MHLOExecutableRef* out_executable);
MHLOStatusCode mhlo_compile_n(MHLOClientRef client, const char* mlir_text, size_t mlir_length,
                              MHLOExecutableRef* out_executable);
MHLOStatusCode mhlo_compile_with_config(MHLOClientRef client, const char* mlir_text,
                                        const MHLOCompileConfig* config, MHLOExecutableRef* out_executable);

/* ---- executable (reference: metalhlo.h:180-243) ---- */
void mhlo_executable_destroy(MHLOExecutableRef executable);
int32_t mhlo_executable_input_count(MHLOExecutableRef executable);
int32_t mhlo_executable_output_count(MHLOExecutableRef executable);
/* out_shape (room for the rank), out_rank and out_element_type may each be NULL. */
MHLOStatusCode mhlo_executable_input_type(MHLOExecutableRef executable, int32_t index, int64_t* out_shape,
                                          int32_t* out_rank, MHLOElementType* out_element_type);
MHLOStatusCode mhlo_executable_output_type(MHLOExecutableRef executable, int32_t index, int64_t* out_shape,
                                           int32_t* out_rank, MHLOElementType* out_element_type);
MHLOStatusCode mhlo_executable_get_stats(MHLOExecutableRef executable, MHLOExecutionStats* out_stats);
void mhlo_executable_reset_stats(MHLOExecutableRef executable);

/* ---- buffers (reference: metalhlo.h:260-310) ---- */
MHLOStatusCode mhlo_buffer_create(MHLOClientRef client, const void* data, size_t data_size, const int64_t* shape,
                                  int32_t rank, MHLOElementType element_type, MHLOBufferRef* out_buffer);
MHLOStatusCode mhlo_buffer_create_uninitialized(MHLOClientRef client, const int64_t* shape, int32_t rank,
                                                MHLOElementType element_type, MHLOBufferRef* out_buffer);
void mhlo_buffer_destroy(MHLOBufferRef buffer);
void mhlo_buffer_shape(MHLOBufferRef buffer, int64_t* out_shape, int32_t* out_rank);
int32_t mhlo_buffer_rank(MHLOBufferRef buffer);
MHLOElementType mhlo_buffer_element_type(MHLOBufferRef buffer);
size_t mhlo_buffer_byte_count(MHLOBufferRef buffer);
MHLOStatusCode mhlo_buffer_to_host(MHLOBufferRef buffer, void* out_data, size_t data_size);

/* ---- execution (reference: metalhlo.h:325-388) ----
 * out_outputs must have room for mhlo_executable_output_count handles; each is a new buffer owned by the caller.
 * The *_with_timing variant reports seconds: encode = host time spent enqueueing, gpu = device time between CUDA
 * events around the program, total = wall clock of the call. */
MHLOStatusCode mhlo_execute(MHLOExecutableRef executable, const MHLOBufferRef* inputs, int32_t num_inputs,
                            MHLOBufferRef* out_outputs, int32_t* out_num_outputs);
MHLOStatusCode mhlo_execute_with_timing(MHLOExecutableRef executable, const MHLOBufferRef* inputs,
                                        int32_t num_inputs, MHLOBufferRef* out_outputs, int32_t* out_num_outputs,
                                        double* out_encode_time, double* out_gpu_time, double* out_total_time);
MHLOStatusCode mhlo_execute_with_profile(MHLOExecutableRef executable, const MHLOBufferRef* inputs,
                                         int32_t num_inputs, MHLOBufferRef* out_outputs, int32_t* out_num_outputs,
                                         MHLOExecutionProfile* out_profile);

/* ---- additions of this backend (no counterpart in the reference's header) ----
 * Introspection for tests and benchmarks, and execution on device memory the caller already owns. */
/* Host-only (no CUDA device needed): parse, run the pass pipeline of the given level, return the module text
 * (free with mhlo_free_string). */
MHLOStatusCode mhlo_b200_optimize_text(const char* mlir_text, int32_t optimization_level, char** out_text);
/* Host-only: lowers the module to the executor's step list without touching a device. *out_steps = one step label
 * per line (free with mhlo_free_string); out_launches / out_arena_bytes may be NULL. */
MHLOStatusCode mhlo_b200_plan_text(const char* mlir_text, int32_t optimization_level, char** out_steps,
                                   int32_t* out_launches, int64_t* out_arena_bytes);
/* MLIR bytecode (magic "ML\xEFR": the VHLO portable artifact JAX hands a plugin) -> StableHLO text. No bytecode reader
 * is linked; as in the reference (Sources/PJRTMetalHLO/PJRTExecutable.swift:23-239) the interpreter named by
 * METALHLO_PYTHON runs a jaxlib helper script (METALHLO_BYTECODE_HELPER; default jax_plugins/metalhlo/bytecode_to_text.py
 * of this package) with the bytecode on stdin and prints the text; METALHLO_HELPER_TIMEOUT_S bounds it. *out_text is
 * malloc'd (mhlo_free_string). mhlo_compile_n and the PJRT plugin convert bytecode programs the same way. */
MHLOStatusCode mhlo_b200_bytecode_to_text(const void* bytecode, size_t size, char** out_text);
/* CUDA devices visible to this process, and a client bound to one of them (mhlo_client_create takes METALHLO_DEVICE /
 * LOCAL_RANK, else device 0). A process may hold one client per GPU; the PJRT plugin does so when it exposes several
 * devices. The reference has one Metal device per client (Sources/MetalHLO/Client.swift). */
int32_t mhlo_b200_device_count(void);
MHLOStatusCode mhlo_b200_client_create_on_device(int32_t device_ordinal, MHLOClientRef* out_client);
/*
 * Batch sharding. The reference runs every program on one device (Sources/PJRTMetalHLO/PJRTExecutable.swift:1830-1848
 * fixes num_replicas = num_partitions = 1 and :2033-2036 refuses several devices). Here a program whose results are,
 * slice by slice along one axis, functions of the same slice of its batched arguments is split into shard_count equal
 * shards with no exchange on the data path; each GPU (one process per GPU, or one PJRT device each) compiles and runs
 * one shard. The proof is a propagation of the split axis through every operator; a program that mixes elements along
 * the split axis (a reduction, contraction, sort, window or gather over it) is refused with
 * MHLO_ERROR_UNSUPPORTED_OP and the operator's name.
 *   mhlo_b200_compile_sharded    compiles shard shard_index. input_axes (one per argument: split axis, or -1 for a
 *                                replicated argument) may be NULL: then every argument whose leading extent equals the
 *                                first argument's is split along axis 0. The executable's types are one shard's.
 *   mhlo_b200_executable_sharding  count, index and the split axis of each argument / result (-1: replicated).
 *   mhlo_b200_shard_text         host-only: the rewritten function as text (free with mhlo_free_string).
 * A client created with METALHLO_SHARD_COUNT / METALHLO_SHARD_INDEX in the environment applies the same split to every
 * mhlo_compile* call.
 */
MHLOStatusCode mhlo_b200_compile_sharded(MHLOClientRef client, const char* mlir_text, const MHLOCompileConfig* config,
                                         int32_t shard_count, int32_t shard_index, const int32_t* input_axes,
                                         int32_t num_input_axes, MHLOExecutableRef* out_executable);
MHLOStatusCode mhlo_b200_executable_sharding(MHLOExecutableRef executable, int32_t* out_count, int32_t* out_index,
                                             int32_t* out_input_axes, int32_t* out_output_axes);
MHLOStatusCode mhlo_b200_shard_text(const char* mlir_text, int32_t shard_count, int32_t shard_index,
                                    const int32_t* input_axes, int32_t num_input_axes, char** out_text,
                                    int32_t* out_input_axes, int32_t* out_output_axes);
/* Host-only views of the static memory planner (Sources/MetalHLOCore/Memory/StaticMemoryPlanner.swift:175-253): the
 * planner alone on n buffers (sizes, inclusive live ranges in steps -> 256-byte aligned arena offsets and the arena size
 * rounded to 4096), and the plan of a module as lines "bytes first last offset" (free with mhlo_free_string). */
MHLOStatusCode mhlo_b200_plan_intervals(const int64_t* bytes, const int32_t* first, const int32_t* last, int32_t n,
                                        int64_t* out_offsets, int64_t* out_total);
MHLOStatusCode mhlo_b200_plan_memory_text(const char* mlir_text, int32_t optimization_level, char** out_lines,
                                          int64_t* out_arena_bytes);
/* StableHLO text after the pass pipeline; free with mhlo_free_string. */
char* mhlo_b200_executable_optimized_text(MHLOExecutableRef executable);
/* Kernel launches one execution enqueues. */
int32_t mhlo_b200_executable_launch_count(MHLOExecutableRef executable);
/* Bytes of the statically planned arena that holds every intermediate. */
int64_t mhlo_b200_executable_arena_bytes(MHLOExecutableRef executable);
/* Executions of this program that were served by replaying a recorded CUDA graph. A program is recorded when it runs a
 * second time on the same stream with the same input and output addresses (mhlo_b200_execute_on_device with buffers
 * the caller keeps); METALHLO_CUDA_GRAPH=0 turns recording off. */
int64_t mhlo_b200_executable_graph_replays(MHLOExecutableRef executable);
/* Newline-separated labels of the launch list; free with mhlo_free_string. */
char* mhlo_b200_executable_steps(MHLOExecutableRef executable);
/* Device address of a buffer's storage (dense row-major). */
void* mhlo_b200_buffer_device_pointer(MHLOBufferRef buffer);

/* Complex tensors. MHLOElementType has no complex entry (Sources/CMetalHLO/include/metalhlo.h:61-75): a parameter or
 * result typed tensor<..xcomplex<f32|f64>> in the program is a float buffer of (re, im) pairs with one more dimension of
 * extent 2, and that is the shape and type the functions above report for it. These two tell a host with a complex buffer
 * type of its own (PJRT's C64 / C128) which ones they are: 1 complex, 0 not, -1 index out of range. */
int32_t mhlo_b200_executable_input_is_complex(MHLOExecutableRef executable, int32_t index);
int32_t mhlo_b200_executable_output_is_complex(MHLOExecutableRef executable, int32_t index);

/*
 * mhlo_buffer_to_host without the wait: the copy is queued on the client's transfer stream behind everything already
 * queued on its compute stream, and done(user) runs on a driver thread when the bytes are in out_data (pinned memory for
 * the copy to run beside the next program). done must not call into this library. The buffer may be destroyed at any
 * time afterwards: destruction waits for transfers out of it. An extension: the reference's buffers copy synchronously
 * (Sources/MetalHLO/CAPI: mhlo_buffer_to_host).
 */
MHLOStatusCode mhlo_b200_buffer_to_host_async(MHLOBufferRef buffer, void* out_data, size_t data_size, void (*done)(void*), void* user);
/* Enqueues the program on `stream` (a cudaStream_t) reading/writing caller-owned dense device tensors of the
 * executable's declared types. Does not synchronise; the only device allocations are stream-ordered scratch of split
 * reductions. On a non-default stream, repeated calls with the same addresses replay a recorded CUDA graph. */
MHLOStatusCode mhlo_b200_execute_on_device(MHLOExecutableRef executable, const void* const* input_ptrs,
                                           void* const* output_ptrs, void* stream);


/* ---- kernel tuning (reference: Sources/MetalHLOCore/Tuning/TuningDatabase.swift:15-290, AutoTuner.swift:225-764;
 * the reference exposes these only to Swift callers). One database per process, opened from `path` (or from
 * $METALHLO_TUNING_DB on first use). Executables compiled afterwards look their fused LayerNorm / RMSNorm / softmax
 * launches up in it by (operation, shape, dtype, device name) and fall back to the library's heuristics. */
/* Opens (and loads, when the file exists) the process database. NULL path: $METALHLO_TUNING_DB. */
MHLOStatusCode mhlo_b200_tuning_open(const char* path);
/* Entries currently held; -1 when no database is open. */
int64_t mhlo_b200_tuning_count(void);
/* Measures every candidate launch configuration of a row kernel on the client's device (5 warm-up + 20 timed
 * launches each, median) and stores the best. kernel: "fused_layer_norm" | "fused_rms_norm" | "fused_softmax".
 * max_trials <= 0: all candidates. *out_record_json (optional) receives the stored record; free with mhlo_free_string. */
MHLOStatusCode mhlo_b200_tuning_tune_row_kernel(MHLOClientRef client, const char* kernel, MHLOElementType element_type,
                                                int64_t rows, int64_t hidden, int32_t max_trials, char** out_record_json);
/* The same for the tensor-core GEMM, over {tile width 128 | 256, TMA ring depth, one CTA per tile | a pair of CTAs per
 * 256 x 256 tile} (the tile knobs of Sources/MetalHLOCore/Tuning/AutoTuner.swift:31-103 on this hardware), for
 * [batch, m, k] . [batch, k, n] of bf16 / f16 operands; a_transposed / b_transposed: the operand is stored with its
 * other dimension contiguous. The record is stored under the key the compiler looks up when it lowers the same
 * dot_general or fused_matmul_bias_activation; executables compiled afterwards launch the stored configuration. */
MHLOStatusCode mhlo_b200_tuning_tune_gemm(MHLOClientRef client, MHLOElementType element_type, MHLOElementType out_element_type,
                                          int64_t batch, int64_t m, int64_t n, int64_t k, bool a_transposed, bool b_transposed,
                                          int32_t max_trials, char** out_record_json);
/* The same for the tensor-core attention kernel (head_dim 64 or 128, bf16 / f16) over its tile orders
 * (AutoTuner.swift:81-103: the attention block options). bshd: tensors laid out [batch, sequence, heads, head_dim]. */
MHLOStatusCode mhlo_b200_tuning_tune_attention(MHLOClientRef client, MHLOElementType element_type, int64_t batch, int64_t heads,
                                               int64_t seq_q, int64_t seq_k, int64_t head_dim, bool causal, bool bshd,
                                               int32_t max_trials, char** out_record_json);
/* Merges records given as a database document (the file format: {"version": 1, "entries": [key, result, ...]});
 * existing keys win unless overwrite. Host-only. *out_taken (optional) = entries taken. */
MHLOStatusCode mhlo_b200_tuning_merge_json(const char* database_json, bool overwrite, int32_t* out_taken);
/* The whole database as JSON text (the file format); free with mhlo_free_string. NULL when none is open. */
char* mhlo_b200_tuning_to_json(void);
/* Writes the file if anything changed. */
MHLOStatusCode mhlo_b200_tuning_save(void);
/* Merges another database file (existing keys win unless overwrite); *out_taken (optional) = entries taken. */
MHLOStatusCode mhlo_b200_tuning_import(const char* other_path, bool overwrite, int32_t* out_taken);
/* Drops entries older than max_age_days; returns how many, -1 when no database is open. */
int32_t mhlo_b200_tuning_prune(double max_age_days);
/* Forgets every entry (the file changes on the next save). */
void mhlo_b200_tuning_clear(void);

#ifdef __cplusplus
}
#endif
#endif /* METALHLO_H */
