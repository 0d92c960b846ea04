/*
 * pjrt_host.h — C ABI of libpjrt_host.so, a minimal PJRT *host*.
 *
 * It loads a PJRT plugin by path, takes its table from GetPjrtApi and drives it through the PJRT C API only
 * (PJRT_Plugin_Initialize, PJRT_Client_Create, PJRT_Client_BufferFromHostBuffer, PJRT_Client_Compile with a serialized
 * CompileOptionsProto, PJRT_LoadedExecutable_Execute over one or several devices, PJRT_Buffer_ToHostBuffer) — the calls
 * XLA / JAX make and the reference's plugin tests exercise (Tests/PJRTMetalHLOTests/PJRTPluginTests.swift:160-467).
 * It exists so that the parity tests and the benchmark reach pjrt_plugin_metalhlo_b200.so the way a framework does,
 * without jaxlib. Every function returns 0 on success; pjrt_host_last_error() gives the message otherwise.
 */
#ifndef PJRT_HOST_H_
#define PJRT_HOST_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* pjrt_host_last_error(void);

/* dlopen + GetPjrtApi + Plugin_Initialize + Client_Create; *out_host owns the client. */
int pjrt_host_open(const char* plugin_path, void** out_host);
void pjrt_host_close(void* host);
int pjrt_host_api_version(void* host, int* major, int* minor);
int pjrt_host_platform_name(void* host, char* out, size_t cap);

/* Addressable devices of the client, in the client's order, and their PJRT ids. */
int pjrt_host_device_count(void* host);
int pjrt_host_device_id(void* host, int index, int64_t* out_id);

/* Dense row-major host array -> buffer on addressable device `device_index`; `type` is a PJRT_Buffer_Type value. */
int pjrt_host_buffer_from_host(void* host, const void* data, int type, const int64_t* dims, int rank, int device_index,
                               void** out_buffer);
/* Element type, dimensions (up to 8) and host size of a buffer; any output may be NULL. */
int pjrt_host_buffer_describe(void* host, void* buffer, int* out_type, int64_t* out_dims, int* out_rank, size_t* out_bytes);
int pjrt_host_buffer_to_host(void* host, void* buffer, void* dst, size_t bytes);
/* The same in two halves: PJRT_Buffer_ToHostBuffer now, PJRT_Event_Await (which also destroys the event) later, so that
 * the caller can execute the next program while the bytes travel. */
int pjrt_host_buffer_to_host_start(void* host, void* buffer, void* dst, size_t bytes, void** out_event);
int pjrt_host_event_await(void* host, void* event);
void pjrt_host_buffer_destroy(void* host, void* buffer);

/*
 * Compiles `program` (format "mlir": StableHLO text or MLIR bytecode) for num_replicas x num_partitions devices;
 * device_ids (replica-major, may be NULL) becomes the DeviceAssignmentProto of the compile options. num_replicas = 0
 * sends no compile options at all.
 */
int pjrt_host_compile(void* host, const char* program, size_t size, int num_replicas, int num_partitions, const int64_t* device_ids,
                      void** out_executable);
int pjrt_host_executable_num_outputs(void* executable);
int pjrt_host_executable_num_devices(void* executable);
void pjrt_host_executable_destroy(void* host, void* executable);

/*
 * One PJRT_LoadedExecutable_Execute over num_devices devices: args = [num_devices][num_args] buffers,
 * outs = [num_devices][num_outputs] (filled in). Returns after every device's completion event is ready.
 */
int pjrt_host_execute(void* host, void* executable, void* const* args, int num_devices, int num_args, void** outs);

#ifdef __cplusplus
}
#endif
#endif /* PJRT_HOST_H_ */
