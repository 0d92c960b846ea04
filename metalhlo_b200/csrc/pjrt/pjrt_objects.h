// Object model of the PJRT plugin: the concrete structs behind PJRT's opaque handles.
//
// The plugin is a thin layer over the mhlo_* C API (include/metalhlo.h): a PJRT client owns one MHLOClientRef, a
// loaded executable one MHLOExecutableRef, a buffer one MHLOBufferRef. It mirrors the reference plugin
// (Sources/PJRTMetalHLO/*.swift): one device, one memory space named "device", synchronous transfers and execution
// whose events are complete when they are returned.
//
// pjrt_c_api.h is the OpenXLA header (PJRT C API 0.90). It is not part of this repository; the build takes its
// directory from PJRT_INCLUDE.
#pragma once

#include <atomic>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <condition_variable>
#include <mutex>
#include <string>
#include <vector>

#include "metalhlo.h"
#include "pjrt_c_api.h"

struct PJRT_Error {
    PJRT_Error_Code code;
    std::string message;
};

// Events are reference counted because a buffer keeps its ready event while every PJRT_Buffer_ReadyEvent caller
// receives a handle it must destroy (PJRTEvent.swift:14-100).
struct PJRT_Event {
    std::mutex mu;
    std::condition_variable cv;  // signalled when a pending event becomes ready
    bool ready = true;
    std::unique_ptr<PJRT_Error> error;  // set when the awaited work failed
    std::vector<std::pair<PJRT_Event_OnReadyCallback, void*>> callbacks;
    std::atomic<int> refs{1};
};

struct PJRT_DeviceDescription {
    int id = 0;
    int process_index = 0;
    std::string kind, debug_string, to_string;
    // attribute storage: names/strings are kept alive by the vectors below
    std::vector<std::string> attr_names, attr_strings;
    std::vector<PJRT_NamedValue> attributes;
};

struct PJRT_Memory {
    int id = 0;
    int kind_id = 0;
    std::string kind, debug_string, to_string;
    std::vector<PJRT_Device*> devices;
};

struct PJRT_Device {
    PJRT_Client* client = nullptr;
    int index = 0;                 // position among the client's devices = PJRT device id = local hardware id
    int cuda_ordinal = 0;
    MHLOClientRef mhlo = nullptr;  // the C API client bound to this GPU
    PJRT_DeviceDescription description;
    std::vector<PJRT_Memory*> memories;
};

struct PJRT_TopologyDescription {
    std::string platform_name, platform_version;
    std::vector<PJRT_DeviceDescription*> descriptions;
    std::string serialized;
};

struct PJRT_Client {
    MHLOClientRef mhlo = nullptr;  // device 0's
    std::string platform_name, platform_version;
    std::vector<std::unique_ptr<PJRT_Device>> owned_devices;
    std::vector<std::unique_ptr<PJRT_Memory>> owned_memories;
    std::vector<PJRT_Device*> devices;
    std::vector<PJRT_Memory*> memories;
    PJRT_TopologyDescription topology;
    std::atomic<int64_t> live_buffer_bytes{0}, peak_buffer_bytes{0}, num_allocs{0};
};

struct PJRT_Buffer {
    PJRT_Client* client = nullptr;
    PJRT_Device* device = nullptr;  // where the data lives
    MHLOBufferRef mhlo = nullptr;  // null after PJRT_Buffer_Delete
    PJRT_Buffer_Type type = PJRT_Buffer_Type_INVALID;
    std::vector<int64_t> dims;
    std::vector<int64_t> minor_to_major;  // dense row-major: rank-1 .. 0
    size_t bytes = 0;
    PJRT_Event* ready = nullptr;
    std::atomic<int> external_refs{0};
};

// Immutable description of a compiled program; shared by the loaded executable and every PJRT_Executable handle
// PJRT_LoadedExecutable_GetExecutable gives out (PJRTExecutable.swift:266-400).
struct ExecutableMeta {
    std::string name;
    std::string mlir;         // the text that was compiled; what Serialize stores
    std::string fingerprint;  // hex hash of the text
    std::string serialized;   // [u32 version = 1][u64 length][text], built on first use
    std::mutex mu;
    size_t num_outputs = 0;
    int64_t num_replicas = 1;
    std::vector<PJRT_Buffer_Type> output_types;
    std::vector<int64_t> output_dims;      // all outputs' dims concatenated
    std::vector<size_t> output_dim_sizes;  // rank of each output
    std::vector<bool> output_complex;      // the output is C64 / C128 here and a float tensor of (re, im) pairs below
    std::vector<const char*> output_memory_kinds;
    std::vector<size_t> output_memory_kind_sizes;
    int64_t code_bytes = 0, argument_bytes = 0, output_bytes = 0, temp_bytes = 0;
};

struct PJRT_Executable {
    std::shared_ptr<ExecutableMeta> meta;
};

// One program loaded on num_replicas devices: replica r runs `replicas[r]` (the same program, compiled by that device's
// client) on `devices[r]`. The reference loads on its single device only (PJRTExecutable.swift:1830-1848).
struct PJRT_LoadedExecutable {
    PJRT_Client* client = nullptr;
    MHLOExecutableRef mhlo = nullptr;  // replica 0's
    std::vector<MHLOExecutableRef> replicas;
    std::vector<PJRT_Device*> devices;
    std::shared_ptr<ExecutableMeta> meta;
    bool deleted = false;
};

namespace pjrt_b200 {

PJRT_Error* make_error(PJRT_Error_Code code, const std::string& message);
PJRT_Error* unimplemented(const char* function_name);
PJRT_Event* new_ready_event();
PJRT_Event* new_pending_event();          // becomes ready through event_complete()
void event_complete(PJRT_Event* e);        // marks a pending event ready, wakes waiters, runs its callbacks; drops one reference
void event_retain(PJRT_Event* e);
void event_release(PJRT_Event* e);

// PJRT element type <-> the C API's element type; false when the type has no counterpart (PJRTBuffer.swift:58-95).
bool to_mhlo_type(PJRT_Buffer_Type t, MHLOElementType* out);
PJRT_Buffer_Type from_mhlo_type(MHLOElementType t);
size_t storage_bytes_per_element(MHLOElementType t);

PJRT_Buffer* wrap_buffer(PJRT_Client* client, MHLOBufferRef ref, PJRT_Device* device = nullptr);
// Presents a float buffer of (re, im) pairs as the complex buffer one rank lower that PJRT knows (C64 / C128): the C API
// below has no complex element type (Sources/CMetalHLO/include/metalhlo.h:61-75); the bytes are the same.
void present_as_complex(PJRT_Buffer* b);
std::string hex_hash(const std::string& text);

// Fills every table entry the plugin implements; each group lives in its own translation unit.
void fill_core_api(PJRT_Api* api);        // errors, plugin, events
void fill_client_api(PJRT_Api* api);      // client, devices, memories, topology
void fill_buffer_api(PJRT_Api* api);      // buffers and transfers
void fill_executable_api(PJRT_Api* api);  // compile, executables, execution

}  // namespace pjrt_b200

#define PJRT_B200_REQUIRE(cond, msg) \
    do {                             \
        if (!(cond)) return pjrt_b200::make_error(PJRT_Error_Code_INVALID_ARGUMENT, msg); \
    } while (0)
