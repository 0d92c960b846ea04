// A small PJRT *host*: loads a PJRT plugin by path, fetches its table through GetPjrtApi and drives it the way XLA / JAX
// do — Plugin_Initialize, Client_Create, BufferFromHostBuffer, Compile (with a serialized CompileOptionsProto),
// LoadedExecutable_Execute over one or several devices, ToHostBuffer. It holds no knowledge of the plugin's internals:
// everything goes through the PJRT C API structs. Exposed as plain C functions (libpjrt_host.so) so that the parity
// tests and the benchmark can reach the plugin from Python without jaxlib.
//
// The calls follow what the reference's plugin tests exercise (Tests/PJRTMetalHLOTests/PJRTPluginTests.swift:160-467).
#include <dlfcn.h>

#include <cstdint>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "pjrt_c_api.h"

namespace {

std::mutex g_mu;
std::string g_error;

int fail(const std::string& m) {
    std::lock_guard<std::mutex> lock(g_mu);
    g_error = m;
    return 1;
}

struct Host {
    void* lib = nullptr;
    const PJRT_Api* api = nullptr;
    PJRT_Client* client = nullptr;
    std::vector<PJRT_Device*> devices;  // addressable devices, in the client's order

    std::string take(PJRT_Error* e) const {
        if (!e) return "";
        PJRT_Error_Message_Args m{};
        m.struct_size = PJRT_Error_Message_Args_STRUCT_SIZE;
        m.error = e;
        api->PJRT_Error_Message(&m);
        std::string s(m.message, m.message_size);
        PJRT_Error_Destroy_Args d{};
        d.struct_size = PJRT_Error_Destroy_Args_STRUCT_SIZE;
        d.error = e;
        api->PJRT_Error_Destroy(&d);
        return s.empty() ? "(empty PJRT error message)" : s;
    }
    void drop_event(PJRT_Event* ev) const {
        if (!ev) return;
        PJRT_Event_Destroy_Args a{};
        a.struct_size = PJRT_Event_Destroy_Args_STRUCT_SIZE;
        a.event = ev;
        api->PJRT_Event_Destroy(&a);
    }
    std::string await(PJRT_Event* ev) const {
        if (!ev) return "";
        PJRT_Event_Await_Args w{};
        w.struct_size = PJRT_Event_Await_Args_STRUCT_SIZE;
        w.event = ev;
        std::string e = take(api->PJRT_Event_Await(&w));
        drop_event(ev);
        return e;
    }
};

struct LoadedExe {
    PJRT_LoadedExecutable* loaded = nullptr;
    size_t num_outputs = 0;
    size_t num_devices = 1;  // replicas x partitions the program was compiled for
};

// ---- protobuf wire format, just enough for CompileOptionsProto{executable_build_options{num_replicas, num_partitions,
// device_assignment}} (xla/pjrt/proto/compile_options.proto, xla/xla_data.proto) ----
void put_varint(std::string* s, uint64_t v) {
    while (v >= 0x80) {
        s->push_back(static_cast<char>(v | 0x80));
        v >>= 7;
    }
    s->push_back(static_cast<char>(v));
}
void put_int_field(std::string* s, int field, int64_t v) {
    put_varint(s, static_cast<uint64_t>(field) << 3);
    put_varint(s, static_cast<uint64_t>(v));
}
void put_bytes_field(std::string* s, int field, const std::string& body) {
    put_varint(s, (static_cast<uint64_t>(field) << 3) | 2);
    put_varint(s, body.size());
    s->append(body);
}

std::string compile_options(int num_replicas, int num_partitions, const int64_t* device_ids) {
    std::string build;
    put_int_field(&build, 1, -1);  // device_ordinal: unset
    put_int_field(&build, 4, num_replicas);
    put_int_field(&build, 5, num_partitions);
    if (device_ids) {
        // DeviceAssignmentProto: replica_count = 1, computation_count = 2, computation_devices = 3 (one per partition,
        // each listing the device id of every replica)
        std::string assign;
        put_int_field(&assign, 1, num_replicas);
        put_int_field(&assign, 2, num_partitions);
        for (int p = 0; p < num_partitions; ++p) {
            std::string comp;
            for (int r = 0; r < num_replicas; ++r) put_int_field(&comp, 1, device_ids[r * num_partitions + p]);
            put_bytes_field(&assign, 3, comp);
        }
        put_bytes_field(&build, 9, assign);
    }
    std::string opts;
    put_bytes_field(&opts, 3, build);
    return opts;
}

}  // namespace

extern "C" {

const char* pjrt_host_last_error(void) {
    std::lock_guard<std::mutex> lock(g_mu);
    return g_error.c_str();
}

int pjrt_host_open(const char* plugin_path, void** out_host) {
    if (!plugin_path || !out_host) return fail("pjrt_host_open: null argument");
    *out_host = nullptr;
    Host* h = new Host();
    h->lib = dlopen(plugin_path, RTLD_NOW | RTLD_LOCAL);
    if (!h->lib) {
        std::string why = dlerror();
        delete h;
        return fail("dlopen failed: " + why);
    }
    using GetApi = const PJRT_Api* (*)(void);
    auto get = reinterpret_cast<GetApi>(dlsym(h->lib, "GetPjrtApi"));
    if (!get || !(h->api = get())) {
        delete h;
        return fail("GetPjrtApi missing or returned NULL");
    }
    PJRT_Plugin_Initialize_Args init{};
    init.struct_size = PJRT_Plugin_Initialize_Args_STRUCT_SIZE;
    std::string e = h->take(h->api->PJRT_Plugin_Initialize(&init));
    if (!e.empty()) { delete h; return fail("PJRT_Plugin_Initialize: " + e); }
    PJRT_Client_Create_Args cc{};
    cc.struct_size = PJRT_Client_Create_Args_STRUCT_SIZE;
    e = h->take(h->api->PJRT_Client_Create(&cc));
    if (!e.empty()) { delete h; return fail("PJRT_Client_Create: " + e); }
    h->client = cc.client;
    PJRT_Client_AddressableDevices_Args ad{};
    ad.struct_size = PJRT_Client_AddressableDevices_Args_STRUCT_SIZE;
    ad.client = h->client;
    e = h->take(h->api->PJRT_Client_AddressableDevices(&ad));
    if (!e.empty()) { delete h; return fail("PJRT_Client_AddressableDevices: " + e); }
    h->devices.assign(ad.addressable_devices, ad.addressable_devices + ad.num_addressable_devices);
    *out_host = h;
    return 0;
}

void pjrt_host_close(void* host) {
    Host* h = static_cast<Host*>(host);
    if (!h) return;
    if (h->client) {
        PJRT_Client_Destroy_Args cd{};
        cd.struct_size = PJRT_Client_Destroy_Args_STRUCT_SIZE;
        cd.client = h->client;
        h->take(h->api->PJRT_Client_Destroy(&cd));
    }
    delete h;  // the plugin stays loaded: its table is static data other hosts of this process may hold
}

int pjrt_host_api_version(void* host, int* major, int* minor) {
    Host* h = static_cast<Host*>(host);
    if (!h) return fail("null host");
    if (major) *major = h->api->pjrt_api_version.major_version;
    if (minor) *minor = h->api->pjrt_api_version.minor_version;
    return 0;
}

int pjrt_host_device_count(void* host) { return host ? static_cast<int>(static_cast<Host*>(host)->devices.size()) : 0; }

int pjrt_host_device_id(void* host, int index, int64_t* out_id) {
    Host* h = static_cast<Host*>(host);
    if (!h || index < 0 || index >= static_cast<int>(h->devices.size()) || !out_id) return fail("device index out of range");
    PJRT_Device_GetDescription_Args g{};
    g.struct_size = PJRT_Device_GetDescription_Args_STRUCT_SIZE;
    g.device = h->devices[index];
    std::string e = h->take(h->api->PJRT_Device_GetDescription(&g));
    if (!e.empty()) return fail(e);
    PJRT_DeviceDescription_Id_Args id{};
    id.struct_size = PJRT_DeviceDescription_Id_Args_STRUCT_SIZE;
    id.device_description = g.device_description;
    e = h->take(h->api->PJRT_DeviceDescription_Id(&id));
    if (!e.empty()) return fail(e);
    *out_id = id.id;
    return 0;
}

int pjrt_host_platform_name(void* host, char* out, size_t cap) {
    Host* h = static_cast<Host*>(host);
    if (!h || !out || cap == 0) return fail("null argument");
    PJRT_Client_PlatformName_Args a{};
    a.struct_size = PJRT_Client_PlatformName_Args_STRUCT_SIZE;
    a.client = h->client;
    std::string e = h->take(h->api->PJRT_Client_PlatformName(&a));
    if (!e.empty()) return fail(e);
    const size_t n = a.platform_name_size < cap - 1 ? a.platform_name_size : cap - 1;
    std::memcpy(out, a.platform_name, n);
    out[n] = 0;
    return 0;
}

// Host array -> buffer on addressable device `device_index`. `type` is a PJRT_Buffer_Type value.
int pjrt_host_buffer_from_host(void* host, const void* data, int type, const int64_t* dims, int rank, int device_index,
                               void** out_buffer) {
    Host* h = static_cast<Host*>(host);
    if (!h || !out_buffer) return fail("null argument");
    if (device_index < 0 || device_index >= static_cast<int>(h->devices.size())) return fail("device index out of range");
    PJRT_Client_BufferFromHostBuffer_Args a{};
    a.struct_size = PJRT_Client_BufferFromHostBuffer_Args_STRUCT_SIZE;
    a.client = h->client;
    a.data = data;
    a.type = static_cast<PJRT_Buffer_Type>(type);
    a.dims = dims;
    a.num_dims = static_cast<size_t>(rank);
    a.host_buffer_semantics = PJRT_HostBufferSemantics_kImmutableOnlyDuringCall;
    a.device = h->devices[device_index];
    std::string e = h->take(h->api->PJRT_Client_BufferFromHostBuffer(&a));
    if (!e.empty()) return fail("BufferFromHostBuffer: " + e);
    e = h->await(a.done_with_host_buffer);
    if (!e.empty()) return fail("done_with_host_buffer: " + e);
    *out_buffer = a.buffer;
    return 0;
}

int pjrt_host_buffer_describe(void* host, void* buffer, int* out_type, int64_t* out_dims, int* out_rank, size_t* out_bytes) {
    Host* h = static_cast<Host*>(host);
    if (!h || !buffer) return fail("null argument");
    PJRT_Buffer* b = static_cast<PJRT_Buffer*>(buffer);
    PJRT_Buffer_ElementType_Args t{};
    t.struct_size = PJRT_Buffer_ElementType_Args_STRUCT_SIZE;
    t.buffer = b;
    std::string e = h->take(h->api->PJRT_Buffer_ElementType(&t));
    if (!e.empty()) return fail(e);
    PJRT_Buffer_Dimensions_Args d{};
    d.struct_size = PJRT_Buffer_Dimensions_Args_STRUCT_SIZE;
    d.buffer = b;
    e = h->take(h->api->PJRT_Buffer_Dimensions(&d));
    if (!e.empty()) return fail(e);
    if (out_type) *out_type = static_cast<int>(t.type);
    if (out_rank) *out_rank = static_cast<int>(d.num_dims);
    if (out_dims) for (size_t i = 0; i < d.num_dims && i < 8; ++i) out_dims[i] = d.dims[i];
    if (out_bytes) {
        PJRT_Buffer_ToHostBuffer_Args q{};  // dst == NULL asks for the size
        q.struct_size = PJRT_Buffer_ToHostBuffer_Args_STRUCT_SIZE;
        q.src = b;
        e = h->take(h->api->PJRT_Buffer_ToHostBuffer(&q));
        h->drop_event(q.event);
        if (!e.empty()) return fail(e);
        *out_bytes = q.dst_size;
    }
    return 0;
}

int pjrt_host_buffer_to_host(void* host, void* buffer, void* dst, size_t bytes) {
    Host* h = static_cast<Host*>(host);
    if (!h || !buffer || !dst) return fail("null argument");
    PJRT_Buffer_ToHostBuffer_Args a{};
    a.struct_size = PJRT_Buffer_ToHostBuffer_Args_STRUCT_SIZE;
    a.src = static_cast<PJRT_Buffer*>(buffer);
    a.dst = dst;
    a.dst_size = bytes;
    std::string e = h->take(h->api->PJRT_Buffer_ToHostBuffer(&a));
    if (!e.empty()) return fail("ToHostBuffer: " + e);
    e = h->await(a.event);
    if (!e.empty()) return fail("ToHostBuffer event: " + e);
    return 0;
}

// Starts the transfer and returns its event in *out_event; pjrt_host_event_await waits for it (and frees it).
int pjrt_host_buffer_to_host_start(void* host, void* buffer, void* dst, size_t bytes, void** out_event) {
    Host* h = static_cast<Host*>(host);
    if (!h || !buffer || !dst || !out_event) return fail("null argument");
    *out_event = nullptr;
    PJRT_Buffer_ToHostBuffer_Args a{};
    a.struct_size = PJRT_Buffer_ToHostBuffer_Args_STRUCT_SIZE;
    a.src = static_cast<PJRT_Buffer*>(buffer);
    a.dst = dst;
    a.dst_size = bytes;
    std::string e = h->take(h->api->PJRT_Buffer_ToHostBuffer(&a));
    if (!e.empty()) return fail("ToHostBuffer: " + e);
    *out_event = a.event;
    return 0;
}

int pjrt_host_event_await(void* host, void* event) {
    Host* h = static_cast<Host*>(host);
    if (!h || !event) return fail("null argument");
    const std::string e = h->await(static_cast<PJRT_Event*>(event));
    if (!e.empty()) return fail("event: " + e);
    return 0;
}

void pjrt_host_buffer_destroy(void* host, void* buffer) {
    Host* h = static_cast<Host*>(host);
    if (!h || !buffer) return;
    PJRT_Buffer_Destroy_Args a{};
    a.struct_size = PJRT_Buffer_Destroy_Args_STRUCT_SIZE;
    a.buffer = static_cast<PJRT_Buffer*>(buffer);
    h->take(h->api->PJRT_Buffer_Destroy(&a));
}

// Compiles `program` (format "mlir": StableHLO text or MLIR bytecode) for num_replicas x num_partitions devices.
// device_ids (may be null) = the assignment, replica-major. num_replicas = 0 sends no compile options at all.
int pjrt_host_compile(void* host, const char* program, size_t size, int num_replicas, int num_partitions, const int64_t* device_ids,
                      void** out_executable) {
    Host* h = static_cast<Host*>(host);
    if (!h || !program || !out_executable) return fail("null argument");
    *out_executable = nullptr;
    PJRT_Program prog{};
    prog.struct_size = PJRT_Program_STRUCT_SIZE;
    prog.code = const_cast<char*>(program);
    prog.code_size = size;
    prog.format = "mlir";
    prog.format_size = 4;
    std::string opts;
    if (num_replicas > 0) opts = compile_options(num_replicas, num_partitions > 0 ? num_partitions : 1, device_ids);
    PJRT_Client_Compile_Args a{};
    a.struct_size = PJRT_Client_Compile_Args_STRUCT_SIZE;
    a.client = h->client;
    a.program = &prog;
    a.compile_options = opts.data();
    a.compile_options_size = opts.size();
    std::string e = h->take(h->api->PJRT_Client_Compile(&a));
    if (!e.empty()) return fail("Compile: " + e);
    LoadedExe* x = new LoadedExe();
    x->loaded = a.executable;
    x->num_devices = static_cast<size_t>((num_replicas > 0 ? num_replicas : 1) * (num_partitions > 0 ? num_partitions : 1));
    PJRT_LoadedExecutable_GetExecutable_Args ge{};
    ge.struct_size = PJRT_LoadedExecutable_GetExecutable_Args_STRUCT_SIZE;
    ge.loaded_executable = x->loaded;
    e = h->take(h->api->PJRT_LoadedExecutable_GetExecutable(&ge));
    if (e.empty()) {
        PJRT_Executable_NumOutputs_Args no{};
        no.struct_size = PJRT_Executable_NumOutputs_Args_STRUCT_SIZE;
        no.executable = ge.executable;
        e = h->take(h->api->PJRT_Executable_NumOutputs(&no));
        x->num_outputs = no.num_outputs;
        PJRT_Executable_Destroy_Args de{};
        de.struct_size = PJRT_Executable_Destroy_Args_STRUCT_SIZE;
        de.executable = ge.executable;
        h->take(h->api->PJRT_Executable_Destroy(&de));
    }
    if (!e.empty()) {
        PJRT_LoadedExecutable_Destroy_Args d{};
        d.struct_size = PJRT_LoadedExecutable_Destroy_Args_STRUCT_SIZE;
        d.executable = x->loaded;
        h->take(h->api->PJRT_LoadedExecutable_Destroy(&d));
        delete x;
        return fail("NumOutputs: " + e);
    }
    *out_executable = x;
    return 0;
}

int pjrt_host_executable_num_outputs(void* executable) { return executable ? static_cast<int>(static_cast<LoadedExe*>(executable)->num_outputs) : 0; }
int pjrt_host_executable_num_devices(void* executable) { return executable ? static_cast<int>(static_cast<LoadedExe*>(executable)->num_devices) : 0; }

void pjrt_host_executable_destroy(void* host, void* executable) {
    Host* h = static_cast<Host*>(host);
    LoadedExe* x = static_cast<LoadedExe*>(executable);
    if (!h || !x) return;
    PJRT_LoadedExecutable_Destroy_Args d{};
    d.struct_size = PJRT_LoadedExecutable_Destroy_Args_STRUCT_SIZE;
    d.executable = x->loaded;
    h->take(h->api->PJRT_LoadedExecutable_Destroy(&d));
    delete x;
}

// One Execute call over num_devices devices. args = [num_devices][num_args] buffers, outs = [num_devices][num_outputs]
// (filled in). Waits for every device's completion event before it returns.
int pjrt_host_execute(void* host, void* executable, void* const* args, int num_devices, int num_args, void** outs) {
    Host* h = static_cast<Host*>(host);
    LoadedExe* x = static_cast<LoadedExe*>(executable);
    if (!h || !x || !outs || (num_args > 0 && !args)) return fail("null argument");
    if (num_devices < 1) return fail("num_devices < 1");
    std::vector<PJRT_Buffer* const*> arg_lists(static_cast<size_t>(num_devices));
    std::vector<PJRT_Buffer**> out_lists(static_cast<size_t>(num_devices));
    for (int d = 0; d < num_devices; ++d) {
        arg_lists[d] = reinterpret_cast<PJRT_Buffer* const*>(args) + static_cast<size_t>(d) * num_args;
        out_lists[d] = reinterpret_cast<PJRT_Buffer**>(outs) + static_cast<size_t>(d) * x->num_outputs;
    }
    std::vector<PJRT_Event*> done(static_cast<size_t>(num_devices), nullptr);
    PJRT_ExecuteOptions opts{};
    opts.struct_size = PJRT_ExecuteOptions_STRUCT_SIZE;
    PJRT_LoadedExecutable_Execute_Args a{};
    a.struct_size = PJRT_LoadedExecutable_Execute_Args_STRUCT_SIZE;
    a.executable = x->loaded;
    a.options = &opts;
    a.argument_lists = arg_lists.data();
    a.num_devices = static_cast<size_t>(num_devices);
    a.num_args = static_cast<size_t>(num_args);
    a.output_lists = out_lists.data();
    a.device_complete_events = done.data();
    std::string e = h->take(h->api->PJRT_LoadedExecutable_Execute(&a));
    if (!e.empty()) return fail("Execute: " + e);
    std::string first;
    for (PJRT_Event* ev : done) {
        std::string w = h->await(ev);
        if (first.empty()) first = w;
    }
    if (!first.empty()) return fail("Execute completion: " + first);
    return 0;
}

}  // extern "C"
