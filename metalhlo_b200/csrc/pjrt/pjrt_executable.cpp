// PJRT compile, executable and execution entries (reference: Sources/PJRTMetalHLO/PJRTExecutable.swift:266-400 for
// the executable objects, :1660-1815 for compile, :1820-2208 for the getters, Execute and DeserializeAndLoad).
#include <cstdio>
#include <cstdlib>

#include "pjrt_objects.h"

namespace pjrt_b200 {
namespace {

const char kMemoryKind[] = "device";
constexpr uint32_t kSerialVersion = 1;  // [u32 version][u64 text length][text], PJRTExecutable.swift:345-365

MHLOOptimizationLevel env_opt_level() {
    const char* v = std::getenv("METALHLO_OPT_LEVEL");
    if (!v) return MHLO_OPT_O2;
    const std::string s(v);
    if (s == "O0") return MHLO_OPT_O0;
    if (s == "O1") return MHLO_OPT_O1;
    if (s == "O3") return MHLO_OPT_O3;
    return MHLO_OPT_O2;
}

std::shared_ptr<ExecutableMeta> describe(MHLOExecutableRef exe, const std::string& name, const std::string& text) {
    auto m = std::make_shared<ExecutableMeta>();
    m->name = name;
    m->mlir = text;
    m->fingerprint = hex_hash(text);
    m->num_outputs = static_cast<size_t>(mhlo_executable_output_count(exe));
    for (size_t i = 0; i < m->num_outputs; ++i) {
        int32_t rank = 0;
        MHLOElementType et = MHLO_F32;
        mhlo_executable_output_type(exe, static_cast<int32_t>(i), nullptr, &rank, nullptr);
        std::vector<int64_t> shape(static_cast<size_t>(rank));
        mhlo_executable_output_type(exe, static_cast<int32_t>(i), shape.data(), &rank, &et);
        m->output_types.push_back(from_mhlo_type(et));
        m->output_dim_sizes.push_back(static_cast<size_t>(rank));
        int64_t count = 1;
        for (int64_t d : shape) {
            m->output_dims.push_back(d);
            count *= d;
        }
        m->output_bytes += count * static_cast<int64_t>(storage_bytes_per_element(et));
        m->output_memory_kinds.push_back(kMemoryKind);
        m->output_memory_kind_sizes.push_back(sizeof(kMemoryKind) - 1);
    }
    const int32_t inputs = mhlo_executable_input_count(exe);
    for (int32_t i = 0; i < inputs; ++i) {
        int32_t rank = 0;
        MHLOElementType et = MHLO_F32;
        mhlo_executable_input_type(exe, i, nullptr, &rank, nullptr);
        std::vector<int64_t> shape(static_cast<size_t>(rank));
        mhlo_executable_input_type(exe, i, shape.data(), &rank, &et);
        int64_t count = 1;
        for (int64_t d : shape) count *= d;
        m->argument_bytes += count * static_cast<int64_t>(storage_bytes_per_element(et));
    }
    m->temp_bytes = mhlo_b200_executable_arena_bytes(exe);
    return m;
}

PJRT_Error* compile_text(PJRT_Client* client, const std::string& text, MHLOOptimizationLevel level, const std::string& name,
                         const char* failure_prefix, PJRT_LoadedExecutable** out) {
    MHLOCompileConfig config;
    mhlo_compile_config_init(&config);
    config.optimization_level = level;
    MHLOExecutableRef exe = nullptr;
    if (mhlo_compile_with_config(client->mhlo, text.c_str(), &config, &exe) != MHLO_OK || !exe)
        return make_error(PJRT_Error_Code_INTERNAL, std::string(failure_prefix) + mhlo_get_last_error());
    auto* loaded = new PJRT_LoadedExecutable();
    loaded->client = client;
    loaded->mhlo = exe;
    loaded->meta = describe(exe, name, text);
    *out = loaded;
    return nullptr;
}

// The program is StableHLO text. MLIR bytecode (magic "ML\xEFR") is what JAX sends; the reference converts it to text
// with a jaxlib helper process (PJRTExecutable.swift:1680-1697). No MLIR bytecode reader is linked here, so bytecode
// is refused with a message that says what to send instead.
PJRT_Error* client_compile(PJRT_Client_Compile_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args or client");
    PJRT_B200_REQUIRE(args->program, "NULL program");
    PJRT_B200_REQUIRE(args->program->code, "NULL program code");
    const char* code = args->program->code;
    const size_t size = args->program->code_size;
    if (size >= 4 && static_cast<unsigned char>(code[0]) == 0x4D && static_cast<unsigned char>(code[1]) == 0x4C &&
        static_cast<unsigned char>(code[2]) == 0xEF && static_cast<unsigned char>(code[3]) == 0x52)
        return make_error(PJRT_Error_Code_UNIMPLEMENTED,
                          "Bytecode conversion failed: this build has no MLIR bytecode reader; pass the module as StableHLO text");
    const std::string text(code, size);
    if (const char* dir = std::getenv("METALHLO_DUMP_MLIR")) {
        const std::string path = std::string(dir) + "/mlir_" + hex_hash(text) + ".txt";
        if (FILE* f = std::fopen(path.c_str(), "w")) {
            std::fwrite(text.data(), 1, text.size(), f);
            std::fclose(f);
        }
    }
    return compile_text(args->client, text, env_opt_level(), "metalhlo_program", "Compilation failed: ", &args->executable);
}

// ---- PJRT_Executable getters ----
PJRT_Error* executable_destroy(PJRT_Executable_Destroy_Args* args) {
    if (args && args->executable) delete args->executable;
    return nullptr;
}

PJRT_Error* executable_name(PJRT_Executable_Name_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    args->executable_name = args->executable->meta->name.c_str();
    args->executable_name_size = args->executable->meta->name.size();
    return nullptr;
}

PJRT_Error* executable_num_replicas(PJRT_Executable_NumReplicas_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    args->num_replicas = 1;
    return nullptr;
}

PJRT_Error* executable_num_partitions(PJRT_Executable_NumPartitions_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    args->num_partitions = 1;
    return nullptr;
}

PJRT_Error* executable_num_outputs(PJRT_Executable_NumOutputs_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    args->num_outputs = args->executable->meta->num_outputs;
    return nullptr;
}

PJRT_Error* executable_code_size(PJRT_Executable_SizeOfGeneratedCodeInBytes_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    args->size_in_bytes = 0;  // kernels are precompiled into the library; a program adds no device code
    return nullptr;
}

PJRT_Error* executable_cost_analysis(PJRT_Executable_GetCostAnalysis_Args* args) {
    PJRT_B200_REQUIRE(args, "NULL args");
    args->num_properties = 0;
    args->properties = nullptr;
    return nullptr;
}

PJRT_Error* executable_output_memory_kinds(PJRT_Executable_OutputMemoryKinds_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    ExecutableMeta& m = *args->executable->meta;
    args->num_outputs = m.num_outputs;
    args->memory_kinds = m.output_memory_kinds.data();
    args->memory_kind_sizes = m.output_memory_kind_sizes.data();
    return nullptr;
}

// The reference leaves this entry unimplemented (PJRTExecutable.swift:1895-1899). Here it follows PJRT's two-call
// protocol: a NULL code pointer asks for the size, otherwise the text that was compiled is copied out as "mlir".
PJRT_Error* executable_optimized_program(PJRT_Executable_OptimizedProgram_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable && args->program, "NULL args");
    static const char kFormat[] = "mlir";
    const std::string& text = args->executable->meta->mlir;
    args->program->format = kFormat;
    args->program->format_size = sizeof(kFormat) - 1;
    if (!args->program->code) {
        args->program->code_size = text.size();
        return nullptr;
    }
    if (args->program->code_size < text.size()) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "OptimizedProgram: code buffer too small");
    std::memcpy(args->program->code, text.data(), text.size());
    args->program->code_size = text.size();
    return nullptr;
}

// The bytes stay owned by the executable's description and live as long as any handle on it
// (PJRTExecutable.swift:1901-1918); the deleter therefore has nothing to free.
PJRT_Error* executable_serialize(PJRT_Executable_Serialize_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    ExecutableMeta& m = *args->executable->meta;
    {
        std::lock_guard<std::mutex> lock(m.mu);
        if (m.serialized.empty()) {
            const uint32_t version = kSerialVersion;
            const uint64_t length = m.mlir.size();
            m.serialized.append(reinterpret_cast<const char*>(&version), sizeof version);
            m.serialized.append(reinterpret_cast<const char*>(&length), sizeof length);
            m.serialized.append(m.mlir);
        }
    }
    args->serialized_bytes = m.serialized.data();
    args->serialized_bytes_size = m.serialized.size();
    args->serialized_executable = nullptr;
    args->serialized_executable_deleter = [](PJRT_SerializedExecutable*) {};
    return nullptr;
}

PJRT_Error* executable_output_element_types(PJRT_Executable_OutputElementTypes_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    args->output_types = args->executable->meta->output_types.data();
    args->num_output_types = args->executable->meta->num_outputs;
    return nullptr;
}

PJRT_Error* executable_output_dimensions(PJRT_Executable_OutputDimensions_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    ExecutableMeta& m = *args->executable->meta;
    args->num_outputs = m.num_outputs;
    args->dims = m.output_dims.data();
    args->dim_sizes = m.output_dim_sizes.data();
    return nullptr;
}

PJRT_Error* executable_fingerprint(PJRT_Executable_Fingerprint_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    args->executable_fingerprint = args->executable->meta->fingerprint.c_str();
    args->executable_fingerprint_size = args->executable->meta->fingerprint.size();
    return nullptr;
}

// Unimplemented in the reference (PJRTExecutable.swift:1957-1961); the static plan makes the figures cheap here:
// arguments and outputs from the signature, temporaries = the planned arena.
PJRT_Error* executable_memory_stats(PJRT_Executable_GetCompiledMemoryStats_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    const ExecutableMeta& m = *args->executable->meta;
    args->generated_code_size_in_bytes = 0;
    args->argument_size_in_bytes = m.argument_bytes;
    args->output_size_in_bytes = m.output_bytes;
    args->alias_size_in_bytes = 0;
    args->temp_size_in_bytes = m.temp_bytes;
    args->host_generated_code_size_in_bytes = 0;
    args->host_argument_size_in_bytes = 0;
    args->host_output_size_in_bytes = 0;
    args->host_alias_size_in_bytes = 0;
    args->host_temp_size_in_bytes = 0;
    args->peak_memory_in_bytes = m.argument_bytes + m.output_bytes + m.temp_bytes;
    args->total_size_in_bytes = m.argument_bytes + m.output_bytes + m.temp_bytes;
    return nullptr;
}

// ---- PJRT_LoadedExecutable ----
PJRT_Error* loaded_destroy(PJRT_LoadedExecutable_Destroy_Args* args) {
    if (!args || !args->executable) return nullptr;
    if (args->executable->mhlo) mhlo_executable_destroy(args->executable->mhlo);
    delete args->executable;
    return nullptr;
}

PJRT_Error* loaded_get_executable(PJRT_LoadedExecutable_GetExecutable_Args* args) {
    PJRT_B200_REQUIRE(args && args->loaded_executable, "NULL args");
    args->executable = new PJRT_Executable{args->loaded_executable->meta};
    return nullptr;
}

PJRT_Error* loaded_addressable_devices(PJRT_LoadedExecutable_AddressableDevices_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    args->addressable_devices = args->executable->client->devices.data();
    args->num_addressable_devices = args->executable->client->devices.size();
    return nullptr;
}

PJRT_Error* loaded_delete(PJRT_LoadedExecutable_Delete_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    args->executable->deleted = true;
    return nullptr;
}

PJRT_Error* loaded_is_deleted(PJRT_LoadedExecutable_IsDeleted_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    args->is_deleted = args->executable->deleted;
    return nullptr;
}

// Single-device, synchronous (PJRTExecutable.swift:2024-2110): inputs from argument_lists[0], fresh output buffers
// into output_lists[0], and a completion event that is ready on return.
PJRT_Error* loaded_execute(PJRT_LoadedExecutable_Execute_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    PJRT_LoadedExecutable* loaded = args->executable;
    if (args->num_devices > 1) return make_error(PJRT_Error_Code_UNIMPLEMENTED, "Multi-device execution not supported");
    if (loaded->deleted) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "Execution failed: executable was deleted");
    std::vector<MHLOBufferRef> inputs;
    if (args->num_devices > 0 && args->num_args > 0) {
        PJRT_B200_REQUIRE(args->argument_lists && args->argument_lists[0], "NULL argument list for device 0");
        for (size_t i = 0; i < args->num_args; ++i) {
            PJRT_Buffer* b = args->argument_lists[0][i];
            if (!b) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "NULL buffer at argument index " + std::to_string(i));
            if (!b->mhlo) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "deleted buffer at argument index " + std::to_string(i));
            inputs.push_back(b->mhlo);
        }
    }
    std::vector<MHLOBufferRef> outputs(loaded->meta->num_outputs, nullptr);
    int32_t produced = 0;
    const MHLOStatusCode st = mhlo_execute(loaded->mhlo, inputs.data(), static_cast<int32_t>(inputs.size()), outputs.data(), &produced);
    if (st != MHLO_OK) return make_error(PJRT_Error_Code_INTERNAL, std::string("Execution failed: ") + mhlo_get_last_error());
    const bool want_outputs = args->output_lists && args->num_devices > 0 && args->output_lists[0];
    for (int32_t i = 0; i < produced; ++i) {
        if (want_outputs) args->output_lists[0][i] = wrap_buffer(loaded->client, outputs[static_cast<size_t>(i)]);
        else mhlo_buffer_destroy(outputs[static_cast<size_t>(i)]);
    }
    if (args->device_complete_events && args->num_devices > 0) args->device_complete_events[0] = new_ready_event();
    return nullptr;
}

// DeviceAssignmentProto for one replica, one computation on device 0 (PJRTExecutable.swift:2112-2145):
// field 1 (replica_count) = 1, field 2 (computation_count) = 1, field 3 = {field 1 (replica_device_ids) = 0}.
PJRT_Error* loaded_device_assignment(PJRT_LoadedExecutable_GetDeviceAssignment_Args* args) {
    PJRT_B200_REQUIRE(args, "NULL args");
    static const unsigned char kProto[] = {0x08, 0x01, 0x10, 0x01, 0x1A, 0x02, 0x08, 0x00};
    auto* copy = static_cast<unsigned char*>(std::malloc(sizeof kProto));
    std::memcpy(copy, kProto, sizeof kProto);
    args->serialized_bytes = reinterpret_cast<const char*>(copy);
    args->serialized_bytes_size = sizeof kProto;
    args->serialized_device_assignment = reinterpret_cast<PJRT_DeviceAssignmentSerialized*>(copy);
    args->serialized_device_assignment_deleter = [](PJRT_DeviceAssignmentSerialized* p) { std::free(p); };
    return nullptr;
}

PJRT_Error* loaded_fingerprint(PJRT_LoadedExecutable_Fingerprint_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    args->executable_fingerprint = args->executable->meta->fingerprint.c_str();
    args->executable_fingerprint_size = args->executable->meta->fingerprint.size();
    return nullptr;
}

// Re-compiles the stored text at O2 (PJRTExecutable.swift:2160-2208).
PJRT_Error* deserialize_and_load(PJRT_Executable_DeserializeAndLoad_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args or client");
    PJRT_B200_REQUIRE(args->serialized_executable, "NULL serialized bytes");
    const char* bytes = args->serialized_executable;
    const size_t size = args->serialized_executable_size;
    PJRT_B200_REQUIRE(size >= 12, "Serialized data too short");
    uint32_t version = 0;
    uint64_t length = 0;
    std::memcpy(&version, bytes, 4);
    std::memcpy(&length, bytes + 4, 8);
    if (version != kSerialVersion) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "Unknown serialization version: " + std::to_string(version));
    PJRT_B200_REQUIRE(length <= size - 12, "Serialized data truncated");
    const std::string text(bytes + 12, static_cast<size_t>(length));
    return compile_text(args->client, text, MHLO_OPT_O2, "metalhlo_deserialized", "Deserialization re-compilation failed: ",
                        &args->loaded_executable);
}

}  // namespace

void fill_executable_api(PJRT_Api* api) {
    api->PJRT_Client_Compile = client_compile;
    api->PJRT_Executable_Destroy = executable_destroy;
    api->PJRT_Executable_Name = executable_name;
    api->PJRT_Executable_NumReplicas = executable_num_replicas;
    api->PJRT_Executable_NumPartitions = executable_num_partitions;
    api->PJRT_Executable_NumOutputs = executable_num_outputs;
    api->PJRT_Executable_SizeOfGeneratedCodeInBytes = executable_code_size;
    api->PJRT_Executable_GetCostAnalysis = executable_cost_analysis;
    api->PJRT_Executable_OutputMemoryKinds = executable_output_memory_kinds;
    api->PJRT_Executable_OptimizedProgram = executable_optimized_program;
    api->PJRT_Executable_Serialize = executable_serialize;
    api->PJRT_Executable_OutputElementTypes = executable_output_element_types;
    api->PJRT_Executable_OutputDimensions = executable_output_dimensions;
    api->PJRT_Executable_Fingerprint = executable_fingerprint;
    api->PJRT_Executable_GetCompiledMemoryStats = executable_memory_stats;
    api->PJRT_Executable_DeserializeAndLoad = deserialize_and_load;
    api->PJRT_LoadedExecutable_Destroy = loaded_destroy;
    api->PJRT_LoadedExecutable_GetExecutable = loaded_get_executable;
    api->PJRT_LoadedExecutable_AddressableDevices = loaded_addressable_devices;
    api->PJRT_LoadedExecutable_Delete = loaded_delete;
    api->PJRT_LoadedExecutable_IsDeleted = loaded_is_deleted;
    api->PJRT_LoadedExecutable_Execute = loaded_execute;
    api->PJRT_LoadedExecutable_GetDeviceAssignment = loaded_device_assignment;
    api->PJRT_LoadedExecutable_Fingerprint = loaded_fingerprint;
}

}  // namespace pjrt_b200
