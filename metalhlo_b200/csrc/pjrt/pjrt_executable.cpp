// PJRT compile, executable and execution entries (reference: Sources/PJRTMetalHLO/PJRTExecutable.swift:266-400 for
// the executable objects, :1660-1815 for compile, :1820-2208 for the getters, Execute and DeserializeAndLoad).
#include <thread>
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
        // a complex result is a float tensor of (re, im) pairs below this layer: C64 / C128 of one rank less here
        const bool cx = mhlo_b200_executable_output_is_complex(exe, static_cast<int32_t>(i)) == 1 && rank > 0 && shape.back() == 2 &&
                        (et == MHLO_F32 || et == MHLO_F64);
        m->output_complex.push_back(cx);
        m->output_types.push_back(cx ? (et == MHLO_F32 ? PJRT_Buffer_Type_C64 : PJRT_Buffer_Type_C128) : from_mhlo_type(et));
        m->output_dim_sizes.push_back(static_cast<size_t>(cx ? rank - 1 : rank));
        int64_t count = 1;
        for (size_t k = 0; k < shape.size(); ++k) {
            if (!cx || k + 1 < shape.size()) m->output_dims.push_back(shape[k]);
            count *= shape[k];
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

// ---- the part of CompileOptionsProto this plugin honours (xla/pjrt/proto/compile_options.proto): field 3
// executable_build_options { 4 num_replicas, 5 num_partitions, 9 device_assignment { 3 computation_devices { 1 replica_device_ids } } }.
// The reference ignores the options and fixes both counts at 1 (PJRTExecutable.swift:1830-1848). ----
struct BuildOptions {
    int64_t num_replicas = 1, num_partitions = 1;
    std::vector<int64_t> replica_devices;  // device id of replica r (partition 0), when an assignment was sent
};

struct ProtoReader {
    const unsigned char* p;
    const unsigned char* end;
    bool ok = true;
    uint64_t varint() {
        uint64_t v = 0;
        for (int shift = 0; shift < 64 && p < end; shift += 7) {
            const unsigned char b = *p++;
            v |= static_cast<uint64_t>(b & 0x7f) << shift;
            if (!(b & 0x80)) return v;
        }
        ok = false;
        return 0;
    }
    // next field: number, wire type, and for length-delimited fields the payload range
    bool next(int* field, int* wire, uint64_t* value, ProtoReader* sub) {
        if (p >= end || !ok) return false;
        const uint64_t key = varint();
        *field = static_cast<int>(key >> 3);
        *wire = static_cast<int>(key & 7);
        if (*wire == 0) *value = varint();
        else if (*wire == 2) {
            const uint64_t n = varint();
            if (!ok || n > static_cast<uint64_t>(end - p)) { ok = false; return false; }
            *sub = ProtoReader{p, p + n};
            p += n;
        } else if (*wire == 1) { if (end - p < 8) { ok = false; return false; } p += 8; }
        else if (*wire == 5) { if (end - p < 4) { ok = false; return false; } p += 4; }
        else { ok = false; return false; }
        return ok;
    }
};

bool parse_build_options(const char* data, size_t size, BuildOptions* out) {
    if (!data || size == 0) return true;
    ProtoReader top{reinterpret_cast<const unsigned char*>(data), reinterpret_cast<const unsigned char*>(data) + size};
    int field, wire;
    uint64_t value;
    ProtoReader sub{nullptr, nullptr};
    while (top.next(&field, &wire, &value, &sub)) {
        if (field != 3 || wire != 2) continue;
        ProtoReader build = sub, inner{nullptr, nullptr};
        while (build.next(&field, &wire, &value, &inner)) {
            if (field == 4 && wire == 0) out->num_replicas = static_cast<int64_t>(value);
            else if (field == 5 && wire == 0) out->num_partitions = static_cast<int64_t>(value);
            else if (field == 9 && wire == 2) {
                ProtoReader assign = inner, comp{nullptr, nullptr};
                bool first_computation = true;
                while (assign.next(&field, &wire, &value, &comp)) {
                    if (field != 3 || wire != 2 || !first_computation) continue;
                    first_computation = false;
                    ProtoReader ids = comp, packed{nullptr, nullptr};
                    while (ids.next(&field, &wire, &value, &packed)) {
                        if (field != 1) continue;
                        if (wire == 0) out->replica_devices.push_back(static_cast<int64_t>(value));
                        else if (wire == 2) while (packed.p < packed.end && packed.ok) out->replica_devices.push_back(static_cast<int64_t>(packed.varint()));
                    }
                }
            }
        }
        if (!build.ok) return false;
    }
    return top.ok;
}

// Compiles `text` once per replica, each on its own device's client. Replica r runs on the r-th device of the assignment,
// else on device r.
PJRT_Error* compile_text(PJRT_Client* client, const std::string& text, MHLOOptimizationLevel level, const std::string& name,
                         const char* failure_prefix, PJRT_LoadedExecutable** out, const BuildOptions& options = BuildOptions()) {
    if (options.num_partitions != 1)
        return make_error(PJRT_Error_Code_UNIMPLEMENTED, std::string(failure_prefix) + "num_partitions = " + std::to_string(options.num_partitions) +
                                                             ": programs are not partitioned across devices (replicas are)");
    const size_t replicas = options.num_replicas < 1 ? 1 : static_cast<size_t>(options.num_replicas);
    if (replicas > client->devices.size())
        return make_error(PJRT_Error_Code_INVALID_ARGUMENT, std::string(failure_prefix) + std::to_string(replicas) + " replicas on a client with " +
                                                                std::to_string(client->devices.size()) + " device(s); set METALHLO_NUM_GPUS");
    MHLOCompileConfig config;
    mhlo_compile_config_init(&config);
    config.optimization_level = level;
    auto* loaded = new PJRT_LoadedExecutable();
    loaded->client = client;
    auto undo = [&](PJRT_Error* e) {
        for (MHLOExecutableRef x : loaded->replicas) mhlo_executable_destroy(x);
        delete loaded;
        return e;
    };
    for (size_t r = 0; r < replicas; ++r) {
        int64_t id = r < options.replica_devices.size() ? options.replica_devices[r] : static_cast<int64_t>(r);
        if (id < 0 || id >= static_cast<int64_t>(client->devices.size()))
            return undo(make_error(PJRT_Error_Code_INVALID_ARGUMENT, std::string(failure_prefix) + "device assignment names device " + std::to_string(id)));
        PJRT_Device* dev = client->devices[static_cast<size_t>(id)];
        MHLOExecutableRef exe = nullptr;
        if (mhlo_compile_with_config(dev->mhlo, text.c_str(), &config, &exe) != MHLO_OK || !exe)
            return undo(make_error(PJRT_Error_Code_INTERNAL, std::string(failure_prefix) + mhlo_get_last_error()));
        loaded->replicas.push_back(exe);
        loaded->devices.push_back(dev);
    }
    loaded->mhlo = loaded->replicas[0];
    loaded->meta = describe(loaded->mhlo, name, text);
    loaded->meta->num_replicas = static_cast<int64_t>(replicas);
    *out = loaded;
    return nullptr;
}

// The program is StableHLO text, or MLIR bytecode (magic "ML\xEFR", what JAX sends), which a jaxlib helper process turns
// into text first, as in the reference (PJRTExecutable.swift:1680-1697).
PJRT_Error* client_compile(PJRT_Client_Compile_Args* args) {
    PJRT_B200_REQUIRE(args && args->client, "NULL args or client");
    PJRT_B200_REQUIRE(args->program, "NULL program");
    PJRT_B200_REQUIRE(args->program->code, "NULL program code");
    const char* code = args->program->code;
    const size_t size = args->program->code_size;
    std::string converted;
    if (size >= 4 && static_cast<unsigned char>(code[0]) == 0x4D && static_cast<unsigned char>(code[1]) == 0x4C &&
        static_cast<unsigned char>(code[2]) == 0xEF && static_cast<unsigned char>(code[3]) == 0x52) {
        char* out = nullptr;
        if (mhlo_b200_bytecode_to_text(code, size, &out) != MHLO_OK || !out) {
            const char* m = mhlo_get_last_error();
            return make_error(PJRT_Error_Code_INTERNAL, m ? m : "Bytecode conversion failed");
        }
        converted = out;
        mhlo_free_string(out);
    }
    const std::string text = converted.empty() ? std::string(code, size) : converted;
    if (const char* dir = std::getenv("METALHLO_DUMP_MLIR")) {
        const std::string path = std::string(dir) + "/mlir_" + hex_hash(text) + ".txt";
        if (FILE* f = std::fopen(path.c_str(), "w")) {
            std::fwrite(text.data(), 1, text.size(), f);
            std::fclose(f);
        }
    }
    BuildOptions options;
    if (!parse_build_options(args->compile_options, args->compile_options_size, &options))
        return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "Compilation failed: malformed compile options");
    return compile_text(args->client, text, env_opt_level(), "metalhlo_program", "Compilation failed: ", &args->executable, options);
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
    args->num_replicas = static_cast<size_t>(args->executable->meta->num_replicas);
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
    for (MHLOExecutableRef x : args->executable->replicas) mhlo_executable_destroy(x);
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
    args->addressable_devices = args->executable->devices.data();
    args->num_addressable_devices = args->executable->devices.size();
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

// Synchronous (PJRTExecutable.swift:2024-2110): replica d takes its inputs from argument_lists[d], writes fresh output
// buffers into output_lists[d], and its completion event is ready on return. Several replicas run at the same time, one
// host thread per device (the reference refuses num_devices > 1, PJRTExecutable.swift:2033-2036). With execute_device set,
// the one argument list runs on that device's replica.
PJRT_Error* loaded_execute(PJRT_LoadedExecutable_Execute_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    PJRT_LoadedExecutable* loaded = args->executable;
    if (loaded->deleted) return make_error(PJRT_Error_Code_FAILED_PRECONDITION, "Execution failed: executable was deleted");
    const size_t replicas = loaded->replicas.size();
    size_t first = 0, count = args->num_devices;
    if (args->execute_device) {
        if (args->num_devices != 1) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "Execution failed: execute_device takes one argument list");
        bool found = false;
        for (size_t r = 0; r < replicas; ++r)
            if (loaded->devices[r] == args->execute_device) { first = r; found = true; }
        if (!found) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "Execution failed: the executable is not loaded on execute_device");
    } else if (count > replicas) {
        return make_error(replicas == 1 ? PJRT_Error_Code_UNIMPLEMENTED : PJRT_Error_Code_INVALID_ARGUMENT,
                          "Multi-device execution not supported: " + std::to_string(count) + " argument lists for " + std::to_string(replicas) +
                              " replica(s); compile with num_replicas");
    }
    if (count == 0) count = 1;
    std::vector<std::vector<MHLOBufferRef>> inputs(count);
    for (size_t d = 0; d < count && args->num_devices > 0 && args->num_args > 0; ++d) {
        PJRT_B200_REQUIRE(args->argument_lists && args->argument_lists[d], "NULL argument list");
        for (size_t i = 0; i < args->num_args; ++i) {
            PJRT_Buffer* b = args->argument_lists[d][i];
            if (!b) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "NULL buffer at argument index " + std::to_string(i));
            if (!b->mhlo) return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "deleted buffer at argument index " + std::to_string(i));
            if (b->device != loaded->devices[first + d])
                return make_error(PJRT_Error_Code_INVALID_ARGUMENT, "argument " + std::to_string(i) + " of replica " + std::to_string(first + d) +
                                                                        " lives on device " + std::to_string(b->device ? b->device->index : -1) +
                                                                        ", the replica runs on device " + std::to_string(loaded->devices[first + d]->index));
            inputs[d].push_back(b->mhlo);
        }
    }
    const size_t n_out = loaded->meta->num_outputs;
    std::vector<std::vector<MHLOBufferRef>> outputs(count, std::vector<MHLOBufferRef>(n_out, nullptr));
    std::vector<int32_t> produced(count, 0);
    std::vector<MHLOStatusCode> status(count, MHLO_OK);
    std::vector<std::string> messages(count);
    auto run_one = [&](size_t d) {
        status[d] = mhlo_execute(loaded->replicas[first + d], inputs[d].data(), static_cast<int32_t>(inputs[d].size()), outputs[d].data(), &produced[d]);
        if (status[d] != MHLO_OK) {
            const char* m = mhlo_get_last_error();
            messages[d] = m ? m : "unknown error";
        }
    };
    if (count == 1) {
        run_one(0);
    } else {
        std::vector<std::thread> workers;
        for (size_t d = 0; d < count; ++d) workers.emplace_back(run_one, d);
        for (std::thread& w : workers) w.join();
    }
    for (size_t d = 0; d < count; ++d) {
        if (status[d] == MHLO_OK) continue;
        for (size_t e = 0; e < count; ++e)
            for (int32_t i = 0; i < produced[e]; ++i)
                if (status[e] == MHLO_OK && outputs[e][static_cast<size_t>(i)]) mhlo_buffer_destroy(outputs[e][static_cast<size_t>(i)]);
        return make_error(PJRT_Error_Code_INTERNAL, "Execution failed" + (count > 1 ? " on replica " + std::to_string(first + d) : std::string()) + ": " + messages[d]);
    }
    for (size_t d = 0; d < count; ++d) {
        const bool want_outputs = args->output_lists && args->num_devices > 0 && args->output_lists[d];
        for (int32_t i = 0; i < produced[d]; ++i) {
            if (want_outputs) {
                args->output_lists[d][i] = wrap_buffer(loaded->client, outputs[d][static_cast<size_t>(i)], loaded->devices[first + d]);
                if (loaded->meta->output_complex[static_cast<size_t>(i)]) present_as_complex(args->output_lists[d][i]);
            }
            else mhlo_buffer_destroy(outputs[d][static_cast<size_t>(i)]);
        }
        if (args->device_complete_events && args->num_devices > 0) args->device_complete_events[d] = new_ready_event();
    }
    return nullptr;
}

// DeviceAssignmentProto of the loaded program (PJRTExecutable.swift:2112-2145 writes the one-replica form): field 1
// replica_count, field 2 computation_count = 1, field 3 = one computation listing the device id of every replica.
PJRT_Error* loaded_device_assignment(PJRT_LoadedExecutable_GetDeviceAssignment_Args* args) {
    PJRT_B200_REQUIRE(args && args->executable, "NULL args");
    std::string comp;
    for (PJRT_Device* d : args->executable->devices) {
        comp.push_back(0x08);
        comp.push_back(static_cast<char>(d->index & 0x7f));  // device ids stay below 128
    }
    std::string proto;
    proto.push_back(0x08);
    proto.push_back(static_cast<char>(args->executable->devices.size() & 0x7f));
    proto.push_back(0x10);
    proto.push_back(0x01);
    proto.push_back(0x1A);
    proto.push_back(static_cast<char>(comp.size()));
    proto += comp;
    auto* copy = static_cast<unsigned char*>(std::malloc(proto.size()));
    std::memcpy(copy, proto.data(), proto.size());
    args->serialized_bytes = reinterpret_cast<const char*>(copy);
    args->serialized_bytes_size = proto.size();
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
