// Self-test of the PJRT plugin through its one exported symbol, the way a PJRT host (XLA, JAX) drives it.
//   pjrt_selftest <plugin.so> host     checks that need no GPU: table, version, error objects
//   pjrt_selftest <plugin.so> device   the above plus client, transfers, compile, execute, serialize
// The cases follow the reference's plugin tests (Tests/PJRTMetalHLOTests/PJRTPluginTests.swift:160-460).
// Prints one "PASS <case>" or "FAIL <case>: <why>" line per case; the exit code is the number of failures.
#include <dlfcn.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "pjrt_c_api.h"

static const PJRT_Api* api = nullptr;
static int failures = 0;

static void report(const char* name, bool ok, const std::string& why = "") {
    if (ok) std::printf("PASS %s\n", name);
    else {
        std::printf("FAIL %s: %s\n", name, why.c_str());
        ++failures;
    }
}

static std::string take_error(PJRT_Error* e) {
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
    return s.empty() ? "(empty message)" : s;
}

static void destroy_event(PJRT_Event* ev) {
    if (!ev) return;
    PJRT_Event_Destroy_Args a{};
    a.struct_size = PJRT_Event_Destroy_Args_STRUCT_SIZE;
    a.event = ev;
    api->PJRT_Event_Destroy(&a);
}

static void destroy_buffer(PJRT_Buffer* b) {
    if (!b) return;
    PJRT_Buffer_Destroy_Args a{};
    a.struct_size = PJRT_Buffer_Destroy_Args_STRUCT_SIZE;
    a.buffer = b;
    api->PJRT_Buffer_Destroy(&a);
}

static void destroy_loaded(PJRT_LoadedExecutable* e) {
    if (!e) return;
    PJRT_LoadedExecutable_Destroy_Args a{};
    a.struct_size = PJRT_LoadedExecutable_Destroy_Args_STRUCT_SIZE;
    a.executable = e;
    api->PJRT_LoadedExecutable_Destroy(&a);
}

static PJRT_Buffer* make_buffer(PJRT_Client* c, const void* data, PJRT_Buffer_Type type, const std::vector<int64_t>& dims,
                                const int64_t* byte_strides, std::string* err) {
    PJRT_Client_BufferFromHostBuffer_Args a{};
    a.struct_size = PJRT_Client_BufferFromHostBuffer_Args_STRUCT_SIZE;
    a.client = c;
    a.data = data;
    a.type = type;
    a.dims = dims.data();
    a.num_dims = dims.size();
    a.byte_strides = byte_strides;
    a.num_byte_strides = byte_strides ? dims.size() : 0;
    a.host_buffer_semantics = PJRT_HostBufferSemantics_kImmutableOnlyDuringCall;
    *err = take_error(api->PJRT_Client_BufferFromHostBuffer(&a));
    if (!err->empty()) return nullptr;
    if (a.done_with_host_buffer) {
        PJRT_Event_IsReady_Args r{};
        r.struct_size = PJRT_Event_IsReady_Args_STRUCT_SIZE;
        r.event = a.done_with_host_buffer;
        api->PJRT_Event_IsReady(&r);
        if (!r.is_ready) *err = "done_with_host_buffer is not ready";
        destroy_event(a.done_with_host_buffer);
    }
    return a.buffer;
}

static std::string read_buffer(PJRT_Buffer* b, void* dst, size_t bytes) {
    PJRT_Buffer_ToHostBuffer_Args q{};
    q.struct_size = PJRT_Buffer_ToHostBuffer_Args_STRUCT_SIZE;
    q.src = b;
    std::string e = take_error(api->PJRT_Buffer_ToHostBuffer(&q));  // dst == NULL: size query
    destroy_event(q.event);
    if (!e.empty()) return e;
    if (q.dst_size != bytes) return "size query gave " + std::to_string(q.dst_size) + ", expected " + std::to_string(bytes);
    PJRT_Buffer_ToHostBuffer_Args a{};
    a.struct_size = PJRT_Buffer_ToHostBuffer_Args_STRUCT_SIZE;
    a.src = b;
    a.dst = dst;
    a.dst_size = bytes;
    e = take_error(api->PJRT_Buffer_ToHostBuffer(&a));
    destroy_event(a.event);
    return e;
}

static PJRT_LoadedExecutable* compile(PJRT_Client* c, const std::string& text, std::string* err) {
    PJRT_Program prog{};
    prog.struct_size = PJRT_Program_STRUCT_SIZE;
    prog.code = const_cast<char*>(text.data());
    prog.code_size = text.size();
    prog.format = "mlir";
    prog.format_size = 4;
    PJRT_Client_Compile_Args a{};
    a.struct_size = PJRT_Client_Compile_Args_STRUCT_SIZE;
    a.client = c;
    a.program = &prog;
    *err = take_error(api->PJRT_Client_Compile(&a));
    return err->empty() ? a.executable : nullptr;
}

static std::string execute(PJRT_LoadedExecutable* exe, const std::vector<PJRT_Buffer*>& inputs, std::vector<PJRT_Buffer*>* outputs) {
    PJRT_ExecuteOptions opts{};
    opts.struct_size = PJRT_ExecuteOptions_STRUCT_SIZE;
    PJRT_Buffer* const* arg_list = inputs.data();
    PJRT_Buffer** out_list = outputs->data();
    PJRT_Event* done = nullptr;
    PJRT_LoadedExecutable_Execute_Args a{};
    a.struct_size = PJRT_LoadedExecutable_Execute_Args_STRUCT_SIZE;
    a.executable = exe;
    a.options = &opts;
    a.argument_lists = &arg_list;
    a.num_devices = 1;
    a.num_args = inputs.size();
    a.output_lists = &out_list;
    a.device_complete_events = &done;
    std::string e = take_error(api->PJRT_LoadedExecutable_Execute(&a));
    if (e.empty() && done) {
        PJRT_Event_Await_Args w{};
        w.struct_size = PJRT_Event_Await_Args_STRUCT_SIZE;
        w.event = done;
        e = take_error(api->PJRT_Event_Await(&w));
    }
    destroy_event(done);
    return e;
}

static std::string add_module(int n) {
    const std::string t = "tensor<" + std::to_string(n) + "xf32>";
    return "module @m {\n  func.func @main(%arg0: " + t + ", %arg1: " + t + ") -> (" + t + ") {\n    %0 = stablehlo.add %arg0, %arg1 : " + t +
           "\n    return %0 : " + t + "\n  }\n}\n";
}

// ---- cases that need no GPU ----
static void host_cases() {
    report("api_version", api->pjrt_api_version.major_version == PJRT_API_MAJOR && api->pjrt_api_version.minor_version == PJRT_API_MINOR &&
                              api->struct_size == PJRT_Api_STRUCT_SIZE,
           "version " + std::to_string(api->pjrt_api_version.major_version) + "." + std::to_string(api->pjrt_api_version.minor_version));
    const bool populated = api->PJRT_Error_Destroy && api->PJRT_Error_Message && api->PJRT_Error_GetCode && api->PJRT_Plugin_Initialize &&
                           api->PJRT_Event_Await && api->PJRT_Event_OnReady && api->PJRT_Client_Create && api->PJRT_Client_Destroy &&
                           api->PJRT_Client_Compile && api->PJRT_Client_BufferFromHostBuffer && api->PJRT_LoadedExecutable_Execute &&
                           api->PJRT_Buffer_ToHostBuffer && api->PJRT_Buffer_Destroy && api->PJRT_Executable_Serialize &&
                           api->PJRT_Executable_DeserializeAndLoad && api->PJRT_Client_TopologyDescription && api->PJRT_Device_MemoryStats &&
                           api->PJRT_Memory_Kind && api->PJRT_Buffer_CopyRawToHost && api->PJRT_LoadedExecutable_GetDeviceAssignment;
    report("required_functions", populated, "a required table entry is NULL");

    // error lifecycle: a call that must fail, then message, code, destroy
    PJRT_Error_GetCode_Args bad{};
    bad.struct_size = PJRT_Error_GetCode_Args_STRUCT_SIZE;
    PJRT_Error* e = api->PJRT_Error_GetCode(&bad);  // NULL error inside
    bool ok = e != nullptr;
    std::string msg;
    if (e) {
        PJRT_Error_GetCode_Args code{};
        code.struct_size = PJRT_Error_GetCode_Args_STRUCT_SIZE;
        code.error = e;
        PJRT_Error* e2 = api->PJRT_Error_GetCode(&code);
        ok = e2 == nullptr && code.code == PJRT_Error_Code_INVALID_ARGUMENT;
        msg = take_error(e);
        ok = ok && msg == "NULL error";
    }
    report("error_lifecycle", ok, "message '" + msg + "'");

    PJRT_Plugin_Initialize_Args init{};
    init.struct_size = PJRT_Plugin_Initialize_Args_STRUCT_SIZE;
    report("plugin_initialize", take_error(api->PJRT_Plugin_Initialize(&init)).empty());

    PJRT_TopologyDescription_PlatformName_Args tn{};
    tn.struct_size = PJRT_TopologyDescription_PlatformName_Args_STRUCT_SIZE;
    std::string te = take_error(api->PJRT_TopologyDescription_PlatformName(&tn));
    report("topology_platform_name", te.empty() && std::string(tn.platform_name, tn.platform_name_size) == "metalhlo", te);

    PJRT_Executable_DeserializeAndLoad_Args d{};
    d.struct_size = PJRT_Executable_DeserializeAndLoad_Args_STRUCT_SIZE;
    std::string de = take_error(api->PJRT_Executable_DeserializeAndLoad(&d));
    report("deserialize_rejects_null", !de.empty(), "no error for NULL client");
}

// ---- cases on the GPU ----
static bool on_ready_fired = false;

static void device_cases() {
    PJRT_Client_Create_Args cc{};
    cc.struct_size = PJRT_Client_Create_Args_STRUCT_SIZE;
    std::string e = take_error(api->PJRT_Client_Create(&cc));
    report("client_create", e.empty() && cc.client, e);
    if (!cc.client) return;
    PJRT_Client* c = cc.client;

    PJRT_Client_PlatformName_Args pn{};
    pn.struct_size = PJRT_Client_PlatformName_Args_STRUCT_SIZE;
    pn.client = c;
    e = take_error(api->PJRT_Client_PlatformName(&pn));
    report("platform_name", e.empty() && std::string(pn.platform_name, pn.platform_name_size) == "metalhlo", e);

    PJRT_Client_Devices_Args dv{};
    dv.struct_size = PJRT_Client_Devices_Args_STRUCT_SIZE;
    dv.client = c;
    e = take_error(api->PJRT_Client_Devices(&dv));
    report("one_device", e.empty() && dv.num_devices == 1, e);

    // device attributes: ane_available (int64) and device_policy (string) are always published
    bool found_ane = false, found_policy = false;
    if (dv.num_devices == 1) {
        PJRT_Device_GetDescription_Args gd{};
        gd.struct_size = PJRT_Device_GetDescription_Args_STRUCT_SIZE;
        gd.device = dv.devices[0];
        api->PJRT_Device_GetDescription(&gd);
        PJRT_DeviceDescription_Attributes_Args at{};
        at.struct_size = PJRT_DeviceDescription_Attributes_Args_STRUCT_SIZE;
        at.device_description = gd.device_description;
        e = take_error(api->PJRT_DeviceDescription_Attributes(&at));
        for (size_t i = 0; i < at.num_attributes; ++i) {
            const std::string name(at.attributes[i].name, at.attributes[i].name_size);
            if (name == "ane_available") found_ane = at.attributes[i].type == PJRT_NamedValue_kInt64 && at.attributes[i].int64_value == 0;
            if (name == "device_policy") found_policy = at.attributes[i].type == PJRT_NamedValue_kString && at.attributes[i].value_size > 0;
        }
        PJRT_Device_DefaultMemory_Args dm{};
        dm.struct_size = PJRT_Device_DefaultMemory_Args_STRUCT_SIZE;
        dm.device = dv.devices[0];
        api->PJRT_Device_DefaultMemory(&dm);
        PJRT_Memory_Kind_Args mk{};
        mk.struct_size = PJRT_Memory_Kind_Args_STRUCT_SIZE;
        mk.memory = dm.memory;
        std::string me = dm.memory ? take_error(api->PJRT_Memory_Kind(&mk)) : "no default memory";
        report("memory_kind_device", me.empty() && std::string(mk.kind, mk.kind_size) == "device", me);
    }
    report("device_attributes", found_ane && found_policy, "ane_available / device_policy missing");

    // host -> device -> host round trip
    const float src[4] = {1.f, 2.f, 3.f, 4.f};
    PJRT_Buffer* b = make_buffer(c, src, PJRT_Buffer_Type_F32, {4}, nullptr, &e);
    bool ok = b != nullptr && e.empty();
    if (ok) {
        PJRT_Buffer_ElementType_Args et{};
        et.struct_size = PJRT_Buffer_ElementType_Args_STRUCT_SIZE;
        et.buffer = b;
        api->PJRT_Buffer_ElementType(&et);
        float back[4] = {0, 0, 0, 0};
        e = read_buffer(b, back, sizeof back);
        ok = e.empty() && et.type == PJRT_Buffer_Type_F32 && std::memcmp(src, back, sizeof src) == 0;
    }
    report("buffer_round_trip", ok, e);

    // the ready event: complete, awaitable, and OnReady fires at once
    if (b) {
        PJRT_Buffer_ReadyEvent_Args re{};
        re.struct_size = PJRT_Buffer_ReadyEvent_Args_STRUCT_SIZE;
        re.buffer = b;
        e = take_error(api->PJRT_Buffer_ReadyEvent(&re));
        PJRT_Event_OnReady_Args on{};
        on.struct_size = PJRT_Event_OnReady_Args_STRUCT_SIZE;
        on.event = re.event;
        on.callback = [](PJRT_Error* err, void* flag) {
            *static_cast<bool*>(flag) = err == nullptr;
        };
        on.user_arg = &on_ready_fired;
        if (e.empty()) e = take_error(api->PJRT_Event_OnReady(&on));
        destroy_event(re.event);
        report("event_on_ready", e.empty() && on_ready_fired, e);
    }

    // strided host data (a transposed view of a 2x3 matrix) lands dense and row-major
    {
        const float m[6] = {1, 2, 3, 4, 5, 6};  // 2x3 row-major
        const int64_t strides[2] = {4, 12};     // read it as 3x2 = its transpose
        PJRT_Buffer* t = make_buffer(c, m, PJRT_Buffer_Type_F32, {3, 2}, strides, &e);
        float back[6] = {};
        if (t && e.empty()) e = read_buffer(t, back, sizeof back);
        const float want[6] = {1, 4, 2, 5, 3, 6};
        report("strided_host_buffer", t && e.empty() && std::memcmp(back, want, sizeof want) == 0, e);
        destroy_buffer(t);
    }

    // raw partial copy and its range check
    if (b) {
        float two[2] = {0, 0};
        PJRT_Buffer_CopyRawToHost_Args raw{};
        raw.struct_size = PJRT_Buffer_CopyRawToHost_Args_STRUCT_SIZE;
        raw.buffer = b;
        raw.dst = two;
        raw.offset = 4;
        raw.transfer_size = 8;
        e = take_error(api->PJRT_Buffer_CopyRawToHost(&raw));
        destroy_event(raw.event);
        bool raw_ok = e.empty() && two[0] == 2.f && two[1] == 3.f;
        raw.offset = 12;
        raw.event = nullptr;
        PJRT_Error* over = api->PJRT_Buffer_CopyRawToHost(&raw);
        PJRT_Error_GetCode_Args code{};
        code.struct_size = PJRT_Error_GetCode_Args_STRUCT_SIZE;
        code.error = over;
        if (over) api->PJRT_Error_GetCode(&code);
        raw_ok = raw_ok && over && code.code == PJRT_Error_Code_OUT_OF_RANGE;
        take_error(over);
        report("copy_raw_to_host", raw_ok, e);
    }

    // compile + execute stablehlo.add: [1,2,3,4] + [5,6,7,8] = [6,8,10,12]
    PJRT_LoadedExecutable* exe = compile(c, add_module(4), &e);
    report("compile_add", exe != nullptr, e);
    if (exe && b) {
        const float rhs[4] = {5.f, 6.f, 7.f, 8.f};
        std::string e2;
        PJRT_Buffer* b2 = make_buffer(c, rhs, PJRT_Buffer_Type_F32, {4}, nullptr, &e2);
        std::vector<PJRT_Buffer*> outs(1, nullptr);
        e = b2 ? execute(exe, {b, b2}, &outs) : e2;
        float got[4] = {};
        if (e.empty() && outs[0]) e = read_buffer(outs[0], got, sizeof got);
        report("execute_add", e.empty() && got[0] == 6.f && got[1] == 8.f && got[2] == 10.f && got[3] == 12.f, e);

        // output description of the executable
        PJRT_LoadedExecutable_GetExecutable_Args ge{};
        ge.struct_size = PJRT_LoadedExecutable_GetExecutable_Args_STRUCT_SIZE;
        ge.loaded_executable = exe;
        e = take_error(api->PJRT_LoadedExecutable_GetExecutable(&ge));
        if (ge.executable) {
            PJRT_Executable_NumOutputs_Args no{};
            no.struct_size = PJRT_Executable_NumOutputs_Args_STRUCT_SIZE;
            no.executable = ge.executable;
            api->PJRT_Executable_NumOutputs(&no);
            PJRT_Executable_OutputDimensions_Args od{};
            od.struct_size = PJRT_Executable_OutputDimensions_Args_STRUCT_SIZE;
            od.executable = ge.executable;
            api->PJRT_Executable_OutputDimensions(&od);
            PJRT_Executable_OutputElementTypes_Args ot{};
            ot.struct_size = PJRT_Executable_OutputElementTypes_Args_STRUCT_SIZE;
            ot.executable = ge.executable;
            api->PJRT_Executable_OutputElementTypes(&ot);
            report("executable_outputs", no.num_outputs == 1 && od.num_outputs == 1 && od.dim_sizes[0] == 1 && od.dims[0] == 4 &&
                                             ot.num_output_types == 1 && ot.output_types[0] == PJRT_Buffer_Type_F32,
                   "wrong output description");

            // serialize -> deserialize -> execute: [3,5] + [5,10] = [8,15] in the reference's test; here the same program
            PJRT_Executable_Serialize_Args se{};
            se.struct_size = PJRT_Executable_Serialize_Args_STRUCT_SIZE;
            se.executable = ge.executable;
            e = take_error(api->PJRT_Executable_Serialize(&se));
            bool ser_ok = e.empty() && se.serialized_bytes_size > 12;
            uint32_t version = 0;
            uint64_t length = 0;
            if (ser_ok) {
                std::memcpy(&version, se.serialized_bytes, 4);
                std::memcpy(&length, se.serialized_bytes + 4, 8);
                ser_ok = version == 1 && length == se.serialized_bytes_size - 12;
            }
            report("serialize_format", ser_ok, e);
            if (ser_ok) {
                PJRT_Executable_DeserializeAndLoad_Args dl{};
                dl.struct_size = PJRT_Executable_DeserializeAndLoad_Args_STRUCT_SIZE;
                dl.client = c;
                dl.serialized_executable = se.serialized_bytes;
                dl.serialized_executable_size = se.serialized_bytes_size;
                e = take_error(api->PJRT_Executable_DeserializeAndLoad(&dl));
                std::vector<PJRT_Buffer*> outs2(1, nullptr);
                if (e.empty() && dl.loaded_executable) e = execute(dl.loaded_executable, {b2, b2}, &outs2);
                float got2[4] = {};
                if (e.empty() && outs2[0]) e = read_buffer(outs2[0], got2, sizeof got2);
                report("deserialize_and_execute", e.empty() && got2[0] == 10.f && got2[3] == 16.f, e);
                destroy_buffer(outs2[0]);
                destroy_loaded(dl.loaded_executable);
            }
            PJRT_Executable_Fingerprint_Args fp{};
            fp.struct_size = PJRT_Executable_Fingerprint_Args_STRUCT_SIZE;
            fp.executable = ge.executable;
            e = take_error(api->PJRT_Executable_Fingerprint(&fp));
            report("fingerprint", e.empty() && fp.executable_fingerprint_size == 16, e);
            PJRT_Executable_Destroy_Args xd{};
            xd.struct_size = PJRT_Executable_Destroy_Args_STRUCT_SIZE;
            xd.executable = ge.executable;
            api->PJRT_Executable_Destroy(&xd);
        }
        destroy_buffer(outs[0]);
        destroy_buffer(b2);
    }

    // a fused program through the plugin: softmax over rows of a 64 x 512 matrix (rows sum to one, ordering kept)
    {
        const int rows = 64, cols = 512;
        const std::string t = "tensor<64x512xf32>", r = "tensor<64xf32>";
        const std::string text =
            "module @s {\n  func.func @main(%x: " + t + ") -> (" + t + ") {\n"
            "    %ninf = stablehlo.constant dense<0xFF800000> : tensor<f32>\n"
            "    %zero = stablehlo.constant dense<0.0> : tensor<f32>\n"
            "    %mx = stablehlo.reduce(%x init: %ninf) applies stablehlo.maximum across dimensions = [1] : (" + t + ", tensor<f32>) -> " + r + "\n"
            "    %mb = stablehlo.broadcast_in_dim %mx, dims = [0] : (" + r + ") -> " + t + "\n"
            "    %d = stablehlo.subtract %x, %mb : " + t + "\n"
            "    %ex = stablehlo.exponential %d : " + t + "\n"
            "    %s = stablehlo.reduce(%ex init: %zero) applies stablehlo.add across dimensions = [1] : (" + t + ", tensor<f32>) -> " + r + "\n"
            "    %sb = stablehlo.broadcast_in_dim %s, dims = [0] : (" + r + ") -> " + t + "\n"
            "    %y = stablehlo.divide %ex, %sb : " + t + "\n"
            "    return %y : " + t + "\n  }\n}\n";
        std::vector<float> x(static_cast<size_t>(rows) * cols), y(x.size());
        for (size_t i = 0; i < x.size(); ++i) x[i] = std::sin(0.37f * static_cast<float>(i)) * 3.f;
        PJRT_LoadedExecutable* sm = compile(c, text, &e);
        PJRT_Buffer* xb = sm ? make_buffer(c, x.data(), PJRT_Buffer_Type_F32, {rows, cols}, nullptr, &e) : nullptr;
        std::vector<PJRT_Buffer*> outs(1, nullptr);
        if (sm && xb) e = execute(sm, {xb}, &outs);
        if (e.empty() && outs[0]) e = read_buffer(outs[0], y.data(), y.size() * sizeof(float));
        double worst = 0;
        if (e.empty())
            for (int i = 0; i < rows; ++i) {
                double mx = -1e30, sum = 0;
                for (int j = 0; j < cols; ++j) mx = std::max(mx, static_cast<double>(x[static_cast<size_t>(i) * cols + j]));
                for (int j = 0; j < cols; ++j) sum += std::exp(x[static_cast<size_t>(i) * cols + j] - mx);
                for (int j = 0; j < cols; ++j) {
                    const double want = std::exp(x[static_cast<size_t>(i) * cols + j] - mx) / sum;
                    worst = std::max(worst, std::fabs(y[static_cast<size_t>(i) * cols + j] - want) / (std::fabs(want) + 1e-12));
                }
            }
        report("execute_softmax", sm && e.empty() && worst < 1e-5, e.empty() ? "worst relative error " + std::to_string(worst) : e);
        destroy_buffer(outs[0]);
        destroy_buffer(xb);
        destroy_loaded(sm);
    }

    // the module shape jax.jit prints: @main calls a private function from inside a counted loop. Three trips of
    // x -> 2 * x + 1 take [1, 2, 3, 4] to [15, 23, 31, 39].
    {
        const std::string text =
            "module @jit_f attributes {mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {\n"
            "  func.func public @main(%arg0: tensor<4xf32>) -> (tensor<4xf32> {jax.result_info = \"\"}) {\n"
            "    %c = stablehlo.constant dense<0> : tensor<i32>\n"
            "    %0:2 = stablehlo.while(%iterArg = %c, %iterArg_0 = %arg0) : tensor<i32>, tensor<4xf32>\n"
            "     cond {\n"
            "      %c_1 = stablehlo.constant dense<3> : tensor<i32>\n"
            "      %1 = stablehlo.compare  LT, %iterArg, %c_1,  SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>\n"
            "      stablehlo.return %1 : tensor<i1>\n"
            "    } do {\n"
            "      %c_1 = stablehlo.constant dense<1> : tensor<i32>\n"
            "      %1 = stablehlo.add %iterArg, %c_1 : tensor<i32>\n"
            "      %2 = call @step(%iterArg_0) : (tensor<4xf32>) -> tensor<4xf32>\n"
            "      stablehlo.return %1, %2 : tensor<i32>, tensor<4xf32>\n"
            "    }\n"
            "    return %0#1 : tensor<4xf32>\n"
            "  }\n"
            "  func.func private @step(%arg0: tensor<4xf32>) -> tensor<4xf32> {\n"
            "    %cst = stablehlo.constant dense<2.000000e+00> : tensor<4xf32>\n"
            "    %cst_0 = stablehlo.constant dense<1.000000e+00> : tensor<4xf32>\n"
            "    %0 = stablehlo.multiply %arg0, %cst : tensor<4xf32>\n"
            "    %1 = stablehlo.add %0, %cst_0 : tensor<4xf32>\n"
            "    return %1 : tensor<4xf32>\n"
            "  }\n"
            "}\n";
        PJRT_LoadedExecutable* loop = compile(c, text, &e);
        const float in4[4] = {1.f, 2.f, 3.f, 4.f};
        std::string e2;
        PJRT_Buffer* xb = loop ? make_buffer(c, in4, PJRT_Buffer_Type_F32, {4}, nullptr, &e2) : nullptr;
        std::vector<PJRT_Buffer*> outs(1, nullptr);
        if (loop && xb) e = execute(loop, {xb}, &outs);
        float got[4] = {};
        if (e.empty() && outs[0]) e = read_buffer(outs[0], got, sizeof got);
        report("execute_loop_with_call", loop && e.empty() && got[0] == 15.f && got[1] == 23.f && got[2] == 31.f && got[3] == 39.f, e + e2);
        destroy_buffer(outs[0]);
        destroy_buffer(xb);
        destroy_loaded(loop);
    }

    // complex values: a C64 argument goes down as (re, im) float pairs, an RFFT spectrum comes back up as C64
    {
        const char* text =
            "module @cx {\n"
            "  func.func @main(%arg0: tensor<8xf32>, %arg1: tensor<5xcomplex<f32>>) -> (tensor<5xcomplex<f32>>, tensor<5xf32>) {\n"
            "    %0 = stablehlo.fft %arg0, type = RFFT, length = [8] : (tensor<8xf32>) -> tensor<5xcomplex<f32>>\n"
            "    %1 = stablehlo.add %0, %arg1 : tensor<5xcomplex<f32>>\n"
            "    %2 = stablehlo.imag %arg1 : (tensor<5xcomplex<f32>>) -> tensor<5xf32>\n"
            "    return %1, %2 : tensor<5xcomplex<f32>>, tensor<5xf32>\n"
            "  }\n"
            "}\n";
        PJRT_LoadedExecutable* cx = compile(c, text, &e);
        const float x8[8] = {1.f, 2.f, 3.f, 4.f, 5.f, 6.f, 7.f, 8.f};
        const float z5[10] = {10.f, 1.f, 20.f, 2.f, 30.f, 3.f, 40.f, 4.f, 50.f, 5.f};  // (re, im) x 5
        std::string e2, e3;
        PJRT_Buffer* xb = cx ? make_buffer(c, x8, PJRT_Buffer_Type_F32, {8}, nullptr, &e2) : nullptr;
        PJRT_Buffer* zb = cx ? make_buffer(c, z5, PJRT_Buffer_Type_C64, {5}, nullptr, &e3) : nullptr;
        bool ok = cx && xb && zb;
        if (ok) {
            PJRT_Buffer_ElementType_Args et{};
            et.struct_size = PJRT_Buffer_ElementType_Args_STRUCT_SIZE;
            et.buffer = zb;
            api->PJRT_Buffer_ElementType(&et);
            PJRT_Buffer_Dimensions_Args dm{};
            dm.struct_size = PJRT_Buffer_Dimensions_Args_STRUCT_SIZE;
            dm.buffer = zb;
            api->PJRT_Buffer_Dimensions(&dm);
            ok = et.type == PJRT_Buffer_Type_C64 && dm.num_dims == 1 && dm.dims[0] == 5;
        }
        std::vector<PJRT_Buffer*> outs(2, nullptr);
        if (ok) e = execute(cx, {xb, zb}, &outs);
        float spec[10] = {}, im[5] = {};
        if (ok && e.empty() && outs[0]) e = read_buffer(outs[0], spec, sizeof spec);
        if (ok && e.empty() && outs[1]) e = read_buffer(outs[1], im, sizeof im);
        if (ok && e.empty()) {
            PJRT_Buffer_ElementType_Args et{};
            et.struct_size = PJRT_Buffer_ElementType_Args_STRUCT_SIZE;
            et.buffer = outs[0];
            api->PJRT_Buffer_ElementType(&et);
            PJRT_Buffer_Dimensions_Args dm{};
            dm.struct_size = PJRT_Buffer_Dimensions_Args_STRUCT_SIZE;
            dm.buffer = outs[0];
            api->PJRT_Buffer_Dimensions(&dm);
            // bin 0 of the spectrum is the sum (36), bin 4 the alternating sum (-4); both real
            ok = et.type == PJRT_Buffer_Type_C64 && dm.num_dims == 1 && dm.dims[0] == 5 && std::fabs(spec[0] - 46.f) < 1e-4f &&
                 std::fabs(spec[1] - 1.f) < 1e-4f && std::fabs(spec[8] - 46.f) < 1e-4f && std::fabs(spec[9] - 5.f) < 1e-4f && im[2] == 3.f;
        }
        report("complex_buffers_and_rfft", ok && e.empty(), e + e2 + e3);
        destroy_buffer(outs[0]);
        destroy_buffer(outs[1]);
        destroy_buffer(xb);
        destroy_buffer(zb);
        destroy_loaded(cx);
    }

    // compile errors surface as PJRT errors with the compiler's message
    {
        PJRT_LoadedExecutable* badexe = compile(c, "module { func.func @main() -> tensor<f32> { %0 = stablehlo.nonsense : tensor<f32> return %0 : tensor<f32> } }", &e);
        report("compile_error_reported", badexe == nullptr && e.rfind("Compilation failed", 0) == 0, e);
        destroy_loaded(badexe);
        const char bytecode[] = {'M', 'L', '\xEF', 'R', 0, 0, 0, 0};
        PJRT_LoadedExecutable* bc = compile(c, std::string(bytecode, sizeof bytecode), &e);
        report("bytecode_refused", bc == nullptr && e.find("Bytecode") != std::string::npos, e);
    }

    // memory accounting and buffer deletion
    if (dv.num_devices == 1 && b) {
        PJRT_Device_MemoryStats_Args ms{};
        ms.struct_size = PJRT_Device_MemoryStats_Args_STRUCT_SIZE;
        ms.device = dv.devices[0];
        api->PJRT_Device_MemoryStats(&ms);
        const int64_t before = ms.bytes_in_use;
        PJRT_Buffer_Delete_Args del{};
        del.struct_size = PJRT_Buffer_Delete_Args_STRUCT_SIZE;
        del.buffer = b;
        api->PJRT_Buffer_Delete(&del);
        PJRT_Buffer_IsDeleted_Args isd{};
        isd.struct_size = PJRT_Buffer_IsDeleted_Args_STRUCT_SIZE;
        isd.buffer = b;
        api->PJRT_Buffer_IsDeleted(&isd);
        api->PJRT_Device_MemoryStats(&ms);
        report("delete_and_memory_stats", isd.is_deleted && before - ms.bytes_in_use == 16 && ms.bytes_in_use == 0,
               "bytes_in_use " + std::to_string(before) + " -> " + std::to_string(ms.bytes_in_use));
    }
    destroy_buffer(b);
    destroy_loaded(exe);

    PJRT_Client_Destroy_Args cd{};
    cd.struct_size = PJRT_Client_Destroy_Args_STRUCT_SIZE;
    cd.client = c;
    report("client_destroy", take_error(api->PJRT_Client_Destroy(&cd)).empty());
}

int main(int argc, char** argv) {
    if (argc < 3) {
        std::fprintf(stderr, "usage: %s <plugin.so> host|device\n", argv[0]);
        return 64;
    }
    void* lib = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
    if (!lib) {
        std::printf("FAIL load: %s\n", dlerror());
        return 1;
    }
    using GetApi = const PJRT_Api* (*)(void);
    auto get = reinterpret_cast<GetApi>(dlsym(lib, "GetPjrtApi"));
    if (!get || !(api = get())) {
        std::printf("FAIL load: GetPjrtApi missing or returned NULL\n");
        return 1;
    }
    std::printf("PASS load\n");
    host_cases();
    if (std::string(argv[2]) == "device") device_cases();
    std::printf("%d failure(s)\n", failures);
    return failures;
}
