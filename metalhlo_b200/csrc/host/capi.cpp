// The mhlo_* C API (include/metalhlo.h) over the C++ compiler core and libmhlo_cuda.so. Behaviour follows
// Sources/CMetalHLO/CInterface.swift:202-1010: opaque retained handles, MHLOStatusCode returns, a process-global
// last-error string that is NULL when clear, synchronous execution with new output buffers per call, and
// per-executable execution statistics.
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../../include/metalhlo.h"
#include "../../../include/mhlo_cuda.h"
#include "compiler.h"
#include "tuning.h"

using namespace mhlo;

namespace {

std::mutex g_error_mu;
std::string g_error;
bool g_has_error = false;

int set_error(int code, const std::string& msg) {
    std::lock_guard<std::mutex> lock(g_error_mu);
    g_error = msg;
    g_has_error = true;
    return code;
}

struct Client {
    // METALHLO_SHARD_COUNT / METALHLO_SHARD_INDEX: every program this client compiles is split over that many equal
    // batch shards and this client builds and runs the shard with that index (one process per GPU, one shard each).
    int shard_count = 1, shard_index = 0;
    int device = 0;
    void* stream = nullptr;
    void* copy_stream = nullptr;  // device-to-host transfers that run beside the next program (mhlo_b200_buffer_to_host_async)
    void* copy_fence = nullptr;   // event that orders such a transfer behind the work already queued on `stream`
    std::mutex mu;
    // in-process executable cache keyed by (text, level): MetalHLOCompiler.swift:730-782 keeps the same
    std::map<std::string, std::shared_ptr<Executable>> cache;
    int64_t cache_hits = 0, cache_misses = 0;
    // Device memory of destroyed buffers, kept for the next buffer of the same size: a serving loop creates and destroys
    // the same few shapes over and over, and cudaMalloc / cudaFree cost far more than the transfers they bracket are
    // allowed to (the reference allocates and zero-fills per call, IntegratedExecutor.swift:170-215).
    // Bounded by METALHLO_BUFFER_POOL_MB (default 8192, 0 = off); everything goes back to the driver with the client.
    std::multimap<size_t, void*> pool;
    size_t pooled_bytes = 0, pool_limit = 0;
};

size_t pool_limit_from_env() {
    const char* v = std::getenv("METALHLO_BUFFER_POOL_MB");
    const long long mb = v && *v ? std::atoll(v) : 8192;
    return mb <= 0 ? 0 : static_cast<size_t>(mb) << 20;
}

// Takes exactly `bytes` from the pool or the driver. Pool memory was released only after its client's stream had
// drained, so it is free of pending work.
int pool_alloc(Client* c, size_t bytes, void** out) {
    {
        std::lock_guard<std::mutex> lock(c->mu);
        auto it = c->pool.find(bytes);
        if (it != c->pool.end()) {
            *out = it->second;
            c->pooled_bytes -= bytes;
            c->pool.erase(it);
            return 0;
        }
    }
    int st = mhlo_cuda_alloc(bytes, out);
    if (st != 0) {
        // out of memory with blocks parked in the pool: give them back and try once more
        std::multimap<size_t, void*> drained;
        {
            std::lock_guard<std::mutex> lock(c->mu);
            drained.swap(c->pool);
            c->pooled_bytes = 0;
        }
        if (drained.empty()) return st;
        for (auto& kv : drained) mhlo_cuda_free(kv.second);
        st = mhlo_cuda_alloc(bytes, out);
    }
    return st;
}

void pool_release(Client* c, void* dev, size_t bytes) {
    if (!dev) return;
    {
        std::lock_guard<std::mutex> lock(c->mu);
        // (blocks of a few KB are cheap to allocate afresh; anything larger is kept: cudaFree waits for the whole device,
        // a transfer on the copy stream included, which is exactly what a serving loop's per-step input buffer must not do)
        if (bytes >= 4096 && c->pooled_bytes + bytes <= c->pool_limit) {
            c->pool.emplace(bytes, dev);
            c->pooled_bytes += bytes;
            return;
        }
    }
    mhlo_cuda_free(dev);
}

struct ExecutableHandle {
    Client* client;
    std::shared_ptr<Executable> exe;
    ExecutionStats stats;
};

struct Buffer {
    Client* client;
    void* dev = nullptr;
    TensorType type;
    size_t bytes = 0;
    void* copy_done = nullptr;  // recorded behind the latest asynchronous transfer out of this buffer
};

// I1 tensors occupy one byte per element on the device (mhlo_element_type_size reports 0 for I1, as the
// reference does, so callers size bool buffers themselves).
size_t buffer_bytes(const TensorType& t) { return static_cast<size_t>(t.bytes()); }

MHLOStatusCode make_buffer(Client* c, const TensorType& t, Buffer** out) {
    std::unique_ptr<Buffer> b(new Buffer());
    b->client = c;
    b->type = t;
    b->bytes = buffer_bytes(t);
    if (mhlo_cuda_device_set(c->device) != 0) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_NO_DEVICE, mhlo_cuda_last_error()));
    if (b->bytes > 0 && pool_alloc(c, b->bytes, &b->dev) != 0)
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_BUFFER_FAILED, mhlo_cuda_last_error()));
    *out = b.release();
    return MHLO_OK;
}

bool valid_dtype(int t) { return t >= 0 && t <= 12; }

MHLOStatusCode run(ExecutableHandle* h, const MHLOBufferRef* inputs, int32_t num_inputs, MHLOBufferRef* out_outputs,
                   int32_t* out_num_outputs, double* encode_s, double* gpu_s, double* total_s) {
    if (!h) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "executable is null"));
    if (!out_outputs) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "out_outputs is null"));
    if (!out_num_outputs) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "out_num_outputs is null"));
    Executable& exe = *h->exe;
    Client* c = h->client;
    if (num_inputs != exe.num_inputs())
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INPUT_MISMATCH, "Input count mismatch: expected " +
                                                     std::to_string(exe.num_inputs()) + ", got " + std::to_string(num_inputs)));
    std::vector<const void*> in_ptrs(static_cast<size_t>(num_inputs));
    for (int i = 0; i < num_inputs; ++i) {
        if (!inputs || !inputs[i]) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "Input " + std::to_string(i) + " is null"));
        const Buffer* b = static_cast<const Buffer*>(inputs[i]);
        if (b->type != exe.input_type(i))
            return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INPUT_MISMATCH, "Input " + std::to_string(i) + " is " + b->type.str() +
                                                         ", executable expects " + exe.input_type(i).str()));
        in_ptrs[static_cast<size_t>(i)] = b->dev;
    }
    {
        std::lock_guard<std::mutex> lock(g_error_mu);
        g_has_error = false;
    }
    const auto t0 = std::chrono::steady_clock::now();
    if (mhlo_cuda_device_set(c->device) != 0) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_NO_DEVICE, mhlo_cuda_last_error()));
    std::vector<Buffer*> outs;
    std::vector<void*> out_ptrs;
    auto cleanup = [&]() { for (Buffer* b : outs) { pool_release(b->client, b->dev, b->bytes); delete b; } };
    for (int i = 0; i < exe.num_outputs(); ++i) {
        Buffer* b = nullptr;
        MHLOStatusCode st = make_buffer(c, exe.output_type(i), &b);
        if (st != MHLO_OK) { cleanup(); return st; }
        outs.push_back(b);
        out_ptrs.push_back(b->dev);
    }
    void *ev0 = nullptr, *ev1 = nullptr;
    const bool timed = gpu_s != nullptr;
    if (timed) { mhlo_cuda_event_create(&ev0); mhlo_cuda_event_create(&ev1); mhlo_cuda_event_record(ev0, c->stream); }
    int st;
    bool words = false;
    std::chrono::steady_clock::time_point t1;
    {
        std::lock_guard<std::mutex> lock(c->mu);  // one caller at a time on the client's stream and arena, until the stream has drained
        st = exe.execute(in_ptrs.data(), out_ptrs.data(), c->stream);
        t1 = std::chrono::steady_clock::now();
        if (timed) mhlo_cuda_event_record(ev1, c->stream);
        // The tensor-core kernels bound every wait and record a code instead of hanging; the words ride back behind the
        // program on the same stream, so a kernel that gave up fails this call instead of returning partly written outputs.
        words = st == 0 && mhlo_cuda_device_error_fetch(c->stream) == 0;
        if (st == 0 && mhlo_cuda_stream_sync(c->stream) != 0) { st = MHLO_ERROR_EXECUTION_FAILED; set_error(st, mhlo_cuda_last_error()); }
        else if (st != 0) set_error(st, exe.last_error());
    }
    if (st == 0 && words) {
        int32_t code = 0;
        if (mhlo_cuda_device_error_take(&code) != 0 && code != 0) {
            st = MHLO_ERROR_EXECUTION_FAILED;
            set_error(st, std::string("Execution failed: ") + mhlo_cuda_last_error());
        }
    }
    if (timed) {
        float ms = 0;
        if (st == 0) mhlo_cuda_event_elapsed_ms(ev0, ev1, &ms);
        *gpu_s = ms * 1e-3;
        mhlo_cuda_event_destroy(ev0);
        mhlo_cuda_event_destroy(ev1);
    }
    if (st != 0) { cleanup(); return static_cast<MHLOStatusCode>(st); }
    const auto t2 = std::chrono::steady_clock::now();
    const double total = std::chrono::duration<double>(t2 - t0).count();
    if (encode_s) *encode_s = std::chrono::duration<double>(t1 - t0).count();
    if (total_s) *total_s = total;
    h->stats.count += 1;
    h->stats.last_ms = total * 1e3;
    h->stats.total_ms += total * 1e3;
    *out_num_outputs = static_cast<int32_t>(outs.size());
    for (size_t i = 0; i < outs.size(); ++i) out_outputs[i] = outs[i];
    return MHLO_OK;
}

MHLOStatusCode compile_impl(Client* c, const std::string& text, const MHLOCompileConfig* config, MHLOExecutableRef* out,
                            const ShardSpec* shard = nullptr) {
    if (!c) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "client is null"));
    if (!out) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "out_executable is null"));
    *out = nullptr;
    CompileOptions opt;
    if (shard) opt.shard = *shard;
    else { opt.shard.count = c->shard_count; opt.shard.index = c->shard_index; }
    if (config) {
        if (config->optimization_level < 0 || config->optimization_level > 3)
            return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "optimization_level out of range"));
        opt.opt_level = config->optimization_level;
        opt.enable_caching = config->enable_caching;
        opt.enable_debug_info = config->enable_debug_info;
    }
    if (const char* env = std::getenv("METALHLO_OPT_LEVEL"))
        if (!config && env[0] >= '0' && env[0] <= '3') opt.opt_level = env[0] - '0';
    if (mhlo_cuda_device_set(c->device) != 0) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_NO_DEVICE, mhlo_cuda_last_error()));
    std::string key = std::to_string(opt.opt_level) + "|" + std::to_string(opt.shard.count) + "/" + std::to_string(opt.shard.index) + ":";
    for (int a : opt.shard.input_axes) key += std::to_string(a) + ",";
    key += "|" + text;
    std::shared_ptr<Executable> exe;
    {
        std::lock_guard<std::mutex> lock(c->mu);
        if (opt.enable_caching) {
            auto it = c->cache.find(key);
            if (it != c->cache.end()) { exe = it->second; ++c->cache_hits; }
        }
    }
    if (!exe) {
        try {
            exe = std::shared_ptr<Executable>(Executable::compile(text, opt).release());
        } catch (const CompileError& e) {
            return static_cast<MHLOStatusCode>(set_error(e.code, e.what()));
        } catch (const std::exception& e) {
            return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_COMPILATION_FAILED, e.what()));
        }
        std::lock_guard<std::mutex> lock(c->mu);
        ++c->cache_misses;
        if (opt.enable_caching) c->cache[key] = exe;
    }
    ExecutableHandle* h = new ExecutableHandle();
    h->client = c;
    h->exe = exe;
    *out = h;
    return MHLO_OK;
}

}  // namespace

extern "C" {

const char* mhlo_version(void) { return "0.2.0"; }

const char* mhlo_get_last_error(void) {
    std::lock_guard<std::mutex> lock(g_error_mu);
    return g_has_error ? g_error.c_str() : nullptr;
}

void mhlo_clear_error(void) {
    std::lock_guard<std::mutex> lock(g_error_mu);
    g_has_error = false;
    g_error.clear();
}

size_t mhlo_element_type_size(MHLOElementType type) {
    if (type == MHLO_I1) return 0;
    return valid_dtype(type) ? dtype_size(static_cast<DType>(type)) : 0;
}

void mhlo_free_string(const char* str) { std::free(const_cast<char*>(str)); }

static MHLOStatusCode client_create_impl(MHLOClientRef* out_client, int forced_device);

MHLOStatusCode mhlo_client_create(MHLOClientRef* out_client) { return client_create_impl(out_client, -1); }

// A client bound to CUDA device `device_ordinal` (mhlo_client_create takes METALHLO_DEVICE / LOCAL_RANK, else device 0).
// One process may hold one client per GPU: each has its own stream, buffer pool and executable cache.
MHLOStatusCode mhlo_b200_client_create_on_device(int32_t device_ordinal, MHLOClientRef* out_client) {
    if (device_ordinal < 0) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "negative device ordinal"));
    return client_create_impl(out_client, device_ordinal);
}

int32_t mhlo_b200_device_count(void) {
    int n = 0;
    return mhlo_cuda_device_count(&n) == 0 ? n : 0;
}

static MHLOStatusCode client_create_impl(MHLOClientRef* out_client, int forced_device) {
    if (!out_client) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "out_client is null"));
    *out_client = nullptr;
    int n = 0;
    if (mhlo_cuda_device_count(&n) != 0 || n == 0)
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_NO_DEVICE, std::string("No CUDA device available: ") + mhlo_cuda_last_error()));
    std::unique_ptr<Client> c(new Client());
    c->pool_limit = pool_limit_from_env();
    // one process drives one GPU: LOCAL_RANK picks it when several ranks share a box
    if (const char* sc = std::getenv("METALHLO_SHARD_COUNT")) {
        c->shard_count = std::atoi(sc);
        if (const char* si = std::getenv("METALHLO_SHARD_INDEX")) c->shard_index = std::atoi(si);
        if (c->shard_count < 1 || c->shard_index < 0 || c->shard_index >= c->shard_count)
            return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "METALHLO_SHARD_COUNT / METALHLO_SHARD_INDEX out of range"));
    }
    if (forced_device >= 0) {
        if (forced_device >= n)
            return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_NO_DEVICE, "CUDA device " + std::to_string(forced_device) + " does not exist (" +
                                                         std::to_string(n) + " visible)"));
        c->device = forced_device;
    } else if (const char* lr = std::getenv("METALHLO_DEVICE")) c->device = std::atoi(lr);
    else if (const char* lr2 = std::getenv("LOCAL_RANK")) c->device = std::atoi(lr2) % n;
    if (c->device < 0 || c->device >= n) c->device = 0;
    if (mhlo_cuda_device_set(c->device) != 0 || mhlo_cuda_stream_create(&c->stream) != 0)
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_NO_DEVICE, mhlo_cuda_last_error()));
    *out_client = c.release();
    return MHLO_OK;
}

void mhlo_client_destroy(MHLOClientRef client) {
    Client* c = static_cast<Client*>(client);
    if (!c) return;
    mhlo_cuda_device_set(c->device);
    c->cache.clear();
    for (auto& kv : c->pool) mhlo_cuda_free(kv.second);
    c->pool.clear();
    if (c->copy_stream) { mhlo_cuda_stream_sync(c->copy_stream); mhlo_cuda_stream_destroy(c->copy_stream); }
    if (c->copy_fence) mhlo_cuda_event_destroy(c->copy_fence);
    if (c->stream) mhlo_cuda_stream_destroy(c->stream);
    delete c;
}

char* mhlo_client_device_name(MHLOClientRef client) {
    Client* c = static_cast<Client*>(client);
    if (!c) return nullptr;
    char name[256];
    if (mhlo_cuda_device_name(c->device, name, sizeof name) != 0) return nullptr;
    return strdup(name);
}

void mhlo_compile_config_init(MHLOCompileConfig* out_config) {
    if (!out_config) return;
    out_config->optimization_level = MHLO_OPT_O2;
    out_config->enable_caching = true;
    out_config->enable_debug_info = false;
    out_config->device_policy = MHLO_DEVICE_GPU_ONLY;
}

bool mhlo_ane_available(void) { return false; }

MHLOStatusCode mhlo_compile(MHLOClientRef client, const char* mlir_text, MHLOExecutableRef* out_executable) {
    if (!mlir_text) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "mlir_text is null"));
    return compile_impl(static_cast<Client*>(client), mlir_text, nullptr, out_executable);
}

MHLOStatusCode mhlo_compile_n(MHLOClientRef client, const char* mlir_text, size_t mlir_length, MHLOExecutableRef* out_executable) {
    if (!mlir_text) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "mlir_text is null"));
    if (is_mlir_bytecode(mlir_text, mlir_length)) {
        std::string text, why;
        if (!bytecode_to_text(mlir_text, mlir_length, &text, &why)) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_PARSE_FAILED, why));
        return compile_impl(static_cast<Client*>(client), text, nullptr, out_executable);
    }
    return compile_impl(static_cast<Client*>(client), std::string(mlir_text, mlir_length), nullptr, out_executable);
}

MHLOStatusCode mhlo_compile_with_config(MHLOClientRef client, const char* mlir_text, const MHLOCompileConfig* config,
                                        MHLOExecutableRef* out_executable) {
    if (!mlir_text) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "mlir_text is null"));
    return compile_impl(static_cast<Client*>(client), mlir_text, config, out_executable);
}

void mhlo_executable_destroy(MHLOExecutableRef executable) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    if (!h) return;
    mhlo_cuda_device_set(h->client->device);
    delete h;
}

int32_t mhlo_executable_input_count(MHLOExecutableRef executable) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    return h ? h->exe->num_inputs() : 0;
}

int32_t mhlo_executable_output_count(MHLOExecutableRef executable) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    return h ? h->exe->num_outputs() : 0;
}

static MHLOStatusCode describe(const TensorType& t, int64_t* out_shape, int32_t* out_rank, MHLOElementType* out_type) {
    if (out_shape) for (int d = 0; d < t.rank(); ++d) out_shape[d] = t.shape[d];
    if (out_rank) *out_rank = t.rank();
    if (out_type) *out_type = static_cast<MHLOElementType>(t.dtype);
    return MHLO_OK;
}

MHLOStatusCode mhlo_executable_input_type(MHLOExecutableRef executable, int32_t index, int64_t* out_shape, int32_t* out_rank,
                                          MHLOElementType* out_element_type) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    if (!h) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "executable is null"));
    if (index < 0 || index >= h->exe->num_inputs()) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "Input index out of range"));
    return describe(h->exe->input_type(index), out_shape, out_rank, out_element_type);
}

MHLOStatusCode mhlo_executable_output_type(MHLOExecutableRef executable, int32_t index, int64_t* out_shape, int32_t* out_rank,
                                           MHLOElementType* out_element_type) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    if (!h) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "executable is null"));
    if (index < 0 || index >= h->exe->num_outputs()) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "Output index out of range"));
    return describe(h->exe->output_type(index), out_shape, out_rank, out_element_type);
}

// 1 when input / output `index` was a complex tensor in the program text: its buffer is then the float tensor of
// (re, im) pairs, one dimension longer, that mhlo_executable_{input,output}_type reports. 0 otherwise, -1 for a bad index.
int32_t mhlo_b200_executable_input_is_complex(MHLOExecutableRef executable, int32_t index) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    if (!h || index < 0 || index >= h->exe->num_inputs()) return -1;
    return h->exe->input_type(index).was_complex ? 1 : 0;
}

int32_t mhlo_b200_executable_output_is_complex(MHLOExecutableRef executable, int32_t index) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    if (!h || index < 0 || index >= h->exe->num_outputs()) return -1;
    return h->exe->output_type(index).was_complex ? 1 : 0;
}

MHLOStatusCode mhlo_executable_get_stats(MHLOExecutableRef executable, MHLOExecutionStats* out_stats) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    if (!h) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "executable is null"));
    if (!out_stats) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "out_stats is null"));
    out_stats->execution_count = h->stats.count;
    out_stats->total_execution_time_ms = h->stats.total_ms;
    out_stats->last_execution_time_ms = h->stats.last_ms;
    out_stats->average_execution_time_ms = h->stats.count ? h->stats.total_ms / static_cast<double>(h->stats.count) : 0.0;
    return MHLO_OK;
}

void mhlo_executable_reset_stats(MHLOExecutableRef executable) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    if (h) h->stats = ExecutionStats();
}

MHLOStatusCode mhlo_buffer_create(MHLOClientRef client, const void* data, size_t data_size, const int64_t* shape, int32_t rank,
                                  MHLOElementType element_type, MHLOBufferRef* out_buffer) {
    Client* c = static_cast<Client*>(client);
    if (!c) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "client is null"));
    if (!out_buffer) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "out_buffer is null"));
    *out_buffer = nullptr;
    if (rank < 0 || rank > MHLO_CUDA_MAX_RANK || (rank > 0 && !shape)) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "bad shape or rank"));
    if (!valid_dtype(element_type)) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "unknown element type"));
    TensorType t;
    t.dtype = static_cast<DType>(element_type);
    for (int d = 0; d < rank; ++d) {
        if (shape[d] < 0) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "negative dimension"));
        t.shape.push_back(shape[d]);
    }
    const size_t need = buffer_bytes(t);
    if (data_size != need)
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_BUFFER_FAILED, "Data size mismatch: expected " + std::to_string(need) +
                                                     " bytes for " + t.str() + ", got " + std::to_string(data_size)));
    if (need > 0 && !data) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "data is null"));
    Buffer* b = nullptr;
    MHLOStatusCode st = make_buffer(c, t, &b);
    if (st != MHLO_OK) return st;
    bool copied = true;
    if (need > 0) {
        std::lock_guard<std::mutex> lock(c->mu);  // the client's stream is used by one caller at a time (an execution may be capturing on it)
        copied = mhlo_cuda_upload(b->dev, data, need, c->stream) == 0 && mhlo_cuda_stream_sync(c->stream) == 0;
    }
    if (!copied) {
        set_error(MHLO_ERROR_TRANSFER_FAILED, mhlo_cuda_last_error());
        mhlo_cuda_free(b->dev);
        delete b;
        return MHLO_ERROR_TRANSFER_FAILED;
    }
    *out_buffer = b;
    return MHLO_OK;
}

MHLOStatusCode mhlo_buffer_create_uninitialized(MHLOClientRef client, const int64_t* shape, int32_t rank, MHLOElementType element_type,
                                                MHLOBufferRef* out_buffer) {
    Client* c = static_cast<Client*>(client);
    if (!c) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "client is null"));
    if (!out_buffer) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "out_buffer is null"));
    *out_buffer = nullptr;
    if (rank < 0 || rank > MHLO_CUDA_MAX_RANK || (rank > 0 && !shape) || !valid_dtype(element_type))
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "bad shape, rank or element type"));
    TensorType t;
    t.dtype = static_cast<DType>(element_type);
    for (int d = 0; d < rank; ++d) {
        if (shape[d] < 0) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "negative dimension"));
        t.shape.push_back(shape[d]);
    }
    Buffer* b = nullptr;
    MHLOStatusCode st = make_buffer(c, t, &b);
    if (st != MHLO_OK) return st;
    if (b->bytes) {
        std::lock_guard<std::mutex> lock(c->mu);
        mhlo_cuda_memset(b->dev, 0, b->bytes, c->stream);  // the reference's fresh MTLBuffers read as zero
    }
    *out_buffer = b;
    return MHLO_OK;
}

void mhlo_buffer_destroy(MHLOBufferRef buffer) {
    Buffer* b = static_cast<Buffer*>(buffer);
    if (!b) return;
    mhlo_cuda_device_set(b->client->device);
    {
        std::lock_guard<std::mutex> lock(b->client->mu);
        mhlo_cuda_stream_sync(b->client->stream);
        if (b->copy_done) {  // a transfer out of this buffer may still be reading it (other buffers' transfers are not waited for)
            mhlo_cuda_event_sync(b->copy_done);
            mhlo_cuda_event_destroy(b->copy_done);
        }
    }
    pool_release(b->client, b->dev, b->bytes);
    delete b;
}

void mhlo_buffer_shape(MHLOBufferRef buffer, int64_t* out_shape, int32_t* out_rank) {
    Buffer* b = static_cast<Buffer*>(buffer);
    if (!b) return;
    if (out_shape) for (int d = 0; d < b->type.rank(); ++d) out_shape[d] = b->type.shape[d];
    if (out_rank) *out_rank = b->type.rank();
}

int32_t mhlo_buffer_rank(MHLOBufferRef buffer) { return buffer ? static_cast<Buffer*>(buffer)->type.rank() : 0; }

MHLOElementType mhlo_buffer_element_type(MHLOBufferRef buffer) {
    return buffer ? static_cast<MHLOElementType>(static_cast<Buffer*>(buffer)->type.dtype) : MHLO_F32;
}

size_t mhlo_buffer_byte_count(MHLOBufferRef buffer) { return buffer ? static_cast<Buffer*>(buffer)->bytes : 0; }

MHLOStatusCode mhlo_buffer_to_host(MHLOBufferRef buffer, void* out_data, size_t data_size) {
    Buffer* b = static_cast<Buffer*>(buffer);
    if (!b) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "buffer is null"));
    if (!out_data) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "out_data is null"));
    if (b->bytes > data_size)
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_TRANSFER_FAILED, "Output buffer too small: need " + std::to_string(b->bytes) +
                                                     ", got " + std::to_string(data_size)));
    if (b->bytes == 0) return MHLO_OK;
    bool ok;
    {
        std::lock_guard<std::mutex> lock(b->client->mu);
        ok = mhlo_cuda_device_set(b->client->device) == 0 && mhlo_cuda_download(out_data, b->dev, b->bytes, b->client->stream) == 0 &&
             mhlo_cuda_stream_sync(b->client->stream) == 0;
    }
    if (!ok) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_TRANSFER_FAILED, mhlo_cuda_last_error()));
    return MHLO_OK;
}

MHLOStatusCode mhlo_b200_buffer_to_host_async(MHLOBufferRef buffer, void* out_data, size_t data_size, void (*done)(void*), void* user) {
    Buffer* b = static_cast<Buffer*>(buffer);
    if (!b) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "buffer is null"));
    if (!out_data || !done) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "out_data or the completion function is null"));
    if (b->bytes > data_size)
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_TRANSFER_FAILED, "Output buffer too small: need " + std::to_string(b->bytes) +
                                                     ", got " + std::to_string(data_size)));
    Client* c = b->client;
    bool ok;
    {
        std::lock_guard<std::mutex> lock(c->mu);
        ok = mhlo_cuda_device_set(c->device) == 0;
        if (ok && !c->copy_stream) ok = mhlo_cuda_stream_create(&c->copy_stream) == 0 && mhlo_cuda_event_create(&c->copy_fence) == 0;
        // behind whatever is queued on the client's stream (the program that wrote the buffer), then on its own
        ok = ok && mhlo_cuda_event_record(c->copy_fence, c->stream) == 0 && mhlo_cuda_stream_wait_event(c->copy_stream, c->copy_fence) == 0;
        if (ok && b->bytes) ok = mhlo_cuda_download(out_data, b->dev, b->bytes, c->copy_stream) == 0;
        if (ok && !b->copy_done) ok = mhlo_cuda_event_create(&b->copy_done) == 0;
        ok = ok && mhlo_cuda_event_record(b->copy_done, c->copy_stream) == 0;  // what the buffer's destruction waits for
        ok = ok && mhlo_cuda_stream_host_callback(c->copy_stream, done, user) == 0;
    }
    if (!ok) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_TRANSFER_FAILED, mhlo_cuda_last_error()));
    return MHLO_OK;
}

MHLOStatusCode mhlo_execute(MHLOExecutableRef executable, const MHLOBufferRef* inputs, int32_t num_inputs, MHLOBufferRef* out_outputs,
                            int32_t* out_num_outputs) {
    return run(static_cast<ExecutableHandle*>(executable), inputs, num_inputs, out_outputs, out_num_outputs, nullptr, nullptr, nullptr);
}

MHLOStatusCode mhlo_execute_with_timing(MHLOExecutableRef executable, const MHLOBufferRef* inputs, int32_t num_inputs,
                                        MHLOBufferRef* out_outputs, int32_t* out_num_outputs, double* out_encode_time,
                                        double* out_gpu_time, double* out_total_time) {
    double enc = 0, gpu = 0, tot = 0;
    MHLOStatusCode st = run(static_cast<ExecutableHandle*>(executable), inputs, num_inputs, out_outputs, out_num_outputs, &enc, &gpu, &tot);
    if (out_encode_time) *out_encode_time = enc;
    if (out_gpu_time) *out_gpu_time = gpu;
    if (out_total_time) *out_total_time = tot;
    return st;
}

MHLOStatusCode mhlo_execute_with_profile(MHLOExecutableRef executable, const MHLOBufferRef* inputs, int32_t num_inputs,
                                         MHLOBufferRef* out_outputs, int32_t* out_num_outputs, MHLOExecutionProfile* out_profile) {
    double enc = 0, gpu = 0, tot = 0;
    MHLOStatusCode st = run(static_cast<ExecutableHandle*>(executable), inputs, num_inputs, out_outputs, out_num_outputs, &enc, &gpu, &tot);
    if (out_profile) {
        std::memset(out_profile, 0, sizeof *out_profile);
        out_profile->partition_count = 1;
        out_profile->gpu_partition_count = 1;
        out_profile->gpu_time_ms = gpu * 1e3;
        out_profile->total_time_ms = tot * 1e3;
    }
    return st;
}

// ---- introspection used by the tests and the benchmark (not part of the reference's header) --------------------------

// Writes the optimised module (StableHLO text after the pass pipeline) into a malloc'd string; free with mhlo_free_string.
char* mhlo_b200_executable_optimized_text(MHLOExecutableRef executable) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    return h ? strdup(h->exe->optimized_text().c_str()) : nullptr;
}

// Host-only: parses `mlir_text`, runs the pass pipeline of `optimization_level` and returns the resulting module as
// text (malloc'd; free with mhlo_free_string). Needs no CUDA device, so the compiler core can be tested anywhere.
MHLOStatusCode mhlo_b200_optimize_text(const char* mlir_text, int32_t optimization_level, char** out_text) {
    if (!mlir_text || !out_text) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "null argument"));
    *out_text = nullptr;
    try {
        Module m = parse_module(mlir_text);
        Function f = flatten_main(m);
        CompileOptions opt;
        opt.opt_level = optimization_level;
        run_pass_pipeline(f, opt);
        optimize_loop_bodies(f, opt);
        *out_text = strdup(print_function(f).c_str());
        return MHLO_OK;
    } catch (const CompileError& e) {
        return static_cast<MHLOStatusCode>(set_error(e.code, e.what()));
    } catch (const std::exception& e) {
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_COMPILATION_FAILED, e.what()));
    }
}

// Host-only: lowers `mlir_text` to the executor's step list without touching a device. *out_steps receives one step
// label per line (malloc'd; free with mhlo_free_string); *out_launches and *out_arena_bytes (either may be null) the
// kernel launches per execution and the planned scratch arena.
MHLOStatusCode mhlo_b200_plan_text(const char* mlir_text, int32_t optimization_level, char** out_steps, int32_t* out_launches,
                                   int64_t* out_arena_bytes) {
    if (!mlir_text || !out_steps) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "null argument"));
    *out_steps = nullptr;
    try {
        CompileOptions opt;
        opt.opt_level = optimization_level;
        std::unique_ptr<Executable> exe = Executable::plan_only(mlir_text, opt);
        std::string s;
        for (const std::string& l : exe->step_labels()) s += l + "\n";
        *out_steps = strdup(s.c_str());
        if (out_launches) *out_launches = exe->num_kernel_launches();
        if (out_arena_bytes) *out_arena_bytes = exe->arena_bytes();
        return MHLO_OK;
    } catch (const CompileError& e) {
        return static_cast<MHLOStatusCode>(set_error(e.code, e.what()));
    } catch (const std::exception& e) {
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_COMPILATION_FAILED, e.what()));
    }
}

// ---- static memory plan, for inspection ----

// Host-only: the planner alone. n buffers with sizes and inclusive live ranges [first, last] in steps; out_offsets receives
// the arena offset of each and *out_total the arena size (StaticMemoryPlanner.plan, Memory/StaticMemoryPlanner.swift:175-253).
MHLOStatusCode mhlo_b200_plan_intervals(const int64_t* bytes, const int32_t* first, const int32_t* last, int32_t n, int64_t* out_offsets,
                                        int64_t* out_total) {
    if (n < 0 || (n > 0 && (!bytes || !first || !last || !out_offsets)) || !out_total)
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "null argument"));
    std::vector<PlanInterval> ivs(static_cast<size_t>(n));
    for (int32_t i = 0; i < n; ++i) {
        if (bytes[i] < 0 || first[i] > last[i]) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "negative size or empty live range"));
        ivs[static_cast<size_t>(i)].bytes = bytes[i];
        ivs[static_cast<size_t>(i)].first = first[i];
        ivs[static_cast<size_t>(i)].last = last[i];
    }
    *out_total = plan_memory(&ivs);
    for (int32_t i = 0; i < n; ++i) out_offsets[i] = ivs[static_cast<size_t>(i)].offset;
    return MHLO_OK;
}

// Host-only: the arena plan of a module: one line "bytes first last offset" per intermediate buffer (malloc'd; free with
// mhlo_free_string), *out_arena_bytes the planned arena.
MHLOStatusCode mhlo_b200_plan_memory_text(const char* mlir_text, int32_t optimization_level, char** out_lines, int64_t* out_arena_bytes) {
    if (!mlir_text || !out_lines) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "null argument"));
    *out_lines = nullptr;
    try {
        CompileOptions opt;
        opt.opt_level = optimization_level;
        std::unique_ptr<Executable> exe = Executable::plan_only(mlir_text, opt);
        std::string s;
        for (const PlanInterval& p : exe->plan_intervals())
            s += std::to_string(p.bytes) + " " + std::to_string(p.first) + " " + std::to_string(p.last) + " " + std::to_string(p.offset) + "\n";
        *out_lines = strdup(s.c_str());
        if (out_arena_bytes) *out_arena_bytes = exe->arena_bytes();
        return MHLO_OK;
    } catch (const CompileError& e) {
        return static_cast<MHLOStatusCode>(set_error(e.code, e.what()));
    } catch (const std::exception& e) {
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_COMPILATION_FAILED, e.what()));
    }
}

// ---- MLIR bytecode ----

// MLIR bytecode ("ML\xEFR...", what JAX sends) -> StableHLO text through the jaxlib helper process; *out_text is malloc'd
// (free with mhlo_free_string). mhlo_compile_n accepts bytecode directly and converts it the same way.
MHLOStatusCode mhlo_b200_bytecode_to_text(const void* bytecode, size_t size, char** out_text) {
    if (!bytecode || !out_text) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "null argument"));
    *out_text = nullptr;
    if (!is_mlir_bytecode(static_cast<const char*>(bytecode), size))
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "not MLIR bytecode (the magic ML\\xEFR is missing)"));
    std::string text, why;
    if (!bytecode_to_text(static_cast<const char*>(bytecode), size, &text, &why)) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_PARSE_FAILED, why));
    *out_text = strdup(text.c_str());
    return MHLO_OK;
}

// ---- batch sharding ------------------------------------------------------------------------------------------------

namespace {
ShardSpec make_spec(int32_t count, int32_t index, const int32_t* input_axes, int32_t num_axes) {
    ShardSpec s;
    s.count = count;
    s.index = index;
    if (input_axes) s.input_axes.assign(input_axes, input_axes + num_axes);
    return s;
}
}  // namespace

// Compiles shard `shard_index` of `shard_count` equal batch shards of the program. input_axes (num_input_axes entries, one
// per argument: the split axis or -1 for replicated) may be NULL: then every argument whose leading extent equals the
// first argument's is split along axis 0. The executable's input and output types are those of one shard. Fails with
// MHLO_ERROR_UNSUPPORTED_OP, naming the operator, when the shards would depend on one another.
MHLOStatusCode mhlo_b200_compile_sharded(MHLOClientRef client, const char* mlir_text, const MHLOCompileConfig* config, int32_t shard_count,
                                         int32_t shard_index, const int32_t* input_axes, int32_t num_input_axes, MHLOExecutableRef* out_executable) {
    if (!mlir_text) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "mlir_text is null"));
    if (shard_count < 1 || shard_index < 0 || shard_index >= shard_count)
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "shard index / count out of range"));
    const ShardSpec spec = make_spec(shard_count, shard_index, input_axes, num_input_axes);
    return compile_impl(static_cast<Client*>(client), mlir_text, config, out_executable, &spec);
}

// How an executable was split: shard count and index, and per argument / result the split axis (-1: replicated) and the
// extents before the split (rank entries each, concatenated; any pointer may be NULL).
MHLOStatusCode mhlo_b200_executable_sharding(MHLOExecutableRef executable, int32_t* out_count, int32_t* out_index, int32_t* out_input_axes,
                                             int32_t* out_output_axes) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    if (!h) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "executable is null"));
    const ShardPlan& p = h->exe->shard_plan();
    if (out_count) *out_count = p.count;
    if (out_index) *out_index = p.index;
    if (out_input_axes) for (size_t i = 0; i < p.input_axes.size(); ++i) out_input_axes[i] = p.input_axes[i];
    if (out_output_axes) for (size_t i = 0; i < p.output_axes.size(); ++i) out_output_axes[i] = p.output_axes[i];
    return MHLO_OK;
}

// Host-only: the analysis and rewrite alone. *out_text receives the function that computes the shard (malloc'd; free with
// mhlo_free_string); out_input_axes / out_output_axes (may be NULL) one entry per argument / result.
MHLOStatusCode mhlo_b200_shard_text(const char* mlir_text, int32_t shard_count, int32_t shard_index, const int32_t* input_axes,
                                    int32_t num_input_axes, char** out_text, int32_t* out_input_axes, int32_t* out_output_axes) {
    if (!mlir_text || !out_text) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "null argument"));
    *out_text = nullptr;
    try {
        Module m = parse_module(mlir_text);
        Function f = flatten_main(m);
        const ShardPlan p = shard_function(f, make_spec(shard_count, shard_index, input_axes, num_input_axes));
        *out_text = strdup(print_function(f).c_str());
        if (out_input_axes) for (size_t i = 0; i < p.input_axes.size(); ++i) out_input_axes[i] = p.input_axes[i];
        if (out_output_axes) for (size_t i = 0; i < p.output_axes.size(); ++i) out_output_axes[i] = p.output_axes[i];
        return MHLO_OK;
    } catch (const CompileError& e) {
        return static_cast<MHLOStatusCode>(set_error(e.code, e.what()));
    } catch (const std::exception& e) {
        return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_COMPILATION_FAILED, e.what()));
    }
}

// ---- kernel tuning -----------------------------------------------------------------------------------------------

MHLOStatusCode mhlo_b200_tuning_open(const char* path) {
    if (path && *path) {
        TuningDatabase::open_global(path);
        return MHLO_OK;
    }
    if (!TuningDatabase::global()) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "no path given and METALHLO_TUNING_DB is not set"));
    return MHLO_OK;
}

int64_t mhlo_b200_tuning_count(void) {
    TuningDatabase* db = TuningDatabase::global();
    return db ? static_cast<int64_t>(db->count()) : -1;
}

MHLOStatusCode mhlo_b200_tuning_tune_row_kernel(MHLOClientRef client, const char* kernel, MHLOElementType element_type, int64_t rows,
                                                int64_t hidden, int32_t max_trials, char** out_record_json) {
    if (out_record_json) *out_record_json = nullptr;
    Client* c = static_cast<Client*>(client);
    if (!c || !kernel) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "null client or kernel name"));
    TuningDatabase* db = TuningDatabase::global();
    if (!db) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "no tuning database is open"));
    if (mhlo_cuda_device_set(c->device) != 0) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_NO_DEVICE, mhlo_cuda_last_error()));
    TuningRecord rec;
    std::string why;
    const int st = tune_row_kernel(kernel, static_cast<int>(element_type), rows, hidden, max_trials, db, &rec, &why);
    if (st == MHLO_CUDA_INVALID_ARGUMENT) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, why));
    if (st != MHLO_CUDA_OK) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_EXECUTION_FAILED, why));
    if (out_record_json) {
        char buf[512];
        snprintf(buf, sizeof buf,
                 "{\"bestConfig\": {\"threads\": %d, \"vectorsPerThread\": %d, \"ctasPerSM\": %d}, \"measuredTime\": %.9g, "
                 "\"gbytesPerSecond\": %.6g, \"configsTried\": %d}",
                 rec.best.threads, rec.best.vectors_per_thread, rec.best.ctas_per_sm, rec.measured_time_s, rec.gbytes_per_s, rec.configs_tried);
        *out_record_json = strdup(buf);
    }
    return MHLO_OK;
}

namespace {
char* record_json(const TuningRecord& rec) {
    char buf[640];
    snprintf(buf, sizeof buf,
             "{\"bestConfig\": {\"tileM\": %d, \"tileN\": %d, \"tileK\": %d, \"stages\": %d, \"ctaGroup\": %d, \"tileOrder\": %d}, "
             "\"measuredTime\": %.9g, \"gflops\": %.6g, \"gbytesPerSecond\": %.6g, \"configsTried\": %d}",
             rec.best.tile_m, rec.best.tile_n, rec.best.tile_k, rec.best.stages, rec.best.cta_group, rec.best.tile_order, rec.measured_time_s,
             rec.gflops, rec.gbytes_per_s, rec.configs_tried);
    return strdup(buf);
}
}  // namespace

// Times every configuration of the tensor-core GEMM on [batch, m, k] . [batch, k, n] (operands of element_type, result of
// out_element_type; a_transposed / b_transposed: the operand is stored with the other dimension contiguous) and stores the
// best in the open database under the key the compiler looks up for the same dot_general.
MHLOStatusCode mhlo_b200_tuning_tune_gemm(MHLOClientRef client, MHLOElementType element_type, MHLOElementType out_element_type, int64_t batch,
                                          int64_t m, int64_t n, int64_t k, bool a_transposed, bool b_transposed, int32_t max_trials,
                                          char** out_record_json) {
    if (out_record_json) *out_record_json = nullptr;
    Client* c = static_cast<Client*>(client);
    if (!c) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "null client"));
    TuningDatabase* db = TuningDatabase::global();
    if (!db) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "no tuning database is open"));
    if (mhlo_cuda_device_set(c->device) != 0) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_NO_DEVICE, mhlo_cuda_last_error()));
    GemmCase gc;
    gc.dtype = static_cast<int>(element_type); gc.out_dtype = static_cast<int>(out_element_type);
    gc.batch = batch; gc.m = m; gc.n = n; gc.k = k;
    gc.a_k_major = !a_transposed; gc.b_k_major = b_transposed;
    TuningRecord rec;
    std::string why;
    const int st = tune_gemm(gc, max_trials, db, &rec, &why);
    if (st == MHLO_CUDA_INVALID_ARGUMENT) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, why));
    if (st != MHLO_CUDA_OK) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_EXECUTION_FAILED, why));
    if (out_record_json) *out_record_json = record_json(rec);
    return MHLO_OK;
}

// The same for the tensor-core attention kernel on Q [batch, heads, seq_q, head_dim], K / V [batch, heads, seq_k, head_dim]
// (bshd: the tensors are laid out [batch, sequence, heads, head_dim]).
MHLOStatusCode mhlo_b200_tuning_tune_attention(MHLOClientRef client, MHLOElementType element_type, int64_t batch, int64_t heads, int64_t seq_q,
                                               int64_t seq_k, int64_t head_dim, bool causal, bool bshd, int32_t max_trials, char** out_record_json) {
    if (out_record_json) *out_record_json = nullptr;
    Client* c = static_cast<Client*>(client);
    if (!c) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "null client"));
    TuningDatabase* db = TuningDatabase::global();
    if (!db) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "no tuning database is open"));
    if (mhlo_cuda_device_set(c->device) != 0) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_NO_DEVICE, mhlo_cuda_last_error()));
    AttentionCase ac;
    ac.dtype = static_cast<int>(element_type);
    ac.batch = batch; ac.heads = heads; ac.seq_q = seq_q; ac.seq_k = seq_k; ac.head_dim = head_dim; ac.causal = causal; ac.bshd = bshd;
    TuningRecord rec;
    std::string why;
    const int st = tune_attention(ac, max_trials, db, &rec, &why);
    if (st == MHLO_CUDA_INVALID_ARGUMENT) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, why));
    if (st != MHLO_CUDA_OK) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_EXECUTION_FAILED, why));
    if (out_record_json) *out_record_json = record_json(rec);
    return MHLO_OK;
}

MHLOStatusCode mhlo_b200_tuning_merge_json(const char* database_json, bool overwrite, int32_t* out_taken) {
    if (out_taken) *out_taken = 0;
    TuningDatabase* db = TuningDatabase::global();
    if (!db) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "no tuning database is open"));
    if (!database_json) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "null document"));
    std::string why;
    const int taken = db->merge_json(database_json, overwrite, &why);
    if (taken < 0) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_PARSE_FAILED, why));
    if (out_taken) *out_taken = taken;
    return MHLO_OK;
}

char* mhlo_b200_tuning_to_json(void) {
    TuningDatabase* db = TuningDatabase::global();
    return db ? strdup(db->to_json().c_str()) : nullptr;
}

MHLOStatusCode mhlo_b200_tuning_save(void) {
    TuningDatabase* db = TuningDatabase::global();
    if (!db) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "no tuning database is open"));
    if (!db->save()) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_TRANSFER_FAILED, "cannot write " + db->path()));
    return MHLO_OK;
}

MHLOStatusCode mhlo_b200_tuning_import(const char* other_path, bool overwrite, int32_t* out_taken) {
    if (out_taken) *out_taken = 0;
    TuningDatabase* db = TuningDatabase::global();
    if (!db || !other_path) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "no tuning database is open, or null path"));
    const int taken = db->import_from(other_path, overwrite);
    if (out_taken) *out_taken = taken;
    return MHLO_OK;
}

int32_t mhlo_b200_tuning_prune(double max_age_days) {
    TuningDatabase* db = TuningDatabase::global();
    return db ? db->prune(max_age_days, static_cast<double>(std::time(nullptr))) : -1;
}

void mhlo_b200_tuning_clear(void) {
    if (TuningDatabase* db = TuningDatabase::global()) db->clear();
}

// Kernel launches one execution enqueues, the arena size and a newline-separated list of step labels.
int32_t mhlo_b200_executable_launch_count(MHLOExecutableRef executable) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    return h ? h->exe->num_kernel_launches() : 0;
}
int64_t mhlo_b200_executable_graph_replays(MHLOExecutableRef executable) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    return h ? h->exe->graph_replays : 0;
}

int64_t mhlo_b200_executable_arena_bytes(MHLOExecutableRef executable) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    return h ? h->exe->arena_bytes() : 0;
}
char* mhlo_b200_executable_steps(MHLOExecutableRef executable) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    if (!h) return nullptr;
    std::string s;
    for (const std::string& l : h->exe->step_labels()) s += l + "\n";
    return strdup(s.c_str());
}
// Device pointer of a buffer, so that a caller holding device memory (torch, another library) can run kernels on
// it or time device-resident execution.
void* mhlo_b200_buffer_device_pointer(MHLOBufferRef buffer) { return buffer ? static_cast<Buffer*>(buffer)->dev : nullptr; }
// Runs the executable on caller-provided device pointers and stream (no allocation, no synchronisation).
MHLOStatusCode mhlo_b200_execute_on_device(MHLOExecutableRef executable, const void* const* input_ptrs, void* const* output_ptrs,
                                           void* stream) {
    ExecutableHandle* h = static_cast<ExecutableHandle*>(executable);
    if (!h) return static_cast<MHLOStatusCode>(set_error(MHLO_ERROR_INVALID_ARGUMENT, "executable is null"));
    const int st = h->exe->execute(input_ptrs, output_ptrs, stream);
    if (st != 0) set_error(st, h->exe->last_error());
    return static_cast<MHLOStatusCode>(st);
}

}  // extern "C"
