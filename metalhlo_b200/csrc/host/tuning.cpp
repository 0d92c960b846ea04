// Tuning database (JSON persistence) and the row-kernel auto-tuner. See tuning.h.
#include "tuning.h"
#include "numeric.h"

#include <algorithm>
#include <cmath>
#include <functional>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <ctime>
#include <fstream>
#include <sstream>
#include <vector>

#include "../../../include/mhlo_cuda.h"

namespace mhlo {

bool TuningKey::operator<(const TuningKey& o) const {
    if (op_type != o.op_type) return op_type < o.op_type;
    if (dtype != o.dtype) return dtype < o.dtype;
    if (device != o.device) return device < o.device;
    return shapes < o.shapes;
}
bool TuningKey::operator==(const TuningKey& o) const { return !(*this < o) && !(o < *this); }

std::string TuningConfig::description() const {
    char buf[160];
    snprintf(buf, sizeof buf, "tile[%dx%dx%d]_stages%d_threads%d_vec%d_ctas%d_group%d_order%d", tile_m, tile_n, tile_k, stages, threads,
             vectors_per_thread, ctas_per_sm, cta_group, tile_order);
    return buf;
}

// ---- a small JSON reader: objects, arrays, strings, numbers, true/false/null ------------------------------------
namespace {

struct JsonValue {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<JsonValue> items;                            // Array
    std::vector<std::pair<std::string, JsonValue>> members;  // Object
    const JsonValue* find(const std::string& key) const {
        for (const auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
    double number_or(const std::string& key, double dflt) const {
        const JsonValue* v = find(key);
        return v && v->kind == Number ? v->num : dflt;
    }
    std::string string_or(const std::string& key, const std::string& dflt) const {
        const JsonValue* v = find(key);
        return v && v->kind == String ? v->str : dflt;
    }
};

class JsonReader {
  public:
    explicit JsonReader(const std::string& t) : t_(t) {}
    bool parse(JsonValue* out, std::string* why) {
        if (!value(out)) {
            *why = "JSON error near offset " + std::to_string(p_) + ": " + err_;
            return false;
        }
        ws();
        if (p_ != t_.size()) {
            *why = "trailing characters after JSON value";
            return false;
        }
        return true;
    }

  private:
    void ws() {
        while (p_ < t_.size() && (t_[p_] == ' ' || t_[p_] == '\n' || t_[p_] == '\t' || t_[p_] == '\r')) ++p_;
    }
    bool fail(const char* m) {
        if (err_.empty()) err_ = m;
        return false;
    }
    bool literal(const char* word) {
        const size_t n = std::char_traits<char>::length(word);
        if (t_.compare(p_, n, word) != 0) return fail("unknown literal");
        p_ += n;
        return true;
    }
    bool string(std::string* out) {
        if (p_ >= t_.size() || t_[p_] != '"') return fail("expected string");
        ++p_;
        out->clear();
        while (p_ < t_.size() && t_[p_] != '"') {
            char c = t_[p_++];
            if (c == '\\') {
                if (p_ >= t_.size()) return fail("bad escape");
                const char e = t_[p_++];
                switch (e) {
                    case 'n': c = '\n'; break;
                    case 't': c = '\t'; break;
                    case 'r': c = '\r'; break;
                    case 'b': c = '\b'; break;
                    case 'f': c = '\f'; break;
                    case 'u': {
                        if (p_ + 4 > t_.size()) return fail("bad \\u escape");
                        const unsigned code = static_cast<unsigned>(std::strtoul(t_.substr(p_, 4).c_str(), nullptr, 16));
                        p_ += 4;
                        c = code < 128 ? static_cast<char>(code) : '?';
                        break;
                    }
                    default: c = e;
                }
            }
            out->push_back(c);
        }
        if (p_ >= t_.size()) return fail("unterminated string");
        ++p_;
        return true;
    }
    bool value(JsonValue* out) {
        ws();
        if (p_ >= t_.size()) return fail("unexpected end");
        const char c = t_[p_];
        if (c == '{') {
            out->kind = JsonValue::Object;
            ++p_;
            ws();
            if (p_ < t_.size() && t_[p_] == '}') { ++p_; return true; }
            while (true) {
                ws();
                std::string key;
                if (!string(&key)) return false;
                ws();
                if (p_ >= t_.size() || t_[p_] != ':') return fail("expected ':'");
                ++p_;
                JsonValue v;
                if (!value(&v)) return false;
                out->members.emplace_back(std::move(key), std::move(v));
                ws();
                if (p_ < t_.size() && t_[p_] == ',') { ++p_; continue; }
                if (p_ < t_.size() && t_[p_] == '}') { ++p_; return true; }
                return fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            out->kind = JsonValue::Array;
            ++p_;
            ws();
            if (p_ < t_.size() && t_[p_] == ']') { ++p_; return true; }
            while (true) {
                JsonValue v;
                if (!value(&v)) return false;
                out->items.push_back(std::move(v));
                ws();
                if (p_ < t_.size() && t_[p_] == ',') { ++p_; continue; }
                if (p_ < t_.size() && t_[p_] == ']') { ++p_; return true; }
                return fail("expected ',' or ']'");
            }
        }
        if (c == '"') {
            out->kind = JsonValue::String;
            return string(&out->str);
        }
        if (c == 't') { out->kind = JsonValue::Bool; out->b = true; return literal("true"); }
        if (c == 'f') { out->kind = JsonValue::Bool; out->b = false; return literal("false"); }
        if (c == 'n') { out->kind = JsonValue::Null; return literal("null"); }
        char* end = nullptr;
        out->num = std::strtod(t_.c_str() + p_, &end);
        if (end == t_.c_str() + p_) return fail("expected a value");
        out->kind = JsonValue::Number;
        p_ = static_cast<size_t>(end - t_.c_str());
        return true;
    }
    const std::string& t_;
    size_t p_ = 0;
    std::string err_;
};

std::string quoted(const std::string& s) {
    std::string o = "\"";
    for (char c : s) {
        if (c == '"' || c == '\\') { o.push_back('\\'); o.push_back(c); }
        else if (c == '\n') o += "\\n";
        else if (static_cast<unsigned char>(c) < 0x20) o += "?";
        else o.push_back(c);
    }
    return o + "\"";
}

std::string number(double v) {
    char buf[64];
    if (v == std::floor(v) && std::fabs(v) < 1e15) snprintf(buf, sizeof buf, "%.0f", v);
    else snprintf(buf, sizeof buf, "%.9g", v);
    return buf;
}

constexpr double kSwiftReferenceDate = 978307200.0;  // 2001-01-01T00:00:00Z: Swift's JSONEncoder writes dates relative to it

}  // namespace

// ---- database ---------------------------------------------------------------------------------------------------

TuningDatabase::TuningDatabase(std::string path) : path_(std::move(path)) {
    if (path_.empty()) return;
    std::ifstream in(path_);
    if (!in) return;
    std::stringstream ss;
    ss << in.rdbuf();
    std::string why;
    if (!from_json(ss.str(), &why)) fprintf(stderr, "Warning: Failed to load tuning database %s: %s\n", path_.c_str(), why.c_str());
    dirty_ = false;
}

bool TuningDatabase::get(const TuningKey& key, TuningRecord* out) const {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = entries_.find(key);
    if (it == entries_.end()) return false;
    if (out) *out = it->second;
    return true;
}

void TuningDatabase::store(const TuningKey& key, const TuningRecord& record) {
    std::lock_guard<std::mutex> lock(mu_);
    entries_[key] = record;
    dirty_ = true;
}

bool TuningDatabase::remove(const TuningKey& key) {
    std::lock_guard<std::mutex> lock(mu_);
    const bool had = entries_.erase(key) > 0;
    dirty_ = dirty_ || had;
    return had;
}

void TuningDatabase::clear() {
    std::lock_guard<std::mutex> lock(mu_);
    dirty_ = dirty_ || !entries_.empty();
    entries_.clear();
}

size_t TuningDatabase::count() const {
    std::lock_guard<std::mutex> lock(mu_);
    return entries_.size();
}

std::vector<TuningKey> TuningDatabase::keys() const {
    std::lock_guard<std::mutex> lock(mu_);
    std::vector<TuningKey> out;
    for (const auto& e : entries_) out.push_back(e.first);
    return out;
}

std::string TuningDatabase::to_json() const {
    std::lock_guard<std::mutex> lock(mu_);
    std::string o = "{\n  \"version\": 1,\n  \"entries\": [";
    bool first = true;
    for (const auto& e : entries_) {
        const TuningKey& k = e.first;
        const TuningRecord& r = e.second;
        o += first ? "\n" : ",\n";
        first = false;
        o += "    {\"opType\": " + quoted(k.op_type) + ", \"shapes\": [";
        for (size_t i = 0; i < k.shapes.size(); ++i) {
            o += i ? ", [" : "[";
            for (size_t j = 0; j < k.shapes[i].size(); ++j) o += (j ? ", " : "") + std::to_string(k.shapes[i][j]);
            o += "]";
        }
        o += "], \"dtype\": " + quoted(k.dtype) + ", \"deviceID\": " + quoted(k.device) + "},\n";
        const TuningConfig& c = r.best;
        o += "    {\"bestConfig\": {\"tileM\": " + std::to_string(c.tile_m) + ", \"tileN\": " + std::to_string(c.tile_n) + ", \"tileK\": " +
             std::to_string(c.tile_k) + ", \"stages\": " + std::to_string(c.stages) + ", \"threads\": " + std::to_string(c.threads) +
             ", \"vectorsPerThread\": " + std::to_string(c.vectors_per_thread) + ", \"ctasPerSM\": " + std::to_string(c.ctas_per_sm) + ", \"ctaGroup\": " +
             std::to_string(c.cta_group) + ", \"tileOrder\": " + std::to_string(c.tile_order) +
             "}, \"measuredTime\": " + number(r.measured_time_s) + ", \"gflops\": " + number(r.gflops) + ", \"gbytesPerSecond\": " +
             number(r.gbytes_per_s) + ", \"configsTried\": " + std::to_string(r.configs_tried) + ", \"timestamp\": " +
             number(r.timestamp - kSwiftReferenceDate) + "}";
    }
    o += "\n  ],\n  \"savedAt\": " + number(static_cast<double>(std::time(nullptr)) - kSwiftReferenceDate) + "\n}\n";
    return o;
}

bool TuningDatabase::from_json(const std::string& text, std::string* why) {
    JsonValue root;
    JsonReader reader(text);
    if (!reader.parse(&root, why)) return false;
    const JsonValue* entries = root.kind == JsonValue::Object ? root.find("entries") : nullptr;
    if (!entries || entries->kind != JsonValue::Array || entries->items.size() % 2 != 0) {
        *why = "no alternating key/value \"entries\" array";
        return false;
    }
    std::map<TuningKey, TuningRecord> loaded;
    for (size_t i = 0; i + 1 < entries->items.size(); i += 2) {
        const JsonValue& k = entries->items[i];
        const JsonValue& r = entries->items[i + 1];
        if (k.kind != JsonValue::Object || r.kind != JsonValue::Object) {
            *why = "entry " + std::to_string(i / 2) + " is not an object pair";
            return false;
        }
        TuningKey key;
        key.op_type = k.string_or("opType", "");
        key.dtype = k.string_or("dtype", "");
        key.device = k.string_or("deviceID", "");
        if (const JsonValue* shapes = k.find("shapes"))
            for (const JsonValue& s : shapes->items) {
                std::vector<int64_t> dims;
                for (const JsonValue& d : s.items) dims.push_back(static_cast<int64_t>(d.num));
                key.shapes.push_back(dims);
            }
        TuningRecord rec;
        if (const JsonValue* c = r.find("bestConfig")) {
            rec.best.tile_m = static_cast<int32_t>(c->number_or("tileM", 0));
            rec.best.tile_n = static_cast<int32_t>(c->number_or("tileN", 0));
            rec.best.tile_k = static_cast<int32_t>(c->number_or("tileK", 0));
            rec.best.stages = static_cast<int32_t>(c->number_or("stages", 0));
            rec.best.threads = static_cast<int32_t>(c->number_or("threads", 0));
            rec.best.vectors_per_thread = static_cast<int32_t>(c->number_or("vectorsPerThread", 0));
            rec.best.ctas_per_sm = static_cast<int32_t>(c->number_or("ctasPerSM", 0));
            rec.best.cta_group = static_cast<int32_t>(c->number_or("ctaGroup", 0));
            rec.best.tile_order = static_cast<int32_t>(c->number_or("tileOrder", 0));
        }
        rec.measured_time_s = r.number_or("measuredTime", 0);
        rec.gflops = r.number_or("gflops", 0);
        rec.gbytes_per_s = r.number_or("gbytesPerSecond", 0);
        rec.configs_tried = static_cast<int32_t>(r.number_or("configsTried", 0));
        rec.timestamp = r.number_or("timestamp", 0) + kSwiftReferenceDate;
        loaded[key] = rec;
    }
    std::lock_guard<std::mutex> lock(mu_);
    entries_ = std::move(loaded);
    dirty_ = true;
    return true;
}

bool TuningDatabase::save() {
    if (path_.empty()) return false;
    {
        std::lock_guard<std::mutex> lock(mu_);
        if (!dirty_) return true;
    }
    const std::string text = to_json();
    const std::string tmp = path_ + ".tmp";
    {
        std::ofstream out(tmp, std::ios::trunc);
        if (!out) return false;
        out << text;
        if (!out.good()) return false;
    }
    if (std::rename(tmp.c_str(), path_.c_str()) != 0) return false;  // atomic replace: a reader never sees half a file
    std::lock_guard<std::mutex> lock(mu_);
    dirty_ = false;
    return true;
}

int TuningDatabase::merge_json(const std::string& text, bool overwrite, std::string* why) {
    TuningDatabase other("");
    if (!other.from_json(text, why)) return -1;
    int taken = 0;
    std::lock_guard<std::mutex> lock(mu_);
    for (const auto& e : other.entries_) {
        if (!overwrite && entries_.count(e.first)) continue;
        entries_[e.first] = e.second;
        ++taken;
    }
    dirty_ = dirty_ || taken > 0;
    return taken;
}

int TuningDatabase::import_from(const std::string& other_path, bool overwrite) {
    TuningDatabase other(other_path);
    int taken = 0;
    std::lock_guard<std::mutex> lock(mu_);
    for (const auto& e : other.entries_) {
        if (!overwrite && entries_.count(e.first)) continue;
        entries_[e.first] = e.second;
        ++taken;
    }
    dirty_ = dirty_ || taken > 0;
    return taken;
}

int TuningDatabase::prune(double max_age_days, double now_epoch_s) {
    std::lock_guard<std::mutex> lock(mu_);
    int dropped = 0;
    for (auto it = entries_.begin(); it != entries_.end();) {
        if (now_epoch_s - it->second.timestamp > max_age_days * 86400.0) {
            it = entries_.erase(it);
            ++dropped;
        } else {
            ++it;
        }
    }
    dirty_ = dirty_ || dropped > 0;
    return dropped;
}

namespace {
std::mutex g_global_mu;
TuningDatabase* g_global = nullptr;
bool g_global_probed = false;
}  // namespace

TuningDatabase* TuningDatabase::global() {
    std::lock_guard<std::mutex> lock(g_global_mu);
    if (!g_global && !g_global_probed) {
        g_global_probed = true;
        const char* path = std::getenv("METALHLO_TUNING_DB");
        if (path && *path) g_global = new TuningDatabase(path);
    }
    return g_global;
}

TuningDatabase* TuningDatabase::open_global(const std::string& path) {
    std::lock_guard<std::mutex> lock(g_global_mu);
    if (g_global) g_global->save();
    g_global = new TuningDatabase(path);
    g_global_probed = true;
    return g_global;
}

// ---- tuner ------------------------------------------------------------------------------------------------------

std::vector<TuningConfig> row_kernel_candidates(int64_t hidden, int elem_bytes) {
    std::vector<TuningConfig> out;
    const int64_t per_vec = 16 / elem_bytes;
    const int64_t nvec = hidden / per_vec;
    std::vector<int> thread_counts = {64, 128, 256, 512, 1024};
    // CTAs of whole warps that cover the row exactly (no idle threads, no predicates)
    for (int vecs : {1, 2, 4, 8})
        if (nvec % (32LL * vecs) == 0 && nvec / vecs <= 1024) thread_counts.push_back(static_cast<int>(nvec / vecs));
    std::sort(thread_counts.begin(), thread_counts.end());
    thread_counts.erase(std::unique(thread_counts.begin(), thread_counts.end()), thread_counts.end());
    for (int threads : thread_counts)
        for (int vecs : {1, 2, 4, 8}) {
            const int64_t cover = static_cast<int64_t>(threads) * vecs * per_vec;
            // a row must fit the registers of one CTA, and a CTA more than four times wider than the row wastes threads
            if (cover < hidden || cover >= hidden * 4) continue;
            for (int ctas : {0, 2, 4, 8, 16}) {
                if (ctas * threads > 2048) continue;
                TuningConfig c;
                c.threads = threads;
                c.vectors_per_thread = vecs;
                c.ctas_per_sm = ctas;
                out.push_back(c);
            }
        }
    return out;
}

int tune_row_kernel(const std::string& kind, int dtype, int64_t rows, int64_t hidden, int max_trials, TuningDatabase* db, TuningRecord* out,
                    std::string* why) {
    const size_t elem = mhlo_cuda_dtype_size(dtype);
    if (elem == 0 || rows < 1 || hidden < 1) {
        *why = "tune_row_kernel: bad dtype or shape";
        return MHLO_CUDA_INVALID_ARGUMENT;
    }
    if (kind != "fused_layer_norm" && kind != "fused_rms_norm" && kind != "fused_softmax") {
        *why = "tune_row_kernel: unknown kernel " + kind;
        return MHLO_CUDA_INVALID_ARGUMENT;
    }
    const size_t bytes = static_cast<size_t>(rows) * static_cast<size_t>(hidden) * elem;
    void *x = nullptr, *y = nullptr, *g = nullptr, *e0 = nullptr, *e1 = nullptr;
    auto cleanup = [&] {
        if (x) mhlo_cuda_free(x);
        if (y) mhlo_cuda_free(y);
        if (g) mhlo_cuda_free(g);
        if (e0) mhlo_cuda_event_destroy(e0);
        if (e1) mhlo_cuda_event_destroy(e1);
    };
    auto failed = [&](int st) {
        *why = mhlo_cuda_last_error();
        cleanup();
        return st;
    };
    int st;
    if ((st = mhlo_cuda_alloc(bytes, &x)) || (st = mhlo_cuda_alloc(bytes, &y)) || (st = mhlo_cuda_alloc(static_cast<size_t>(hidden) * elem, &g)) ||
        (st = mhlo_cuda_event_create(&e0)) || (st = mhlo_cuda_event_create(&e1)))
        return failed(st);
    // zeros are a valid input for all three kernels (gamma = 0 does not change the traffic or the instruction stream)
    if ((st = mhlo_cuda_memset(x, 0, bytes, nullptr)) || (st = mhlo_cuda_memset(g, 0, static_cast<size_t>(hidden) * elem, nullptr))) return failed(st);
    auto launch = [&](const mhlo_cuda_row_tuning* t) {
        if (kind == "fused_layer_norm") return mhlo_cuda_layer_norm(dtype, x, g, g, y, rows, hidden, 1e-5f, t, nullptr);
        if (kind == "fused_rms_norm") return mhlo_cuda_rms_norm(dtype, x, g, y, rows, hidden, 1e-5f, t, nullptr);
        return mhlo_cuda_softmax(dtype, x, y, rows, hidden, 1, t, nullptr);
    };
    std::vector<TuningConfig> candidates = row_kernel_candidates(hidden, static_cast<int>(elem));
    TuningConfig dflt;  // all zero: the library's own choice competes too
    candidates.insert(candidates.begin(), dflt);
    if (max_trials > 0 && static_cast<int>(candidates.size()) > max_trials) candidates.resize(static_cast<size_t>(max_trials));
    constexpr int kWarmup = 5, kTimed = 20;  // AutoTuner.swift:242-245
    TuningRecord best;
    best.measured_time_s = 1e30;
    int tried = 0;
    for (const TuningConfig& c : candidates) {
        mhlo_cuda_row_tuning t{c.threads, c.vectors_per_thread, c.ctas_per_sm};
        const mhlo_cuda_row_tuning* tp = (c.threads || c.vectors_per_thread || c.ctas_per_sm) ? &t : nullptr;
        if (launch(tp) != MHLO_CUDA_OK) continue;  // the kernel rejects combinations it cannot run
        ++tried;
        for (int i = 1; i < kWarmup; ++i) launch(tp);
        std::vector<float> ms(kTimed, 0.f);
        bool ok = true;
        for (int i = 0; i < kTimed && ok; ++i) {
            ok = mhlo_cuda_event_record(e0, nullptr) == MHLO_CUDA_OK && launch(tp) == MHLO_CUDA_OK && mhlo_cuda_event_record(e1, nullptr) == MHLO_CUDA_OK &&
                 mhlo_cuda_event_elapsed_ms(e0, e1, &ms[static_cast<size_t>(i)]) == MHLO_CUDA_OK;
        }
        if (!ok) return failed(MHLO_CUDA_EXECUTION_FAILED);
        std::sort(ms.begin(), ms.end());
        const double median_s = 0.5 * (ms[kTimed / 2 - 1] + ms[kTimed / 2]) * 1e-3;
        if (median_s < best.measured_time_s) {
            best.best = c;
            best.measured_time_s = median_s;
        }
    }
    if (tried == 0) {
        *why = "tune_row_kernel: no candidate could be launched";
        cleanup();
        return MHLO_CUDA_EXECUTION_FAILED;
    }
    best.configs_tried = tried;
    best.gbytes_per_s = 2.0 * static_cast<double>(bytes) / best.measured_time_s / 1e9;
    best.timestamp = static_cast<double>(std::time(nullptr));
    cleanup();
    if (db) {
        TuningKey key;
        key.op_type = kind;
        key.shapes = {{rows, hidden}};
        key.dtype = dtype == MHLO_DT_BF16 ? "bf16" : dtype == MHLO_DT_F16 ? "f16" : "f32";
        char name[256] = "";
        int ordinal = 0;
        mhlo_cuda_device_current(&ordinal);
        mhlo_cuda_device_name(ordinal, name, sizeof name);
        key.device = name;
        db->store(key, best);
    }
    if (out) *out = best;
    return MHLO_CUDA_OK;
}

std::string current_device_name() {
    char name[256] = "";
    int ordinal = 0;
    if (mhlo_cuda_device_current(&ordinal) == MHLO_CUDA_OK) mhlo_cuda_device_name(ordinal, name, sizeof name);
    return name;
}

namespace {

const char* dtype_key(int dtype) { return dtype == MHLO_DT_BF16 ? "bf16" : dtype == MHLO_DT_F16 ? "f16" : "f32"; }

// 5 warm-up + 20 timed launches of `launch`, median in seconds (AutoTuner.swift:242-245, 479-513); < 0 when a launch failed.
double median_seconds(const std::function<int()>& launch, void* e0, void* e1) {
    constexpr int kWarmup = 5, kTimed = 20;
    for (int i = 0; i < kWarmup; ++i)
        if (launch() != MHLO_CUDA_OK) return -1;
    std::vector<float> ms(kTimed, 0.f);
    for (int i = 0; i < kTimed; ++i) {
        if (mhlo_cuda_event_record(e0, nullptr) != MHLO_CUDA_OK || launch() != MHLO_CUDA_OK || mhlo_cuda_event_record(e1, nullptr) != MHLO_CUDA_OK ||
            mhlo_cuda_event_elapsed_ms(e0, e1, &ms[static_cast<size_t>(i)]) != MHLO_CUDA_OK)
            return -1;
    }
    std::sort(ms.begin(), ms.end());
    return 0.5 * (ms[kTimed / 2 - 1] + ms[kTimed / 2]) * 1e-3;
}

}  // namespace

std::vector<TuningConfig> gemm_candidates(int64_t m, int64_t n, int64_t k) {
    std::vector<TuningConfig> out;
    auto add = [&](int tile_n, int stages, int group) {
        TuningConfig c;
        c.tile_m = 128 * group;
        c.tile_n = tile_n;
        c.tile_k = 64;
        c.stages = stages;
        c.cta_group = group;
        out.push_back(c);
    };
    const int k_blocks = static_cast<int>((k + 63) / 64);
    for (int stages : {6, 4, 3}) {
        if (stages != 6 && stages > k_blocks + 1) continue;  // a ring deeper than the K loop is the same as the full one
        add(128, stages, 1);
    }
    if (n > 128) {
        for (int stages : {4, 3, 2}) add(256, stages, 1);
        if (m > 128)
            for (int stages : {6, 5, 4, 3}) add(256, stages, 2);
    }
    return out;
}

TuningKey GemmCase::key(const std::string& device) const {
    TuningKey k;
    k.op_type = "dot_general";
    k.shapes = {{batch, m, this->k}, {batch, this->k, n}, {a_k_major ? 1 : 0, b_k_major ? 1 : 0, out_dtype}};
    k.dtype = dtype_key(dtype);
    k.device = device;
    return k;
}

namespace {
// Fills a device buffer with 16-bit floats drawn once from (-1, 1) on the host (a 2 MB block, repeated).
int fill_random_16(void* dev, size_t bytes, int dtype) {
    static std::vector<uint16_t> block[2];
    std::vector<uint16_t>& src = block[dtype == MHLO_DT_BF16 ? 1 : 0];
    if (src.empty()) {
        src.resize(1 << 20);
        uint64_t state = 0x9E3779B97F4A7C15ull;
        for (uint16_t& w : src) {
            state = state * 6364136223846793005ull + 1442695040888963407ull;
            const float v = static_cast<float>(static_cast<int32_t>(state >> 40) - (1 << 23)) / static_cast<float>(1 << 23);  // (-1, 1)
            uint8_t raw[2];
            encode_float(dtype == MHLO_DT_BF16 ? DType::BF16 : DType::F16, v, raw);
            w = static_cast<uint16_t>(raw[0] | (raw[1] << 8));
        }
    }
    const size_t chunk = src.size() * sizeof(uint16_t);
    if (bytes == 0) return MHLO_CUDA_OK;
    int st = mhlo_cuda_upload(dev, src.data(), std::min(chunk, bytes), nullptr);
    for (size_t off = chunk; st == MHLO_CUDA_OK && off < bytes; off += chunk)
        st = mhlo_cuda_copy(static_cast<uint8_t*>(dev) + off, dev, std::min(chunk, bytes - off), nullptr);
    return st;
}
}  // namespace

int tune_gemm(const GemmCase& c, int max_trials, TuningDatabase* db, TuningRecord* out, std::string* why) {
    if ((c.dtype != MHLO_DT_BF16 && c.dtype != MHLO_DT_F16) || c.batch < 1 || c.m < 1 || c.n < 1 || c.k < 1) {
        *why = "tune_gemm: bf16 / f16 operands and positive extents expected";
        return MHLO_CUDA_INVALID_ARGUMENT;
    }
    const size_t out_es = mhlo_cuda_dtype_size(c.out_dtype);
    if (out_es == 0) { *why = "tune_gemm: bad output dtype"; return MHLO_CUDA_INVALID_ARGUMENT; }
    const size_t a_bytes = static_cast<size_t>(c.batch * c.m * c.k) * 2, b_bytes = static_cast<size_t>(c.batch * c.k * c.n) * 2,
                 c_bytes = static_cast<size_t>(c.batch * c.m * c.n) * out_es;
    void *a = nullptr, *b = nullptr, *d = nullptr, *e0 = nullptr, *e1 = nullptr;
    auto cleanup = [&] {
        if (a) mhlo_cuda_free(a);
        if (b) mhlo_cuda_free(b);
        if (d) mhlo_cuda_free(d);
        if (e0) mhlo_cuda_event_destroy(e0);
        if (e1) mhlo_cuda_event_destroy(e1);
    };
    auto failed = [&](int st) {
        *why = mhlo_cuda_last_error();
        cleanup();
        return st;
    };
    int st;
    if ((st = mhlo_cuda_alloc(a_bytes, &a)) || (st = mhlo_cuda_alloc(b_bytes, &b)) || (st = mhlo_cuda_alloc(c_bytes, &d)) ||
        (st = mhlo_cuda_event_create(&e0)) || (st = mhlo_cuda_event_create(&e1)))
        return failed(st);
    // Random operands, not zeros: the instruction stream does not depend on the values, but the power the tensor cores
    // draw does, and under the board's power cap the clocks (and with them the ranking of the candidates) follow it.
    if ((st = fill_random_16(a, a_bytes, c.dtype)) || (st = fill_random_16(b, b_bytes, c.dtype))) return failed(st);
    const int64_t as[4] = {0, c.m * c.k, c.a_k_major ? c.k : 1, c.a_k_major ? 1 : c.m};
    const int64_t bs[4] = {0, c.k * c.n, c.b_k_major ? 1 : c.n, c.b_k_major ? c.k : 1};
    std::vector<TuningConfig> candidates = gemm_candidates(c.m, c.n, c.k);
    candidates.insert(candidates.begin(), TuningConfig());  // the library's own choice competes too
    if (max_trials > 0 && static_cast<int>(candidates.size()) > max_trials) candidates.resize(static_cast<size_t>(max_trials));
    TuningRecord best;
    best.measured_time_s = 1e30;
    int tried = 0;
    for (const TuningConfig& cand : candidates) {
        mhlo_cuda_gemm_tuning t{cand.tile_n, cand.stages, cand.cta_group, 0};
        const mhlo_cuda_gemm_tuning* tp = cand.is_default() ? nullptr : &t;
        const double sec = median_seconds([&] {
            return mhlo_cuda_gemm_tuned(c.dtype, c.out_dtype, a, as, b, bs, d, 1, c.batch, c.m, c.n, c.k, nullptr, MHLO_EPILOGUE_NONE, tp, nullptr);
        }, e0, e1);
        if (sec < 0) continue;
        ++tried;
        if (sec < best.measured_time_s) {
            best.best = cand;
            best.measured_time_s = sec;
        }
    }
    int32_t device_code = 0;
    mhlo_cuda_device_error(&device_code);
    cleanup();
    if (tried == 0 || device_code != 0) {
        *why = tried == 0 ? "tune_gemm: no candidate could be launched" : "tune_gemm: a kernel gave up on a bounded wait";
        return MHLO_CUDA_EXECUTION_FAILED;
    }
    best.configs_tried = tried;
    best.gflops = 2.0 * static_cast<double>(c.batch) * c.m * c.n * c.k / best.measured_time_s / 1e9;
    best.gbytes_per_s = static_cast<double>(a_bytes + b_bytes + c_bytes) / best.measured_time_s / 1e9;
    best.timestamp = static_cast<double>(std::time(nullptr));
    if (db) db->store(c.key(current_device_name()), best);
    if (out) *out = best;
    return MHLO_CUDA_OK;
}

TuningKey AttentionCase::key(const std::string& device) const {
    TuningKey k;
    k.op_type = "fused_scaled_dot_product_attention";
    k.shapes = {{batch, heads, seq_q, head_dim}, {batch, heads, seq_k, head_dim}, {causal ? 1 : 0, bshd ? 1 : 0}};
    k.dtype = dtype_key(dtype);
    k.device = device;
    return k;
}

int tune_attention(const AttentionCase& c, int max_trials, TuningDatabase* db, TuningRecord* out, std::string* why) {
    if ((c.dtype != MHLO_DT_BF16 && c.dtype != MHLO_DT_F16) || (c.head_dim != 64 && c.head_dim != 128) || c.batch < 1 || c.heads < 1 ||
        c.seq_q < 1 || c.seq_k < 1) {
        *why = "tune_attention: bf16 / f16 operands with head dimension 64 or 128 expected (the tensor-core kernel's domain)";
        return MHLO_CUDA_INVALID_ARGUMENT;
    }
    const size_t q_bytes = static_cast<size_t>(c.batch * c.heads * c.seq_q * c.head_dim) * 2, kv_bytes = static_cast<size_t>(c.batch * c.heads * c.seq_k * c.head_dim) * 2;
    void *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr, *e0 = nullptr, *e1 = nullptr;
    auto cleanup = [&] {
        for (void* p : {q, k, v, o})
            if (p) mhlo_cuda_free(p);
        if (e0) mhlo_cuda_event_destroy(e0);
        if (e1) mhlo_cuda_event_destroy(e1);
    };
    auto failed = [&](int st) {
        *why = mhlo_cuda_last_error();
        cleanup();
        return st;
    };
    int st;
    if ((st = mhlo_cuda_alloc(q_bytes, &q)) || (st = mhlo_cuda_alloc(kv_bytes, &k)) || (st = mhlo_cuda_alloc(kv_bytes, &v)) ||
        (st = mhlo_cuda_alloc(q_bytes, &o)) || (st = mhlo_cuda_event_create(&e0)) || (st = mhlo_cuda_event_create(&e1)))
        return failed(st);
    if ((st = fill_random_16(q, q_bytes, c.dtype)) || (st = fill_random_16(k, kv_bytes, c.dtype)) || (st = fill_random_16(v, kv_bytes, c.dtype)))
        return failed(st);
    auto strides = [&](int64_t seq, int64_t* s) {
        if (c.bshd) { s[0] = seq * c.heads * c.head_dim; s[1] = c.head_dim; s[2] = c.heads * c.head_dim; }
        else { s[0] = c.heads * seq * c.head_dim; s[1] = seq * c.head_dim; s[2] = c.head_dim; }
    };
    int64_t qs[3], ks[3];
    strides(c.seq_q, qs);
    strides(c.seq_k, ks);
    std::vector<TuningConfig> candidates(3);
    candidates[1].tile_order = 1;
    candidates[2].tile_order = 2;
    if (max_trials > 0 && static_cast<int>(candidates.size()) > max_trials) candidates.resize(static_cast<size_t>(max_trials));
    TuningRecord best;
    best.measured_time_s = 1e30;
    int tried = 0;
    const float scale = 1.0f / std::sqrt(static_cast<float>(c.head_dim));
    for (const TuningConfig& cand : candidates) {
        mhlo_cuda_attention_tuning t{cand.tile_order, {0, 0, 0}};
        const mhlo_cuda_attention_tuning* tp = cand.is_default() ? nullptr : &t;
        const double sec = median_seconds([&] {
            return mhlo_cuda_attention_tuned(c.dtype, q, qs, k, ks, v, ks, nullptr, o, qs, c.batch, c.heads, c.seq_q, c.seq_k, c.head_dim, scale,
                                             c.causal ? 1 : 0, tp, nullptr);
        }, e0, e1);
        if (sec < 0) continue;
        ++tried;
        if (sec < best.measured_time_s) {
            best.best = cand;
            best.measured_time_s = sec;
        }
    }
    int32_t device_code = 0;
    mhlo_cuda_device_error(&device_code);
    cleanup();
    if (tried == 0 || device_code != 0) {
        *why = tried == 0 ? "tune_attention: no candidate could be launched" : "tune_attention: a kernel gave up on a bounded wait";
        return MHLO_CUDA_EXECUTION_FAILED;
    }
    best.configs_tried = tried;
    best.gflops = 4.0 * static_cast<double>(c.batch) * c.heads * c.seq_q * c.seq_k * c.head_dim * (c.causal ? 0.5 : 1.0) / best.measured_time_s / 1e9;
    best.timestamp = static_cast<double>(std::time(nullptr));
    if (db) db->store(c.key(current_device_name()), best);
    if (out) *out = best;
    return MHLO_CUDA_OK;
}

}  // namespace mhlo
