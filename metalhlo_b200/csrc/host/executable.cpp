// Lowers an optimised function to a list of device launches over a statically planned arena and runs it.
//
// Role in the reference: CodeGenerator.generateWithViews + buildBindings + calculateDispatch
// (Sources/MetalHLOCore/Compiler/CodeGenerator.swift:103-166,5380-5879) decide, per op, which kernel runs on
// which buffers; StaticMemoryPlanner places intermediates; IntegratedExecutor.execute
// (Sources/MetalHLOCore/Runtime/IntegratedExecutor.swift:150-270) walks the list. Here the kernels are the AOT
// sm_100a entry points of libmhlo_cuda.so, and reshape / transpose / broadcast_in_dim / slice / reverse never
// launch anything: they become strided views that the consuming kernel reads directly.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <numeric>

#include "../../../include/mhlo_cuda.h"
#include "compiler.h"
#include "tuning.h"
#include "numeric.h"

namespace mhlo {

// ---- tiny JSON field readers (backend_config of fused custom calls) -------------------------------------------------

static size_t json_find(const std::string& j, const std::string& key) {
    const std::string pat = "\"" + key + "\"";
    size_t p = j.find(pat);
    if (p == std::string::npos) return p;
    p = j.find(':', p + pat.size());
    if (p == std::string::npos) return p;
    ++p;
    while (p < j.size() && std::isspace(static_cast<unsigned char>(j[p]))) ++p;
    return p;
}
double json_number(const std::string& j, const std::string& key, double dflt) {
    size_t p = json_find(j, key);
    if (p == std::string::npos) return dflt;
    char* end = nullptr;
    double v = std::strtod(j.c_str() + p, &end);
    return end == j.c_str() + p ? dflt : v;
}
bool json_bool(const std::string& j, const std::string& key, bool dflt) {
    size_t p = json_find(j, key);
    if (p == std::string::npos) return dflt;
    if (j.compare(p, 4, "true") == 0) return true;
    if (j.compare(p, 5, "false") == 0) return false;
    return json_number(j, key, dflt ? 1 : 0) != 0;
}
std::string json_string(const std::string& j, const std::string& key, const std::string& dflt) {
    size_t p = json_find(j, key);
    if (p == std::string::npos || j[p] != '"') return dflt;
    size_t e = j.find('"', p + 1);
    return e == std::string::npos ? dflt : j.substr(p + 1, e - p - 1);
}
std::vector<int64_t> json_int_array(const std::string& j, const std::string& key) {
    std::vector<int64_t> out;
    size_t p = json_find(j, key);
    if (p == std::string::npos || j[p] != '[') return out;
    ++p;
    while (p < j.size() && j[p] != ']') {
        char* end = nullptr;
        long long v = std::strtoll(j.c_str() + p, &end, 10);
        if (end == j.c_str() + p) { ++p; continue; }
        out.push_back(v);
        p = static_cast<size_t>(end - j.c_str());
    }
    return out;
}

// ---- memory planner ---------------------------------------------------------------------------------------------------

int64_t plan_memory(std::vector<PlanInterval>* buffers) {
    std::vector<int> order(buffers->size());
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(),
                     [&](int a, int b) { return (*buffers)[a].bytes > (*buffers)[b].bytes; });
    auto align = [](int64_t v) { return (v + 255) / 256 * 256; };
    std::vector<int> placed;
    int64_t total = 0;
    for (int id : order) {
        PlanInterval& b = (*buffers)[id];
        if (b.bytes == 0) { b.offset = 0; continue; }
        // candidate offsets: 0 and the end of every placed buffer that is live at the same time
        std::vector<std::pair<int64_t, int64_t>> busy;
        for (int o : placed) {
            const PlanInterval& q = (*buffers)[o];
            if (q.last < b.first || b.last < q.first) continue;
            busy.emplace_back(q.offset, q.offset + align(q.bytes));
        }
        std::sort(busy.begin(), busy.end());
        int64_t best = -1, best_gap = INT64_MAX, cursor = 0;
        const int64_t need = align(b.bytes);
        for (const auto& iv : busy) {
            if (iv.first - cursor >= need && iv.first - cursor < best_gap) { best = cursor; best_gap = iv.first - cursor; }
            cursor = std::max(cursor, iv.second);
        }
        if (best < 0) best = cursor;  // no gap fits: append after the last conflicting buffer
        b.offset = best;
        total = std::max(total, best + need);
        placed.push_back(id);
    }
    return (total + 4095) / 4096 * 4096;
}

// ---- lowering -----------------------------------------------------------------------------------------------------------

namespace {

struct View {
    int buf = -1;
    int64_t offset = 0;  // elements
    std::vector<int64_t> strides;
    TensorType type;
};

struct Buffer {
    enum Kind { Input, Const, Arena, Output } kind = Arena;
    int index = 0;  // input / output ordinal
    int64_t bytes = 0;
    int64_t offset = 0;  // byte offset inside the const pool / arena
    int first = -1, last = -1;
};

std::vector<int64_t> dense_strides(const std::vector<int64_t>& shape) {
    std::vector<int64_t> s(shape.size());
    int64_t m = 1;
    for (int d = static_cast<int>(shape.size()) - 1; d >= 0; --d) { s[d] = m; m *= shape[d]; }
    return s;
}

// A view whose leading dimensions repeat (stride 0) over a dense block that holds whole rows of the last axis, e.g. a
// [sequence, hidden] table broadcast over the batch: the block as a dense view of its own, and how many rows it has.
bool repeated_rows(const View& v, View* block, int64_t* block_rows) {
    const int rank = v.type.rank();
    if (rank < 2) return false;
    int d0 = 0;
    while (d0 < rank - 1 && (v.strides[d0] == 0 || v.type.shape[d0] == 1)) ++d0;
    if (d0 == 0) return false;
    int64_t expect = 1, rows = 1;
    for (int d = rank - 1; d >= d0; --d) {
        if (v.type.shape[d] != 1 && v.strides[d] != expect) return false;
        expect *= v.type.shape[d];
        if (d < rank - 1) rows *= v.type.shape[d];
    }
    if (expect == 0) return false;
    block->buf = v.buf;
    block->offset = v.offset;
    block->type = v.type;
    block->type.shape.assign(v.type.shape.begin() + d0, v.type.shape.end());
    block->strides = dense_strides(block->type.shape);
    *block_rows = rows;
    return true;
}

bool is_dense(const View& v) {
    int64_t expect = 1;
    for (int d = v.type.rank() - 1; d >= 0; --d) {
        if (v.type.shape[d] == 1) continue;
        if (v.strides[d] != expect) return false;
        expect *= v.type.shape[d];
    }
    return true;
}

// numpy's no-copy reshape: can `v` be viewed with `shape` without moving data?
bool reshape_view(const View& v, const std::vector<int64_t>& shape, View* out) {
    std::vector<int64_t> os, ost;  // old dims without extent 1
    for (int d = 0; d < v.type.rank(); ++d)
        if (v.type.shape[d] != 1) { os.push_back(v.type.shape[d]); ost.push_back(v.strides[d]); }
    std::vector<int64_t> ns(shape.size(), 0);
    size_t oi = 0, ni = 0;
    const size_t on = os.size(), nn = shape.size();
    int64_t count = 1;
    for (int64_t d : shape) count *= d;
    if (count == 0) { out->strides = dense_strides(shape); return true; }
    while (ni < nn && oi < on) {
        if (shape[ni] == 1) { ns[ni++] = 0; continue; }
        int64_t np = shape[ni], op = os[oi];
        size_t oj = oi + 1, nj = ni + 1;
        while (np != op) {
            if (np < op) { if (nj >= nn) return false; np *= shape[nj++]; }
            else { if (oj >= on) return false; op *= os[oj++]; }
        }
        for (size_t k = oi; k + 1 < oj; ++k)
            if (ost[k] != ost[k + 1] * os[k + 1]) return false;  // old dims of this group are not mergeable
        int64_t st = ost[oj - 1];
        for (size_t k = nj; k-- > ni;) {
            ns[k] = st;
            st *= shape[k];
        }
        oi = oj;
        ni = nj;
    }
    for (; ni < nn; ++ni) { if (shape[ni] != 1) return false; ns[ni] = 0; }
    if (oi < on) return false;
    out->strides = ns;
    return true;
}

int ew_opcode(const std::string& n) {
    static const std::map<std::string, int> table = {
        {"add", MHLO_EW_ADD}, {"subtract", MHLO_EW_SUB}, {"multiply", MHLO_EW_MUL}, {"divide", MHLO_EW_DIV},
        {"remainder", MHLO_EW_REM}, {"maximum", MHLO_EW_MAX}, {"minimum", MHLO_EW_MIN}, {"power", MHLO_EW_POW},
        {"atan2", MHLO_EW_ATAN2}, {"and", MHLO_EW_AND}, {"or", MHLO_EW_OR}, {"xor", MHLO_EW_XOR},
        {"shift_left", MHLO_EW_SHL}, {"shift_right_arithmetic", MHLO_EW_SHR_A}, {"shift_right_logical", MHLO_EW_SHR_L},
        {"negate", MHLO_EW_NEG}, {"abs", MHLO_EW_ABS}, {"exponential", MHLO_EW_EXP}, {"exponential_minus_one", MHLO_EW_EXPM1},
        {"log", MHLO_EW_LOG}, {"log_plus_one", MHLO_EW_LOG1P}, {"sqrt", MHLO_EW_SQRT}, {"rsqrt", MHLO_EW_RSQRT},
        {"cbrt", MHLO_EW_CBRT}, {"tanh", MHLO_EW_TANH}, {"logistic", MHLO_EW_LOGISTIC}, {"sine", MHLO_EW_SIN},
        {"cosine", MHLO_EW_COS}, {"tan", MHLO_EW_TAN}, {"floor", MHLO_EW_FLOOR}, {"ceil", MHLO_EW_CEIL},
        {"round_nearest_afz", MHLO_EW_ROUND_AFZ}, {"round_nearest_even", MHLO_EW_ROUND_EVEN}, {"sign", MHLO_EW_SIGN},
        {"not", MHLO_EW_NOT}, {"is_finite", MHLO_EW_IS_FINITE}, {"popcnt", MHLO_EW_POPCNT},
        {"count_leading_zeros", MHLO_EW_CLZ}, {"convert", MHLO_EW_COPY}, {"select", MHLO_EW_SELECT},
        {"clamp", MHLO_EW_CLAMP}, {"copy", MHLO_EW_COPY}, {"optimization_barrier", MHLO_EW_COPY},
        {"gelu_tanh", MHLO_EW_GELU_TANH}, {"gelu_erf", MHLO_EW_GELU_ERF}, {"silu", MHLO_EW_SILU}, {"relu", MHLO_EW_RELU},
        {"erf", MHLO_EW_ERF},
    };
    auto it = table.find(n);
    return it == table.end() ? -1 : it->second;
}

}  // namespace

int elementwise_opcode(const std::string& name) { return ew_opcode(name); }

// Launch configuration of a fused row kernel from the process tuning database, when it holds one for this operation,
// shape, dtype and device (TuningDatabase.get in the reference's compile path, Tuning/AutoTuner.swift:301-333).
bool lookup_row_tuning(const std::string& kind, int64_t rows, int64_t hidden, DType dt, mhlo_cuda_row_tuning* out) {
    TuningDatabase* db = TuningDatabase::global();
    if (!db) return false;
    static std::string device_name = [] {
        char name[256] = "";
        int ordinal = 0;
        if (mhlo_cuda_device_current(&ordinal) == MHLO_CUDA_OK) mhlo_cuda_device_name(ordinal, name, sizeof name);
        return std::string(name);
    }();
    TuningKey key;
    key.op_type = kind;
    key.shapes = {{rows, hidden}};
    key.dtype = dt == DType::BF16 ? "bf16" : dt == DType::F16 ? "f16" : "f32";
    key.device = device_name;
    TuningRecord rec;
    if (!db->get(key, &rec)) return false;
    if (!rec.best.threads && !rec.best.vectors_per_thread && !rec.best.ctas_per_sm) return false;  // the default won
    *out = mhlo_cuda_row_tuning{rec.best.threads, rec.best.vectors_per_thread, rec.best.ctas_per_sm};
    return true;
}

// The same for the tensor-core GEMM and attention kernels: a stored record whose configuration is not the library's own
// choice becomes the launch's tuning argument.
bool lookup_gemm_tuning(const GemmCase& c, mhlo_cuda_gemm_tuning* out) {
    TuningDatabase* db = TuningDatabase::global();
    if (!db || (c.dtype != MHLO_DT_BF16 && c.dtype != MHLO_DT_F16)) return false;
    static const std::string device_name = current_device_name();
    TuningRecord rec;
    if (!db->get(c.key(device_name), &rec) || rec.best.is_default()) return false;
    *out = mhlo_cuda_gemm_tuning{rec.best.tile_n, rec.best.stages, rec.best.cta_group, 0};
    return true;
}

bool lookup_attention_tuning(const AttentionCase& c, mhlo_cuda_attention_tuning* out) {
    TuningDatabase* db = TuningDatabase::global();
    if (!db) return false;
    static const std::string device_name = current_device_name();
    TuningRecord rec;
    if (!db->get(c.key(device_name), &rec) || rec.best.is_default()) return false;
    *out = mhlo_cuda_attention_tuning{rec.best.tile_order, {0, 0, 0}};
    return true;
}

class Lowering {
  public:
    Lowering(const Function& f, Executable* exe) : f_(f), exe_(exe), views_(f.values.size()), have_(f.values.size(), false) {}

    void run() {
        for (size_t i = 0; i < f_.args.size(); ++i) {
            Buffer b;
            b.kind = Buffer::Input;
            b.index = static_cast<int>(i);
            b.bytes = f_.type_of(f_.args[i]).bytes();
            set(f_.args[i], dense_view(add_buffer(b), f_.type_of(f_.args[i])));
            exe_->input_types_.push_back(f_.type_of(f_.args[i]));
            exe_->input_types_.back().was_complex = i < f_.arg_complex.size() && f_.arg_complex[i];
        }
        open_parameter_converts();
        for (const Op& op : f_.ops) {
            if (op.dead) continue;
            if (op.name == "return") { lower_return(op); break; }
            lower(op);
        }
        plan();
    }

  private:
    const Function& f_;
    Executable* exe_;
    std::vector<View> views_;
    std::vector<bool> have_;
    std::vector<Buffer> buffers_;

    using Ctx = Executable::Ctx;

    // ---- buffers and views ----------------------------------------------------------------------------------------
    int add_buffer(const Buffer& b) { buffers_.push_back(b); return static_cast<int>(buffers_.size()) - 1; }
    int new_arena(int64_t bytes) { Buffer b; b.kind = Buffer::Arena; b.bytes = bytes; return add_buffer(b); }
    static View dense_view(int buf, const TensorType& t) { View v; v.buf = buf; v.type = t; v.strides = dense_strides(t.shape); return v; }
    void set(int value, const View& v) { views_[value] = v; have_[value] = true; }
    const View& get(int value) const {
        if (!have_[value]) fail_compile("internal: value " + f_.values[value].name + " used before it is lowered");
        return views_[value];
    }
    int step_index() const { return static_cast<int>(exe_->steps_.size()); }
    void touch(int buf) {
        Buffer& b = buffers_[buf];
        const int s = step_index();
        if (b.first < 0) b.first = s;
        b.last = std::max(b.last, s);
    }
    void keep_alive(const View& v) { touch(v.buf); }

    // Resolved at run time: base pointer of a buffer.
    std::function<char*(const Ctx&)> resolver(int buf) {
        // The buffer table is final only after plan(); capture the index and look it up through a shared copy.
        auto table = table_;
        return [table, buf](const Ctx& c) -> char* {
            const Buffer& b = (*table)[buf];
            switch (b.kind) {
                case Buffer::Input: return static_cast<char*>(const_cast<void*>(c.inputs[b.index]));
                case Buffer::Output: return static_cast<char*>(c.outputs[b.index]);
                case Buffer::Const: return c.consts + b.offset;
                default: return c.arena + b.offset;
            }
        };
    }
    std::shared_ptr<std::vector<Buffer>> table_ = std::make_shared<std::vector<Buffer>>();

    struct DevView {  // a View whose pointer is resolved per call
        std::function<char*(const Ctx&)> base;
        mhlo_cuda_view v;
        int64_t byte_offset;
    };
    DevView dev(const View& v) {
        if (v.type.rank() > MHLO_CUDA_MAX_RANK) fail_unsupported("tensor rank above 8: " + v.type.str());
        DevView d;
        d.base = resolver(v.buf);
        std::memset(&d.v, 0, sizeof d.v);
        d.v.dtype = static_cast<int>(v.type.dtype);
        d.v.rank = v.type.rank();
        for (int i = 0; i < v.type.rank(); ++i) { d.v.shape[i] = v.type.shape[i]; d.v.stride[i] = v.strides[i]; }
        d.byte_offset = v.offset * static_cast<int64_t>(dtype_size(v.type.dtype));
        return d;
    }
    static mhlo_cuda_view bind(const DevView& d, const Ctx& c) {
        mhlo_cuda_view v = d.v;
        v.base = d.base(c) + d.byte_offset;
        return v;
    }

    // Steps go to the executable's list, or to the list of a loop region while one is being lowered.
    std::vector<Executable::Step>* sink_ = nullptr;
    std::string detail_;  // result type of the op being lowered
    void add_step(const std::string& label, std::function<int(const Ctx&)> run, int launches = 1) {
        Executable::Step s;
        s.label = label;
        s.detail = detail_;
        s.run = std::move(run);
        s.launches = launches;
        (sink_ ? *sink_ : exe_->steps_).push_back(std::move(s));
        exe_->launches_per_run_ += launches;
    }

    // Copies a view into a fresh dense arena buffer (the only place a transpose / broadcast / slice costs a launch).
    View materialize(const View& v, const std::string& why) {
        if (is_dense(v)) return v;
        View out = dense_view(new_arena(v.type.bytes()), v.type);
        copy_view(v, out, "copy(" + why + ")");
        return out;
    }
    // A dense view whose element 0 is at the buffer start (needed when a raw pointer is handed to a kernel that
    // takes an offset-free base is NOT required: pointers carry the offset). Kept for clarity.
    void copy_view(const View& src, const View& dst, const std::string& label) {
        DevView s = dev(src), d = dev(dst);
        keep_alive(src);
        keep_alive(dst);
        add_step(label, [s, d](const Ctx& c) {
            mhlo_cuda_view sv = bind(s, c), dv = bind(d, c);
            mhlo_cuda_ew_inst inst = {MHLO_EW_COPY, 0, 0, 0, 0.0};
            return mhlo_cuda_elementwise_to_view(&sv, 1, &inst, 1, &dv, c.stream);
        });
    }

    // Broadcasts a view to `shape` (numpy-style trailing alignment is NOT used: StableHLO operands already have
    // the result rank except for scalars, which broadcast everywhere).
    static View expand_to(const View& v, const std::vector<int64_t>& shape) {
        if (v.type.shape == shape) return v;
        View o = v;
        o.type.shape = shape;
        o.strides.assign(shape.size(), 0);
        if (v.type.rank() == static_cast<int>(shape.size()))
            for (size_t d = 0; d < shape.size(); ++d) o.strides[d] = v.type.shape[d] == shape[d] ? v.strides[d] : 0;
        return o;
    }

    // Elementwise program over `ins` (each already of the output shape) into a new dense buffer.
    View emit_elementwise(const std::vector<View>& ins, const std::vector<mhlo_cuda_ew_inst>& prog, const TensorType& out_t,
                          const std::string& label) {
        View out = dense_view(new_arena(out_t.bytes()), out_t);
        std::vector<DevView> dv;
        for (const View& v : ins) { dv.push_back(dev(expand_to(v, out_t.shape))); keep_alive(v); }
        keep_alive(out);
        DevView dout = dev(out);
        add_step(label, [dv, dout, prog, out_t](const Ctx& c) {
            mhlo_cuda_view in[MHLO_CUDA_EW_MAX_INPUTS];
            for (size_t i = 0; i < dv.size(); ++i) in[i] = bind(dv[i], c);
            mhlo_cuda_view o = bind(dout, c);
            return mhlo_cuda_elementwise(in, static_cast<int>(dv.size()), prog.data(), static_cast<int>(prog.size()),
                                         const_cast<void*>(o.base), static_cast<int>(out_t.dtype), out_t.shape.data(),
                                         out_t.rank(), c.stream);
        });
        return out;
    }

    // ---- per-op lowering --------------------------------------------------------------------------------------------
    // ---- dtype conversions of whole function parameters, gathered into one launch at the start of the program --------
    // A module whose parameters arrive as fp32 and which computes in 16 bit converts every weight once per run (148
    // converts in the GPT-2 module, most of them a few KB). They depend on nothing but the inputs, so they all run in
    // step 0 as one batched launch instead of one launch each.
    struct ParamConvert {
        std::function<char*(const Ctx&)> src, dst;
        int64_t count;
        int32_t src_dtype, dst_dtype;
    };
    std::shared_ptr<std::vector<ParamConvert>> param_converts_;

    static bool batchable_float(DType d) { return d == DType::F32 || d == DType::F16 || d == DType::BF16; }
    bool is_parameter_convert(const Op& op) const {
        if (op.name != "convert" || op.operands.size() != 1 || op.results.empty()) return false;
        const int v = op.operands[0];
        if (!have_[v]) return false;
        const View& x = views_[v];
        if (buffers_[x.buf].kind != Buffer::Input || x.offset != 0 || !is_dense(x)) return false;
        const TensorType& rt = op.result_types[0];
        if (!batchable_float(x.type.dtype) || !batchable_float(rt.dtype)) return false;
        return x.type.dtype == rt.dtype || x.type.dtype == DType::F32 || rt.dtype == DType::F32;
    }
    // Reserves step 0 for the batch when at least two converts qualify (called when only the parameters have views).
    void open_parameter_converts() {
        int n = 0;
        for (const Op& op : f_.ops) n += !op.dead && is_parameter_convert(op);
        if (n < 2) return;
        param_converts_ = std::make_shared<std::vector<ParamConvert>>();
        auto jobs = param_converts_;
        add_step("convert_parameters(x" + std::to_string(n) + ")", [jobs](const Ctx& c) {
            std::vector<mhlo_cuda_convert_job> list(jobs->size());
            for (size_t i = 0; i < jobs->size(); ++i) {
                const ParamConvert& j = (*jobs)[i];
                list[i] = mhlo_cuda_convert_job{j.src(c), j.dst(c), j.count, j.src_dtype, j.dst_dtype};
            }
            return mhlo_cuda_convert_many(list.data(), static_cast<int32_t>(list.size()), c.stream);
        }, (n + 95) / 96);
    }
    void lower_parameter_convert(const Op& op) {
        const View& x = get(op.operands[0]);
        const TensorType& rt = op.result_types[0];
        View out = dense_view(new_arena(rt.bytes()), rt);
        // both buffers are in use from step 0 on, whatever the position of the convert in the program
        buffers_[x.buf].first = 0;
        buffers_[out.buf].first = 0;
        buffers_[out.buf].last = std::max(buffers_[out.buf].last, 0);
        param_converts_->push_back(ParamConvert{resolver(x.buf), resolver(out.buf), rt.count(), static_cast<int32_t>(x.type.dtype),
                                                static_cast<int32_t>(rt.dtype)});
        set(op.results[0], out);
    }

    void lower(const Op& op) {
        const std::string& n = op.name;
        if (op.results.empty()) return;  // ops without results have no effect here
        const TensorType& rt = op.result_types[0];
        detail_ = rt.str();
        if (param_converts_ && is_parameter_convert(op)) return lower_parameter_convert(op);
        if (n == "constant") return lower_constant(op);
        if (n == "reshape" || n == "bitcast" || n == "dynamic_reshape") return lower_reshape(op);
        if (n == "bitcast_convert") return lower_bitcast_convert(op);
        if (n == "dynamic_pad") {  // the padding amounts are operands; they must be constants of the module
            if (op.operands.size() != 5) fail_compile("dynamic_pad takes five operands");
            Op p = op;
            p.name = "pad";
            p.operands.resize(2);
            p.attrs["edge_padding_low"] = Attr::make_ints(constant_ints(op.operands[2], "dynamic_pad: edge_padding_low"));
            p.attrs["edge_padding_high"] = Attr::make_ints(constant_ints(op.operands[3], "dynamic_pad: edge_padding_high"));
            p.attrs["interior_padding"] = Attr::make_ints(constant_ints(op.operands[4], "dynamic_pad: interior_padding"));
            return lower_pad(p);
        }
        if (n == "dynamic_gather") {
            if (op.operands.size() != 3) fail_compile("dynamic_gather takes three operands");
            Op g = op;
            g.name = "gather";
            g.operands.resize(2);
            g.attrs["slice_sizes"] = Attr::make_ints(constant_ints(op.operands[2], "dynamic_gather: slice_sizes"));
            return lower_gather(g);
        }
        if (n == "batch_norm_inference") return lower_batch_norm_inference(op);
        if (n == "get_dimension_size") {  // shapes are static: the extent is a constant
            const View& x = get(op.operands[0]);
            const int64_t d = op.int_attr("dimension", 0);
            if (d < 0 || d >= x.type.rank()) fail_compile("get_dimension_size: dimension out of range");
            std::vector<mhlo_cuda_ew_inst> prog = {{MHLO_EW_IMM, 0, 0, 0, static_cast<double>(x.type.shape[static_cast<size_t>(d)])}};
            return set(op.results[0], emit_elementwise({}, prog, rt, "get_dimension_size"));
        }
        if (n == "transpose") {
            const View& x = get(op.operands[0]);
            std::vector<int64_t> perm = op.int_list("permutation");
            if (static_cast<int>(perm.size()) != x.type.rank()) fail_compile("transpose: permutation rank mismatch");
            View o = x;
            o.type = rt;
            for (size_t d = 0; d < perm.size(); ++d) o.strides[d] = x.strides[perm[d]];
            return set(op.results[0], o);
        }
        if (n == "broadcast_in_dim" || n == "dynamic_broadcast_in_dim") {  // the dynamic form's result type is static here
            const View& x = get(op.operands[0]);
            std::vector<int64_t> dims = op.int_list("broadcast_dimensions");
            if (static_cast<int>(dims.size()) != x.type.rank()) fail_compile("broadcast_in_dim: dims rank mismatch");
            View o = x;
            o.type = rt;
            o.strides.assign(rt.shape.size(), 0);
            for (size_t d = 0; d < dims.size(); ++d)
                o.strides[dims[d]] = (x.type.shape[d] == 1 && rt.shape[dims[d]] != 1) ? 0 : x.strides[d];
            return set(op.results[0], o);
        }
        if (n == "broadcast") {  // leading broadcast_sizes
            const View& x = get(op.operands[0]);
            View o = x;
            o.type = rt;
            const size_t lead = rt.shape.size() - x.type.shape.size();
            o.strides.assign(rt.shape.size(), 0);
            for (size_t d = 0; d < x.strides.size(); ++d) o.strides[lead + d] = x.strides[d];
            return set(op.results[0], o);
        }
        if (n == "slice") {
            const View& x = get(op.operands[0]);
            std::vector<int64_t> st = op.int_list("start_indices"), sd = op.int_list("strides");
            if (sd.empty()) sd.assign(st.size(), 1);
            View o = x;
            o.type = rt;
            for (size_t d = 0; d < st.size(); ++d) { o.offset += st[d] * x.strides[d]; o.strides[d] = x.strides[d] * sd[d]; }
            return set(op.results[0], o);
        }
        if (n == "reverse") {
            const View& x = get(op.operands[0]);
            View o = x;
            for (int64_t d : op.int_list("dimensions")) {
                o.offset += (x.type.shape[d] - 1) * x.strides[d];
                o.strides[d] = -x.strides[d];
            }
            return set(op.results[0], o);
        }
        if (n == "iota" || n == "dynamic_iota") {
            std::vector<mhlo_cuda_ew_inst> prog = {{MHLO_EW_IOTA, 0, 0, 0, static_cast<double>(op.int_attr("iota_dimension", 0))}};
            return set(op.results[0], emit_elementwise({}, prog, rt, "iota"));
        }
        if (n == "compare") {
            static const std::map<std::string, int> dir = {{"EQ", MHLO_EW_CMP_EQ}, {"NE", MHLO_EW_CMP_NE}, {"LT", MHLO_EW_CMP_LT},
                                                           {"LE", MHLO_EW_CMP_LE}, {"GT", MHLO_EW_CMP_GT}, {"GE", MHLO_EW_CMP_GE}};
            auto it = dir.find(op.str_attr("comparison_direction"));
            if (it == dir.end()) fail_compile("compare without a comparison_direction");
            const View& lhs = get(op.operands[0]);
            if (op.str_attr("compare_type") == "TOTALORDER" && is_float(lhs.type.dtype)) {
                // -NaN < -inf < .. < -0 < +0 < .. < +inf < +NaN: read the operands as signed integers of the same width and
                // flip the magnitude bits of the negative ones; the integer comparison of the results is the total order
                const size_t es = dtype_size(lhs.type.dtype);
                const DType as_int = es == 2 ? DType::I16 : es == 4 ? DType::I32 : DType::I64;
                View a = lhs, b = get(op.operands[1]);
                a.type.dtype = as_int;
                b.type.dtype = as_int;
                const double top = static_cast<double>(8 * es - 1);
                std::vector<mhlo_cuda_ew_inst> prog = {
                    {MHLO_EW_IMM, 0, 0, 0, top},      // r2 = width - 1
                    {MHLO_EW_IMM, 0, 0, 0, 1.0},      // r3 = 1
                    {MHLO_EW_SHR_A, 0, 2, 0, 0.0},    // r4 = all ones where a is negative
                    {MHLO_EW_SHR_L, 4, 3, 0, 0.0},    // r5 = the magnitude mask of those
                    {MHLO_EW_XOR, 0, 5, 0, 0.0},      // r6 = ordered key of a
                    {MHLO_EW_SHR_A, 1, 2, 0, 0.0},    // r7
                    {MHLO_EW_SHR_L, 7, 3, 0, 0.0},    // r8
                    {MHLO_EW_XOR, 1, 8, 0, 0.0},      // r9 = ordered key of b
                    {it->second, 6, 9, 0, 0.0},
                };
                return set(op.results[0], emit_elementwise({a, b}, prog, rt, "compare.totalorder"));
            }
            std::vector<mhlo_cuda_ew_inst> prog = {{it->second, 0, 1, 0, 0.0}};
            return set(op.results[0], emit_elementwise({lhs, get(op.operands[1])}, prog, rt, "compare"));
        }
        if (n == "concatenate") return lower_concatenate(op);
        if (n == "pad") return lower_pad(op);
        if (n == "reduce") return lower_reduce(op);
        if (n == "dot_general" || n == "dot") return lower_dot(op);
        if (n == "gather") return lower_gather(op);
        if (n == "convolution") return lower_convolution(op);
        if (n == "dynamic_conv") {  // the padding is an operand ([spatial dims, 2]); it must be a constant of the module
            if (op.operands.size() != 3) fail_compile("dynamic_conv takes three operands");
            Op c = op;
            c.name = "convolution";
            c.operands.resize(2);
            c.attrs["padding"] = Attr::make_ints(constant_ints(op.operands[2], "dynamic_conv: padding"));
            return lower_convolution(c);
        }
        if (n == "reduce_window") return lower_reduce_window(op);
        if (n == "while") return lower_while(op);
        if (n == "scatter") return lower_scatter(op);
        if (n == "select_and_scatter") return lower_select_and_scatter(op);
        if (n == "sort") return lower_sort(op);
        if (n == "dynamic_slice") return lower_dynamic_slice(op);
        if (n == "dynamic_update_slice") return lower_dynamic_update_slice(op);
        if (n == "custom_call") return lower_custom_call(op);
        if (n == "cholesky") return lower_cholesky(op);
        if (n == "triangular_solve") return lower_triangular_solve(op);
        if (n == "rng_bit_generator") return lower_rng_bit_generator(op);
        if (n == "rng") return lower_rng(op);
        if (n == "fft") return lower_fft(op);
        if (n == "tuple" || n == "get_tuple_element" || n == "if" || n == "case" || n == "call" ||
            n == "map" || n == "all_reduce" || n == "all_gather")
            fail_unsupported("operation stablehlo." + n + " is outside this backend's operator surface");
        if (n == "reduce_precision") {
            // `format = e5m10` in the pretty form, exponent_bits / mantissa_bits in the generic one
            int64_t e = op.int_attr("exponent_bits", -1), m = op.int_attr("mantissa_bits", -1);
            const std::string fmt = op.str_attr("format");
            if (fmt.size() >= 4 && fmt[0] == 'e') {
                const size_t mpos = fmt.find('m');
                if (mpos != std::string::npos) { e = std::atoll(fmt.substr(1, mpos - 1).c_str()); m = std::atoll(fmt.substr(mpos + 1).c_str()); }
            }
            if (e < 1 || m < 0 || e > 11 || m > 52 || !is_float(rt.dtype)) fail_unsupported("reduce_precision: format e" + std::to_string(e) + "m" + std::to_string(m));
            mhlo_cuda_ew_inst inst = {MHLO_EW_REDUCE_PRECISION, 0, 0, 0, static_cast<double>(e * 64 + m)};
            return set(op.results[0], emit_elementwise({get(op.operands[0])}, {inst}, rt, n));
        }
        const int code = ew_opcode(n);
        if (code >= 0) {
            std::vector<View> ins;
            for (int v : op.operands) ins.push_back(get(v));
            if (ins.empty() || ins.size() > 3) fail_compile("elementwise op " + n + " with " + std::to_string(ins.size()) + " operands");
            mhlo_cuda_ew_inst inst = {code, 0, ins.size() > 1 ? 1 : 0, ins.size() > 2 ? 2 : 0, 0.0};
            return set(op.results[0], emit_elementwise(ins, {inst}, rt, n));
        }
        fail_unsupported("unsupported operation: " + (op.dialect.empty() ? "" : op.dialect + ".") + n);
    }

    void lower_constant(const Op& op) {
        const Attr* val = op.attr("value");
        const TensorType& rt = op.result_types[0];
        if (!val || val->kind != Attr::Dense) fail_compile("constant without a dense value");
        Buffer b;
        b.kind = Buffer::Const;
        const size_t es = dtype_size(rt.dtype);
        std::vector<uint8_t> bytes = val->dense;
        const bool splat = val->splat || (bytes.size() == es && rt.count() != 1);
        if (!splat && static_cast<int64_t>(bytes.size()) != rt.bytes())
            fail_compile("constant payload of " + std::to_string(bytes.size()) + " bytes does not match " + rt.str());
        // 256-byte aligned slot in the pool
        size_t off = (exe_->const_pool_.size() + 255) / 256 * 256;
        exe_->const_pool_.resize(off + std::max<size_t>(bytes.size(), 1), 0);
        if (!bytes.empty()) std::memcpy(exe_->const_pool_.data() + off, bytes.data(), bytes.size());
        b.offset = static_cast<int64_t>(off);
        b.bytes = static_cast<int64_t>(bytes.size());
        View v = dense_view(add_buffer(b), rt);
        if (splat) v.strides.assign(rt.shape.size(), 0);
        set(op.results[0], v);
    }

    void lower_reshape(const Op& op) {
        const View& x = get(op.operands[0]);
        const TensorType& rt = op.result_types[0];
        View o = x;
        o.type = rt;
        if (x.type.dtype != rt.dtype) {
            if (dtype_size(x.type.dtype) != dtype_size(rt.dtype) || !is_dense(x)) fail_unsupported("bitcast between element sizes");
        }
        if (reshape_view(x, rt.shape, &o)) return set(op.results[0], o);
        View m = materialize(x, "reshape");
        o = m;
        o.type = rt;
        o.strides = dense_strides(rt.shape);
        set(op.results[0], o);
    }

    // stablehlo.bitcast_convert: the same bits under another element type. Equal element sizes re-type the view; a
    // narrower result gains a minor dimension of (old size / new size), a wider one loses it.
    void lower_bitcast_convert(const Op& op) {
        const View& x = get(op.operands[0]);
        const TensorType& rt = op.result_types[0];
        const int64_t from = static_cast<int64_t>(dtype_size(x.type.dtype)), to = static_cast<int64_t>(dtype_size(rt.dtype));
        if (x.type.dtype == DType::I1 || rt.dtype == DType::I1) fail_unsupported("bitcast_convert of i1");
        if (from == to) {
            if (x.type.shape != rt.shape) fail_compile("bitcast_convert: " + x.type.str() + " -> " + rt.str());
            View o = x;
            o.type = rt;
            return set(op.results[0], o);
        }
        if (x.type.bytes() != rt.bytes()) fail_compile("bitcast_convert: " + x.type.str() + " -> " + rt.str());
        View m = materialize(x, "bitcast_convert");
        if ((m.offset * from) % to != 0) fail_unsupported("bitcast_convert of a misaligned view");
        View o = m;
        o.type = rt;
        o.offset = m.offset * from / to;
        o.strides = dense_strides(rt.shape);
        set(op.results[0], o);
    }

    // Integer payload of a value that the module defines as a constant.
    std::vector<int64_t> constant_ints(int value, const std::string& what) {
        const View& v = get(value);
        const Buffer& b = buffers_[v.buf];
        if (b.kind != Buffer::Const || is_float(v.type.dtype)) fail_unsupported(what + " must be an integer constant");
        const size_t es = dtype_size(v.type.dtype);
        std::vector<int64_t> out;
        const int64_t n = v.type.count();
        std::vector<int64_t> idx(static_cast<size_t>(v.type.rank()), 0);  // row-major walk over a view of any rank
        for (int64_t i = 0; i < n; ++i) {
            int64_t at = v.offset;
            for (int d = 0; d < v.type.rank(); ++d) at += idx[static_cast<size_t>(d)] * v.strides[static_cast<size_t>(d)];
            for (int d = v.type.rank() - 1; d >= 0; --d) {
                if (++idx[static_cast<size_t>(d)] < v.type.shape[static_cast<size_t>(d)]) break;
                idx[static_cast<size_t>(d)] = 0;
            }
            const uint8_t* p = exe_->const_pool_.data() + b.offset + at * static_cast<int64_t>(es);
            uint64_t raw = 0;
            for (size_t k = 0; k < es; ++k) raw |= static_cast<uint64_t>(p[k]) << (8 * k);
            if (!is_unsigned(v.type.dtype) && es < 8 && (raw >> (8 * es - 1)) & 1) raw |= ~0ull << (8 * es);
            out.push_back(static_cast<int64_t>(raw));
        }
        return out;
    }

    // stablehlo.batch_norm_inference: (x - mean) * rsqrt(variance + epsilon) * scale + offset with the four statistics
    // broadcast along feature_index; one elementwise launch.
    void lower_batch_norm_inference(const Op& op) {
        if (op.operands.size() != 5) fail_compile("batch_norm_inference takes five operands");
        const TensorType& rt = op.result_types[0];
        const View& x = get(op.operands[0]);
        const int64_t axis = op.int_attr("feature_index", 0);
        if (axis < 0 || axis >= rt.rank()) fail_compile("batch_norm_inference: feature_index out of range");
        const Attr* ea = op.attr("epsilon");
        const double eps = ea ? ea->as_float() : 0.0;
        std::vector<View> ins = {x};
        for (int i = 1; i < 5; ++i) {  // scale, offset, mean, variance: [C] viewed as [1, .., C, .., 1]
            const View& s = get(op.operands[static_cast<size_t>(i)]);
            if (s.type.rank() != 1 || s.type.shape[0] != rt.shape[static_cast<size_t>(axis)])
                fail_compile("batch_norm_inference: statistics must have the feature dimension's length");
            View b = s;
            b.type.shape = rt.shape;
            b.strides.assign(rt.shape.size(), 0);
            b.strides[static_cast<size_t>(axis)] = s.strides[0];
            ins.push_back(b);
        }
        // registers: inputs 0..4 (x, scale, offset, mean, variance), the result of instruction i at 5 + i
        std::vector<mhlo_cuda_ew_inst> prog = {
            {MHLO_EW_SUB, 0, 3, 0, 0.0},    // r5 = x - mean
            {MHLO_EW_IMM, 0, 0, 0, eps},    // r6 = epsilon
            {MHLO_EW_ADD, 4, 6, 0, 0.0},    // r7 = variance + epsilon
            {MHLO_EW_RSQRT, 7, 0, 0, 0.0},  // r8
            {MHLO_EW_MUL, 5, 8, 0, 0.0},    // r9
            {MHLO_EW_MUL, 9, 1, 0, 0.0},    // r10 = .. * scale
            {MHLO_EW_ADD, 10, 2, 0, 0.0},   // r11 = .. + offset
        };
        set(op.results[0], emit_elementwise(ins, prog, rt, "batch_norm_inference"));
    }

    void lower_concatenate(const Op& op) {
        const TensorType& rt = op.result_types[0];
        const int64_t dim = op.int_attr("dimension", 0);
        View out = dense_view(new_arena(rt.bytes()), rt);
        int64_t at = 0;
        for (int v : op.operands) {
            const View& x = get(v);
            View dst = out;
            dst.type.shape = x.type.shape;
            dst.offset = at * out.strides[dim];
            copy_view(x, dst, "concatenate");
            at += x.type.shape[dim];
        }
        set(op.results[0], out);
    }

    void lower_pad(const Op& op) {
        const TensorType& rt = op.result_types[0];
        View x = get(op.operands[0]);
        const View& pv = get(op.operands[1]);
        std::vector<int64_t> lo = op.int_list("edge_padding_low"), hi = op.int_list("edge_padding_high"),
                             in = op.int_list("interior_padding");
        if (in.empty()) in.assign(lo.size(), 0);
        View out = dense_view(new_arena(rt.bytes()), rt);
        copy_view(expand_to(pv, rt.shape), out, "pad.fill");
        // negative edge padding trims the operand first
        View dst = out;
        for (size_t d = 0; d < lo.size(); ++d) {
            const int64_t step = in[d] + 1;
            int64_t first = 0, count = x.type.shape[d];
            // operand element j lands at lo + j*step; keep those inside [0, out extent)
            while (count > 0 && lo[d] + first * step < 0) { ++first; --count; }
            while (count > 0 && lo[d] + (first + count - 1) * step >= rt.shape[d]) --count;
            x.offset += first * x.strides[d];
            x.type.shape[d] = count;
            dst.offset += (lo[d] + first * step) * out.strides[d];
            dst.strides[d] = out.strides[d] * step;
            dst.type.shape[d] = count;
        }
        if (x.type.count() > 0) copy_view(x, dst, "pad.interior");
        set(op.results[0], out);
    }

    void lower_reduce(const Op& op) {
        const size_t n_in = op.operands.size() / 2;
        std::string red = op.str_attr("reducer");
        static const std::map<std::string, int> kinds = {
            {"add", MHLO_REDUCE_SUM}, {"maximum", MHLO_REDUCE_MAX}, {"minimum", MHLO_REDUCE_MIN}, {"multiply", MHLO_REDUCE_PROD},
            {"and", MHLO_REDUCE_AND}, {"or", MHLO_REDUCE_OR}, {"xor", MHLO_REDUCE_XOR}, {"argmax", MHLO_REDUCE_ARGMAX},
            {"argmin", MHLO_REDUCE_ARGMIN}};
        auto it = kinds.find(red);
        if (it == kinds.end()) fail_unsupported("reduce with a reducer body this backend does not recognise (" + red + ")");
        int kind = it->second;
        const bool arg = kind == MHLO_REDUCE_ARGMAX || kind == MHLO_REDUCE_ARGMIN;
        if ((arg && n_in != 2) || (!arg && n_in != 1)) fail_unsupported("variadic reduce other than the argmax/argmin form");
        const View& x = get(op.operands[0]);
        // the reduce kernels accumulate every integer type in a signed 64-bit register: sums, products and bitwise reducers
        // wrap correctly, but an ordering of ui64 values at or above 2^63 would come out wrong
        if (x.type.dtype == DType::UI64 && (kind == MHLO_REDUCE_MAX || kind == MHLO_REDUCE_MIN || arg))
            fail_unsupported("reduce: maximum / minimum / argmax / argmin over ui64 is outside this backend's operator surface");
        std::vector<int64_t> dims = op.int_list("dimensions");
        std::vector<bool> reduced(x.type.rank(), false);
        for (int64_t d : dims) reduced[d] = true;
        View p = x;
        p.type.shape.clear();
        p.strides.clear();
        int kept = 0;
        for (int d = 0; d < x.type.rank(); ++d)
            if (!reduced[d]) { p.type.shape.push_back(x.type.shape[d]); p.strides.push_back(x.strides[d]); ++kept; }
        for (int d = 0; d < x.type.rank(); ++d)
            if (reduced[d]) { p.type.shape.push_back(x.type.shape[d]); p.strides.push_back(x.strides[d]); }
        if (arg && dims.size() != 1) fail_unsupported("argmax/argmin over more than one dimension");
        const TensorType& rt = op.result_types[0];
        View out = dense_view(new_arena(rt.bytes()), rt);
        View iout;
        DevView dio;
        bool has_index = false;
        if (arg) {
            const TensorType& it2 = op.result_types[1];
            if (it2.dtype != DType::I32 && it2.dtype != DType::I64) fail_unsupported("argmax index type " + it2.str());
            iout = dense_view(new_arena(it2.bytes()), it2);
            dio = dev(iout);
            has_index = true;
        }
        View init = materialize(get(op.operands[n_in]), "reduce.init");
        DevView dp = dev(p), dout = dev(out), dinit = dev(init);
        keep_alive(x); keep_alive(out); keep_alive(init);
        if (has_index) keep_alive(iout);
        const int index_dtype = has_index ? static_cast<int>(op.result_types[1].dtype) : MHLO_DT_I32;
        add_step("reduce." + red, [dp, dout, dinit, dio, has_index, kept, kind, index_dtype](const Ctx& c) {
            mhlo_cuda_view in = bind(dp, c);
            return mhlo_cuda_reduce(&in, kept, kind, bind(dinit, c).base, const_cast<void*>(bind(dout, c).base),
                                    has_index ? const_cast<void*>(bind(dio, c).base) : nullptr, index_dtype, c.stream);
        });
        set(op.results[0], out);
        if (arg) set(op.results[1], iout);
    }

    // Merges a group of (extent, stride) pairs into as few dims as their strides allow.
    static void merge_group(std::vector<int64_t>* shape, std::vector<int64_t>* stride) {
        std::vector<int64_t> s, t;
        for (size_t i = 0; i < shape->size(); ++i) {
            if ((*shape)[i] == 1) continue;
            if (!s.empty() && t.back() == (*stride)[i] * (*shape)[i]) { s.back() *= (*shape)[i]; t.back() = (*stride)[i]; }
            else { s.push_back((*shape)[i]); t.push_back((*stride)[i]); }
        }
        *shape = s;
        *stride = t;
    }

    void lower_dot(const Op& op) {
        View a = get(op.operands[0]), b = get(op.operands[1]);
        const TensorType& rt = op.result_types[0];
        std::vector<int64_t> lb, rb, lc, rc;
        if (op.name == "dot") {
            lc = {a.type.rank() - 1};
            rc = {0};
        } else {
            lb = op.int_list("lhs_batching_dimensions"); rb = op.int_list("rhs_batching_dimensions");
            lc = op.int_list("lhs_contracting_dimensions"); rc = op.int_list("rhs_contracting_dimensions");
        }
        auto rest = [](int rank, const std::vector<int64_t>& x, const std::vector<int64_t>& y) {
            std::vector<int64_t> r;
            for (int d = 0; d < rank; ++d)
                if (std::find(x.begin(), x.end(), d) == x.end() && std::find(y.begin(), y.end(), d) == y.end()) r.push_back(d);
            return r;
        };
        std::vector<int64_t> lf = rest(a.type.rank(), lb, lc), rf = rest(b.type.rank(), rb, rc);
        struct Grp { std::vector<int64_t> shape, stride; };
        auto group = [](const View& v, const std::vector<int64_t>& dims) {
            Grp g;
            for (int64_t d : dims) { g.shape.push_back(v.type.shape[d]); g.stride.push_back(v.strides[d]); }
            return g;
        };
        auto extent = [](const Grp& g) { int64_t n = 1; for (int64_t d : g.shape) n *= d; return n; };
        // try the views as they are; if a group does not merge far enough, copy that operand into the canonical
        // [batch.., free.., contracting..] (lhs) / [batch.., contracting.., free..] (rhs) order and retry once
        for (int attempt = 0; attempt < 2; ++attempt) {
            Grp am = group(a, lf), ak = group(a, lc), bk = group(b, rc), bn = group(b, rf);
            Grp ab = group(a, lb), bb = group(b, rb);
            const int64_t M = extent(am), N = extent(bn), K = extent(ak), B = extent(ab);
            merge_group(&am.shape, &am.stride);
            merge_group(&bn.shape, &bn.stride);
            // contracting dims must merge identically on both sides
            {
                std::vector<int64_t> s, ta, tb;
                for (size_t i = 0; i < ak.shape.size(); ++i) {
                    if (ak.shape[i] == 1) continue;
                    if (!s.empty() && ta.back() == ak.stride[i] * ak.shape[i] && tb.back() == bk.stride[i] * bk.shape[i]) {
                        s.back() *= ak.shape[i]; ta.back() = ak.stride[i]; tb.back() = bk.stride[i];
                    } else { s.push_back(ak.shape[i]); ta.push_back(ak.stride[i]); tb.push_back(bk.stride[i]); }
                }
                ak.shape = s; ak.stride = ta; bk.shape = s; bk.stride = tb;
            }
            {
                std::vector<int64_t> s, ta, tb;
                for (size_t i = 0; i < ab.shape.size(); ++i) {
                    if (ab.shape[i] == 1) continue;
                    if (!s.empty() && ta.back() == ab.stride[i] * ab.shape[i] && tb.back() == bb.stride[i] * bb.shape[i]) {
                        s.back() *= ab.shape[i]; ta.back() = ab.stride[i]; tb.back() = bb.stride[i];
                    } else { s.push_back(ab.shape[i]); ta.push_back(ab.stride[i]); tb.push_back(bb.stride[i]); }
                }
                ab.shape = s; ab.stride = ta; bb.shape = s; bb.stride = tb;
            }
            const bool a_ok = am.shape.size() <= 1 && ak.shape.size() <= 1 && ab.shape.size() <= 2;
            const bool b_ok = bn.shape.size() <= 1 && bk.shape.size() <= 1 && bb.shape.size() <= 2;
            if (a_ok && b_ok) {
                int64_t as[4] = {0, 0, 0, 0}, bs[4] = {0, 0, 0, 0};
                int64_t b0 = 1, b1 = 1;
                if (ab.shape.size() == 2) { b0 = ab.shape[0]; b1 = ab.shape[1]; as[0] = ab.stride[0]; as[1] = ab.stride[1]; bs[0] = bb.stride[0]; bs[1] = bb.stride[1]; }
                else if (ab.shape.size() == 1) { b1 = ab.shape[0]; as[1] = ab.stride[0]; bs[1] = bb.stride[0]; }
                as[2] = am.shape.empty() ? 0 : am.stride[0];
                as[3] = ak.shape.empty() ? 0 : ak.stride[0];
                bs[2] = bk.shape.empty() ? 0 : bk.stride[0];
                bs[3] = bn.shape.empty() ? 0 : bn.stride[0];
                (void)B;
                View out = dense_view(new_arena(rt.bytes()), rt);
                DevView da = dev(a), db = dev(b), dc = dev(out);
                keep_alive(a); keep_alive(b); keep_alive(out);
                const int in_dt = static_cast<int>(a.type.dtype), out_dt = static_cast<int>(rt.dtype);
                std::array<int64_t, 4> asv = {as[0], as[1], as[2], as[3]}, bsv = {bs[0], bs[1], bs[2], bs[3]};
                GemmCase gc;
                gc.dtype = in_dt; gc.out_dtype = out_dt; gc.batch = b0 * b1; gc.m = M; gc.n = N; gc.k = K;
                gc.a_k_major = as[3] == 1 || K == 1; gc.b_k_major = bs[2] == 1 || K == 1;
                mhlo_cuda_gemm_tuning gt{0, 0, 0, 0};
                const bool tuned = lookup_gemm_tuning(gc, &gt);
                add_step(tuned ? "dot_general [tuned]" : "dot_general", [=](const Ctx& c) {
                    return mhlo_cuda_gemm_tuned(in_dt, out_dt, bind(da, c).base, asv.data(), bind(db, c).base, bsv.data(),
                                                const_cast<void*>(bind(dc, c).base), b0, b1, M, N, K, nullptr, MHLO_EPILOGUE_NONE,
                                                tuned ? &gt : nullptr, c.stream);
                });
                return set(op.results[0], out);
            }
            if (attempt == 1) fail_compile("internal: dot_general operands did not canonicalise");
            if (!a_ok) {
                std::vector<int64_t> perm = lb;
                perm.insert(perm.end(), lf.begin(), lf.end());
                perm.insert(perm.end(), lc.begin(), lc.end());
                a = permuted_copy(a, perm, "dot.lhs");
                const int nb = static_cast<int>(lb.size()), nf = static_cast<int>(lf.size()), nc = static_cast<int>(lc.size());
                lb.clear(); lf.clear(); lc.clear();
                for (int i = 0; i < nb; ++i) lb.push_back(i);
                for (int i = 0; i < nf; ++i) lf.push_back(nb + i);
                for (int i = 0; i < nc; ++i) lc.push_back(nb + nf + i);
            }
            if (!b_ok) {
                std::vector<int64_t> perm = rb;
                perm.insert(perm.end(), rc.begin(), rc.end());
                perm.insert(perm.end(), rf.begin(), rf.end());
                b = permuted_copy(b, perm, "dot.rhs");
                const int nb = static_cast<int>(rb.size()), nc = static_cast<int>(rc.size()), nf = static_cast<int>(rf.size());
                rb.clear(); rc.clear(); rf.clear();
                for (int i = 0; i < nb; ++i) rb.push_back(i);
                for (int i = 0; i < nc; ++i) rc.push_back(nb + i);
                for (int i = 0; i < nf; ++i) rf.push_back(nb + nc + i);
            }
        }
    }

    View permuted_copy(const View& v, const std::vector<int64_t>& perm, const std::string& why) {
        View p = v;
        p.type.shape.clear();
        p.strides.clear();
        for (int64_t d : perm) { p.type.shape.push_back(v.type.shape[d]); p.strides.push_back(v.strides[d]); }
        View out = dense_view(new_arena(p.type.bytes()), p.type);
        copy_view(p, out, "copy(" + why + ")");
        return out;
    }

    // stablehlo.convolution. Floating-point convolutions without batch groups become a patch matrix and one GEMM
    // (batched over feature groups) on the tensor-core path; everything else runs the direct kernel. Both read the
    // operands through their views, so no layout needs a copy.
    void lower_convolution(const Op& op) {
        if (op.operands.size() != 2) fail_compile("convolution takes two operands");
        set(op.results[0], convolution_view(op, nullptr, MHLO_EPILOGUE_NONE, nullptr));
    }

    // act(convolution(x, w) + bias), the reference's FusedConvBiasActHandler (Compiler/CustomCallHandlers.swift:563-640): the
    // call carries the convolution's attributes; bias (one value per output feature) and activation ride in the product's
    // epilogue when the convolution runs as patch matrix x kernel matrix, and follow as one elementwise step otherwise.
    void lower_fused_conv_bias_act(const Op& op, const std::string& cfg) {
        if (op.operands.size() < 2) fail_unsupported("fused_conv_bias_act takes x, the weights and an optional bias");
        const TensorType& rt = op.result_types[0];
        const bool has_bias = json_bool(cfg, "has_bias", true) && op.operands.size() >= 3;
        const std::string act = json_string(cfg, "activation", "none");
        int epi = MHLO_EPILOGUE_NONE, ew = -1;
        if (act == "relu") { epi = MHLO_EPILOGUE_RELU; ew = MHLO_EW_RELU; }
        else if (act == "sigmoid" || act == "logistic") { epi = MHLO_EPILOGUE_SIGMOID; ew = MHLO_EW_LOGISTIC; }
        else if (act == "tanh") { epi = MHLO_EPILOGUE_TANH; ew = MHLO_EW_TANH; }
        else if (act == "silu" || act == "swish") { epi = MHLO_EPILOGUE_SILU; ew = MHLO_EW_SILU; }
        else if (act != "none") fail_unsupported("fused_conv_bias_act: activation '" + act + "'");
        const int64_t ofd = op.int_attr("output_feature_dimension", rt.rank() - 1);
        View bias;
        if (has_bias) {
            bias = get(op.operands[2]);
            if (bias.type.count() != rt.shape[static_cast<size_t>(ofd)] || bias.type.dtype != rt.dtype)
                fail_unsupported("fused_conv_bias_act: bias " + bias.type.str() + " for " + rt.str());
            bias = materialize(expand_to(bias, {rt.shape[static_cast<size_t>(ofd)]}), "fused_conv_bias_act.bias");
        }
        bool fused = false;
        View y = convolution_view(op, has_bias ? &bias : nullptr, epi, &fused);
        if (fused || (!has_bias && ew < 0)) return set(op.results[0], y);
        std::vector<View> ins = {y};
        std::vector<mhlo_cuda_ew_inst> prog;
        int cur = 0;
        if (has_bias) {
            View spread = bias;  // one value per output feature, repeated along every other dimension
            spread.type.shape = rt.shape;
            spread.strides.assign(rt.shape.size(), 0);
            spread.strides[static_cast<size_t>(ofd)] = 1;
            ins.push_back(spread);
            prog.push_back({MHLO_EW_ADD, 0, 1, 0, 0.0});
            cur = 2;
        }
        if (ew >= 0) prog.push_back({ew, cur, cur, cur, 0.0});
        set(op.results[0], emit_elementwise(ins, prog, rt, "fused_conv_bias_act.epilogue"));
    }

    // The convolution as a view of its result. bias / epilogue: asked to ride in the product's epilogue; *fused says whether they did.
    View convolution_view(const Op& op, const View* bias, int epilogue, bool* fused) {
        if (fused) *fused = false;
        const View& x = get(op.operands[0]);
        const View& w = get(op.operands[1]);
        const TensorType& rt = op.result_types[0];
        const int rank = x.type.rank(), ns = rank - 2;
        if (ns < 0 || ns > MHLO_CUDA_CONV_MAX_SPATIAL || w.type.rank() != rank || rt.rank() != rank)
            fail_unsupported("convolution of rank " + std::to_string(rank));
        if (w.type.dtype != x.type.dtype || rt.dtype != x.type.dtype) fail_unsupported("convolution with mixed element types");
        auto dim = [&](const char* k) {
            const int64_t d = op.int_attr(k, -1);
            if (d < 0 || d >= rank) fail_compile(std::string("convolution: ") + k + " out of range");
            return static_cast<size_t>(d);
        };
        auto dims = [&](const char* k) {
            std::vector<int64_t> v = op.int_list(k);
            if (static_cast<int>(v.size()) != ns) fail_compile(std::string("convolution: ") + k + " must list the spatial dimensions");
            for (int64_t d : v) if (d < 0 || d >= rank) fail_compile(std::string("convolution: ") + k + " out of range");
            return v;
        };
        const size_t ib = dim("input_batch_dimension"), ifd = dim("input_feature_dimension"), ki = dim("kernel_input_feature_dimension"),
                     ko = dim("kernel_output_feature_dimension"), ob = dim("output_batch_dimension"), ofd = dim("output_feature_dimension");
        const std::vector<int64_t> isp = dims("input_spatial_dimensions"), ksp = dims("kernel_spatial_dimensions"), osp = dims("output_spatial_dimensions");
        mhlo_cuda_conv c;
        std::memset(&c, 0, sizeof c);
        c.n_spatial = ns;
        c.batch = x.type.shape[ib];
        c.in_features = x.type.shape[ifd];
        c.out_features = w.type.shape[ko];
        c.feature_group_count = op.int_attr("feature_group_count", 1);
        c.batch_group_count = op.int_attr("batch_group_count", 1);
        if (c.feature_group_count < 1 || c.batch_group_count < 1 || (c.feature_group_count > 1 && c.batch_group_count > 1))
            fail_compile("convolution: bad feature_group_count / batch_group_count");
        if (c.in_features % c.feature_group_count || c.out_features % c.feature_group_count || c.out_features % c.batch_group_count ||
            c.batch % c.batch_group_count || w.type.shape[ki] != c.in_features / c.feature_group_count)
            fail_compile("convolution: group counts do not match the feature dimensions");
        auto list = [&](const char* k, size_t want, int64_t dflt) {
            std::vector<int64_t> v = op.int_list(k);
            if (v.empty()) v.assign(want, dflt);
            if (v.size() != want) fail_compile(std::string("convolution: ") + k + " has the wrong length");
            return v;
        };
        const std::vector<int64_t> st = list("window_strides", ns, 1), pad = list("padding", 2 * ns, 0), ld = list("lhs_dilation", ns, 1),
                                   rd = list("rhs_dilation", ns, 1), rev = list("window_reversal", ns, 0);
        int64_t out_positions = 1, kernel_volume = 1;
        for (int d = 0; d < ns; ++d) {
            c.in_size[d] = x.type.shape[static_cast<size_t>(isp[d])];
            c.kernel_size[d] = w.type.shape[static_cast<size_t>(ksp[d])];
            c.out_size[d] = rt.shape[static_cast<size_t>(osp[d])];
            c.stride[d] = st[d];
            c.pad_low[d] = pad[2 * d];
            c.lhs_dilation[d] = ld[d];
            c.rhs_dilation[d] = rd[d];
            c.reverse[d] = rev[d] ? 1 : 0;
            if (st[d] < 1 || ld[d] < 1 || rd[d] < 1) fail_compile("convolution: strides and dilations must be positive");
            // the result type must agree with the window arithmetic
            const int64_t dil_in = c.in_size[d] > 0 ? (c.in_size[d] - 1) * ld[d] + 1 : 0;
            const int64_t dil_k = c.kernel_size[d] > 0 ? (c.kernel_size[d] - 1) * rd[d] + 1 : 0;
            const int64_t padded = dil_in + pad[2 * d] + pad[2 * d + 1];
            const int64_t expect = (padded < dil_k || dil_k == 0) ? 0 : (padded - dil_k) / st[d] + 1;
            if (expect != c.out_size[d]) fail_compile("convolution: result type " + rt.str() + " does not match the window (dimension " + std::to_string(d) + ")");
            c.in_spatial_stride[d] = x.strides[static_cast<size_t>(isp[d])];
            c.kernel_spatial_stride[d] = w.strides[static_cast<size_t>(ksp[d])];
            out_positions *= c.out_size[d];
            kernel_volume *= c.kernel_size[d];
        }
        c.in_batch_stride = x.strides[ib];
        c.in_feature_stride = x.strides[ifd];
        c.kernel_in_stride = w.strides[ki];
        c.kernel_out_stride = w.strides[ko];
        if (rt.shape[ob] != c.batch / c.batch_group_count || rt.shape[ofd] != c.out_features)
            fail_compile("convolution: result type " + rt.str() + " does not match the batch / feature sizes");
        const int dt = static_cast<int>(x.type.dtype);
        const int64_t G = c.feature_group_count, Og = c.out_features / G, Cg = c.in_features / G;
        const bool gemm_path = is_float(x.type.dtype) && x.type.dtype != DType::F64 && c.batch_group_count == 1 && (G == 1 || Og >= 8) &&
                               !std::getenv("METALHLO_CONV_DIRECT") && rt.count() > 0 && kernel_volume * Cg > 0;
        DevView dx = dev(x), dw = dev(w);
        keep_alive(x);
        keep_alive(w);
        if (!gemm_path) {
            View out = dense_view(new_arena(rt.bytes()), rt);
            c.out_batch_stride = out.strides[ob];
            c.out_feature_stride = out.strides[ofd];
            for (int d = 0; d < ns; ++d) c.out_spatial_stride[d] = out.strides[static_cast<size_t>(osp[d])];
            DevView dout = dev(out);
            keep_alive(out);
            add_step("convolution", [=](const Ctx& cx) {
                return mhlo_cuda_convolution(dt, bind(dx, cx).base, bind(dw, cx).base, const_cast<void*>(bind(dout, cx).base), &c, cx.stream);
            });
            return out;
        }
        // ---- two spatial dimensions, dense NHWC input and HWIO filter, window strides up to 8, one group, 16-bit tensors with channels in
        // multiples of 64: the tensor-core kernel reads the input itself (no patch matrix)
        {
            bool direct = ns == 2 && G == 1 && (x.type.dtype == DType::F16 || x.type.dtype == DType::BF16) && c.in_features % 64 == 0 &&
                          c.out_features % 8 == 0 && !std::getenv("METALHLO_CONV_PATCHES");
            for (int d = 0; d < ns && direct; ++d) direct = st[d] >= 1 && st[d] <= 8 && ld[d] == 1 && rev[d] == 0 && pad[2 * d] >= 0 && pad[2 * d + 1] >= 0;
            if (direct) {
                const int64_t H = c.in_size[0], W = c.in_size[1], C = c.in_features, O = c.out_features;
                direct = is_dense(x) && c.in_feature_stride == 1 && c.in_spatial_stride[1] == C && c.in_spatial_stride[0] == W * C &&
                         c.in_batch_stride == H * W * C && c.kernel_out_stride == 1 && c.kernel_in_stride == O &&
                         c.kernel_spatial_stride[1] == C * O && c.kernel_spatial_stride[0] == c.kernel_size[1] * C * O && is_dense(w);
            }
            if (direct) {
                TensorType canon_t;
                canon_t.dtype = rt.dtype;
                canon_t.shape = {c.batch, c.out_size[0], c.out_size[1], c.out_features};
                View canon = dense_view(new_arena(rt.bytes()), canon_t);
                DevView dcanon = dev(canon), dbias;
                keep_alive(canon);
                const bool with_bias = bias != nullptr;
                if (with_bias) { dbias = dev(*bias); keep_alive(*bias); }
                const int out_dt = static_cast<int>(rt.dtype);
                if (fused) *fused = true;
                const mhlo_cuda_conv cc = c;
                const int64_t pad_top = pad[0], pad_left = pad[2], dil_h = rd[0], dil_w = rd[1], stride_h = st[0], stride_w = st[1];
                add_step(with_bias || epilogue != MHLO_EPILOGUE_NONE ? "convolution.tensor_core+epilogue" : "convolution.tensor_core", [=](const Ctx& cx) {
                    return mhlo_cuda_conv2d_nhwc_strided(dt, out_dt, bind(dx, cx).base, bind(dw, cx).base, const_cast<void*>(bind(dcanon, cx).base), cc.batch,
                                                         cc.in_size[0], cc.in_size[1], cc.in_features, cc.kernel_size[0], cc.kernel_size[1], cc.out_features,
                                                         cc.out_size[0], cc.out_size[1], pad_top, pad_left, dil_h, dil_w, stride_h, stride_w,
                                                         with_bias ? bind(dbias, cx).base : nullptr, epilogue, cx.stream);
                });
                View out = canon;
                out.type = rt;
                out.strides.assign(static_cast<size_t>(rank), 0);
                out.strides[ob] = canon.strides[0];
                for (int d = 0; d < ns; ++d) out.strides[static_cast<size_t>(osp[d])] = canon.strides[static_cast<size_t>(d) + 1];
                out.strides[ofd] = canon.strides[3];
                return out;
            }
        }
        // ---- patch matrix + GEMM
        const int64_t M = c.batch * out_positions, Kc = kernel_volume * Cg, pitch = (Kc + 7) / 8 * 8;
        TensorType cols_t;
        cols_t.dtype = x.type.dtype;
        cols_t.shape = {G, M, pitch};
        View cols = dense_view(new_arena(cols_t.bytes()), cols_t);
        DevView dcols = dev(cols);
        keep_alive(cols);
        add_step("convolution.patches", [=](const Ctx& cx) {
            return mhlo_cuda_im2col(dt, bind(dx, cx).base, const_cast<void*>(bind(dcols, cx).base), pitch, &c, cx.stream);
        });
        // the kernel as [spatial.., input feature, output feature], then as the matrix [Kc, O]
        View wc = w;
        wc.type.shape.clear();
        wc.strides.clear();
        for (int d = 0; d < ns; ++d) { wc.type.shape.push_back(c.kernel_size[d]); wc.strides.push_back(c.kernel_spatial_stride[d]); }
        wc.type.shape.push_back(Cg);
        wc.strides.push_back(c.kernel_in_stride);
        wc.type.shape.push_back(c.out_features);
        wc.strides.push_back(c.kernel_out_stride);
        View wm = wc;
        if (!reshape_view(wc, {Kc, c.out_features}, &wm)) {
            wc = materialize(wc, "convolution.kernel");
            wm = wc;
            if (!reshape_view(wc, {Kc, c.out_features}, &wm)) fail_compile("internal: dense kernel did not reshape");
        }
        wm.type.shape = {Kc, c.out_features};
        DevView dwm = dev(wm);
        keep_alive(wm);
        TensorType prod_t;
        prod_t.dtype = rt.dtype;
        prod_t.shape = {G, M, Og};
        View prod = dense_view(new_arena(prod_t.bytes()), prod_t);
        DevView dprod = dev(prod);
        keep_alive(cols);
        keep_alive(prod);
        std::array<int64_t, 4> as = {0, M * pitch, pitch, 1}, bs = {0, Og * wm.strides[1], wm.strides[0], wm.strides[1]};
        // bias and activation in the product's epilogue: one bias vector for the whole product, so one group only
        const bool in_epilogue = G == 1 && (bias != nullptr || epilogue != MHLO_EPILOGUE_NONE);
        DevView dbias;
        if (in_epilogue && bias) { dbias = dev(*bias); keep_alive(*bias); }
        const bool with_bias = in_epilogue && bias != nullptr;
        const int epi = in_epilogue ? epilogue : MHLO_EPILOGUE_NONE;
        if (fused) *fused = in_epilogue;
        add_step(in_epilogue ? "convolution.gemm+epilogue" : "convolution.gemm", [=](const Ctx& cx) {
            return mhlo_cuda_gemm(dt, dt, bind(dcols, cx).base, as.data(), bind(dwm, cx).base, bs.data(), const_cast<void*>(bind(dprod, cx).base), 1, G,
                                  M, Og, Kc, with_bias ? bind(dbias, cx).base : nullptr, epi, cx.stream);
        });
        // [G, batch, spatial.., Og] -> canonical [batch, spatial.., O] -> the result's own dimension order
        View canon = prod;
        canon.type.shape.clear();
        canon.strides.clear();
        canon.type.shape.push_back(c.batch);
        canon.strides.push_back(out_positions * Og);
        int64_t inner = out_positions;
        for (int d = 0; d < ns; ++d) {
            inner /= std::max<int64_t>(1, c.out_size[d]);
            canon.type.shape.push_back(c.out_size[d]);
            canon.strides.push_back(inner * Og);
        }
        if (G == 1) {
            canon.type.shape.push_back(Og);
            canon.strides.push_back(1);
        } else {
            canon.type.shape.push_back(G);
            canon.strides.push_back(M * Og);
            canon.type.shape.push_back(Og);
            canon.strides.push_back(1);
            View dense = dense_view(new_arena(rt.bytes()), canon.type);
            copy_view(canon, dense, "convolution.groups");
            canon = dense;
            std::vector<int64_t> merged(canon.type.shape.begin(), canon.type.shape.end() - 2);
            merged.push_back(c.out_features);
            canon.type.shape = merged;
            canon.strides = dense_strides(merged);
        }
        View out = canon;
        out.type = rt;
        out.strides.assign(static_cast<size_t>(rank), 0);
        out.strides[ob] = canon.strides[0];
        for (int d = 0; d < ns; ++d) out.strides[static_cast<size_t>(osp[d])] = canon.strides[static_cast<size_t>(d) + 1];
        out.strides[ofd] = canon.strides[static_cast<size_t>(ns) + 1];
        return out;
    }

    // stablehlo.reduce_window of one operand with a recognised reducer; the operand is read through its view.
    void lower_reduce_window(const Op& op) {
        if (op.operands.size() != 2) fail_unsupported("variadic reduce_window");
        static const std::map<std::string, int> kinds = {{"add", MHLO_REDUCE_SUM}, {"maximum", MHLO_REDUCE_MAX}, {"minimum", MHLO_REDUCE_MIN},
                                                         {"multiply", MHLO_REDUCE_PROD}, {"and", MHLO_REDUCE_AND}, {"or", MHLO_REDUCE_OR},
                                                         {"xor", MHLO_REDUCE_XOR}};
        auto it = kinds.find(op.str_attr("reducer"));
        if (it == kinds.end()) fail_unsupported("reduce_window with a reducer body this backend does not recognise (" + op.str_attr("reducer") + ")");
        const int kind = it->second;
        const View& x = get(op.operands[0]);
        View init = materialize(get(op.operands[1]), "reduce_window.init");
        const TensorType& rt = op.result_types[0];
        const int rank = x.type.rank();
        if (rank > MHLO_CUDA_MAX_RANK) fail_unsupported("tensor rank above 8: " + x.type.str());
        mhlo_cuda_window w;
        std::memset(&w, 0, sizeof w);
        w.rank = rank;
        auto fill = [&](const char* key, int64_t* dst, int64_t dflt) {
            std::vector<int64_t> v = op.int_list(key);
            if (!v.empty() && static_cast<int>(v.size()) != rank) fail_compile(std::string("reduce_window: ") + key + " does not match the operand's rank");
            for (int d = 0; d < rank; ++d) dst[d] = v.empty() ? dflt : v[static_cast<size_t>(d)];
        };
        fill("window_dimensions", w.size, 1);
        fill("window_strides", w.stride, 1);
        fill("base_dilations", w.base_dilation, 1);
        fill("window_dilations", w.window_dilation, 1);
        std::vector<int64_t> pad = op.int_list("padding");  // [rank][2], row-major
        if (!pad.empty() && static_cast<int>(pad.size()) != 2 * rank) fail_compile("reduce_window: padding must be rank x 2");
        for (int d = 0; d < rank; ++d) w.pad_low[d] = pad.empty() ? 0 : pad[static_cast<size_t>(2 * d)];
        View out = dense_view(new_arena(rt.bytes()), rt);
        DevView dx = dev(x), di = dev(init), dout = dev(out);
        keep_alive(x); keep_alive(init); keep_alive(out);
        const std::vector<int64_t> oshape = rt.shape;
        add_step("reduce_window", [=](const Ctx& c) {
            mhlo_cuda_view xv = bind(dx, c);
            return mhlo_cuda_reduce_window(&xv, &w, kind, bind(di, c).base, const_cast<void*>(bind(dout, c).base), oshape.data(), c.stream);
        });
        set(op.results[0], out);
    }

    // stablehlo.while whose trip count is not static: the loop runs on the host. The loop-carried values live in arena
    // buffers that both regions read; each iteration launches the condition's steps, reads the predicate back (one byte,
    // one stream synchronisation), launches the body's steps and copies the body's results into the carried buffers (in
    // two phases, through temporaries, so that a result that is a view of another carried value is read before that
    // value is overwritten). Such a program is not replayed as a CUDA graph.
    void lower_while(const Op& op) {
        if (op.regions.size() != 2) fail_compile("while needs a condition and a body");
        const size_t n = op.operands.size();
        const Region& cond = *op.regions[0];
        const Region& body = *op.regions[1];
        if (cond.args.size() != n || body.args.size() != n || op.results.size() != n) fail_compile("while: region arguments do not match the operands");
        std::vector<View> state;
        for (size_t i = 0; i < n; ++i) {
            const TensorType& t = f_.type_of(op.operands[i]);
            View st = dense_view(new_arena(std::max<int64_t>(t.bytes(), 1)), t);
            copy_view(get(op.operands[i]), st, "while.init");
            state.push_back(st);
            set(cond.args[i], st);
            set(body.args[i], st);
        }
        auto lower_region = [&](const Region& r, std::vector<Executable::Step>* steps, std::vector<int>* returned) {
            std::vector<Executable::Step>* outer = sink_;
            sink_ = steps;
            bool done = false;
            for (const Op& ro : r.ops) {
                if (ro.dead) continue;
                if (ro.name == "return") { *returned = ro.operands; done = true; break; }
                lower(ro);
            }
            sink_ = outer;
            if (!done) fail_compile("while: a region does not return");
        };
        auto cond_steps = std::make_shared<std::vector<Executable::Step>>();
        auto body_steps = std::make_shared<std::vector<Executable::Step>>();
        std::vector<int> cond_ret, body_ret;
        lower_region(cond, cond_steps.get(), &cond_ret);
        if (cond_ret.size() != 1 || f_.type_of(cond_ret[0]).count() != 1) fail_compile("while: the condition must return one scalar");
        View pred;
        {
            std::vector<Executable::Step>* outer = sink_;
            sink_ = cond_steps.get();
            // the predicate as one byte in its own buffer (0 / 1), whatever view or integer type the region produced
            TensorType pt;
            pt.dtype = DType::I1;
            pred = dense_view(new_arena(256), pt);
            View src = get(cond_ret[0]);
            src.type.shape.clear();
            src.strides.clear();
            DevView ds = dev(src), dp = dev(pred);
            keep_alive(src); keep_alive(pred);
            add_step("while.predicate", [ds, dp](const Ctx& c) {
                mhlo_cuda_view sv = bind(ds, c), dv = bind(dp, c);
                mhlo_cuda_ew_inst inst = {MHLO_EW_COPY, 0, 0, 0, 0.0};
                return mhlo_cuda_elementwise_to_view(&sv, 1, &inst, 1, &dv, c.stream);
            });
            sink_ = outer;
        }
        lower_region(body, body_steps.get(), &body_ret);
        if (body_ret.size() != n) fail_compile("while: the body must return one value per operand");
        {
            std::vector<Executable::Step>* outer = sink_;
            sink_ = body_steps.get();
            std::vector<std::pair<size_t, View>> staged;
            for (size_t i = 0; i < n; ++i) {
                const View& r = get(body_ret[i]);
                if (r.buf == state[i].buf && r.offset == state[i].offset && r.strides == state[i].strides) continue;  // carried unchanged
                View tmp = dense_view(new_arena(std::max<int64_t>(state[i].type.bytes(), 1)), state[i].type);
                copy_view(r, tmp, "while.stage");
                staged.emplace_back(i, tmp);
            }
            for (const auto& st : staged) copy_view(st.second, state[st.first], "while.carry");
            sink_ = outer;
        }
        DevView dpred = dev(pred);
        for (const View& st : state) keep_alive(st);
        keep_alive(pred);
        exe_->host_control_ = true;
        const int per_iteration = static_cast<int>(cond_steps->size() + body_steps->size());
        add_step("while(" + std::to_string(per_iteration) + " steps per iteration)", [cond_steps, body_steps, dpred](const Ctx& c) -> int {
            constexpr int64_t kMaxIterations = 100000000;  // a loop that never ends is reported, not run forever
            for (int64_t it = 0; it < kMaxIterations; ++it) {
                for (const Executable::Step& s : *cond_steps)
                    if (int st = s.run(c)) return st;
                unsigned char flag = 0;
                if (int st = mhlo_cuda_download(&flag, bind(dpred, c).base, 1, c.stream)) return st;
                if (int st = mhlo_cuda_stream_sync(c.stream)) return st;
                if (!flag) return 0;
                for (const Executable::Step& s : *body_steps)
                    if (int st = s.run(c)) return st;
            }
            return static_cast<int>(MHLO_CUDA_EXECUTION_FAILED);  // more than 1e8 iterations
        }, 0);
        for (size_t i = 0; i < n; ++i) set(op.results[i], state[i]);
    }

    // stablehlo.select_and_scatter: the result is filled with the init value, then every source element is combined
    // into the position its window selects.
    void lower_select_and_scatter(const Op& op) {
        if (op.operands.size() != 3) fail_compile("select_and_scatter takes three operands");
        static const std::map<std::string, int> cmps = {{"GE", MHLO_EW_CMP_GE}, {"GT", MHLO_EW_CMP_GT}, {"LE", MHLO_EW_CMP_LE}, {"LT", MHLO_EW_CMP_LT}};
        static const std::map<std::string, int> modes = {{"add", MHLO_SCATTER_ADD}, {"multiply", MHLO_SCATTER_MUL}, {"maximum", MHLO_SCATTER_MAX},
                                                         {"minimum", MHLO_SCATTER_MIN}};
        auto ci = cmps.find(op.str_attr("select_direction"));
        auto mi = modes.find(op.str_attr("reducer"));
        if (ci == cmps.end()) fail_unsupported("select_and_scatter with a select body other than one GE / GT / LE / LT compare of its arguments");
        if (mi == modes.end()) fail_unsupported("select_and_scatter with a scatter body this backend does not recognise (" + op.str_attr("reducer") + ")");
        const int cmp = ci->second, mode = mi->second;
        const View& x = get(op.operands[0]);
        View source = materialize(get(op.operands[1]), "select_and_scatter.source");
        View init = materialize(get(op.operands[2]), "select_and_scatter.init");
        const TensorType& rt = op.result_types[0];
        const int rank = x.type.rank();
        if (rank > MHLO_CUDA_MAX_RANK || source.type.rank() != rank) fail_unsupported("select_and_scatter of rank " + std::to_string(rank));
        mhlo_cuda_window w;
        std::memset(&w, 0, sizeof w);
        w.rank = rank;
        std::vector<int64_t> size = op.int_list("window_dimensions"), stride = op.int_list("window_strides"), pad = op.int_list("padding");
        if (static_cast<int>(size.size()) != rank) fail_compile("select_and_scatter: window_dimensions does not match the operand's rank");
        if (!stride.empty() && static_cast<int>(stride.size()) != rank) fail_compile("select_and_scatter: window_strides does not match the operand's rank");
        if (!pad.empty() && static_cast<int>(pad.size()) != 2 * rank) fail_compile("select_and_scatter: padding must be rank x 2");
        for (int d = 0; d < rank; ++d) {
            w.size[d] = size[static_cast<size_t>(d)];
            w.stride[d] = stride.empty() ? 1 : stride[static_cast<size_t>(d)];
            w.base_dilation[d] = w.window_dilation[d] = 1;
            w.pad_low[d] = pad.empty() ? 0 : pad[static_cast<size_t>(2 * d)];
            const int64_t hi = pad.empty() ? 0 : pad[static_cast<size_t>(2 * d + 1)];
            const int64_t padded = x.type.shape[static_cast<size_t>(d)] + w.pad_low[d] + hi;
            const int64_t windows = padded < w.size[d] ? 0 : (padded - w.size[d]) / w.stride[d] + 1;
            if (windows != source.type.shape[static_cast<size_t>(d)]) fail_compile("select_and_scatter: source shape does not match the windows of the operand");
        }
        View out = dense_view(new_arena(rt.bytes()), rt);
        copy_view(expand_to(init, rt.shape), out, "select_and_scatter.fill");
        DevView dx = dev(x), ds = dev(source), di = dev(init), dout = dev(out);
        keep_alive(x); keep_alive(source); keep_alive(init); keep_alive(out);
        const std::vector<int64_t> sshape = source.type.shape;
        add_step("select_and_scatter", [=](const Ctx& c) {
            mhlo_cuda_view xv = bind(dx, c);
            return mhlo_cuda_select_and_scatter(&xv, bind(ds, c).base, sshape.data(), bind(di, c).base, &w, cmp, mode,
                                                const_cast<void*>(bind(dout, c).base), c.stream);
        });
        set(op.results[0], out);
    }

    // stablehlo.scatter of one operand: the operand is copied into the result, then the updates are combined in place.
    void lower_scatter(const Op& op) {
        if (op.operands.size() != 3) fail_unsupported("variadic scatter");
        static const std::map<std::string, int> modes = {{"set", MHLO_SCATTER_SET}, {"add", MHLO_SCATTER_ADD}, {"multiply", MHLO_SCATTER_MUL},
                                                         {"maximum", MHLO_SCATTER_MAX}, {"minimum", MHLO_SCATTER_MIN}};
        auto it = modes.find(op.str_attr("reducer"));
        if (it == modes.end()) fail_unsupported("scatter with an update computation this backend does not recognise (" + op.str_attr("reducer") + ")");
        const int mode = it->second;
        const TensorType& rt = op.result_types[0];
        View indices = index_view(get(op.operands[1]), "scatter.indices", true);
        View updates = materialize(get(op.operands[2]), "scatter.updates");
        View out = dense_view(new_arena(rt.bytes()), rt);
        copy_view(get(op.operands[0]), out, "scatter.operand");
        mhlo_cuda_scatter_dims g;
        std::memset(&g, 0, sizeof g);
        auto fill = [&](const char* key, int32_t* dst, int32_t* count) {
            std::vector<int64_t> v = op.int_list(key);
            if (v.size() > MHLO_CUDA_MAX_RANK) fail_unsupported(std::string("scatter: ") + key + " longer than 8");
            for (size_t i = 0; i < v.size(); ++i) dst[i] = static_cast<int32_t>(v[i]);
            if (count) *count = static_cast<int32_t>(v.size());
        };
        fill("update_window_dims", g.update_window_dims, &g.n_update_window_dims);
        fill("inserted_window_dims", g.inserted_window_dims, &g.n_inserted_window_dims);
        fill("input_batching_dims", g.input_batching_dims, &g.n_input_batching);
        fill("scatter_indices_batching_dims", g.scatter_indices_batching_dims, nullptr);
        fill("scatter_dims_to_operand_dims", g.scatter_dims_to_operand_dims, &g.n_scatter_dims_to_operand);
        g.index_vector_dim = static_cast<int32_t>(op.int_attr("index_vector_dim", indices.type.rank()));
        DevView din = dev(indices), dup = dev(updates), dout = dev(out);
        keep_alive(indices); keep_alive(updates); keep_alive(out);
        const TensorType ot = rt, it_ = indices.type, ut = updates.type;
        add_step("scatter", [=](const Ctx& c) {
            return mhlo_cuda_scatter(const_cast<void*>(bind(dout, c).base), static_cast<int>(ot.dtype), ot.shape.data(), ot.rank(), bind(din, c).base,
                                     static_cast<int>(it_.dtype), it_.shape.data(), it_.rank(), bind(dup, c).base, ut.shape.data(), ut.rank(), &g,
                                     mode, c.stream);
        });
        set(op.results[0], out);
    }

    // stablehlo.cholesky: [..., n, n] -> the lower (or upper) factor, other triangle zero.
    void lower_cholesky(const Op& op) {
        if (op.operands.size() != 1) fail_compile("cholesky takes one operand");
        View a = materialize(get(op.operands[0]), "cholesky.operand");
        const TensorType& t = a.type;
        if (t.rank() < 2 || t.shape[t.rank() - 1] != t.shape[t.rank() - 2] || !is_float(t.dtype)) fail_unsupported("cholesky of " + t.str());
        const int64_t n = t.shape[t.rank() - 1], batch = n ? t.count() / (n * n) : 0;
        const Attr* la = op.attr("lower");
        const int lower = la ? (la->kind == Attr::Bool ? la->b : la->i != 0) : 0;  // the specification's default is false
        View out = dense_view(new_arena(t.bytes()), op.result_types[0]);
        DevView da = dev(a), dout = dev(out);
        keep_alive(a); keep_alive(out);
        const int dt = static_cast<int>(t.dtype);
        add_step("cholesky", [=](const Ctx& c) {
            return mhlo_cuda_cholesky(dt, bind(da, c).base, const_cast<void*>(bind(dout, c).base), batch, n, lower, c.stream);
        });
        set(op.results[0], out);
    }

    // stablehlo.fft over the last one to three axes. Complex tensors are float tensors of (re, im) pairs by the time they
    // get here, whether the text had complex types or gave the pairs as floats the way the reference's kernels take them
    // (Sources/MetalHLOCore/Compiler/CodeGenerator.swift:2701-2830), so only element counts are checked. One launch per
    // axis: the half transform on the innermost axis first (RFFT) or last (IRFFT), the others in place.
    void lower_fft(const Op& op) {
        if (op.operands.size() != 1) fail_compile("fft takes one operand");
        std::string kind;
        for (const char* key : {"fft_type", "type"}) {
            const Attr* a = op.attr(key);
            if (!a) continue;
            std::vector<std::string> words = {a->s};
            for (const Attr& e : a->elems) words.push_back(e.s);
            for (const auto& kv : a->dict) { words.push_back(kv.first); words.push_back(kv.second.s); }
            for (const std::string& w : words) {  // "RFFT", or "fft_type RFFT" out of #stablehlo<fft_type RFFT>
                const std::string last = w.substr(w.find_last_of(' ') == std::string::npos ? 0 : w.find_last_of(' ') + 1);
                if (last == "FFT" || last == "IFFT" || last == "RFFT" || last == "IRFFT") kind = last;
            }
        }
        if (kind.empty()) fail_compile("fft without an fft_type of FFT, IFFT, RFFT or IRFFT");
        const std::vector<int64_t> len = op.int_list("fft_length");
        if (len.empty() || len.size() > 3) fail_unsupported("fft over " + std::to_string(len.size()) + " axes");
        int64_t points = 1, half_points = 1;
        for (size_t k = 0; k < len.size(); ++k) {
            if (len[k] < 1) fail_compile("fft_length entries must be positive");
            points *= len[k];
            half_points *= k + 1 == len.size() ? len[k] / 2 + 1 : len[k];
        }
        View in = materialize(get(op.operands[0]), "fft.operand");
        const TensorType& it = in.type;
        const TensorType& rt = op.result_types[0];
        if ((it.dtype != DType::F32 && it.dtype != DType::F64) || rt.dtype != it.dtype) fail_unsupported("fft from " + it.str() + " to " + rt.str());
        const bool real_in = kind == "RFFT", real_out = kind == "IRFFT";
        const int64_t in_per = real_in ? points : 2 * (real_out ? half_points : points);
        const int64_t out_per = real_out ? points : 2 * (real_in ? half_points : points);
        if (it.count() % in_per != 0 || rt.count() != it.count() / in_per * out_per)
            fail_compile("fft " + kind + " of length " + std::to_string(points) + ": " + it.str() + " -> " + rt.str() + " do not hold the same number of transforms");
        const int64_t batch = it.count() / in_per;
        View out = dense_view(new_arena(rt.bytes()), rt);
        const int dt = static_cast<int>(it.dtype);
        struct Pass { int kind; int from, to; int64_t outer, n, inner; };  // buffers: 0 operand, 1 result, 2 scratch
        std::vector<Pass> passes;
        const int r = static_cast<int>(len.size());
        auto inner_of = [&](int axis, bool halved) {
            int64_t m = 1;
            for (int k = axis + 1; k < r; ++k) m *= (halved && k == r - 1) ? len[k] / 2 + 1 : len[k];
            return m;
        };
        auto outer_of = [&](int axis) {
            int64_t m = batch;
            for (int k = 0; k < axis; ++k) m *= len[k];
            return m;
        };
        bool scratch = false;
        if (kind == "FFT" || kind == "IFFT") {
            const int k = kind == "IFFT" ? 1 : 0;
            for (int axis = r - 1; axis >= 0; --axis)
                passes.push_back({k, axis == r - 1 ? 0 : 1, 1, outer_of(axis), len[axis], inner_of(axis, false)});
        } else if (real_in) {
            passes.push_back({2, 0, 1, outer_of(r - 1), len[r - 1], 1});
            for (int axis = r - 2; axis >= 0; --axis) passes.push_back({0, 1, 1, outer_of(axis), len[axis], inner_of(axis, true)});
        } else {
            scratch = r > 1;
            for (int axis = 0; axis < r - 1; ++axis) passes.push_back({1, axis == 0 ? 0 : 2, 2, outer_of(axis), len[axis], inner_of(axis, true)});
            passes.push_back({3, scratch ? 2 : 0, 1, outer_of(r - 1), len[r - 1], 1});
        }
        View tmp;
        if (scratch) tmp = dense_view(new_arena(it.bytes()), it);
        // lines too long for the one-launch kernel's shared memory go pass by pass through two more buffers
        int64_t long_bytes = 0;
        int launches = 0;
        for (const Pass& p : passes) {
            const int64_t need = mhlo_cuda_fft_axis_scratch_bytes(dt, p.outer, p.n, p.inner);
            long_bytes = std::max(long_bytes, need);
            int stages = 0;
            while ((int64_t{1} << stages) < p.n) ++stages;
            launches += need > 0 ? stages : 1;
        }
        View lng;
        if (long_bytes > 0) {
            TensorType bytes_t;
            bytes_t.dtype = DType::UI8;
            bytes_t.shape = {long_bytes};
            lng = dense_view(new_arena(long_bytes), bytes_t);
        }
        DevView din = dev(in), dout = dev(out), dtmp, dlng;
        keep_alive(in); keep_alive(out);
        if (scratch) { dtmp = dev(tmp); keep_alive(tmp); }
        if (long_bytes > 0) { dlng = dev(lng); keep_alive(lng); }
        add_step("fft." + kind, [=](const Ctx& c) {
            const void* bufs[3] = {bind(din, c).base, bind(dout, c).base, scratch ? bind(dtmp, c).base : nullptr};
            void* lp = long_bytes > 0 ? const_cast<void*>(bind(dlng, c).base) : nullptr;
            for (const Pass& p : passes) {
                const int rc = mhlo_cuda_fft_axis_long(dt, p.kind, bufs[p.from], const_cast<void*>(bufs[p.to]), lp, p.outer, p.n, p.inner, c.stream);
                if (rc != 0) return rc;
            }
            return 0;
        }, launches);
        set(op.results[0], out);
    }

    // stablehlo.rng(a, b, shape): values between two scalars. The operator carries no state, so each one gets 16 bytes of
    // its own in the executable's constant pool: key = a hash of its position in the program, counter = 0 at load; the
    // kernel advances the counter on the device, so executions (and graph replays) continue the stream.
    void lower_rng(const Op& op) {
        if (op.operands.size() != 3) fail_compile("rng takes a, b and the shape");
        const TensorType& rt = op.result_types[0];
        View a = materialize(get(op.operands[0]), "rng.a"), b = materialize(get(op.operands[1]), "rng.b");
        if (a.type.count() != 1 || b.type.count() != 1 || a.type.dtype != rt.dtype || b.type.dtype != rt.dtype || rt.dtype == DType::I1)
            fail_unsupported("rng of " + rt.str() + " between " + a.type.str() + " and " + b.type.str());
        // `distribution = NORMAL` in the pretty form, rng_distribution = #stablehlo<rng_distribution NORMAL> in the generic one
        std::string dist;
        for (const char* key : {"rng_distribution", "distribution"}) {
            const Attr* d = op.attr(key);
            if (!d) continue;
            if (d->s == "UNIFORM" || d->s == "NORMAL") dist = d->s;
            for (const Attr& e : d->elems)
                if (e.s == "UNIFORM" || e.s == "NORMAL") dist = e.s;
            for (const auto& kv : d->dict)
                if (kv.first == "UNIFORM" || kv.first == "NORMAL" || kv.second.s == "UNIFORM" || kv.second.s == "NORMAL")
                    dist = (kv.first == "UNIFORM" || kv.first == "NORMAL") ? kv.first : kv.second.s;
            if (dist.empty()) dist = d->s.empty() ? "?" : d->s;
        }
        if (dist.empty()) dist = "UNIFORM";
        if (dist != "UNIFORM" && dist != "NORMAL") fail_unsupported("rng with distribution '" + dist + "'");
        const int normal = dist == "NORMAL";
        if (normal && !is_float(rt.dtype)) fail_unsupported("rng: a normal distribution of " + rt.str());
        Buffer sb;
        sb.kind = Buffer::Const;
        const size_t off = (exe_->const_pool_.size() + 255) / 256 * 256;
        exe_->const_pool_.resize(off + 16, 0);
        uint64_t key = 0x9E3779B97F4A7C15ull * (static_cast<uint64_t>(step_index()) + 1) ^ 0xD1B54A32D192ED03ull;
        std::memcpy(exe_->const_pool_.data() + off, &key, 8);
        sb.offset = static_cast<int64_t>(off);
        sb.bytes = 16;
        TensorType stt;
        stt.dtype = DType::UI64;
        stt.shape = {2};
        View st = dense_view(add_buffer(sb), stt);
        View out = dense_view(new_arena(rt.bytes()), rt);
        DevView da = dev(a), db = dev(b), dst = dev(st), dout = dev(out);
        keep_alive(a); keep_alive(b); keep_alive(st); keep_alive(out);
        const int dt = static_cast<int>(rt.dtype);
        const int64_t count = rt.count();
        add_step(normal ? "rng.normal" : "rng.uniform", [=](const Ctx& c) {
            return mhlo_cuda_rng(dt, normal, const_cast<void*>(bind(dst, c).base), bind(da, c).base, bind(db, c).base, const_cast<void*>(bind(dout, c).base),
                                 count, c.stream);
        }, 2);
        set(op.results[0], out);
    }

    // stablehlo.rng_bit_generator: (state) -> (new state, bits). The state is two 64-bit words {key, counter} (a third word,
    // as the Philox form carries, passes through unchanged).
    void lower_rng_bit_generator(const Op& op) {
        if (op.operands.size() != 1 || op.results.size() != 2) fail_compile("rng_bit_generator takes a state and gives the new state and the bits");
        View st = materialize(get(op.operands[0]), "rng_bit_generator.state");
        const TensorType& stt = st.type;
        const TensorType& ot = op.result_types[1];
        if (stt.dtype != DType::UI64 || stt.rank() != 1 || stt.shape[0] < 2 || stt.shape[0] > 3 || !(op.result_types[0] == stt))
            fail_unsupported("rng_bit_generator with a state of " + stt.str() + " (two or three ui64 words expected)");
        if (is_float(ot.dtype) || ot.dtype == DType::I1) fail_unsupported("rng_bit_generator of " + ot.str());
        View ns = dense_view(new_arena(stt.bytes()), stt), out = dense_view(new_arena(ot.bytes()), ot);
        DevView dst = dev(st), dns = dev(ns), dout = dev(out);
        keep_alive(st); keep_alive(ns); keep_alive(out);
        const int64_t count = ot.count(), extra_words = stt.shape[0] - 2;
        const int es = static_cast<int>(dtype_size(ot.dtype));
        add_step("rng_bit_generator", [=](const Ctx& c) {
            char* nsp = const_cast<char*>(static_cast<const char*>(bind(dns, c).base));
            if (extra_words > 0) {
                const int st2 = mhlo_cuda_copy(nsp + 16, static_cast<const char*>(bind(dst, c).base) + 16, static_cast<size_t>(8 * extra_words), c.stream);
                if (st2 != 0) return st2;
            }
            return mhlo_cuda_rng_bit_generator(bind(dst, c).base, nsp, const_cast<void*>(bind(dout, c).base), count, es, c.stream);
        }, extra_words > 0 ? 2 : 1);
        set(op.results[0], ns);
        set(op.results[1], out);
    }

    // stablehlo.triangular_solve: op(a) x = b or x op(a) = b with a [..., m, m] triangular.
    void lower_triangular_solve(const Op& op) {
        if (op.operands.size() != 2) fail_compile("triangular_solve takes two operands");
        View a = materialize(get(op.operands[0]), "triangular_solve.a"), b = materialize(get(op.operands[1]), "triangular_solve.b");
        const TensorType& at = a.type;
        const TensorType& bt = b.type;
        if (at.rank() < 2 || bt.rank() != at.rank() || at.shape[at.rank() - 1] != at.shape[at.rank() - 2] || !is_float(at.dtype) || bt.dtype != at.dtype)
            fail_unsupported("triangular_solve of " + at.str() + " and " + bt.str());
        auto flag = [&](const char* key) {
            const Attr* x = op.attr(key);
            return x ? (x->kind == Attr::Bool ? (x->b ? 1 : 0) : (x->i != 0 ? 1 : 0)) : 0;
        };
        const int left_side = flag("left_side"), lower = flag("lower"), unit = flag("unit_diagonal");
        std::string tr = op.str_attr("transpose_a", "NO_TRANSPOSE");
        if (const Attr* ta = op.attr("transpose_a"))  // #stablehlo<transpose TRANSPOSE> arrives as a dictionary or keyword list
            if (tr.empty() || tr == "NO_TRANSPOSE")
                for (const Attr& e : ta->elems)
                    if (e.kind == Attr::Keyword || e.kind == Attr::String) tr = e.s;
        int transpose = 0;
        if (tr.find("NO_TRANSPOSE") != std::string::npos) transpose = 0;
        else if (tr.find("TRANSPOSE") != std::string::npos || tr.find("ADJOINT") != std::string::npos) transpose = 1;  // real types: the adjoint is the transpose
        else fail_unsupported("triangular_solve: transpose_a = " + tr);
        const int64_t m = at.shape[at.rank() - 1];
        const int64_t n = left_side ? bt.shape[bt.rank() - 1] : bt.shape[bt.rank() - 2];
        if ((left_side ? bt.shape[bt.rank() - 2] : bt.shape[bt.rank() - 1]) != m) fail_compile("triangular_solve: the shapes of a and b do not agree");
        const int64_t batch = m ? at.count() / (m * m) : 0;
        if (batch * m * n != bt.count()) fail_compile("triangular_solve: batch dimensions of a and b differ");
        View out = dense_view(new_arena(bt.bytes()), op.result_types[0]);
        DevView da = dev(a), db = dev(b), dout = dev(out);
        keep_alive(a); keep_alive(b); keep_alive(out);
        const int dt = static_cast<int>(at.dtype);
        add_step("triangular_solve", [=](const Ctx& c) {
            return mhlo_cuda_triangular_solve(dt, bind(da, c).base, bind(db, c).base, const_cast<void*>(bind(dout, c).base), batch, m, n, left_side, lower,
                                              unit, transpose, c.stream);
        });
        set(op.results[0], out);
    }

    // stablehlo.sort: every operand permuted by the order of the first one along `dimension`.
    void lower_sort(const Op& op) {
        const size_t n = op.operands.size();
        if (n < 1 || n > MHLO_CUDA_SORT_MAX_OPERANDS || op.results.size() != n) fail_unsupported("sort of " + std::to_string(n) + " operands");
        const std::string order = op.str_attr("sort_order");
        if (order != "ascending" && order != "descending")
            fail_unsupported("sort with a comparator other than one LT / GT compare of the first operand");
        std::vector<View> ins, outs;
        for (size_t j = 0; j < n; ++j) {
            ins.push_back(materialize(get(op.operands[j]), "sort.operand"));
            if (ins[j].type.shape != ins[0].type.shape) fail_compile("sort: operands of different shapes");
            outs.push_back(dense_view(new_arena(op.result_types[j].bytes()), op.result_types[j]));
        }
        const TensorType kt = ins[0].type;
        int64_t dim = op.int_attr("dimension", -1);
        if (dim < 0) dim += kt.rank();
        if (kt.rank() < 1 || dim < 0 || dim >= kt.rank()) fail_compile("sort: dimension out of range");
        const int64_t scratch_bytes = mhlo_cuda_sort_scratch_bytes(kt.shape.data(), kt.rank(), static_cast<int32_t>(dim));
        if (scratch_bytes < 0) fail_compile("sort: bad shape");
        View scratch;
        const bool has_scratch = scratch_bytes > 0;
        if (has_scratch) {
            TensorType st;
            st.dtype = DType::UI8;
            st.shape = {scratch_bytes};
            scratch = dense_view(new_arena(scratch_bytes), st);
        }
        std::vector<DevView> din, dout;
        std::vector<int32_t> dts;
        for (size_t j = 0; j < n; ++j) {
            din.push_back(dev(ins[j]));
            dout.push_back(dev(outs[j]));
            dts.push_back(static_cast<int32_t>(ins[j].type.dtype));
            keep_alive(ins[j]);
            keep_alive(outs[j]);
        }
        DevView dscratch;
        if (has_scratch) { dscratch = dev(scratch); keep_alive(scratch); }
        const int descending = (order == "descending" ? 1 : 0) | (op.str_attr("sort_compare_type") == "FLOAT" ? 2 : 0);
        int launches = 1;
        if (has_scratch) {  // keys, chunk sort, then per merge size its global stages and one chunk merge, apply
            int64_t padded = 1;
            while (padded < kt.shape[static_cast<size_t>(dim)]) padded <<= 1;
            launches = 3;
            for (int64_t k = 2 * MHLO_CUDA_SORT_SMEM_MAX; k <= padded; k <<= 1) {
                for (int64_t j = k >> 1; j >= MHLO_CUDA_SORT_SMEM_MAX; j >>= 1) ++launches;
                ++launches;
            }
        }
        add_step("sort", [=](const Ctx& c) {
            const void* in[MHLO_CUDA_SORT_MAX_OPERANDS];
            void* out[MHLO_CUDA_SORT_MAX_OPERANDS];
            for (size_t j = 0; j < din.size(); ++j) { in[j] = bind(din[j], c).base; out[j] = const_cast<void*>(bind(dout[j], c).base); }
            void* sc = has_scratch ? const_cast<void*>(bind(dscratch, c).base) : nullptr;
            return mhlo_cuda_sort(in, out, dts.data(), static_cast<int32_t>(din.size()), kt.shape.data(), kt.rank(), static_cast<int32_t>(dim),
                                  descending, sc, scratch_bytes, c.stream);
        }, launches);
        for (size_t j = 0; j < n; ++j) set(op.results[j], outs[j]);
    }

    void lower_gather(const Op& op) {
        View operand = materialize(get(op.operands[0]), "gather.operand");
        View indices = index_view(get(op.operands[1]), "gather.indices", true);
        const TensorType& rt = op.result_types[0];
        mhlo_cuda_gather_dims g;
        std::memset(&g, 0, sizeof g);
        auto fill = [&](const char* key, int32_t* dst, int32_t* count) {
            std::vector<int64_t> v = op.int_list(key);
            if (v.size() > MHLO_CUDA_MAX_RANK) fail_unsupported(std::string("gather: ") + key + " longer than 8");
            for (size_t i = 0; i < v.size(); ++i) dst[i] = static_cast<int32_t>(v[i]);
            if (count) *count = static_cast<int32_t>(v.size());
        };
        fill("offset_dims", g.offset_dims, &g.n_offset_dims);
        fill("collapsed_slice_dims", g.collapsed_slice_dims, &g.n_collapsed);
        fill("operand_batching_dims", g.operand_batching_dims, &g.n_operand_batching);
        fill("start_indices_batching_dims", g.start_indices_batching_dims, nullptr);
        fill("start_index_map", g.start_index_map, &g.n_start_index_map);
        g.index_vector_dim = static_cast<int32_t>(op.int_attr("index_vector_dim", indices.type.rank()));
        std::vector<int64_t> ss = op.int_list("slice_sizes");
        if (static_cast<int>(ss.size()) != operand.type.rank()) fail_compile("gather: slice_sizes rank mismatch");
        for (size_t i = 0; i < ss.size(); ++i) g.slice_sizes[i] = ss[i];
        View out = dense_view(new_arena(rt.bytes()), rt);
        DevView dop = dev(operand), din = dev(indices), dout = dev(out);
        keep_alive(operand); keep_alive(indices); keep_alive(out);
        const TensorType ot = operand.type, it = indices.type, rtt = rt;
        add_step("gather", [=](const Ctx& c) {
            return mhlo_cuda_gather(bind(dop, c).base, static_cast<int>(dtype_size(ot.dtype)), ot.shape.data(), ot.rank(),
                                    bind(din, c).base, static_cast<int>(it.dtype), it.shape.data(), it.rank(), &g,
                                    const_cast<void*>(bind(dout, c).base), rtt.shape.data(), rtt.rank(), c.stream);
        });
        set(op.results[0], out);
    }

    // Index operands in the types the index kernels read (i32, i64; ui32 too where `ui32_ok`): any other integer type is
    // widened to i64 by one small elementwise launch first (a ui64 index of 2^63 or more would wrap: no tensor is that long).
    View index_view(const View& v, const std::string& why, bool ui32_ok) {
        const DType d = v.type.dtype;
        if (d == DType::I32 || d == DType::I64 || (ui32_ok && d == DType::UI32)) return materialize(v, why);
        if (is_float(d)) fail_compile(why + " must be an integer tensor, not " + v.type.str());
        TensorType wide = v.type;
        wide.dtype = DType::I64;
        mhlo_cuda_ew_inst widen = {MHLO_EW_COPY, 0, 0, 0, 0.0};
        return emit_elementwise({v}, {widen}, wide, "convert(" + why + ")");
    }

    void lower_dynamic_slice(const Op& op) {
        View operand = materialize(get(op.operands[0]), "dynamic_slice.operand");
        const TensorType& rt = op.result_types[0];
        std::vector<DevView> idx;
        DType idt = DType::I32;
        for (size_t i = 1; i < op.operands.size(); ++i) {
            View iv = index_view(get(op.operands[i]), "dynamic_slice.index", false);
            idt = iv.type.dtype;
            idx.push_back(dev(iv));
            keep_alive(iv);
        }
        if (static_cast<int>(idx.size()) != operand.type.rank()) fail_compile("dynamic_slice: one start index per dimension expected");
        View out = dense_view(new_arena(rt.bytes()), rt);
        DevView dop = dev(operand), dout = dev(out);
        keep_alive(operand); keep_alive(out);
        const TensorType ot = operand.type, rtt = rt;
        const int index_dtype = static_cast<int>(idt);
        add_step("dynamic_slice", [=](const Ctx& c) {
            const void* ptrs[MHLO_CUDA_MAX_RANK];
            for (size_t i = 0; i < idx.size(); ++i) ptrs[i] = bind(idx[i], c).base;
            return mhlo_cuda_dynamic_slice(bind(dop, c).base, static_cast<int>(dtype_size(ot.dtype)), ot.shape.data(), ot.rank(),
                                           ptrs, index_dtype, rtt.shape.data(), const_cast<void*>(bind(dout, c).base), c.stream);
        });
        set(op.results[0], out);
    }

    void lower_dynamic_update_slice(const Op& op) {
        const View& operand = get(op.operands[0]);
        View update = materialize(get(op.operands[1]), "dynamic_update_slice.update");
        const TensorType& rt = op.result_types[0];
        View out = dense_view(new_arena(rt.bytes()), rt);
        copy_view(operand, out, "dynamic_update_slice.copy");
        std::vector<DevView> idx;
        DType idt = DType::I32;
        for (size_t i = 2; i < op.operands.size(); ++i) {
            View iv = index_view(get(op.operands[i]), "dynamic_update_slice.index", false);
            idt = iv.type.dtype;
            idx.push_back(dev(iv));
            keep_alive(iv);
        }
        DevView dup = dev(update), dout = dev(out);
        keep_alive(update); keep_alive(out);
        const TensorType ut = update.type, rtt = rt;
        const int index_dtype = static_cast<int>(idt);
        add_step("dynamic_update_slice", [=](const Ctx& c) {
            const void* ptrs[MHLO_CUDA_MAX_RANK];
            for (size_t i = 0; i < idx.size(); ++i) ptrs[i] = bind(idx[i], c).base;
            return mhlo_cuda_dynamic_update_slice(const_cast<void*>(bind(dout, c).base), static_cast<int>(dtype_size(rtt.dtype)),
                                                  rtt.shape.data(), rtt.rank(), bind(dup, c).base, ut.shape.data(), ptrs,
                                                  index_dtype, c.stream);
        });
        set(op.results[0], out);
    }

    void lower_custom_call(const Op& op);
    void lower_return(const Op& op);
    void plan();
};

// ---- fused custom calls ------------------------------------------------------------------------------------------------

void Lowering::lower_custom_call(const Op& op) {
    const std::string target = op.str_attr("call_target_name");
    const std::string cfg = op.str_attr("backend_config");
    const TensorType& rt = op.result_types[0];
    auto operand = [&](size_t i) -> const View& {
        if (i >= op.operands.size()) fail_compile("custom_call @" + target + " needs at least " + std::to_string(i + 1) + " operands");
        return get(op.operands[i]);
    };
    auto last_axis_only = [&](const std::vector<int64_t>& axes, int rank) {
        return axes.empty() || (axes.size() == 1 && (axes[0] == -1 || axes[0] == rank - 1));
    };
    if (target == "fused_layer_norm" || target == "fused_rms_norm") {
        const bool ln = target == "fused_layer_norm";
        View x = materialize(operand(0), target);
        if (!last_axis_only(json_int_array(cfg, "axes"), x.type.rank())) fail_unsupported(target + " over an axis other than the last");
        const int64_t hidden = x.type.rank() ? x.type.shape.back() : 1;
        const int64_t rows = hidden ? x.type.count() / hidden : 0;
        bool has_g = op.operands.size() > 1, has_b = ln && op.operands.size() > 2;
        View g, b;
        if (has_g) g = materialize(expand_to(operand(1), {hidden}), target + ".gamma");
        if (has_b) b = materialize(expand_to(operand(2), {hidden}), target + ".beta");
        if (has_g && !is_dense(g)) g = materialize(g, "gamma");
        const float eps = static_cast<float>(json_number(cfg, "eps", json_number(cfg, "epsilon", 1e-5)));
        View out = dense_view(new_arena(rt.bytes()), rt);
        DevView dx = dev(x), dg, db, dout = dev(out);
        keep_alive(x); keep_alive(out);
        if (has_g) { dg = dev(g); keep_alive(g); }
        if (has_b) { db = dev(b); keep_alive(b); }
        const int dt = static_cast<int>(x.type.dtype);
        mhlo_cuda_row_tuning tuning{0, 0, 0};
        const bool tuned = lookup_row_tuning(target, rows, hidden, x.type.dtype, &tuning);
        add_step(tuned ? target + " [tuned]" : target, [=](const Ctx& c) {
            const void* gp = has_g ? bind(dg, c).base : nullptr;
            const void* bp = has_b ? bind(db, c).base : nullptr;
            const mhlo_cuda_row_tuning* tp = tuned ? &tuning : nullptr;
            if (ln) return mhlo_cuda_layer_norm(dt, bind(dx, c).base, gp, bp, const_cast<void*>(bind(dout, c).base), rows, hidden, eps, tp, c.stream);
            return mhlo_cuda_rms_norm(dt, bind(dx, c).base, gp, const_cast<void*>(bind(dout, c).base), rows, hidden, eps, tp, c.stream);
        });
        return set(op.results[0], out);
    }
    if (target == "fused_add_layer_norm" || target == "fused_add_rms_norm") {
        // results: [0] the sum a + b (the residual stream), [1] its norm
        const bool ln = target == "fused_add_layer_norm";
        if (op.results.size() != 2) fail_compile(target + " must have two results");
        View addend_block;
        int64_t addend_rows = 0;  // > 0: one addend is a block of that many rows repeated down the other
        int dense_side = -1;
        for (int side = 0; side < 2 && dense_side < 0; ++side)
            if (is_dense(operand(side)) && !is_dense(operand(1 - side)) && repeated_rows(operand(1 - side), &addend_block, &addend_rows))
                dense_side = side;
        if (dense_side < 0) addend_rows = 0;
        if (dense_side < 0 && (!is_dense(operand(0)) || !is_dense(operand(1)))) {
            // a broadcast or transposed addend would have to be copied first: the strided elementwise add reads it in
            // place, and the norm then runs on its result
            mhlo_cuda_ew_inst add_inst = {ew_opcode("add"), 0, 1, 0, 0.0};
            View sum = emit_elementwise({operand(0), operand(1)}, {add_inst}, op.result_types[0], "add");
            set(op.results[0], sum);
            Op plain = op;
            plain.operands[0] = op.results[0];
            plain.operands.erase(plain.operands.begin() + 1);
            plain.results = {op.results[1]};
            plain.result_types = {op.result_types[1]};
            plain.attrs["call_target_name"] = Attr::make_string(ln ? "fused_layer_norm" : "fused_rms_norm");
            return lower_custom_call(plain);
        }
        View a = materialize(operand(dense_side == 1 ? 1 : 0), target + ".a");
        View r = dense_side >= 0 ? materialize(addend_block, target + ".b") : materialize(operand(1), target + ".b");
        if (!last_axis_only(json_int_array(cfg, "axes"), a.type.rank())) fail_unsupported(target + " over an axis other than the last");
        const int64_t hidden = a.type.rank() ? a.type.shape.back() : 1;
        const int64_t rows = hidden ? a.type.count() / hidden : 0;
        const bool has_g = op.operands.size() > 2, has_b = ln && op.operands.size() > 3;
        View g, b;
        if (has_g) g = materialize(expand_to(operand(2), {hidden}), target + ".gamma");
        if (has_b) b = materialize(expand_to(operand(3), {hidden}), target + ".beta");
        const float eps = static_cast<float>(json_number(cfg, "eps", json_number(cfg, "epsilon", 1e-5)));
        const TensorType& st = op.result_types[0];
        const TensorType& yt = op.result_types[1];
        View sum = dense_view(new_arena(st.bytes()), st), out = dense_view(new_arena(yt.bytes()), yt);
        DevView da = dev(a), dr = dev(r), dg, db, dsum = dev(sum), dout = dev(out);
        keep_alive(a); keep_alive(r); keep_alive(sum); keep_alive(out);
        if (has_g) { dg = dev(g); keep_alive(g); }
        if (has_b) { db = dev(b); keep_alive(b); }
        const int dt = static_cast<int>(a.type.dtype);
        mhlo_cuda_row_tuning tuning{0, 0, 0};
        const bool tuned = lookup_row_tuning(ln ? "fused_layer_norm" : "fused_rms_norm", rows, hidden, a.type.dtype, &tuning);
        add_step(addend_rows > 0 ? target + " [repeated addend]" : target, [=](const Ctx& c) {
            const void* gp = has_g ? bind(dg, c).base : nullptr;
            const void* bp = has_b ? bind(db, c).base : nullptr;
            const mhlo_cuda_row_tuning* tp = tuned ? &tuning : nullptr;
            void* sp = const_cast<void*>(bind(dsum, c).base);
            void* yp = const_cast<void*>(bind(dout, c).base);
            if (addend_rows > 0) {
                if (ln) return mhlo_cuda_add_layer_norm_rows(dt, bind(da, c).base, bind(dr, c).base, addend_rows, gp, bp, sp, yp, rows, hidden, eps, tp, c.stream);
                return mhlo_cuda_add_rms_norm_rows(dt, bind(da, c).base, bind(dr, c).base, addend_rows, gp, sp, yp, rows, hidden, eps, tp, c.stream);
            }
            if (ln) return mhlo_cuda_add_layer_norm(dt, bind(da, c).base, bind(dr, c).base, gp, bp, sp, yp, rows, hidden, eps, tp, c.stream);
            return mhlo_cuda_add_rms_norm(dt, bind(da, c).base, bind(dr, c).base, gp, sp, yp, rows, hidden, eps, tp, c.stream);
        });
        set(op.results[0], sum);
        return set(op.results[1], out);
    }
    if (target == "fused_softmax") {
        View x = materialize(operand(0), target);
        int64_t axis = static_cast<int64_t>(json_number(cfg, "axis", -1));
        if (axis < 0) axis += x.type.rank();
        if (axis < 0 || axis >= std::max(1, x.type.rank())) fail_compile("fused_softmax: axis out of range");
        int64_t outer = 1, inner = 1;
        for (int d = 0; d < axis; ++d) outer *= x.type.shape[d];
        for (int d = static_cast<int>(axis) + 1; d < x.type.rank(); ++d) inner *= x.type.shape[d];
        const int64_t len = x.type.rank() ? x.type.shape[axis] : 1;
        View out = dense_view(new_arena(rt.bytes()), rt);
        DevView dx = dev(x), dout = dev(out);
        keep_alive(x); keep_alive(out);
        const int dt = static_cast<int>(x.type.dtype);
        mhlo_cuda_row_tuning tuning{0, 0, 0};
        const bool tuned = inner == 1 && lookup_row_tuning(target, outer, len, x.type.dtype, &tuning);
        add_step(tuned ? target + " [tuned]" : target, [=](const Ctx& c) {
            return mhlo_cuda_softmax(dt, bind(dx, c).base, const_cast<void*>(bind(dout, c).base), outer, len, inner, tuned ? &tuning : nullptr, c.stream);
        });
        return set(op.results[0], out);
    }
    if (target == "fused_gelu" || target == "fused_silu" || target == "fused_relu") {
        int code = MHLO_EW_RELU;
        if (target == "fused_gelu") code = json_bool(cfg, "approximate", true) ? MHLO_EW_GELU_TANH : MHLO_EW_GELU_ERF;
        if (target == "fused_silu") code = MHLO_EW_SILU;
        mhlo_cuda_ew_inst inst = {code, 0, 0, 0, 0.0};
        return set(op.results[0], emit_elementwise({operand(0)}, {inst}, rt, target));
    }
    if (target == "fused_elementwise") {
        // program: attribute "_program" = array of [opcode, a, b, c, imm] built by producer-consumer fusion
        const Attr* pa = op.attr("_program");
        if (!pa || pa->kind != Attr::Array) fail_unsupported("fused_elementwise without a program attribute");
        std::vector<mhlo_cuda_ew_inst> prog;
        for (const Attr& e : pa->elems) {
            if (e.elems.size() != 5) fail_compile("fused_elementwise: malformed instruction");
            mhlo_cuda_ew_inst inst;
            inst.op = static_cast<int>(e.elems[0].i);
            inst.a = static_cast<int>(e.elems[1].i);
            inst.b = static_cast<int>(e.elems[2].i);
            inst.c = static_cast<int>(e.elems[3].i);
            inst.imm = e.elems[4].as_float();
            prog.push_back(inst);
        }
        std::vector<View> ins;
        for (int v : op.operands) ins.push_back(get(v));
        return set(op.results[0], emit_elementwise(ins, prog, rt, target));
    }
    if (target == "fused_conv_bias_act") return lower_fused_conv_bias_act(op, cfg);
    if (target == "fused_matmul_bias_activation") {
        // act(x . w + bias): x [.., M, K] (leading dims flattened), w [K, N], bias [N] (optional)
        View x = materialize(operand(0), target + ".x"), w = operand(1);
        if (w.type.rank() != 2) fail_unsupported(target + ": weight must be rank 2");
        const int64_t K = w.type.shape[0], N = w.type.shape[1];
        const int64_t M = K ? x.type.count() / K : 0;
        const bool has_residual = json_bool(cfg, "has_residual", false);  // the last operand: a tensor of the result's type added to the product
        const bool has_bias = json_bool(cfg, "has_bias", op.operands.size() > (has_residual ? 3u : 2u));
        if (op.operands.size() != 2u + (has_bias ? 1u : 0u) + (has_residual ? 1u : 0u)) fail_unsupported(target + ": operand count does not match has_bias / has_residual");
        View bias, residual;
        if (has_bias) bias = materialize(expand_to(operand(2), {N}), target + ".bias");
        if (has_residual) {
            residual = operand(static_cast<int>(op.operands.size()) - 1);
            if (!(residual.type == rt)) fail_unsupported(target + ": the residual must have the result's type");
            if (!is_dense(residual)) residual = materialize(residual, target + ".residual");
        }
        const std::string act = json_string(cfg, "activation", "none");
        int epi = MHLO_EPILOGUE_NONE;
        if (act == "gelu" || act == "gelu_tanh") epi = MHLO_EPILOGUE_GELU_TANH;
        else if (act == "gelu_erf") epi = MHLO_EPILOGUE_GELU_ERF;
        else if (act == "relu") epi = MHLO_EPILOGUE_RELU;
        else if (act == "silu") epi = MHLO_EPILOGUE_SILU;
        else if (act == "tanh") epi = MHLO_EPILOGUE_TANH;
        else if (act == "sigmoid" || act == "logistic") epi = MHLO_EPILOGUE_SIGMOID;
        else if (act != "none") fail_unsupported(target + ": activation '" + act + "'");
        if (has_residual && epi != MHLO_EPILOGUE_NONE) fail_unsupported(target + ": a residual goes with activation 'none'");
        View out = dense_view(new_arena(rt.bytes()), rt);
        DevView dx = dev(x), dw = dev(w), dbias, dres, dout = dev(out);
        keep_alive(x); keep_alive(w); keep_alive(out);
        if (has_bias) { dbias = dev(bias); keep_alive(bias); }
        if (has_residual) { dres = dev(residual); keep_alive(residual); }
        const int in_dt = static_cast<int>(x.type.dtype), out_dt = static_cast<int>(rt.dtype);
        std::array<int64_t, 4> as = {0, 0, K, 1}, bs = {0, 0, w.strides[0], w.strides[1]};
        GemmCase gc;
        gc.dtype = in_dt; gc.out_dtype = out_dt; gc.batch = 1; gc.m = M; gc.n = N; gc.k = K;
        gc.a_k_major = true; gc.b_k_major = w.strides[0] == 1 || K == 1;
        mhlo_cuda_gemm_tuning gt{0, 0, 0, 0};
        const bool tuned = lookup_gemm_tuning(gc, &gt);
        add_step(tuned ? target + " [tuned]" : target, [=](const Ctx& c) {
            if (has_residual)
                return mhlo_cuda_gemm_residual(in_dt, out_dt, bind(dx, c).base, as.data(), bind(dw, c).base, bs.data(),
                                               const_cast<void*>(bind(dout, c).base), 1, 1, M, N, K, has_bias ? bind(dbias, c).base : nullptr,
                                               bind(dres, c).base, tuned ? &gt : nullptr, c.stream);
            return mhlo_cuda_gemm_tuned(in_dt, out_dt, bind(dx, c).base, as.data(), bind(dw, c).base, bs.data(),
                                        const_cast<void*>(bind(dout, c).base), 1, 1, M, N, K, has_bias ? bind(dbias, c).base : nullptr,
                                        epi, tuned ? &gt : nullptr, c.stream);
        });
        return set(op.results[0], out);
    }
    if (target == "fused_scaled_dot_product_attention") {
        // q [B,H,Sq,D], k/v [B,H,Sk,D] in logical order; the views may be permutations of other layouts as long as D
        // is contiguous. Output dense [B,H,Sq,D] unless "output_layout":"BSHD" asks for [B,Sq,H,D].
        View q = operand(0), k = operand(1), v = operand(2);
        if (q.type.rank() == 3) {  // [BH,S,D] -> [1,BH,S,D]
            for (View* t : {&q, &k, &v}) { t->type.shape.insert(t->type.shape.begin(), 1); t->strides.insert(t->strides.begin(), 0); }
        }
        if (q.type.rank() != 4) fail_unsupported(target + ": rank-3 or rank-4 operands expected, got " + q.type.str());
        for (View* t : {&q, &k, &v})
            if (t->strides[3] != 1 && t->type.shape[3] != 1) *t = materialize(*t, target + ".operand");
        const bool has_mask = json_bool(cfg, "has_mask", false) && op.operands.size() > 3;
        View mask;
        if (has_mask) {
            const int64_t sq = q.type.shape[2], sk = k.type.shape[2];
            mask = operand(3);
            if (mask.type.count() != sq * sk) fail_unsupported(target + ": only a [Sq,Sk] additive mask shared by all heads is supported");
            View m2 = mask;
            if (!reshape_view(mask, {sq, sk}, &m2)) { m2 = materialize(mask, "mask"); m2.strides = {sk, 1}; }
            m2.type.shape = {sq, sk};
            mask = materialize(m2, target + ".mask");
        }
        const float scale = static_cast<float>(json_number(cfg, "scale", 1.0));
        const bool causal = json_bool(cfg, "is_causal", false);
        const bool bshd_out = json_string(cfg, "output_layout", "BHSD") == "BSHD";
        View out = dense_view(new_arena(rt.bytes()), rt);
        DevView dq = dev(q), dk = dev(k), dv = dev(v), dm, dout = dev(out);
        keep_alive(q); keep_alive(k); keep_alive(v); keep_alive(out);
        if (has_mask) { dm = dev(mask); keep_alive(mask); }
        const int dt = static_cast<int>(q.type.dtype);
        const int64_t B = q.type.shape[0], H = q.type.shape[1], Sq = q.type.shape[2], D = q.type.shape[3], Sk = k.type.shape[2];
        std::array<int64_t, 3> qs = {q.strides[0], q.strides[1], q.strides[2]}, ks = {k.strides[0], k.strides[1], k.strides[2]},
                               vs = {v.strides[0], v.strides[1], v.strides[2]};
        std::array<int64_t, 3> os = bshd_out ? std::array<int64_t, 3>{Sq * H * D, D, H * D} : std::array<int64_t, 3>{H * Sq * D, Sq * D, D};
        AttentionCase ac;
        ac.dtype = dt; ac.batch = B; ac.heads = H; ac.seq_q = Sq; ac.seq_k = Sk; ac.head_dim = D; ac.causal = causal;
        ac.bshd = H > 1 && q.strides[1] == D;  // heads interleaved inside a token: the [batch, sequence, head, dim] layout
        mhlo_cuda_attention_tuning at{0, {0, 0, 0}};
        const bool tuned = !has_mask && lookup_attention_tuning(ac, &at);
        add_step(tuned ? target + " [tuned]" : target, [=](const Ctx& c) {
            return mhlo_cuda_attention_tuned(dt, bind(dq, c).base, qs.data(), bind(dk, c).base, ks.data(), bind(dv, c).base, vs.data(),
                                             has_mask ? bind(dm, c).base : nullptr, const_cast<void*>(bind(dout, c).base), os.data(), B, H, Sq,
                                             Sk, D, scale, causal ? 1 : 0, tuned ? &at : nullptr, c.stream);
        });
        return set(op.results[0], out);
    }
    fail_unsupported("custom_call target @" + target + " is not provided by this backend");
}

void Lowering::lower_return(const Op& op) {
    std::set<int> claimed;
    for (size_t i = 0; i < op.operands.size(); ++i) {
        const View& v = get(op.operands[i]);
        exe_->output_types_.push_back(v.type);
        exe_->output_types_.back().was_complex = i < f_.result_complex.size() && f_.result_complex[i];
        Buffer& b = buffers_[v.buf];
        const bool whole = b.kind == Buffer::Arena && v.offset == 0 && is_dense(v) && b.bytes == v.type.bytes() &&
                           !claimed.count(v.buf) && v.type.count() > 0;
        bool zero_stride = false;
        for (size_t d = 0; d < v.strides.size(); ++d) zero_stride |= v.strides[d] == 0 && v.type.shape[d] > 1;
        if (whole && !zero_stride) {
            // the producing kernel writes straight into the caller's output buffer
            b.kind = Buffer::Output;
            b.index = static_cast<int>(i);
            claimed.insert(v.buf);
            continue;
        }
        Buffer ob;
        ob.kind = Buffer::Output;
        ob.index = static_cast<int>(i);
        ob.bytes = v.type.bytes();
        View dst = dense_view(add_buffer(ob), v.type);
        if (v.type.count() > 0) copy_view(v, dst, "copy(output)");
    }
}

void Lowering::plan() {
    std::vector<PlanInterval> ivs;
    std::vector<int> ids;
    for (size_t i = 0; i < buffers_.size(); ++i) {
        if (buffers_[i].kind != Buffer::Arena) continue;
        PlanInterval p;
        p.bytes = buffers_[i].bytes;
        p.first = std::max(0, buffers_[i].first);
        p.last = std::max(p.first, buffers_[i].last);
        ivs.push_back(p);
        ids.push_back(static_cast<int>(i));
    }
    const bool no_reuse = std::getenv("METALHLO_NO_REUSE") || std::getenv("METALHLO_DEBUG_NO_BUFFER_REUSE");
    if (no_reuse)
        for (PlanInterval& p : ivs) { p.first = 0; p.last = step_index(); }
    exe_->arena_bytes_ = plan_memory(&ivs);
    exe_->plan_intervals_ = ivs;
    for (size_t k = 0; k < ids.size(); ++k) buffers_[ids[k]].offset = ivs[k].offset;
    *table_ = buffers_;
}

// ---- Executable --------------------------------------------------------------------------------------------------------

Executable::~Executable() {
    for (GraphSlot& g : graph_slots_)
        if (g.graph) mhlo_cuda_graph_destroy(g.graph);
    if (const_dev_) mhlo_cuda_free(const_dev_);
    if (arena_dev_) mhlo_cuda_free(arena_dev_);
}

std::unique_ptr<Executable> Executable::plan_only(const std::string& mlir, const CompileOptions& options) {
    Module m = parse_module(mlir);
    Function f = flatten_main(m);
    std::unique_ptr<Executable> exe(new Executable());
    exe->shard_plan_ = shard_function(f, options.shard);
    exe->pass_log_ = run_pass_pipeline(f, options);
    optimize_loop_bodies(f, options);
    exe->optimized_text_ = print_function(f);
    Lowering lower(f, exe.get());
    lower.run();
    return exe;
}

std::unique_ptr<Executable> Executable::compile(const std::string& mlir, const CompileOptions& options) {
    Module m = parse_module(mlir);
    Function f = flatten_main(m);
    if (std::getenv("METALHLO_DUMP_MLIR")) fprintf(stderr, "[metalhlo] parsed module:\n%s\n", print_function(f).c_str());
    std::unique_ptr<Executable> exe(new Executable());
    exe->shard_plan_ = shard_function(f, options.shard);
    exe->pass_log_ = run_pass_pipeline(f, options);
    optimize_loop_bodies(f, options);
    exe->optimized_text_ = print_function(f);
    if (std::getenv("METALHLO_DUMP_OPTIMIZED")) fprintf(stderr, "[metalhlo] optimized module:\n%s\n", exe->optimized_text_.c_str());
    Lowering lower(f, exe.get());
    lower.run();
    if (!exe->const_pool_.empty()) {
        void* p = nullptr;
        if (mhlo_cuda_alloc(exe->const_pool_.size(), &p) != 0) throw CompileError(6, std::string("constant pool: ") + mhlo_cuda_last_error());
        exe->const_dev_ = static_cast<char*>(p);
        if (mhlo_cuda_upload(p, exe->const_pool_.data(), exe->const_pool_.size(), nullptr) != 0 || mhlo_cuda_stream_sync(nullptr) != 0)
            throw CompileError(9, std::string("constant upload: ") + mhlo_cuda_last_error());
    }
    if (exe->arena_bytes_ > 0) {
        void* p = nullptr;
        if (mhlo_cuda_alloc(static_cast<size_t>(exe->arena_bytes_), &p) != 0)
            throw CompileError(6, std::string("arena of ") + std::to_string(exe->arena_bytes_) + " bytes: " + mhlo_cuda_last_error());
        exe->arena_dev_ = static_cast<char*>(p);
    }
    return exe;
}

int Executable::run_steps(const Ctx& c, bool debug, bool profile) {
    void* stream = c.stream;
    void *e0 = nullptr, *e1 = nullptr;
    if (profile) { mhlo_cuda_event_create(&e0); mhlo_cuda_event_create(&e1); }
    std::map<std::string, std::pair<int, double>> by_label;
    const char* profile_env = std::getenv("METALHLO_PROFILE_GPU");
    const bool every_step = profile && profile_env && profile_env[0] == '2';  // METALHLO_PROFILE_GPU=2: one line per step
    for (size_t i = 0; i < steps_.size(); ++i) {
        if (debug) fprintf(stderr, "[metalhlo] step %zu: %s\n", i, steps_[i].label.c_str());
        if (profile) mhlo_cuda_event_record(e0, stream);
        const int st = steps_[i].run(c);
        if (st != 0) {
            error_ = "step " + std::to_string(i) + " (" + steps_[i].label + "): " + mhlo_cuda_last_error();
            return st;
        }
        if (profile) {
            float ms = 0;
            mhlo_cuda_event_record(e1, stream);
            mhlo_cuda_event_elapsed_ms(e0, e1, &ms);
            auto& slot = by_label[steps_[i].label];
            slot.first += 1;
            slot.second += ms;
            if (ms > 0.5f || every_step)
                fprintf(stderr, "[metalhlo] step %zu %-40s %-28s %.3f ms\n", i, steps_[i].label.c_str(), steps_[i].detail.c_str(), ms);
        }
    }
    if (profile) {
        for (const auto& kv : by_label) fprintf(stderr, "[metalhlo] %-44s x%-4d %.3f ms\n", kv.first.c_str(), kv.second.first, kv.second.second);
        mhlo_cuda_event_destroy(e0);
        mhlo_cuda_event_destroy(e1);
    }
    return 0;
}

int Executable::execute(const void* const* inputs, void* const* outputs, void* stream) {
    Ctx c{inputs, outputs, arena_dev_, const_dev_, stream};
    const bool debug = std::getenv("METALHLO_DEBUG_DISPATCH") != nullptr;
    // METALHLO_PROFILE_GPU: per-step device times from CUDA events (synchronises after every step)
    const bool profile = std::getenv("METALHLO_PROFILE_GPU") != nullptr;
    static const bool graphs_enabled = [] {
        const char* v = std::getenv("METALHLO_CUDA_GRAPH");
        return !(v && std::string(v) == "0");
    }();
    // Graph replay needs a capturable stream, a program worth recording and no per-step host work.
    constexpr size_t kMinStepsForGraph = 8, kMaxSlots = 4;
    if (!graphs_enabled || !graphs_usable_ || host_control_ || stream == nullptr || debug || profile || steps_.size() < kMinStepsForGraph)
        return run_steps(c, debug, profile);

    std::vector<const void*> key;
    key.push_back(stream);
    for (size_t i = 0; i < input_types_.size(); ++i) key.push_back(inputs[i]);
    for (size_t i = 0; i < output_types_.size(); ++i) key.push_back(outputs[i]);
    ++graph_clock_;
    GraphSlot* slot = nullptr;
    for (GraphSlot& s : graph_slots_)
        if (s.key == key) { slot = &s; break; }
    if (slot == nullptr) {
        // first time with these buffers: run launch by launch and remember the combination
        if (graph_slots_.size() < kMaxSlots) {
            graph_slots_.emplace_back();
            slot = &graph_slots_.back();
        } else {
            slot = &graph_slots_[0];
            for (GraphSlot& s : graph_slots_)
                if (s.last_use < slot->last_use) slot = &s;
            if (slot->graph) mhlo_cuda_graph_destroy(slot->graph);
            slot->graph = nullptr;
        }
        slot->key = key;
        slot->last_use = graph_clock_;
        return run_steps(c, false, false);
    }
    slot->last_use = graph_clock_;
    if (slot->graph == nullptr) {
        // second time: record the launch list (nothing executes while recording), then fall through to the replay
        if (mhlo_cuda_graph_capture_begin(stream) != MHLO_CUDA_OK) return run_steps(c, false, false);  // e.g. the caller is recording
        const int st = run_steps(c, false, false);
        void* graph = nullptr;
        const int end = mhlo_cuda_graph_capture_end(stream, &graph);
        if (st != 0 || end != MHLO_CUDA_OK || graph == nullptr) {
            if (graph) mhlo_cuda_graph_destroy(graph);
            graphs_usable_ = false;  // something in this program cannot be recorded: stay with plain launches
            return run_steps(c, false, false);
        }
        slot->graph = graph;
    }
    if (mhlo_cuda_graph_launch(slot->graph, stream) != MHLO_CUDA_OK) {
        error_ = std::string("graph launch: ") + mhlo_cuda_last_error();
        return MHLO_CUDA_EXECUTION_FAILED;
    }
    ++graph_replays;
    return 0;
}

std::vector<std::string> Executable::step_labels() const {
    std::vector<std::string> l;
    for (const Step& s : steps_) l.push_back(s.label);
    return l;
}

}  // namespace mhlo
