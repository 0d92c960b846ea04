// The optimisation pipeline: simplification -> canonicalisation -> pattern fusion -> generic fusion -> layout ->
// scheduling -> cleanup, one sweep, in the registration order of the reference's PassManager
// (Sources/MetalHLOCore/Compiler/PassManager.swift:121-237). Pattern-fusion passes rewrite a matched subgraph to a
// stablehlo.custom_call with the reference's target names and a JSON backend_config
// (fused_scaled_dot_product_attention, fused_layer_norm, fused_rms_norm, fused_softmax, fused_gelu,
// fused_matmul_bias_activation, fused_elementwise). Unlike the reference, scale / eps / causal are read from the
// matched graph, so a fused program computes what the unfused one does.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <sstream>

#include "../../../include/mhlo_cuda.h"
#include "compiler.h"
#include "numeric.h"

namespace mhlo {

int elementwise_opcode(const std::string& name);  // executable.cpp

namespace {

// ---- helpers over the def-use graph -----------------------------------------------------------------------------

struct Graph {
    Function& f;
    std::vector<std::vector<int>> users;
    explicit Graph(Function& fn) : f(fn), users(fn.users()) {}
    const Op* def(int v) const {
        const int d = f.values[v].def_op;
        return d >= 0 && d < static_cast<int>(f.ops.size()) && !f.ops[d].dead ? &f.ops[d] : nullptr;
    }
    Op* def_mut(int v) { return const_cast<Op*>(def(v)); }
    int def_index(int v) const { return f.values[v].def_op; }
    bool is(int v, const char* name) const { const Op* o = def(v); return o && o->name == name; }
    size_t n_users(int v) const { return users[v].size(); }
    const TensorType& type(int v) const { return f.values[v].type; }
};

// Scalar value of a constant reached through broadcast_in_dim / reshape / convert chains.
bool scalar_constant(const Graph& g, int v, double* out) {
    for (int hops = 0; hops < 8; ++hops) {
        const Op* o = g.def(v);
        if (!o) return false;
        if (o->name == "constant") {
            const Attr* a = o->attr("value");
            if (!a || a->kind != Attr::Dense) return false;
            const size_t es = dtype_size(a->dense_type.dtype);
            if (!(a->splat || a->dense.size() == es)) return false;
            *out = decode_as_double(a->dense_type.dtype, a->dense.data());
            return true;
        }
        if (o->name == "broadcast_in_dim" || o->name == "reshape" || o->name == "convert" || o->name == "broadcast") { v = o->operands[0]; continue; }
        return false;
    }
    return false;
}

// Follows broadcast_in_dim / reshape back to the value being broadcast.
int strip_broadcast(const Graph& g, int v) {
    for (int hops = 0; hops < 4; ++hops) {
        const Op* o = g.def(v);
        if (o && (o->name == "broadcast_in_dim" || o->name == "reshape")) v = o->operands[0];
        else break;
    }
    return v;
}

Attr dense_scalar(DType t, double v) {
    Attr a;
    a.kind = Attr::Dense;
    a.dense_type.dtype = t;
    a.dense.resize(dtype_size(t));
    encode_scalar(t, v, static_cast<int64_t>(v), a.dense.data());
    return a;
}

void replace_uses(Function& f, int from, int to) {
    std::function<void(std::vector<Op>&)> walk = [&](std::vector<Op>& ops) {
        for (Op& o : ops) {
            for (int& v : o.operands) if (v == from) v = to;
            for (auto& r : o.regions) walk(r->ops);
        }
    };
    walk(f.ops);
}

int count_live(const Function& f) {
    int n = 0;
    for (const Op& o : f.ops) n += !o.dead;
    return n;
}

bool has_side_effect(const Op& o) { return o.name == "return" || o.results.empty(); }

// ---- simplification -------------------------------------------------------------------------------------------------

bool dce(Function& f) {
    bool any = false;
    for (;;) {
        std::vector<int> uses(f.values.size(), 0);
        for (const Op& o : f.ops) {
            if (o.dead) continue;
            for (int v : o.operands) ++uses[v];
            std::function<void(const Region&)> walk = [&](const Region& r) {
                for (const Op& q : r.ops) { for (int v : q.operands) ++uses[v]; for (const auto& s : q.regions) walk(*s); }
            };
            for (const auto& r : o.regions) walk(*r);
        }
        bool changed = false;
        for (Op& o : f.ops) {
            if (o.dead || has_side_effect(o)) continue;
            bool used = false;
            for (int r : o.results) used |= uses[r] > 0;
            if (!used) { o.dead = true; changed = true; }
        }
        if (!changed) break;
        any = true;
    }
    if (any) f.compact();
    return any;
}

bool is_splat_value(const Graph& g, int v, double want) {
    double c;
    return scalar_constant(g, v, &c) && c == want;
}

// The algebraic rules of the reference's simplifier (Sources/MetalHLOCore/Optimizer/AlgebraicSimplifier.swift:68-94):
// x+0, x*1, x*0, x-0, x/1, x-x, x/x, -(-x), exp(log x), log(exp x), reshape(reshape), reshape to the same type,
// identity transpose, transpose(transpose), and folding of unary/binary ops over splat constants.
bool algebraic_simplify(Function& f, int max_iters) {
    bool any = false;
    for (int it = 0; it < max_iters; ++it) {
        Graph g(f);
        bool changed = false;
        for (size_t i = 0; i < f.ops.size(); ++i) {
            Op& o = f.ops[i];
            if (o.dead || o.results.size() != 1) continue;
            const int r = o.results[0];
            const TensorType& rt = o.result_types[0];
            auto forward = [&](int to) {
                if (g.type(to) != rt) return false;
                replace_uses(f, r, to);
                o.dead = true;
                changed = true;
                return true;
            };
            auto to_constant = [&](double v) {
                o.name = "constant";
                o.operands.clear();
                o.attrs.clear();
                Attr a = dense_scalar(rt.dtype, v);
                a.dense_type = rt;
                a.splat = rt.count() != 1;
                o.attrs["value"] = a;
                changed = true;
            };
            const std::string& n = o.name;
            if (n == "add") {
                if (is_splat_value(g, o.operands[1], 0) && forward(o.operands[0])) continue;
                if (is_splat_value(g, o.operands[0], 0) && forward(o.operands[1])) continue;
            } else if (n == "subtract") {
                if (is_splat_value(g, o.operands[1], 0) && forward(o.operands[0])) continue;
                if (o.operands[0] == o.operands[1] && !is_float(rt.dtype)) { to_constant(0); continue; }
            } else if (n == "multiply") {
                if (is_splat_value(g, o.operands[1], 1) && forward(o.operands[0])) continue;
                if (is_splat_value(g, o.operands[0], 1) && forward(o.operands[1])) continue;
                if (!is_float(rt.dtype) && (is_splat_value(g, o.operands[0], 0) || is_splat_value(g, o.operands[1], 0))) { to_constant(0); continue; }
            } else if (n == "divide") {
                if (is_splat_value(g, o.operands[1], 1) && forward(o.operands[0])) continue;
            } else if (n == "negate") {
                if (g.is(o.operands[0], "negate") && forward(g.def(o.operands[0])->operands[0])) continue;
            } else if (n == "exponential") {
                if (g.is(o.operands[0], "log") && forward(g.def(o.operands[0])->operands[0])) continue;
            } else if (n == "log") {
                if (g.is(o.operands[0], "exponential") && forward(g.def(o.operands[0])->operands[0])) continue;
            } else if (n == "reshape") {
                if (g.type(o.operands[0]) == rt && forward(o.operands[0])) continue;
                if (g.is(o.operands[0], "reshape")) { o.operands[0] = g.def(o.operands[0])->operands[0]; changed = true; continue; }
            } else if (n == "transpose") {
                std::vector<int64_t> p = o.int_list("permutation");
                bool ident = true;
                for (size_t d = 0; d < p.size(); ++d) ident &= p[d] == static_cast<int64_t>(d);
                if (ident && forward(o.operands[0])) continue;
                if (g.is(o.operands[0], "transpose")) {
                    const Op* in = g.def(o.operands[0]);
                    std::vector<int64_t> q = in->int_list("permutation"), c(p.size());
                    for (size_t d = 0; d < p.size(); ++d) c[d] = q[p[d]];
                    o.attrs["permutation"] = Attr::make_ints(c);
                    o.operands[0] = in->operands[0];
                    changed = true;
                    continue;
                }
            } else if (n == "convert") {
                if (g.type(o.operands[0]) == rt && forward(o.operands[0])) continue;
            }
            // constant folding over scalar/splat constants (float types only fold exactly representable cases
            // through the same double arithmetic the device would round from)
            if (o.operands.size() <= 2 && !o.operands.empty() && n != "constant" && n != "convert" && n != "reshape" &&
                n != "broadcast_in_dim" && n != "transpose") {
                const int code = elementwise_opcode(n);
                double a = 0, b = 0;
                bool ok = code >= 0 && scalar_constant(g, o.operands[0], &a) && g.is(o.operands[0], "constant");
                if (ok && o.operands.size() == 2) ok = scalar_constant(g, o.operands[1], &b) && g.is(o.operands[1], "constant");
                if (ok && is_float(rt.dtype) && rt.dtype == g.type(o.operands[0]).dtype) {
                    double v;
                    bool folded = true;
                    switch (code) {
                        case MHLO_EW_ADD: v = a + b; break;
                        case MHLO_EW_SUB: v = a - b; break;
                        case MHLO_EW_MUL: v = a * b; break;
                        case MHLO_EW_DIV: v = a / b; break;
                        case MHLO_EW_MAX: v = (a != a || b != b) ? std::nan("") : std::fmax(a, b); break;  // a NaN goes through, as in the kernels
                        case MHLO_EW_MIN: v = (a != a || b != b) ? std::nan("") : std::fmin(a, b); break;
                        case MHLO_EW_NEG: v = -a; break;
                        case MHLO_EW_SQRT: v = std::sqrt(a); break;
                        case MHLO_EW_RSQRT: v = 1.0 / std::sqrt(a); break;
                        default: folded = false; v = 0;
                    }
                    if (folded) {
                        // round through the element type the way the device store would
                        uint8_t buf[8];
                        encode_float(rt.dtype, rt.dtype == DType::F32 ? static_cast<double>(static_cast<float>(v)) : v, buf);
                        to_constant(decode_as_double(rt.dtype, buf));
                        continue;
                    }
                }
            }
        }
        if (!changed) break;
        any = true;
        f.compact();
        dce(f);
    }
    return any;
}

std::string op_key(const Function& f, const Op& o) {
    std::ostringstream k;
    k << o.dialect << "." << o.name << "(";
    for (int v : o.operands) k << v << ",";
    k << ")";
    for (const auto& kv : o.attrs) {
        k << kv.first << "=";
        const Attr& a = kv.second;
        switch (a.kind) {
            case Attr::Int: k << a.i; break;
            case Attr::Float: k << a.f; break;
            case Attr::Bool: k << a.b; break;
            case Attr::String: case Attr::Keyword: k << a.s; break;
            case Attr::IntArray: for (int64_t x : a.ints) k << x << ","; break;
            case Attr::Dense: k << a.dense_type.str() << ":" << a.splat << ":"; k.write(reinterpret_cast<const char*>(a.dense.data()), static_cast<std::streamsize>(a.dense.size())); break;
            default: k << "#" << reinterpret_cast<uintptr_t>(&a); break;  // never equal
        }
        k << ";";
    }
    for (const TensorType& t : o.result_types) k << t.str();
    (void)f;
    return k.str();
}

bool cse(Function& f) {
    std::map<std::string, int> seen;
    bool changed = false;
    for (size_t i = 0; i < f.ops.size(); ++i) {
        Op& o = f.ops[i];
        if (o.dead || has_side_effect(o) || !o.regions.empty() || o.results.size() != 1) continue;
        if (o.name == "rng") continue;  // two draws with the same bounds are two different tensors
        if (o.name == "constant" && o.attr("value") && o.attr("value")->dense.size() > 4096) continue;
        const std::string key = op_key(f, o);
        auto it = seen.find(key);
        if (it == seen.end()) { seen[key] = static_cast<int>(i); continue; }
        replace_uses(f, o.results[0], f.ops[it->second].results[0]);
        o.dead = true;
        changed = true;
    }
    if (changed) f.compact();
    return changed;
}

// ---- canonicalisation ------------------------------------------------------------------------------------------------

bool canonicalize_reshape(Function& f) {
    Graph g(f);
    bool changed = false;
    for (Op& o : f.ops) {
        if (o.dead || o.name != "reshape") continue;
        if (g.type(o.operands[0]) == o.result_types[0]) { replace_uses(f, o.results[0], o.operands[0]); o.dead = true; changed = true; continue; }
        if (g.is(o.operands[0], "reshape")) { o.operands[0] = g.def(o.operands[0])->operands[0]; changed = true; }
    }
    if (changed) { f.compact(); dce(f); }
    return changed;
}

bool canonicalize_transpose(Function& f) {
    Graph g(f);
    bool changed = false;
    for (Op& o : f.ops) {
        if (o.dead || o.name != "transpose") continue;
        std::vector<int64_t> p = o.int_list("permutation");
        bool ident = true;
        for (size_t d = 0; d < p.size(); ++d) ident &= p[d] == static_cast<int64_t>(d);
        if (ident) { replace_uses(f, o.results[0], o.operands[0]); o.dead = true; changed = true; continue; }
        if (g.is(o.operands[0], "transpose")) {
            const Op* in = g.def(o.operands[0]);
            std::vector<int64_t> q = in->int_list("permutation"), c(p.size());
            for (size_t d = 0; d < p.size(); ++d) c[d] = q[p[d]];
            o.attrs["permutation"] = Attr::make_ints(c);
            o.operands[0] = in->operands[0];
            changed = true;
        }
    }
    if (changed) { f.compact(); dce(f); }
    return changed;
}

bool canonicalize_broadcast(Function& f) {
    Graph g(f);
    bool changed = false;
    for (Op& o : f.ops) {
        if (o.dead || o.name != "broadcast_in_dim") continue;
        std::vector<int64_t> dims = o.int_list("broadcast_dimensions");
        const TensorType& it = g.type(o.operands[0]);
        if (it == o.result_types[0]) {
            bool ident = true;
            for (size_t d = 0; d < dims.size(); ++d) ident &= dims[d] == static_cast<int64_t>(d);
            if (ident) { replace_uses(f, o.results[0], o.operands[0]); o.dead = true; changed = true; continue; }
        }
        if (g.is(o.operands[0], "broadcast_in_dim")) {  // broadcast of a broadcast composes
            const Op* in = g.def(o.operands[0]);
            std::vector<int64_t> inner = in->int_list("broadcast_dimensions"), c(inner.size());
            for (size_t d = 0; d < inner.size(); ++d) c[d] = dims[inner[d]];
            // only when the inner op did not expand an extent-1 dim that the outer one then maps (keeps it simple)
            const TensorType& src = g.type(in->operands[0]);
            bool simple = true;
            for (size_t d = 0; d < inner.size(); ++d) simple &= src.shape[d] == in->result_types[0].shape[inner[d]] || src.shape[d] == 1;
            if (simple) { o.attrs["broadcast_dimensions"] = Attr::make_ints(c); o.operands[0] = in->operands[0]; changed = true; }
        }
    }
    if (changed) { f.compact(); dce(f); }
    return changed;
}

// ---- pattern fusion ---------------------------------------------------------------------------------------------------

std::string fmt_double(double v) {
    char b[64];
    std::snprintf(b, sizeof b, "%.17g", v);
    return b;
}

// Turns op `root` into custom_call @target(operands) {backend_config}; the matched interior dies by DCE.
void make_custom_call(Op& root, const std::string& target, const std::vector<int>& operands, const std::string& config) {
    root.name = "custom_call";
    root.dialect = "stablehlo";
    root.operands = operands;
    root.attrs.clear();
    root.regions.clear();
    root.attrs["call_target_name"] = Attr::make_string(target);
    root.attrs["backend_config"] = Attr::make_string(config);
}

// softmax over one axis: div(e, bcast(reduce_add(e))) with e = exp(sub(x, bcast(reduce_max(x)))).
// Reference detector: Sources/MetalHLOCore/Compiler/Analyzer.swift:513-619.
struct SoftmaxMatch { int x = -1; int64_t axis = -1; std::vector<int> interior; };

bool match_softmax(const Graph& g, int root_value, SoftmaxMatch* m) {
    const Op* div = g.def(root_value);
    if (!div || div->name != "divide") return false;
    const int e = div->operands[0];
    const Op* ex = g.def(e);
    if (!ex || ex->name != "exponential") return false;
    const int sum_v = strip_broadcast(g, div->operands[1]);
    const Op* sum = g.def(sum_v);
    if (!sum || sum->name != "reduce" || sum->str_attr("reducer") != "add" || sum->operands[0] != e) return false;
    std::vector<int64_t> dims = sum->int_list("dimensions");
    if (dims.size() != 1) return false;
    const Op* sub = g.def(ex->operands[0]);
    if (!sub || sub->name != "subtract") return false;
    const int x = sub->operands[0];
    const int max_v = strip_broadcast(g, sub->operands[1]);
    const Op* mx = g.def(max_v);
    if (!mx || mx->name != "reduce" || mx->str_attr("reducer") != "maximum" || mx->operands[0] != x) return false;
    if (mx->int_list("dimensions") != dims) return false;
    // exp feeds only the sum and the divide; sub only exp; the reduces only their broadcasts
    if (g.n_users(e) != 2 || g.n_users(sub->results[0]) != 1) return false;
    if (g.type(x) != g.type(root_value)) return false;
    m->x = x;
    m->axis = dims[0];
    return true;
}

bool fuse_softmax(Function& f) {
    Graph g(f);
    bool changed = false;
    for (Op& o : f.ops) {
        if (o.dead || o.name != "divide" || o.results.size() != 1) continue;
        SoftmaxMatch m;
        if (!match_softmax(g, o.results[0], &m)) continue;
        if (!is_float(g.type(m.x).dtype) || g.type(m.x).dtype == DType::F64) continue;
        make_custom_call(o, "fused_softmax", {m.x}, "{\"axis\":" + std::to_string(m.axis) + "}");
        changed = true;
    }
    if (changed) dce(f);
    return changed;
}

// mean over the last axis written as reduce_add(x)/N or reduce_add(x)*(1/N); returns the reduced operand.
bool match_mean_last(const Graph& g, int v, int* x_out) {
    v = strip_broadcast(g, v);
    const Op* o = g.def(v);
    if (!o) return false;
    double c;
    int red = -1;
    if (o->name == "divide" && scalar_constant(g, o->operands[1], &c)) red = o->operands[0];
    else if (o->name == "multiply" && scalar_constant(g, o->operands[1], &c)) { red = o->operands[0]; c = 1.0 / c; }
    else if (o->name == "multiply" && scalar_constant(g, o->operands[0], &c)) { red = o->operands[1]; c = 1.0 / c; }
    else return false;
    red = strip_broadcast(g, red);
    const Op* r = g.def(red);
    if (!r || r->name != "reduce" || r->str_attr("reducer") != "add") return false;
    const TensorType& xt = g.type(r->operands[0]);
    std::vector<int64_t> dims = r->int_list("dimensions");
    if (dims.size() != 1 || dims[0] != xt.rank() - 1) return false;
    if (std::fabs(c - static_cast<double>(xt.shape.back())) > 1e-3 * c) return false;
    *x_out = r->operands[0];
    return true;
}

// rsqrt(var + eps) or 1/sqrt(var + eps); returns the variance-like value and eps.
bool match_inv_std(const Graph& g, int v, int* var_out, double* eps_out, bool* is_divisor) {
    v = strip_broadcast(g, v);
    const Op* o = g.def(v);
    if (!o) return false;
    int inner = -1;
    if (o->name == "rsqrt") { inner = o->operands[0]; *is_divisor = false; }
    else if (o->name == "sqrt") { inner = o->operands[0]; *is_divisor = true; }
    else if (o->name == "divide" && is_splat_value(g, o->operands[0], 1) && g.is(o->operands[1], "sqrt")) { inner = g.def(o->operands[1])->operands[0]; *is_divisor = false; }
    else return false;
    const Op* add = g.def(inner);
    if (!add || add->name != "add") return false;
    double eps;
    if (scalar_constant(g, add->operands[1], &eps)) *var_out = add->operands[0];
    else if (scalar_constant(g, add->operands[0], &eps)) *var_out = add->operands[1];
    else return false;
    *eps_out = eps;
    return true;
}

// Peels "t * bcast(gamma)" and "+ bcast(beta)" layers (either operand order) off a normalised value.
// gamma/beta must be vectors over the last axis.
int vector_over_last_axis(const Graph& g, int v, const TensorType& full) {
    const Op* o = g.def(v);
    if (!o || o->name != "broadcast_in_dim") return -1;
    const TensorType& st = g.type(o->operands[0]);
    std::vector<int64_t> dims = o->int_list("broadcast_dimensions");
    if (st.rank() == 1 && dims.size() == 1 && dims[0] == full.rank() - 1 && st.shape[0] == full.shape.back()) return o->operands[0];
    return -1;
}

struct NormMatch { bool rms = false; int x = -1, gamma = -1, beta = -1; double eps = 1e-5; };

// LayerNorm: ((x - mean(x)) * rsqrt(mean((x-mean)^2) + eps)) [* gamma] [+ beta]   (or "/ sqrt(..)")
// RMSNorm:   (x * rsqrt(mean(x^2) + eps)) [* gamma]
// Reference detectors: Analyzer.swift:726-1083.
bool match_norm_core(const Graph& g, int v, NormMatch* m) {
    const Op* o = g.def(v);
    if (!o || (o->name != "multiply" && o->name != "divide")) return false;
    for (int side = 0; side < 2; ++side) {
        if (o->name == "divide" && side == 1) break;
        const int num = o->operands[side], other = o->operands[1 - side];
        int var_v;
        double eps;
        bool divisor;
        if (!match_inv_std(g, other, &var_v, &eps, &divisor)) continue;
        if (divisor != (o->name == "divide")) continue;
        int sq_src;
        if (!match_mean_last(g, var_v, &sq_src)) continue;
        const Op* sq = g.def(sq_src);
        if (!sq || sq->name != "multiply" || sq->operands[0] != sq->operands[1]) continue;
        const int squared = sq->operands[0];
        if (squared != num) continue;
        // num is either x (RMS) or x - mean(x) (LayerNorm)
        const Op* c = g.def(num);
        int mean_src;
        if (c && c->name == "subtract" && match_mean_last(g, c->operands[1], &mean_src) && mean_src == c->operands[0]) {
            m->rms = false;
            m->x = c->operands[0];
        } else {
            m->rms = true;
            m->x = num;
        }
        m->eps = eps;
        return g.type(m->x) == g.type(v);
    }
    return false;
}

bool fuse_norm(Function& f) {
    bool any = false;
    for (;;) {
        Graph g(f);
        bool changed = false;
        // roots in reverse order so the outermost affine layer is seen first
        for (size_t idx = f.ops.size(); idx-- > 0;) {
            Op& o = f.ops[idx];
            if (o.dead || o.results.size() != 1) continue;
            const TensorType& rt = o.result_types[0];
            if (!is_float(rt.dtype) || rt.dtype == DType::F64 || rt.rank() < 1) continue;
            NormMatch m;
            int core = o.results[0];
            int gamma = -1, beta = -1;
            // optional + beta
            if (o.name == "add") {
                for (int s = 0; s < 2; ++s) {
                    int b = vector_over_last_axis(g, o.operands[1 - s], rt);
                    if (b >= 0) { beta = b; core = o.operands[s]; break; }
                }
                if (beta < 0) continue;
            }
            // optional * gamma
            const Op* c = g.def(core);
            if (c && c->name == "multiply") {
                for (int s = 0; s < 2; ++s) {
                    int gm = vector_over_last_axis(g, c->operands[1 - s], rt);
                    if (gm >= 0 && match_norm_core(g, c->operands[s], &m)) { gamma = gm; break; }
                }
            }
            if (gamma < 0 && !match_norm_core(g, core, &m)) continue;
            if (m.rms && beta >= 0) continue;  // RMSNorm has no shift: leave "+ beta" to a separate op
            if (core != o.results[0] && g.n_users(core) != 1) continue;
            std::string cfg = "{\"eps\":" + fmt_double(m.eps) + ",\"axes\":[-1]}";
            const int root_result = o.results[0];
            const DType dt = rt.dtype;
            const int64_t hidden = rt.shape.back();
            std::vector<int> operands = {m.x};
            std::string target = m.rms ? "fused_rms_norm" : "fused_layer_norm";
            if (m.rms) {
                if (gamma >= 0) operands.push_back(gamma);
            } else if (gamma >= 0 || beta >= 0) {
                // fused_layer_norm takes (x, gamma, beta): a missing factor becomes a constant vector. add_op
                // inserts into f.ops, so `o` must not be touched after this point.
                size_t at = idx;
                auto const_vec = [&](double val) {
                    Op k;
                    k.name = "constant";
                    k.dialect = "stablehlo";
                    TensorType t;
                    t.dtype = dt;
                    t.shape = {hidden};
                    Attr a = dense_scalar(dt, val);
                    a.dense_type = t;
                    a.splat = true;
                    k.attrs["value"] = a;
                    return f.add_op(k, t, at++);
                };
                const int gv = gamma >= 0 ? gamma : const_vec(1.0);
                const int bv = beta >= 0 ? beta : const_vec(0.0);
                operands.push_back(gv);
                operands.push_back(bv);
            }
            for (Op& q : f.ops)
                if (!q.dead && q.results.size() == 1 && q.results[0] == root_result) {
                    make_custom_call(q, target, operands, cfg);
                    break;
                }
            changed = true;
            break;  // the graph changed: rebuild use lists
        }
        if (!changed) break;
        any = true;
        dce(f);
    }
    return any;
}

// Recognises a single-input elementwise subgraph by evaluating it at probe points and comparing with the
// closed forms of the activations the runtime fuses. More permissive than the reference's structural matcher
// (Analyzer.swift:1084-1527, constants within +-0.01) and insensitive to how the polynomial is factored.
struct Cone { int input = -1; std::vector<int> ops; };

bool eval_cone(const Graph& g, int v, int input, double x, double* out, int depth = 0) {
    if (v == input) { *out = x; return true; }
    if (depth > 24) return false;
    double c;
    if (scalar_constant(g, v, &c)) { *out = c; return true; }
    const Op* o = g.def(v);
    if (!o || o->operands.empty() || o->operands.size() > 2) return false;
    if (o->name == "broadcast_in_dim" || o->name == "reshape") return false;
    double a, b = 0;
    if (!eval_cone(g, o->operands[0], input, x, &a, depth + 1)) return false;
    if (o->operands.size() == 2 && !eval_cone(g, o->operands[1], input, x, &b, depth + 1)) return false;
    const std::string& n = o->name;
    if (n == "add") *out = a + b;
    else if (n == "subtract") *out = a - b;
    else if (n == "multiply") *out = a * b;
    else if (n == "divide") *out = a / b;
    else if (n == "negate") *out = -a;
    else if (n == "tanh") *out = std::tanh(a);
    else if (n == "exponential") *out = std::exp(a);
    else if (n == "logistic") *out = 1.0 / (1.0 + std::exp(-a));
    else if (n == "power") *out = std::pow(a, b);
    else if (n == "maximum") *out = std::fmax(a, b);
    else if (n == "sqrt") *out = std::sqrt(a);
    else if (n == "convert") *out = a;
    else if (n == "custom_call" && o->str_attr("call_target_name") == "erf") *out = std::erf(a);
    else if (n == "erf") *out = std::erf(a);
    else return false;
    return true;
}

bool cone_op(const Op* o) {
    static const char* kOps[] = {"add", "subtract", "multiply", "divide", "negate", "tanh", "exponential", "logistic", "power",
                                 "maximum", "sqrt", "erf", "convert"};
    if (!o) return false;
    for (const char* k : kOps)
        if (o->name == k) return true;
    return o->name == "custom_call" && o->str_attr("call_target_name") == "erf";
}

// True when every path from v upwards ends at `input` or at a scalar constant, passing only through elementwise ops.
bool cone_closed(const Graph& g, int v, int input, int depth = 0) {
    if (v == input) return true;
    double c;
    if (scalar_constant(g, v, &c)) return true;
    const Op* o = g.def(v);
    if (!cone_op(o) || depth > 24) return false;
    for (int x : o->operands)
        if (!cone_closed(g, x, input, depth + 1)) return false;
    return true;
}

// Values reachable upwards from v through elementwise ops: the candidates for "the x of f(x)".
void cone_values(const Graph& g, int v, std::vector<int>* out, int depth = 0) {
    if (std::find(out->begin(), out->end(), v) != out->end()) return;
    double c;
    if (scalar_constant(g, v, &c)) return;
    out->push_back(v);
    const Op* o = g.def(v);
    if (!cone_op(o) || depth > 24) return;
    for (int x : o->operands) cone_values(g, x, out, depth + 1);
}

// Residual add feeding a norm: y = norm(a + b) where the sum is also the residual stream read later.
//   s = add(a, b); y = custom_call @fused_layer_norm(s, gamma, beta)
// becomes one op with two results,
//   s, y = custom_call @fused_add_layer_norm(a, b, gamma, beta)
// whose kernel reads a and b once, writes the rounded sum and normalises it in registers (the sum is not read back).
// Every other user of the sum has to come after the norm in program order. The reference registers
// "residual-chain-fusion" without an implementation (Compiler/PassManager.swift:214-221).
bool fuse_residual_norm(Function& f) {
    Graph g(f);
    bool changed = false;
    for (size_t idx = 0; idx < f.ops.size(); ++idx) {
        Op& o = f.ops[idx];
        if (o.dead || o.name != "custom_call" || o.results.size() != 1 || o.operands.empty()) continue;
        const std::string target = o.str_attr("call_target_name");
        if (target != "fused_layer_norm" && target != "fused_rms_norm") continue;
        const int s = o.operands[0];
        Op* add = g.def_mut(s);
        if (!add || add->name != "add" || add->operands.size() != 2 || add->results.size() != 1) continue;
        const TensorType& st = g.type(s);
        if (!is_float(st.dtype) || st.dtype == DType::F64) continue;
        if (!(g.type(add->operands[0]) == st) || !(g.type(add->operands[1]) == st)) continue;
        bool ordered = true;
        for (int user : g.users[s]) ordered = ordered && user >= static_cast<int>(idx);
        // gamma / beta must not be computed from the sum itself
        for (size_t k = 1; k < o.operands.size(); ++k) ordered = ordered && o.operands[k] != s;
        if (!ordered) continue;
        const int y = o.results[0];
        const TensorType yt = o.result_types[0];
        std::vector<int> operands = {add->operands[0], add->operands[1]};
        for (size_t k = 1; k < o.operands.size(); ++k) operands.push_back(o.operands[k]);
        o.operands = operands;
        o.attrs["call_target_name"] = Attr::make_string(target == "fused_layer_norm" ? "fused_add_layer_norm" : "fused_add_rms_norm");
        o.results = {s, y};
        o.result_types = {st, yt};
        add->dead = true;
        add->results.clear();
        changed = true;
    }
    if (changed) f.compact();
    return changed;
}

bool fuse_activations(Function& f) {
    Graph g(f);
    bool changed = false;
    static const double probes[] = {-6.0, -2.5, -1.0, -0.3, 0.0, 0.2, 0.9, 1.7, 3.0, 7.5};
    for (size_t idx = f.ops.size(); idx-- > 0;) {
        Op& o = f.ops[idx];
        if (o.dead || o.name != "multiply" || o.results.size() != 1) continue;
        const TensorType& rt = o.result_types[0];
        if (!is_float(rt.dtype) || rt.dtype == DType::F64) continue;
        std::vector<int> cands;
        cone_values(g, o.results[0], &cands);
        // nearest candidates first: the latest-defined value that closes the cone is the function's argument
        std::sort(cands.begin(), cands.end(), [&](int a, int b) { return g.def_index(a) > g.def_index(b); });
        int input = -1;
        bool gelu_t = false, gelu_e = false, silu = false;
        for (int cand : cands) {
            if (cand == o.results[0] || g.type(cand) != rt || !cone_closed(g, o.results[0], cand)) continue;
            bool gt_ok = true, ge_ok = true, sl_ok = true;
            for (double x : probes) {
                double y;
                if (!eval_cone(g, o.results[0], cand, x, &y)) { gt_ok = ge_ok = sl_ok = false; break; }
                const double gt = 0.5 * x * (1 + std::tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)));
                const double ge = 0.5 * x * (1 + std::erf(x * 0.7071067811865476));
                const double sl = x / (1 + std::exp(-x));
                gt_ok &= std::fabs(y - gt) < 2e-3 * (1 + std::fabs(y));  // the reference accepts constants within +-0.01
                ge_ok &= std::fabs(y - ge) < 1e-6 * (1 + std::fabs(y));
                sl_ok &= std::fabs(y - sl) < 1e-6 * (1 + std::fabs(y));
            }
            if (gt_ok || ge_ok || sl_ok) { input = cand; gelu_t = gt_ok; gelu_e = ge_ok; silu = sl_ok; break; }
        }
        if (input < 0) continue;
        // the tanh form needs an actual tanh in the cone, the erf form an erf
        if (gelu_e) make_custom_call(o, "fused_gelu", {input}, "{\"approximate\":false}");
        else if (silu) make_custom_call(o, "fused_silu", {input}, "{}");
        else if (gelu_t) make_custom_call(o, "fused_gelu", {input}, "{\"approximate\":true}");
        else continue;
        changed = true;
    }
    if (changed) dce(f);
    return changed;
}

// ---- attention -----------------------------------------------------------------------------------------------------------

struct DotDims { std::vector<int64_t> lb, rb, lc, rc; };
DotDims dot_dims(const Op& o) {
    return {o.int_list("lhs_batching_dimensions"), o.int_list("rhs_batching_dimensions"),
            o.int_list("lhs_contracting_dimensions"), o.int_list("rhs_contracting_dimensions")};
}

// iota(dim a) >= iota(dim b) over a [Sq,Sk] (possibly broadcast) predicate: the causal mask.
bool is_causal_predicate(const Graph& g, int v, int rank) {
    v = strip_broadcast(g, v);
    const Op* c = g.def(v);
    if (!c || c->name != "compare") return false;
    const std::string dir = c->str_attr("comparison_direction");
    const Op* a = g.def(strip_broadcast(g, c->operands[0]));
    const Op* b = g.def(strip_broadcast(g, c->operands[1]));
    if (!a || !b || a->name != "iota" || b->name != "iota") return false;
    const TensorType& t = c->result_types[0];
    if (t.rank() < 2 || t.shape[t.rank() - 1] != t.shape[t.rank() - 2]) return false;
    const int64_t qa = t.rank() - 2, ka = t.rank() - 1;
    const int64_t da = a->int_attr("iota_dimension", -1), db = b->int_attr("iota_dimension", -1);
    (void)rank;
    // query index >= key index, written either way round
    if (dir == "GE" && da == qa && db == ka) return true;
    if (dir == "LE" && da == ka && db == qa) return true;
    return false;
}

// Matches softmax(scale * q.k^T [causal]) . v with q,k,v laid out [B,H,S,D] or [B,S,H,D] (batch dims b,h) and
// rewrites the PV dot into fused_scaled_dot_product_attention. Reference: AttentionFusionPass
// (PassManager.swift:594-708) and Analyzer.swift:631-723, which assume scale = 1/sqrt(D) and no mask.
bool fuse_attention(Function& f) {
    bool any = false;
    for (;;) {
        Graph g(f);
        bool changed = false;
        for (size_t idx = 0; idx < f.ops.size() && !changed; ++idx) {
            Op& pv = f.ops[idx];
            if (pv.dead || pv.name != "dot_general") continue;
            const TensorType& ot = pv.result_types[0];
            if (ot.rank() != 4 || !is_float(ot.dtype) || ot.dtype == DType::F64) continue;
            SoftmaxMatch sm;
            if (!match_softmax(g, pv.operands[0], &sm)) continue;
            const TensorType& pt = g.type(pv.operands[0]);
            if (sm.axis != pt.rank() - 1 || g.n_users(pv.operands[0]) != 1) continue;
            // P [b,h,q,k] . V: batch [0,1] x rb, contracting [3] x [key axis of V]
            DotDims d2 = dot_dims(pv);
            if (d2.lb != std::vector<int64_t>{0, 1} || d2.lc != std::vector<int64_t>{3} || d2.rb.size() != 2 || d2.rc.size() != 1) continue;
            // scores chain: [select causal] <- [mul/div scale] <- dot(q,k)
            int s = sm.x;
            bool causal = false;
            double scale = 1.0;
            // walk down from the softmax input
            auto single_use_or_softmax_input = [&](int v) { return v == sm.x ? g.n_users(v) == 2 : g.n_users(v) == 1; };
            bool ok = true;
            for (int hops = 0; hops < 4 && ok; ++hops) {
                const Op* o = g.def(s);
                if (!o) { ok = false; break; }
                if (!single_use_or_softmax_input(s)) { ok = false; break; }
                double c;
                if (o->name == "select" && is_causal_predicate(g, o->operands[0], pt.rank()) && scalar_constant(g, o->operands[2], &c) &&
                    (c <= -1e4 || std::isinf(c))) { causal = true; s = o->operands[1]; continue; }
                if (o->name == "multiply" && scalar_constant(g, o->operands[1], &c)) { scale *= c; s = o->operands[0]; continue; }
                if (o->name == "multiply" && scalar_constant(g, o->operands[0], &c)) { scale *= c; s = o->operands[1]; continue; }
                if (o->name == "divide" && scalar_constant(g, o->operands[1], &c)) { scale /= c; s = o->operands[0]; continue; }
                break;
            }
            if (!ok) continue;
            const Op* qk = g.def(s);
            if (!qk || qk->name != "dot_general" || !single_use_or_softmax_input(s)) continue;
            DotDims d1 = dot_dims(*qk);
            if (d1.lb.size() != 2 || d1.rb.size() != 2 || d1.lc.size() != 1 || d1.rc.size() != 1) continue;
            int q = qk->operands[0], k = qk->operands[1], v = pv.operands[1];
            // a scale folded into q: multiply(q, const)
            {
                const Op* qo = g.def(q);
                double c;
                if (qo && qo->name == "multiply" && g.n_users(q) == 1) {
                    if (scalar_constant(g, qo->operands[1], &c)) { scale *= c; q = qo->operands[0]; }
                    else if (scalar_constant(g, qo->operands[0], &c)) { scale *= c; q = qo->operands[1]; }
                }
            }
            const TensorType &qt = g.type(q), &kt = g.type(k), &vt = g.type(v);
            if (qt.rank() != 4 || kt.rank() != 4 || vt.rank() != 4) continue;
            // permutations that bring each operand to [b, h, s, d]
            auto perm_of = [](const std::vector<int64_t>& batch, int64_t contract_or_feature_last, int rank, bool contract_is_d) {
                std::vector<int64_t> p = batch;
                int64_t other = -1;
                for (int d = 0; d < rank; ++d)
                    if (std::find(batch.begin(), batch.end(), d) == batch.end() && d != contract_or_feature_last) other = d;
                if (contract_is_d) { p.push_back(other); p.push_back(contract_or_feature_last); }
                else { p.push_back(contract_or_feature_last); p.push_back(other); }
                return p;
            };
            std::vector<int64_t> qp = perm_of(d1.lb, d1.lc[0], 4, true);    // q: contract over D, free = Sq
            std::vector<int64_t> kp = perm_of(d1.rb, d1.rc[0], 4, true);    // k: contract over D, free = Sk
            std::vector<int64_t> vp = perm_of(d2.rb, d2.rc[0], 4, false);   // v: contract over Sk, free = D
            // result of the first dot must be [b,h,q,k] (batch dims first is what dot_general produces)
            const int64_t B = qt.shape[qp[0]], H = qt.shape[qp[1]], Sq = qt.shape[qp[2]], D = qt.shape[qp[3]];
            const int64_t Sk = kt.shape[kp[2]];
            if (kt.shape[kp[0]] != B || kt.shape[kp[1]] != H || kt.shape[kp[3]] != D) continue;
            if (vt.shape[vp[0]] != B || vt.shape[vp[1]] != H || vt.shape[vp[2]] != Sk || vt.shape[vp[3]] != D) continue;
            if (pt.shape != std::vector<int64_t>{B, H, Sq, Sk} || ot.shape != std::vector<int64_t>{B, H, Sq, D}) continue;
            if (causal && Sq != Sk) continue;
            auto transposed = [&](int val, const std::vector<int64_t>& perm) {
                bool ident = true;
                for (size_t d = 0; d < perm.size(); ++d) ident &= perm[d] == static_cast<int64_t>(d);
                if (ident) return val;
                Op t;
                t.name = "transpose";
                t.dialect = "stablehlo";
                t.operands = {val};
                t.attrs["permutation"] = Attr::make_ints(perm);
                TensorType tt = g.type(val);
                for (size_t d = 0; d < perm.size(); ++d) tt.shape[d] = g.type(val).shape[perm[d]];
                return f.add_op(t, tt, idx);
            };
            const int root_result = pv.results[0];
            const int q4 = transposed(q, qp);
            const int k4 = transposed(k, kp);
            const int v4 = transposed(v, vp);
            Op* root = nullptr;
            for (Op& cand : f.ops)
                if (!cand.dead && cand.results.size() == 1 && cand.results[0] == root_result) root = &cand;
            std::string cfg = "{\"scale\":" + fmt_double(scale) + ",\"is_causal\":" + (causal ? "true" : "false") +
                              ",\"has_mask\":false,\"num_heads\":" + std::to_string(H) + ",\"head_dim\":" + std::to_string(D) + "}";
            // When the only consumer transposes [B,H,S,D] to [B,S,H,D] (the layout the following reshape + dense layer
            // wants), let the kernel write that layout directly instead of materialising a transposed copy.
            Op* only_user = nullptr;
            int n_users = 0;
            for (Op& cand : f.ops) {
                if (cand.dead) continue;
                for (int v : cand.operands)
                    if (v == root_result) { ++n_users; only_user = &cand; }
            }
            if (n_users == 1 && only_user->name == "transpose" && only_user->int_list("permutation") == std::vector<int64_t>{0, 2, 1, 3}) {
                cfg.insert(cfg.size() - 1, ",\"output_layout\":\"BSHD\"");
                make_custom_call(*only_user, "fused_scaled_dot_product_attention", {q4, k4, v4}, cfg);
                root->dead = true;
            } else {
                make_custom_call(*root, "fused_scaled_dot_product_attention", {q4, k4, v4}, cfg);
            }
            changed = true;
        }
        if (!changed) break;
        any = true;
        dce(f);
    }
    return any;
}

// ---- matmul + bias + activation -------------------------------------------------------------------------------------------

// act(dot(x, w) + bcast(bias)) with w rank 2 contracting its first dim and x contracting its last.
// Reference: PassManager.swift:1436-1570 (which always records activation "none"); here the activation found in the
// graph is recorded.
bool fuse_matmul_bias_act(Function& f) {
    bool any = false;
    for (;;) {
        Graph g(f);
        bool changed = false;
        for (size_t idx = f.ops.size(); idx-- > 0 && !changed;) {
            Op& o = f.ops[idx];
            if (o.dead || o.results.size() != 1) continue;
            const TensorType& rt = o.result_types[0];
            if (!is_float(rt.dtype) || rt.dtype == DType::F64) continue;
            std::string act = "none";
            int v = o.results[0];
            const Op* cur = &o;
            if (cur->name == "custom_call") {
                const std::string t = cur->str_attr("call_target_name");
                if (t == "fused_gelu") act = json_bool(cur->str_attr("backend_config"), "approximate", true) ? "gelu_tanh" : "gelu_erf";
                else if (t == "fused_silu") act = "silu";
                else if (t == "fused_relu") act = "relu";
                else continue;
                v = cur->operands[0];
            } else if (cur->name == "tanh" || cur->name == "logistic") {
                act = cur->name == "tanh" ? "tanh" : "sigmoid";
                v = cur->operands[0];
            } else if (cur->name == "maximum" && (is_splat_value(g, cur->operands[1], 0) || is_splat_value(g, cur->operands[0], 0))) {
                act = "relu";
                v = is_splat_value(g, cur->operands[1], 0) ? cur->operands[0] : cur->operands[1];
            } else if (cur->name != "add") {
                continue;
            }
            if (act != "none" && g.n_users(v) != 1) continue;
            const Op* add = g.def(v);
            int bias = -1, dot_v = -1;
            if (add && add->name == "add") {
                for (int s = 0; s < 2; ++s) {
                    int b = vector_over_last_axis(g, add->operands[1 - s], rt);
                    if (b >= 0 && g.is(add->operands[s], "dot_general")) { bias = b; dot_v = add->operands[s]; }
                    else if (b >= 0 && g.is(add->operands[s], "dot")) { bias = b; dot_v = add->operands[s]; }
                }
                if (dot_v < 0) continue;
                if (g.n_users(dot_v) != 1) continue;
            } else if (act != "none" && add && (add->name == "dot_general" || add->name == "dot")) {
                dot_v = v;
            } else {
                continue;
            }
            const Op* dot = g.def(dot_v);
            const int x = dot->operands[0], w = dot->operands[1];
            const TensorType &xt = g.type(x), &wt = g.type(w);
            if (wt.rank() != 2 || xt.rank() < 1) continue;
            if (dot->name == "dot_general") {
                DotDims d = dot_dims(*dot);
                if (!d.lb.empty() || !d.rb.empty() || d.lc != std::vector<int64_t>{xt.rank() - 1} || d.rc != std::vector<int64_t>{0}) continue;
            } else if (xt.rank() > 2) continue;
            std::vector<int> operands = {x, w};
            if (bias >= 0) operands.push_back(bias);
            make_custom_call(o, "fused_matmul_bias_activation", operands,
                             "{\"activation\":\"" + act + "\",\"has_bias\":" + (bias >= 0 ? "true" : "false") + "}");
            changed = true;
        }
        if (!changed) break;
        any = true;
        dce(f);
    }
    return any;
}

// Residual add behind a projection: s = add(r, y) with y = fused_matmul_bias_activation(x, w[, bias]) without activation
// and no other user. The sum moves into the product's epilogue,
//   s = custom_call @fused_matmul_bias_activation(x, w[, bias], r) {has_residual}
// which adds r before the one rounding to the result type, so y is never written or read back. The fused op takes the
// place of the add, where r and the product's operands are all defined. Part of "residual-chain-fusion", which the
// reference registers without an implementation (Compiler/PassManager.swift:214-221).
bool fuse_matmul_residual(Function& f) {
    Graph g(f);
    bool changed = false;
    for (size_t idx = 0; idx < f.ops.size(); ++idx) {
        Op& o = f.ops[idx];
        if (o.dead || o.name != "add" || o.operands.size() != 2 || o.results.size() != 1) continue;
        const TensorType st = o.result_types[0];
        if (!is_float(st.dtype) || st.dtype == DType::F64) continue;
        for (int side = 0; side < 2; ++side) {
            const int y = o.operands[side], r = o.operands[1 - side];
            Op* mm = g.def_mut(y);
            if (!mm || mm->dead || mm->results.size() != 1 || y == r) continue;
            if (g.n_users(y) != 1 || !(g.type(y) == st) || !(g.type(r) == st)) continue;
            std::string cfg;
            if (mm->name == "custom_call") {
                if (mm->str_attr("call_target_name") != "fused_matmul_bias_activation") continue;
                cfg = mm->str_attr("backend_config");
                if (cfg.find("\"activation\":\"none\"") == std::string::npos || cfg.find("has_residual") != std::string::npos) continue;
            } else if (mm->name == "dot_general" || mm->name == "dot") {
                // a bare product x [.., K] . w [K, N], the form matmul-bias-act-fusion takes when a bias or activation follows
                if (mm->operands.size() != 2) continue;
                const TensorType &xt = g.type(mm->operands[0]), &wt = g.type(mm->operands[1]);
                if (wt.rank() != 2 || xt.rank() < 1) continue;
                if (mm->name == "dot_general") {
                    DotDims d = dot_dims(*mm);
                    if (!d.lb.empty() || !d.rb.empty() || d.lc != std::vector<int64_t>{xt.rank() - 1} || d.rc != std::vector<int64_t>{0}) continue;
                } else if (xt.rank() > 2) continue;
                cfg = "{\"activation\":\"none\",\"has_bias\":false}";
            } else {
                continue;
            }
            std::vector<int> operands = mm->operands;
            operands.push_back(r);
            std::string fused_cfg = cfg;
            fused_cfg.insert(fused_cfg.rfind('}'), ",\"has_residual\":true");
            make_custom_call(o, "fused_matmul_bias_activation", operands, fused_cfg);
            mm->dead = true;
            mm->results.clear();
            changed = true;
            break;
        }
    }
    if (changed) f.compact();
    return changed;
}

// convolution -> add(broadcast_in_dim(bias)) -> optional relu / sigmoid / tanh / silu becomes
//   custom_call @fused_conv_bias_act(x, w, bias) {the convolution's attributes, activation, has_bias}
// as in the reference (detector Compiler/Analyzer.swift:405-495, rewrite Compiler/PassManager.swift:1325-1410). The bias is one
// value per output feature; the convolution and the sum have no other user. Here the fused call saves the separate
// elementwise step: bias and activation ride in the epilogue of the convolution's product.
bool fuse_conv_bias_act(Function& f) {
    Graph g(f);
    bool changed = false;
    for (size_t idx = 0; idx < f.ops.size(); ++idx) {
        Op& conv = f.ops[idx];
        if (conv.dead || conv.name != "convolution" || conv.results.size() != 1 || conv.operands.size() != 2) continue;
        const int y = conv.results[0];
        const TensorType yt = conv.result_types[0];
        if (!is_float(yt.dtype) || g.n_users(y) != 1) continue;
        Op* add = nullptr;
        for (int u : g.users[y]) add = &f.ops[static_cast<size_t>(u)];
        if (!add || add->dead || add->name != "add" || add->operands.size() != 2 || add->results.size() != 1) continue;
        const int bcast_v = add->operands[0] == y ? add->operands[1] : add->operands[0];
        if (bcast_v == y) continue;
        const Op* bc = g.def(bcast_v);
        if (!bc || bc->name != "broadcast_in_dim" || bc->operands.size() != 1) continue;
        const int64_t ofd = conv.int_attr("output_feature_dimension", yt.rank() - 1);
        const TensorType& bt = g.type(bc->operands[0]);
        if (bt.rank() != 1 || bt.dtype != yt.dtype || bc->int_list("broadcast_dimensions") != std::vector<int64_t>{ofd} ||
            bt.shape[0] != yt.shape[static_cast<size_t>(ofd)] || !(bc->result_types[0] == yt))
            continue;
        Op* root = add;
        std::string act = "none";
        const int s = add->results[0];
        if (g.n_users(s) == 1) {
            Op* a = nullptr;
            for (int u : g.users[s]) a = &f.ops[static_cast<size_t>(u)];
            if (a && !a->dead && a->results.size() == 1 && a->result_types[0] == yt) {
                double zero = 1.0;
                if (a->name == "maximum" && a->operands.size() == 2) {
                    const int other = a->operands[0] == s ? a->operands[1] : a->operands[0];
                    if (other != s && scalar_constant(g, other, &zero) && zero == 0.0) { act = "relu"; root = a; }
                } else if (a->name == "logistic") { act = "sigmoid"; root = a; }
                else if (a->name == "tanh") { act = "tanh"; root = a; }
                else if (a->name == "custom_call" && a->operands.size() == 1 &&
                         (a->str_attr("call_target_name") == "fused_silu" || a->str_attr("call_target_name") == "fused_relu")) {
                    act = a->str_attr("call_target_name") == "fused_silu" ? "silu" : "relu";
                    root = a;
                }
            }
        }
        const std::map<std::string, Attr> conv_attrs = conv.attrs;
        make_custom_call(*root, "fused_conv_bias_act", {conv.operands[0], conv.operands[1], bc->operands[0]},
                         "{\"activation\":\"" + act + "\",\"has_bias\":true}");
        for (const auto& kv : conv_attrs) root->attrs[kv.first] = kv.second;
        if (root != add) { add->dead = true; add->results.clear(); }
        conv.dead = true;
        conv.results.clear();
        changed = true;
    }
    if (changed) {
        f.compact();
        dce(f);
    }
    return changed;
}

// ---- producer-consumer fusion of elementwise chains -----------------------------------------------------------------------

bool fusable_elementwise(const Op& o) {
    static const char* names[] = {"add", "subtract", "multiply", "divide", "maximum", "minimum", "negate", "abs", "exponential",
                                  "log", "sqrt", "rsqrt", "tanh", "logistic", "sine", "cosine", "floor", "ceil", "sign",
                                  "exponential_minus_one", "log_plus_one", "power", "select", "clamp", "compare", "convert"};
    if (o.results.size() != 1) return false;
    if (o.name == "compare" && o.str_attr("compare_type") == "TOTALORDER") return false;  // lowered on the bit patterns
    for (const char* n : names)
        if (o.name == n) return true;
    return false;
}

// Greedy: an elementwise op whose only user is another elementwise op of the same shape is folded into that user;
// chains become one fused_elementwise custom call carrying an instruction list for the device interpreter.
// Reference: Sources/MetalHLOCore/Optimizer/ProducerConsumerFusion.swift:86-589 (linear chains, <= 50 ops).
bool fuse_producer_consumer(Function& f) {
    Graph g(f);
    bool changed = false;
    std::vector<bool> absorbed(f.ops.size(), false);
    for (size_t idx = f.ops.size(); idx-- > 0;) {
        Op& root = f.ops[idx];
        if (root.dead || absorbed[idx] || !fusable_elementwise(root)) continue;
        const TensorType& rt = root.result_types[0];
        if (rt.dtype == DType::F64) continue;
        // grow the set of ops computed inside the kernel: single-use producers with the root's shape
        std::vector<int> members = {static_cast<int>(idx)};
        std::vector<int> inputs;  // external values, in first-use order
        bool grew = true;
        while (grew && members.size() < MHLO_CUDA_EW_MAX_INSTS - 2) {
            grew = false;
            for (size_t mi = 0; mi < members.size() && !grew; ++mi) {
                for (int v : f.ops[members[mi]].operands) {
                    const int d = g.def_index(v);
                    if (d < 0 || f.ops[d].dead || absorbed[d]) continue;
                    if (std::find(members.begin(), members.end(), d) != members.end()) continue;
                    const Op& p = f.ops[d];
                    if (!fusable_elementwise(p) || g.n_users(v) != 1) continue;
                    if (p.result_types[0].shape != rt.shape) continue;
                    // do not mix integer arithmetic into a float-domain program (see mhlo_cuda_elementwise)
                    const bool p_int = !is_float(p.result_types[0].dtype) && p.name != "compare";
                    if (p_int && is_float(rt.dtype) && p.name != "convert") continue;
                    members.push_back(d);
                    grew = true;
                    break;
                }
            }
        }
        if (members.size() < 2) continue;
        std::sort(members.begin(), members.end());
        // count distinct external inputs
        for (int m : members)
            for (int v : f.ops[m].operands) {
                const int d = g.def_index(v);
                const bool internal = d >= 0 && std::find(members.begin(), members.end(), d) != members.end();
                if (!internal && std::find(inputs.begin(), inputs.end(), v) == inputs.end()) inputs.push_back(v);
            }
        if (inputs.size() > MHLO_CUDA_EW_MAX_INPUTS) continue;
        // operands must already have the output shape or be scalars (the kernel broadcasts by stride 0)
        bool shapes_ok = true;
        for (int v : inputs) shapes_ok &= g.type(v).shape == rt.shape || g.type(v).count() == 1;
        if (!shapes_ok) continue;
        std::map<int, int> reg;  // value id -> register
        for (size_t i = 0; i < inputs.size(); ++i) reg[inputs[i]] = static_cast<int>(i);
        Attr prog;
        prog.kind = Attr::Array;
        std::string names;
        int next = static_cast<int>(inputs.size());
        bool ok = true;
        for (int m : members) {
            const Op& p = f.ops[m];
            int code = elementwise_opcode(p.name);
            if (p.name == "compare") {
                static const std::map<std::string, int> dir = {{"EQ", MHLO_EW_CMP_EQ}, {"NE", MHLO_EW_CMP_NE}, {"LT", MHLO_EW_CMP_LT},
                                                               {"LE", MHLO_EW_CMP_LE}, {"GT", MHLO_EW_CMP_GT}, {"GE", MHLO_EW_CMP_GE}};
                auto it = dir.find(p.str_attr("comparison_direction"));
                code = it == dir.end() ? -1 : it->second;
            }
            if (code < 0) { ok = false; break; }
            auto r = [&](size_t k) { return k < p.operands.size() ? reg[p.operands[k]] : 0; };
            auto push = [&](int op, int a, int b, int c, double imm) {
                Attr inst;
                inst.kind = Attr::Array;
                inst.elems = {Attr::make_int(op), Attr::make_int(a), Attr::make_int(b), Attr::make_int(c), Attr::make_float(imm)};
                prog.elems.push_back(inst);
                return next++;
            };
            int res = push(code, r(0), r(1), r(2), 0.0);
            // keep the rounding point an unfused f16/bf16 op would have had
            const DType pd = p.result_types[0].dtype;
            if (m != members.back() && (pd == DType::F16 || pd == DType::BF16))
                res = push(MHLO_EW_ROUND_TO, res, res, res, static_cast<double>(static_cast<int>(pd)));
            reg[p.results[0]] = res;
            names += (names.empty() ? "\"" : ",\"") + p.name + "\"";
        }
        if (!ok || prog.elems.size() > MHLO_CUDA_EW_MAX_INSTS) continue;
        for (int m : members)
            if (m != static_cast<int>(idx)) absorbed[m] = true;
        make_custom_call(root, "fused_elementwise", inputs,
                         "{\"operations\":[" + names + "],\"num_ops\":" + std::to_string(members.size()) + "}");
        root.attrs["_program"] = prog;
        changed = true;
    }
    if (changed) dce(f);
    return changed;
}

// ---- layout ------------------------------------------------------------------------------------------------------------------

// Rewrites every dot_general so that lhs = [batch.., free.., contracting..] and rhs = [batch.., contracting.., free..]
// by inserting transposes (Sources/MetalHLOCore/Optimizer/Canonicalizers.swift:903-1091). In this backend a
// transpose is a strided view, so the canonical form costs nothing at run time.
bool canonicalize_dot_layout(Function& f) {
    bool any = false;
    for (size_t idx = 0; idx < f.ops.size(); ++idx) {
        if (f.ops[idx].dead || f.ops[idx].name != "dot_general") continue;
        const int result = f.ops[idx].results[0];
        DotDims d = dot_dims(f.ops[idx]);
        const int lhs = f.ops[idx].operands[0], rhs = f.ops[idx].operands[1];
        const TensorType lt = f.type_of(lhs), rt = f.type_of(rhs);
        auto rest = [](int rank, const std::vector<int64_t>& x, const std::vector<int64_t>& y) {
            std::vector<int64_t> r;
            for (int k = 0; k < rank; ++k)
                if (std::find(x.begin(), x.end(), k) == x.end() && std::find(y.begin(), y.end(), k) == y.end()) r.push_back(k);
            return r;
        };
        std::vector<int64_t> lf = rest(lt.rank(), d.lb, d.lc), rf = rest(rt.rank(), d.rb, d.rc);
        std::vector<int64_t> lp = d.lb, rp = d.rb;
        lp.insert(lp.end(), lf.begin(), lf.end());
        lp.insert(lp.end(), d.lc.begin(), d.lc.end());
        rp.insert(rp.end(), d.rc.begin(), d.rc.end());
        rp.insert(rp.end(), rf.begin(), rf.end());
        auto ident = [](const std::vector<int64_t>& p) { for (size_t k = 0; k < p.size(); ++k) if (p[k] != static_cast<int64_t>(k)) return false; return true; };
        if (ident(lp) && ident(rp)) continue;
        size_t at = idx;
        auto transposed = [&](int val, const std::vector<int64_t>& perm) {
            if (ident(perm)) return val;
            Op t;
            t.name = "transpose";
            t.dialect = "stablehlo";
            t.operands = {val};
            t.attrs["permutation"] = Attr::make_ints(perm);
            TensorType src = f.type_of(val), tt = src;
            for (size_t k = 0; k < perm.size(); ++k) tt.shape[k] = src.shape[perm[k]];
            int v = f.add_op(t, tt, at);
            ++at;
            return v;
        };
        const int nl = transposed(lhs, lp), nr = transposed(rhs, rp);
        Op* dot = nullptr;
        for (Op& c : f.ops) if (!c.dead && c.results.size() == 1 && c.results[0] == result) dot = &c;
        const int nb = static_cast<int>(d.lb.size()), nlf = static_cast<int>(lf.size()), nc = static_cast<int>(d.lc.size());
        std::vector<int64_t> b, lc, rc;
        for (int k = 0; k < nb; ++k) b.push_back(k);
        for (int k = 0; k < nc; ++k) { lc.push_back(nb + nlf + k); rc.push_back(nb + k); }
        dot->operands = {nl, nr};
        dot->attrs["lhs_batching_dimensions"] = Attr::make_ints(b);
        dot->attrs["rhs_batching_dimensions"] = Attr::make_ints(b);
        dot->attrs["lhs_contracting_dimensions"] = Attr::make_ints(lc);
        dot->attrs["rhs_contracting_dimensions"] = Attr::make_ints(rc);
        for (const char* k : {"dot_dimension_numbers", "batching_dims.lhs", "batching_dims.rhs", "contracting_dims.lhs", "contracting_dims.rhs"}) dot->attrs.erase(k);
        idx = at;
        any = true;
    }
    return any;
}

// Greedy list schedule: among the ops whose operands are ready, run the one with the most operand bytes first
// (Sources/MetalHLOCore/Compiler/PassManager.swift:1645-1724), ties by original position.
bool schedule_memory_aware(Function& f) {
    f.compact();
    const size_t n = f.ops.size();
    if (n < 3) return false;
    std::vector<int> pending(n, 0);
    std::vector<std::vector<int>> consumers(n);
    for (size_t i = 0; i < n; ++i) {
        std::set<int> deps;
        std::function<void(const Op&)> collect = [&](const Op& o) {
            for (int v : o.operands) { const int d = f.values[v].def_op; if (d >= 0 && d != static_cast<int>(i)) deps.insert(d); }
            for (const auto& r : o.regions) for (const Op& q : r->ops) collect(q);
        };
        collect(f.ops[i]);
        pending[i] = static_cast<int>(deps.size());
        for (int d : deps) consumers[d].push_back(static_cast<int>(i));
    }
    std::vector<int> order;
    std::vector<bool> done(n, false);
    std::vector<int> ready;
    for (size_t i = 0; i + 1 < n; ++i) if (pending[i] == 0) ready.push_back(static_cast<int>(i));
    auto weight = [&](int i) { int64_t b = 0; for (int v : f.ops[i].operands) b += f.values[v].type.bytes(); return b; };
    while (!ready.empty()) {
        size_t best = 0;
        for (size_t k = 1; k < ready.size(); ++k) {
            const int64_t wb = weight(ready[best]), wk = weight(ready[k]);
            if (wk > wb || (wk == wb && ready[k] < ready[best])) best = k;
        }
        const int i = ready[best];
        ready.erase(ready.begin() + static_cast<long>(best));
        order.push_back(i);
        done[i] = true;
        for (int c : consumers[i]) if (--pending[c] == 0 && c != static_cast<int>(n) - 1) ready.push_back(c);
    }
    if (order.size() != n - 1) return false;  // cycle or region dependency we do not model: keep program order
    bool moved = false;
    for (size_t k = 0; k < order.size(); ++k) moved |= order[k] != static_cast<int>(k);
    if (!moved) return false;
    std::vector<Op> ops;
    for (int i : order) ops.push_back(std::move(f.ops[i]));
    ops.push_back(std::move(f.ops[n - 1]));
    f.ops.swap(ops);
    f.compact();
    return true;
}

struct PassDef {
    const char* name;
    std::function<bool(Function&)> run;
};

const std::vector<PassDef>& registry() {
    static const std::vector<PassDef> passes = {
        // phase 1: simplification
        {"constant-folding", [](Function& f) { return algebraic_simplify(f, 1); }},
        {"algebraic-simplifier", [](Function& f) { return algebraic_simplify(f, 10); }},
        {"dead-code-elimination", dce},
        {"common-subexpr-elim", cse},
        // phase 2: canonicalisation
        {"reshape-canonicalizer", canonicalize_reshape},
        {"transpose-canonicalizer", canonicalize_transpose},
        {"broadcast-canonicalizer", canonicalize_broadcast},
        // phase 3: pattern fusion
        {"transformer-block-fusion", [](Function&) { return false; }},  // a no-op in the reference as well
        {"attention-fusion", fuse_attention},
        {"ffn-fusion", [](Function&) { return false; }},  // the reference's FFN rewrite drops biases; the matmul+bias+act fusion covers the chain
        {"norm-fusion", fuse_norm},
        {"batch-norm-fusion", [](Function&) { return false; }},  // CNN-only pattern, outside this backend's surface
        {"gelu-fusion", fuse_activations},
        {"softmax-fusion", fuse_softmax},
        {"matmul-bias-act-fusion", fuse_matmul_bias_act},
        {"conv-bias-act-fusion", fuse_conv_bias_act},
        // phase 4: generic fusion
        {"producer-consumer-fusion", fuse_producer_consumer},
        {"sibling-fusion", [](Function&) { return false; }},            // analysis-only in the reference
        {"elementwise-chain-fusion", [](Function&) { return false; }},  // no-op in the reference
        // phase 5: cross-layer
        {"cross-layer-fusion", [](Function&) { return false; }},
        {"residual-chain-fusion", [](Function& f) {
             // norms first: reading both addends in the norm kernel measured cheaper than reading the residual in the product's
             // epilogue (GPT-2-small layer products: +16 us per product against 4 us saved per norm); a product takes the sums
             // that feed no norm, where the alternative is an elementwise pass of its own
             const bool norms = fuse_residual_norm(f);
             const bool products = fuse_matmul_residual(f);
             return products || norms;
         }},
        // phase 6: layout
        {"layout-assignment", [](Function&) { return false; }},  // analysis-only in the reference
        {"transpose-folding", canonicalize_transpose},
        {"copy-elimination", [](Function& f) {
             Graph g(f);
             bool changed = false;
             for (Op& o : f.ops)
                 if (!o.dead && (o.name == "copy" || o.name == "optimization_barrier") && o.results.size() == 1 && o.operands.size() == 1) {
                     replace_uses(f, o.results[0], o.operands[0]);
                     o.dead = true;
                     changed = true;
                 }
             if (changed) f.compact();
             return changed;
         }},
        // phase 7: scheduling
        {"memory-aware-scheduler", schedule_memory_aware},
        // phase 8: cleanup
        {"dot-general-layout-canonicalize", canonicalize_dot_layout},
        {"final-dce", dce},
    };
    return passes;
}

}  // namespace

const std::vector<std::string>& all_pass_names() {
    static std::vector<std::string> names;
    if (names.empty())
        for (const PassDef& p : registry()) names.push_back(p.name);
    return names;
}

std::set<std::string> passes_for_level(int level) {
    std::set<std::string> s;
    if (level <= 0) return s;
    s = {"constant-folding", "algebraic-simplifier", "dead-code-elimination", "dot-general-layout-canonicalize"};
    if (level == 1) return s;
    for (const char* p : {"common-subexpr-elim", "reshape-canonicalizer", "transpose-canonicalizer", "broadcast-canonicalizer",
                          "producer-consumer-fusion", "batch-norm-fusion", "final-dce"})
        s.insert(p);
    if (level == 2) return s;
    for (const std::string& p : all_pass_names()) s.insert(p);
    return s;
}

std::vector<PassRecord> run_pass_pipeline(Function& f, const CompileOptions& options) {
    std::set<std::string> enabled = options.has_enabled_set ? options.enabled_passes : passes_for_level(options.opt_level);
    for (const std::string& d : options.disabled_passes) enabled.erase(d);
    if (const char* env = std::getenv("METALHLO_DISABLED_PASSES")) {
        std::stringstream ss(env);
        std::string tok;
        while (std::getline(ss, tok, ',')) enabled.erase(tok);
    }
    const bool debug = std::getenv("METALHLO_DEBUG_PASSES") != nullptr;
    std::vector<PassRecord> log;
    for (const PassDef& p : registry()) {
        PassRecord r;
        r.name = p.name;
        r.ops_before = count_live(f);
        if (enabled.count(p.name)) {
            r.ran = true;
            r.changed = p.run(f);
            f.compact();
        }
        r.ops_after = count_live(f);
        if (debug && r.ran) fprintf(stderr, "[metalhlo] pass %-34s %s ops %d -> %d\n", p.name, r.changed ? "changed" : "no-op  ", r.ops_before, r.ops_after);
        log.push_back(r);
    }
    return log;
}

}  // namespace mhlo
