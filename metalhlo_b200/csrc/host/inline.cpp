// Flattening of the module a jitted JAX function lowers to: `call`s of private functions are inlined into @main and
// `stablehlo.while` loops with a static trip count (what lax.fori_loop emits) are unrolled, so that the straight-line
// executor can run them. The reference does both on the module text before compiling
// (Sources/PJRTMetalHLO/PJRTExecutable.swift:458-1657: inlineSimpleCallWrapper, inlineCallsInBody,
// unrollStaticWhileLoops, iterated until nothing changes); here they work on the parsed IR. `stablehlo.if` and
// `stablehlo.case` become straight-line code too: every branch is computed and the results are picked with `select`,
// which is exact because StableHLO ops have no side effects (the reference runs them through MPSGraph's if/else,
// Sources/MetalHLOCore/MPSGraph/MPSGraphCompiler.swift, with the same results).
#include <cmath>
#include <functional>
#include <map>

#include "compiler.h"
#include "numeric.h"

namespace mhlo {

int elementwise_opcode(const std::string& name);  // executable.cpp

namespace {

constexpr int kMaxInlineRounds = 64;     // nesting depth of calls
constexpr int64_t kMaxTripCount = 4096;  // loops longer than this stay loops (and are rejected by the executor)
constexpr size_t kMaxUnrolledOps = 2000000;

// Copies ops from `src` into `dst`, giving every value they define a fresh id in dst. Values that are not in the map
// are taken to be visible at the destination as they are (only valid when src and dst are the same function).
struct Cloner {
    Function& dst;
    const Function& src;
    bool same_function;
    std::map<int, int> map;

    int remap(int v) const {
        auto it = map.find(v);
        if (it != map.end()) return it->second;
        if (!same_function) fail_compile("internal: value " + src.values[v].name + " of an inlined function has no definition at the call site");
        return v;
    }
    int fresh(int v) {
        const int nv = dst.new_value(src.values[v].type, src.values[v].name);
        map[v] = nv;
        return nv;
    }
    Op clone(const Op& o) {
        Op c = o;
        for (int& v : c.operands) v = remap(v);
        c.regions.clear();
        for (const auto& r : o.regions) {
            auto nr = std::make_shared<Region>();
            for (int a : r->args) nr->args.push_back(fresh(a));
            for (const Op& ro : r->ops) nr->ops.push_back(clone(ro));
            c.regions.push_back(nr);
        }
        for (int& v : c.results) v = fresh(v);
        return c;
    }
};

void apply_alias(Op& o, const std::map<int, int>& alias) {
    if (alias.empty()) return;
    for (int& v : o.operands) {
        for (auto it = alias.find(v); it != alias.end(); it = alias.find(v)) v = it->second;
    }
    for (auto& r : o.regions)
        for (Op& ro : r->ops) apply_alias(ro, alias);
}

const Function* find_function(const Module& m, const std::string& name) {
    for (const Function& f : m.functions)
        if (f.name == name) return &f;
    return nullptr;
}

// ---- while analysis -------------------------------------------------------------------------------------------------

const Op* def_in(const std::vector<Op>& ops, int v) {
    for (const Op& o : ops)
        for (int r : o.results)
            if (r == v) return &o;
    return nullptr;
}

// Scalar integer constant defined in `inner` (a region) or among the top-level ops `outer`.
bool int_constant(const std::vector<Op>& outer, const std::vector<Op>& inner, int v, int64_t* out) {
    const Op* o = def_in(inner, v);
    if (!o) o = def_in(outer, v);
    if (!o || o->name != "constant") return false;
    const Attr* a = o->attr("value");
    if (!a || a->kind != Attr::Dense || o->result_types.empty()) return false;
    const TensorType& t = o->result_types[0];  // the payload is stored in the result's element type
    if (t.count() != 1 || is_float(t.dtype) || t.dtype == DType::I1) return false;
    const size_t es = dtype_size(t.dtype);
    if (a->dense.size() < es || es > 8) return false;
    uint64_t raw = 0;
    for (size_t i = 0; i < es; ++i) raw |= static_cast<uint64_t>(a->dense[i]) << (8 * i);
    if (!is_unsigned(t.dtype) && es < 8 && (raw >> (8 * es - 1)) & 1) raw |= ~0ull << (8 * es);  // sign-extend
    *out = static_cast<int64_t>(raw);
    return true;
}

struct LoopShape {
    int counter = -1;  // index of the iteration argument that counts
    int64_t init = 0, limit = 0, step = 0;
    std::string direction;
    int64_t trips = 0;
};

bool compare(const std::string& dir, int64_t a, int64_t b) {
    if (dir == "LT") return a < b;
    if (dir == "LE") return a <= b;
    if (dir == "GT") return a > b;
    if (dir == "GE") return a >= b;
    if (dir == "NE") return a != b;
    return false;
}

// cond: return(compare(dir, iter_k, const)); body: result_k = add/subtract(iter_k, const); init_k constant.
// `f` = the top-level ops that precede the loop.
bool analyse_loop(const std::vector<Op>& f, const Op& w, LoopShape* shape) {
    if (w.regions.size() != 2) return false;
    const Region& cond = *w.regions[0];
    const Region& body = *w.regions[1];
    if (cond.ops.empty() || body.ops.empty() || cond.ops.back().name != "return" || body.ops.back().name != "return") return false;
    if (cond.ops.back().operands.size() != 1 || body.ops.back().operands.size() != w.operands.size()) return false;
    const Op* cmp = def_in(cond.ops, cond.ops.back().operands[0]);
    if (!cmp || cmp->name != "compare" || cmp->operands.size() != 2) return false;
    std::string dir = cmp->str_attr("comparison_direction");
    int k = -1;
    int64_t limit = 0;
    for (int side = 0; side < 2 && k < 0; ++side) {
        for (size_t i = 0; i < cond.args.size(); ++i)
            if (cmp->operands[side] == cond.args[i] && int_constant(f, cond.ops, cmp->operands[1 - side], &limit)) {
                k = static_cast<int>(i);
                if (side == 1) {  // const <dir> iter  ==  iter <mirrored dir> const
                    if (dir == "LT") dir = "GT"; else if (dir == "LE") dir = "GE"; else if (dir == "GT") dir = "LT"; else if (dir == "GE") dir = "LE";
                }
                break;
            }
    }
    if (k < 0) return false;
    const Op* upd = def_in(body.ops, body.ops.back().operands[static_cast<size_t>(k)]);
    if (!upd || (upd->name != "add" && upd->name != "subtract") || upd->operands.size() != 2) return false;
    int64_t step = 0;
    if (upd->operands[0] == body.args[static_cast<size_t>(k)] && int_constant(f, body.ops, upd->operands[1], &step)) {
        if (upd->name == "subtract") step = -step;
    } else if (upd->name == "add" && upd->operands[1] == body.args[static_cast<size_t>(k)] && int_constant(f, body.ops, upd->operands[0], &step)) {
    } else {
        return false;
    }
    int64_t init = 0;
    if (step == 0 || !int_constant(f, {}, w.operands[static_cast<size_t>(k)], &init)) return false;
    int64_t trips = 0;
    for (int64_t i = init; compare(dir, i, limit); i += step)
        if (++trips > kMaxTripCount) return false;
    shape->counter = k;
    shape->init = init;
    shape->limit = limit;
    shape->step = step;
    shape->direction = dir;
    shape->trips = trips;
    return true;
}

}  // namespace

bool inline_calls(Module& m) {
    Function& main = m.main();
    bool changed = false;
    for (int round = 0; round < kMaxInlineRounds; ++round) {
        bool any = false;
        std::vector<Op> out;
        std::map<int, int> alias;  // results of removed calls -> the values that replace them
        for (Op& op : main.ops) {
            apply_alias(op, alias);
            // stablehlo.composite names the private function that implements it: it is a call of that function
            const bool composite = !op.dead && op.name == "composite" && op.attr("decomposition");
            if (op.dead || (op.name != "call" && !composite)) {
                out.push_back(std::move(op));
                continue;
            }
            std::string callee_name = composite ? op.str_attr("decomposition") : op.str_attr("callee");
            if (!callee_name.empty() && callee_name[0] == '@') callee_name.erase(0, 1);
            const Function* callee = find_function(m, callee_name);
            if (!callee) fail_compile("call to unknown function @" + callee_name);
            if (callee == &main) fail_unsupported("recursive call of @" + callee_name);
            if (callee->args.size() != op.operands.size()) fail_compile("call of @" + callee_name + " with the wrong number of arguments");
            Cloner c{main, *callee, false, {}};
            for (size_t i = 0; i < callee->args.size(); ++i) c.map[callee->args[i]] = op.operands[i];
            for (const Op& co : callee->ops) {
                if (co.dead) continue;
                if (co.name == "return") {
                    if (co.operands.size() != op.results.size()) fail_compile("call of @" + callee_name + " binds the wrong number of results");
                    for (size_t r = 0; r < op.results.size(); ++r) alias[op.results[r]] = c.remap(co.operands[r]);
                    break;
                }
                out.push_back(c.clone(co));
            }
            any = true;
        }
        main.ops.swap(out);
        main.compact();
        if (!any) break;
        changed = true;
        if (round + 1 == kMaxInlineRounds) fail_unsupported("calls nested deeper than " + std::to_string(kMaxInlineRounds));
    }
    return changed;
}

bool unroll_static_whiles(Function& f) {
    bool changed = false;
    for (int round = 0; round < kMaxInlineRounds; ++round) {  // an unrolled body may contain further loops
        bool any = false;
        std::vector<Op> out;
        std::map<int, int> alias;
        for (Op& op : f.ops) {
            apply_alias(op, alias);
            LoopShape shape;
            if (op.dead || op.name != "while" || !analyse_loop(out, op, &shape)) {
                out.push_back(std::move(op));
                continue;
            }
            const Region& body = *op.regions[1];
            if (static_cast<size_t>(shape.trips) * body.ops.size() + out.size() > kMaxUnrolledOps)
                fail_unsupported("unrolling a loop of " + std::to_string(shape.trips) + " iterations would exceed " + std::to_string(kMaxUnrolledOps) + " operations");
            std::vector<int> current = op.operands;
            const Op counter_init = *def_in(out, op.operands[static_cast<size_t>(shape.counter)]);  // a scalar integer constant
            for (int64_t t = 0; t < shape.trips; ++t) {
                if (t > 0) {
                    // the counter of iteration t is known: give the body a constant instead of a chain of scalar adds
                    Op k = counter_init;
                    const int64_t value = shape.init + t * shape.step;
                    Attr& payload = k.attrs["value"];
                    const size_t es = dtype_size(k.result_types[0].dtype);
                    payload.dense.assign(es, 0);
                    for (size_t b = 0; b < es; ++b) payload.dense[b] = static_cast<uint8_t>(static_cast<uint64_t>(value) >> (8 * b));
                    payload.splat = true;
                    k.results = {f.new_value(k.result_types[0], "")};
                    current[static_cast<size_t>(shape.counter)] = k.results[0];
                    out.push_back(k);
                }
                Cloner c{f, f, true, {}};
                for (size_t i = 0; i < body.args.size(); ++i) c.map[body.args[i]] = current[i];
                std::vector<int> next = current;
                for (const Op& bo : body.ops) {
                    if (bo.name == "return") {
                        for (size_t i = 0; i < next.size(); ++i) next[i] = c.remap(bo.operands[i]);
                        break;
                    }
                    out.push_back(c.clone(bo));
                }
                current.swap(next);
            }
            for (size_t r = 0; r < op.results.size(); ++r) alias[op.results[r]] = current[r];
            any = true;
        }
        f.ops.swap(out);
        f.compact();
        if (!any) break;
        changed = true;
    }
    return changed;
}

namespace {

Op scalar_constant(Function& f, DType dt, int64_t value) {
    Op k;
    k.name = "constant";
    k.dialect = "stablehlo";
    TensorType t;
    t.dtype = dt;
    Attr a;
    a.kind = Attr::Dense;
    a.dense_type = t;
    a.splat = true;
    const size_t es = dtype_size(dt);
    a.dense.assign(es, 0);
    for (size_t b = 0; b < es && b < 8; ++b) a.dense[b] = static_cast<uint8_t>(static_cast<uint64_t>(value) >> (8 * b));
    k.attrs["value"] = a;
    k.result_types = {t};
    k.results = {f.new_value(t, "")};
    return k;
}

Op simple_op(Function& f, const std::string& name, std::vector<int> operands, const TensorType& rt) {
    Op o;
    o.name = name;
    o.dialect = "stablehlo";
    o.operands = std::move(operands);
    o.result_types = {rt};
    o.results = {f.new_value(rt, "")};
    return o;
}

}  // namespace

bool flatten_conditionals(Function& f) {
    bool changed = false;
    for (int round = 0; round < kMaxInlineRounds; ++round) {  // a branch may hold further conditionals
        bool any = false;
        std::vector<Op> out;
        std::map<int, int> alias;
        for (Op& op : f.ops) {
            apply_alias(op, alias);
            if (op.dead || (op.name != "if" && op.name != "case")) {
                out.push_back(std::move(op));
                continue;
            }
            const bool is_if = op.name == "if";
            if (op.operands.size() != 1 || op.regions.empty() || (is_if && op.regions.size() != 2))
                fail_compile("stablehlo." + op.name + " with " + std::to_string(op.operands.size()) + " operands and " +
                             std::to_string(op.regions.size()) + " branches");
            const TensorType st = f.type_of(op.operands[0]);  // a copy: new values reallocate the table
            if (st.count() != 1) fail_compile("stablehlo." + op.name + ": the selector must be a scalar, got " + st.str());
            std::vector<std::vector<int>> branch_results;
            for (const auto& r : op.regions) {
                Cloner c{f, f, true, {}};
                std::vector<int> res;
                bool returned = false;
                for (const Op& bo : r->ops) {
                    if (bo.name == "return") {
                        for (int v : bo.operands) res.push_back(c.remap(v));
                        returned = true;
                        break;
                    }
                    out.push_back(c.clone(bo));
                }
                if (!returned || res.size() != op.results.size())
                    fail_compile("stablehlo." + op.name + ": a branch returns " + std::to_string(res.size()) + " values for " +
                                 std::to_string(op.results.size()) + " results");
                branch_results.push_back(res);
            }
            TensorType pred_t;
            pred_t.dtype = DType::I1;
            std::vector<int> current = branch_results.back();  // `if`: the false branch; `case`: the default branch
            for (int b = static_cast<int>(branch_results.size()) - 2; b >= 0; --b) {
                int pred = op.operands[0];
                if (!is_if) {
                    Op k = scalar_constant(f, st.dtype, b);
                    Op eq = simple_op(f, "compare", {op.operands[0], k.results[0]}, pred_t);
                    eq.attrs["comparison_direction"] = Attr::make_string("EQ");
                    pred = eq.results[0];
                    out.push_back(k);
                    out.push_back(eq);
                }
                for (size_t r = 0; r < current.size(); ++r) {
                    Op sel = simple_op(f, "select", {pred, branch_results[static_cast<size_t>(b)][r], current[r]}, op.result_types[r]);
                    current[r] = sel.results[0];
                    out.push_back(sel);
                }
            }
            for (size_t r = 0; r < op.results.size(); ++r) alias[op.results[r]] = current[r];
            any = true;
        }
        f.ops.swap(out);
        f.compact();
        if (!any) break;
        changed = true;
    }
    return changed;
}

// stablehlo.map applies a scalar computation to every element: its body becomes the same ops on whole tensors. The
// dimensions attribute must list every dimension in order (the only form the specification allows).
bool flatten_maps(Function& f) {
    bool changed = false;
    for (int round = 0; round < kMaxInlineRounds; ++round) {
        bool any = false;
        std::vector<Op> out;
        std::map<int, int> alias;
        for (Op& op : f.ops) {
            apply_alias(op, alias);
            if (op.dead || op.name != "map") {
                out.push_back(std::move(op));
                continue;
            }
            if (op.regions.size() != 1 || op.results.size() != 1 || op.regions[0]->args.size() != op.operands.size())
                fail_compile("stablehlo.map: one computation with one argument per operand expected");
            const std::vector<int64_t> shape = op.result_types[0].shape;
            const Region& body = *op.regions[0];
            Cloner c{f, f, true, {}};
            for (size_t i = 0; i < body.args.size(); ++i) c.map[body.args[i]] = op.operands[i];
            int result = -1;
            for (const Op& bo : body.ops) {
                if (bo.name == "return") {
                    if (bo.operands.size() != 1) fail_compile("stablehlo.map: the computation must return one value");
                    result = c.remap(bo.operands[0]);
                    break;
                }
                if (!bo.regions.empty()) fail_unsupported("stablehlo.map: nested regions in the computation");
                Op lifted = c.clone(bo);
                // scalars computed from the arguments become tensors of the map's shape; constants stay scalars and
                // broadcast where they are used
                bool from_args = false;
                for (int v : lifted.operands) from_args |= f.values[v].type.shape == shape && !shape.empty();
                if (from_args) {
                    if (elementwise_opcode(lifted.name) < 0 && lifted.name != "compare")
                        fail_unsupported("stablehlo.map: " + lifted.name + " in the computation is not elementwise");
                    for (size_t r = 0; r < lifted.results.size(); ++r) {
                        lifted.result_types[r].shape = shape;
                        f.values[lifted.results[r]].type.shape = shape;
                    }
                }
                out.push_back(lifted);
            }
            if (result < 0) fail_compile("stablehlo.map: the computation does not return");
            if (f.values[result].type.shape != shape) {  // the body ignored its arguments: broadcast the scalar
                Op b = simple_op(f, "broadcast_in_dim", {result}, op.result_types[0]);
                b.attrs["broadcast_dimensions"] = Attr::make_ints({});
                result = b.results[0];
                out.push_back(b);
            }
            alias[op.results[0]] = result;
            any = true;
        }
        f.ops.swap(out);
        f.compact();
        if (!any) break;
        changed = true;
    }
    return changed;
}

// chlo.top_k(x, k): the k largest entries of the last dimension and their positions, ties in index order. Rewritten to
// iota + stable descending sort of (x, iota) + two slices, which the sort kernel and zero-copy slices then run.
// stablehlo.optimization_barrier is the identity on each of its operands (it only fences compiler motion): its results
// are replaced by its operands, whatever their number.
bool drop_optimization_barriers(Function& f) {
    bool changed = false;
    std::vector<Op> out;
    std::map<int, int> alias;
    for (Op& op : f.ops) {
        apply_alias(op, alias);
        if (!op.dead && op.name == "optimization_barrier" && op.results.size() == op.operands.size()) {
            for (size_t i = 0; i < op.results.size(); ++i) alias[op.results[i]] = op.operands[i];
            changed = true;
            continue;
        }
        out.push_back(std::move(op));
    }
    f.ops.swap(out);
    if (changed) f.compact();
    return changed;
}

// stablehlo.tuple / get_tuple_element: a tuple is only a name for a list of values (nested tuples included), so every
// get_tuple_element of a tuple built in the same function is replaced by the member it names and the tuple itself goes
// away once nothing reads it. A tuple that crosses the function's boundary stays and is refused by the lowering: buffers
// of the C API are tensors (Sources/CMetalHLO/include/metalhlo.h).
bool fold_tuples(Function& f) {
    bool any = false;
    for (const Op& op : f.ops) any = any || (!op.dead && (op.name == "tuple" || op.name == "get_tuple_element"));
    if (!any) return false;
    bool changed = false;
    std::map<int, std::vector<int>> members;  // tuple value -> its members
    std::map<int, int> alias;
    std::vector<Op> out;
    for (Op& op : f.ops) {
        apply_alias(op, alias);
        if (!op.dead && op.name == "tuple" && op.results.size() == 1) members[op.results[0]] = op.operands;
        if (!op.dead && op.name == "get_tuple_element" && op.operands.size() == 1 && op.results.size() == 1) {
            const std::vector<int64_t> idx = op.int_list("indices");
            const int64_t k = !idx.empty() ? idx[0] : op.int_attr("index", -1);
            auto it = members.find(op.operands[0]);
            if (it != members.end()) {
                if (k < 0 || k >= static_cast<int64_t>(it->second.size())) fail_compile("get_tuple_element: index " + std::to_string(k) + " outside the tuple");
                alias[op.results[0]] = it->second[static_cast<size_t>(k)];
                changed = true;
                continue;
            }
        }
        out.push_back(std::move(op));
    }
    f.ops.swap(out);
    // tuples nothing reads any more
    const std::vector<std::vector<int>> users = f.users();
    for (size_t i = f.ops.size(); i-- > 0;) {
        Op& op = f.ops[i];
        if (op.name == "tuple" && op.results.size() == 1 && users[static_cast<size_t>(op.results[0])].empty()) {
            bool read_later = false;  // by a tuple that is itself still alive
            for (const Op& other : f.ops)
                if (!other.dead && &other != &op)
                    for (int v : other.operands) read_later = read_later || v == op.results[0];
            if (!read_later) { op.dead = true; changed = true; }
        }
    }
    if (changed) f.compact();
    return changed;
}

bool flatten_top_k(Function& f) {
    bool any = false;
    std::vector<Op> out;
    for (Op& op : f.ops) {
        if (op.dead || op.name != "top_k") {
            out.push_back(std::move(op));
            continue;
        }
        if (op.operands.size() != 1 || op.results.size() != 2) fail_compile("top_k takes one operand and gives values and indices");
        const TensorType xt = f.type_of(op.operands[0]);
        const int rank = xt.rank();
        const int64_t k = op.int_attr("k", -1);
        if (rank < 1 || k < 0 || k > xt.shape.back()) fail_compile("top_k: k out of range for " + xt.str());
        TensorType it = xt;
        it.dtype = op.result_types[1].dtype;
        Op iota = simple_op(f, "iota", {}, it);
        iota.attrs["iota_dimension"] = Attr::make_int(rank - 1);
        Op sort;
        sort.name = "sort";
        sort.dialect = "stablehlo";
        sort.operands = {op.operands[0], iota.results[0]};
        sort.result_types = {xt, it};
        sort.results = {f.new_value(xt, ""), f.new_value(it, "")};
        sort.attrs["dimension"] = Attr::make_int(rank - 1);
        sort.attrs["is_stable"] = Attr::make_bool(true);
        sort.attrs["sort_order"] = Attr::make_string("descending");
        std::vector<int64_t> start(static_cast<size_t>(rank), 0), limit = xt.shape, stride(static_cast<size_t>(rank), 1);
        limit.back() = k;
        out.push_back(iota);
        out.push_back(sort);
        for (int r = 0; r < 2; ++r) {
            Op sl;
            sl.name = "slice";
            sl.dialect = "stablehlo";
            sl.operands = {sort.results[static_cast<size_t>(r)]};
            sl.result_types = {op.result_types[static_cast<size_t>(r)]};
            sl.results = {op.results[static_cast<size_t>(r)]};  // the slices define the top_k's own result values
            sl.attrs["start_indices"] = Attr::make_ints(start);
            sl.attrs["limit_indices"] = Attr::make_ints(limit);
            sl.attrs["strides"] = Attr::make_ints(stride);
            out.push_back(sl);
        }
        any = true;
    }
    f.ops.swap(out);
    f.compact();
    return any;
}

namespace {

// Runs `pass` (which works on f.ops) on the region bodies of the loops that stay loops, innermost included, by letting
// each body stand in for the function's op list while the pass runs.
bool sweep_loop_regions(Function& f, const std::function<bool()>& pass, int depth) {
    bool changed = false;
    std::vector<std::shared_ptr<Region>> regions;
    for (Op& op : f.ops)
        if (!op.dead && op.name == "while")
            for (auto& r : op.regions) regions.push_back(r);
    for (auto& r : regions) {
        std::vector<Op> saved;
        saved.swap(f.ops);
        f.ops.swap(r->ops);
        changed |= pass();
        if (depth < 8) changed |= sweep_loop_regions(f, pass, depth + 1);
        f.ops.swap(r->ops);
        saved.swap(f.ops);
    }
    return changed;
}

}  // namespace

void optimize_loop_bodies(Function& f, const CompileOptions& options) {
    sweep_loop_regions(f, [&]() {
        f.compact();  // link the values to the ops of this body; values from outside count as opaque
        run_pass_pipeline(f, options);
        return false;
    }, 0);
    f.compact();
}

// The reference's custom-call handlers beyond the ones this backend has kernels for, restated as the StableHLO ops their
// MPSGraph bodies compute (Sources/MetalHLOCore/Compiler/CustomCallHandlers.swift): fused_batch_norm (:405-447),
// fused_rope (:715-845), fused_ffn (:848-925), fused_depth_attention (:1075-1135); fused_conv_bias_act is lowered as it is. A module
// that arrives with these targets already in it (written by hand, or by the reference's own passes) then lowers like the
// unfused program; the pass pipeline may fuse the pieces again in this backend's own way.
bool expand_fused_custom_calls(Function& f) {
    bool any = false;
    std::vector<Op> out;
    auto emit = [&](Op o) { const int v = o.results[0]; out.push_back(std::move(o)); return v; };
    auto float_splat = [&](const TensorType& t, double value) {
        Op k;
        k.name = "constant";
        k.dialect = "stablehlo";
        Attr a;
        a.kind = Attr::Dense;
        a.dense_type = t;
        a.splat = true;
        a.dense.assign(dtype_size(t.dtype), 0);
        encode_scalar(t.dtype, value, static_cast<int64_t>(value), a.dense.data());
        k.attrs["value"] = a;
        k.result_types = {t};
        k.results = {f.new_value(t, "")};
        return emit(std::move(k));
    };
    auto unary = [&](const char* name, int x) { return emit(simple_op(f, name, {x}, f.type_of(x))); };
    auto binary = [&](const char* name, int a, int b) { return emit(simple_op(f, name, {a, b}, f.type_of(a))); };
    auto slice_last = [&](int x, int64_t lo, int64_t hi) {
        TensorType t = f.type_of(x);
        std::vector<int64_t> st(t.shape.size(), 0), lim = t.shape, strides(t.shape.size(), 1);
        st.back() = lo;
        lim.back() = hi;
        t.shape.back() = hi - lo;
        Op o = simple_op(f, "slice", {x}, t);
        o.attrs["start_indices"] = Attr::make_ints(st);
        o.attrs["limit_indices"] = Attr::make_ints(lim);
        o.attrs["strides"] = Attr::make_ints(strides);
        return emit(std::move(o));
    };
    // v spread to `to` by the trailing-dimension rule of the reference's graph arithmetic (extents equal or 1)
    auto broadcast_trailing = [&](int v, const TensorType& to, const std::string& what) {
        const TensorType vt = f.type_of(v);
        if (vt.shape == to.shape) return v;
        const int shift = to.rank() - vt.rank();
        if (shift < 0) fail_unsupported(what + ": " + vt.str() + " has more dimensions than " + to.str());
        std::vector<int64_t> dims;
        for (int d = 0; d < vt.rank(); ++d) {
            if (vt.shape[d] != 1 && vt.shape[d] != to.shape[d + shift]) fail_unsupported(what + ": " + vt.str() + " does not spread over " + to.str());
            dims.push_back(d + shift);
        }
        TensorType rt = to;
        rt.dtype = vt.dtype;
        Op o = simple_op(f, "broadcast_in_dim", {v}, rt);
        o.attrs["broadcast_dimensions"] = Attr::make_ints(dims);
        return emit(std::move(o));
    };
    auto matmul_call = [&](int x, int w, const std::string& act, const std::string& what) {
        const TensorType xt = f.type_of(x), wt = f.type_of(w);
        if (wt.rank() != 2 || xt.rank() < 1 || xt.shape.back() != wt.shape[0]) fail_unsupported(what + ": " + xt.str() + " . " + wt.str());
        TensorType rt = xt;
        rt.shape.back() = wt.shape[1];
        Op o = simple_op(f, "custom_call", {x, w}, rt);
        o.attrs["call_target_name"] = Attr::make_string("fused_matmul_bias_activation");
        o.attrs["backend_config"] = Attr::make_string("{\"activation\":\"" + act + "\",\"has_bias\":false}");
        return emit(std::move(o));
    };
    // the last op of an expansion takes the custom call's result value
    auto finish = [&](int v, const Op& call) {
        if (!(f.type_of(v) == call.result_types[0]))
            fail_unsupported("@" + call.str_attr("call_target_name") + ": the operands give " + f.type_of(v).str() + ", the call declares " + call.result_types[0].str());
        Op& last = out.back();
        if (last.results.size() != 1 || last.results[0] != v) {  // the value is an operand passed through: copy it
            Op c = simple_op(f, "copy", {v}, f.type_of(v));
            out.push_back(std::move(c));
        }
        out.back().results = call.results;
    };
    for (Op& op : f.ops) {
        // uniform_quantize(x, scale) = convert(round(x / scale)) and uniform_dequantize(q, scale) = convert(q) * scale: the
        // reference's two-operand forms, scale an ordinary tensor (Compiler/MPSGraphCompiler.swift:3615-3640), not the
        // specification's quantised element types, which neither backend has
        if (!op.dead && (op.name == "uniform_quantize" || op.name == "uniform_dequantize") && op.operands.size() == 2 && op.results.size() == 1) {
            const Op call = op;
            any = true;
            const TensorType rt = call.result_types[0], xt = f.type_of(call.operands[0]);
            if (call.name == "uniform_quantize") {
                if (!is_float(xt.dtype) || is_float(rt.dtype)) fail_unsupported("uniform_quantize from " + xt.str() + " to " + rt.str());
                const int s = broadcast_trailing(call.operands[1], xt, "uniform_quantize");
                int q = unary("round_nearest_even", binary("divide", call.operands[0], s));
                // quantisation saturates at the ends of the storage type (a bare convert of an out-of-range float need not)
                const int bits = static_cast<int>(dtype_size(rt.dtype)) * 8;
                if (rt.dtype != DType::I1 && bits <= 32) {
                    const bool uns = is_unsigned(rt.dtype);
                    double lo = uns ? 0.0 : -std::ldexp(1.0, bits - 1), hi = std::ldexp(1.0, uns ? bits : bits - 1) - 1.0;
                    if (bits == 32) hi = uns ? 4294967040.0 : 2147483520.0;  // the largest floats below 2^32 and 2^31
                    Op cl = simple_op(f, "clamp", {float_splat(xt, lo), q, float_splat(xt, hi)}, xt);
                    q = emit(std::move(cl));
                }
                finish(emit(simple_op(f, "convert", {q}, rt)), call);
            } else {
                if (!is_float(rt.dtype)) fail_unsupported("uniform_dequantize from " + xt.str() + " to " + rt.str());
                const int x = emit(simple_op(f, "convert", {call.operands[0]}, rt));
                finish(binary("multiply", x, broadcast_trailing(call.operands[1], rt, "uniform_dequantize")), call);
            }
            continue;
        }
        const std::string target = !op.dead && op.name == "custom_call" ? op.str_attr("call_target_name") : "";
        if (target != "fused_batch_norm" && target != "fused_rope" && target != "fused_ffn" && target != "fused_depth_attention") {
            out.push_back(std::move(op));
            continue;
        }
        if (op.results.size() != 1) fail_unsupported("@" + target + " gives one result");
        const std::string cfg = op.str_attr("backend_config", "{}");
        const Op call = op;
        any = true;
        if (target == "fused_batch_norm") {
            // (x - mean) / sqrt(variance + eps) * gamma + beta with the statistics along x's last dimension
            if (call.operands.size() < 5) fail_unsupported("@fused_batch_norm takes x, gamma, beta, mean, variance");
            const TensorType xt = f.type_of(call.operands[0]);
            for (int i = 1; i < 5; ++i) {
                const TensorType st = f.type_of(call.operands[i]);
                if (xt.rank() < 1 || st.rank() != 1 || st.shape[0] != xt.shape.back())
                    fail_unsupported("@fused_batch_norm: statistics of shape " + st.str() + " for " + xt.str() + " (one value per element of the last dimension expected)");
            }
            Op bn = simple_op(f, "batch_norm_inference", {call.operands[0], call.operands[1], call.operands[2], call.operands[3], call.operands[4]}, xt);
            bn.attrs["epsilon"] = Attr::make_float(json_number(cfg, "eps", json_number(cfg, "epsilon", 1e-5)));
            bn.attrs["feature_index"] = Attr::make_int(xt.rank() - 1);
            finish(emit(std::move(bn)), call);
        } else if (target == "fused_ffn") {
            // act(x . up) . down; no biases, as in the reference's handler
            if (call.operands.size() < 3) fail_unsupported("@fused_ffn takes x, the up-projection and the down-projection");
            std::string act = json_string(cfg, "activation", "gelu");
            if (act == "gelu" || act == "gelu_approximate" || act == "geluApproximate") act = "gelu_tanh";
            else if (act == "gelu_exact") act = "gelu_erf";
            else if (act == "swish") act = "silu";
            else if (act != "relu" && act != "sigmoid" && act != "tanh" && act != "silu") act = "none";
            const int h = matmul_call(call.operands[0], call.operands[1], act, "@fused_ffn");
            finish(matmul_call(h, call.operands[2], "none", "@fused_ffn"), call);
        } else if (target == "fused_rope") {
            // rotation of the two halves of the last dimension: [x1 cos - x2 sin, x1 sin + x2 cos]
            if (call.operands.size() < 2) fail_unsupported("@fused_rope takes x and the frequencies");
            const int x = call.operands[0], fr = call.operands[1];
            const TensorType xt = f.type_of(x), ft = f.type_of(fr);
            if (xt.rank() < 2 || ft.rank() < 1 || xt.shape.back() % 2 != 0) fail_unsupported("@fused_rope: " + xt.str() + " with frequencies " + ft.str());
            const int64_t hd = xt.shape.back(), half = hd / 2;
            const int x1 = slice_last(x, 0, half), x2 = slice_last(x, half, hd);
            int c, s;
            if (ft.shape.back() == hd) {            // cosines in the first half, sines in the second
                c = slice_last(fr, 0, half);
                s = slice_last(fr, half, hd);
            } else if (ft.shape.back() == half) {   // angles
                c = unary("cosine", fr);
                s = unary("sine", fr);
            } else {                                 // cosines as given; sines from a third operand, else the sine of the operand
                c = fr;
                s = call.operands.size() >= 3 ? call.operands[2] : unary("sine", fr);
            }
            const TensorType ht = f.type_of(x1);
            c = broadcast_trailing(c, ht, "@fused_rope");
            s = broadcast_trailing(s, ht, "@fused_rope");
            const int o1 = binary("subtract", binary("multiply", x1, c), binary("multiply", x2, s));
            const int o2 = binary("add", binary("multiply", x1, s), binary("multiply", x2, c));
            Op cat = simple_op(f, "concatenate", {o1, o2}, xt);
            cat.attrs["dimension"] = Attr::make_int(xt.rank() - 1);
            finish(emit(std::move(cat)), call);
        } else {  // fused_depth_attention: softmax(q . k^T * scale) . v over a short key axis
            if (call.operands.size() < 3) fail_unsupported("@fused_depth_attention takes query, keys and values");
            const int q = call.operands[0], k = call.operands[1], v = call.operands[2];
            const TensorType qt = f.type_of(q), kt = f.type_of(k), vt = f.type_of(v);
            if (kt.rank() != 3 || vt.rank() != 3 || (qt.rank() != 3 && qt.rank() != 2) || qt.shape[0] != kt.shape[0] || qt.shape.back() != kt.shape[2] ||
                vt.shape[0] != kt.shape[0] || vt.shape[1] != kt.shape[1])
                fail_unsupported("@fused_depth_attention: query " + qt.str() + ", keys " + kt.str() + ", values " + vt.str());
            auto batched_dot = [&](int a, int b, int64_t a_contract, int64_t b_contract, std::vector<int64_t> shape) {
                TensorType rt = f.type_of(a);
                rt.shape = std::move(shape);
                Op d = simple_op(f, "dot_general", {a, b}, rt);
                d.attrs["lhs_batching_dimensions"] = Attr::make_ints({0});
                d.attrs["rhs_batching_dimensions"] = Attr::make_ints({0});
                d.attrs["lhs_contracting_dimensions"] = Attr::make_ints({a_contract});
                d.attrs["rhs_contracting_dimensions"] = Attr::make_ints({b_contract});
                return emit(std::move(d));
            };
            const bool q3 = qt.rank() == 3;
            const int64_t B = kt.shape[0], depth = kt.shape[1];
            std::vector<int64_t> score_shape = q3 ? std::vector<int64_t>{B, qt.shape[1], depth} : std::vector<int64_t>{B, depth};
            int sc = batched_dot(q, k, qt.rank() - 1, 2, score_shape);
            const double scale = json_number(cfg, "scale", 1.0);
            if (scale != 1.0) sc = binary("multiply", sc, float_splat(f.type_of(sc), scale));
            Op sm = simple_op(f, "custom_call", {sc}, f.type_of(sc));
            sm.attrs["call_target_name"] = Attr::make_string("fused_softmax");
            sm.attrs["backend_config"] = Attr::make_string("{\"axis\":-1}");
            const int w = emit(std::move(sm));
            std::vector<int64_t> out_shape = q3 ? std::vector<int64_t>{B, qt.shape[1], vt.shape[2]} : std::vector<int64_t>{B, vt.shape[2]};
            finish(batched_dot(w, v, f.type_of(w).rank() - 1, 1, out_shape), call);
        }
    }
    f.ops.swap(out);
    if (any) f.compact();
    return any;
}

Function flatten_main(Module& m) {
    // calls, loops and conditionals can hide each other (a loop body that calls, a callee that loops or branches): repeat
    // until nothing changes
    Function& main = m.main();
    auto all = [&]() {
        const bool a = inline_calls(m);
        const bool b = unroll_static_whiles(main);
        const bool c = flatten_conditionals(main);
        const bool d = flatten_maps(main);
        const bool e = flatten_top_k(main);
        const bool g = drop_optimization_barriers(main) | fold_tuples(main);
        const bool h = expand_fused_custom_calls(main);
        return a || b || c || d || e || g || h;
    };
    for (int round = 0; round < kMaxInlineRounds; ++round) {
        const bool top = all();
        const bool inner = sweep_loop_regions(main, all, 0);  // bodies of the loops whose trip count is not static
        if (!top && !inner) break;
    }
    main.compact();
    return main;
}

}  // namespace mhlo
