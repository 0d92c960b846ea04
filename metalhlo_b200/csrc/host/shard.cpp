// Batch sharding of a StableHLO function over equal, contiguous shards of one axis.
//
// The reference runs every program on one device (Sources/PJRTMetalHLO/PJRTExecutable.swift:1830-1848 fixes
// num_replicas = num_partitions = 1, :2033-2036 refuses several devices). Here a program whose results are, slice by
// slice along one axis, functions of the same slice of its batched arguments can be split over several GPUs with no
// exchange on the data path. This file proves that property and rewrites the function to compute one shard.
//
// The proof is a forward propagation over the flattened @main: every value is either replicated (the same on every
// shard) or split along one axis. Each operator has a rule that derives the split axis of its results from those of its
// operands, or refuses: a contraction, reduction, window, sort or gather that mixes elements along the split axis makes
// the shards depend on one another, and the function is rejected with the operator named. Replicated values that meet a
// split value in an elementwise operator (broadcast masks, position tables, constants) are re-derived at shard extent by
// cloning their defining chain, or sliced when that chain is not a pure broadcast.
//
// The rewrite itself only shrinks types (and the few attributes that spell out extents): the operators, their order and
// their fusion patterns stay as they were, so the pass pipeline sees the same graph at a smaller batch.
#include <algorithm>
#include <map>
#include <set>

#include "compiler.h"

namespace mhlo {
namespace {

const std::set<std::string>& elementwise_ops() {
    static const std::set<std::string> s = {
        "add", "subtract", "multiply", "divide", "maximum", "minimum", "power", "remainder", "atan2", "and", "or", "xor", "not",
        "shift_left", "shift_right_arithmetic", "shift_right_logical", "compare", "select", "clamp", "convert", "negate", "abs",
        "exponential", "exponential_minus_one", "log", "log_plus_one", "logistic", "tanh", "tan", "sine", "cosine", "sqrt",
        "rsqrt", "cbrt", "floor", "ceil", "round_nearest_afz", "round_nearest_even", "sign", "popcnt", "count_leading_zeros",
        "is_finite", "erf", "reduce_precision", "copy"};
    return s;
}

int64_t product(const std::vector<int64_t>& s, size_t from, size_t to) {
    int64_t p = 1;
    for (size_t i = from; i < to; ++i) p *= s[i];
    return p;
}

int position(const std::vector<int64_t>& v, int64_t x) {
    for (size_t i = 0; i < v.size(); ++i)
        if (v[i] == x) return static_cast<int>(i);
    return -1;
}

struct Sharder {
    Function& f;
    const int n, k;                       // shard count and this shard's index
    std::vector<Op> old;                  // the function's ops as they came in
    std::vector<Op> out;                  // the rewritten op list, in program order
    std::vector<int> axis;                // per value: -1 replicated, else the split axis
    std::vector<TensorType> full;         // per value: its type before the split
    std::map<std::pair<int, int>, int> sharded_copy;  // (replicated value, axis) -> value that holds this shard of it

    Sharder(Function& fn, int count, int index) : f(fn), n(count), k(index) {
        old = f.ops;
        axis.assign(f.values.size(), -1);
        full.reserve(f.values.size());
        for (const Value& v : f.values) full.push_back(v.type);
    }

    [[noreturn]] void refuse(const Op& op, const std::string& why) const {
        fail_unsupported("cannot split the batch over " + std::to_string(n) + " shards: stablehlo." + op.name + " " + why);
    }

    int new_value(const TensorType& shard_type, const TensorType& full_type, int ax) {
        const int v = f.new_value(shard_type);
        axis.push_back(ax);
        full.push_back(full_type);
        return v;
    }

    static TensorType shrunk(TensorType t, int ax, int count) {
        t.shape[static_cast<size_t>(ax)] /= count;
        return t;
    }

    void mark(int v, int ax, const Op& op) {
        if (ax < 0) return;
        const TensorType& t = full[static_cast<size_t>(v)];
        if (ax >= t.rank() || t.shape[static_cast<size_t>(ax)] % n != 0)
            refuse(op, "yields " + t.str() + ", whose axis " + std::to_string(ax) + " does not divide into the shards");
        axis[static_cast<size_t>(v)] = ax;
        f.values[static_cast<size_t>(v)].type = shrunk(t, ax, n);
    }

    // This shard of replicated value v along axis d, as a value of the rewritten function.
    int demand(int v, int d, const Op& user) {
        if (axis[static_cast<size_t>(v)] == d) return v;
        if (axis[static_cast<size_t>(v)] >= 0) refuse(user, "combines values split along different axes");
        const auto key = std::make_pair(v, d);
        auto it = sharded_copy.find(key);
        if (it != sharded_copy.end()) return it->second;
        const TensorType ft = full[static_cast<size_t>(v)];
        if (d >= ft.rank() || ft.shape[static_cast<size_t>(d)] % n != 0) refuse(user, "needs a shard of " + ft.str() + " along axis " + std::to_string(d));
        const TensorType st = shrunk(ft, d, n);
        const int def = v < static_cast<int>(f.values.size()) ? f.values[static_cast<size_t>(v)].def_op : -1;
        int result = -1;
        if (def >= 0 && def < static_cast<int>(old.size()) && old[static_cast<size_t>(def)].results.size() == 1 &&
            old[static_cast<size_t>(def)].results[0] == v) {
            const Op& o = old[static_cast<size_t>(def)];
            Op c = o;
            bool cloned = false;
            if (o.name == "broadcast_in_dim") {
                const std::vector<int64_t> dims = o.int_list("broadcast_dimensions");
                const int od = position(dims, d);
                const TensorType& ot = full[static_cast<size_t>(o.operands[0])];
                if (od < 0 || ot.shape[static_cast<size_t>(od)] == 1) cloned = true;  // the axis is made by the broadcast itself
                else if (ot.shape[static_cast<size_t>(od)] == ft.shape[static_cast<size_t>(d)]) {
                    c.operands[0] = demand(o.operands[0], od, user);
                    cloned = true;
                }
            } else if (o.name == "constant") {
                auto a = c.attrs.find("value");
                if (a != c.attrs.end() && a->second.kind == Attr::Dense && a->second.splat) {
                    a->second.dense_type = st;
                    cloned = true;
                }
            } else if (o.name == "iota") {
                cloned = o.int_attr("iota_dimension", 0) != d;
            } else if (elementwise_ops().count(o.name)) {
                for (int& operand : c.operands) {
                    const TensorType& ot = full[static_cast<size_t>(operand)];
                    if (ot.shape == ft.shape) operand = demand(operand, d, user);
                    else if (ot.rank() != 0) refuse(o, "has operands of different shapes");
                }
                cloned = true;
            }
            if (cloned) {
                result = new_value(st, ft, d);
                c.results = {result};
                c.result_types = {st};
                out.push_back(std::move(c));
            }
        }
        if (result < 0) {
            // anything else: cut this shard out of the replicated tensor
            Op s;
            s.name = "slice";
            s.dialect = "stablehlo";
            s.operands = {v};
            std::vector<int64_t> start(static_cast<size_t>(ft.rank()), 0), limit = ft.shape, stride(static_cast<size_t>(ft.rank()), 1);
            const int64_t len = ft.shape[static_cast<size_t>(d)] / n;
            start[static_cast<size_t>(d)] = len * k;
            limit[static_cast<size_t>(d)] = len * (k + 1);
            s.attrs["start_indices"] = Attr::make_ints(start);
            s.attrs["limit_indices"] = Attr::make_ints(limit);
            s.attrs["strides"] = Attr::make_ints(stride);
            result = new_value(st, ft, d);
            s.results = {result};
            s.result_types = {st};
            out.push_back(std::move(s));
        }
        sharded_copy[key] = result;
        return result;
    }

    int ax(int v) const { return axis[static_cast<size_t>(v)]; }
    const TensorType& ft(int v) const { return full[static_cast<size_t>(v)]; }

    // The one axis the split operands agree on (refuses a mix); -1 when none is split.
    int common_axis(const Op& op, size_t first, size_t last) const {
        int d = -1;
        for (size_t i = first; i < last; ++i) {
            const int a = ax(op.operands[i]);
            if (a < 0) continue;
            if (d >= 0 && a != d) refuse(op, "combines values split along different axes");
            d = a;
        }
        return d;
    }

    void set_results(Op& op, int d) {
        for (size_t r = 0; r < op.results.size(); ++r) {
            mark(op.results[r], d, op);
            op.result_types[r] = f.values[static_cast<size_t>(op.results[r])].type;
        }
    }

    bool region_reads_split_value(const Region& r) const {
        for (const Op& o : r.ops) {
            for (int v : o.operands)
                if (ax(v) >= 0) return true;
            for (const auto& sub : o.regions)
                if (region_reads_split_value(*sub)) return true;
        }
        return false;
    }

    void rewrite(Op op) {
        bool any = false;
        for (int v : op.operands) any = any || ax(v) >= 0;
        for (const auto& r : op.regions)
            if (region_reads_split_value(*r)) refuse(op, "has a body that reads a split value of the enclosing function");
        if (!any || op.name == "return") {  // replicated computation: every shard does the same
            out.push_back(std::move(op));
            return;
        }
        const std::string& nm = op.name;
        const int r0 = op.results.empty() ? -1 : op.results[0];
        if (r0 < 0) refuse(op, "has no result");
        if (elementwise_ops().count(nm)) {
            const int d = common_axis(op, 0, op.operands.size());
            const TensorType rt = ft(r0);
            for (int& v : op.operands) {
                if (ft(v).shape == rt.shape) v = demand(v, d, op);
                else if (ft(v).rank() != 0) refuse(op, "has operands of different shapes");
            }
            set_results(op, d);
        } else if (nm == "broadcast_in_dim") {
            const std::vector<int64_t> dims = op.int_list("broadcast_dimensions");
            const int od = ax(op.operands[0]);
            const int d = static_cast<int>(dims[static_cast<size_t>(od)]);
            if (ft(op.operands[0]).shape[static_cast<size_t>(od)] != ft(r0).shape[static_cast<size_t>(d)])
                refuse(op, "expands the split axis");
            set_results(op, d);
        } else if (nm == "reshape" || nm == "dynamic_reshape") {
            if (nm == "dynamic_reshape") refuse(op, "of a split value");
            const int od = ax(op.operands[0]);
            const std::vector<int64_t>& in = ft(op.operands[0]).shape;
            const std::vector<int64_t>& o = ft(r0).shape;
            const int64_t prefix = product(in, 0, static_cast<size_t>(od));
            int d = -1;
            for (size_t j = 0; j < o.size(); ++j)
                if (product(o, 0, j) == prefix && o[j] % n == 0 && o[j] > 1) { d = static_cast<int>(j); break; }
            if (d < 0) refuse(op, "regroups the split axis " + ft(op.operands[0]).str() + " -> " + ft(r0).str());
            set_results(op, d);
        } else if (nm == "transpose") {
            const int d = position(op.int_list("permutation"), ax(op.operands[0]));
            if (d < 0) refuse(op, "has a malformed permutation");
            set_results(op, d);
        } else if (nm == "dot_general") {
            const std::vector<int64_t> lb = op.int_list("lhs_batching_dimensions"), rb = op.int_list("rhs_batching_dimensions"),
                                       lc = op.int_list("lhs_contracting_dimensions"), rc = op.int_list("rhs_contracting_dimensions");
            const int la = ax(op.operands[0]), ra = ax(op.operands[1]);
            auto free_position = [](int rank, const std::vector<int64_t>& b, const std::vector<int64_t>& c, int a) {
                int p = 0;
                for (int i = 0; i < rank; ++i) {
                    if (position(b, i) >= 0 || position(c, i) >= 0) continue;
                    if (i == a) return p;
                    ++p;
                }
                return -1;
            };
            auto free_count = [](int rank, const std::vector<int64_t>& b, const std::vector<int64_t>& c) {
                return rank - static_cast<int>(b.size()) - static_cast<int>(c.size());
            };
            int d = -1;
            if (la >= 0 && position(lc, la) >= 0) refuse(op, "contracts over the split axis");
            if (ra >= 0 && position(rc, ra) >= 0) refuse(op, "contracts over the split axis");
            if (la >= 0 && position(lb, la) >= 0) {
                const int i = position(lb, la);
                op.operands[1] = demand(op.operands[1], static_cast<int>(rb[static_cast<size_t>(i)]), op);
                d = i;
            } else if (ra >= 0 && position(rb, ra) >= 0) {
                const int i = position(rb, ra);
                op.operands[0] = demand(op.operands[0], static_cast<int>(lb[static_cast<size_t>(i)]), op);
                d = i;
            } else if (la >= 0) {
                if (ra >= 0) refuse(op, "has both operands split along free axes");
                d = static_cast<int>(lb.size()) + free_position(ft(op.operands[0]).rank(), lb, lc, la);
            } else {
                d = static_cast<int>(lb.size()) + free_count(ft(op.operands[0]).rank(), lb, lc) + free_position(ft(op.operands[1]).rank(), rb, rc, ra);
            }
            set_results(op, d);
        } else if (nm == "reduce") {
            const size_t n_in = op.operands.size() / 2;
            for (size_t i = n_in; i < op.operands.size(); ++i)
                if (ax(op.operands[i]) >= 0) refuse(op, "has a split initial value");
            const int od = common_axis(op, 0, n_in);
            const std::vector<int64_t> dims = op.int_list("dimensions");
            if (position(dims, od) >= 0) refuse(op, "reduces over the split axis");
            for (size_t i = 0; i < n_in; ++i) op.operands[i] = demand(op.operands[i], od, op);
            int d = od;
            for (int64_t x : dims) d -= x < od ? 1 : 0;
            set_results(op, d);
        } else if (nm == "gather") {
            if (ax(op.operands[0]) >= 0) refuse(op, "reads from a split table");
            const int id = ax(op.operands[1]);
            const int64_t ivd = op.int_attr("index_vector_dim", ft(op.operands[1]).rank());
            if (id == ivd) refuse(op, "has its index vectors split");
            if (!op.int_list("operand_batching_dims").empty()) refuse(op, "with batching dimensions");
            int batch_pos = 0;
            for (int i = 0; i < id; ++i) batch_pos += i != ivd ? 1 : 0;
            const std::vector<int64_t> offset = op.int_list("offset_dims");
            int d = -1, seen = 0;
            for (int j = 0; j < ft(r0).rank(); ++j) {
                if (position(offset, j) >= 0) continue;
                if (seen++ == batch_pos) { d = j; break; }
            }
            if (d < 0) refuse(op, "has no result axis for the split index axis");
            set_results(op, d);
        } else if (nm == "concatenate") {
            const int d = common_axis(op, 0, op.operands.size());
            if (op.int_attr("dimension", 0) == d) refuse(op, "joins along the split axis");
            for (int& v : op.operands) v = demand(v, d, op);
            set_results(op, d);
        } else if (nm == "slice") {
            const int d = ax(op.operands[0]);
            std::vector<int64_t> start = op.int_list("start_indices"), limit = op.int_list("limit_indices"), stride = op.int_list("strides");
            const int64_t extent = ft(op.operands[0]).shape[static_cast<size_t>(d)];
            if (start[static_cast<size_t>(d)] != 0 || limit[static_cast<size_t>(d)] != extent || (!stride.empty() && stride[static_cast<size_t>(d)] != 1))
                refuse(op, "cuts the split axis");
            limit[static_cast<size_t>(d)] = extent / n;
            op.attrs["limit_indices"] = Attr::make_ints(limit);
            set_results(op, d);
        } else if (nm == "dynamic_slice") {
            const int d = ax(op.operands[0]);
            for (size_t i = 1; i < op.operands.size(); ++i)
                if (ax(op.operands[i]) >= 0) refuse(op, "has a split start index");
            std::vector<int64_t> sizes = op.int_list("slice_sizes");
            const int64_t extent = ft(op.operands[0]).shape[static_cast<size_t>(d)];
            if (sizes.size() <= static_cast<size_t>(d) || sizes[static_cast<size_t>(d)] != extent) refuse(op, "cuts the split axis");
            sizes[static_cast<size_t>(d)] = extent / n;
            op.attrs["slice_sizes"] = Attr::make_ints(sizes);
            set_results(op, d);
        } else if (nm == "pad") {
            const int d = ax(op.operands[0]);
            if (ax(op.operands[1]) >= 0) refuse(op, "has a split padding value");
            for (const char* key : {"edge_padding_low", "edge_padding_high", "interior_padding"}) {
                const std::vector<int64_t> p = op.int_list(key);
                if (p.size() > static_cast<size_t>(d) && p[static_cast<size_t>(d)] != 0) refuse(op, "pads the split axis");
            }
            set_results(op, d);
        } else if (nm == "reverse") {
            const int d = ax(op.operands[0]);
            if (position(op.int_list("dimensions"), d) >= 0) refuse(op, "reverses the split axis");
            set_results(op, d);
        } else if (nm == "convolution") {
            if (ax(op.operands[1]) >= 0) refuse(op, "has a split kernel");
            if (op.int_attr("batch_group_count", 1) != 1) refuse(op, "with batch groups");
            if (ax(op.operands[0]) != op.int_attr("input_batch_dimension", 0)) refuse(op, "is split along a feature or spatial axis");
            set_results(op, static_cast<int>(op.int_attr("output_batch_dimension", 0)));
        } else if (nm == "reduce_window") {
            if (op.operands.size() != 2 || ax(op.operands[1]) >= 0) refuse(op, "with several operands or a split initial value");
            const int d = ax(op.operands[0]);
            auto at = [&](const char* key, int64_t dflt) {
                const std::vector<int64_t> v = op.int_list(key);
                return v.size() > static_cast<size_t>(d) ? v[static_cast<size_t>(d)] : dflt;
            };
            const std::vector<int64_t> pad = op.int_list("padding");
            const bool padded = pad.size() >= 2 * static_cast<size_t>(d) + 2 && (pad[2 * static_cast<size_t>(d)] != 0 || pad[2 * static_cast<size_t>(d) + 1] != 0);
            if (at("window_dimensions", 1) != 1 || at("window_strides", 1) != 1 || at("base_dilations", 1) != 1 || at("window_dilations", 1) != 1 || padded)
                refuse(op, "slides its window along the split axis");
            set_results(op, d);
        } else if (nm == "batch_norm_inference") {
            for (size_t i = 1; i < op.operands.size(); ++i)
                if (ax(op.operands[i]) >= 0) refuse(op, "has split statistics");
            const int d = ax(op.operands[0]);
            if (op.int_attr("feature_index", -1) == d) refuse(op, "normalises along the split axis");
            set_results(op, d);
        } else if (nm == "sort") {
            const int d = common_axis(op, 0, op.operands.size());
            int64_t sd = op.int_attr("dimension", -1);
            if (sd < 0) sd += ft(op.operands[0]).rank();
            if (sd == d) refuse(op, "orders along the split axis");
            for (int& v : op.operands) v = demand(v, d, op);
            set_results(op, d);
        } else if (nm == "custom_call") {
            const std::string target = op.str_attr("call_target_name");
            const int d = ax(op.operands[0]);
            const int rank = ft(op.operands[0]).rank();
            auto rest_replicated = [&](size_t from) {
                for (size_t i = from; i < op.operands.size(); ++i)
                    if (ax(op.operands[i]) >= 0) refuse(op, "@" + target + " has a split parameter operand");
            };
            if (target == "fused_conv_bias_act") {  // the convolution's rule; the bias is a parameter
                if (op.operands.size() < 2 || ax(op.operands[1]) >= 0) refuse(op, "@" + target + " has a split kernel");
                if (op.int_attr("batch_group_count", 1) != 1) refuse(op, "@" + target + " with batch groups");
                if (d != op.int_attr("input_batch_dimension", 0)) refuse(op, "@" + target + " is split along a feature or spatial axis");
                rest_replicated(2);
                set_results(op, static_cast<int>(op.int_attr("output_batch_dimension", 0)));
                out.push_back(std::move(op));
                return;
            }
            if (target == "fused_scaled_dot_product_attention") {
                if (rank != 4 || d > 1) refuse(op, "@" + target + " is split along the sequence or head dimension");
                for (size_t i = 0; i < 3 && i < op.operands.size(); ++i) op.operands[i] = demand(op.operands[i], d, op);
                rest_replicated(3);
            } else if (target == "fused_layer_norm" || target == "fused_rms_norm" || target == "fused_softmax" || target == "fused_gelu" ||
                       target == "fused_silu" || target == "fused_matmul_bias_activation") {
                if (d == rank - 1) refuse(op, "@" + target + " is split along the axis it works on");
                // a product's residual (its last operand) has the result's shape and is split with the activations
                const bool residual = target == "fused_matmul_bias_activation" && op.operands.size() > 2 &&
                                      op.str_attr("backend_config").find("\"has_residual\":true") != std::string::npos;
                if (residual) {
                    const int r = op.operands.back();
                    op.operands.pop_back();
                    rest_replicated(1);
                    op.operands.push_back(demand(r, d, op));
                } else {
                    rest_replicated(1);
                }
            } else {
                refuse(op, "@" + target + " of a split value");
            }
            set_results(op, d);
        } else {
            refuse(op, "has no rule for split operands");
        }
        out.push_back(std::move(op));
    }
};

}  // namespace

ShardPlan shard_function(Function& f, const ShardSpec& spec) {
    if (spec.count < 1 || spec.index < 0 || spec.index >= spec.count) fail_compile("shard index / count out of range");
    ShardPlan plan;
    plan.count = spec.count;
    plan.index = spec.index;
    for (int a : f.args) plan.full_input_types.push_back(f.type_of(a));
    plan.full_output_types = f.result_types;
    plan.input_axes.assign(f.args.size(), -1);
    plan.output_axes.assign(f.result_types.size(), -1);
    if (spec.count == 1) return plan;

    // which arguments are split: as given, else every argument whose leading extent equals the first argument's
    // (the batch), else the first argument alone
    std::vector<std::vector<int>> attempts;
    if (!spec.input_axes.empty()) {
        if (spec.input_axes.size() != f.args.size()) fail_compile("shard axes: one entry per argument expected");
        attempts.push_back(spec.input_axes);
    } else {
        if (f.args.empty() || f.type_of(f.args[0]).rank() == 0) fail_unsupported("cannot split the batch: the first argument has no axes");
        const int64_t batch = f.type_of(f.args[0]).shape[0];
        std::vector<int> all(f.args.size(), -1), first(f.args.size(), -1);
        for (size_t i = 0; i < f.args.size(); ++i) {
            const TensorType& t = f.type_of(f.args[i]);
            if (t.rank() > 0 && t.shape[0] == batch) all[i] = 0;
        }
        first[0] = 0;
        attempts.push_back(all);
        if (all != first) attempts.push_back(first);
    }
    std::string first_error;
    for (const std::vector<int>& axes : attempts) {
        Function g = f;
        try {
            Sharder s(g, spec.count, spec.index);
            Op dummy;
            dummy.name = "func argument";
            for (size_t i = 0; i < g.args.size(); ++i) s.mark(g.args[i], axes[i], dummy);
            for (Op& op : s.old) {
                if (op.dead) continue;
                s.rewrite(op);
            }
            g.ops = std::move(s.out);
            const std::vector<int> rets = g.return_values();
            g.result_types.clear();
            for (size_t i = 0; i < rets.size(); ++i) {
                plan.output_axes[i] = s.axis[static_cast<size_t>(rets[i])];
                g.result_types.push_back(g.type_of(rets[i]));
            }
            plan.input_axes = axes;
            // drop what only the replicated originals of re-derived values used
            for (;;) {
                const std::vector<std::vector<int>> users = g.users();
                bool removed = false;
                for (Op& op : g.ops) {
                    if (op.dead || op.name == "return" || op.results.empty()) continue;
                    bool used = false;
                    for (int r : op.results) used = used || !users[static_cast<size_t>(r)].empty();
                    if (!used) { op.dead = true; removed = true; }
                }
                if (!removed) break;
            }
            g.compact();
            f = std::move(g);
            return plan;
        } catch (const CompileError& e) {
            if (first_error.empty()) first_error = e.what();
        }
    }
    fail_unsupported(first_error);
}

}  // namespace mhlo
