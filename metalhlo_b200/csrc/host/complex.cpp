// Complex values without a complex element type. The parser reads tensor<AxBxcomplex<f32>> as the float tensor
// tensor<AxBx2xf32> that stores it as (re, im) pairs and marks the type; this step rewrites every operation that
// touches a marked value into operations on those float tensors, so that nothing behind the parser knows about
// complex numbers. The pair layout is also the one the reference's FFT kernels read and write on float tensors
// (Sources/MetalHLOCore/Compiler/CodeGenerator.swift:2701-2830: "interleaved real/imag"), its element-type enum
// having no complex entry either (Sources/CMetalHLO/include/metalhlo.h:61-75): a complex argument or result of
// @main therefore crosses the C API as a float buffer with one more dimension of extent 2.
//
//   complex(re, im)            -> concatenate of the two parts on a new last axis
//   real / imag                -> slice of the last axis, reshaped
//   add / subtract / negate / convert / select / data movement -> the same operation with the extra axis
//   multiply / divide / abs / exponential / compare EQ, NE -> real arithmetic on the sliced parts
//   fft                        -> stays one operation (FFT, IFFT, RFFT, IRFFT over the last 1 to 3 axes)
// Any other operation on a complex operand is refused with status 4.
#include <functional>

#include "ir.h"

namespace mhlo {
namespace {

struct Rewriter {
    Function& f;
    std::vector<Op> out;

    int emit(const std::string& name, const std::vector<int>& operands, const TensorType& t,
             const std::map<std::string, Attr>& attrs = {}) {
        Op o;
        o.name = name;
        o.dialect = "stablehlo";
        o.operands = operands;
        o.attrs = attrs;
        TensorType plain = t;
        plain.was_complex = false;
        const int v = f.new_value(plain);
        o.results = {v};
        o.result_types = {plain};
        out.push_back(std::move(o));
        return v;
    }
    const TensorType& type(int v) const { return f.values[v].type; }

    // part 0 (re) or 1 (im) of a pair tensor, with the pair axis kept ([..., 1])
    int part_keep(int z, int which) {
        const TensorType& zt = type(z);
        TensorType t = zt;
        t.shape.back() = 1;
        std::vector<int64_t> start(zt.rank(), 0), limit = zt.shape, strides(zt.rank(), 1);
        start.back() = which;
        limit.back() = which + 1;
        return emit("slice", {z}, t, {{"start_indices", Attr::make_ints(start)}, {"limit_indices", Attr::make_ints(limit)},
                                      {"strides", Attr::make_ints(strides)}});
    }
    int drop_pair_axis(int v) {
        TensorType t = type(v);
        t.shape.pop_back();
        return emit("reshape", {v}, t);
    }
    int pairs(int re_keep, int im_keep) {
        TensorType t = type(re_keep);
        const int64_t axis = t.rank() - 1;
        t.shape.back() = 2;
        return emit("concatenate", {re_keep, im_keep}, t, {{"dimension", Attr::make_int(axis)}});
    }
    int binary(const char* name, int a, int b) { return emit(name, {a, b}, type(a)); }
    int unary(const char* name, int a) { return emit(name, {a}, type(a)); }
    int zeros(const TensorType& t) {
        Attr a;
        a.kind = Attr::Dense;
        a.dense_type = t;
        a.dense_type.was_complex = false;
        a.splat = t.count() != 1;
        a.dense.assign(dtype_size(t.dtype), 0);
        return emit("constant", {}, t, {{"value", a}});
    }
};

bool touches_complex(const Function& f, const Op& o) {
    for (const TensorType& t : o.result_types)
        if (t.was_complex) return true;
    for (int v : o.operands)
        if (f.values[v].type.was_complex) return true;
    return false;
}

void refuse_regions(const Function& f, const Op& o) {
    for (const auto& r : o.regions) {
        for (int a : r->args)
            if (f.values[a].type.was_complex) fail_unsupported("complex values inside the region of stablehlo." + o.name);
        for (const Op& inner : r->ops) {
            if (touches_complex(f, inner)) fail_unsupported("complex values inside the region of stablehlo." + o.name);
            refuse_regions(f, inner);
        }
    }
}

}  // namespace

void legalize_complex(Function& f) {
    bool any = false;
    for (const Value& v : f.values) any = any || v.type.was_complex;
    for (const Op& o : f.ops) any = any || o.name == "real" || o.name == "imag";  // also defined on real operands
    for (const TensorType& t : f.result_types) any = any || t.was_complex;
    if (!any) return;

    Rewriter rw{f, {}};
    std::map<int, int> replaced;  // result of a rewritten op -> the value that now holds it
    auto mapped = [&](int v) {
        auto it = replaced.find(v);
        return it == replaced.end() ? v : it->second;
    };
    for (Op& op : f.ops) {
        for (int& v : op.operands) v = mapped(v);
        refuse_regions(f, op);
        if (!touches_complex(f, op) && (op.name == "real" || op.name == "imag") && op.operands.size() == 1) {
            // of a real tensor: the tensor itself, and zeros
            replaced[op.results[0]] = op.name == "real" ? op.operands[0] : rw.zeros(op.result_types[0]);
            continue;
        }
        if (!touches_complex(f, op) || op.name == "return" || op.name == "call" || op.name == "constant" ||
            op.name == "optimization_barrier") {
            rw.out.push_back(op);
            continue;
        }
        const std::string& n = op.name;
        const bool result_complex = !op.result_types.empty() && op.result_types[0].was_complex;
        auto operand_complex = [&](size_t k) { return k < op.operands.size() && f.values[op.operands[k]].type.was_complex; };
        auto done = [&](int v) {  // the value that stands in for the result stays marked while later operations are rewritten
            replaced[op.results[0]] = v;
            f.values[v].type.was_complex = result_complex;
        };

        if (n == "complex") {
            if (op.operands.size() != 2) fail_parse("stablehlo.complex takes two operands");
            TensorType keep = rw.type(op.operands[0]);
            keep.shape.push_back(1);
            done(rw.pairs(rw.emit("reshape", {op.operands[0]}, keep), rw.emit("reshape", {op.operands[1]}, keep)));
        } else if ((n == "real" || n == "imag") && operand_complex(0)) {
            done(rw.drop_pair_axis(rw.part_keep(op.operands[0], n == "imag")));
        } else if (n == "abs" && operand_complex(0)) {
            const int re = rw.part_keep(op.operands[0], 0), im = rw.part_keep(op.operands[0], 1);
            const int sum = rw.binary("add", rw.binary("multiply", re, re), rw.binary("multiply", im, im));
            done(rw.drop_pair_axis(rw.emit("sqrt", {sum}, rw.type(sum))));
        } else if ((n == "multiply" || n == "divide") && operand_complex(0) && operand_complex(1)) {
            const int ar = rw.part_keep(op.operands[0], 0), ai = rw.part_keep(op.operands[0], 1);
            const int br = rw.part_keep(op.operands[1], 0), bi = rw.part_keep(op.operands[1], 1);
            if (n == "multiply") {
                const int re = rw.binary("subtract", rw.binary("multiply", ar, br), rw.binary("multiply", ai, bi));
                const int im = rw.binary("add", rw.binary("multiply", ar, bi), rw.binary("multiply", ai, br));
                done(rw.pairs(re, im));
            } else {  // a * conj(b) / |b|^2
                const int den = rw.binary("add", rw.binary("multiply", br, br), rw.binary("multiply", bi, bi));
                const int re = rw.binary("add", rw.binary("multiply", ar, br), rw.binary("multiply", ai, bi));
                const int im = rw.binary("subtract", rw.binary("multiply", ai, br), rw.binary("multiply", ar, bi));
                done(rw.pairs(rw.binary("divide", re, den), rw.binary("divide", im, den)));
            }
        } else if ((n == "add" || n == "subtract") && operand_complex(0) && operand_complex(1)) {
            rw.out.push_back(op);
        } else if ((n == "negate" || n == "reshape" || n == "reverse" || n == "concatenate" || n == "copy") && operand_complex(0)) {
            rw.out.push_back(op);
        } else if (n == "convert" && operand_complex(0) && result_complex) {
            rw.out.push_back(op);
        } else if (n == "convert" && !operand_complex(0) && result_complex) {  // real -> complex: imaginary part zero
            TensorType keep = op.result_types[0];
            keep.shape.back() = 1;
            TensorType real_t = keep;
            real_t.shape.pop_back();
            const int re = rw.emit("reshape", {rw.emit("convert", {op.operands[0]}, real_t)}, keep);
            done(rw.pairs(re, rw.zeros(keep)));
        } else if (n == "convert" && operand_complex(0) && !result_complex) {  // the imaginary part is dropped
            const int re = rw.drop_pair_axis(rw.part_keep(op.operands[0], 0));
            done(rw.emit("convert", {re}, op.result_types[0]));
        } else if (n == "exponential" && operand_complex(0)) {  // e^re (cos im + i sin im)
            const int re = rw.part_keep(op.operands[0], 0), im = rw.part_keep(op.operands[0], 1);
            const int mag = rw.unary("exponential", re);
            done(rw.pairs(rw.binary("multiply", mag, rw.unary("cosine", im)), rw.binary("multiply", mag, rw.unary("sine", im))));
        } else if (n == "compare" && operand_complex(0) && operand_complex(1)) {
            std::string dir;
            for (const auto& kv : op.attrs)
                for (const char* d : {"EQ", "NE"})
                    if (kv.second.s == d || kv.second.s == std::string("comparison_direction ") + d) dir = d;
            if (dir.empty()) fail_unsupported("stablehlo.compare of complex operands in a direction other than EQ and NE");
            TensorType bt = rw.type(op.operands[0]);
            bt.shape.back() = 1;
            bt.dtype = DType::I1;
            int part[2];
            for (int k = 0; k < 2; ++k) {
                Op c = op;
                c.operands = {rw.part_keep(op.operands[0], k), rw.part_keep(op.operands[1], k)};
                part[k] = rw.emit("compare", c.operands, bt, c.attrs);
            }
            done(rw.drop_pair_axis(rw.binary(dir == "EQ" ? "and" : "or", part[0], part[1])));
        } else if (n == "select" && result_complex && op.operands.size() == 3) {
            const TensorType& pt = rw.type(op.operands[0]);
            TensorType wide = op.result_types[0];
            wide.dtype = pt.dtype;
            std::vector<int64_t> dims;
            for (int d = 0; d < pt.rank(); ++d) dims.push_back(d);
            const int pred = rw.emit("broadcast_in_dim", {op.operands[0]}, wide, {{"broadcast_dimensions", Attr::make_ints(dims)}});
            Op sel = op;
            sel.operands[0] = pred;
            rw.out.push_back(sel);
        } else if (n == "transpose" && operand_complex(0)) {
            std::vector<int64_t> perm = op.int_list("permutation");
            perm.push_back(static_cast<int64_t>(perm.size()));
            op.attrs["permutation"] = Attr::make_ints(perm);
            rw.out.push_back(op);
        } else if (n == "broadcast_in_dim" && operand_complex(0)) {
            std::vector<int64_t> dims = op.int_list("broadcast_dimensions");
            dims.push_back(op.result_types[0].rank() - 1);
            op.attrs["broadcast_dimensions"] = Attr::make_ints(dims);
            rw.out.push_back(op);
        } else if (n == "slice" && operand_complex(0)) {
            std::vector<int64_t> start = op.int_list("start_indices"), limit = op.int_list("limit_indices"), strides = op.int_list("strides");
            if (strides.empty()) strides.assign(start.size(), 1);
            start.push_back(0);
            limit.push_back(2);
            strides.push_back(1);
            op.attrs["start_indices"] = Attr::make_ints(start);
            op.attrs["limit_indices"] = Attr::make_ints(limit);
            op.attrs["strides"] = Attr::make_ints(strides);
            rw.out.push_back(op);
        } else if (n == "fft") {
            rw.out.push_back(op);  // the lowering takes pairs; the types already have the pair axis
        } else {
            fail_unsupported("stablehlo." + n + " on complex operands is not supported (complex, real, imag, abs, add, subtract, "
                             "multiply, divide, negate, exponential, compare EQ / NE, convert, select, fft and data movement are)");
        }
        if (!rw.out.empty())
            for (TensorType& t : rw.out.back().result_types) t.was_complex = false;
    }
    f.ops.swap(rw.out);
    f.arg_complex.clear();
    f.result_complex.clear();
    for (int a : f.args) f.arg_complex.push_back(f.values[a].type.was_complex);
    for (const TensorType& t : f.result_types) f.result_complex.push_back(t.was_complex);
    for (Value& v : f.values) v.type.was_complex = false;
    for (TensorType& t : f.result_types) t.was_complex = false;
    for (Op& o : f.ops)
        for (TensorType& t : o.result_types) t.was_complex = false;
    for (Value& v : f.values)
        if (v.def_op >= 0) v.def_op = -2;
    for (size_t i = 0; i < f.ops.size(); ++i)
        for (size_t r = 0; r < f.ops[i].results.size(); ++r) {
            f.values[f.ops[i].results[r]].def_op = static_cast<int>(i);
            f.values[f.ops[i].results[r]].def_result = static_cast<int>(r);
        }
}

}  // namespace mhlo
