// Function-level IR utilities: op insertion, return access, compaction, use lists, and a printer that writes
// a function back as StableHLO text in the generic-friendly pretty form the parser reads.
#include <algorithm>
#include <cstdio>
#include <functional>
#include <sstream>

#include "ir.h"
#include "numeric.h"

namespace mhlo {

int Function::add_op(Op op, const TensorType& t, size_t before) {
    int v = new_value(t);
    op.results = {v};
    op.result_types = {t};
    ops.insert(ops.begin() + static_cast<long>(before), std::move(op));
    for (size_t i = 0; i < ops.size(); ++i)
        for (size_t r = 0; r < ops[i].results.size(); ++r) {
            values[ops[i].results[r]].def_op = static_cast<int>(i);
            values[ops[i].results[r]].def_result = static_cast<int>(r);
        }
    return v;
}

std::vector<int> Function::return_values() const {
    if (ops.empty() || ops.back().name != "return") return {};
    return ops.back().operands;
}

void Function::set_return_values(const std::vector<int>& v) { ops.back().operands = v; }

void Function::compact() {
    std::vector<Op> kept;
    kept.reserve(ops.size());
    for (Op& o : ops)
        if (!o.dead) kept.push_back(std::move(o));
    ops.swap(kept);
    for (Value& v : values)
        if (v.def_op >= 0) v.def_op = -2;  // re-linked below; -2 = defined by a removed op or inside a region
    for (size_t i = 0; i < ops.size(); ++i)
        for (size_t r = 0; r < ops[i].results.size(); ++r) {
            values[ops[i].results[r]].def_op = static_cast<int>(i);
            values[ops[i].results[r]].def_result = static_cast<int>(r);
        }
}

static void collect_region_uses(const Region& r, int op_index, std::vector<std::vector<int>>* users) {
    for (const Op& o : r.ops) {
        for (int v : o.operands) (*users)[v].push_back(op_index);
        for (const auto& sub : o.regions) collect_region_uses(*sub, op_index, users);
    }
}

std::vector<std::vector<int>> Function::users() const {
    std::vector<std::vector<int>> u(values.size());
    for (size_t i = 0; i < ops.size(); ++i) {
        if (ops[i].dead) continue;
        for (int v : ops[i].operands) u[v].push_back(static_cast<int>(i));
        for (const auto& r : ops[i].regions) collect_region_uses(*r, static_cast<int>(i), &u);
    }
    return u;
}

// ---- printer ------------------------------------------------------------------------------------------------

static std::string ints(const std::vector<int64_t>& v) {
    std::string s = "[";
    for (size_t i = 0; i < v.size(); ++i) s += (i ? ", " : "") + std::to_string(v[i]);
    return s + "]";
}

static std::string dense_text(const Attr& a) {
    const TensorType& t = a.dense_type;
    const size_t es = dtype_size(t.dtype);
    const size_t n = es ? a.dense.size() / es : 0;
    auto elem = [&](size_t k) {
        char buf[64];
        const uint8_t* p = a.dense.data() + k * es;
        if (is_float(t.dtype)) {
            double v = decode_as_double(t.dtype, p);
            if (std::isnan(v) || std::isinf(v)) {  // the element's own bit pattern, in the width of its type
                static const char* hex = "0123456789ABCDEF";
                std::string s = "0x";
                for (size_t b = es; b-- > 0;) { s += hex[p[b] >> 4]; s += hex[p[b] & 15]; }
                return s;
            }
            std::snprintf(buf, sizeof buf, "%.9g", v);
            std::string s = buf;
            if (s.find_first_of(".e") == std::string::npos) s += ".0";
            return s;
        }
        if (t.dtype == DType::I1) return std::string(p[0] ? "true" : "false");
        if (t.dtype == DType::UI64) { uint64_t v; std::memcpy(&v, p, 8); return std::to_string(v); }
        return std::to_string(decode_as_int(t.dtype, p));
    };
    if (n == 0) return "dense<>";
    if (a.splat || n == 1) return "dense<" + elem(0) + ">";
    if (n > 64) {  // large payloads print as raw bytes
        static const char* hex = "0123456789ABCDEF";
        std::string s = "dense<\"0x";
        for (uint8_t b : a.dense) { s += hex[b >> 4]; s += hex[b & 15]; }
        return s + "\">";
    }
    // nested brackets following the shape
    std::string s;
    std::vector<int64_t> idx(t.shape.size(), 0);
    size_t k = 0;
    std::function<void(int)> rec = [&](int d) {
        if (d == t.rank()) { s += elem(k++); return; }
        s += "[";
        for (int64_t i = 0; i < t.shape[d]; ++i) { if (i) s += ", "; rec(d + 1); }
        s += "]";
    };
    rec(0);
    return "dense<" + s + ">";
}

static std::string attr_text(const Attr& a) {
    switch (a.kind) {
        case Attr::Int: return std::to_string(a.i);
        case Attr::Float: { char b[64]; std::snprintf(b, sizeof b, "%.9g", a.f); std::string s = b; if (s.find_first_of(".en") == std::string::npos) s += ".0"; return s; }
        case Attr::Bool: return a.b ? "true" : "false";
        case Attr::String: {
            std::string s = "\"";
            for (char c : a.s) { if (c == '"' || c == '\\') s += '\\'; s += c; }
            return s + "\"";
        }
        case Attr::Keyword: return a.s;
        case Attr::IntArray: return ints(a.ints);
        case Attr::Array: { std::string s = "["; for (size_t i = 0; i < a.elems.size(); ++i) s += (i ? ", " : "") + attr_text(a.elems[i]); return s + "]"; }
        case Attr::Dict: { std::string s = "{"; bool first = true; for (const auto& kv : a.dict) { s += (first ? "" : ", ") + kv.first + " = " + attr_text(kv.second); first = false; } return s + "}"; }
        case Attr::Dense: return dense_text(a) + " : " + a.dense_type.str();
        default: return "unit";
    }
}

static std::string vname(int v) { return "%v" + std::to_string(v); }

static void print_op(const Function& f, const Op& o, int indent, std::ostringstream& os);

static void print_region(const Function& f, const Region& r, int indent, std::ostringstream& os) {
    os << "{\n" << std::string(indent + 2, ' ') << "^bb0(";
    for (size_t i = 0; i < r.args.size(); ++i)
        os << (i ? ", " : "") << vname(r.args[i]) << ": " << f.values[r.args[i]].type.str();
    os << "):\n";
    for (const Op& o : r.ops) print_op(f, o, indent + 4, os);
    os << std::string(indent, ' ') << "}";
}

static void print_op(const Function& f, const Op& o, int indent, std::ostringstream& os) {
    os << std::string(indent, ' ');
    if (o.name == "return") {
        os << (indent > 4 ? "stablehlo.return" : "return");
        for (size_t i = 0; i < o.operands.size(); ++i) os << (i ? ", " : " ") << vname(o.operands[i]);
        if (!o.operands.empty()) {
            os << " : ";
            for (size_t i = 0; i < o.operands.size(); ++i) os << (i ? ", " : "") << f.values[o.operands[i]].type.str();
        }
        os << "\n";
        return;
    }
    for (size_t i = 0; i < o.results.size(); ++i) os << (i ? ", " : "") << vname(o.results[i]);
    if (!o.results.empty()) os << " = ";
    os << "\"" << (o.dialect.empty() ? "" : o.dialect + ".") << o.name << "\"(";
    for (size_t i = 0; i < o.operands.size(); ++i) os << (i ? ", " : "") << vname(o.operands[i]);
    os << ")";
    if (!o.regions.empty()) {  // "op"(operands) ({region}, {region}) {attrs}
        os << " (";
        for (size_t i = 0; i < o.regions.size(); ++i) { if (i) os << ", "; print_region(f, *o.regions[i], indent, os); }
        os << ")";
    }
    bool first = true;
    for (const auto& kv : o.attrs) {
        if (kv.first[0] == '_' || kv.first.find('.') != std::string::npos) continue;
        if (kv.second.kind == Attr::Dict && (kv.first == "dot_dimension_numbers" || kv.first == "dimension_numbers")) continue;
        os << (first ? " {" : ", ") << kv.first << " = " << attr_text(kv.second);
        first = false;
    }
    if (!first) os << "}";
    os << " : (";
    for (size_t i = 0; i < o.operands.size(); ++i) os << (i ? ", " : "") << f.values[o.operands[i]].type.str();
    os << ") -> ";
    if (o.result_types.size() == 1) os << o.result_types[0].str();
    else {
        os << "(";
        for (size_t i = 0; i < o.result_types.size(); ++i) os << (i ? ", " : "") << o.result_types[i].str();
        os << ")";
    }
    os << "\n";
}

std::string print_function(const Function& f) {
    std::ostringstream os;
    os << "module {\n  func.func @" << f.name << "(";
    for (size_t i = 0; i < f.args.size(); ++i) os << (i ? ", " : "") << vname(f.args[i]) << ": " << f.values[f.args[i]].type.str();
    os << ") -> (";
    for (size_t i = 0; i < f.result_types.size(); ++i) os << (i ? ", " : "") << f.result_types[i].str();
    os << ") {\n";
    for (const Op& o : f.ops)
        if (!o.dead) print_op(f, o, 4, os);
    os << "  }\n}\n";
    return os.str();
}

}  // namespace mhlo
