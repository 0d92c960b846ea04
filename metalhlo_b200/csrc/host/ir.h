// In-memory form of a StableHLO module as the compiler core sees it: SSA values, operations with typed
// results and an attribute dictionary, functions and regions. Plays the role of HLOModule / HLOFunction /
// HLOOperation / HLOAttributes / TensorType in the reference
// (Sources/MetalHLOCore/IR/{HLOModule,HLOOpKind,Attributes,TensorType}.swift).
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace mhlo {

// Element types in the numbering of MHLOElementType (Sources/CMetalHLO/include/metalhlo.h:61-75).
enum class DType : int {
    F16 = 0, F32 = 1, F64 = 2, BF16 = 3, I1 = 4, I8 = 5, I16 = 6, I32 = 7, I64 = 8,
    UI8 = 9, UI16 = 10, UI32 = 11, UI64 = 12
};

inline size_t dtype_size(DType t) {
    switch (t) {
        case DType::F16: case DType::BF16: case DType::I16: case DType::UI16: return 2;
        case DType::F32: case DType::I32: case DType::UI32: return 4;
        case DType::F64: case DType::I64: case DType::UI64: return 8;
        default: return 1;
    }
}
inline bool is_float(DType t) { return t == DType::F16 || t == DType::F32 || t == DType::F64 || t == DType::BF16; }
inline bool is_unsigned(DType t) { return t >= DType::UI8; }
const char* dtype_name(DType t);
bool dtype_from_name(const std::string& s, DType* out);

struct TensorType {
    DType dtype = DType::F32;
    std::vector<int64_t> shape;
    // Set by the parser on tensor<...xcomplex<f32|f64>>: the type is then already the float tensor with a trailing
    // dimension of 2 (re, im) that stores it; the mark only tells the complex legalisation which operations to
    // rewrite, is cleared by it and takes no part in comparisons.
    bool was_complex = false;
    int rank() const { return static_cast<int>(shape.size()); }
    int64_t count() const {
        int64_t n = 1;
        for (int64_t d : shape) n *= d;
        return n;
    }
    int64_t bytes() const { return count() * static_cast<int64_t>(dtype_size(dtype)); }
    bool operator==(const TensorType& o) const { return dtype == o.dtype && shape == o.shape; }
    bool operator!=(const TensorType& o) const { return !(*this == o); }
    std::string str() const;
};

// Errors carry the MHLO status code they map to at the C boundary.
struct CompileError : std::runtime_error {
    int code;
    CompileError(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};
[[noreturn]] void fail_parse(const std::string& m);        // status 3
[[noreturn]] void fail_unsupported(const std::string& m);  // status 4
[[noreturn]] void fail_compile(const std::string& m);      // status 5

// Attribute values: the subset of MLIR attribute syntax StableHLO text uses.
struct Attr {
    enum Kind { None, Int, Float, Bool, String, IntArray, Array, Dict, Dense, Keyword } kind = None;
    int64_t i = 0;
    double f = 0;
    bool b = false;
    std::string s;                      // String / Keyword text
    std::vector<int64_t> ints;          // IntArray
    std::vector<Attr> elems;            // Array of anything
    std::map<std::string, Attr> dict;   // Dict (also #stablehlo.xxx<...> bodies)
    // Dense: raw little-endian bytes in the element type of `dense_type`; a splat holds one element.
    std::vector<uint8_t> dense;
    TensorType dense_type;
    bool splat = false;

    static Attr make_int(int64_t v) { Attr a; a.kind = Int; a.i = v; a.f = static_cast<double>(v); return a; }
    static Attr make_float(double v) { Attr a; a.kind = Float; a.f = v; return a; }
    static Attr make_bool(bool v) { Attr a; a.kind = Bool; a.b = v; a.i = v; return a; }
    static Attr make_string(const std::string& v) { Attr a; a.kind = String; a.s = v; return a; }
    static Attr make_ints(const std::vector<int64_t>& v) { Attr a; a.kind = IntArray; a.ints = v; return a; }
    const Attr* get(const std::string& key) const {
        auto it = dict.find(key);
        return it == dict.end() ? nullptr : &it->second;
    }
    // Integer list view of Int / IntArray / Array-of-Int attributes.
    std::vector<int64_t> as_ints() const;
    double as_float() const { return kind == Int ? static_cast<double>(i) : f; }
};

struct Region;

struct Op {
    std::string name;                    // without dialect prefix: "add", "dot_general", "custom_call", "return"
    std::string dialect;                 // "stablehlo", "func", "chlo", ...
    std::vector<int> operands;           // value ids
    std::vector<int> results;            // value ids
    std::vector<TensorType> result_types;
    std::map<std::string, Attr> attrs;
    std::vector<std::shared_ptr<Region>> regions;
    bool dead = false;                   // tombstone used by passes; compacted by Function::compact()

    const Attr* attr(const std::string& k) const {
        auto it = attrs.find(k);
        return it == attrs.end() ? nullptr : &it->second;
    }
    std::vector<int64_t> int_list(const std::string& k) const {
        const Attr* a = attr(k);
        return a ? a->as_ints() : std::vector<int64_t>{};
    }
    int64_t int_attr(const std::string& k, int64_t dflt) const {
        const Attr* a = attr(k);
        return a && (a->kind == Attr::Int) ? a->i : dflt;
    }
    std::string str_attr(const std::string& k, const std::string& dflt = "") const {
        const Attr* a = attr(k);
        return a && (a->kind == Attr::String || a->kind == Attr::Keyword) ? a->s : dflt;
    }
};

struct Value {
    TensorType type;
    int def_op = -1;      // index into Function::ops, or -1 for a function / block argument
    int def_result = 0;   // which result of def_op
    std::string name;     // textual name (%arg0, %3) for diagnostics
};

struct Region {
    std::vector<int> args;   // value ids (in the enclosing function's value table)
    std::vector<Op> ops;
};

struct Function {
    std::string name;
    std::vector<int> args;            // value ids of the parameters
    std::vector<Value> values;        // every SSA value of the function, regions included
    std::vector<Op> ops;              // top-level body in program order; the last one is the return
    std::vector<TensorType> result_types;
    // Which parameters / results were complex tensors in the text (they are float tensors of (re, im) pairs here); empty
    // when none was. Filled by legalize_complex for hosts that have a complex buffer type of their own (PJRT).
    std::vector<bool> arg_complex, result_complex;

    int new_value(const TensorType& t, const std::string& name = "") {
        Value v;
        v.type = t;
        v.name = name;
        values.push_back(v);
        return static_cast<int>(values.size()) - 1;
    }
    // Appends an op producing one result of type t before the return; returns the result value id.
    int add_op(Op op, const TensorType& t, size_t before);
    std::vector<int> return_values() const;
    void set_return_values(const std::vector<int>& v);
    // Drops dead ops and re-links Value::def_op.
    void compact();
    // users[v] = indices of ops using value v (regions are scanned too).
    std::vector<std::vector<int>> users() const;
    const TensorType& type_of(int v) const { return values[v].type; }
};

struct Module {
    std::string name;
    std::vector<Function> functions;
    const Function& main() const;
    Function& main();
};

// Rewrites every operation on complex values into operations on float tensors with a trailing (re, im) dimension
// (complex.cpp); called by parse_module on each function.
void legalize_complex(Function& f);
// Parses StableHLO text (pretty and generic op forms) into a Module. Throws CompileError(3, ...).
Module parse_module(const std::string& text);
// Prints a function back as StableHLO text (used for METALHLO_DUMP_OPTIMIZED and by the tests).
std::string print_function(const Function& f);

}  // namespace mhlo
