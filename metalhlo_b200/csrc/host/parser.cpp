// Recursive-descent parser for StableHLO text: the dialect the reference's hand-written parser accepts
// (Sources/MetalHLOCore/Parser/Parser.swift:31-2778, Lexer.swift) - `module`/`func.func` shells, pretty and
// generic operation forms, tensor types over the 13 element types, dense constants (scalars, nested lists,
// hex bit patterns, raw "0x.." byte strings), #stablehlo.dot/#stablehlo.gather attribute bodies, reduce with
// either an `applies` clause or a reducer region, and custom_call with a backend_config string.
//
// It works on characters rather than tokens because MLIR's shaped-type syntax (2x3xf32) does not tokenise.
#include <cctype>
#include <cmath>
#include <cstring>
#include <sstream>

#include "ir.h"
#include "numeric.h"

namespace mhlo {

void fail_parse(const std::string& m) { throw CompileError(3, m); }
void fail_unsupported(const std::string& m) { throw CompileError(4, m); }
void fail_compile(const std::string& m) { throw CompileError(5, m); }

static const char* kDTypeNames[] = {"f16", "f32", "f64", "bf16", "i1", "i8", "i16", "i32", "i64",
                                    "ui8", "ui16", "ui32", "ui64"};
const char* dtype_name(DType t) { return kDTypeNames[static_cast<int>(t)]; }
bool dtype_from_name(const std::string& s, DType* out) {
    for (int i = 0; i < 13; ++i)
        if (s == kDTypeNames[i]) {
            *out = static_cast<DType>(i);
            return true;
        }
    // signless/signed spellings that appear in StableHLO text
    if (s == "si8") { *out = DType::I8; return true; }
    if (s == "si16") { *out = DType::I16; return true; }
    if (s == "si32") { *out = DType::I32; return true; }
    if (s == "si64") { *out = DType::I64; return true; }
    return false;
}

std::string TensorType::str() const {
    std::string s = "tensor<";
    for (int64_t d : shape) s += std::to_string(d) + "x";
    return s + dtype_name(dtype) + ">";
}

std::vector<int64_t> Attr::as_ints() const {
    if (kind == Int) return {i};
    if (kind == IntArray) return ints;
    std::vector<int64_t> out;
    if (kind == Array)
        for (const Attr& e : elems) out.push_back(e.kind == Float ? static_cast<int64_t>(e.f) : e.i);
    if (kind == Dense && !is_float(dense_type.dtype)) {  // dense<[[0, 0], [1, 1]]> : tensor<2x2xi64>, row-major
        const size_t es = dtype_size(dense_type.dtype);
        const int64_t n = dense_type.count();
        for (int64_t k = 0; k < n && es > 0 && es <= 8; ++k) {
            const size_t at = splat ? 0 : static_cast<size_t>(k) * es;
            if (at + es > dense.size()) break;
            uint64_t raw = 0;
            for (size_t b = 0; b < es; ++b) raw |= static_cast<uint64_t>(dense[at + b]) << (8 * b);
            if (!is_unsigned(dense_type.dtype) && es < 8 && (raw >> (8 * es - 1)) & 1) raw |= ~0ull << (8 * es);
            out.push_back(static_cast<int64_t>(raw));
        }
    }
    return out;
}

namespace {

struct Lit {  // one scalar of a dense literal, before the element type is known
    bool is_float = false, is_hex = false, is_bool = false;
    int64_t i = 0;
    uint64_t u = 0;
    double f = 0;
};

struct DensePending {
    std::vector<Lit> lits;
    std::string raw_hex;  // "0x..." byte string form
    bool nested = false;  // had brackets (not a splat)
    bool pairs = false;   // elements written as (re, im)
};

class Parser {
  public:
    explicit Parser(const std::string& t) : s_(t) {}

    Module parse() {
        Module m;
        skip();
        if (peek_word("module")) {
            word();
            skip();
            if (cur() == '@') { ++p_; m.name = ident(); }
            else if (cur() == '"') m.name = string_lit();
            skip();
            if (peek_word("attributes")) { word(); skip(); skip_balanced('{', '}'); }
            expect('{');
            parse_module_body(m);
            expect('}');
        } else {
            parse_module_body(m);
        }
        if (m.functions.empty()) fail_parse("module has no func.func");
        return m;
    }

  private:
    const std::string& s_;
    size_t p_ = 0;
    Function* fn_ = nullptr;
    std::map<std::string, int> names_;

    // ---- character level ------------------------------------------------------------------------------
    char cur() const { return p_ < s_.size() ? s_[p_] : '\0'; }
    char at(size_t k) const { return p_ + k < s_.size() ? s_[p_ + k] : '\0'; }
    bool eof() { skip(); return p_ >= s_.size(); }
    void skip() {
        for (;;) {
            while (p_ < s_.size() && std::isspace(static_cast<unsigned char>(s_[p_]))) ++p_;
            if (cur() == '/' && at(1) == '/') {
                while (p_ < s_.size() && s_[p_] != '\n') ++p_;
                continue;
            }
            break;
        }
    }
    [[noreturn]] void error(const std::string& what) {
        int line = 1;
        for (size_t i = 0; i < p_ && i < s_.size(); ++i) line += s_[i] == '\n';
        std::string ctx = s_.substr(p_, 40);
        for (char& c : ctx) if (c == '\n') c = ' ';
        fail_parse("line " + std::to_string(line) + ": " + what + " near '" + ctx + "'");
    }
    void expect(char c) {
        skip();
        if (cur() != c) error(std::string("expected '") + c + "'");
        ++p_;
    }
    bool accept(char c) {
        skip();
        if (cur() == c) { ++p_; return true; }
        return false;
    }
    bool accept_str(const char* t) {
        skip();
        size_t n = std::strlen(t);
        if (s_.compare(p_, n, t) == 0) { p_ += n; return true; }
        return false;
    }
    static bool ident_char(char c) { return std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '.' || c == '$'; }
    std::string ident() {
        size_t b = p_;
        while (ident_char(cur())) ++p_;
        if (p_ == b) error("expected identifier");
        return s_.substr(b, p_ - b);
    }
    std::string word() { skip(); return ident(); }
    bool peek_word(const char* w) {
        skip();
        size_t n = std::strlen(w);
        return s_.compare(p_, n, w) == 0 && !ident_char(at(n));
    }
    std::string string_lit() {
        skip();
        if (cur() != '"') error("expected string");
        ++p_;
        std::string out;
        while (p_ < s_.size() && s_[p_] != '"') {
            if (s_[p_] == '\\' && p_ + 1 < s_.size()) {
                char n = s_[p_ + 1];
                if (n == 'n') { out += '\n'; p_ += 2; }
                else if (n == 't') { out += '\t'; p_ += 2; }
                else if (n == '"' || n == '\\') { out += n; p_ += 2; }
                else if (std::isxdigit(static_cast<unsigned char>(n)) && p_ + 2 < s_.size()) {
                    out += static_cast<char>(std::stoi(s_.substr(p_ + 1, 2), nullptr, 16));
                    p_ += 3;
                } else { out += n; p_ += 2; }
            } else {
                out += s_[p_++];
            }
        }
        if (cur() != '"') error("unterminated string");
        ++p_;
        return out;
    }
    void skip_balanced(char open, char close) {
        skip();
        if (cur() != open) error(std::string("expected '") + open + "'");
        int depth = 0;
        while (p_ < s_.size()) {
            char c = s_[p_];
            if (c == '"') { string_lit(); continue; }
            if (c == open) ++depth;
            else if (c == close && --depth == 0) { ++p_; return; }
            ++p_;
        }
        error("unbalanced delimiter");
    }
    std::string value_name() {
        skip();
        if (cur() != '%') error("expected SSA value");
        size_t b = p_++;
        while (ident_char(cur()) || cur() == '-') ++p_;
        if (cur() == '#' && std::isdigit(static_cast<unsigned char>(at(1)))) {
            ++p_;
            while (std::isdigit(static_cast<unsigned char>(cur()))) ++p_;
        }
        return s_.substr(b, p_ - b);
    }
    int lookup(const std::string& name) {
        auto it = names_.find(name);
        if (it == names_.end()) {
            // "%0" may name the first result of a multi-result op bound as "%0#0"
            it = names_.find(name + "#0");
            if (it == names_.end()) fail_parse("use of undefined value " + name);
        }
        return it->second;
    }

    // ---- numbers --------------------------------------------------------------------------------------
    Lit number() {
        skip();
        Lit l;
        if (peek_word("true")) { word(); l.is_bool = true; l.i = 1; l.u = 1; l.f = 1; return l; }
        if (peek_word("false")) { word(); l.is_bool = true; return l; }
        size_t b = p_;
        bool neg = false;
        if (cur() == '-' || cur() == '+') { neg = cur() == '-'; ++p_; }
        if (cur() == '0' && (at(1) == 'x' || at(1) == 'X')) {
            p_ += 2;
            size_t hb = p_;
            while (std::isxdigit(static_cast<unsigned char>(cur()))) ++p_;
            l.is_hex = true;
            l.u = std::stoull(s_.substr(hb, p_ - hb), nullptr, 16);
            l.i = static_cast<int64_t>(l.u);
            l.f = static_cast<double>(l.u);
            return l;
        }
        if (s_.compare(p_, 3, "inf") == 0) { p_ += 3; l.is_float = true; l.f = neg ? -INFINITY : INFINITY; return l; }
        if (s_.compare(p_, 3, "nan") == 0 || s_.compare(p_, 3, "NaN") == 0) { p_ += 3; l.is_float = true; l.f = NAN; return l; }
        while (std::isdigit(static_cast<unsigned char>(cur()))) ++p_;
        if (cur() == '.' || cur() == 'e' || cur() == 'E') {
            l.is_float = true;
            if (cur() == '.') { ++p_; while (std::isdigit(static_cast<unsigned char>(cur()))) ++p_; }
            if (cur() == 'e' || cur() == 'E') {
                ++p_;
                if (cur() == '-' || cur() == '+') ++p_;
                while (std::isdigit(static_cast<unsigned char>(cur()))) ++p_;
            }
        }
        std::string t = s_.substr(b, p_ - b);
        if (t.empty() || t == "-" || t == "+") error("expected number");
        if (l.is_float) {
            l.f = std::strtod(t.c_str(), nullptr);
        } else {
            if (neg) { l.i = std::strtoll(t.c_str(), nullptr, 10); l.u = static_cast<uint64_t>(l.i); }
            else { l.u = std::strtoull(t.c_str(), nullptr, 10); l.i = static_cast<int64_t>(l.u); }
            l.f = neg ? static_cast<double>(l.i) : static_cast<double>(l.u);
        }
        return l;
    }

    // ---- types ----------------------------------------------------------------------------------------
    bool at_type() {
        skip();
        return peek_word("tensor") || peek_word("tuple") || peek_word("none") || peek_word("index") ||
               peek_word("!stablehlo.token") || (cur() == '!' );
    }
    TensorType type() {
        skip();
        if (cur() == '!') {  // !stablehlo.token and friends: carried as an empty i1 tensor
            while (ident_char(cur()) || cur() == '!') ++p_;
            if (cur() == '<') skip_balanced('<', '>');
            TensorType t; t.dtype = DType::I1; return t;
        }
        std::string w = ident();
        if (w == "tuple") {  // tuples are flattened by the callers that can meet them; keep the first element
            expect('<');
            TensorType first;
            bool have = false;
            skip();
            while (cur() != '>') {
                TensorType t = type();
                if (!have) { first = t; have = true; }
                if (!accept(',')) break;
                skip();
            }
            expect('>');
            return first;
        }
        if (w != "tensor") {
            DType d;
            if (dtype_from_name(w, &d)) { TensorType t; t.dtype = d; return t; }  // bare scalar type
            error("unsupported type '" + w + "'");
        }
        expect('<');
        TensorType t;
        for (;;) {
            skip();
            if (std::isdigit(static_cast<unsigned char>(cur()))) {
                size_t b = p_;
                while (std::isdigit(static_cast<unsigned char>(cur()))) ++p_;
                if (cur() == 'x') {
                    t.shape.push_back(std::stoll(s_.substr(b, p_ - b)));
                    ++p_;
                    continue;
                }
                error("malformed tensor shape");
            }
            if (cur() == '?' || cur() == '*') error("dynamic shapes are not supported");
            break;
        }
        std::string e = ident();
        if (e == "complex") {  // stored as (re, im) pairs of the part type: one more dimension of extent 2
            expect('<');
            e = ident();
            expect('>');
            if (e != "f32" && e != "f64") error("complex<" + e + "> is not supported (complex<f32> and complex<f64> are)");
            t.shape.push_back(2);
            t.was_complex = true;
        }
        if (!dtype_from_name(e, &t.dtype)) error("unsupported element type '" + e + "'");
        skip();
        if (cur() == ',') { ++p_; skip(); while (cur() != '>' && p_ < s_.size()) { if (cur() == '<') skip_balanced('<', '>'); else ++p_; } }  // encoding attr
        expect('>');
        return t;
    }
    // "(t, t) -> t", "(t) -> (t, t)", "t", "t, t" (select's pred/result pair): returns (inputs, results)
    void signature(std::vector<TensorType>* ins, std::vector<TensorType>* outs) {
        skip();
        if (cur() == '(') {
            ++p_;
            skip();
            while (cur() != ')') {
                ins->push_back(type());
                if (!accept(',')) break;
                skip();
            }
            expect(')');
            if (!accept_str("->")) error("expected '->' in function type");
            skip();
            if (cur() == '(') {
                ++p_;
                skip();
                while (cur() != ')') {
                    outs->push_back(type());
                    if (!accept(',')) break;
                    skip();
                }
                expect(')');
            } else {
                outs->push_back(type());
            }
            return;
        }
        // bare type list: every type is both an operand type and (the last one) the result type
        std::vector<TensorType> ts;
        ts.push_back(type());
        while (accept(',')) ts.push_back(type());
        if (accept_str("->")) {  // "t -> t"
            *ins = ts;
            skip();
            if (cur() == '(') {
                ++p_;
                skip();
                while (cur() != ')') { outs->push_back(type()); if (!accept(',')) break; skip(); }
                expect(')');
            } else outs->push_back(type());
            return;
        }
        *ins = ts;
        outs->push_back(ts.back());
    }

    // ---- attributes -----------------------------------------------------------------------------------
    DensePending dense_body() {  // after "dense<", consumes through '>'
        DensePending d;
        skip();
        if (cur() == '>') { ++p_; return d; }
        if (cur() == '"') {
            d.raw_hex = string_lit();
            expect('>');
            return d;
        }
        int depth = 0;
        for (;;) {
            skip();
            if (cur() == '[') { ++depth; ++p_; d.nested = true; continue; }
            if (cur() == ']') { --depth; ++p_; continue; }
            if (cur() == ',') { ++p_; continue; }
            if (cur() == '>' && depth == 0) { ++p_; break; }
            if (cur() == '(' || cur() == ')') { ++p_; d.pairs = true; continue; }  // (re, im) of a complex element
            d.lits.push_back(number());
        }
        return d;
    }
    Attr finalize_dense(const DensePending& d, const TensorType& t) {
        Attr a;
        a.kind = Attr::Dense;
        a.dense_type = t;
        const size_t es = dtype_size(t.dtype);
        const int64_t n = t.count();
        if (!d.raw_hex.empty()) {
            if (d.raw_hex.size() < 2 || d.raw_hex[0] != '0' || (d.raw_hex[1] != 'x' && d.raw_hex[1] != 'X'))
                fail_parse("dense string constant must start with 0x");
            std::vector<uint8_t> raw;
            for (size_t i = 2; i + 1 < d.raw_hex.size(); i += 2)
                raw.push_back(static_cast<uint8_t>(std::stoi(d.raw_hex.substr(i, 2), nullptr, 16)));
            if (raw.size() == es && n != 1) { a.splat = true; a.dense = raw; return a; }
            if (static_cast<int64_t>(raw.size()) != n * static_cast<int64_t>(es))
                fail_parse("dense hex constant has " + std::to_string(raw.size()) + " bytes, type " + t.str() +
                           " needs " + std::to_string(n * es));
            a.dense = raw;
            return a;
        }
        if (d.lits.empty()) {
            if (n != 0) fail_parse("empty dense<> for non-empty type " + t.str());
            return a;
        }
        if (t.was_complex && d.lits.size() == 2 && n != 2 && !d.nested) {  // one (re, im) for every element
            DensePending all;
            all.nested = true;
            for (int64_t k = 0; k < n / 2; ++k) { all.lits.push_back(d.lits[0]); all.lits.push_back(d.lits[1]); }
            return finalize_dense(all, t);
        }
        const bool splat = d.lits.size() == 1 && (n != 1 || !d.nested);
        if (!splat && static_cast<int64_t>(d.lits.size()) != n)
            fail_parse("dense literal has " + std::to_string(d.lits.size()) + " elements, type " + t.str() +
                       " needs " + std::to_string(n));
        a.splat = splat && n != 1;
        a.dense.resize(d.lits.size() * es);
        for (size_t k = 0; k < d.lits.size(); ++k) {
            const Lit& l = d.lits[k];
            uint8_t* dst = a.dense.data() + k * es;
            if (is_float(t.dtype)) {
                if (l.is_hex) {  // hex integers inside a float dense<> are IEEE bit patterns
                    uint64_t bits = l.u;
                    std::memcpy(dst, &bits, es);
                } else {
                    encode_float(t.dtype, l.f, dst);
                }
            } else if (t.dtype == DType::I1) {
                dst[0] = (l.is_float ? l.f != 0 : l.u != 0) ? 1 : 0;
            } else {
                int64_t v = l.is_float ? static_cast<int64_t>(l.f) : l.i;
                std::memcpy(dst, &v, es);  // little endian: low bytes first
            }
        }
        return a;
    }

    Attr attr_value() {
        skip();
        char c = cur();
        if (c == '"') {
            Attr a = Attr::make_string(string_lit());
            maybe_type_suffix();
            return a;
        }
        if (c == '[') {
            ++p_;
            Attr a;
            a.kind = Attr::Array;
            skip();
            while (cur() != ']') {
                a.elems.push_back(attr_value());
                if (!accept(',')) break;
                skip();
            }
            expect(']');
            bool all_int = true;
            for (const Attr& e : a.elems) all_int &= e.kind == Attr::Int;
            if (all_int) {
                Attr r = Attr::make_ints({});
                for (const Attr& e : a.elems) r.ints.push_back(e.i);
                return r;
            }
            return a;
        }
        if (c == '{') return attr_dict('{', '}');
        if (c == '#') {  // #stablehlo.dot<...>, #stablehlo<comparison_direction GT>, #stablehlo.gather<...>
            ++p_;
            std::string tag = ident();
            skip();
            if (cur() != '<') { Attr a; a.kind = Attr::Keyword; a.s = tag; return a; }
            size_t save = p_;
            ++p_;
            skip();
            if (tag == "stablehlo.conv" && cur() == '[') {
                Attr a = conv_dimension_spec();
                expect('>');
                return a;
            }
            // enum form: "<comparison_direction GT>" / "<precision DEFAULT>"
            if (ident_char(cur())) {
                size_t q = p_;
                std::string first = ident();
                skip();
                if (cur() != '=' ) {
                    Attr a;
                    a.kind = Attr::Keyword;
                    if (ident_char(cur())) a.s = ident(); else a.s = first;
                    skip();
                    while (cur() != '>' && p_ < s_.size()) ++p_;
                    expect('>');
                    return a;
                }
                p_ = q;
            }
            p_ = save;
            return attr_dict('<', '>');
        }
        if (peek_word("dense")) {
            word();
            expect('<');
            DensePending d = dense_body();
            expect(':');
            TensorType t = type();
            return finalize_dense(d, t);
        }
        if (peek_word("array")) {  // array<i64: 1, 2> / array<i64>
            word();
            expect('<');
            word();
            Attr a = Attr::make_ints({});
            if (accept(':')) {
                skip();
                while (cur() != '>') {
                    Lit l = number();
                    a.ints.push_back(l.is_float ? static_cast<int64_t>(l.f) : l.i);
                    if (!accept(',')) break;
                }
            }
            expect('>');
            return a;
        }
        if (peek_word("true") || peek_word("false")) { Attr a = Attr::make_bool(word() == "true"); return a; }
        if (peek_word("unit")) { word(); return Attr::make_bool(true); }
        if (c == '@') { ++p_; Attr a; a.kind = Attr::Keyword; a.s = ident(); return a; }
        if (std::isdigit(static_cast<unsigned char>(c)) || c == '-' || c == '+') {
            Lit l = number();
            Attr a = l.is_float ? Attr::make_float(l.f) : Attr::make_int(l.i);
            maybe_type_suffix();
            return a;
        }
        if (at_type()) { TensorType t = type(); Attr a; a.kind = Attr::Keyword; a.s = t.str(); return a; }
        if (ident_char(c)) {
            Attr a;
            a.kind = Attr::Keyword;
            a.s = ident();
            skip();
            if (cur() == '<') skip_balanced('<', '>');
            return a;
        }
        error("unsupported attribute syntax");
    }
    // Convolution layout "[b, 0, 1, f]x[0, 1, i, o]->[b, 0, 1, f]" (input x kernel -> output; b = batch, f = feature,
    // i / o = kernel input / output feature, k = spatial dimension k) as a dictionary of the nine dimension attributes.
    Attr conv_dimension_spec() {
        Attr d;
        d.kind = Attr::Dict;
        auto side = [&](const char* batch_key, char batch_c, const char* feature_key, char feature_c, const char* spatial_key) {
            skip();
            expect('[');
            std::map<int64_t, int64_t> spatial;
            int64_t pos = 0;
            skip();
            while (cur() != ']') {
                if (std::isdigit(static_cast<unsigned char>(cur()))) {
                    spatial[number().i] = pos;
                } else {
                    const std::string w = ident();
                    if (w.size() != 1 || (w[0] != batch_c && w[0] != feature_c)) error("unexpected '" + w + "' in a convolution layout");
                    d.dict[w[0] == batch_c ? batch_key : feature_key] = Attr::make_int(pos);
                }
                ++pos;
                if (!accept(',')) break;
                skip();
            }
            expect(']');
            std::vector<int64_t> sp;
            for (const auto& kv : spatial) sp.push_back(kv.second);
            d.dict[spatial_key] = Attr::make_ints(sp);
        };
        side("input_batch_dimension", 'b', "input_feature_dimension", 'f', "input_spatial_dimensions");
        skip();
        if (cur() != 'x') error("expected 'x' in a convolution layout");
        ++p_;
        side("kernel_input_feature_dimension", 'i', "kernel_output_feature_dimension", 'o', "kernel_spatial_dimensions");
        skip();
        if (!accept_str("->")) error("expected '->' in a convolution layout");
        side("output_batch_dimension", 'b', "output_feature_dimension", 'f', "output_spatial_dimensions");
        return d;
    }

    void maybe_type_suffix() {  // "1 : i64", "1.0 : f32", "0 : index"; a tensor type after ':' belongs to the op
        size_t save = p_;
        skip();
        if (cur() == ':') {
            ++p_;
            skip();
            if (ident_char(cur())) {
                std::string w = ident();
                DType d;
                if (dtype_from_name(w, &d) || w == "index") return;
            }
        }
        p_ = save;
    }
    Attr attr_dict(char open, char close) {
        expect(open);
        Attr a;
        a.kind = Attr::Dict;
        skip();
        while (cur() != close) {
            std::string key;
            skip();
            if (cur() == '"') key = string_lit(); else key = ident();
            // strip dialect prefixes on discardable attributes (mhlo.sharding, stablehlo.foo)
            skip();
            if (cur() == '=') {
                ++p_;
                a.dict[key] = attr_value();
            } else {
                a.dict[key] = Attr::make_bool(true);  // unit attribute
            }
            if (!accept(',')) break;
            skip();
        }
        expect(close);
        return a;
    }

    // ---- module / function ----------------------------------------------------------------------------
    void parse_module_body(Module& m) {
        for (;;) {
            skip();
            if (p_ >= s_.size() || cur() == '}') return;
            if (peek_word("func.func")) {
                m.functions.push_back(function());
            } else {
                // anything else at module level (sdy.mesh, attribute aliases) is skipped statement-wise
                while (p_ < s_.size() && cur() != '\n') {
                    if (cur() == '{') { skip_balanced('{', '}'); continue; }
                    if (cur() == '<') { skip_balanced('<', '>'); continue; }
                    ++p_;
                }
            }
        }
    }

    Function function() {
        word();  // func.func
        skip();
        if (peek_word("private") || peek_word("public")) word();
        expect('@');
        Function f;
        f.name = ident();
        fn_ = &f;
        names_.clear();
        expect('(');
        skip();
        while (cur() != ')') {
            std::string n = value_name();
            expect(':');
            TensorType t = type();
            skip();
            if (cur() == '{') skip_balanced('{', '}');  // argument attributes
            skip();
            if (peek_word("loc")) { word(); skip_balanced('(', ')'); }
            int v = f.new_value(t, n);
            f.args.push_back(v);
            names_[n] = v;
            if (!accept(',')) break;
            skip();
        }
        expect(')');
        if (accept_str("->")) {
            skip();
            if (cur() == '(') {
                ++p_;
                skip();
                while (cur() != ')') {
                    f.result_types.push_back(type());
                    skip();
                    if (cur() == '{') skip_balanced('{', '}');
                    if (!accept(',')) break;
                    skip();
                }
                expect(')');
            } else {
                f.result_types.push_back(type());
                skip();
                if (cur() == '{') { /* result attrs or body? a body starts a new line with ops; attrs are {name = ..} */
                    size_t save = p_;
                    ++p_;
                    skip();
                    bool is_attr = ident_char(cur()) && !peek_word("return") && !peek_word("func.return") &&
                                   !peek_word("stablehlo.return") && s_.compare(p_, 10, "stablehlo.") != 0 &&
                                   s_.compare(p_, 5, "chlo.") != 0;
                    if (is_attr) {
                        // could still be an op like "check.expect..": attribute dicts always have '=' or ',' or '}' next
                        size_t q = p_;
                        ident();
                        skip();
                        is_attr = cur() == '=' || cur() == '}' || cur() == ',';
                        p_ = q;
                    }
                    p_ = save;
                    if (is_attr) skip_balanced('{', '}');
                }
            }
        }
        skip();
        if (peek_word("attributes")) { word(); skip(); skip_balanced('{', '}'); }
        expect('{');
        block(&f.ops, /*top=*/true);
        expect('}');
        if (f.ops.empty() || f.ops.back().name != "return") {
            Op r;
            r.name = "return";
            r.dialect = "func";
            f.ops.push_back(r);
        }
        if (f.result_types.empty())
            for (int v : f.ops.back().operands) f.result_types.push_back(f.values[v].type);
        for (size_t i = 0; i < f.ops.size(); ++i)
            for (size_t r = 0; r < f.ops[i].results.size(); ++r) {
                f.values[f.ops[i].results[r]].def_op = static_cast<int>(i);
                f.values[f.ops[i].results[r]].def_result = static_cast<int>(r);
            }
        fn_ = nullptr;
        return f;
    }

    // Parses operations until the closing '}' of the enclosing block (not consumed).
    void block(std::vector<Op>* ops, bool top) {
        for (;;) {
            skip();
            if (p_ >= s_.size()) error("unexpected end of input inside a block");
            if (cur() == '}') return;
            if (cur() == '^') {  // block label with arguments: ^bb0(%a: t, %b: t):
                while (cur() != '(' && cur() != ':') ++p_;
                if (cur() == '(') {
                    ++p_;
                    skip();
                    while (cur() != ')') {
                        std::string n = value_name();
                        expect(':');
                        TensorType t = type();
                        skip();
                        if (peek_word("loc")) { word(); skip_balanced('(', ')'); }
                        int v = fn_->new_value(t, n);
                        names_[n] = v;
                        pending_block_args_.push_back(v);
                        if (!accept(',')) break;
                        skip();
                    }
                    expect(')');
                }
                expect(':');
                continue;
            }
            ops->push_back(operation());
            (void)top;
        }
    }
    std::vector<int> pending_block_args_;

    std::shared_ptr<Region> region() {  // at '{'
        expect('{');
        auto r = std::make_shared<Region>();
        std::vector<int> saved;
        saved.swap(pending_block_args_);
        block(&r->ops, false);
        r->args = pending_block_args_;
        pending_block_args_.swap(saved);
        expect('}');
        return r;
    }

    // ---- operations -----------------------------------------------------------------------------------
    Op operation() {
        skip();
        std::vector<std::string> result_names;
        int declared_results = -1;
        if (cur() == '%') {
            for (;;) {
                std::string n = value_name();
                skip();
                if (cur() == ':' && std::isdigit(static_cast<unsigned char>(at(1)))) {  // %0:2
                    ++p_;
                    Lit l = number();
                    declared_results = static_cast<int>(l.i);
                }
                result_names.push_back(n);
                if (!accept(',')) break;
            }
            expect('=');
        }
        skip();
        Op op;
        std::vector<TensorType> in_types;
        if (cur() == '"') {
            std::string full = string_lit();
            split_name(full, &op);
            generic_op(&op, &in_types);
        } else {
            std::string full = ident();
            split_name(full, &op);
            pretty_op(&op, &in_types);
        }
        skip();
        if (peek_word("loc")) { word(); skip_balanced('(', ')'); }
        // bind results
        if (declared_results > 0 && result_names.size() == 1) {
            if (static_cast<int>(op.result_types.size()) < declared_results)
                op.result_types.resize(declared_results, op.result_types.empty() ? TensorType() : op.result_types[0]);
            for (int r = 0; r < declared_results; ++r) {
                std::string n = result_names[0] + "#" + std::to_string(r);
                int v = fn_->new_value(op.result_types[r], n);
                op.results.push_back(v);
                names_[n] = v;
            }
        } else {
            if (result_names.size() > 1 && op.result_types.size() == 1 && in_types.size() == result_names.size())
                op.result_types = in_types;  // "%a, %b = op %x, %y : t0, t1": one type per result
            if (op.result_types.size() < result_names.size())
                fail_parse("operation " + op.name + " binds " + std::to_string(result_names.size()) +
                           " results but its type lists " + std::to_string(op.result_types.size()));
            op.result_types.resize(result_names.size());
            for (size_t r = 0; r < result_names.size(); ++r) {
                int v = fn_->new_value(op.result_types[r], result_names[r]);
                op.results.push_back(v);
                names_[result_names[r]] = v;
            }
        }
        return op;
    }

    static void split_name(const std::string& full, Op* op) {
        size_t dot = full.find('.');
        if (dot == std::string::npos) { op->dialect = ""; op->name = full; }
        else { op->dialect = full.substr(0, dot); op->name = full.substr(dot + 1); }
        if (full == "return" || full == "func.return" || full == "stablehlo.return") op->name = "return";
        if (full == "func.call" || full == "call") { op->name = "call"; op->dialect = "func"; }
    }

    void operand_list(Op* op, char close) {
        skip();
        while (cur() != close) {
            op->operands.push_back(lookup(value_name()));
            if (!accept(',')) break;
            skip();
        }
        expect(close);
    }

    void merge_attrs(Op* op, const Attr& dict) {
        for (const auto& kv : dict.dict) op->attrs[kv.first] = kv.second;
    }

    // "stablehlo.op"(%a, %b) <{props}> ({region}, {region}) {attrs} : (types) -> types
    void generic_op(Op* op, std::vector<TensorType>* in_types) {
        expect('(');
        operand_list(op, ')');
        skip();
        if (cur() == '<' && at(1) == '{') {
            ++p_;
            merge_attrs(op, attr_dict('{', '}'));
            expect('>');
        }
        skip();
        if (cur() == '(' ) {
            size_t save = p_;
            ++p_;
            skip();
            if (cur() == '{') {
                for (;;) {
                    op->regions.push_back(region());
                    if (!accept(',')) break;
                }
                expect(')');
            } else {
                p_ = save;
            }
        }
        skip();
        if (cur() == '{') merge_attrs(op, attr_dict('{', '}'));
        expect(':');
        signature(in_types, &op->result_types);
        normalise(op);
    }

    // stablehlo.op <items> {attrs} : signature, where an item is an operand, a keyword, key = value, a slice
    // spec, a dense literal, @symbol(operands) or a parenthesised reduce operand group.
    void pretty_op(Op* op, std::vector<TensorType>* in_types) {
        DensePending dense;
        bool have_dense = false;
        std::vector<std::string> keywords;
        if (op->name == "reduce" && accept('(')) {  // stablehlo.reduce(%x init: %i), (%y init: %j) applies ...
            std::vector<int> inputs, inits;
            for (;;) {
                inputs.push_back(lookup(value_name()));
                skip();
                if (!accept_str("init")) error("expected 'init:' in reduce");
                expect(':');
                inits.push_back(lookup(value_name()));
                expect(')');
                if (accept(',')) { expect('('); continue; }
                break;
            }
            op->operands = inputs;
            op->operands.insert(op->operands.end(), inits.begin(), inits.end());
        } else if (op->name == "while" && accept('(')) {
            // stablehlo.while(%iter = %init, ...) : types [attributes {...}] cond {..} do {..}
            // The iteration arguments are block arguments shared by both regions (regions[0] = cond, regions[1] = body).
            std::vector<int> iter_vals;
            skip();
            while (cur() != ')') {
                std::string n = value_name();
                expect('=');
                int v = lookup(value_name());
                op->operands.push_back(v);
                int bv = fn_->new_value(fn_->values[v].type, n);
                names_[n] = bv;
                iter_vals.push_back(bv);
                if (!accept(',')) break;
                skip();
            }
            expect(')');
            skip();
            if (accept(':')) {
                for (;;) {
                    op->result_types.push_back(type());
                    skip();
                    if (!accept(',')) break;
                }
            }
            skip();
            if (peek_word("attributes")) { word(); skip(); merge_attrs(op, attr_dict('{', '}')); skip(); }
            for (const char* introducer : {"cond", "do"}) {
                skip();
                if (!peek_word(introducer)) error(std::string("expected '") + introducer + "' region of stablehlo.while");
                word();
                skip();
                auto r = region();
                r->args = iter_vals;
                op->regions.push_back(r);
            }
            for (size_t i = 0; i < iter_vals.size() && i < op->result_types.size(); ++i) fn_->values[iter_vals[i]].type = op->result_types[i];
            return;
        }
        for (;;) {
            skip();
            char c = cur();
            if (c == ':' || c == '{' || c == '\0' || c == '}') break;
            if (c == ',') { ++p_; continue; }
            if (c == '%') { op->operands.push_back(lookup(value_name())); continue; }
            if (c == '@') {  // custom_call @target(%a, %b)
                ++p_;
                op->attrs["call_target_name"] = Attr::make_string(ident());
                if (op->name == "call") op->attrs["callee"] = op->attrs["call_target_name"];
                skip();
                if (cur() == '(') { ++p_; operand_list(op, ')'); }
                continue;
            }
            if (c == '[') {  // slice spec [a:b:c, ...] or a bare index list
                ++p_;
                std::vector<int64_t> start, limit, stride, plain;
                bool is_slice = false;
                skip();
                while (cur() != ']') {
                    Lit a = number();
                    skip();
                    if (cur() == ':') {
                        is_slice = true;
                        ++p_;
                        Lit b = number();
                        int64_t st = 1;
                        skip();
                        if (cur() == ':') { ++p_; st = number().i; }
                        start.push_back(a.i); limit.push_back(b.i); stride.push_back(st);
                    } else {
                        plain.push_back(a.i);
                    }
                    if (!accept(',')) break;
                    skip();
                }
                expect(']');
                if (is_slice) {
                    op->attrs["start_indices"] = Attr::make_ints(start);
                    op->attrs["limit_indices"] = Attr::make_ints(limit);
                    op->attrs["strides"] = Attr::make_ints(stride);
                } else {
                    op->attrs["indices"] = Attr::make_ints(plain);
                }
                continue;
            }
            if (c == '(') {  // reducer(...) block header of the pretty reduce with a region, or call operands
                if (op->name == "call" || op->name == "convolution") { ++p_; operand_list(op, ')'); continue; }
                if (op->name == "top_k") {  // chlo.top_k(%x, k = 5)
                    ++p_;
                    skip();
                    while (cur() != ')') {
                        if (cur() == '%') {
                            op->operands.push_back(lookup(value_name()));
                        } else {
                            const std::string key = ident();
                            expect('=');
                            op->attrs[key] = attr_value();
                        }
                        if (!accept(',')) break;
                        skip();
                    }
                    expect(')');
                    continue;
                }
                skip_balanced('(', ')');
                continue;
            }
            if (c == '<' && at(1) == '{') { ++p_; merge_attrs(op, attr_dict('{', '}')); expect('>'); continue; }
            if (peek_word("dense")) {
                word();
                expect('<');
                dense = dense_body();
                have_dense = true;
                continue;
            }
            if (ident_char(c)) {
                size_t save = p_;
                std::string w = ident();
                skip();
                if (w == "applies") {  // applies stablehlo.add across dimensions = [1]
                    std::string r = ident();
                    op->attrs["reducer"] = Attr::make_string(r.substr(r.find('.') + 1));
                    continue;
                }
                if (w == "across") continue;
                if (w == "reducer" || w == "cond" || w == "do") {  // region introducer
                    if (w == "reducer") { while (cur() == '(') { skip_balanced('(', ')'); skip(); } }
                    if (cur() == '{') op->regions.push_back(region());
                    continue;
                }
                if (cur() == '=') {
                    ++p_;
                    skip();
                    // "batching_dims = [0] x [0]" style pairs
                    if (w == "dim_numbers") {  // [b, 0, 1, f]x[0, 1, i, o]->[b, 0, 1, f]
                        op->attrs["dimension_numbers"] = conv_dimension_spec();
                        continue;
                    }
                    Attr v = attr_value();
                    skip();
                    if (cur() == 'x' && !ident_char(at(1))) {
                        ++p_;
                        Attr rhs = attr_value();
                        op->attrs[w + ".lhs"] = v;
                        op->attrs[w + ".rhs"] = rhs;
                    } else {
                        op->attrs[w] = v;
                    }
                    continue;
                }
                (void)save;
                keywords.push_back(w);
                continue;
            }
            if (c == '#') { op->attrs["_attr" + std::to_string(op->attrs.size())] = attr_value(); continue; }
            if (c == '"') { keywords.push_back(string_lit()); continue; }
            error("unexpected token in operation " + op->name);
        }
        skip();
        if (cur() == '{') {
            // attribute dictionary or (for reduce/while in pretty form) a region
            size_t save = p_;
            ++p_;
            skip();
            bool looks_like_region = cur() == '^' || cur() == '%' || s_.compare(p_, 10, "stablehlo.") == 0 ||
                                     peek_word("return") || peek_word("func.return");
            p_ = save;
            if (looks_like_region) op->regions.push_back(region());
            else merge_attrs(op, attr_dict('{', '}'));
        }
        skip();
        if (op->name == "return") {
            if (accept(':')) { std::vector<TensorType> outs; signature(in_types, &outs); }
            return;
        }
        if (cur() == ':') {
            ++p_;
            signature(in_types, &op->result_types);
        }
        skip();
        if (op->name == "reduce" && peek_word("reducer")) {
            // jax prints the body after the type: reducer(%a: t, %b: t) (%c: t, %d: t) { ... }
            word();
            std::vector<int> args;
            skip();
            while (cur() == '(') {
                ++p_;
                skip();
                while (cur() != ')') {
                    std::string n = value_name();
                    expect(':');
                    TensorType t = type();
                    skip();
                    if (peek_word("loc")) { word(); skip_balanced('(', ')'); }
                    int v = fn_->new_value(t, n);
                    names_[n] = v;
                    args.push_back(v);
                    if (!accept(',')) break;
                    skip();
                }
                expect(')');
                skip();
            }
            auto r = region();
            // the printed order is (lhs0, rhs0) (lhs1, rhs1): block arguments are lhs0, lhs1, rhs0, rhs1
            std::vector<int> ordered;
            for (size_t k = 0; k < args.size(); k += 2) ordered.push_back(args[k]);
            for (size_t k = 1; k < args.size(); k += 2) ordered.push_back(args[k]);
            r->args = ordered;
            op->regions.push_back(r);
        }
        if (have_dense) {
            if (op->result_types.empty()) fail_parse("constant without a type");
            op->attrs["value"] = finalize_dense(dense, op->result_types[0]);
        }
        if (!keywords.empty()) {
            Attr k;
            k.kind = Attr::Array;
            for (const std::string& w : keywords) { Attr e; e.kind = Attr::Keyword; e.s = w; k.elems.push_back(e); }
            op->attrs["_keywords"] = k;
        }
        // select prints "pred_type, value_type": the result is the value type
        normalise(op);
    }

    // Brings the attribute spellings of the pretty and generic forms to one canonical set.
    void normalise(Op* op) {
        auto rename = [&](const char* from, const char* to) {
            auto it = op->attrs.find(from);
            if (it != op->attrs.end() && !op->attrs.count(to)) { op->attrs[to] = it->second; op->attrs.erase(from); }
        };
        const std::string& n = op->name;
        if (n == "constant") {
            const Attr* v = op->attr("value");
            if (v && v->kind == Attr::Dense && !op->result_types.empty() && v->dense_type != op->result_types[0] &&
                v->dense_type.count() == op->result_types[0].count()) {
                op->attrs["value"].dense_type = op->result_types[0];
            }
        }
        if (n == "broadcast_in_dim" || n == "transpose" || n == "reverse") {
            rename("dims", n == "broadcast_in_dim" ? "broadcast_dimensions" : (n == "transpose" ? "permutation" : "dimensions"));
            rename("dimensions", n == "broadcast_in_dim" ? "broadcast_dimensions" : (n == "transpose" ? "permutation" : "dimensions"));
        }
        if (n == "concatenate" || n == "get_dimension_size") { rename("dim", "dimension"); }
        if (n == "fft") { rename("type", "fft_type"); rename("length", "fft_length"); }
        if (n == "iota" || n == "dynamic_iota") { rename("dim", "iota_dimension"); rename("dimension", "iota_dimension"); }
        if (n == "reduce") {
            rename("dims", "dimensions");
            // classify the reducer region when there is no `applies` clause
            if (!op->attr("reducer") && !op->regions.empty()) op->attrs["reducer"] = Attr::make_string(classify_reducer(*op->regions[0]));
        }
        if (n == "compare") {
            if (const Attr* kw = op->attr("_keywords")) {
                for (const Attr& e : kw->elems) {
                    if (e.s == "EQ" || e.s == "NE" || e.s == "LT" || e.s == "LE" || e.s == "GT" || e.s == "GE")
                        op->attrs["comparison_direction"] = Attr::make_string(e.s);
                    else if (e.s == "FLOAT" || e.s == "SIGNED" || e.s == "UNSIGNED" || e.s == "TOTALORDER")
                        op->attrs["compare_type"] = Attr::make_string(e.s);
                }
            }
            for (const char* k : {"comparison_direction", "compare_type"})
                if (const Attr* a = op->attr(k))
                    if (a->kind == Attr::Keyword) op->attrs[k] = Attr::make_string(a->s);
        }
        if (n == "dot_general") {
            if (const Attr* d = op->attr("dot_dimension_numbers")) {
                for (const char* k : {"lhs_batching_dimensions", "rhs_batching_dimensions", "lhs_contracting_dimensions",
                                      "rhs_contracting_dimensions"})
                    if (const Attr* x = d->get(k)) op->attrs[k] = Attr::make_ints(x->as_ints());
            }
            for (const Attr* d : {op->attr("_attr0"), op->attr("_attr1")})
                if (d && d->kind == Attr::Dict)
                    for (const char* k : {"lhs_batching_dimensions", "rhs_batching_dimensions",
                                          "lhs_contracting_dimensions", "rhs_contracting_dimensions"})
                        if (const Attr* x = d->get(k)) op->attrs[k] = Attr::make_ints(x->as_ints());
            auto pair = [&](const char* base, const char* l, const char* r) {
                if (const Attr* a = op->attr(std::string(base) + ".lhs")) op->attrs[l] = Attr::make_ints(a->as_ints());
                if (const Attr* a = op->attr(std::string(base) + ".rhs")) op->attrs[r] = Attr::make_ints(a->as_ints());
            };
            pair("batching_dims", "lhs_batching_dimensions", "rhs_batching_dimensions");
            pair("contracting_dims", "lhs_contracting_dimensions", "rhs_contracting_dimensions");
            for (const char* k : {"lhs_batching_dimensions", "rhs_batching_dimensions", "lhs_contracting_dimensions",
                                  "rhs_contracting_dimensions"})
                if (!op->attr(k)) op->attrs[k] = Attr::make_ints({});
        }
        if (n == "gather" || n == "dynamic_gather" || n == "scatter") {
            const char* key = n == "scatter" ? "scatter_dimension_numbers" : "dimension_numbers";
            if (const Attr* d = op->attr(key))
                for (const auto& kv : d->dict) op->attrs[kv.first] = kv.second.kind == Attr::Int || kv.second.kind == Attr::IntArray || kv.second.kind == Attr::Array ? (kv.second.kind == Attr::Int ? kv.second : Attr::make_ints(kv.second.as_ints())) : kv.second;
        }
        if (n == "reduce_window" && !op->attr("reducer") && !op->regions.empty())
            op->attrs["reducer"] = Attr::make_string(classify_reducer(*op->regions[0]));
        if (n == "scatter" && !op->attr("reducer") && !op->regions.empty()) {
            // the update computation takes (current, update): returning the update itself is an assignment
            const Region& r = *op->regions[0];
            if (r.ops.size() == 1 && r.ops[0].name == "return" && r.args.size() == 2 && r.ops[0].operands.size() == 1 &&
                r.ops[0].operands[0] == r.args[1])
                op->attrs["reducer"] = Attr::make_string("set");
            else
                op->attrs["reducer"] = Attr::make_string(r.ops.size() == 2 ? classify_reducer(r) : "unknown");
        }
        if (n == "select_and_scatter" && op->regions.size() == 2) {
            // select(a, b): one compare of the two arguments; scatter(a, b): one arithmetic op
            const Region& sel = *op->regions[0];
            std::string dir = "unknown";
            if (sel.ops.size() == 2 && sel.ops[0].name == "compare" && sel.args.size() == 2 && sel.ops[1].name == "return" &&
                sel.ops[1].operands.size() == 1 && sel.ops[1].operands[0] == sel.ops[0].results[0]) {
                const Op& c = sel.ops[0];
                dir = c.str_attr("comparison_direction");
                if (c.operands[0] == sel.args[1] && c.operands[1] == sel.args[0])  // b <dir> a  ==  a <mirrored dir> b
                    dir = dir == "GE" ? "LE" : dir == "GT" ? "LT" : dir == "LE" ? "GE" : dir == "LT" ? "GT" : "unknown";
                else if (!(c.operands[0] == sel.args[0] && c.operands[1] == sel.args[1]))
                    dir = "unknown";
            }
            op->attrs["select_direction"] = Attr::make_string(dir);
            op->attrs["reducer"] = Attr::make_string(op->regions[1]->ops.size() == 2 ? classify_reducer(*op->regions[1]) : "unknown");
        }
        if (n == "sort" && !op->regions.empty()) {
            // comparator(lhs0, rhs0, lhs1, rhs1, ..): one strict compare of the first operand's pair gives the order
            const Region& r = *op->regions[0];
            std::string order = "unknown";
            if (r.ops.size() == 2 && r.ops[0].name == "compare" && r.ops[1].name == "return" && r.args.size() >= 2 &&
                r.ops[1].operands.size() == 1 && r.ops[1].operands[0] == r.ops[0].results[0]) {
                const Op& c = r.ops[0];
                std::string dir = c.str_attr("comparison_direction");
                const bool straight = c.operands[0] == r.args[0] && c.operands[1] == r.args[1];
                const bool swapped = c.operands[0] == r.args[1] && c.operands[1] == r.args[0];
                if ((dir == "LT" || dir == "GT") && (straight || swapped))
                    order = ((dir == "LT") == straight) ? "ascending" : "descending";
                // the comparison type decides how zeros and the sign of integers are read: FLOAT holds -0 = +0, TOTALORDER
                // orders them; SIGNED / UNSIGNED must agree with the key's element type
                const std::string ctype = c.str_attr("compare_type");
                const DType kd = fn_->values[r.args[0]].type.dtype;
                if (ctype == "SIGNED" && (is_unsigned(kd) || is_float(kd))) order = "unknown";
                if (ctype == "UNSIGNED" && !(is_unsigned(kd) || kd == DType::I1)) order = "unknown";
                if (ctype == "TOTALORDER" && !is_float(kd)) order = "unknown";
                op->attrs["sort_compare_type"] = Attr::make_string(ctype.empty() && is_float(kd) ? "FLOAT" : ctype);
            }
            op->attrs["sort_order"] = Attr::make_string(order);
        }
        if (n == "convolution" || n == "dynamic_conv") normalise_convolution(op);
        if (n == "dynamic_slice") { rename("sizes", "slice_sizes"); }
        if (n == "pad") { rename("low", "edge_padding_low"); rename("high", "edge_padding_high"); rename("interior", "interior_padding"); }
        if (n == "custom_call") {
            if (const Attr* a = op->attr("call_target_name"))
                if (a->kind == Attr::Keyword) op->attrs["call_target_name"] = Attr::make_string(a->s);
            // the fused convolution call carries the attributes of the convolution it stands for
            if (op->str_attr("call_target_name") == "fused_conv_bias_act") normalise_convolution(op);
        }
        if (n == "select" && op->result_types.size() == 1 && !op->operands.empty()) {
            // "tensor<i1>, tensor<f32>" was parsed as a bare list: result = last, already handled
        }
    }

    // Flattens [[a, b], [c, d]] (Array of IntArray), dense<..> : tensor<Nx2xi64> or a flat list to a flat integer list.
    static std::vector<int64_t> nested_ints(const Attr& a) {
        if (a.kind != Attr::Array) return a.as_ints();
        std::vector<int64_t> out;
        for (const Attr& e : a.elems) {
            std::vector<int64_t> part = e.kind == Attr::Bool ? std::vector<int64_t>{e.b ? 1 : 0} : nested_ints(e);
            out.insert(out.end(), part.begin(), part.end());
        }
        return out;
    }

    // Canonical convolution attributes: the nine dimension numbers (default NHWC x HWIO -> NHWC, the layout of the
    // short form "stablehlo.convolution %x, %w window_strides = [..], padding = [[..]]"), window_strides, padding
    // (flat, rank x 2), lhs_dilation, rhs_dilation, window_reversal, feature_group_count, batch_group_count.
    void normalise_convolution(Op* op) {
        if (op->operands.size() < 2 || op->result_types.empty()) return;  // two operands, or a fused call's x, w, bias
        const int rank = fn_->values[op->operands[0]].type.rank();
        const int ns = rank - 2;
        if (ns < 0) fail_parse("convolution of a tensor of rank " + std::to_string(rank));
        if (const Attr* d = op->attr("dimension_numbers")) {
            if (d->kind == Attr::Dict) {
                const Attr dict = *d;
                for (const auto& kv : dict.dict) op->attrs[kv.first] = kv.second.kind == Attr::Int ? kv.second : Attr::make_ints(nested_ints(kv.second));
            }
            op->attrs.erase("dimension_numbers");
        }
        if (const Attr* w = op->attr("window")) {
            if (w->kind == Attr::Dict) {
                const Attr dict = *w;
                static const std::map<std::string, std::string> keys = {{"stride", "window_strides"}, {"pad", "padding"}, {"lhs_dilate", "lhs_dilation"},
                                                                        {"rhs_dilate", "rhs_dilation"}, {"reverse", "window_reversal"}};
                for (const auto& kv : dict.dict) {
                    auto it = keys.find(kv.first);
                    if (it == keys.end()) fail_parse("convolution: unknown window attribute '" + kv.first + "'");
                    op->attrs[it->second] = Attr::make_ints(nested_ints(kv.second));
                }
            }
            op->attrs.erase("window");
        }
        for (const char* k : {"window_strides", "padding", "lhs_dilation", "rhs_dilation", "window_reversal"})
            if (const Attr* a = op->attr(k)) op->attrs[k] = Attr::make_ints(nested_ints(*a));
        auto dflt_int = [&](const char* k, int64_t v) { if (!op->attr(k)) op->attrs[k] = Attr::make_int(v); };
        auto dflt_list = [&](const char* k, int64_t first) {
            if (op->attr(k)) return;
            std::vector<int64_t> v;
            for (int i = 0; i < ns; ++i) v.push_back(first + i);
            op->attrs[k] = Attr::make_ints(v);
        };
        dflt_int("input_batch_dimension", 0);
        dflt_int("input_feature_dimension", rank - 1);
        dflt_list("input_spatial_dimensions", 1);
        dflt_int("kernel_input_feature_dimension", rank - 2);
        dflt_int("kernel_output_feature_dimension", rank - 1);
        dflt_list("kernel_spatial_dimensions", 0);
        dflt_int("output_batch_dimension", 0);
        dflt_int("output_feature_dimension", rank - 1);
        dflt_list("output_spatial_dimensions", 1);
        dflt_int("feature_group_count", 1);
        dflt_int("batch_group_count", 1);
        op->attrs.erase("precision_config");
    }

    static std::string classify_reducer(const Region& r) {
        // a reducer body is a single arithmetic op (add/maximum/minimum/multiply/and/or) followed by return, or
        // the compare/select idiom of argmax/argmin (direction GT/GE -> max, LT/LE -> min)
        std::string arith;
        std::string cmp;
        int selects = 0;
        for (const Op& o : r.ops) {
            if (o.name == "add" || o.name == "maximum" || o.name == "minimum" || o.name == "multiply" || o.name == "and" ||
                o.name == "or" || o.name == "xor")
                if (arith.empty()) arith = o.name;
            if (o.name == "compare" && cmp.empty()) cmp = o.str_attr("comparison_direction");
            if (o.name == "select") ++selects;
        }
        if (selects > 0 && !cmp.empty()) return (cmp == "GT" || cmp == "GE") ? "argmax" : (cmp == "LT" || cmp == "LE") ? "argmin" : "unknown";
        if (!arith.empty() && r.ops.size() <= 2) return arith;
        if (!arith.empty()) return arith;
        return "unknown";
    }
};

}  // namespace

Module parse_module(const std::string& text) {
    Parser p(text);
    Module m = p.parse();
    for (Function& f : m.functions) legalize_complex(f);
    return m;
}

const Function& Module::main() const {
    for (const Function& f : functions)
        if (f.name == "main") return f;
    return functions.front();
}
Function& Module::main() { return const_cast<Function&>(static_cast<const Module*>(this)->main()); }

}  // namespace mhlo
