"""numpy interpreter for StableHLO text — TEST INFRASTRUCTURE ONLY (the module-level parity oracle).

It evaluates a module the way the reference lowers it, op by op (unfused semantics; the reference requires every
optimisation level to agree with that, Tests/MetalHLOTests/Conformance/OptimizationCorrectnessTests.swift:19-24):
floating-point values are carried in float64 whatever their declared element type, integers in their own numpy
dtype so that wrap-around and truncation are exact. Semantics follow
Sources/MetalHLOCore/Compiler/MPSGraphCompiler.swift:814-1144 (dot_general, broadcast_in_dim, reduce/argmax),
Sources/MetalHLOCore/Compiler/CodeGenerator.swift:1012-1075 (convert = C cast), :1133-1292 (gather with clamped start
indices), :1977-2005 (iota) and the fused custom-call handlers in Compiler/CustomCallHandlers.swift.

The parser here is independent of the product's C++ parser on purpose: both read the same dialect
(Sources/MetalHLOCore/Parser/Parser.swift) and the tests compare their results.

Pinned against the reference's vendored StableHLO interpreter suite
(Tests/MetalHLOTests/Conformance/StableHLO/interpret/*.mlir, `check.expect_*` goldens) by tests/test_interp_suite.py.
"""
from __future__ import annotations

import json
import math
import re

import numpy as np

try:
    import ml_dtypes

    _BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    _BF16 = None

INT_DTYPES = {"i1": np.bool_, "i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64, "ui8": np.uint8,
              "ui16": np.uint16, "ui32": np.uint32, "ui64": np.uint64, "si8": np.int8, "si16": np.int16,
              "si32": np.int32, "si64": np.int64}
FLOAT_DTYPES = ("f16", "f32", "f64", "bf16")
COMPLEX_DTYPES = ("complex<f32>", "complex<f64>")  # carried as complex128


class Unsupported(Exception):
    pass


class TType:
    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), dtype

    @property
    def is_float(self):
        return self.dtype in FLOAT_DTYPES

    @property
    def is_complex(self):
        return self.dtype in COMPLEX_DTYPES

    def np_dtype(self):
        if self.is_complex:
            return np.complex128
        return np.float64 if self.is_float else INT_DTYPES[self.dtype]

    def __repr__(self):
        return "tensor<" + "x".join([str(d) for d in self.shape] + [self.dtype]) + ">"


def round_to(arr, dtype):
    """Rounds float64 values to the precision of a storage dtype (used when a convert asks for it)."""
    if dtype in COMPLEX_DTYPES:
        return arr.astype(np.complex64).astype(np.complex128) if dtype == "complex<f32>" else arr
    if dtype == "f32":
        return arr.astype(np.float32).astype(np.float64)
    if dtype == "f16":
        with np.errstate(over="ignore"):
            return arr.astype(np.float16).astype(np.float64)
    if dtype == "bf16" and _BF16 is not None:
        return arr.astype(np.float32).astype(_BF16).astype(np.float64)
    return arr


def _storage_dtype(dtype):
    """numpy dtype with the bit layout of a StableHLO element type (floats are carried as float64 elsewhere)."""
    if dtype in FLOAT_DTYPES:
        if dtype == "bf16":
            if _BF16 is None:
                raise Unsupported("bf16 bit patterns need ml_dtypes")
            return _BF16
        return {"f16": np.float16, "f32": np.float32, "f64": np.float64}[dtype]
    return INT_DTYPES[dtype]


class Scanner:
    def __init__(self, text):
        self.s, self.p = text, 0

    def ws(self):
        s = self.s
        while self.p < len(s):
            if s[self.p].isspace():
                self.p += 1
            elif s.startswith("//", self.p):
                e = s.find("\n", self.p)
                self.p = len(s) if e < 0 else e
            else:
                break

    def peek(self, n=1):
        self.ws()
        return self.s[self.p:self.p + n]

    def accept(self, tok):
        self.ws()
        if self.s.startswith(tok, self.p):
            self.p += len(tok)
            return True
        return False

    def expect(self, tok):
        if not self.accept(tok):
            raise SyntaxError(f"expected {tok!r} at {self.s[self.p:self.p + 40]!r}")

    _ident = re.compile(r"[A-Za-z_][A-Za-z0-9_.$]*")
    _value = re.compile(r"%[A-Za-z0-9_.$\-]+(#\d+)?")
    _number = re.compile(r"[-+]?(0x[0-9a-fA-F]+|inf|nan|NaN|(\d+\.?\d*([eE][-+]?\d+)?|\.\d+([eE][-+]?\d+)?))")

    def ident(self):
        self.ws()
        m = self._ident.match(self.s, self.p)
        if not m:
            raise SyntaxError(f"expected identifier at {self.s[self.p:self.p + 40]!r}")
        self.p = m.end()
        return m.group()

    def value(self):
        self.ws()
        m = self._value.match(self.s, self.p)
        if not m:
            raise SyntaxError(f"expected SSA value at {self.s[self.p:self.p + 40]!r}")
        self.p = m.end()
        return m.group()

    def number_token(self):
        self.ws()
        for kw in ("true", "false"):
            if self.s.startswith(kw, self.p):
                self.p += len(kw)
                return kw
        m = self._number.match(self.s, self.p)
        if not m:
            raise SyntaxError(f"expected number at {self.s[self.p:self.p + 40]!r}")
        self.p = m.end()
        return m.group()

    def string(self):
        self.ws()
        assert self.s[self.p] == '"'
        out, p = [], self.p + 1
        while self.s[p] != '"':
            if self.s[p] == "\\":
                nxt = self.s[p + 1]
                if nxt in "\"\\":
                    out.append(nxt); p += 2
                elif nxt == "n":
                    out.append("\n"); p += 2
                elif nxt == "t":
                    out.append("\t"); p += 2
                else:
                    out.append(chr(int(self.s[p + 1:p + 3], 16))); p += 3
            else:
                out.append(self.s[p]); p += 1
        self.p = p + 1
        return "".join(out)

    def balanced(self, open_c, close_c):
        self.ws()
        assert self.s[self.p] == open_c, self.s[self.p:self.p + 30]
        depth, p = 0, self.p
        while True:
            c = self.s[p]
            if c == '"':
                q = p + 1
                while self.s[q] != '"':
                    q += 2 if self.s[q] == "\\" else 1
                p = q
            elif c == open_c:
                depth += 1
            elif c == close_c:
                depth -= 1
                if depth == 0:
                    body = self.s[self.p + 1:p]
                    self.p = p + 1
                    return body
            p += 1

    def type(self):
        self.ws()
        if self.peek() == "!":
            self.ident_bang()
            return TType((), "i1")
        w = self.ident()
        if w == "tuple":
            body = self.balanced("<", ">")
            return Scanner(body).type() if body.strip() else TType((), "i1")
        if w != "tensor":
            if w in INT_DTYPES or w in FLOAT_DTYPES:
                return TType((), w)
            raise Unsupported(f"type {w}")
        body = self.balanced("<", ">").split(",")[0].strip()
        m = re.match(r"((?:(?:\d+|\?|\*)x)*)(.*)$", body)
        parts = m.group(1).split("x")[:-1]
        if any(p in ("?", "*") for p in parts):
            raise Unsupported("dynamic shape")
        dt = m.group(2).strip()
        if dt not in INT_DTYPES and dt not in FLOAT_DTYPES and dt not in COMPLEX_DTYPES:
            raise Unsupported(f"element type {dt}")
        return TType([int(p) for p in parts], dt)

    def ident_bang(self):
        self.p += 1
        self.ident()
        if self.peek() == "<":
            self.balanced("<", ">")


def parse_number(tok, ttype):
    if tok == "true":
        return True
    if tok == "false":
        return False
    neg = tok.startswith("-")
    body = tok.lstrip("+-")
    if body.startswith("0x"):
        bits = int(body, 16)
        if ttype.is_float:
            width = {"f16": 2, "bf16": 2, "f32": 4, "f64": 8}[ttype.dtype]
            raw = bits.to_bytes(width, "little")
            if ttype.dtype == "bf16":
                return float(np.frombuffer(raw + b"", dtype=np.uint16).astype(np.uint32).__lshift__(16).view(np.float32)[0])
            return float(np.frombuffer(raw, dtype={"f16": np.float16, "f32": np.float32, "f64": np.float64}[ttype.dtype])[0])
        return -bits if neg else bits
    if body in ("inf",):
        return -math.inf if neg else math.inf
    if body.lower() == "nan":
        return math.nan
    if ttype.is_float:
        return float(tok)
    return int(float(tok)) if ("." in tok or "e" in tok.lower()) else int(tok)


def dense_value(body, ttype):
    """Array of a dense<...> body for a tensor type (floats as float64, ints in their dtype)."""
    body = body.strip()
    npdt = ttype.np_dtype()
    n = int(np.prod(ttype.shape, dtype=np.int64)) if ttype.shape else 1
    if body == "":
        return np.zeros(ttype.shape, dtype=npdt)
    if body.startswith('"'):
        raw = bytes.fromhex(Scanner(body).string()[2:])
        store = {"f16": np.float16, "f32": np.float32, "f64": np.float64}.get(ttype.dtype, INT_DTYPES.get(ttype.dtype))
        if ttype.dtype == "bf16":
            arr = (np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif ttype.dtype == "i1":
            arr = np.frombuffer(raw, dtype=np.uint8) != 0
        else:
            arr = np.frombuffer(raw, dtype=store)
        if arr.size == 1 and n != 1:
            arr = np.full(ttype.shape, arr[0])
        return arr.reshape(ttype.shape).astype(npdt)
    if ttype.is_complex:
        part = TType((), ttype.dtype[len("complex<"):-1])
        nums = [parse_number(x, part) for x in
                re.findall(r"[-+]?(?:0x[0-9a-fA-F]+|inf|nan|NaN|\d+\.?\d*(?:[eE][-+]?\d+)?|\.\d+(?:[eE][-+]?\d+)?)", body)]
        vals = np.array(nums[0::2]) + 1j * np.array(nums[1::2])
        if vals.size == 1 and (n != 1 or "[" not in body):
            return np.full(ttype.shape, vals[0], dtype=np.complex128)
        return vals.astype(np.complex128).reshape(ttype.shape)
    if "(" in body:
        raise Unsupported("complex constant")
    toks = re.findall(r"true|false|[-+]?(?:0x[0-9a-fA-F]+|inf|nan|NaN|\d+\.?\d*(?:[eE][-+]?\d+)?|\.\d+(?:[eE][-+]?\d+)?)", body)
    vals = [parse_number(t, ttype) for t in toks]
    if not ttype.is_float and ttype.dtype != "i1":
        info = np.iinfo(npdt)
        vals = [((v - info.min) % (info.max - info.min + 1)) + info.min if not info.min <= v <= info.max else v for v in vals]
    if len(vals) == 1 and (n != 1 or "[" not in body):
        return np.full(ttype.shape, vals[0], dtype=npdt)
    return np.array(vals, dtype=npdt).reshape(ttype.shape)


class Op:
    __slots__ = ("name", "operands", "results", "types", "attrs", "regions", "in_types", "bare_type_list")

    def __init__(self):
        self.name, self.operands, self.results, self.types, self.attrs, self.regions, self.in_types = "", [], [], [], {}, [], []
        self.bare_type_list = False  # the signature was "t0, t1" without parentheses or arrow


class Region:
    def __init__(self):
        self.args, self.ops = [], []


class Func:
    def __init__(self):
        self.name, self.args, self.arg_types, self.ops, self.result_types = "", [], [], [], []


class ModuleParser(Scanner):
    def parse(self):
        funcs = []
        self.ws()
        if self.accept("module"):
            self.ws()
            if self.peek() == "@":
                self.p += 1
                self.ident()
            elif self.peek() == '"':
                self.string()
            if self.accept("attributes"):
                self.balanced("{", "}")
            self.expect("{")
        while True:
            self.ws()
            if self.p >= len(self.s) or self.peek() == "}":
                break
            if self.s.startswith("func.func", self.p):
                funcs.append(self.func())
            else:
                e = self.s.find("\n", self.p)
                self.p = len(self.s) if e < 0 else e
        return funcs

    def func(self):
        self.expect("func.func")
        for vis in ("private", "public"):
            self.accept(vis)
        self.expect("@")
        f = Func()
        f.name = self.ident()
        self.expect("(")
        while self.peek() != ")":
            f.args.append(self.value())
            self.expect(":")
            f.arg_types.append(self.type())
            if self.peek() == "{":
                self.balanced("{", "}")
            if self.peek(3) == "loc":
                self.ident(); self.balanced("(", ")")
            if not self.accept(","):
                break
        self.expect(")")
        if self.accept("->"):
            if self.peek() == "(":
                self.p += 1
                while self.peek() != ")":
                    f.result_types.append(self.type())
                    if self.peek() == "{":
                        self.balanced("{", "}")
                    if not self.accept(","):
                        break
                self.expect(")")
            else:
                f.result_types.append(self.type())
                if self.peek() == "{":
                    save = self.p
                    body = self.balanced("{", "}")
                    if re.match(r"\s*(%|return|func\.return|stablehlo\.|check\.|chlo\.|\^)", body) or body.strip() == "":
                        self.p = save
        if self.accept("attributes"):
            self.balanced("{", "}")
        self.expect("{")
        f.ops = self.block()[1]
        self.expect("}")
        return f

    def block(self):
        args, ops = [], []
        while True:
            self.ws()
            if self.peek() == "}":
                return args, ops
            if self.peek() == "^":
                self.p += 1
                self.ident()
                if self.accept("("):
                    while self.peek() != ")":
                        name = self.value()
                        self.expect(":")
                        t = self.type()
                        if self.peek(3) == "loc":
                            self.ident(); self.balanced("(", ")")
                        args.append((name, t))
                        if not self.accept(","):
                            break
                    self.expect(")")
                self.expect(":")
                continue
            ops.append(self.operation())

    def region(self):
        self.expect("{")
        r = Region()
        r.args, r.ops = self.block()
        self.expect("}")
        return r

    def operation(self):
        op = Op()
        names, declared = [], None
        if self.peek() == "%":
            while True:
                n = self.value()
                m = re.match(r":(\d+)", self.s[self.p:])
                if m:
                    declared = int(m.group(1))
                    self.p += m.end()
                names.append(n)
                if not self.accept(","):
                    break
            self.expect("=")
        self.ws()
        if self.peek() == '"':
            op.name = self.string()
            self.generic(op)
        else:
            op.name = self.ident()
            self.pretty(op)
        if self.peek(3) == "loc":
            self.ident(); self.balanced("(", ")")
        for k in ("stablehlo.", "chlo.", "func.", "mhlo."):
            if op.name.startswith(k):
                op.name = op.name[len(k):]
        if declared:
            op.results = [f"{names[0]}#{i}" for i in range(declared)]
        else:
            op.results = names
        if len(op.results) > 1 and getattr(op, "bare_type_list", False) and len(op.in_types) == len(op.results):
            op.types = list(op.in_types)  # "%a, %b = op %x, %y : t0, t1": one type per result
        return op

    def operands(self, op, close):
        while self.peek() != close:
            op.operands.append(self.value())
            if not self.accept(","):
                break
        self.expect(close)

    def signature(self, op):
        ins, outs = [], []
        if self.peek() == "(":
            self.p += 1
            while self.peek() != ")":
                ins.append(self.type())
                if not self.accept(","):
                    break
            self.expect(")")
            self.expect("->")
            if self.peek() == "(":
                self.p += 1
                while self.peek() != ")":
                    outs.append(self.type())
                    if not self.accept(","):
                        break
                self.expect(")")
            else:
                outs.append(self.type())
        else:
            ts = [self.type()]
            while self.accept(","):
                ts.append(self.type())
            if self.accept("->"):
                ins = ts
                if self.peek() == "(":  # "t -> (t0, t1)"
                    self.p += 1
                    outs = []
                    while self.peek() != ")":
                        outs.append(self.type())
                        if not self.accept(","):
                            break
                    self.expect(")")
                else:
                    outs = [self.type()]
            else:
                ins, outs = ts, [ts[-1]]
                op.bare_type_list = True
        op.in_types, op.types = ins, outs

    def attr(self):
        self.ws()
        c = self.peek()
        if c == '"':
            v = self.string()
            self.type_suffix()
            return v
        if c == "[":
            self.p += 1
            out = []
            while self.peek() != "]":
                out.append(self.attr())
                if not self.accept(","):
                    break
            self.expect("]")
            return out
        if c == "{":
            return self.attr_dict("{", "}")
        if c == "#":
            self.p += 1
            tag = self.ident()
            if self.peek() != "<":
                return tag
            if tag == "stablehlo.conv":
                self.expect("<")
                spec = self.conv_dimension_spec()
                self.expect(">")
                return spec
            save = self.p
            body = self.balanced("<", ">")
            if "=" not in body:
                return body.split()[-1] if body.split() else tag
            self.p = save
            return self.attr_dict("<", ">")
        if self.s.startswith("dense", self.p):
            self.p += 5
            body = self.balanced("<", ">")
            self.expect(":")
            t = self.type()
            return ("dense", body, t)
        if self.s.startswith("array", self.p):
            self.p += 5
            body = self.balanced("<", ">")
            vals = body.split(":", 1)[1] if ":" in body else ""
            return [{"true": 1, "false": 0}.get(x, x) if x in ("true", "false") else int(x) for x in vals.replace(" ", "").split(",") if x]
        if c == "@":
            self.p += 1
            return self.ident()
        m = re.match(r"true|false|unit", self.s[self.p:])
        if m and not (self.s[self.p + m.end()].isalnum() or self.s[self.p + m.end()] == "_"):
            self.p += m.end()
            return m.group() != "false"
        if c.isdigit() or c in "-+":
            tok = self.number_token()
            self.type_suffix()
            if tok.lower().lstrip("+-").startswith("0x"):
                return int(tok, 16)
            return float(tok) if ("." in tok or "e" in tok.lower() or "inf" in tok or "nan" in tok.lower()) else int(tok)
        w = self.ident()
        if w in ("tensor", "tuple"):
            self.balanced("<", ">")
            return w
        if self.peek() == "<":
            self.balanced("<", ">")
        return w

    def type_suffix(self):
        # "1 : i64" / "1.0 : f32" / "0 : index"; a tensor type after ':' belongs to the operation, not the number
        m = re.match(r"\s*:\s*(index|[su]?i\d+|bf16|f\d+)\b", self.s[self.p:])
        if m:
            self.p += m.end()

    def attr_dict(self, o, c):
        self.expect(o)
        d = {}
        while self.peek() != c:
            key = self.string() if self.peek() == '"' else self.ident()
            if self.accept("="):
                d[key] = self.attr()
            else:
                d[key] = True
            if not self.accept(","):
                break
        self.expect(c)
        return d

    def generic(self, op):
        self.expect("(")
        self.operands(op, ")")
        if self.peek(2) == "<{":
            self.p += 1
            op.attrs.update(self.attr_dict("{", "}"))
            self.expect(">")
        if self.peek() == "(":
            save = self.p
            self.p += 1
            if self.peek() == "{":
                while True:
                    op.regions.append(self.region())
                    if not self.accept(","):
                        break
                self.expect(")")
            else:
                self.p = save
        if self.peek() == "{":
            op.attrs.update(self.attr_dict("{", "}"))
        self.expect(":")
        self.signature(op)

    def conv_dimension_spec(self):
        """'[b, 0, 1, f]x[0, 1, i, o]->[b, 0, 1, f]' as the nine dimension attributes of stablehlo.convolution."""
        out = {}

        def side(batch_key, batch_c, feature_key, feature_c, spatial_key):
            body = self.balanced("[", "]")
            spatial = {}
            for pos, tok in enumerate(t.strip() for t in body.split(",")):
                if tok.isdigit():
                    spatial[int(tok)] = pos
                elif tok == batch_c:
                    out[batch_key] = pos
                elif tok == feature_c:
                    out[feature_key] = pos
                else:
                    raise Unsupported(f"convolution layout token {tok!r}")
            out[spatial_key] = [spatial[k] for k in sorted(spatial)]

        self.ws()
        side("input_batch_dimension", "b", "input_feature_dimension", "f", "input_spatial_dimensions")
        self.expect("x")
        side("kernel_input_feature_dimension", "i", "kernel_output_feature_dimension", "o", "kernel_spatial_dimensions")
        self.expect("->")
        side("output_batch_dimension", "b", "output_feature_dimension", "f", "output_spatial_dimensions")
        return out

    def pretty(self, op):
        kw = []
        name = op.name.split(".")[-1]
        if name == "reduce" and self.accept("("):
            ins, inits = [], []
            while True:
                ins.append(self.value())
                self.expect("init")
                self.expect(":")
                inits.append(self.value())
                self.expect(")")
                if self.accept(","):
                    self.expect("(")
                    continue
                break
            op.operands = ins + inits
        if name == "while" and self.accept("("):
            # stablehlo.while(%iterArg = %init, ...) : types cond { ... } do { ... }: both regions see the iteration arguments
            iters = []
            while self.peek() != ")":
                it_name = self.value()
                self.expect("=")
                op.operands.append(self.value())
                iters.append(it_name)
                if not self.accept(","):
                    break
            self.expect(")")
            self.expect(":")
            while True:
                op.types.append(self.type())
                if not self.accept(","):
                    break
            if self.accept("attributes"):
                self.balanced("{", "}")
            for word in ("cond", "do"):
                self.expect(word)
                r = self.region()
                r.args = [(n, t) for n, t in zip(iters, op.types)]
                op.regions.append(r)
            op.in_types = list(op.types)
            op.attrs["_kw"] = kw
            return
        while True:
            self.ws()
            c = self.peek()
            if c in (":", "{", "}", ""):
                break
            if c == ",":
                self.p += 1
            elif c == "%":
                op.operands.append(self.value())
            elif c == "@":
                self.p += 1
                op.attrs["call_target_name"] = self.ident()
                if self.accept("("):
                    self.operands(op, ")")
            elif c == "[":
                body = self.balanced("[", "]")
                if ":" in body:
                    st, li, sd = [], [], []
                    for part in body.split(","):
                        f = [int(x) for x in part.strip().split(":")]
                        st.append(f[0]); li.append(f[1]); sd.append(f[2] if len(f) > 2 else 1)
                    op.attrs.update(start_indices=st, limit_indices=li, strides=sd)
                else:
                    op.attrs["indices"] = [int(x) for x in body.split(",") if x.strip()]
            elif c == "(" and name == "convolution":
                self.p += 1
                self.operands(op, ")")
            elif c == "(" and name == "top_k":  # chlo.top_k(%x, k = 5)
                self.p += 1
                while self.peek() != ")":
                    if self.peek() == "%":
                        op.operands.append(self.value())
                    else:
                        key = self.ident()
                        self.expect("=")
                        op.attrs[key] = self.attr()
                    if not self.accept(","):
                        break
                self.expect(")")
            elif c == "(":
                self.balanced("(", ")")
            elif self.peek(2) == "<{":
                self.p += 1
                op.attrs.update(self.attr_dict("{", "}"))
                self.expect(">")
            elif self.s.startswith("dense", self.p):
                self.p += 5
                op.attrs["_dense"] = self.balanced("<", ">")
            elif c == "#":
                v = self.attr()
                if isinstance(v, dict):
                    op.attrs.update(v)
            elif c == '"':
                kw.append(self.string())
            else:
                w = self.ident()
                if w == "applies":
                    op.attrs["reducer"] = self.ident().split(".")[-1]
                elif w == "across":
                    pass
                elif w in ("reducer", "cond", "do"):
                    while self.peek() == "(":
                        self.balanced("(", ")")
                    if self.peek() == "{":
                        op.regions.append(self.region())
                elif w == "dim_numbers" and self.accept("="):
                    op.attrs["dimension_numbers"] = self.conv_dimension_spec()
                elif self.accept("="):
                    v = self.attr()
                    self.ws()
                    if self.s.startswith("x", self.p) and not (self.s[self.p + 1].isalnum() or self.s[self.p + 1] == "_"):
                        self.p += 1
                        op.attrs[w + ".lhs"], op.attrs[w + ".rhs"] = v, self.attr()
                    else:
                        op.attrs[w] = v
                else:
                    kw.append(w)
        if self.peek() == "{":
            save = self.p
            body = self.balanced("{", "}")
            self.p = save
            if re.match(r"\s*(\^|%|stablehlo\.|return|func\.return)", body):
                op.regions.append(self.region())
            else:
                op.attrs.update(self.attr_dict("{", "}"))
        if name in ("return",) or op.name in ("return", "func.return", "stablehlo.return"):
            if self.accept(":"):
                self.signature(op)
            return
        if self.accept(":"):
            self.signature(op)
        self.ws()
        if name == "reduce" and self.s.startswith("reducer", self.p):
            self.ident()
            r_args = []
            while self.peek() == "(":
                self.p += 1
                while self.peek() != ")":
                    an = self.value()
                    self.expect(":")
                    r_args.append((an, self.type()))
                    if not self.accept(","):
                        break
                self.expect(")")
            r = self.region()
            r.args = r_args[0::2] + r_args[1::2]
            op.regions.append(r)
        op.attrs["_kw"] = kw


def parse(text):
    return ModuleParser(text).parse()


# ---- evaluation ------------------------------------------------------------------------------------------------------

_DIRS = {"EQ": np.equal, "NE": np.not_equal, "LT": np.less, "LE": np.less_equal, "GT": np.greater, "GE": np.greater_equal}


def _ints(v):
    if v is None:
        return []
    if isinstance(v, (int, np.integer)):
        return [int(v)]
    return [int(x) for x in v]


def _wrap(arr, ttype):
    """Brings a numpy result to the carrier dtype of its declared type."""
    if ttype.is_float:
        return np.asarray(arr, dtype=np.float64)
    if ttype.is_complex:
        return np.asarray(arr, dtype=np.complex128)
    return np.asarray(arr).astype(ttype.np_dtype())


def _float_to_int(arr, ttype):
    # C cast: toward zero; out-of-range and NaN follow the device conversion (saturate, NaN -> 0)
    dt = ttype.np_dtype()
    if dt == np.bool_:
        return arr != 0
    info = np.iinfo(dt)
    a = np.nan_to_num(np.trunc(arr), nan=0.0, posinf=float(info.max), neginf=float(info.min))
    a = np.clip(a, float(info.min), float(info.max))
    top = a >= float(info.max)  # float(info.max) is 2^63 / 2^64 for the 64-bit types: past what astype can take
    return np.where(top, info.max, np.where(top, 0.0, a).astype(dt)).astype(dt)


def _total_order_key(values, dtype):
    """uint64 keys whose unsigned order is the total order of the values (-NaN < -inf < .. < -0 < +0 < .. < +NaN)."""
    if dtype in FLOAT_DTYPES:
        if dtype == "f64":
            b = np.ascontiguousarray(values, dtype=np.float64).view(np.uint64)
            return np.where(b >> np.uint64(63), ~b, b | np.uint64(1 << 63))
        b = np.ascontiguousarray(values.astype(np.float32)).view(np.uint32).astype(np.uint64)
        flipped = np.where(b >> np.uint64(31), b ^ np.uint64(0xFFFFFFFF), b | np.uint64(0x80000000))
        return flipped
    v = np.asarray(values)
    if v.dtype == np.bool_:
        return v.astype(np.uint64)
    if np.issubdtype(v.dtype, np.signedinteger):
        return (v.astype(np.int64).view(np.uint64)) ^ np.uint64(1 << 63)
    return v.astype(np.uint64)


def _with_attrs(op, **extra):
    import copy
    o = copy.copy(op)
    o.attrs = dict(op.attrs)
    o.attrs.update(extra)
    return o


_COMPLEX_OPS = ("complex", "real", "imag", "abs", "add", "subtract", "multiply", "divide", "negate", "convert", "select", "fft", "exponential", "compare",
                "reshape", "transpose", "broadcast_in_dim", "slice", "concatenate", "reverse", "constant", "call",
                "optimization_barrier")


class Interpreter:
    def __init__(self, round_floats: bool = False, funcs=None):
        self.round_floats = round_floats
        self.funcs = {f.name: f for f in (funcs or [])}

    def op_call(self, op, a, t):
        """func.call: the callee is interpreted on the argument arrays (no inlining)."""
        callee = self.funcs.get(op.attrs.get("call_target_name") or op.attrs.get("callee"))
        if callee is None:
            raise Unsupported(f"call of unknown function {op.attrs}")
        env = {name: x for name, x in zip(callee.args, a)}
        return self._run_ops(callee.ops, env)

    def op_while(self, op, a, t, env):
        """stablehlo.while: the loop is run, condition first, for as long as the condition region returns true."""
        cond, body = op.regions
        state = list(a)
        for _ in range(1_000_000):
            scope = dict(env)
            scope.update({name: x for (name, _), x in zip(cond.args, state)})
            if not bool(np.asarray(self._run_ops(cond.ops, scope)[0]).reshape(())):
                return state
            scope = dict(env)
            scope.update({name: x for (name, _), x in zip(body.args, state)})
            state = self._run_ops(body.ops, scope)
        raise Unsupported("while loop did not terminate within 1e6 iterations")

    def op_branch(self, op, a, env):
        """stablehlo.if / stablehlo.case: only the selected region is interpreted (if: true branch first; case: an
        index outside [0, N) selects the last branch)."""
        sel = np.asarray(a[0]).reshape(())
        if op.name == "if":
            k = 0 if bool(sel) else 1
        else:
            k = int(sel)
            if k < 0 or k >= len(op.regions):
                k = len(op.regions) - 1
        return self._run_ops(op.regions[k].ops, dict(env))

    def _apply(self, region, env, values):
        """Runs a region on scalar arguments and returns its results."""
        scope = dict(env)
        scope.update({name: np.asarray(v) for (name, _), v in zip(region.args, values)})
        return self._run_ops(region.ops, scope)

    def region_map(self, op, a, env):
        """stablehlo.map: the computation is applied to each tuple of corresponding elements."""
        t = op.types[0]
        out = np.empty(t.shape, dtype=np.float64 if t.is_float else t.np_dtype())
        for idx in np.ndindex(*t.shape):
            out[idx] = self._apply(op.regions[0], env, [x[idx] for x in a])[0].reshape(())
        return out

    def op_top_k(self, op, a, t):
        """chlo.top_k: the k largest entries along the last dimension (total order, NaN largest) and their positions,
        equal entries in index order."""
        k = int(op.attrs["k"])
        x = a[0]
        key = _total_order_key(x, op.in_types[0].dtype)
        order = np.argsort(~key, axis=-1, kind="stable")[..., :k]
        return [np.take_along_axis(x, order, axis=-1), order.astype(op.types[1].np_dtype())]

    def op_get_dimension_size(self, op, a, t):
        return np.asarray(a[0].shape[int(op.attrs.get("dim", op.attrs.get("dimension", 0)))], dtype=t.np_dtype())

    def region_reduce_window(self, op, a, env):
        """stablehlo.reduce_window: the operand is dilated and padded with the init value, and every window is folded
        through the body region in row-major order, starting from the init value."""
        if len(a) != 2:
            raise Unsupported("variadic reduce_window")
        x, init = a[0], a[1].reshape(())
        t = op.types[0]
        A = op.attrs
        rank = x.ndim
        size = _ints(A.get("window_dimensions"))
        stride = _ints(A.get("window_strides")) or [1] * rank
        bdil = _ints(A.get("base_dilations")) or [1] * rank
        wdil = _ints(A.get("window_dilations")) or [1] * rank
        pad = A.get("padding")
        pad = np.asarray(dense_value(pad[1], pad[2]) if isinstance(pad, tuple) else (pad if pad is not None else np.zeros((rank, 2))), dtype=np.int64).reshape(rank, 2)
        dil_shape = [(n - 1) * b + 1 if n > 0 else 0 for n, b in zip(x.shape, bdil)]
        dil = np.full(dil_shape, init, dtype=x.dtype)
        dil[tuple(slice(None, None, b) for b in bdil)] = x
        padded_shape = [max(0, n + int(lo) + int(hi)) for n, (lo, hi) in zip(dil_shape, pad)]
        padded = np.full(padded_shape, init, dtype=x.dtype)
        src, dst = [], []
        for n, (lo, hi), m in zip(dil_shape, pad, padded_shape):
            s0, s1 = max(0, -int(lo)), n - max(0, -int(hi))
            src.append(slice(s0, max(s0, s1)))
            d0 = max(0, int(lo))
            dst.append(slice(d0, d0 + max(0, s1 - s0)))
        padded[tuple(dst)] = dil[tuple(src)]
        out = np.empty(t.shape, dtype=x.dtype)
        body = op.regions[0]
        for o in np.ndindex(*t.shape):
            acc = init
            for w in np.ndindex(*size):
                pos = tuple(oi * st + wi * wd for oi, st, wi, wd in zip(o, stride, w, wdil))
                acc = self._apply(body, env, [acc, padded[pos]])[0].reshape(())
            out[o] = acc
        return out

    def region_select_and_scatter(self, op, a, env):
        """stablehlo.select_and_scatter: each window of the operand (padded with the init value) keeps the element e
        for which select(kept, e) fails, scanning in row-major order; the source element of the window is combined by
        the scatter region into the result (filled with the init value) at the kept position, unless it is padding."""
        x, source, init = a[0], a[1], a[2].reshape(())
        t = op.types[0]
        A = op.attrs
        rank = x.ndim
        size = _ints(A.get("window_dimensions"))
        stride = _ints(A.get("window_strides")) or [1] * rank
        pad = A.get("padding")
        pad = np.asarray(dense_value(pad[1], pad[2]) if isinstance(pad, tuple) else (pad if pad is not None else np.zeros((rank, 2))), dtype=np.int64).reshape(rank, 2)
        select, scatter = op.regions
        result = np.full(t.shape, init, dtype=x.dtype)
        for s_idx in np.ndindex(*source.shape):
            kept, kept_at = None, None
            for w in np.ndindex(*size):
                pos = tuple(si * st + wi - int(lo) for si, st, wi, (lo, _) in zip(s_idx, stride, w, pad))
                inside = all(0 <= c < n for c, n in zip(pos, x.shape))
                v = x[pos] if inside else init
                if kept is None or not bool(self._apply(select, env, [kept, v])[0].reshape(())):
                    kept, kept_at = v, (pos if inside else None)
            if kept_at is not None:
                result[kept_at] = self._apply(scatter, env, [result[kept_at], source[s_idx]])[0].reshape(())
        return result

    def region_scatter(self, op, a, env):
        """stablehlo.scatter: updates are applied one by one, in row-major order of `updates`, through the update
        computation; an update whose target lies outside the operand is skipped."""
        if len(a) != 3:
            raise Unsupported("variadic scatter")
        A = op.attrs
        d = A.get("scatter_dimension_numbers", A)
        uwd = _ints(d.get("update_window_dims"))
        iwd = _ints(d.get("inserted_window_dims"))
        ib = _ints(d.get("input_batching_dims"))
        sb = _ints(d.get("scatter_indices_batching_dims"))
        sdod = _ints(d.get("scatter_dims_to_operand_dims"))
        ivd = int(d.get("index_vector_dim"))
        result, idx, upd = a[0].copy(), a[1].astype(np.int64), a[2]
        if ivd == idx.ndim:
            idx = idx[..., None]
        idx = np.moveaxis(idx, ivd, -1)
        scatter_dims = [k for k in range(upd.ndim) if k not in uwd]
        window_operand_dims = [k for k in range(result.ndim) if k not in iwd and k not in ib]
        sb_pos = [b - (1 if b > ivd else 0) for b in sb]
        body = op.regions[0]
        for u in np.ndindex(*upd.shape):
            batch = tuple(u[k] for k in scatter_dims)
            target = [0] * result.ndim
            for k, od in enumerate(sdod):
                target[od] = int(idx[batch + (k,)])
            for k, od in enumerate(ib):
                target[od] += batch[sb_pos[k]]
            for k, od in enumerate(window_operand_dims):
                target[od] += u[uwd[k]]
            if all(0 <= c < n for c, n in zip(target, result.shape)):
                result[tuple(target)] = self._apply(body, env, [result[tuple(target)], upd[u]])[0].reshape(())
        return result

    def region_sort(self, op, a, env):
        """stablehlo.sort: slices along `dimension` are put in the order of the comparator region with a stable
        sort (slices longer than 2048 elements use the comparator's recognised LT / GT form on a total-order key)."""
        import functools
        A = op.attrs
        dim = int(A.get("dimension", -1))
        if dim < 0:
            dim += a[0].ndim
        comp = op.regions[0]
        n = a[0].shape[dim]
        moved = [np.moveaxis(x, dim, -1) for x in a]
        outs = [np.empty_like(m) for m in moved]

        def less(i, j, row):
            args = []
            for m in moved:
                args += [m[row + (i,)], m[row + (j,)]]
            return bool(self._apply(comp, env, args)[0].reshape(()))

        direction = None
        if n > 2048:
            cmp_ops = [o for o in comp.ops if o.name.endswith("compare")]
            if len(comp.ops) != 2 or len(cmp_ops) != 1:
                raise Unsupported("long sort with a comparator that is not a single compare")
            c = cmp_ops[0]
            dname = c.attrs.get("comparison_direction") or [k for k in c.attrs.get("_kw", []) if k in _DIRS][0]
            names = [name for name, _ in comp.args]
            straight = list(c.operands) == names[:2]
            if dname not in ("LT", "GT") or (not straight and list(c.operands) != names[1::-1]):
                raise Unsupported("long sort with a comparator other than LT / GT of the first operand")
            direction = "asc" if (dname == "LT") == straight else "desc"
        for row in np.ndindex(*moved[0].shape[:-1]):
            if direction is None:
                order = sorted(range(n), key=functools.cmp_to_key(lambda i, j: -1 if less(i, j, row) else (1 if less(j, i, row) else 0)))
            else:
                key = _total_order_key(moved[0][row], op.in_types[0].dtype)
                order = np.argsort(~key if direction == "desc" else key, kind="stable")
            for m, o in zip(moved, outs):
                o[row] = m[row][np.asarray(order, dtype=np.int64)]
        return [np.moveaxis(o, -1, dim) for o in outs]

    def run(self, func, inputs):
        env = {}
        for name, t, x in zip(func.args, func.arg_types, inputs):
            env[name] = self._input(x, t)
        return self._run_ops(func.ops, env)

    def _input(self, x, t):
        if hasattr(x, "detach"):
            x = x.detach().cpu()
            x = x.double().numpy() if x.is_floating_point() else x.numpy()
        a = np.asarray(x)
        if t.is_complex and not np.iscomplexobj(a):  # (re, im) pairs on a last axis of 2, as the C API carries them
            assert a.shape == t.shape + (2,), (a.shape, t)
            a = a[..., 0].astype(np.float64) + 1j * a[..., 1].astype(np.float64)
        a = a.astype(np.float64) if t.is_float else a.astype(t.np_dtype())
        assert a.shape == t.shape, (a.shape, t)
        return a

    def _run_ops(self, ops, env):
        for op in ops:
            if op.name in ("return", "func.return", "stablehlo.return"):
                return [env[v] for v in op.operands]
            if op.name.startswith("check."):
                continue
            if op.name == "tuple":  # a name for a list of values (nested tuples included)
                env[op.results[0]] = tuple(env[v] for v in op.operands)
                continue
            if op.name == "get_tuple_element":
                idx = op.attrs.get("index", op.attrs.get("indices"))
                env[op.results[0]] = env[op.operands[0]][_ints(idx)[0]]
                continue
            outs = self.eval(op, [env[v] if v in env else env[v + "#0"] for v in op.operands], env)
            if not isinstance(outs, (list, tuple)):
                outs = [outs]
            for name, t, v in zip(op.results, op.types, outs):
                v = _wrap(v, t)
                if self.round_floats and (t.is_float or t.is_complex):
                    v = round_to(v, t.dtype)
                env[name] = v.reshape(t.shape)
        return []

    def eval(self, op, a, env):
        n, t = op.name, (op.types[0] if op.types else None)
        A = op.attrs
        it = op.in_types
        if n not in _COMPLEX_OPS and (any(np.iscomplexobj(x) for x in a) or (t is not None and t.is_complex)):
            # the backend's surface for complex values (csrc/host/complex.cpp); everything else is out of scope for both
            raise Unsupported(f"{n} on complex values")
        if n == "convert" and a and np.iscomplexobj(a[0]) and not t.is_complex:
            a = [np.real(a[0])]  # the imaginary part is dropped
        if n == "compare" and a and np.iscomplexobj(a[0]):
            d = op.attrs.get("comparison_direction") or next((k for k in op.attrs.get("_kw", []) if k in _DIRS), None)
            if d not in ("EQ", "NE"):
                raise Unsupported("compare of complex values in a direction other than EQ and NE")
        if n == "while":
            return self.op_while(op, a, t, env)
        if n in ("if", "case"):
            return self.op_branch(op, a, env)
        if n == "map":
            return self.region_map(op, a, env)
        if n in ("reduce_window", "scatter", "sort", "select_and_scatter"):
            return getattr(self, "region_" + n)(op, a, env)
        f = getattr(self, "op_" + n, None)
        if f is not None:
            return f(op, a, t)
        un = {"negate": np.negative, "abs": np.abs, "exponential": np.exp, "exponential_minus_one": np.expm1, "log": np.log,
              "log_plus_one": np.log1p, "sqrt": np.sqrt, "rsqrt": lambda x: 1.0 / np.sqrt(x), "cbrt": np.cbrt, "tanh": np.tanh,
              "logistic": lambda x: 1.0 / (1.0 + np.exp(-x)), "sine": np.sin, "cosine": np.cos, "tan": np.tan, "floor": np.floor,
              "ceil": np.ceil, "round_nearest_even": np.rint, "sign": np.sign, "is_finite": np.isfinite,
              "round_nearest_afz": lambda x: np.sign(x) * np.floor(np.abs(x) + 0.5),
              "erf": np.vectorize(math.erf, otypes=[np.float64])}
        if n in un:
            with np.errstate(all="ignore"):
                return un[n](a[0])
        if n == "not":
            return np.logical_not(a[0]) if a[0].dtype == np.bool_ else np.invert(a[0])
        if n == "popcnt":
            bits = a[0].dtype.itemsize * 8
            u = a[0].astype(f"uint{bits}")
            return sum(((u >> i) & 1) for i in range(bits)).astype(a[0].dtype)
        if n == "count_leading_zeros":
            bits = a[0].dtype.itemsize * 8
            u = a[0].astype(f"uint{bits}").astype(np.uint64)
            out = np.full(u.shape, bits, dtype=np.int64)
            for i in range(bits):
                out = np.where((u >> np.uint64(i)) != 0, bits - 1 - i, out)
            return out
        with np.errstate(all="ignore"):
            if n == "add":
                return np.logical_or(a[0], a[1]) if a[0].dtype == np.bool_ else a[0] + a[1]
            if n == "subtract":
                return a[0] - a[1]
            if n == "multiply":
                return np.logical_and(a[0], a[1]) if a[0].dtype == np.bool_ else a[0] * a[1]
            if n == "divide":
                if t.is_float or t.is_complex:
                    return a[0] / a[1]
                q = np.where(a[1] == 0, 1, a[1])
                if a[0].dtype.itemsize < 8:
                    r = np.trunc(a[0].astype(np.float64) / q.astype(np.float64))
                else:  # exact integers (|INT64_MIN| does not fit int64): truncation toward zero, wrapped to the type
                    num, den = np.broadcast_arrays(a[0].astype(object), q.astype(object))
                    r = np.empty(num.shape, dtype=object)
                    for idx in np.ndindex(num.shape):
                        n_, d_ = int(num[idx]), int(den[idx])
                        r[idx] = abs(n_) // abs(d_) * (1 if (n_ < 0) == (d_ < 0) else -1)
                    info = np.iinfo(a[0].dtype)
                    span = int(info.max) - int(info.min) + 1
                    r = np.array([((int(v) - int(info.min)) % span) + int(info.min) for v in r.reshape(-1)], dtype=a[0].dtype).reshape(num.shape)
                return np.where(a[1] == 0, -1, r)
            if n == "remainder":
                if t.is_float:
                    return np.fmod(a[0], a[1])
                q = np.where(a[1] == 0, 1, a[1])
                return np.where(a[1] == 0, a[0], np.fmod(a[0], q))
            if n == "maximum":
                return np.maximum(a[0], a[1])
            if n == "minimum":
                return np.minimum(a[0], a[1])
            if n == "power":
                if t.is_float:
                    return np.power(a[0], a[1])
                base, e = a[0].astype(object), a[1].astype(object)
                info = np.iinfo(t.np_dtype())
                out = np.empty(base.shape, dtype=object)
                for idx in np.ndindex(base.shape):
                    b_, e_ = int(base[idx]), int(e[idx])
                    if e_ < 0:
                        v = 1 if b_ == 1 else ((-1 if e_ % 2 else 1) if b_ == -1 else 0)
                    else:
                        v = pow(b_, e_, 1 << 64)
                    v &= (1 << (8 * np.dtype(t.np_dtype()).itemsize)) - 1
                    if info.min < 0 and v > info.max:
                        v -= 1 << (8 * np.dtype(t.np_dtype()).itemsize)
                    out[idx] = v
                return out.astype(t.np_dtype())
            if n == "atan2":
                return np.arctan2(a[0], a[1])
            if n == "and":
                return np.logical_and(a[0], a[1]) if a[0].dtype == np.bool_ else a[0] & a[1]
            if n == "or":
                return np.logical_or(a[0], a[1]) if a[0].dtype == np.bool_ else a[0] | a[1]
            if n == "xor":
                return np.logical_xor(a[0], a[1]) if a[0].dtype == np.bool_ else a[0] ^ a[1]
            if n in ("shift_left", "shift_right_arithmetic", "shift_right_logical"):
                bits = a[0].dtype.itemsize * 8
                sh = a[1].astype(np.int64)
                big = (sh >= bits) | (sh < 0)
                s = np.where(big, 0, sh).astype(a[0].dtype)
                if n == "shift_left":
                    return np.where(big, 0, a[0] << s)
                if n == "shift_right_arithmetic":
                    return np.where(big, np.where(a[0] < 0, -1, 0), a[0] >> s).astype(a[0].dtype)
                u = a[0].astype(f"uint{bits}")
                return np.where(big, 0, u >> s.astype(f"uint{bits}")).astype(a[0].dtype)
        raise Unsupported(f"op {n}")

    def op_reduce_precision(self, op, a, t):
        # stablehlo.reduce_precision: round to nearest even at `m` mantissa bits, then clamp to `e` exponent bits
        fmt = op.attrs.get("format")
        if fmt is not None:
            m_ = re.match(r"e(\d+)m(\d+)", str(fmt if not isinstance(fmt, tuple) else fmt[-1]))
            e, m = int(m_.group(1)), int(m_.group(2))
        else:
            e, m = int(op.attrs["exponent_bits"]), int(op.attrs["mantissa_bits"])
        x = np.ascontiguousarray(a[0], dtype=np.float64)
        bits = x.view(np.uint64).copy()
        sign = bits & np.uint64(1 << 63)
        exp_mask, mant_mask = np.uint64(0x7FF << 52), np.uint64((1 << 52) - 1)
        nan = ((bits & exp_mask) == exp_mask) & ((bits & mant_mask) != 0)
        if m < 52:
            last = np.uint64(1 << (52 - m))
            bias = (last >> np.uint64(1)) - np.uint64(1) + ((bits & last) >> np.uint64(52 - m))
            bits = (bits + bias) & ~(last - np.uint64(1))
        if e < 11:
            full, red = 1023, (1 << (e - 1)) - 1
            ex = bits & exp_mask
            over, under = ex > np.uint64((full + red) << 52), ex <= np.uint64((full - red) << 52)
            bits = np.where(over, sign | exp_mask, np.where(under, sign, bits))
        keep_nan = x.view(np.uint64) if m > 0 else (sign | exp_mask)  # a format without mantissa bits has no NaN
        out = np.where(nan, keep_nan, bits).astype(np.uint64).view(np.float64)
        return out.reshape(a[0].shape)

    def op_cholesky(self, op, a, t):
        # stablehlo.cholesky: the lower (default: upper) factor of every [n, n] matrix, the other triangle zero
        lower = str(op.attrs.get("lower", "false")).lower() in ("true", "1")
        x = np.asarray(a[0], dtype=np.float64)
        with np.errstate(all="ignore"):
            try:
                fac = np.linalg.cholesky(x)
            except np.linalg.LinAlgError:
                fac = np.full_like(x, np.nan)
        return fac if lower else np.swapaxes(fac, -1, -2)

    def op_triangular_solve(self, op, a, t):
        import scipy.linalg

        A = op.attrs
        flag = lambda k: str(A.get(k, "false")).lower() in ("true", "1")  # noqa: E731
        tr = str(A.get("transpose_a", "NO_TRANSPOSE"))
        trans = 0 if "NO_TRANSPOSE" in tr else 1
        x, b = np.asarray(a[0], dtype=np.float64), np.asarray(a[1], dtype=np.float64)
        out = np.empty_like(b)
        for idx in np.ndindex(*x.shape[:-2]):
            m = np.tril(x[idx]) if flag("lower") else np.triu(x[idx])
            if flag("left_side"):
                out[idx] = scipy.linalg.solve_triangular(m, b[idx], trans=trans, lower=flag("lower"), unit_diagonal=flag("unit_diagonal"))
            else:  # x op(a) = b  <=>  op(a)^T x^T = b^T
                out[idx] = scipy.linalg.solve_triangular(m, b[idx].T, trans=1 - trans, lower=flag("lower"), unit_diagonal=flag("unit_diagonal")).T
        return out

    def op_composite(self, op, a, t):
        dec = op.attrs.get("decomposition", "")
        name = str(dec[-1] if isinstance(dec, tuple) else dec).lstrip("@")
        callee = self.funcs.get(name)
        if callee is None:
            raise Unsupported(f"composite without its decomposition @{name}")
        env = {arg: x for arg, x in zip(callee.args, a)}
        return self._run_ops(callee.ops, env)

    # -- structural ops
    def op_constant(self, op, a, t):
        v = op.attrs.get("value")
        arr = dense_value(v[1], t) if v is not None else dense_value(op.attrs["_dense"], t)
        # a constant holds values of its element type: the literal is rounded to it, as the reference serialises
        # constants at their element type (Sources/MetalHLOCore/Compiler/MetalHLOCompiler.swift:487-613)
        return round_to(arr, t.dtype) if t.is_float else arr

    def op_iota(self, op, a, t):
        d = int(op.attrs.get("dim", op.attrs.get("iota_dimension", 0)))
        shape = [1] * len(t.shape)
        shape[d] = t.shape[d]
        return np.broadcast_to(np.arange(t.shape[d]).reshape(shape), t.shape)

    def op_complex(self, op, a, t):
        return a[0] + 1j * a[1]

    def op_real(self, op, a, t):
        return np.real(a[0])

    def op_imag(self, op, a, t):
        return np.imag(a[0])

    def op_fft(self, op, a, t):
        """stablehlo.fft over the last len(fft_length) axes. Complex tensors may also be given as float tensors of
        interleaved (re, im) pairs, the form of the reference's kernels (Compiler/CodeGenerator.swift:2701-2830)."""
        A = op.attrs
        words = " ".join(str(A.get(k, "")) for k in ("fft_type", "type")) + " " + " ".join(map(str, A.get("_kw", [])))
        kind = next(k for k in ("IRFFT", "RFFT", "IFFT", "FFT") if re.search(r"\b" + k + r"\b", words))
        lens = _ints(A.get("fft_length", A.get("length")))
        axes = tuple(range(-len(lens), 0))
        x = a[0]

        def as_complex(arr, tail):
            if np.iscomplexobj(arr):
                return arr
            flat = arr.reshape(-1, 2)
            return (flat[:, 0] + 1j * flat[:, 1]).reshape((-1,) + tuple(tail))

        half = lens[:-1] + [lens[-1] // 2 + 1]
        if kind == "FFT":
            z = np.fft.fftn(as_complex(x, lens), axes=axes)
        elif kind == "IFFT":
            z = np.fft.ifftn(as_complex(x, lens), axes=axes)
        elif kind == "RFFT":
            z = np.fft.rfftn(np.asarray(x, dtype=np.float64).reshape((-1,) + tuple(lens)), s=lens, axes=axes)
        else:
            z = np.fft.irfftn(as_complex(x, half), s=lens, axes=axes)
        if t.is_complex or kind == "IRFFT":
            return z.reshape(t.shape)
        return np.stack([z.real, z.imag], axis=-1).reshape(t.shape)

    def op_convert(self, op, a, t):
        src = op.in_types[0] if op.in_types else None
        x = a[0]
        if t.is_complex:
            return round_to(np.asarray(x).astype(np.complex128), t.dtype)
        if t.is_float:
            return round_to(x.astype(np.float64), t.dtype)  # a convert is a real rounding point
        if x.dtype == np.float64:
            return _float_to_int(x, t)
        if t.dtype == "i1":
            return x != 0
        return x.astype(t.np_dtype())

    def op_compare(self, op, a, t):
        d = op.attrs.get("comparison_direction")
        if d is None:
            d = [k for k in op.attrs.get("_kw", []) if k in _DIRS][0]
        ctype = op.attrs.get("compare_type") or next((k for k in op.attrs.get("_kw", []) if k in ("TOTALORDER", "FLOAT", "SIGNED", "UNSIGNED")), None)
        if ctype == "TOTALORDER" and op.in_types and op.in_types[0].is_float:
            # -NaN < -inf < .. < -0 < +0 < .. < +inf < +NaN: compare order-preserving integer keys
            dt = op.in_types[0].dtype
            return _DIRS[d](_total_order_key(np.asarray(a[0]), dt), _total_order_key(np.asarray(a[1]), dt))
        return _DIRS[d](a[0], a[1])

    def op_select(self, op, a, t):
        return np.where(a[0], a[1], a[2])

    def op_clamp(self, op, a, t):
        return np.minimum(np.maximum(a[1], a[0]), a[2])

    def op_broadcast_in_dim(self, op, a, t):
        dims = _ints(op.attrs.get("dims", op.attrs.get("broadcast_dimensions")))
        shape = [1] * len(t.shape)
        for i, d in enumerate(dims):
            shape[d] = a[0].shape[i]
        return np.broadcast_to(a[0].reshape(shape), t.shape)

    def op_reshape(self, op, a, t):
        return a[0].reshape(t.shape)

    def op_transpose(self, op, a, t):
        return np.transpose(a[0], _ints(op.attrs.get("dims", op.attrs.get("permutation"))))

    def op_reverse(self, op, a, t):
        return np.flip(a[0], axis=tuple(_ints(op.attrs.get("dims", op.attrs.get("dimensions")))))

    def op_slice(self, op, a, t):
        st, li = _ints(op.attrs["start_indices"]), _ints(op.attrs["limit_indices"])
        sd = _ints(op.attrs.get("strides")) or [1] * len(st)
        return a[0][tuple(slice(s, l, k) for s, l, k in zip(st, li, sd))]

    def op_concatenate(self, op, a, t):
        return np.concatenate(a, axis=int(op.attrs.get("dim", op.attrs.get("dimension", 0))))

    def op_pad(self, op, a, t):
        lo = _ints(op.attrs.get("low", op.attrs.get("edge_padding_low")))
        hi = _ints(op.attrs.get("high", op.attrs.get("edge_padding_high")))
        inter = _ints(op.attrs.get("interior", op.attrs.get("interior_padding"))) or [0] * len(lo)
        out = np.full(t.shape, a[1].reshape(()), dtype=a[0].dtype)
        x = a[0]
        src, dst = [], []
        for d in range(x.ndim):
            step = inter[d] + 1
            first, count = 0, x.shape[d]
            while count > 0 and lo[d] + first * step < 0:
                first += 1; count -= 1
            while count > 0 and lo[d] + (first + count - 1) * step >= t.shape[d]:
                count -= 1
            src.append(slice(first, first + count))
            start = lo[d] + first * step
            dst.append(slice(start, start + (count - 1) * step + 1 if count > 0 else start, step))
        out[tuple(dst)] = x[tuple(src)]
        return out

    def op_dot(self, op, a, t):
        return self._dot(a[0], a[1], [], [], [a[0].ndim - 1], [0], t)

    def op_dot_general(self, op, a, t):
        A = op.attrs
        d = A.get("dot_dimension_numbers", A)
        lb = _ints(d.get("lhs_batching_dimensions", A.get("batching_dims.lhs")))
        rb = _ints(d.get("rhs_batching_dimensions", A.get("batching_dims.rhs")))
        lc = _ints(d.get("lhs_contracting_dimensions", A.get("contracting_dims.lhs")))
        rc = _ints(d.get("rhs_contracting_dimensions", A.get("contracting_dims.rhs")))
        return self._dot(a[0], a[1], lb, rb, lc, rc, t)

    def _dot(self, x, y, lb, rb, lc, rc, t):
        lf = [d for d in range(x.ndim) if d not in lb and d not in lc]
        rf = [d for d in range(y.ndim) if d not in rb and d not in rc]
        xs = np.transpose(x, lb + lf + lc)
        ys = np.transpose(y, rb + rc + rf)
        B = int(np.prod([x.shape[d] for d in lb], dtype=np.int64))
        M = int(np.prod([x.shape[d] for d in lf], dtype=np.int64))
        K = int(np.prod([x.shape[d] for d in lc], dtype=np.int64))
        N = int(np.prod([y.shape[d] for d in rf], dtype=np.int64))
        if t.is_float:
            out = np.matmul(xs.reshape(B, M, K).astype(np.float64), ys.reshape(B, K, N).astype(np.float64))
        elif t.dtype == "i1":
            out = np.matmul(xs.reshape(B, M, K).astype(np.int64), ys.reshape(B, K, N).astype(np.int64)) != 0
        else:
            out = np.matmul(xs.reshape(B, M, K).astype(np.int64), ys.reshape(B, K, N).astype(np.int64))
        return out.reshape(t.shape)

    def op_reduce(self, op, a, t):
        n_in = len(a) // 2
        dims = tuple(_ints(op.attrs.get("dimensions", op.attrs.get("dims"))))
        red = op.attrs.get("reducer")
        if red is None and op.regions:
            red = self._classify(op.regions[0])
        x, init = a[0], a[n_in]
        if red in ("argmax", "argmin"):
            assert n_in == 2 and len(dims) == 1
            axis = dims[0]
            xv = np.where(np.isnan(x), np.inf if red == "argmax" else -np.inf, x) if x.dtype == np.float64 else x
            idx = (np.argmax if red == "argmax" else np.argmin)(xv, axis=axis)
            val = np.take_along_axis(x, np.expand_dims(idx, axis), axis=axis).squeeze(axis)
            return [val, idx]
        fns = {"add": np.add, "maximum": np.maximum, "minimum": np.minimum, "multiply": np.multiply,
               "and": np.logical_and if x.dtype == np.bool_ else np.bitwise_and,
               "or": np.logical_or if x.dtype == np.bool_ else np.bitwise_or,
               "xor": np.logical_xor if x.dtype == np.bool_ else np.bitwise_xor}
        if red not in fns:
            raise Unsupported(f"reducer {red}")
        fn = fns[red]
        if x.dtype == np.bool_ and red in ("add", "multiply"):
            fn = np.logical_or if red == "add" else np.logical_and
        with np.errstate(all="ignore"):
            out = fn.reduce(x, axis=dims) if x.size or True else None
            out = fn(out, init.reshape(()).astype(out.dtype) if hasattr(out, "dtype") else init)
        return out

    @staticmethod
    def _classify(region):
        names = [o.name.split(".")[-1] for o in region.ops]
        if "select" in names and "compare" in names:
            cmp = [o for o in region.ops if o.name.endswith("compare")][0]
            d = cmp.attrs.get("comparison_direction") or [k for k in cmp.attrs.get("_kw", []) if k in _DIRS][0]
            return "argmax" if d in ("GT", "GE") else "argmin"
        for n in names:
            if n in ("add", "maximum", "minimum", "multiply", "and", "or", "xor"):
                return n
        return "unknown"

    def op_gather(self, op, a, t):
        A = op.attrs
        d = A.get("dimension_numbers", A)
        offset_dims = _ints(d.get("offset_dims"))
        collapsed = _ints(d.get("collapsed_slice_dims"))
        ob = _ints(d.get("operand_batching_dims"))
        sb = _ints(d.get("start_indices_batching_dims"))
        sim = _ints(d.get("start_index_map"))
        ivd = int(d.get("index_vector_dim"))
        ss = _ints(A.get("slice_sizes"))
        operand, idx = a[0], a[1].astype(np.int64)
        if ivd == idx.ndim:
            idx = idx[..., None]
        idx = np.moveaxis(idx, ivd, -1)  # [...batch, len(sim)]
        batch_shape = idx.shape[:-1]
        out = np.empty(t.shape, dtype=operand.dtype)
        batch_dims_out = [d_ for d_ in range(len(t.shape)) if d_ not in offset_dims]
        kept = [d_ for d_ in range(operand.ndim) if d_ not in collapsed and d_ not in ob]
        # position of each batching dim inside the batch coordinates (index_vector_dim removed)
        sb_pos = [b - (1 if b > ivd else 0) for b in sb]
        for bidx in np.ndindex(*batch_shape):
            start = [0] * operand.ndim
            for k, od in enumerate(sim):
                v = int(idx[bidx + (k,)])
                start[od] = min(max(v, 0), operand.shape[od] - ss[od])
            for k, od in enumerate(ob):
                start[od] = bidx[sb_pos[k]]
            sl = tuple(slice(start[d_], start[d_] + ss[d_]) for d_ in range(operand.ndim))
            piece = operand[sl]
            piece = piece.reshape([ss[d_] for d_ in kept])
            sel = [None] * len(t.shape)
            for k, od in enumerate(batch_dims_out):
                sel[od] = bidx[k]
            for od in offset_dims:
                sel[od] = slice(None)
            out[tuple(sel)] = piece
        return out

    def op_dynamic_slice(self, op, a, t):
        sizes = _ints(op.attrs.get("sizes", op.attrs.get("slice_sizes")))
        x = a[0]
        st = [min(max(int(a[1 + d].reshape(())), 0), x.shape[d] - sizes[d]) for d in range(x.ndim)]
        return x[tuple(slice(s, s + n) for s, n in zip(st, sizes))]

    def op_dynamic_update_slice(self, op, a, t):
        x, u = a[0].copy(), a[1]
        st = [min(max(int(a[2 + d].reshape(())), 0), x.shape[d] - u.shape[d]) for d in range(x.ndim)]
        x[tuple(slice(s, s + n) for s, n in zip(st, u.shape))] = u
        return x

    # -- forms whose shape operands are constants of the module (the result type is static)
    def op_dynamic_reshape(self, op, a, t):
        return a[0].reshape(t.shape)

    def op_dynamic_broadcast_in_dim(self, op, a, t):
        return self.op_broadcast_in_dim(op, a[:1], t)

    def op_dynamic_iota(self, op, a, t):
        return self.op_iota(op, [], t)

    def op_dynamic_pad(self, op, a, t):
        op2 = _with_attrs(op, edge_padding_low=[int(v) for v in a[2]], edge_padding_high=[int(v) for v in a[3]],
                          interior_padding=[int(v) for v in a[4]])
        return self.op_pad(op2, a[:2], t)

    def op_dynamic_gather(self, op, a, t):
        return self.op_gather(_with_attrs(op, slice_sizes=[int(v) for v in a[2]]), a[:2], t)

    def op_bitcast_convert(self, op, a, t):
        """Same bits, other element type; a narrower result gains a minor dimension, a wider one loses it."""
        if "i1" in (op.in_types[0].dtype, t.dtype):
            raise Unsupported("bitcast_convert of i1 (packed bits)")
        raw = np.ascontiguousarray(a[0].astype(_storage_dtype(op.in_types[0].dtype)))
        out = (raw if raw.ndim else raw.reshape(1)).view(_storage_dtype(t.dtype)).reshape(t.shape)
        return out.astype(np.float64) if t.is_float else out

    def op_uniform_quantize(self, op, a, t):
        """The reference's two-operand form: round(x / scale) in the result's integer type
        (Compiler/MPSGraphCompiler.swift:3615-3628), ties to even, saturating like convert."""
        if len(a) != 2:
            raise Unsupported("uniform_quantize with quantised element types")
        with np.errstate(all="ignore"):
            # the quotient is a tensor of the operand's type before it is rounded to an integer
            return _float_to_int(np.rint(round_to(a[0] / a[1], op.in_types[0].dtype)), t)

    def op_uniform_dequantize(self, op, a, t):
        """The reference's two-operand form: float(q) * scale (Compiler/MPSGraphCompiler.swift:3630-3640)."""
        if len(a) != 2:
            raise Unsupported("uniform_dequantize with quantised element types")
        return round_to(np.asarray(a[0]).astype(np.float64), t.dtype) * a[1]

    def op_dynamic_conv(self, op, a, t):
        """stablehlo.dynamic_conv: convolution whose padding is its third operand ([spatial dims, 2])."""
        return self.op_convolution(_with_attrs(op, padding=[int(x) for x in np.asarray(a[2]).reshape(-1)]), a[:2], t)

    def op_convolution(self, op, a, t):
        """stablehlo.convolution: the input is dilated and padded with zeros, and every output element is the dot
        product of a (dilated, possibly reversed) kernel window with the input features of its group."""
        A = op.attrs
        lhs, rhs = a
        rank = lhs.ndim
        ns = rank - 2
        d = dict(A.get("dimension_numbers") or {})
        for k in ("input_batch_dimension", "input_feature_dimension", "input_spatial_dimensions", "kernel_input_feature_dimension",
                  "kernel_output_feature_dimension", "kernel_spatial_dimensions", "output_batch_dimension", "output_feature_dimension",
                  "output_spatial_dimensions"):
            if k in A:
                d[k] = A[k]
        d.setdefault("input_batch_dimension", 0); d.setdefault("input_feature_dimension", rank - 1)
        d.setdefault("input_spatial_dimensions", list(range(1, rank - 1)))
        d.setdefault("kernel_input_feature_dimension", rank - 2); d.setdefault("kernel_output_feature_dimension", rank - 1)
        d.setdefault("kernel_spatial_dimensions", list(range(0, rank - 2)))
        d.setdefault("output_batch_dimension", 0); d.setdefault("output_feature_dimension", rank - 1)
        d.setdefault("output_spatial_dimensions", list(range(1, rank - 1)))
        win = A.get("window") or {}

        def flat(v):
            if v is None:
                return None
            if isinstance(v, tuple) and v and v[0] == "dense":
                return [int(i) for i in np.asarray(dense_value(v[1], v[2])).reshape(-1)]
            return [int(i) for i in np.asarray(v).reshape(-1)]

        def pick(short, long, default):
            v = flat(win.get(short)) if short in win else flat(A.get(long))
            return v if v else default

        stride = pick("stride", "window_strides", [1] * ns)
        pad = pick("pad", "padding", [0] * (2 * ns))
        ldil = pick("lhs_dilate", "lhs_dilation", [1] * ns)
        rdil = pick("rhs_dilate", "rhs_dilation", [1] * ns)
        rev = pick("reverse", "window_reversal", [0] * ns)
        fgc = int(A.get("feature_group_count", 1))
        bgc = int(A.get("batch_group_count", 1))
        # canonical orders: input [B, spatial.., C], kernel [spatial.., I, O], output [B, spatial.., O]
        x = np.transpose(lhs, [d["input_batch_dimension"]] + _ints(d["input_spatial_dimensions"]) + [d["input_feature_dimension"]])
        w = np.transpose(rhs, _ints(d["kernel_spatial_dimensions"]) + [d["kernel_input_feature_dimension"], d["kernel_output_feature_dimension"]])
        wide = np.float64 if x.dtype == np.float64 else (np.uint64 if x.dtype == np.uint64 else np.int64)
        x, w = x.astype(wide), w.astype(wide)
        for k in range(ns):
            if rev[k]:
                w = np.flip(w, axis=k)
        B, C, O = x.shape[0], x.shape[-1], w.shape[-1]
        dil_shape = [(n - 1) * l + 1 if n > 0 else 0 for n, l in zip(x.shape[1:-1], ldil)]
        xd = np.zeros([B] + dil_shape + [C], dtype=wide)
        xd[(slice(None),) + tuple(slice(None, None, l) for l in ldil)] = x
        padded_shape = [max(0, n + pad[2 * k] + pad[2 * k + 1]) for k, n in enumerate(dil_shape)]
        xp = np.zeros([B] + padded_shape + [C], dtype=wide)
        src, dst = [slice(None)], [slice(None)]
        for k, n in enumerate(dil_shape):
            lo, hi = pad[2 * k], pad[2 * k + 1]
            s0, s1 = max(0, -lo), n - max(0, -hi)
            src.append(slice(s0, max(s0, s1)))
            d0 = max(0, lo)
            dst.append(slice(d0, d0 + max(0, s1 - s0)))
        xp[tuple(dst)] = xd[tuple(src)]
        out_sp = [t.shape[i] for i in _ints(d["output_spatial_dimensions"])]
        Bo = B // bgc
        out = np.zeros([Bo] + out_sp + [O], dtype=wide)
        Cg, Og_f, Og_b = C // fgc, O // fgc, O // bgc
        for kidx in np.ndindex(*w.shape[:-2]):
            window = tuple(slice(kk * rd, kk * rd + (n - 1) * st + 1, st) if n > 0 else slice(0, 0)
                           for kk, rd, st, n in zip(kidx, rdil, stride, out_sp))
            patch = xp[(slice(None),) + window]  # [B, out spatial.., C]
            wk = w[kidx]                          # [I, O]
            for oc in range(O):
                g, gb = oc // Og_f, oc // Og_b
                xs = patch[gb * Bo:(gb + 1) * Bo, ..., g * Cg:(g + 1) * Cg]
                with np.errstate(all="ignore"):
                    out[..., oc] += xs @ wk[:, oc]
        perm = [0] * rank
        perm[d["output_batch_dimension"]] = 0
        for k, od in enumerate(_ints(d["output_spatial_dimensions"])):
            perm[od] = 1 + k
        perm[d["output_feature_dimension"]] = rank - 1
        res = np.transpose(out, perm)
        return res if t.is_float else res.astype(t.np_dtype())

    def op_batch_norm_inference(self, op, a, t):
        x, scale, offset, mean, var = a
        axis = int(op.attrs.get("feature_index", 0))
        eps = float(op.attrs.get("epsilon", 0.0))
        shape = [1] * x.ndim
        shape[axis] = x.shape[axis]
        r = lambda v: v.reshape(shape)
        return (x - r(mean)) / np.sqrt(r(var) + eps) * r(scale) + r(offset)

    def op_rng_bit_generator(self, op, a, t):
        """(state) -> (new state, bits): counter-mode Threefry-2x32-20 (Salmon et al. 2011) on state = {key, counter}; word pair
        b is the generator at counter + b; elements of up to 32 bits take one word each, 64-bit elements a pair. The stream is
        implementation-defined by the specification; the reference draws from MPSGraph's generator without reading the state
        (Sources/MetalHLOCore/Compiler/MPSGraphCompiler.swift:4250-4263), so this restates the backend's own choice."""
        state = np.asarray(a[0], dtype=np.uint64)
        ot = op.types[1]
        count = int(np.prod(ot.shape, dtype=np.int64))
        es = np.dtype(ot.np_dtype()).itemsize
        blocks = count if es == 8 else (count + 1) // 2
        key, ctr = int(state[0]), int(state[1])
        c = (np.arange(blocks, dtype=np.uint64) + np.uint64(ctr))
        x0, x1 = (c & np.uint64(0xFFFFFFFF)).astype(np.uint32), (c >> np.uint64(32)).astype(np.uint32)
        k0, k1 = np.uint32(key & 0xFFFFFFFF), np.uint32(key >> 32)
        ks = [k0, k1, k0 ^ k1 ^ np.uint32(0x1BD11BDA)]
        rot = [13, 15, 26, 6, 17, 29, 16, 24]
        with np.errstate(over="ignore"):
            x0 = x0 + ks[0]
            x1 = x1 + ks[1]
            for g in range(5):
                for r in rot[4 * (g % 2):4 * (g % 2) + 4]:
                    x0 = x0 + x1
                    x1 = ((x1 << np.uint32(r)) | (x1 >> np.uint32(32 - r))) ^ x0
                x0 = x0 + ks[(g + 1) % 3]
                x1 = x1 + ks[(g + 2) % 3] + np.uint32(g + 1)
        if es == 8:
            words = x0.astype(np.uint64) | (x1.astype(np.uint64) << np.uint64(32))
        else:
            words = np.stack([x0, x1], axis=1).reshape(-1)[:count]
        unsigned = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[es]
        bits = words.astype(unsigned).view(ot.np_dtype()).reshape(ot.shape)
        new_state = state.copy()
        new_state[1] = np.uint64((ctr + blocks) & 0xFFFFFFFFFFFFFFFF)
        return [new_state, bits]

    def op_optimization_barrier(self, op, a, t):
        return a

    def op_custom_call(self, op, a, t):
        target = op.attrs.get("call_target_name")
        cfg = op.attrs.get("backend_config", "{}")
        cfg = json.loads(cfg) if isinstance(cfg, str) and cfg.strip().startswith("{") else (cfg if isinstance(cfg, dict) else {})
        x = a[0]
        if target == "fused_layer_norm":
            eps = float(cfg.get("eps", 1e-5))
            mean = x.mean(-1, keepdims=True)
            var = ((x - mean) ** 2).mean(-1, keepdims=True)
            y = (x - mean) / np.sqrt(var + eps)
            if len(a) > 1:
                y = y * a[1]
            if len(a) > 2:
                y = y + a[2]
            return y
        if target == "fused_rms_norm":
            eps = float(cfg.get("eps", 1e-5))
            y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
            return y * a[1] if len(a) > 1 else y
        if target == "fused_softmax":
            ax = int(cfg.get("axis", -1))
            e = np.exp(x - x.max(ax, keepdims=True))
            return e / e.sum(ax, keepdims=True)
        if target == "fused_gelu":
            if cfg.get("approximate", True):
                return 0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
            return 0.5 * x * (1 + np.vectorize(math.erf)(x / math.sqrt(2)))
        if target == "fused_silu":
            return x / (1 + np.exp(-x))
        if target == "fused_scaled_dot_product_attention":
            q, k, v = a[0], a[1], a[2]
            s = np.einsum("...qd,...kd->...qk", q, k) * float(cfg.get("scale", 1.0))
            if cfg.get("has_mask") and len(a) > 3:
                s = s + a[3]
            if cfg.get("is_causal"):
                sq, sk = s.shape[-2:]
                s = np.where(np.arange(sk)[None, :] <= np.arange(sq)[:, None], s, -np.inf)  # kv_pos > q_pos is cut
            p = np.exp(s - s.max(-1, keepdims=True))
            p = p / p.sum(-1, keepdims=True)
            return np.einsum("...qk,...kd->...qd", p, v)
        def activate(y, act):
            if act in ("gelu", "gelu_tanh", "gelu_approximate", "geluApproximate"):
                return 0.5 * y * (1 + np.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
            if act in ("gelu_erf", "gelu_exact"):
                return 0.5 * y * (1 + np.vectorize(math.erf)(y / math.sqrt(2)))
            if act == "relu":
                return np.maximum(y, 0)
            if act in ("silu", "swish"):
                return y / (1 + np.exp(-y))
            if act == "tanh":
                return np.tanh(y)
            if act in ("sigmoid", "logistic"):
                return 1 / (1 + np.exp(-y))
            return y

        # The reference's remaining handlers (Sources/MetalHLOCore/Compiler/CustomCallHandlers.swift): batch norm :405-447,
        # convolution + bias + activation :563-640, rotary embedding :715-845, feed-forward :848-925, depth attention :1075-1135
        if target == "fused_batch_norm":
            eps = float(cfg.get("eps", cfg.get("epsilon", 1e-5)))
            return (x - a[3]) / np.sqrt(a[4] + eps) * a[1] + a[2]
        if target == "fused_ffn":
            return activate(x @ a[1], cfg.get("activation", "gelu")) @ a[2]
        if target == "fused_rope":
            hd = x.shape[-1]
            half = hd // 2
            x1, x2, fr = x[..., :half], x[..., half:], a[1]
            if fr.shape[-1] == hd:
                c, s = fr[..., :half], fr[..., half:]
            elif fr.shape[-1] == half:
                c, s = np.cos(fr), np.sin(fr)
            else:
                c, s = fr, (a[2] if len(a) > 2 else np.sin(fr))
            return np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], axis=-1)
        if target == "fused_conv_bias_act":
            y = self.op_convolution(op, a[:2], t)
            if cfg.get("has_bias", True) and len(a) > 2:
                y = y + a[2]
            return activate(y, cfg.get("activation", "none"))
        if target == "fused_depth_attention":
            q, k, v = a[0], a[1], a[2]
            sc = np.einsum("b...h,bdh->b...d", q, k) * float(cfg.get("scale", 1.0))
            w = np.exp(sc - sc.max(-1, keepdims=True))
            w = w / w.sum(-1, keepdims=True)
            return np.einsum("b...d,bdh->b...h", w, v)
        if target == "fused_matmul_bias_activation":
            y = x @ a[1]
            n_plain = len(a) - (1 if cfg.get("has_residual") else 0)
            if n_plain > 2:
                y = y + a[2]
            if cfg.get("has_residual"):
                y = y + a[-1]
            act = cfg.get("activation", "none")
            if act in ("gelu", "gelu_tanh"):
                y = 0.5 * y * (1 + np.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
            elif act == "relu":
                y = np.maximum(y, 0)
            elif act == "silu":
                y = y / (1 + np.exp(-y))
            elif act == "tanh":
                y = np.tanh(y)
            elif act in ("sigmoid", "logistic"):
                y = 1 / (1 + np.exp(-y))
            return y
        raise Unsupported(f"custom_call @{target}")


def evaluate(text, inputs, function: str | None = None, round_floats: bool = False):
    """Runs @main (or `function`) of a StableHLO module on numpy inputs; returns a list of arrays (floats in fp64)."""
    funcs = parse(text)
    f = next((g for g in funcs if g.name == (function or "main")), funcs[0])
    outs = Interpreter(round_floats, funcs).run(f, inputs)
    # complex results leave as (re, im) pairs on a new last axis, the form they cross the C API in
    return [np.stack([o.real, o.imag], axis=-1) if np.iscomplexobj(o) else o for o in outs]
