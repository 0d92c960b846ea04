"""Loader for the StableHLO interpreter suite the reference vendors
(Tests/MetalHLOTests/Conformance/StableHLO/interpret/*.mlir): splits a file into cases on `// -----`, pulls the
`check.expect_*` lines out of each function and rewrites the function so that it returns the checked values.
Same convention as the reference's InterpretTestParser (Tests/MetalHLOTests/Conformance/InterpretTestParser.swift:62-241).

The suite is read from the reference checkout when one is present: the directory named by MHLO_INTERP_SUITE_DIR, else the
checkout beside this repository. Where there is none (the GPU box), the cases come from tests/golden/interp_suite.json.gz,
which tests/golden/make_interp_suite.py wrote from that checkout with this same loader.
"""
from __future__ import annotations

import gzip
import json
import os
import re

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SUITE_DIR = os.environ.get("MHLO_INTERP_SUITE_DIR") or os.path.join(
    os.path.dirname(_ROOT), "reference", "Tests", "MetalHLOTests", "Conformance", "StableHLO", "interpret")
FIXTURE = os.path.join(_ROOT, "tests", "golden", "interp_suite.json.gz")

# the operator surface of this backend (the fused hot path + the data-movement ops around it)
FILES = ["abs", "add", "and", "atan2", "broadcast_in_dim", "cbrt", "ceil", "clamp", "compare", "concatenate", "constant",
         "convert", "cosine", "count_leading_zeros", "divide", "dot_general", "dynamic_slice", "dynamic_update_slice",
         "exponential", "exponential_minus_one", "floor", "gather", "iota", "is_finite", "log", "log_plus_one", "logistic",
         "maximum", "minimum", "multiply", "negate", "not", "or", "pad", "popcnt", "power", "reduce", "remainder", "reshape",
         "reverse", "round_nearest_afz", "round_nearest_even", "rsqrt", "select", "shift_left", "shift_right_arithmetic",
         "shift_right_logical", "sign", "sine", "slice", "sqrt", "subtract", "tan", "tanh", "transpose", "xor",
         # control flow and the operators either side of the fused path
         "bitcast_convert", "call", "case", "if", "while", "dynamic_broadcast_in_dim", "dynamic_gather", "dynamic_iota",
         "dynamic_pad", "dynamic_reshape", "optimization_barrier", "reduce_window", "scatter", "sort", "convolution", "select_and_scatter", "map",
         "get_dimension_size", "reduce_precision", "composite",
         # complex values: (re, im) float pairs behind the parser
         "complex", "real", "imag",
         "tuple_and_get_tuple_element", "dynamic_conv"]


class Case:
    def __init__(self, file, name, text, checks):
        self.file, self.name, self.text, self.checks = file, name, text, checks

    @property
    def id(self):
        return f"{self.file}:{self.name}"


_CHECK = re.compile(r"check\.(expect_eq_const|expect_almost_eq_const|expect_eq|expect_almost_eq|expect_close)\s+(.*?)\s*:\s*(tensor<(?:[^<>]|<[^<>]*>)*>)"
                    r"(?:\s*,\s*tensor<(?:[^<>]|<[^<>]*>)*>)?", re.S)


def _split_dense(rest):
    """'%v, dense<...>' -> ('%v', 'dense body')"""
    m = re.match(r"(%[\w.#\-]+)\s*,\s*dense<(.*)>\s*$", rest, re.S)
    return (m.group(1), m.group(2)) if m else None


def _functions(chunk):
    """Top-level `func.func` definitions of one chunk as (name, start, end of the closing brace)."""
    out = []
    for m in re.finditer(r"func\.func\s+(?:private\s+|public\s+)?@([\w.]+)", chunk):
        if out and m.start() < out[-1][2]:
            continue  # nested inside the previous function (cannot happen in MLIR, but stay safe)
        depth, i = 0, chunk.index("{", m.end())
        while True:
            c = chunk[i]
            if c == "{":
                depth += 1
            elif c == "}":
                depth -= 1
                if depth == 0:
                    break
            i += 1
        out.append((m.group(1), m.start(), i + 1))
    return out


def load_cases(file):
    path = os.path.join(SUITE_DIR, file + ".mlir")
    text = open(path).read()
    cases = []
    for chunk in re.split(r"^// -----\s*$", text, flags=re.M):
        chunk = re.sub(r"^\s*//[^\n]*$", "", chunk, flags=re.M)  # RUN / comment lines
        funcs = _functions(chunk)
        # the function that carries the checks is the test; the others are its callees and are kept as they are
        tests = [f for f in funcs if "check." in chunk[f[1]:f[2]]]
        if len(tests) != 1:
            continue
        name, start, end = tests[0]
        m = re.match(r"func\.func\s+(?:private\s+|public\s+)?@[\w.]+\s*\(\s*\)\s*(?:->\s*[^{]*)?\{", chunk[start:end])
        if not m:
            continue
        body = chunk[start + m.end():end - 1]
        callees = "".join(chunk[s:e] + "\n" for n, s, e in funcs if (n, s, e) != tests[0])
        checks, returns, ret_types = [], [], []
        ok = True

        def repl(cm):
            nonlocal ok
            kind, rest, ttype = cm.group(1), cm.group(2), cm.group(3)
            if kind.endswith("_const"):
                sd = _split_dense(rest)
                if not sd:
                    ok = False
                    return ""
                checks.append({"kind": kind, "value": len(returns), "dense": sd[1], "type": ttype})
                returns.append(sd[0]); ret_types.append(ttype)
            else:
                vals = [v.strip() for v in rest.split(",")][:2]
                if len(vals) != 2 or not all(v.startswith("%") for v in vals):
                    ok = False
                    return ""
                checks.append({"kind": kind, "value": len(returns), "other": len(returns) + 1, "type": ttype})
                returns.extend(vals); ret_types.extend([ttype, ttype])
            return ""

        body = _CHECK.sub(repl, body)
        body = re.sub(r"(func\.)?return\s*$", "", body.rstrip())
        body = re.sub(r"\n\s*(func\.)?return\b[^\n]*", "", body)
        if not ok or not returns or "check." in body:
            continue
        new = (f"func.func @main() -> ({', '.join(ret_types)}) {{\n{body}\n  return {', '.join(returns)} : "
               f"{', '.join(ret_types)}\n}}\n")
        if callees:
            new = "module {\n" + new + callees + "}\n"
        cases.append(Case(file, name, new, checks))
    return cases


def cases_from_checkout():
    out = []
    if not os.path.isdir(SUITE_DIR):
        return out
    for f in FILES:
        if os.path.exists(os.path.join(SUITE_DIR, f + ".mlir")):
            out.extend(load_cases(f))
    return out


def cases_from_fixture():
    if not os.path.exists(FIXTURE):
        return []
    with gzip.open(FIXTURE, "rt") as f:
        doc = json.load(f)
    return [Case(c["file"], c["name"], c["text"], c["checks"]) for c in doc["cases"]]


def all_cases():
    """The suite from the reference checkout; from the committed fixture where there is no checkout."""
    return cases_from_checkout() or cases_from_fixture()


UNSUPPORTED_MARKERS = ("f8E", "f4E", "f6E", "i2>", "i4>", "ui2>", "ui4>", "tf32", "quant", "x?x", "<?x", "token")


def skip_reason(text):
    """Element types outside the backend's 13 (MHLOElementType) put a case out of scope."""
    for bad in UNSUPPORTED_MARKERS:
        if bad in text:
            return bad
    return None


def verify(case, outs):
    """Holds the returned values of one case to its goldens with the reference runner's tolerances: exact for
    expect_eq, 1e-4 for expect_almost_eq / expect_close (Conformance/InterpretTestRunner.swift:37-45); 16-bit floats are
    compared after rounding both sides to the type."""
    import numpy as np

    from oracle import interp

    for chk in case.checks:
        got = np.asarray(outs[chk["value"]])
        t = interp.Scanner(chk["type"]).type()
        want = interp.dense_value(chk["dense"], t) if "dense" in chk else np.asarray(outs[chk["other"]])
        if t.is_complex:  # results leave as (re, im) pairs on a last axis
            want = np.asarray(want, dtype=np.complex128)
            want = np.stack([want.real, want.imag], axis=-1)
            if np.iscomplexobj(got):
                got = np.stack([got.real, got.imag], axis=-1)
            tol = 1e-6 if chk["kind"].startswith("expect_eq") else 1e-4
            np.testing.assert_allclose(got.astype(np.float64), want, rtol=tol, atol=tol, equal_nan=True, err_msg=case.id)
            continue
        if t.is_float:
            tol = 0 if chk["kind"].startswith("expect_eq") else 1e-4
            got = got.astype(np.float64)
            want = np.asarray(want, dtype=np.float64)
            if t.dtype in ("f16", "bf16"):
                want = interp.round_to(want, t.dtype)
                got = interp.round_to(got, t.dtype)
                tol = max(tol, 1e-2)
            elif t.dtype == "f32":
                got = interp.round_to(got, "f32")
                tol = max(tol, 1e-6)
            np.testing.assert_allclose(got, want, rtol=tol, atol=tol, equal_nan=True, err_msg=case.id)
        else:
            np.testing.assert_array_equal(got, np.asarray(want).astype(got.dtype) if got.dtype != np.asarray(want).dtype else want, err_msg=case.id)
