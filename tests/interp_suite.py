"""Loader for the StableHLO interpreter suite the reference vendors
(Tests/MetalHLOTests/Conformance/StableHLO/interpret/*.mlir): splits a file into cases on `// -----`, pulls the
`check.expect_*` lines out of each function and rewrites the function so that it returns the checked values.
Same convention as the reference's InterpretTestParser (Tests/MetalHLOTests/Conformance/InterpretTestParser.swift:62-241).

The suite lives in the reference checkout only; nothing of it is copied into this repository.
"""
from __future__ import annotations

import os
import re

SUITE_DIR = "/root/reference/Tests/MetalHLOTests/Conformance/StableHLO/interpret"

# the operator surface of this backend (SURVEY hot path + the data-movement ops around it)
FILES = ["abs", "add", "and", "atan2", "broadcast_in_dim", "cbrt", "ceil", "clamp", "compare", "concatenate", "constant",
         "convert", "cosine", "count_leading_zeros", "divide", "dot_general", "dynamic_slice", "dynamic_update_slice",
         "exponential", "exponential_minus_one", "floor", "gather", "iota", "is_finite", "log", "log_plus_one", "logistic",
         "maximum", "minimum", "multiply", "negate", "not", "or", "pad", "popcnt", "power", "reduce", "remainder", "reshape",
         "reverse", "round_nearest_afz", "round_nearest_even", "rsqrt", "select", "shift_left", "shift_right_arithmetic",
         "shift_right_logical", "sign", "sine", "slice", "sqrt", "subtract", "tan", "tanh", "transpose", "xor",
         # control flow and the operators either side of the fused path
         "bitcast_convert", "call", "case", "if", "while", "dynamic_broadcast_in_dim", "dynamic_gather", "dynamic_iota",
         "dynamic_pad", "dynamic_reshape", "optimization_barrier", "reduce_window", "scatter", "sort", "convolution", "select_and_scatter", "map"]


class Case:
    def __init__(self, file, name, text, checks):
        self.file, self.name, self.text, self.checks = file, name, text, checks

    @property
    def id(self):
        return f"{self.file}:{self.name}"


_CHECK = re.compile(r"check\.(expect_eq_const|expect_almost_eq_const|expect_eq|expect_almost_eq|expect_close)\s+(.*?)\s*:\s*(tensor<[^>]*>)"
                    r"(?:\s*,\s*tensor<[^>]*>)?", re.S)


def _split_dense(rest):
    """'%v, dense<...>' -> ('%v', 'dense body')"""
    m = re.match(r"(%[\w.#\-]+)\s*,\s*dense<(.*)>\s*$", rest, re.S)
    return (m.group(1), m.group(2)) if m else None


def load_cases(file):
    path = os.path.join(SUITE_DIR, file + ".mlir")
    text = open(path).read()
    cases = []
    for chunk in re.split(r"^// -----\s*$", text, flags=re.M):
        m = re.search(r"func\.func\s+@([\w.]+)\s*\(\s*\)\s*(?:->\s*[^{]*)?\{", chunk)
        if not m:
            continue
        name = m.group(1)
        body_start = m.end()
        body_end = chunk.rfind("}")
        body = chunk[body_start:body_end]
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
        cases.append(Case(file, name, new, checks))
    return cases


def all_cases():
    out = []
    if not os.path.isdir(SUITE_DIR):
        return out
    for f in FILES:
        if os.path.exists(os.path.join(SUITE_DIR, f + ".mlir")):
            out.extend(load_cases(f))
    return out
