#!/usr/bin/env python3
"""MLIR bytecode on stdin -> StableHLO text on stdout.

The PJRT plugin runs this script in the interpreter named by METALHLO_PYTHON when JAX hands it a program as MLIR
bytecode (a VHLO portable artifact): jaxlib deserializes the artifact, the module is printed, and the annotations JAX adds
for its own use are taken out. Same job as the reference's helper (python/jax_plugins/metalhlo/bytecode_to_text.py:13-100
and the script embedded in Sources/PJRTMetalHLO/PJRTExecutable.swift:28-190). This backend's parser reads the generic op
form, `<{...}>` property dictionaries, `array<i64: ...>` and `#stablehlo.gather<...>` attributes and all convolution
spellings as printed, so none of the reference's rewrites of those are needed; what remains is `clean()` below.
"""
import re
import sys


def strip_sharding_constraints(text: str) -> str:
    """`%out = sdy.sharding_constraint %in <...> : type` is the identity: the line goes and %out is renamed to %in inside
    the function that held it (not globally: SSA names repeat across functions)."""
    lines = text.split("\n")
    bounds, start = [], None
    for i, line in enumerate(lines):
        if re.match(r"\s*func\.func\b", line):
            start = i
        elif re.match(r"\s*\}\s*$", line) and start is not None:
            bounds.append((start, i))
            start = None
    for i, line in enumerate(lines):
        m = re.match(r"^\s*(%[\w.#-]+)\s*=\s*sdy\.sharding_constraint\s+(%[\w.#-]+)\b", line)
        if not m:
            continue
        out_name, in_name = m.group(1), m.group(2)
        lo, hi = next(((a, b) for a, b in bounds if a <= i <= b), (0, len(lines) - 1))
        lines[i] = ""
        pat = re.compile(re.escape(out_name) + r"(?![\w.#-])")
        for j in range(lo, hi + 1):
            lines[j] = pat.sub(in_name, lines[j])
    return "\n".join(lines)


def clean(text: str) -> str:
    """Takes JAX's own annotations out of a printed StableHLO module."""
    # module attributes (mhlo.num_partitions, jax.uses_shape_polymorphism, ...), possibly with nested braces
    text = re.sub(r"(module\s+@[\w.$-]+)\s+attributes\s+\{(?:[^{}]|\{[^{}]*\})*\}", r"\1", text)
    # Shardy: mesh declarations, sharding attributes, identity constraints
    text = re.sub(r"^\s*sdy\.mesh\s+@\S+\s*=\s*<[^>]*>\s*$", "", text, flags=re.MULTILINE)
    text = re.sub(r"\s*\{sdy\.sharding\s*=\s*#sdy\.sharding<[^>]*>\}", "", text)
    text = re.sub(r",?\s*sdy\.sharding\s*=\s*#sdy\.sharding(?:_per_value)?<(?:[^<>]|<[^<>]*>)*>", "", text)
    text = strip_sharding_constraints(text)
    # argument / result attributes: {jax.result_info = "..."}, {mhlo.sharding = "..."}, {mhlo.layout_mode = "..."}, {tf.aliasing_output = 0 : i32}
    text = re.sub(r"\s*\{\s*(?:(?:jax|mhlo|tf)\.[\w.]+\s*=\s*(?:\"[^\"]*\"|-?\d+\s*:\s*i\d+|true|false|\[[^\]]*\])\s*,?\s*)+\}", "", text)
    # a composite names a decomposition function: call it
    text = re.sub(r'stablehlo\.composite\s+"[^"]*"\s+([^{]+?)\s*\{[^}]*decomposition\s*=\s*@([\w.$-]+)[^}]*\}', r"func.call @\2(\1)", text)
    text = re.sub(r"\n\s*\n\s*\n", "\n\n", text)
    return text


def deserialize(bytecode: bytes) -> str:
    from jax._src.interpreters.mlir import make_ir_context
    from jaxlib.mlir._mlir_libs import _stablehlo

    ctx = make_ir_context()
    return str(_stablehlo.deserialize_portable_artifact(ctx, bytecode))


def main() -> int:
    bytecode = sys.stdin.buffer.read()
    if bytecode[:4] != b"ML\xefR":
        sys.stderr.write("bytecode_to_text: stdin does not hold MLIR bytecode\n")
        return 2
    sys.stdout.write(clean(deserialize(bytecode)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
