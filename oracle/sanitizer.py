"""Forward-graph text patches, restated from the reference.  Test infrastructure only.

Follows src/compiler/sanitizer.zig:
  apply_stability_patches  :8-111   every `stablehlo.log x` becomes log(x + 1e-4) and every
                                    `stablehlo.divide a, b` becomes a / (b + 1e-4), by inserting a
                                    splat constant and an add in front of the op (line based).
  sanitize_hex_floats      :129-244 bf16 models only: 32-bit hex float literals outside the
                                    resource section become decimals; 0xFF800000 (-inf) becomes
                                    -65504.
The third pass of the reference (:246-314, large splat constants -> scalar + broadcast) does not
change any value and is omitted.

One deliberate difference: the reference matches the substring "stablehlo.log", which also hits
`stablehlo.logistic` and would rewrite a sigmoid into a logarithm.  That only concerns graphs with
SiLU (not the nanochat / nanoGPT families); this restatement patches `stablehlo.log` proper only.
"""
from __future__ import annotations

import re
import struct


def _type_at_end(line: str):
    k = line.rfind(":")
    if k < 0:
        return None
    t = line[k + 1:].strip()
    if t.startswith("tensor<") and "?" not in t:
        return t
    return None


def apply_stability_patches(source: str) -> str:
    out = []
    count = 0
    for line in source.split("\n"):
        is_log = re.search(r"stablehlo\.log(?![a-z_])", line) is not None
        is_div = "stablehlo.divide" in line
        ty = _type_at_end(line) if (is_log or is_div) else None
        if ty is None:
            out.append(line)
            continue
        toks = [t for t in re.split(r"[ =:]+", line.strip()) if t]
        if is_log and len(toks) >= 3:
            res, arg = toks[0], toks[2]
            out.append(f"    %eps_log_{count} = stablehlo.constant dense<1.000000e-4> : {ty}")
            out.append(f"    %safe_log_{count} = stablehlo.add {arg}, %eps_log_{count} : {ty}")
            out.append(f"    {res} = stablehlo.log %safe_log_{count} : {ty}")
            count += 1
        elif is_div and len(toks) >= 4:
            res, lhs, rhs = toks[0], toks[2].rstrip(","), toks[3].rstrip(",")
            out.append(f"    %eps_div_{count} = stablehlo.constant dense<1.000000e-4> : {ty}")
            out.append(f"    %safe_denom_{count} = stablehlo.add {rhs}, %eps_div_{count} : {ty}")
            out.append(f"    {res} = stablehlo.divide {lhs}, %safe_denom_{count} : {ty}")
            count += 1
        else:
            out.append(line)
    return "\n".join(out)


def sanitize_hex_floats(source: str) -> str:
    end = source.find("dialect_resources:")
    if end < 0:
        end = len(source)
    head, tail = source[:end], source[end:]

    def repl(m):
        h = m.group(1)
        if h.upper() == "FF800000":
            return "-6.550400e+04"
        (f,) = struct.unpack("<f", struct.pack("<I", int(h, 16)))
        if f != f:
            return "0x7FC0"
        if f == float("inf"):
            return "0x7F80"
        if f == float("-inf"):
            return "0xFF80"
        return f"{f:.6e}"

    return re.sub(r"0x([0-9A-Fa-f]{8})", repl, head) + tail


def model_dtype_of(source: str) -> str:
    """Element type of the first @main argument (the model dtype of the export)."""
    m = re.search(r"func\.func\s+(?:public\s+)?@main\(%arg0:\s*tensor<[0-9x]*x?([a-z0-9]+)>", source)
    return m.group(1) if m else "f32"


def sanitize(source: str) -> str:
    """The pipeline DiLoCo.init applies to a model file (src/algorithms/diloco.zig:158-177)."""
    s = apply_stability_patches(source)
    if model_dtype_of(source) == "bf16":
        s = sanitize_hex_floats(s)
    return s
