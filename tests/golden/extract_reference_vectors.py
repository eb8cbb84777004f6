#!/usr/bin/env python3
"""Generates tests/golden/reference_vectors.json from the reference's own test sources.

The reference is a Rust workspace that cannot be compiled where this repository is built,
so its known-answer tests are read as TEXT: this script parses
`crates/maidenx_tensor/tests/ops_binary.rs` and `ops_unary.rs` (one `pub fn <op>_test`
per op, one `match` arm per dtype class) and lifts inputs, scalar arguments, expected
outputs and tolerances out of each arm.  The reduction, matmul, padding, fold and MSE vectors are listed
below by hand with the line they come from; every literal listed is checked to be present
in the cited source range before it is written out.

Usage:  python tests/golden/extract_reference_vectors.py /path/to/reference
"""
from __future__ import annotations

import json
import re
import sys
from pathlib import Path

OUT = Path(__file__).resolve().parent / "reference_vectors.json"

INT_CLASS = ["u8", "u16", "u32", "u64", "i8", "i16", "i32", "i64"]
HALF_CLASS = ["bf16", "f16"]
FLOAT_CLASS = ["f32", "f64"]

CONSTS = {}


def parse_scalar(tok: str):
    tok = tok.strip()
    if tok in ("true", "false"):
        return tok == "true"
    m = re.fullmatch(r"(f32|f64)::(INFINITY|NEG_INFINITY|NAN)", tok)
    if m:
        return {"INFINITY": "inf", "NEG_INFINITY": "-inf", "NAN": "nan"}[m.group(2)]
    m = re.fullmatch(r"(-?\d+(?:\.\d+)?)\s*/\s*(-?\d+(?:\.\d+)?)", tok)
    if m:
        return float(m.group(1)) / float(m.group(2))
    tok = re.sub(r"_?(u8|u16|u32|u64|i8|i16|i32|i64|f32|f64|usize)$", "", tok)
    if re.fullmatch(r"-?\d+", tok):
        return int(tok)
    return float(tok)


def parse_vec(expr: str):
    """`vec![...]`, `NAME.to_vec()` or a flat const name."""
    expr = expr.strip()
    m = re.match(r"vec!\[(.*)\]$", expr, re.S)
    if m:
        body = m.group(1).strip()
        if not body:
            return []
        return [parse_scalar(t) for t in body.split(",") if t.strip()]
    m = re.match(r"(\w+)\.to_vec\(\)$", expr)
    if m:
        return CONSTS[m.group(1)]
    m = re.match(r"(\w+)\.iter\(\)\.flatten\(\)\.copied\(\)\.collect\(\)$", expr)
    if m:
        return CONSTS[m.group(1)]
    raise ValueError(f"cannot parse vector expression: {expr!r}")


def load_consts(text: str):
    for m in re.finditer(r"const (\w+): \[+[^=]*= (\[.*?\]);", text, re.S):
        flat = re.sub(r"[\[\]]", " ", m.group(2))
        CONSTS[m.group(1)] = [parse_scalar(t) for t in flat.split(",") if t.strip()]


def split_functions(text: str):
    """Yield (name, first_line_no, body_lines)."""
    lines = text.split("\n")
    starts = [(i, re.match(r"\s*pub fn (\w+)_test\(dtype: DType\)", l)) for i, l in enumerate(lines)]
    starts = [(i, m.group(1)) for i, m in starts if m]
    for k, (i, name) in enumerate(starts):
        end = starts[k + 1][0] if k + 1 < len(starts) else len(lines)
        yield name, i + 1, lines[i:end]


ARM_RE = re.compile(r"^\s{12}((?:DType::\w+\s*\|?\s*)+|_)\s*=>\s*\{")


def split_arms(body_lines, first_line_no):
    arms = []
    cur = None
    for off, l in enumerate(body_lines):
        m = ARM_RE.match(l)
        if m:
            pat = m.group(1).strip()
            dts = "_" if pat == "_" else [d.lower() for d in re.findall(r"DType::(\w+)", pat)]
            cur = {"dtypes": dts, "line": first_line_no + off, "lines": []}
            arms.append(cur)
        elif cur is not None:
            cur["lines"].append(l)
    return arms


def extract_arm(fn: str, arm, file: str, named_scalars=None):
    src = "\n".join(arm["lines"])
    named_scalars = named_scalars or {}
    local = {}
    for m in re.finditer(r"let (\w+) = (vec!\[[^\]]*\]);", src):
        local[m.group(1)] = parse_vec(m.group(2))
    inputs = {}
    for m in re.finditer(r"let (?:mut )?(\w+)\s*=\s*setup_(?:grad_)?tensor\((.*?), dtype\)\?;", src, re.S):
        expr = m.group(2).strip()
        inputs[m.group(1)] = local[expr] if expr in local else parse_vec(expr)
    if not inputs:
        return None
    # the op call: `let result = x.op(args)?;` or in-place `x.op_(&y)?;`
    call = re.search(r"let result = (\w+)\.(\w+)\((.*?)\)\?;", src)
    inplace = False
    if not call:
        call = re.search(r"^\s*(\w+)\.(\w+_)\((.*?)\)\?;", src, re.M)
        inplace = True
    if not call:
        return None
    recv, method, args = call.group(1), call.group(2), call.group(3).strip()
    rec = {"fn": fn, "cite": f"{file}:{arm['line']}", "method": method, "inplace": inplace, "lhs": inputs[recv]}
    if args.startswith("&"):
        rec["rhs"] = inputs[args[1:]]
    elif args:
        rec["scalar"] = named_scalars[args] if args in named_scalars else parse_scalar(args)
    # expected forward values: exact assert_eq on the result, or `let expected = vec![..]` + tolerance
    target = recv if inplace else "result"
    m = re.search(rf"assert_eq!\(\s*{target}\.to_flatten_vec::<(\w+)>\(\)\?,\s*(vec!\[[^\]]*\])\s*\);", src, re.S)
    if m:
        rec["expected"] = parse_vec(m.group(2))
        rec["read_as"] = m.group(1)
        rec["tol"] = {"exact": True}
    elif re.search(rf"\({target}\.to_flatten_vec::<f32>\(\)\?\[0\] - ", src):
        # indexed form: assert!((result.to_flatten_vec::<f32>()?[i] - X).abs() < tol);
        items = re.findall(rf"\(\({target}\.to_flatten_vec::<f32>\(\)\?\[(\d+)\] - (\(-?[0-9.]+\)|-?[0-9.]+)\)\.abs\(\) < ([0-9.e-]+)\)", src)
        vals = {int(i): (parse_scalar(v.strip("()")), float(t)) for i, v, t in items}
        if sorted(vals) != list(range(len(vals))):
            return None
        rec["expected"] = [vals[i][0] for i in range(len(vals))]
        rec["read_as"] = "f32"
        rec["tol"] = {"abs": max(t for _, t in vals.values())}
    else:
        m = re.search(r"let expected = (vec!\[[^\]]*\]);", src)
        if not m:
            return None
        rec["expected"] = parse_vec(m.group(1))
        rec["read_as"] = "f32"
        after = src[m.end():]
        t = re.search(r"\(a - e\)\.abs\(\) < ([0-9.e-]+)( \* e\.abs\(\))?", after)
        if not t:
            return None
        rec["tol"] = {"rel": float(t.group(1))} if t.group(2) else {"abs": float(t.group(1))}
    return rec


def extract_elementwise(ref: Path, file: str):
    text = (ref / file).read_text()
    load_consts(text)
    out = []
    for fn, line, body in split_functions(text):
        arms = split_arms(body, line)
        # scalars bound before the match, e.g. `let alpha = 0.1;`
        named_scalars = {m.group(1): parse_scalar(m.group(2))
                         for m in re.finditer(r"let (\w+) = (-?[0-9.]+(?:f32)?);", "\n".join(body[:4]))}
        named = {d for a in arms if a["dtypes"] != "_" for d in a["dtypes"]}
        for arm in arms:
            try:
                rec = extract_arm(fn, arm, file, named_scalars)
            except (ValueError, KeyError):
                rec = None  # arm built from Rust expressions rather than literals (e.g. elu): not liftable as text
            if rec is None:
                continue
            rec["dtypes"] = [d for d in FLOAT_CLASS if d not in named] if arm["dtypes"] == "_" else arm["dtypes"]
            out.append(rec)
    return out


# ---------------------------------------------------------------------------------------
# Hand-listed vectors (shape-carrying tests).  `needles` must all occur in the cited lines.
# ---------------------------------------------------------------------------------------
D1 = [1.0, 2.0, 3.0, 4.0]
D2 = [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]
U2 = [1, 2, 3, 4]
RED = "crates/maidenx_tensor/tests/ops_reduction.rs"
MM = "crates/maidenx_tensor/tests/ops_matmul.rs"
MSE = "crates/maidenx_nn/src/losses/mse.rs"

REDUCTIONS = [
    # op, input, shape, dim (or target shape), expected, dtype classes, cite(lines), needles
    ("sum", D1, [4], 0, [10.0], "all", (RED, 15, 30), ["x.sum(0, false)", "vec![10.0]"]),
    ("sum", D2, [2, 3], 0, [5.0, 7.0, 9.0], "all", (RED, 31, 45), ["x.sum(0, false)", "vec![5.0, 7.0, 9.0]"]),
    ("sum", D2, [2, 3], 1, [6.0, 15.0], "all", (RED, 46, 59), ["x.sum(1, false)", "vec![6.0, 15.0]"]),
    ("sum_to_shape", D2, [2, 3], [1, 3], [5.0, 7.0, 9.0], "all", (RED, 267, 318), ["x.sum_to_shape(&[1, 3])", "vec![5.0, 7.0, 9.0]"]),
    ("mean", D2, [2, 3], 0, [2.5, 3.5, 4.5], "float", (RED, 337, 430), ["x.mean(0, false)", "vec![2.5, 3.5, 4.5]"]),
    ("max", U2, [2, 2], 0, [3, 4], "int", (RED, 613, 627), ["x.max(0, false)", "vec![3, 4]"]),
    ("max", D2, [2, 3], 0, [4.0, 5.0, 6.0], "float", (RED, 628, 725), ["x.max(0, false)", "vec![4.0, 5.0, 6.0]"]),
    ("min", D2, [2, 3], 0, [1.0, 2.0, 3.0], "float", (RED, 833, 930), ["x.min(0, false)", "vec![1.0, 2.0, 3.0]"]),
]

MATMULS = [
    # a, a_shape, b, b_shape, c, grad_a, grad_b (gradients of sum(c)), cite, needles
    ([1, 2, 3], [3], [4, 5, 6], [3], [32], [4, 5, 6], [1, 2, 3], (MM, 11, 67),
     ["vec![32.0f32]", "vec![4.0f32, 5.0, 6.0]", "vec![1.0f32, 2.0, 3.0]"]),
    ([1, 2, 3, 4, 5, 6], [2, 3], [2, 1, 3], [3], [13, 31], [2, 1, 3, 2, 1, 3], [5, 7, 9], (MM, 69, 128),
     ["vec![13.0f32, 31.0]", "vec![2.0f32, 1.0, 3.0, 2.0, 1.0, 3.0]", "vec![5.0f32, 7.0, 9.0]"]),
    ([2, 3], [2], [1, 2, 3, 4, 5, 6], [2, 3], [14, 19, 24], [6, 15], [2, 2, 2, 3, 3, 3], (MM, 130, 189),
     ["vec![14.0f32, 19.0, 24.0]", "vec![6.0f32, 15.0]", "vec![2.0f32, 2.0, 2.0, 3.0, 3.0, 3.0]"]),
    ([1, 2, 3, 4], [2, 2], [5, 6, 7, 8], [2, 2], [19, 22, 43, 50], [11, 15, 11, 15], [4, 4, 6, 6], (MM, 191, 247),
     ["vec![19.0f32, 22.0, 43.0, 50.0]", "vec![11.0f32, 15.0, 11.0, 15.0]", "vec![4.0f32, 4.0, 6.0, 6.0]"]),
    ([1, 2, 3, 4, 5, 6, 7, 8], [2, 2, 2], [9, 10, 11, 12, 13, 14, 15, 16], [2, 2, 2],
     [31, 34, 71, 78, 155, 166, 211, 226], [19, 23, 19, 23, 27, 31, 27, 31], [4, 4, 6, 6, 12, 12, 14, 14], (MM, 249, 325),
     ["vec![31.0f32, 34.0, 71.0, 78.0, 155.0, 166.0, 211.0, 226.0]", "vec![19.0f32, 23.0, 19.0, 23.0, 27.0, 31.0, 27.0, 31.0]",
      "vec![4.0f32, 4.0, 6.0, 6.0, 12.0, 12.0, 14.0, 14.0]"]),
]

MSE_CASE = {"pred": [2.0, 3.0, 4.0], "target": [1.0, 2.0, 3.0], "loss": 1.0, "grad": [2.0 / 3.0] * 3,
            "cite": (MSE, 45, 79), "needles": ["vec![2.0f32, 3.0, 4.0]", "vec![1.0f32, 2.0, 3.0]", "vec![1.0]", "2.0 / 3.0"]}


PAD = "crates/maidenx_tensor/tests/ops_padding.rs"
X1 = [1.0, 2.0, 3.0, 4.0]                 # TEST_DATA_F32_1D (ops_padding.rs:9)
X2 = [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]       # TEST_DATA_F32_2D flattened (ops_padding.rs:10)
# (mode, input, shape, pads, pad value, expected output, expected grad of the input under backward of sum | None, cite, needles)
PADDINGS = [
    ("constant", X1, [4], [(1, 2)], 0.0, [0.0, 1.0, 2.0, 3.0, 4.0, 0.0, 0.0], [1.0] * 4, (PAD, 116, 131),
     ["x.pad(&[(1, 2)], 0.0)", "vec![0.0, 1.0, 2.0, 3.0, 4.0, 0.0, 0.0]", "vec![1.0, 1.0, 1.0, 1.0]"]),
    ("constant", X2, [2, 3], [(1, 1), (2, 1)], 3.0,
     [3.0] * 8 + [1.0, 2.0, 3.0] + [3.0] * 3 + [4.0, 5.0, 6.0] + [3.0] * 7, [1.0] * 6, (PAD, 133, 151),
     ["x.pad(&[(1, 1), (2, 1)], 3.0)", "3.0, 3.0, 3.0, 3.0, 3.0, 3.0, 3.0, 3.0, 1.0, 2.0, 3.0, 3.0, 3.0, 3.0, 4.0, 5.0, 6.0, 3.0, 3.0, 3.0,",
      "vec![1.0, 1.0, 1.0, 1.0, 1.0, 1.0]"]),
    ("constant", X1, [4], [(0, 2)], 9.9, [1.0, 2.0, 3.0, 4.0, 9.9, 9.9], None, (PAD, 153, 160),
     ["x.pad(&[(0, 2)], 9.9)", "vec![1.0, 2.0, 3.0, 4.0, 9.9, 9.9]"]),
    ("reflection", X1, [4], [(2, 2)], None, [3.0, 2.0, 1.0, 2.0, 3.0, 4.0, 3.0, 2.0], [1.0, 3.0, 3.0, 1.0], (PAD, 237, 254),
     ["x.pad_with_reflection(&[(2, 2)])", "vec![3.0, 2.0, 1.0, 2.0, 3.0, 4.0, 3.0, 2.0]", "vec![1.0, 3.0, 3.0, 1.0]"]),
    ("reflection", X2, [2, 3], [(1, 1), (2, 2)], None,
     [6.0, 5.0, 4.0, 5.0, 6.0, 5.0, 4.0, 3.0, 2.0, 1.0, 2.0, 3.0, 2.0, 1.0, 6.0, 5.0, 4.0, 5.0, 6.0, 5.0, 4.0, 3.0, 2.0, 1.0, 2.0, 3.0, 2.0, 1.0],
     None, (PAD, 256, 267),
     ["x.pad_with_reflection(&[(1, 1), (2, 2)])", "6.0, 5.0, 4.0, 5.0, 6.0, 5.0, 4.0, 3.0, 2.0, 1.0, 2.0, 3.0, 2.0, 1.0, 6.0, 5.0, 4.0, 5.0, 6.0, 5.0,"]),
    ("replication", X1, [4], [(2, 2)], None, [1.0, 1.0, 1.0, 2.0, 3.0, 4.0, 4.0, 4.0], [3.0, 1.0, 1.0, 3.0], (PAD, 370, 386),
     ["x.pad_with_replication(&[(2, 2)])", "vec![1.0, 1.0, 1.0, 2.0, 3.0, 4.0, 4.0, 4.0]", "vec![3.0, 1.0, 1.0, 3.0]"]),
    ("replication", X2, [2, 3], [(1, 1), (2, 2)], None,
     [1.0, 1.0, 1.0, 2.0, 3.0, 3.0, 3.0, 1.0, 1.0, 1.0, 2.0, 3.0, 3.0, 3.0, 4.0, 4.0, 4.0, 5.0, 6.0, 6.0, 6.0, 4.0, 4.0, 4.0, 5.0, 6.0, 6.0, 6.0],
     None, (PAD, 388, 399),
     ["x.pad_with_replication(&[(1, 1), (2, 2)])", "1.0, 1.0, 1.0, 2.0, 3.0, 3.0, 3.0, 1.0, 1.0, 1.0, 2.0, 3.0, 3.0, 3.0, 4.0, 4.0, 4.0, 5.0, 6.0, 6.0,"]),
]
# fold of an unfolded view: (input, shape, unfold dim, window size, step, expected, cite, needles); the unfolded view has
# the window count at `dim` (stride step * stride[dim]) and the window as the next dim (crates/maidenx_core/src/layout.rs:193-250)
FOLDS = [
    ([1.0, 2.0, 3.0, 4.0, 5.0], [5], 0, 2, 1, [1.0, 4.0, 6.0, 8.0, 5.0], (RED, 484, 497),
     ["vec![1.0, 2.0, 3.0, 4.0, 5.0]", "x.unfold(0, 2, 1)", "unfolded.fold(0, 2, 1)", "vec![1.0, 4.0, 6.0, 8.0, 5.0]"]),
    (X2, [2, 3], 1, 2, 1, [1.0, 4.0, 3.0, 4.0, 10.0, 6.0], (RED, 520, 531),
     ["x_2d.unfold(1, 2, 1)", "unfolded_2d.fold(1, 2, 1)", "vec![1.0, 4.0, 3.0, 4.0, 10.0, 6.0]"]),
]


def check_needles(ref: Path, cite, needles):
    file, lo, hi = cite
    lines = (ref / file).read_text().split("\n")[lo - 1:hi]
    chunk = re.sub(r"\s+", " ", " ".join(lines))
    for n in needles:
        if re.sub(r"\s+", " ", n) not in chunk:
            raise SystemExit(f"golden provenance check failed: {n!r} not in {file}:{lo}-{hi}")
    return f"{file}:{lo}-{hi}"


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: extract_reference_vectors.py <path to a checkout of the reference (miniex/maidenx)>")
    ref = Path(sys.argv[1])
    data = {
        "_comment": "Known-answer vectors of the reference's own tests, lifted from its test sources as text by "
                    "tests/golden/extract_reference_vectors.py. Every fixture in those tests is a padded buffer "
                    "viewed from element 1 (crates/maidenx_tensor/tests/utils/mod.rs:30-37), i.e. offset = 1.",
        "binary": extract_elementwise(ref, "crates/maidenx_tensor/tests/ops_binary.rs"),
        "unary": extract_elementwise(ref, "crates/maidenx_tensor/tests/ops_unary.rs"),
        "reduction": [],
        "matmul": [],
    }
    for op, x, shape, arg, exp, classes, cite, needles in REDUCTIONS:
        data["reduction"].append({"op": op, "input": x, "shape": shape, "arg": arg, "expected": exp, "classes": classes,
                                  "cite": check_needles(ref, cite, needles)})
    for a, ash, b, bsh, c, ga, gb, cite, needles in MATMULS:
        data["matmul"].append({"a": a, "a_shape": ash, "b": b, "b_shape": bsh, "c": c, "grad_a": ga, "grad_b": gb,
                               "cite": check_needles(ref, cite, needles)})
    data["padding"] = [{"mode": mode, "input": x, "shape": shape, "pads": [list(p) for p in pads], "value": value, "expected": exp, "grad": grad,
                        "cite": check_needles(ref, cite, needles)} for mode, x, shape, pads, value, exp, grad, cite, needles in PADDINGS]
    data["fold"] = [{"input": x, "shape": shape, "dim": dim, "size": size, "step": step, "expected": exp, "cite": check_needles(ref, cite, needles)}
                    for x, shape, dim, size, step, exp, cite, needles in FOLDS]
    m = dict(MSE_CASE)
    m["cite"] = check_needles(ref, m["cite"], m.pop("needles"))
    data["mse"] = m
    OUT.write_text(json.dumps(data, indent=1) + "\n")
    print(f"wrote {OUT}: {len(data['binary'])} binary, {len(data['unary'])} unary, "
          f"{len(data['reduction'])} reduction, {len(data['matmul'])} matmul records")


if __name__ == "__main__":
    main()
