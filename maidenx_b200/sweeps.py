"""The single-op workloads the benchmark sweeps, with their algorithmic byte counts.

Shapes, value ranges and layouts are the ones the target configurations name:
  * elementwise: 2^28-element tensors viewed as [16384, 16384]; contiguous, transposed lhs
    (strides [1, 16384]), rhs broadcast from [1, 16384] (strides [0, 1]) and contiguous views that
    start at element 1 of their buffers (the reference's test fixtures); add/sub/mul/div
    and exp/relu/gelu/neg in f32 / bf16 / f16, add/mul in i32;
  * reductions: [8192, 16384] sum along dim 0 and dim 1, mean, max in f32 / bf16, i32 sum,
    and the sum_to_shape fold [64, 512, 4096] -> [1, 1, 4096];
  * conv: im2col / col2im for N=64, C=256, H=W=56, 3x3, stride 1, pad 1 in bf16 / f32.
Algorithmic bytes = bytes every correct implementation must move between HBM and the SMs:
each distinct input element read once, each output element written once.
"""
from __future__ import annotations

from dataclasses import dataclass, field

ELEM_SIZE = {"f32": 4, "bf16": 2, "f16": 2, "i32": 4, "f64": 8}


@dataclass
class Case:
    name: str            # e.g. add_bf16/transposed_lhs
    op: str
    dtype: str
    family: str          # binary | unary | reduce | sum_to_shape | im2col | col2im
    metadata: list
    num_els: int
    in_elems: list       # element count of each input buffer
    out_elems: int
    bytes: int           # algorithmic bytes per launch
    extra: dict = field(default_factory=dict)


def elementwise_cases(R: int = 16384, C: int = 16384, dtypes=("f32", "bf16", "f16")):
    n = R * C
    cases = []
    layouts_b = {
        "contiguous": ([R, C, C, 1, C, 1, 0, 0], n, n),
        "transposed_lhs": ([R, C, 1, R, C, 1, 0, 0], n, n),
        "rhs_broadcast": ([R, C, C, 1, 0, 1, 0, 0], n, C),
        # both operands viewed from element 1 of their buffers, as every fixture of the reference's test-suite is
        # (crates/maidenx_tensor/tests/utils/mod.rs:30-37): contiguous, but not 16-byte aligned
        "offset1": ([R, C, C, 1, C, 1, 1, 1], n + 1, n + 1),
    }
    layouts_u = {
        "contiguous": ([R, C, C, 1, 0], n),
        "transposed": ([R, C, 1, R, 0], n),
        "broadcast": ([R, C, 0, 1, 0], C),
        "offset1": ([R, C, C, 1, 1], n + 1),
    }
    for dt in dtypes:
        s = ELEM_SIZE[dt]
        for op in ("add", "sub", "mul", "div"):
            for lname, (meta, la, lb) in layouts_b.items():
                cases.append(Case(f"{op}_{dt}/{lname}", op, dt, "binary", meta, n, [la, lb], n, (min(la, n) + min(lb, n) + n) * s))
        for op in ("exp", "relu", "gelu", "neg"):
            for lname, (meta, la) in layouts_u.items():
                cases.append(Case(f"{op}_{dt}/{lname}", op, dt, "unary", meta, n, [la], n, (min(la, n) + n) * s))
    for op in ("add", "mul"):
        for lname, (meta, la, lb) in layouts_b.items():
            cases.append(Case(f"{op}_i32/{lname}", op, "i32", "binary", meta, n, [la, lb], n, (min(la, n) + min(lb, n) + n) * 4))
    return cases


def reduction_cases(R: int = 8192, C: int = 16384, fold=(64, 512, 4096)):
    n = R * C
    cases = []
    for dt in ("f32", "bf16"):
        s = ELEM_SIZE[dt]
        for op in ("sum", "mean", "max"):
            # metadata = [dims | strides | red_len | red_stride | offset]
            cases.append(Case(f"{op}_{dt}/dim0", op, dt, "reduce", [R, C, C, 1, R, C, 0], n, [n], C, (n + C) * s, {"num_red": 1}))
            cases.append(Case(f"{op}_{dt}/dim1", op, dt, "reduce", [R, C, C, 1, C, 1, 0], n, [n], R, (n + R) * s, {"num_red": 1}))
    cases.append(Case("sum_i32/dim0", "sum", "i32", "reduce", [R, C, C, 1, R, C, 0], n, [n], C, (n + C) * 4, {"num_red": 1}))
    cases.append(Case("sum_i32/dim1", "sum", "i32", "reduce", [R, C, C, 1, C, 1, 0], n, [n], R, (n + R) * 4, {"num_red": 1}))
    a, b, c = fold
    nf = a * b * c
    for dt in ("f32", "bf16"):
        s = ELEM_SIZE[dt]
        meta = [a, b, c, b * c, c, 1, 1, 1, c, 0]
        cases.append(Case(f"sum_to_shape_{dt}/{a}x{b}x{c}->1x1x{c}", "sum_to_shape", dt, "sum_to_shape", meta, nf, [nf], c, (nf + c) * s))
    return cases


def conv_cases(N: int = 64, Cin: int = 256, H: int = 56, W: int = 56, k: int = 3, stride: int = 1, pad: int = 1):
    oh = (H + 2 * pad - k) // stride + 1
    ow = (W + 2 * pad - k) // stride + 1
    x = N * Cin * H * W
    col = N * Cin * k * k * oh * ow
    meta = [N, Cin, H, W, k, k, oh, ow, pad, pad, stride, stride]
    cases = []
    for dt in ("bf16", "f32"):
        s = ELEM_SIZE[dt]
        cases.append(Case(f"conv2d_im2col_{dt}", "conv2d_im2col", dt, "im2col", meta, col, [x], col, (x + col) * s))
        cases.append(Case(f"conv2d_col2im_{dt}", "conv2d_col2im", dt, "col2im", meta, col, [col], x, (x + col) * s))
    return cases


def extras_cases(rows: int = 16384, cols: int = 8192, N: int = 64, C: int = 256, H: int = 56, W: int = 56, pad: int = 1):
    """The crate's remaining families at sizes of the same order as the other sweeps: softmax along the last dim of
    [rows, cols] and along the first dim of [cols / 8, 4 * rows] (a column softmax), the three paddings of an [N, C, H, W]
    image batch by `pad` on each side of H and W, and the backward of the constant padding."""
    cases = []
    n = rows * cols
    for dt in ("f32", "bf16"):
        s = ELEM_SIZE[dt]
        cases.append(Case(f"softmax_{dt}/last_dim", "softmax", dt, "softmax", [rows, cols, cols, 1, 0], n, [n], n, 2 * n * s, {"dim": 1}))
    r2, c2 = cols // 8, rows * 4   # 268 MB at the default size: larger than L2, like every other case
    cases.append(Case("softmax_f32/first_dim", "softmax", "f32", "softmax", [r2, c2, c2, 1, 0], r2 * c2, [r2 * c2], r2 * c2, 2 * r2 * c2 * 4, {"dim": 0}))
    in_dims = [N, C, H, W]
    out_dims = [N, C, H + 2 * pad, W + 2 * pad]
    n_in, n_out = N * C * H * W, N * C * (H + 2 * pad) * (W + 2 * pad)
    meta = in_dims + [C * H * W, H * W, W, 1] + [0] + out_dims + [0, 0, 0, 0, pad, pad, pad, pad]
    for dt in ("f32", "bf16"):
        s = ELEM_SIZE[dt]
        for mode in ("constant", "reflection", "replication"):
            cases.append(Case(f"pad_with_{mode}_{dt}", f"pad_with_{mode}", dt, "pad", meta, n_in, [n_in], n_out, (n_in + n_out) * s,
                              {"n_out": n_out, "constant": mode == "constant"}))
        # the cropped copy reads only the n_in interior elements of grad_out
        cases.append(Case(f"pad_with_constant_backward_{dt}", "pad_with_constant_backward", dt, "pad_backward", meta, n_in, [n_out], n_in,
                          2 * n_in * s, {"n_out": n_out}))
    # fold (the backward of unfold) of a dense [rows, windows, 4] gradient with step 1: every output sums up to 4 windows
    fr, fw, fs = rows, cols // 8 - 3, 4
    f_in, f_out = fr * fw * fs, fr * (fw - 1 + fs)
    cases.append(Case("fold_f32/windows_of_4", "fold", "f32", "fold", [fr, fw, fs, fw * fs, fs, 1, 1, 2, fw - 1 + fs, 1, fs, 0], f_in, [f_in], f_out,
                      (f_in + f_out) * 4, {"rows": fr, "windows": fw, "size": fs}))
    return cases
