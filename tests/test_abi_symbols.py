"""The drop-in boundary, checked without a GPU: every function the public header declares
is exported by libmaidenx_cuda.so, the op symbol set is the one the reference's dispatch
layer references, and the library loads."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

from maidenx_b200 import _lib, _signatures as sig

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "maidenx_cuda.h"
HEADERS = sorted((ROOT / "include").glob("*.h"))  # the public header and the test-only one


def _declared():
    names = set()
    for h in HEADERS:
        src = subprocess.run(["gcc", "-E", "-P", str(h)], check=True, capture_output=True, text=True).stdout
        names |= set(re.findall(r"\b((?:cuda|mx)_[a-z0-9_]+)\s*\(", src))
    return sorted(names)


def _exported():
    out = subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], check=True, capture_output=True, text=True).stdout
    return {l.split()[-1] for l in out.splitlines() if l.strip()}


def test_header_preprocesses_as_c_with_stdbool(tmp_path):
    t = tmp_path / "t.c"
    t.write_text('#include <stdbool.h>\n#include "maidenx_cuda.h"\nbool still_defined = true;\n')
    subprocess.run(["gcc", "-fsyntax-only", "-I", str(HEADER.parent), str(t)], check=True)


def test_library_is_built():
    assert _lib.LIB_PATH.exists(), "run python -m maidenx_b200.build"


def test_every_declared_symbol_is_exported():
    declared = _declared()
    assert len(declared) > 600
    missing = sorted(set(declared) - _exported())
    assert not missing, f"declared in include/*.h but not exported: {missing[:10]} (+{max(0, len(missing) - 10)})"


def test_op_symbol_set_matches_reference_dispatch():
    """237 binary + 295 unary + 64 reduction (sum, max, min, sum_to_shape, fold x12, mean x4) + 24 matmul
    + 8 conv + 72 padding + 4 softmax = the 704 entry points dispatched by crates/maidenx_core/src/be/ops/*.rs,
    be/nn/conv.rs and be/nn/activation.rs."""
    table = list(sig.op_table())
    fam = {}
    for op, d, f in table:
        fam[f] = fam.get(f, 0) + 1
    assert fam["binary"] + fam["binary_bool"] + fam["binary_inplace"] == 237
    assert fam["unary"] + fam["unary_bool"] + fam["unary_const"] + fam["unary_const_bool"] == 295
    assert fam["reduce"] + fam["sum_to_shape"] == 64
    assert fam["pad"] + fam["pad_const"] == 72
    assert fam["softmax"] == 4
    assert len(table) == 704
    assert fam["matmul"] + fam["matmul_backward"] == 24
    assert fam["conv"] == 8
    exported = _exported()
    declared = set(_declared())
    for op, d, _ in table:
        name = f"cuda_{op}_{d.name}"
        assert name in declared, name
        assert name in exported, name


def test_library_loads_and_binds():
    lib = _lib.load()
    assert isinstance(lib, ctypes.CDLL)
    assert lib.mx_last_error() == 0
    assert _lib.op("add", "f32") is not None
    with pytest.raises(KeyError):
        _lib.op("add", "bool")  # never dispatched by the reference (be/ops/binary.rs:245)
