"""CPU-side checks: the C-ABI library loads without a GPU and exports every symbol the public
header declares; host-side helpers agree with the oracle."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    src = open(os.path.join(ROOT, "include", "rew_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(rewb200_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    from rew_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_functions()
    assert len(names) >= 40
    for n in names:
        assert hasattr(lib, n), "declared in include/rew_b200.h but not exported: " + n
    # and the Python binding names exactly the declared set
    assert sorted(_lib.SIGNATURES) == names


def test_config_struct_matches_header_layout():
    from rew_b200 import _lib
    # 8 int32, double (8-aligned at offset 32), float, 12 int32
    assert _lib.Config.theta.offset == 32
    assert _lib.Config.eps.offset == 40
    assert ctypes.sizeof(_lib.Config) == 96


def test_no_gpu_means_a_loud_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from rew_b200 import _lib
    arr = (ctypes.c_int32 * 1)(0)
    assert _lib.lib().rewb200_init(arr, 1) != 0
    assert b"no CUDA device" in _lib.lib().rewb200_last_error()
    with pytest.raises(_lib.RewB200Error):
        from rew_b200 import api
        api.Tensor.from_host(np.zeros(4, np.float32))


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "rew_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, f


def test_tensor_specs_and_bf16_helpers(orc):
    from rew_b200 import weights as W
    cfg = W.tiny_llama()
    specs = W.tensor_specs(cfg)
    assert len(specs) == 1 + 2 * 18 + 4
    assert sum(int(np.prod(s)) for n, s in specs if len(s) == 2 and "embed" not in n) == 1646592  # matmul params
    l8 = W.llama3_8b()
    assert sum(int(np.prod(s)) for n, s in W.tensor_specs(l8) if len(s) == 2 and "embed" not in n) == 7504658432
    moe = W.deepseek_v2_lite()
    assert len(W.tensor_specs(moe)) == 1 + (12 + 6) + 26 * (12 + 2 + 6 * 66) + 4
    x = np.random.default_rng(0).normal(size=100).astype(np.float32)
    assert np.array_equal(W.bf16_round(x), orc.bf16_round(x))
    assert np.array_equal(W.from_bf16_bits(W.to_bf16_bits(x)), orc.bf16_round(x))


def test_header_is_valid_c_and_struct_layout_matches_the_bindings(tmp_path):
    """gcc (C, not C++) compiles a program that includes the public header and prints the layout of
    rewb200_config; the ctypes mirror and the generated Nim object must have the same fields, order, offsets
    and sizes."""
    import subprocess
    from rew_b200 import _lib
    exe = str(tmp_path / "abi_layout")
    src = os.path.join(ROOT, "tests", "c", "abi_layout.c")
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", src, "-o", exe + ".o"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run(["gcc", exe + ".o", "-o", exe, "-L", os.path.dirname(_lib.LIB_PATH), "-lrew_b200",
                        "-Wl,-rpath," + os.path.dirname(_lib.LIB_PATH)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split("\n")
    rows = [l.split() for l in out if l and not l.startswith("sizeof")]
    size_line = [l.split() for l in out if l.startswith("sizeof")][0]
    assert int(size_line[1]) == ctypes.sizeof(_lib.Config) and int(size_line[2]) == _lib.BF16
    fields = [f[0] for f in _lib.Config._fields_]
    assert [r[0] for r in rows] == fields
    for name, off, sz in rows:
        d = getattr(_lib.Config, name)
        assert (d.offset, d.size) == (int(off), int(sz)), name
    nim = open(os.path.join(ROOT, "nim", "rew_b200_abi.nim")).read()
    body = nim[nim.index("RewbConfig*"):nim.index("proc rewb200_init")]
    nim_fields = re.findall(r"^    (\w+)\*: (\w+)$", body, flags=re.M)
    assert [n for n, _ in nim_fields] == fields
    width = {"int32": 4, "cfloat": 4, "cdouble": 8}
    assert [width[t] for _, t in nim_fields] == [int(r[2]) for r in rows]


def test_generated_nim_declarations_are_up_to_date():
    """nim/rew_b200_abi.nim is generated from the header; a header change without regenerating fails here."""
    import subprocess
    import sys
    r = subprocess.run([sys.executable, os.path.join(ROOT, "nim", "gen_importc.py"), "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    nim = open(os.path.join(ROOT, "nim", "rew_b200_abi.nim")).read()
    assert sorted(re.findall(r"^proc (rewb200_\w+)\*", nim, flags=re.M)) == _declared_functions()
    # the hand-written half of the binding only calls what the generated half declares
    hand = open(os.path.join(ROOT, "nim", "rew_b200.nim")).read()
    for name in set(re.findall(r"\b(rewb200_[a-z0-9_]+)\b", hand)):
        assert name in _declared_functions(), name
