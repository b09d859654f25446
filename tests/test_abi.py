"""The C-ABI library: loads, exports every symbol the header declares, matches the header's struct
layout, and fails loudly (never silently falls back) without a GPU."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "trinity_b200.h")


@pytest.fixture(scope="module")
def lib():
    from trinity_b200 import build
    build.build()
    from trinity_b200 import _lib
    return _lib.load()


def header_functions():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    return sorted(set(re.findall(r"\b(tb200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from trinity_b200 import _lib
    declared = header_functions()
    assert len(declared) >= 12
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SYMBOLS, f"{name} has no ctypes signature"
    assert sorted(_lib.SYMBOLS) == declared


def test_struct_layout_matches_header(tmp_path):
    from trinity_b200 import _lib
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "trinity_b200.h"\nint main(){printf("%zu %zu %zu %zu %zu %zu %zu %zu\\n",'
                   'sizeof(tb200_gemm_args),sizeof(tb200_attn_args),sizeof(tb200_ffn_args),'
                   'offsetof(tb200_attn_args,workspace),offsetof(tb200_ffn_args,w_down),offsetof(tb200_gemm_args,split_k),'
                   'sizeof(tb200_kv_compact_args),offsetof(tb200_kv_compact_args,new_len));}')
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    got = [int(v) for v in subprocess.check_output([str(exe)]).split()]
    want = [C.sizeof(_lib.GemmArgs), C.sizeof(_lib.AttnArgs), C.sizeof(_lib.FfnArgs),
            _lib.AttnArgs.workspace.offset, _lib.FfnArgs.w_down.offset, _lib.GemmArgs.split_k.offset,
            C.sizeof(_lib.KvCompactArgs), _lib.KvCompactArgs.new_len.offset]
    assert got == want


def test_strerror_and_version(lib):
    assert lib.tb200_version() >= 1000
    assert lib.tb200_strerror(0) == b"ok"
    for code in (-1, -2, -3, -4, -5):
        assert lib.tb200_strerror(code) not in (b"ok", b"unknown status")


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_calls_fail_loudly_without_a_gpu(lib):
    from trinity_b200 import _lib
    assert lib.tb200_rmsnorm(None, None, None, None, 4, 64, 0.0, _lib.BF16, None) != 0
    args = _lib.GemmArgs(dtype=_lib.BF16, m=16, n=64, k=64)
    assert lib.tb200_gemm(C.byref(args), None) != 0
    a = _lib.AttnArgs(dtype=_lib.BF16)
    assert lib.tb200_attn_forward(C.byref(a), None) != 0
    f = _lib.FfnArgs(dtype=_lib.BF16)
    assert lib.tb200_ffn_forward(C.byref(f), None) != 0
    e = _lib.KvCompactArgs(dtype=_lib.BF16, rows=1, head_dim=128, kv_len=8, src_cache_len=8, dst_cache_len=8, n_idx=2)
    assert lib.tb200_kv_compact_max_keep(C.byref(e)) == 2      # pure host arithmetic: answers without a device
    assert lib.tb200_kv_compact(C.byref(e), None) != 0


def test_ops_reject_cpu_tensors(lib):
    from trinity_b200 import ops
    with pytest.raises(ValueError, match="CUDA tensors"):
        ops.rmsnorm(torch.zeros(4, 64, dtype=torch.bfloat16))


def test_missing_library_is_an_import_error(monkeypatch, tmp_path):
    from trinity_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "trinity_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, f"{f} mentions the oracle"
