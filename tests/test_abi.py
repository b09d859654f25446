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
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "trinity_b200.h"\nint main(){printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n",'
                   'sizeof(tb200_peer_gemm_args),offsetof(tb200_peer_gemm_args,epoch),'
                   'sizeof(tb200_gemm_args),sizeof(tb200_attn_args),sizeof(tb200_ffn_args),'
                   'offsetof(tb200_attn_args,workspace),offsetof(tb200_ffn_args,w_down),offsetof(tb200_gemm_args,split_k),'
                   'sizeof(tb200_kv_compact_args),offsetof(tb200_kv_compact_args,new_len));}')
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    got = [int(v) for v in subprocess.check_output([str(exe)]).split()]
    want = [C.sizeof(_lib.PeerGemmArgs), _lib.PeerGemmArgs.epoch.offset, C.sizeof(_lib.GemmArgs), C.sizeof(_lib.AttnArgs), C.sizeof(_lib.FfnArgs),
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


# ---------------------------------------------------------------- host-side argument checks, no device, no launch
def _gemm_args(**kw):
    from trinity_b200 import _lib
    base = dict(dtype=_lib.BF16, act=0, m=64, n=256, k=512, a=0x10000, b=0x20000, c=0x30000)
    base.update(kw)
    return _lib.GemmArgs(**base)


def test_gemm_check_refuses_misaligned_pointers_on_the_host(lib):
    """Every tensor pointer is touched with 16-byte accesses on some path (TMA, uint4 loads and stores of the K-slice
    finish), so a misaligned one is refused by the host check -- with fake addresses, nothing is launched."""
    assert lib.tb200_gemm_check(C.byref(_gemm_args())) == 0
    for field in ("a", "b", "c"):
        assert lib.tb200_gemm_check(C.byref(_gemm_args(**{field: 0x10008}))) == -1, field
    assert lib.tb200_gemm_check(C.byref(_gemm_args(b2=0x40004))) == -1
    assert lib.tb200_gemm_check(C.byref(_gemm_args(residual=0x40002))) == -1
    assert lib.tb200_gemm_check(C.byref(_gemm_args(row_scale=0x40002))) == -1
    assert lib.tb200_gemm_check(C.byref(_gemm_args(row_scale=0x40004))) == 0       # fp32: 4-byte alignment is enough
    assert lib.tb200_gemm_check(C.byref(_gemm_args(n=250))) == -1                   # n % 8
    assert lib.tb200_gemm_check(C.byref(_gemm_args(c=None))) == -1
    assert lib.tb200_gemm_check(None) == -1


def _attn_args(**kw):
    from trinity_b200 import _lib
    base = dict(dtype=_lib.BF16, flags=0, batch=1, seq=16, hidden=512, n_q_heads=4, n_kv_heads=2, head_dim=128, past=0,
                cache_len=16, sm_scale=1.0, tau=1.0, x=0x1000, wq=0x2000, wk=0x3000, wv=0x4000, k_cache=0x5000, v_cache=0x6000,
                o2=0x7000, aux_dtype=_lib.F32)
    base.update(kw)
    return _lib.AttnArgs(**base)


def test_attn_check_refuses_before_any_launch(lib):
    from trinity_b200 import _lib
    assert lib.tb200_attn_check(C.byref(_attn_args())) == 0
    for field in ("x", "wq", "wk", "wv", "k_cache", "v_cache", "o2"):
        assert lib.tb200_attn_check(C.byref(_attn_args(**{field: 0x1008}))) == -1, field
    assert lib.tb200_attn_check(C.byref(_attn_args(flags=_lib.ATTN_PRENORM, norm_weight=0x8002))) == -1
    # requests without a kernel are refused up front, not after the projection has already written the caches
    both = _attn_args(flags=_lib.ATTN_KEYFORMER | _lib.ATTN_ROCO, noise=0x8000, c_out=0x9000, c_out1=0xa000, c_out2=0xb000)
    assert lib.tb200_attn_check(C.byref(both)) == -2
    long_topk = _attn_args(flags=_lib.ATTN_ROCO, seq=128, past=16384, cache_len=16512, c_out1=0xa000, c_out2=0xb000, topk=8, topk_idx=0xc000)
    assert lib.tb200_attn_check(C.byref(long_topk)) == -2
    assert lib.tb200_attn_check(C.byref(_attn_args(flags=_lib.ATTN_ROCO, c_out1=0xa002, c_out2=0xb000))) == -1
    assert lib.tb200_attn_check(C.byref(_attn_args(flags=_lib.ATTN_ROCO_VARIANCE))) == -1   # variance without ROCO
    assert lib.tb200_attn_check(C.byref(_attn_args(sm_scale=0.0))) == -1


def test_ffn_check_refuses_misaligned_pointers(lib):
    from trinity_b200 import _lib
    base = dict(dtype=_lib.BF16, act=_lib.FFN_SWIGLU, flags=0, tokens=16, hidden=512, inner=1536, x=0x1000, w_gate=0x2000,
                w_up=0x3000, w_down=0x4000, ff2=0x5000)
    assert lib.tb200_ffn_check(C.byref(_lib.FfnArgs(**base))) == 0
    for field in ("x", "w_gate", "w_up", "w_down", "ff2"):
        bad = dict(base)
        bad[field] = 0x1004
        assert lib.tb200_ffn_check(C.byref(_lib.FfnArgs(**bad))) == -1, field
    assert lib.tb200_ffn_check(C.byref(_lib.FfnArgs(**dict(base, ff1=0x6008)))) == -1
    assert lib.tb200_ffn_check(C.byref(_lib.FfnArgs(**dict(base, w_up=None)))) == -1


def test_wait_limit_is_a_host_setting(lib):
    assert lib.tb200_get_wait_limit_cycles() == 4_000_000_000
    assert lib.tb200_set_wait_limit_cycles(10) == -1                # refuses a limit no kernel could meet
    assert lib.tb200_set_wait_limit_cycles(1_000_000) == 0
    assert lib.tb200_get_wait_limit_cycles() == 1_000_000
    assert lib.tb200_set_wait_limit_cycles(4_000_000_000) == 0


def test_chained_launch_is_a_host_setting(lib):
    """On by default; the setter returns what was set before (no device involved)."""
    assert lib.tb200_set_chained_launch(0) == 1
    assert lib.tb200_set_chained_launch(0) == 0
    assert lib.tb200_set_chained_launch(1) == 0
    assert lib.tb200_set_chained_launch(7) == 1                     # any non-zero value means on
    assert lib.tb200_set_chained_launch(1) == 1
