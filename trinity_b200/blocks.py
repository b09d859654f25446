"""What a generated module's ``forward`` calls: map the reference's named tensors onto the C ABI.

Shapes follow the reference drivers (``convert_eval_rms.py:61-107``, ``convert_ffn_llama.py:34-53``):
``X (M,N)``, ``WQ/WK/WV (N,H*D)``, ``K_cache/V_cache (H,P+M,D)``, ``O2 (M,N)``, ``noise (H,M,P+M)``,
``C_out* (H,P+M)``; FFN: ``O2,X (M,N)``, ``WO (N,N)``, ``WFF1a/WFF1b (N,P)``, ``WFF2 (P,N)``.  A leading
batch axis on ``X`` (and the matching caches) is accepted.  Scratch tensors a candidate lists
(``O``, ``C_exp``, ``C_sum``, ...) are accepted and left untouched: the kernels keep their own workspace.
The keyword-only tensors of a generated module (``norm_weight``, ``q_norm_weight``, ``k_norm_weight``,
``topk_idx``) arrive here under those names and are ``None`` when the caller did not pass them.
"""
from __future__ import annotations

from typing import Dict

import torch

from . import _lib as L
from . import ops

_ATTN_FLAGS = {
    "vanilla": 0, "prenorm": L.ATTN_PRENORM, "qknorm": L.ATTN_QKNORM, "qknorm_prenorm": L.ATTN_QKNORM | L.ATTN_PRENORM,
    "keyformer": L.ATTN_KEYFORMER, "keyformer_prenorm": L.ATTN_KEYFORMER | L.ATTN_PRENORM,
    "roco": L.ATTN_ROCO, "roco_prenorm": L.ATTN_ROCO | L.ATTN_PRENORM,
}


def run(kind: str, constants: Dict, t: Dict[str, torch.Tensor]) -> None:
    if kind in _ATTN_FLAGS:
        _run_attention(kind, constants, t)
    elif kind in ("ffn_llama", "ffn_falcon"):
        _run_ffn(kind, constants, t)
    else:
        raise ValueError(f"unknown block family {kind!r}")


def _run_attention(kind: str, c: Dict, t: Dict[str, torch.Tensor]) -> None:
    flags = _ATTN_FLAGS[kind]
    if c.get("CAUSAL"):
        flags |= L.ATTN_CAUSAL
    if c.get("ROCO_VARIANCE") and flags & L.ATTN_ROCO:
        flags |= L.ATTN_ROCO_VARIANCE
    D = int(c["D"])
    past = int(c["P"])
    topk = int(c.get("TOPK", 0))
    idx = t.get("topk_idx")
    if topk and idx is None:
        raise ValueError("TOPK is set in the module constants but no 'topk_idx' tensor was passed")
    if idx is not None and not topk:
        topk = int(idx.shape[-1])
    ops.attn_forward(
        t["X"], t["WQ"], t["WK"], t["WV"], t["K_cache"], t["V_cache"], t["O2"], past=past, head_dim=D, flags=flags,
        sm_scale=float(c.get("SM_SCALE", 1.0)), norm_weight=t.get("norm_weight"), norm_eps=float(c.get("NORM_EPS", 0.0)),
        q_norm_weight=t.get("q_norm_weight"), k_norm_weight=t.get("k_norm_weight"), qk_eps=float(c.get("QK_EPS", 0.0)),
        noise=t.get("noise") if flags & L.ATTN_KEYFORMER else None, tau=float(c.get("TAU", 1.5)),
        c_out=t.get("C_out") if flags & L.ATTN_KEYFORMER else None,
        c_out1=t.get("C_out1") if flags & L.ATTN_ROCO else None, c_out2=t.get("C_out2") if flags & L.ATTN_ROCO else None,
        topk=topk, topk_idx=idx)


def _run_ffn(kind: str, c: Dict, t: Dict[str, torch.Tensor]) -> None:
    tail = kind == "ffn_falcon"
    ops.ffn_forward(
        t["X"], t["WFF1b"], t["WFF1a"], t["WFF2"], t["FF2"] if "FF2" in t else _scratch_like(t["X"], "FF2"),
        act=L.FFN_SWIGLU, flags=L.FFN_NORM | (L.FFN_FALCON_TAIL if tail else 0), o2=t["O2"], wo=t["WO"],
        norm_weight=t.get("norm_weight"), norm_eps=float(c.get("NORM_EPS", 0.0)), tail_divisor=int(c.get("N", 0)) if tail else 0,
        attn_o2=t.get("attn_O2"), ff1=t.get("FF1"), o_ff_norm=t.get("O_FF_norm") if tail else None)


def _scratch_like(x: torch.Tensor, tag: str) -> torch.Tensor:
    ws = ops.Workspace.get(x.device, x.numel() * x.element_size(), "blocks." + tag)
    return ws[: x.numel() * x.element_size()].view(x.dtype).view(x.shape)
