"""CPU oracle for the fused transformer blocks -- TEST INFRASTRUCTURE, NOT PRODUCT.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this module; the shipped path (``trinity_b200``) never does.

fp32 PyTorch restatement of the eager reference classes of youngchan2/Trinity:

* attention: ``baseline/ref_rms.py`` -- ``Vanilla.forward`` :44-82,
  ``PreNorm.forward`` :100-126, ``KeyFormer.forward`` :146-171,
  ``QKNorm.forward`` :237-265, ``RoCo.forward`` :333-357 and their ``Norm*``
  forms (:191-219, :283-314, :376-403);
* the per-key reductions that the eager classes compute and drop
  (``perturb_out`` :166, ``weights_sum`` / ``weights_sqr_sum`` :351-352) are
  summed over queries as the emitted kernels do
  (``evaluation/keyformer/keyformer_falcon_benchmark4358.py:134-141``,
  ``evaluation/roco/roco_falcon_benchmark1620.py:131-136``);
* FFN: ``baseline/ffn_ref.py`` -- ``SimpleFFN.forward`` :24-52 and the Falcon
  tail of ``TRT_Falcon_Ffn...TensorOpsModel.forward`` :114-121.

The reference is MHA, non-causal, unscaled, weight-free and eps-free.  Every
extension (GQA/MQA, causal mask, softmax scale, norm weight + eps, tau, a batch
dimension, column mean/variance, top-k, plain SwiGLU / GELU MLP) is a keyword
whose default is the reference's behaviour, so that at the default parameter
point the functions below reproduce the reference classes (checked against the
classes themselves in ``tests/golden/make_golden.py`` and against the committed
golden vectors in ``tests/test_oracle.py``).

Parity status: pinned at the reference parameter point by golden vectors
generated from the reference classes.  UNPINNED (nothing in the reference
computes them): GELU MLP, top-k indices, causal masking, softmax scale,
GQA/MQA, norm weight/eps, tau != 1.5, column variance, KV-cache eviction
(``kv_compact``: the reference stops at the per-key scores).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

F32 = torch.float32


def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor] = None, eps: float = 0.0) -> torch.Tensor:
    """``x * rsqrt(mean(x^2, -1) [+ eps]) [* weight]`` (``baseline/ref_rms.py:101-102``)."""
    x = x.to(F32)
    variance = x.pow(2).mean(-1, keepdim=True)
    y = x * torch.rsqrt(variance + eps)
    if weight is not None:
        y = y * weight.to(F32)
    return y


def stable_topk(scores: torch.Tensor, k: int) -> torch.Tensor:
    """First ``k`` indices of a stable descending sort along the last axis (ties -> lower index)."""
    order = torch.sort(scores, dim=-1, descending=True, stable=True).indices
    return order[..., :k].to(torch.int32)


def kv_compact(k: torch.Tensor, v: torch.Tensor, idx: torch.Tensor, kv_len: int, keep_recent: int = 0):
    """Eviction step after the per-key scores: per cache row keep the positions ``idx`` names (entries outside
    ``[0, kv_len)`` ignored, duplicates once) and the last ``keep_recent`` ones, packed in ascending position order.

    ``k, v``: ``(..., L, D)``; ``idx``: integer ``(..., n_idx)``.  Returns ``(k_out, v_out, kept_pos, new_len)`` with
    ``k_out, v_out`` ``(..., max_keep, D)`` zero beyond each row's count, ``kept_pos`` ``(..., max_keep)`` padded
    with -1, ``max_keep = min(kv_len, n_idx + keep_recent)``.  Plain loops over rows: parity unpinned (the reference
    defines the layout, ``convert_eval_rms.py:82-83``, and the scores, never the eviction)."""
    lead = k.shape[:-2]
    L, D = k.shape[-2], k.shape[-1]
    n_idx = idx.shape[-1]
    max_keep = min(kv_len, n_idx + keep_recent)
    k2, v2 = k.reshape(-1, L, D), v.reshape(-1, L, D)
    rows = k2.shape[0]
    i2 = idx.reshape(rows, n_idx).to(torch.int64)
    k_out = torch.zeros(rows, max_keep, D, dtype=k.dtype)
    v_out = torch.zeros(rows, max_keep, D, dtype=v.dtype)
    kept = torch.full((rows, max_keep), -1, dtype=torch.int32)
    new_len = torch.zeros(rows, dtype=torch.int32)
    for r in range(rows):
        keep = torch.zeros(kv_len, dtype=torch.bool)
        ok = i2[r][(i2[r] >= 0) & (i2[r] < kv_len)]
        keep[ok] = True
        if keep_recent > 0:
            keep[max(kv_len - keep_recent, 0):] = True
        pos = torch.nonzero(keep).flatten()
        n = pos.numel()
        k_out[r, :n] = k2[r, pos]
        v_out[r, :n] = v2[r, pos]
        kept[r, :n] = pos.to(torch.int32)
        new_len[r] = n
    return (k_out.reshape(*lead, max_keep, D), v_out.reshape(*lead, max_keep, D), kept.reshape(*lead, max_keep),
            new_len.reshape(*lead) if lead else new_len.reshape(()))


def attention_block(
    x: torch.Tensor,
    wq: torch.Tensor,
    wk: torch.Tensor,
    wv: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    past: int,
    head_dim: int,
    prenorm: bool = False,
    norm_weight: Optional[torch.Tensor] = None,
    norm_eps: float = 0.0,
    qknorm: bool = False,
    q_norm_weight: Optional[torch.Tensor] = None,
    k_norm_weight: Optional[torch.Tensor] = None,
    qk_eps: float = 0.0,
    causal: bool = False,
    sm_scale: float = 1.0,
    noise: Optional[torch.Tensor] = None,
    tau: float = 1.5,
    roco: bool = False,
    topk: int = 0,
) -> Dict[str, torch.Tensor]:
    """One fused attention block in fp32.

    Shapes (a leading batch axis ``B`` is optional everywhere; the reference has none):
      x (B,S,N); wq (N,Hq*D); wk, wv (N,Hkv*D); k_cache, v_cache (B,Hkv,>=past+S,D);
      noise (B,Hq,S,past+S).
    Returns a dict with ``O2`` (B,S,Hq*D), ``K_new`` / ``V_new`` (B,Hkv,S,D: the rows
    the block appends at ``[past, past+S)``), ``lse`` (B,Hq,S, natural log) and, when
    asked, ``C_out`` (KeyFormer), ``C_out1`` / ``C_out2`` / ``col_mean`` / ``col_var``
    (RoCo) and ``topk_idx``.

    Op order follows ``baseline/ref_rms.py``: [norm] -> project -> split heads ->
    [q/k norm] -> cat cache -> scores -> softmax -> reductions -> PV -> merge heads.
    """
    batched = x.dim() == 3
    if not batched:
        x = x[None]
        k_cache = k_cache[None]
        v_cache = v_cache[None]
        if noise is not None:
            noise = noise[None]
    B, S, N = x.shape
    D = head_dim
    Hq = wq.shape[1] // D
    Hkv = wk.shape[1] // D
    assert Hq % Hkv == 0
    group = Hq // Hkv
    L = past + S

    x = x.to(F32)
    wq, wk, wv = wq.to(F32), wk.to(F32), wv.to(F32)
    h = rmsnorm(x, norm_weight, norm_eps) if prenorm else x          # ref_rms.py:101-102

    out = {
        "O2": torch.empty(B, S, Hq * D, dtype=F32),
        "K_new": torch.empty(B, Hkv, S, D, dtype=F32),
        "V_new": torch.empty(B, Hkv, S, D, dtype=F32),
        "lse": torch.empty(B, Hq, S, dtype=F32),
    }
    if noise is not None:
        out["C_out"] = torch.empty(B, Hq, L, dtype=F32)
    if roco:
        out["C_out1"] = torch.empty(B, Hq, L, dtype=F32)
        out["C_out2"] = torch.empty(B, Hq, L, dtype=F32)

    if causal:
        qi = torch.arange(S)[:, None]
        kj = torch.arange(L)[None, :]
        visible = kj <= (past + qi)                                   # query i sees keys <= past+i
    for b in range(B):
        q = (h[b] @ wq).view(S, Hq, D).transpose(0, 1)                # ref_rms.py:46-61
        k = (h[b] @ wk).view(S, Hkv, D).transpose(0, 1)
        v = (h[b] @ wv).view(S, Hkv, D).transpose(0, 1)
        if qknorm:                                                    # ref_rms.py:250-253
            q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + qk_eps)
            k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + qk_eps)
            if q_norm_weight is not None:
                q = q * q_norm_weight.to(F32)
            if k_norm_weight is not None:
                k = k * k_norm_weight.to(F32)
        out["K_new"][b] = k
        out["V_new"][b] = v
        kc = torch.cat([k_cache[b, :, :past, :].to(F32), k], dim=1)   # ref_rms.py:71-72
        vc = torch.cat([v_cache[b, :, :past, :].to(F32), v], dim=1)
        o = torch.empty(Hq, S, D, dtype=F32)
        for hq in range(Hq):
            hk = hq // group
            scores = (q[hq] @ kc[hk].transpose(0, 1)) * sm_scale       # ref_rms.py:76
            if causal:
                scores = scores.masked_fill(~visible, float("-inf"))
            weights = torch.softmax(scores, dim=-1)                    # ref_rms.py:77
            out["lse"][b, hq] = torch.logsumexp(scores, dim=-1)
            if noise is not None:                                      # ref_rms.py:164-166
                perturb = (scores + noise[b, hq].to(F32)) / tau
                perturb_out = torch.softmax(perturb, dim=-1)
                out["C_out"][b, hq] = perturb_out.sum(dim=0)
            if roco:                                                   # ref_rms.py:351-352
                out["C_out1"][b, hq] = weights.sum(dim=0)
                out["C_out2"][b, hq] = weights.pow(2).sum(dim=0)
            o[hq] = weights @ vc[hk]                                   # ref_rms.py:79
        out["O2"][b] = o.transpose(0, 1).contiguous().view(S, Hq * D)  # ref_rms.py:80

    if roco:
        # number of queries that can see key j: all S without a mask; S - max(0, j - past) with it
        if causal:
            n_vis = (S - torch.clamp(torch.arange(L) - past, min=0)).to(F32)
        else:
            n_vis = torch.full((L,), float(S))
        out["col_mean"] = out["C_out1"] / n_vis
        out["col_var"] = out["C_out2"] / n_vis - out["col_mean"].pow(2)
    if topk:
        key = out["C_out"] if noise is not None else out["C_out1"]
        out["topk_idx"] = stable_topk(key, topk)
    if not batched:
        out = {name: t[0] for name, t in out.items()}
    return out


def ffn_block(
    x_in: torch.Tensor,
    w_gate: torch.Tensor,
    w_up: Optional[torch.Tensor],
    w_down: torch.Tensor,
    *,
    act: str = "swiglu",
    wo: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    norm: bool = False,
    norm_weight: Optional[torch.Tensor] = None,
    norm_eps: float = 0.0,
    falcon_tail: bool = False,
    tail_divisor: Optional[int] = None,
) -> Dict[str, torch.Tensor]:
    """FFN block in fp32 (``baseline/ffn_ref.py:24-52``; Falcon tail :114-121).

    With ``wo``/``residual``/``norm`` this is the reference block:
      ``a = x_in @ wo + residual`` (``x_in`` is ``O2``); ``h = a / sqrt(sum(a^2)/N)``;
      ``FF2 = (silu(h @ w_gate) * (h @ w_up)) @ w_down`` with gate = ``WFF1b``, up = ``WFF1a``.
    Without them it is the plain MLP on ``x_in``.  ``act='gelu'`` is the exact-erf GELU MLP
    ``gelu(h @ w_gate) @ w_down`` (``w_up`` unused); the reference has no GELU, so this
    choice is unpinned.  ``falcon_tail`` adds ``O_FF = FF2 + h`` and
    ``O_FF_norm = O_FF / sqrt(sum(O_FF^2) / tail_divisor)`` (divisor 4544 in the reference).
    """
    a = x_in.to(F32)
    if wo is not None:
        a = a @ wo.to(F32)                                            # ffn_ref.py:26
    if residual is not None:
        a = a + residual.to(F32)                                      # ffn_ref.py:29
    out = {"attn_O2": a}
    if norm:
        n = a.shape[-1]
        ss = torch.sum(a ** 2, dim=-1, keepdim=True)                  # ffn_ref.py:32
        h = a / torch.sqrt(ss / n + norm_eps)                         # ffn_ref.py:35
        if norm_weight is not None:
            h = h * norm_weight.to(F32)
    else:
        h = a
    g = h @ w_gate.to(F32)                                            # ffn_ref.py:41 (FF1b)
    if act == "swiglu":
        u = h @ w_up.to(F32)                                          # ffn_ref.py:38 (FF1a)
        ff1 = u * (g * torch.sigmoid(g))                              # ffn_ref.py:44-47
    elif act == "gelu":
        ff1 = torch.nn.functional.gelu(g)
    else:
        raise ValueError(act)
    ff2 = ff1 @ w_down.to(F32)                                        # ffn_ref.py:50
    out["FF1"] = ff1
    out["FF2"] = ff2
    if falcon_tail:
        o_ff = ff2 + h                                                # ffn_ref.py:115
        div = tail_divisor if tail_divisor is not None else o_ff.shape[-1]
        o_ff1 = torch.sum(o_ff ** 2, dim=-1, keepdim=True)            # ffn_ref.py:118
        out["O_FF"] = o_ff
        out["O_FF_norm"] = o_ff / torch.sqrt(o_ff1 / div)             # ffn_ref.py:121
    return out


# ----------------------------------------------------------------------------------------------
# Seeded synthetic inputs.  The reference uses no dataset; these are its own distributions
# (``convert_eval_rms.py:127-176``, ``convert_ffn_llama.py:86-99``) and the benchmark configs'.
# ----------------------------------------------------------------------------------------------

class _Rng:
    """Seeded N(0,1) / U(0,1) tensors from numpy's PCG64 stream: identical on every host CPU (torch's CPU
    ``randn`` takes different vector paths on different machines, which would unpin the golden vectors)."""

    def __init__(self, seed: int):
        self.g = np.random.default_rng(seed)

    def randn(self, *shape) -> torch.Tensor:
        return torch.from_numpy(self.g.standard_normal(shape, dtype=np.float32))

    def rand(self, *shape) -> torch.Tensor:
        return torch.from_numpy(self.g.random(shape, dtype=np.float32))


def ref_attention_inputs(M: int, N: int, D: int, P: int, seed: int = 42, std: float = 0.01):
    """Inputs of the reference parity driver (MHA, ``randn * 0.01``, unscaled ``randn`` noise)."""
    H = N // D
    rn = _Rng(seed).randn
    return {
        "X": rn(M, N) * std, "WQ": rn(N, N) * std, "WK": rn(N, N) * std, "WV": rn(N, N) * std,
        "K_cache": rn(H, P + M, D) * std, "V_cache": rn(H, P + M, D) * std,
        "noise": rn(H, M, P + M),
    }


def ref_ffn_inputs(M: int, N: int, P: int, seed: int = 42, std: float = 0.001):
    """Inputs of the reference FFN driver (``randn.clamp(-1,1) * 0.001``)."""
    r = _Rng(seed)
    rn = lambda *s: r.randn(*s).clamp(-1, 1) * std
    return {"O2": rn(M, N), "X": rn(M, N), "WO": rn(N, N), "WFF1a": rn(N, P), "WFF1b": rn(N, P), "WFF2": rn(P, N)}


def gumbel_noise(shape, generator) -> torch.Tensor:
    """Gumbel(0,1) = -log(-log(U)), U clamped to [1e-9, 1-1e-9]; ``generator`` is a torch.Generator or an _Rng."""
    if isinstance(generator, _Rng):
        u = generator.rand(*shape)
    else:
        u = torch.rand(*shape, generator=generator, dtype=F32)
    u = u.clamp_(1e-9, 1 - 1e-9)
    return -torch.log(-torch.log(u))


def bench_attention_inputs(B: int, S: int, N: int, Hq: int, Hkv: int, D: int, seed: int = 0,
                           norm_weights: bool = False, noise: bool = False):
    """x ~ N(0,1); projection weights ~ N(0,0.02); norm weights 1 + N(0,0.02); Gumbel noise."""
    g = _Rng(seed)
    rn = g.randn
    t = {"X": rn(B, S, N), "WQ": rn(N, Hq * D) * 0.02, "WK": rn(N, Hkv * D) * 0.02, "WV": rn(N, Hkv * D) * 0.02}
    if norm_weights:
        t["norm_weight"] = 1 + rn(N) * 0.02
        t["q_norm_weight"] = 1 + rn(D) * 0.02
        t["k_norm_weight"] = 1 + rn(D) * 0.02
    if noise:
        t["noise"] = gumbel_noise((B, Hq, S, S), g)
    return t


def bench_ffn_inputs(M: int, N: int, P: int, seed: int = 0, gated: bool = True):
    rn = _Rng(seed).randn
    t = {"X": rn(M, N), "W_gate": rn(N, P) * 0.02}
    if gated:
        t["W_up"] = rn(N, P) * 0.02
    t["W_down"] = rn(P, N) * 0.02
    return t


LOG2E = math.log2(math.e)
