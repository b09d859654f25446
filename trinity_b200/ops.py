"""Tensor-level wrappers over the C ABI: torch tensors in, raw device pointers across the boundary.

PyTorch is plumbing here (device memory, streams); every operator below runs in libtrinity_b200.so.
All wrappers launch on ``torch.cuda.current_stream()`` and allocate nothing once their workspace has
been cached, so they can be captured in a CUDA graph after one warm-up call.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional

import torch

from . import _lib as L

_DT = {torch.float16: L.F16, torch.bfloat16: L.BF16, torch.float32: L.F32}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("trinity_b200 operators take CUDA tensors (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError("trinity_b200 operators take contiguous tensors")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class Workspace:
    """Scratch buffers the operators hand to the C ABI, one per (device, tag, stream).

    * A buffer only grows, and only outside CUDA-graph capture (the first call sizes it).
    * A buffer that is outgrown is RETIRED, not freed: a CUDA graph captured earlier holds its device address, and
      the caching allocator must not hand that memory to another tensor while the graph can still be replayed.
      ``Workspace.release()`` drops the retired buffers once no such graph is left.
    * Buffers are keyed by the stream the call runs on, so eager calls on two streams never share partial sums; the
      memory is allocated on that stream, so the allocator's stream bookkeeping is right without ``record_stream``.
    * A capture on a stream that has no buffer yet adopts the one a warm-up call sized on another stream (capture
      cannot allocate).  The two streams then share it: do not run that warm-up stream while the graph replays.
    """

    _bufs: Dict[tuple, torch.Tensor] = {}
    _retired: list = []

    @classmethod
    def get(cls, device: torch.device, nbytes: int, tag: str = "default") -> Optional[torch.Tensor]:
        if nbytes == 0:
            return None
        index = device.index if device.index is not None else torch.cuda.current_device()
        key = (index, tag, torch.cuda.current_stream(device).cuda_stream)
        buf = cls._bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            if torch.cuda.is_current_stream_capturing():
                for (i, t, _), other in cls._bufs.items():
                    if i == index and t == tag and other.numel() >= nbytes:
                        if buf is not None:
                            cls._retired.append(buf)
                        cls._bufs[key] = other
                        return other
                raise RuntimeError("workspace must be sized by one call outside CUDA-graph capture first")
            if buf is not None:
                cls._retired.append(buf)
            buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
            cls._bufs[key] = buf
        return buf

    @classmethod
    def release(cls) -> None:
        """Free the buffers that were outgrown.  Call only when no CUDA graph captured before the growth is replayed again."""
        cls._retired.clear()


class FoldedWeights:
    """Projection weights with an RMSNorm weight folded into their rows (``tb200_fold_norm_weight``), kept per set of
    source tensors.  ``(x * r * g) @ W = r * (x @ (diag(g) W))``: with the folded copy the weighted norm in front of a
    projection is a row statistic and a per-row scale in the projection's epilogue, no normalised copy of ``x``.

    A folded copy is made at the first call that sees a (weights, norm weight) combination -- outside CUDA-graph
    capture, like any one-time set-up; under capture an unseen combination runs the unfolded path -- and reused while
    the source tensors are alive and unmodified (their torch version counters are part of the key).  It costs the
    projection's weight bytes once more in HBM; ``FoldedWeights.enabled = False`` turns folding off."""

    enabled = True
    _cache: Dict[tuple, tuple] = {}

    @classmethod
    def get(cls, g: torch.Tensor, *weights: torch.Tensor):
        if not cls.enabled:
            return None
        key = (g.data_ptr(), g._version) + tuple((w.data_ptr(), w._version, tuple(w.shape)) for w in weights)
        hit = cls._cache.get(key)
        if hit is not None:
            return hit[0]
        if torch.cuda.is_current_stream_capturing():
            return None
        lib = L.load()
        folded = []
        for w in weights:
            out = torch.empty_like(w)
            L.check(lib.tb200_fold_norm_weight(_ptr(w), _ptr(g), _ptr(out), w.shape[0], w.shape[1], _dt(w), _stream()), "tb200_fold_norm_weight")
            folded.append(out)
        if len(cls._cache) >= 64:          # a bound, not a policy: drop the oldest entry
            cls._cache.pop(next(iter(cls._cache)))
        cls._cache[key] = (tuple(folded), (g,) + weights)   # the sources are kept alive so that their addresses stay theirs
        return tuple(folded)

    @classmethod
    def clear(cls) -> None:
        cls._cache.clear()


def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor] = None, eps: float = 0.0,
            out: Optional[torch.Tensor] = None, inv_rms: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = L.load()
    cols = x.shape[-1]
    rows = x.numel() // cols
    if out is None:
        out = torch.empty_like(x)
    L.check(lib.tb200_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), _ptr(inv_rms), rows, cols, eps, _dt(x), _stream()), "tb200_rmsnorm")
    return out


def row_inv_rms(x: torch.Tensor, eps: float = 0.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Only the per-row statistic ``rsqrt(mean(x^2) + eps)`` (fp32), for the norm-as-epilogue path."""
    lib = L.load()
    cols = x.shape[-1]
    rows = x.numel() // cols
    if out is None:
        out = torch.empty(rows, dtype=torch.float32, device=x.device)
    L.check(lib.tb200_rmsnorm(_ptr(x), None, None, _ptr(out), rows, cols, eps, _dt(x), _stream()), "tb200_rmsnorm")
    return out


def gemm(a: torch.Tensor, b: torch.Tensor, *, b2: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, act: int = 0, split_k: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = L.load()
    m, k = a.shape
    n = b.shape[1]
    if out is None:
        out = torch.empty(m, n, dtype=a.dtype, device=a.device)
    args = L.GemmArgs(dtype=_dt(a), act=act, m=m, n=n, k=k, a=_ptr(a), b=_ptr(b), b2=_ptr(b2), c=_ptr(out),
                      row_scale=_ptr(row_scale), residual=_ptr(residual), split_k=split_k)
    need = lib.tb200_gemm_workspace_bytes(C.byref(args))
    ws = Workspace.get(a.device, need, "gemm")
    args.workspace, args.workspace_bytes = _ptr(ws), need
    L.check(lib.tb200_gemm(C.byref(args), _stream()), "tb200_gemm")
    return out


def _attn_args(x, wq, wk, wv, k_cache, v_cache, o2, *, past: int, head_dim: int, flags: int = 0,
               sm_scale: float = 1.0, norm_weight=None, norm_eps: float = 0.0, q_norm_weight=None,
               k_norm_weight=None, qk_eps: float = 0.0, noise=None, tau: float = 1.5, c_out=None,
               c_out1=None, c_out2=None, topk: int = 0, topk_idx=None):
    """The argument block of tb200_attn_forward with its workspace attached.  Returns (args, tensors to keep alive)."""
    lib = L.load()
    if x.dim() == 2:
        batch, (seq, hidden) = 1, x.shape
    else:
        batch, seq, hidden = x.shape
    n_q = wq.shape[1] // head_dim
    n_kv = wk.shape[1] // head_dim
    cache_len = k_cache.shape[-2]
    if (flags & L.ATTN_PRENORM) and norm_weight is not None and not (flags & L.ATTN_NORM_FOLDED):
        folded = FoldedWeights.get(norm_weight, wq, wk, wv)
        if folded is not None:
            wq, wk, wv = folded
            flags |= L.ATTN_NORM_FOLDED
    aux = c_out if c_out is not None else c_out1
    args = L.AttnArgs(
        dtype=_dt(x), flags=flags, batch=batch, seq=seq, hidden=hidden, n_q_heads=n_q, n_kv_heads=n_kv,
        head_dim=head_dim, past=past, cache_len=cache_len, sm_scale=sm_scale, norm_eps=norm_eps, qk_eps=qk_eps, tau=tau,
        x=_ptr(x), wq=_ptr(wq), wk=_ptr(wk), wv=_ptr(wv), k_cache=_ptr(k_cache), v_cache=_ptr(v_cache), o2=_ptr(o2),
        norm_weight=_ptr(norm_weight), q_norm_weight=_ptr(q_norm_weight), k_norm_weight=_ptr(k_norm_weight),
        noise=_ptr(noise), c_out=_ptr(c_out), c_out1=_ptr(c_out1), c_out2=_ptr(c_out2),
        aux_dtype=_dt(aux) if aux is not None else L.F32, topk=topk, topk_idx=_ptr(topk_idx))
    need = lib.tb200_attn_workspace_bytes(C.byref(args))
    if need == 0:
        raise L.Tb200Error(-1, "tb200_attn_workspace_bytes")
    ws = Workspace.get(x.device, need, "attn")
    args.workspace, args.workspace_bytes = _ptr(ws), need
    return args, (wq, wk, wv, ws)


def attn_forward(*tensors, timed: bool = False, **kw):
    """The fused attention block: ``attn_forward(x, wq, wk, wv, k_cache, v_cache, o2, past=, head_dim=, flags=, ...)``;
    mutates ``o2``, the cache rows ``[past, past+S)`` and the c_out* tensors.  With ``timed`` the call waits for the
    stream and returns the four stage durations in ms."""
    lib = L.load()
    args, _keep = _attn_args(*tensors, **kw)
    if timed:
        ms = (C.c_float * 4)()
        L.check(lib.tb200_attn_forward_timed(C.byref(args), _stream(), ms), "tb200_attn_forward_timed")
        return list(ms)
    L.check(lib.tb200_attn_forward(C.byref(args), _stream()), "tb200_attn_forward")


def _ffn_args(x, w_gate, w_up, w_down, ff2, *, act: int = L.FFN_SWIGLU, flags: int = 0, o2=None, wo=None,
              norm_weight=None, norm_eps: float = 0.0, tail_divisor: int = 0, attn_o2=None, ff1=None,
              o_ff_norm=None):
    """The argument block of tb200_ffn_forward with its workspace attached.  Returns (args, tensors to keep alive)."""
    lib = L.load()
    hidden = x.shape[-1]
    tokens = x.numel() // hidden
    inner = w_gate.shape[1]
    if (flags & L.FFN_NORM) and norm_weight is not None and not (flags & (L.FFN_NORM_FOLDED | L.FFN_FALCON_TAIL)):
        folded = FoldedWeights.get(norm_weight, *([w_gate] if w_up is None else [w_gate, w_up]))
        if folded is not None:
            w_gate, w_up = folded[0], (folded[1] if w_up is not None else None)
            flags |= L.FFN_NORM_FOLDED
    args = L.FfnArgs(dtype=_dt(x), act=act, flags=flags, tokens=tokens, hidden=hidden, inner=inner, norm_eps=norm_eps,
                     tail_divisor=tail_divisor, x=_ptr(x), o2=_ptr(o2), wo=_ptr(wo), norm_weight=_ptr(norm_weight),
                     w_gate=_ptr(w_gate), w_up=_ptr(w_up), w_down=_ptr(w_down), ff2=_ptr(ff2), attn_o2=_ptr(attn_o2),
                     ff1=_ptr(ff1), o_ff_norm=_ptr(o_ff_norm))
    need = lib.tb200_ffn_workspace_bytes(C.byref(args))
    ws = Workspace.get(x.device, need, "ffn")
    args.workspace, args.workspace_bytes = _ptr(ws), need
    return args, (w_gate, w_up, ws)


def ffn_forward(*tensors, **kw) -> None:
    """The fused FFN block: ``ffn_forward(x, w_gate, w_up, w_down, ff2, act=, flags=, o2=, wo=, ...)``; mutates ``ff2``
    (and ``attn_o2`` / ``ff1`` / ``o_ff_norm`` when given)."""
    args, _keep = _ffn_args(*tensors, **kw)
    L.check(L.load().tb200_ffn_forward(C.byref(args), _stream()), "tb200_ffn_forward")


def layer_forward(attn: dict, ffn: dict) -> None:
    """The attention block and the FFN block that consumes its ``o2`` as ONE call (tb200_layer_forward): one launch chain,
    in which the FFN's first projection starts its weight stream while the attention kernel drains.  ``attn`` and ``ffn``
    hold the arguments of ``attn_forward`` / ``ffn_forward`` (positional tensors under the key ``"tensors"``); the FFN's
    ``o2`` must be the attention block's."""
    a_args, _ka = _attn_args(*attn["tensors"], **{k: v for k, v in attn.items() if k != "tensors"})
    f_args, _kf = _ffn_args(*ffn["tensors"], **{k: v for k, v in ffn.items() if k != "tensors"})
    L.check(L.load().tb200_layer_forward(C.byref(a_args), C.byref(f_args), _stream()), "tb200_layer_forward")


def topk(scores: torch.Tensor, k: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = L.load()
    n = scores.shape[-1]
    rows = scores.numel() // n
    if out is None:
        out = torch.empty(*scores.shape[:-1], k, dtype=torch.int32, device=scores.device)
    L.check(lib.tb200_topk(_ptr(scores), _ptr(out), rows, n, k, _stream()), "tb200_topk")
    return out


def kv_compact(k_src: torch.Tensor, v_src: torch.Tensor, idx: torch.Tensor, kv_len: int, keep_recent: int = 0,
               k_dst: Optional[torch.Tensor] = None, v_dst: Optional[torch.Tensor] = None, kept_pos: Optional[torch.Tensor] = None,
               new_len: Optional[torch.Tensor] = None):
    """Pack the cache positions ``idx`` names (and the last ``keep_recent``) to the front of ``k_dst`` / ``v_dst``.

    ``k_src, v_src``: ``(..., L, D)`` caches, leading axes = batch and kv heads; ``idx``: int32 ``(..., n_idx)`` over the
    same leading axes.  Returns ``(k_dst, v_dst, kept_pos, new_len)``; destination caches are allocated
    ``(..., max_keep, D)`` when not given; ``k_dst=k_src, v_dst=v_src`` packs in place."""
    lib = L.load()
    if idx.dtype != torch.int32:
        raise TypeError("idx must be int32")
    if k_src.shape != v_src.shape or k_src.dtype != v_src.dtype:
        raise ValueError("k_src and v_src must agree in shape and dtype")
    lead = k_src.shape[:-2]
    if tuple(idx.shape[:-1]) != tuple(lead):
        raise ValueError(f"idx leading axes {tuple(idx.shape[:-1])} do not match the caches' {tuple(lead)}")
    rows = 1
    for d in lead:
        rows *= int(d)
    args = L.KvCompactArgs(dtype=_dt(k_src), rows=rows, head_dim=int(k_src.shape[-1]), kv_len=int(kv_len),
                           src_cache_len=int(k_src.shape[-2]), n_idx=int(idx.shape[-1]), keep_recent=int(keep_recent))
    max_keep = int(lib.tb200_kv_compact_max_keep(C.byref(args)))
    dev = k_src.device
    if k_dst is None:
        k_dst = torch.empty(*lead, max_keep, k_src.shape[-1], dtype=k_src.dtype, device=dev)
    if v_dst is None:
        v_dst = torch.empty(*lead, max_keep, k_src.shape[-1], dtype=k_src.dtype, device=dev)
    if k_dst.shape != v_dst.shape or k_dst.dtype != k_src.dtype or v_dst.dtype != k_src.dtype:
        raise ValueError("k_dst and v_dst must agree in shape and share the source dtype")
    if tuple(k_dst.shape[:-2]) != tuple(lead) or k_dst.shape[-1] != k_src.shape[-1]:
        raise ValueError("destination caches must have the source's leading axes and head dimension")
    if kept_pos is None:
        kept_pos = torch.empty(*lead, max_keep, dtype=torch.int32, device=dev)
    if new_len is None:
        new_len = torch.empty(*lead, dtype=torch.int32, device=dev)
    if kept_pos.dtype != torch.int32 or new_len.dtype != torch.int32 or kept_pos.numel() != rows * max_keep or new_len.numel() != rows:
        raise ValueError("kept_pos must be int32 (..., max_keep) and new_len int32 (...)")
    args.dst_cache_len = int(k_dst.shape[-2])
    args.idx, args.k_src, args.v_src = _ptr(idx), _ptr(k_src), _ptr(v_src)
    args.k_dst, args.v_dst, args.kept_pos, args.new_len = _ptr(k_dst), _ptr(v_dst), _ptr(kept_pos), _ptr(new_len)
    L.check(lib.tb200_kv_compact(C.byref(args), _stream()), "tb200_kv_compact")
    return k_dst, v_dst, kept_pos, new_len


def device_status() -> int:
    """Synchronise and return the device error word (0 = healthy); raises on a recorded timeout."""
    code = C.c_int(0)
    status = L.load().tb200_device_status(C.byref(code))
    if status != 0:
        raise L.Tb200Error(status, f"tb200_device_status (device code {code.value})")
    return code.value
