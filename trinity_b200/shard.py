"""Partitioning the fused blocks over the GPUs of one box: one process per GPU, ``torch.distributed`` for
the plumbing.  The reference has no multi-GPU path at all; the blocks are cut where they split naturally:

* attention with several KV heads (Llama GQA): by **KV-head group** -- each rank owns ``Hkv/g`` KV heads and their
  ``Hq/g`` query heads, i.e. column slices of ``WQ/WK/WV`` and the matching heads of the caches, of ``noise`` and of
  the per-key outputs; ``x`` is replicated.  No collective: ``O2`` comes out column-sharded ``(T, Hq*D/g)``, which is
  what a row-parallel ``WO`` consumes.  An all-gather is offered for callers that want the full ``O2``.
* attention with one KV head (Falcon MQA): by **batch** -- no collective, weights replicated.
* KV eviction: by **cache row** (batch x KV head) -- every rank packs its own contiguous share of the rows; the only
  exchange is an optional all-gather of the new row lengths (4 bytes per row), which a scheduler needs in full.
* FFN: tensor-parallel.  Gate/up (or W1) are column-parallel over the inner width, the activation is local, the down
  projection is row-parallel and ends in ONE all-reduce (sum) of ``(T, N)``.  With the ``WO`` prologue, ``WO`` is
  row-parallel on the column-sharded ``O2`` and needs its own all-reduce before the norm, so that the row statistic
  is computed on the complete sum.

The local compute is injectable (``local_ops``): on the GPUs it is ``trinity_b200.ops``; the CPU tests drive the same
sharding and collective logic over ``gloo`` with an fp32 stand-in.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch
import torch.distributed as dist


class CollectiveTimeout(RuntimeError):
    """A collective did not complete within the host-side time limit (a rank that never arrived, a failed link)."""


def wait_collective(work, timeout_s: float, what: str = "collective") -> None:
    """Poll an asynchronous collective until it completes, raises, or ``timeout_s`` passes.

    ``torch.distributed`` surfaces NCCL's asynchronous errors on the work object (``exception()``); a rank that never
    joins shows no error at all, only a collective that does not finish -- the host-side clock here is what turns that
    into a ``CollectiveTimeout`` the caller can act on (drop the rank, rebuild the group) instead of a hang.  The wait
    is on the host: nothing is enqueued behind the collective until it is known to have finished."""
    import time
    deadline = time.monotonic() + timeout_s
    while True:
        if work.is_completed():
            exc = work.exception() if hasattr(work, "exception") else None
            if exc is not None:
                raise RuntimeError(f"{what} failed: {exc}")
            return
        if time.monotonic() > deadline:
            raise CollectiveTimeout(f"{what} did not complete within {timeout_s:.1f} s")
        time.sleep(0.0005)


def all_reduce_checked(t: torch.Tensor, timeout_s: float, group=None) -> None:
    """Sum-all-reduce ``t`` in place, or raise ``CollectiveTimeout`` / ``RuntimeError`` -- never hang."""
    work = dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group, async_op=True)
    wait_collective(work, timeout_s, "all-reduce")


def _world(group=None) -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def head_group_slices(n_q_heads: int, n_kv_heads: int, head_dim: int, rank: int, world: int) -> Tuple[slice, slice]:
    """Column ranges of WQ and of WK/WV owned by ``rank`` when the KV heads are dealt out in contiguous groups."""
    if n_kv_heads % world != 0:
        raise ValueError(f"{n_kv_heads} KV heads cannot be split over {world} ranks; shard by batch instead")
    if n_q_heads % n_kv_heads != 0:
        raise ValueError("n_q_heads must be a multiple of n_kv_heads")
    kv_per = n_kv_heads // world
    q_per = n_q_heads // world
    return (slice(rank * q_per * head_dim, (rank + 1) * q_per * head_dim),
            slice(rank * kv_per * head_dim, (rank + 1) * kv_per * head_dim))


def shard_attention_weights(wq, wk, wv, head_dim: int, rank: int, world: int):
    """This rank's contiguous column slices of the three projection weights."""
    qs, kvs = head_group_slices(wq.shape[1] // head_dim, wk.shape[1] // head_dim, head_dim, rank, world)
    return wq[:, qs].contiguous(), wk[:, kvs].contiguous(), wv[:, kvs].contiguous()


def shard_heads(t: Optional[torch.Tensor], n_heads: int, rank: int, world: int, head_axis: int):
    """The slice of a per-head tensor (cache, noise, c_out*, topk_idx) that belongs to this rank."""
    if t is None:
        return None
    per = n_heads // world
    return t.narrow(head_axis, rank * per, per).contiguous()


def batch_slice(batch: int, rank: int, world: int) -> slice:
    """Contiguous share of the batch for this rank (the first ``batch % world`` ranks take one more)."""
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def gather_columns(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather column shards ``(.., n/g)`` into ``(.., n)``; the optional step after head-group attention."""
    rank, world = _world(group)
    if world == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=-1)


@dataclass
class FfnShard:
    """This rank's slice of the FFN weights."""
    w_gate: torch.Tensor            # (N, P/g)
    w_up: Optional[torch.Tensor]    # (N, P/g) or None (GELU MLP)
    w_down: torch.Tensor            # (P/g, N)
    wo: Optional[torch.Tensor]      # (N/g, N) or None


def shard_ffn_weights(w_gate, w_up, w_down, wo, rank: int, world: int) -> FfnShard:
    P = w_gate.shape[1]
    if P % (8 * world) != 0:
        raise ValueError(f"inner width {P} must be a multiple of 8*{world}")
    p = slice(rank * P // world, (rank + 1) * P // world)
    wo_l = None
    if wo is not None:
        N = wo.shape[0]
        if N % (8 * world) != 0:
            raise ValueError(f"hidden width {N} must be a multiple of 8*{world}")
        wo_l = wo[rank * N // world:(rank + 1) * N // world, :].contiguous()
    return FfnShard(w_gate[:, p].contiguous(), None if w_up is None else w_up[:, p].contiguous(), w_down[p, :].contiguous(), wo_l)


class LocalOps:
    """The three local operators the tensor-parallel FFN needs; the default runs them on the GPU through the C ABI."""

    def gemm(self, a, b, *, b2=None, row_scale=None, residual=None, act=0):
        from . import ops
        return ops.gemm(a, b, b2=b2, row_scale=row_scale, residual=residual, act=act, split_k=0)

    def row_inv_rms(self, a, eps):
        from . import ops
        return ops.row_inv_rms(a, eps)

    def rmsnorm(self, a, weight, eps):
        from . import ops
        return ops.rmsnorm(a, weight, eps)


def tensor_parallel_ffn(x: torch.Tensor, shard: FfnShard, *, act: str = "swiglu", o2_local: Optional[torch.Tensor] = None,
                        norm: bool = False, norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 0.0,
                        falcon_tail: bool = False, group=None, local_ops=None,
                        all_reduce: Optional[Callable[[torch.Tensor], None]] = None,
                        overlap_chunks: Optional[int] = None, peer=None,
                        collective_timeout_s: Optional[float] = None) -> Dict[str, torch.Tensor]:
    """One FFN block, tensor-parallel over the ranks of ``group``.

    ``x`` (T,N) is replicated; ``o2_local`` (T,N/g) is this rank's column shard of the attention output when the block
    starts with ``O2 @ WO + X``.  Returns ``{"FF2": ..}`` (replicated after the all-reduce) or, with ``falcon_tail``,
    ``{"O_FF": FF2 + h, "O_FF_norm": RMSNorm(O_FF)}``.  Residuals are added on rank 0 only, before the all-reduce, so
    that the sum carries them exactly once.

    With ``peer`` (a ``trinity_b200.peer.PeerReduce`` set up for ``(T, N)``) the down projection and its all-reduce are
    ONE pair of kernels that exchange over peer memory: the projection's epilogue stores every 128-row block of its partial
    product into the block owner's staging buffer while its main loop runs on, and a second kernel sums the ranks'
    contributions in rank order and writes the result into every rank's buffer (``tb200_gemm_peer_reduce``).  No NCCL
    call is made for that step; the result is the communicator's buffer, overwritten by the next call.

    ``collective_timeout_s`` puts a host-side clock on every NCCL all-reduce of the block (``all_reduce_checked``): a rank
    that never arrives raises ``CollectiveTimeout`` on the others instead of hanging them.

    With ``overlap_chunks`` > 1 the down projection and its all-reduce are pipelined over that many blocks of token
    rows: the sum of block i travels (asynchronous collective, the library's own stream) while block i+1 is multiplied.
    Off by default: measured on B200s with 4 blocks it is slower than one GEMM and one all-reduce (Llama FFN, 16384
    tokens: 2.26 against 2.08 ms on 2 GPUs, 1.15 against 0.86 ms on 8; Falcon FFN, 32768 tokens: 2.08 against 1.71 ms on
    8) -- the collective's CTAs take SMs from a GEMM that is laid out as one persistent CTA pair per SM pair, and four
    quarter-size all-reduces cost more than one.
    """
    rank, world = _world(group)
    lo = local_ops or LocalOps()
    if overlap_chunks is None:
        overlap_chunks = 1
    if overlap_chunks > 1 and all_reduce is not None:
        raise ValueError("overlap_chunks needs the built-in asynchronous all-reduce")
    if all_reduce is None:
        def all_reduce(t):
            if world > 1:
                if collective_timeout_s is not None:     # host-side watchdog: a rank that never arrives raises instead of hanging
                    all_reduce_checked(t, collective_timeout_s, group)
                else:
                    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    gelu = act == "gelu"
    if gelu == (shard.w_up is not None):
        raise ValueError("SwiGLU needs w_up; the GELU MLP takes none")

    a = x
    if shard.wo is not None:
        if o2_local is None:
            raise ValueError("o2_local is required when the shard carries WO")
        a = lo.gemm(o2_local, shard.wo, residual=x if rank == 0 else None)   # row-parallel WO
        all_reduce(a)
    h, row_scale = a, None
    if norm:
        if norm_weight is not None or falcon_tail:
            h = lo.rmsnorm(a, norm_weight, norm_eps)          # the tail needs h itself as a residual
        else:
            row_scale = lo.row_inv_rms(a, norm_eps)           # norm folded into the next epilogue as a row scale
    if gelu:
        ff1 = lo.gemm(h, shard.w_gate, row_scale=row_scale, act=1)
    else:
        ff1 = lo.gemm(h, shard.w_gate, b2=shard.w_up, row_scale=row_scale)
    if peer is not None and world > 1:
        ff2 = peer.gemm_reduce(ff1, shard.w_down, residual=h if falcon_tail else None)
    elif overlap_chunks > 1 and world > 1:
        T = ff1.shape[0]
        step = -(-T // overlap_chunks)
        if T >= 128 * overlap_chunks:
            step = (step + 127) // 128 * 128                   # whole row tiles of the GEMM per block
        parts, works = [], []
        for r0 in range(0, T, step):
            r1 = min(T, r0 + step)
            part = lo.gemm(ff1[r0:r1], shard.w_down, residual=h[r0:r1] if (falcon_tail and rank == 0) else None)
            works.append(dist.all_reduce(part, op=dist.ReduceOp.SUM, group=group, async_op=True))
            parts.append(part)
        for work in works:
            work.wait()
        ff2 = torch.cat(parts, dim=0)
    else:
        ff2 = lo.gemm(ff1, shard.w_down, residual=h if (falcon_tail and rank == 0) else None)   # row-parallel down
        all_reduce(ff2)
    if not falcon_tail:
        return {"FF2": ff2, "attn_O2": a}
    return {"O_FF": ff2, "O_FF_norm": lo.rmsnorm(ff2, None, 0.0), "attn_O2": a}


def evict_rows(k_cache: torch.Tensor, v_cache: torch.Tensor, idx: torch.Tensor, kv_len: int, keep_recent: int = 0, *,
               compact: Optional[Callable] = None, gather_lengths: bool = True, group=None) -> Dict[str, torch.Tensor]:
    """KV eviction over the ranks: ``k_cache, v_cache (rows, L, D)`` and ``idx (rows, n_idx)`` are the SAME on every
    rank's call in shape (each rank may hold only its own rows' data); rank r packs rows ``batch_slice(rows, r, world)``
    with ``compact`` (default ``trinity_b200.ops.kv_compact``) and returns its share: ``rows`` (the slice), ``k``, ``v``,
    ``kept_pos``, ``new_len``; with ``gather_lengths`` also ``all_new_len (rows,)`` from one all-gather."""
    rank, world = _world(group)
    if k_cache.dim() != 3 or idx.dim() != 2 or idx.shape[0] != k_cache.shape[0]:
        raise ValueError("evict_rows takes (rows, L, D) caches and (rows, n_idx) index lists")
    if compact is None:
        from . import ops
        compact = ops.kv_compact
    rows = k_cache.shape[0]
    mine = batch_slice(rows, rank, world)
    k_new, v_new, kept, n_new = compact(k_cache[mine].contiguous(), v_cache[mine].contiguous(), idx[mine].contiguous(), kv_len, keep_recent)
    out = {"rows": mine, "k": k_new, "v": v_new, "kept_pos": kept, "new_len": n_new}
    if gather_lengths:
        if world == 1:
            out["all_new_len"] = n_new.clone()
        else:  # shares differ by at most one row: pad to the largest share, gather, cut
            width = (rows + world - 1) // world
            padded = torch.zeros(width, dtype=n_new.dtype, device=n_new.device)
            padded[: n_new.numel()] = n_new
            parts = [torch.empty_like(padded) for _ in range(world)]
            dist.all_gather(parts, padded, group=group)
            out["all_new_len"] = torch.cat([parts[r][: (s_.stop - s_.start)] for r in range(world)
                                            for s_ in [batch_slice(rows, r, world)]])
    return out
