"""Multi-rank host logic on CPU: world_size-2 gloo processes drive trinity_b200.shard with an fp32 stand-in for the
local GPU operators and must reproduce the unsharded oracle."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as orc
from trinity_b200 import shard


class Fp32Ops:
    """fp32 torch stand-in for the local operators (the GPU path calls the C ABI instead)."""

    def gemm(self, a, b, *, b2=None, row_scale=None, residual=None, act=0):
        r = a @ b
        if row_scale is not None:
            r = r * row_scale[:, None]
        if b2 is not None:
            u = a @ b2
            if row_scale is not None:
                u = u * row_scale[:, None]
            r = torch.nn.functional.silu(r) * u
        if act == 1:
            r = torch.nn.functional.gelu(r)
        if residual is not None:
            r = r + residual
        return r

    def row_inv_rms(self, a, eps):
        return torch.rsqrt(a.pow(2).mean(-1) + eps)

    def rmsnorm(self, a, weight, eps):
        return orc.rmsnorm(a, weight, eps)


def _teardown():
    """Leave the group without turning a peer's earlier exit into a failure: gloo's teardown raises when the other side
    has already closed its sockets, which says nothing about the result a rank has long handed back."""
    try:
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        pass


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ffn_worker(rank, world, port, case, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    chunks = {"plain3": 3, "tail5": 5}.get(case)       # down projection and all-reduce pipelined over row blocks
    case = case.rstrip("35")
    try:
        t = orc.ref_ffn_inputs(12, 64, 96, seed=5, std=0.3)
        gelu = case == "gelu"
        sh = shard.shard_ffn_weights(t["WFF1b"], None if gelu else t["WFF1a"], t["WFF2"], None if case == "plain" or gelu else t["WO"],
                                     rank, world)
        o2_local = None
        if sh.wo is not None:
            n = t["O2"].shape[1] // world
            o2_local = t["O2"][:, rank * n:(rank + 1) * n].contiguous()
        out = shard.tensor_parallel_ffn(t["X"], sh, act="gelu" if gelu else "swiglu", o2_local=o2_local,
                                        norm=case in ("block", "tail"), falcon_tail=case == "tail", local_ops=Fp32Ops(),
                                        overlap_chunks=chunks)
        if rank == 0:
            ret.put({k: v.clone() for k, v in out.items()})
    finally:
        _teardown()


@pytest.mark.parametrize("case", ["plain", "gelu", "block", "tail", "plain3", "tail5"])
def test_tensor_parallel_ffn_two_ranks(case):
    ctx = mp.get_context("spawn")
    ret = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_ffn_worker, args=(r, 2, port, case, ret)) for r in range(2)]
    for p in procs:
        p.start()
    got = ret.get()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    t = orc.ref_ffn_inputs(12, 64, 96, seed=5, std=0.3)
    case = case.rstrip("35")
    if case == "plain":
        want = orc.ffn_block(t["X"], t["WFF1b"], t["WFF1a"], t["WFF2"])
        torch.testing.assert_close(got["FF2"], want["FF2"], rtol=1e-5, atol=1e-6)
    elif case == "gelu":
        want = orc.ffn_block(t["X"], t["WFF1b"], None, t["WFF2"], act="gelu")
        torch.testing.assert_close(got["FF2"], want["FF2"], rtol=1e-5, atol=1e-6)
    else:
        want = orc.ffn_block(t["O2"], t["WFF1b"], t["WFF1a"], t["WFF2"], wo=t["WO"], residual=t["X"], norm=True,
                             falcon_tail=case == "tail")
        torch.testing.assert_close(got["attn_O2"], want["attn_O2"], rtol=1e-5, atol=1e-6)
        key = "O_FF_norm" if case == "tail" else "FF2"
        torch.testing.assert_close(got[key], want[key], rtol=1e-4, atol=1e-6)


def _attn_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, S, N, Hq, Hkv, D, P = 2, 10, 64, 4, 2, 16, 6
        t = orc.bench_attention_inputs(B, S, N, Hq, Hkv, D, seed=2)
        r = orc._Rng(7)
        kc, vc = r.randn(B, Hkv, P + S, D), r.randn(B, Hkv, P + S, D)
        wq, wk, wv = shard.shard_attention_weights(t["WQ"], t["WK"], t["WV"], D, rank, world)
        out = orc.attention_block(t["X"], wq, wk, wv, shard.shard_heads(kc, Hkv, rank, world, 1), shard.shard_heads(vc, Hkv, rank, world, 1),
                                  past=P, head_dim=D, causal=True, sm_scale=D ** -0.5, roco=True)
        full = shard.gather_columns(out["O2"])
        if rank == 0:
            ret.put((full.clone(), out["C_out1"].clone()))
    finally:
        _teardown()


def test_head_group_sharded_attention_two_ranks():
    ctx = mp.get_context("spawn")
    ret = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_attn_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    full, c1_rank0 = ret.get()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    B, S, N, Hq, Hkv, D, P = 2, 10, 64, 4, 2, 16, 6
    t = orc.bench_attention_inputs(B, S, N, Hq, Hkv, D, seed=2)
    r = orc._Rng(7)
    kc, vc = r.randn(B, Hkv, P + S, D), r.randn(B, Hkv, P + S, D)
    want = orc.attention_block(t["X"], t["WQ"], t["WK"], t["WV"], kc, vc, past=P, head_dim=D, causal=True, sm_scale=D ** -0.5, roco=True)
    torch.testing.assert_close(full, want["O2"], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(c1_rank0, want["C_out1"][:, :2], rtol=1e-5, atol=1e-6)   # rank 0 owns q heads 0..1


def _evict_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        k, v, idx = _evict_inputs()
        out = shard.evict_rows(k, v, idx, kv_len=40, keep_recent=3, compact=orc.kv_compact)
        ret.put((rank, out["rows"].start, out["rows"].stop, out["k"].clone(), out["kept_pos"].clone(), out["all_new_len"].clone()))
    finally:
        _teardown()


def _evict_inputs():
    g = torch.Generator().manual_seed(9)
    rows, L, D = 5, 48, 8          # 5 rows over 2 ranks: shares of 3 and 2
    return (torch.randn(rows, L, D, generator=g), torch.randn(rows, L, D, generator=g),
            torch.randint(-2, 44, (rows, 12), generator=g, dtype=torch.int32))


def test_row_sharded_eviction_two_ranks():
    ctx = mp.get_context("spawn")
    ret = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_evict_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted([ret.get(), ret.get()], key=lambda g: g[0])
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    k, v, idx = _evict_inputs()
    wk, _, wpos, wlen = orc.kv_compact(k, v, idx, 40, 3)
    assert [(g[1], g[2]) for g in got] == [(0, 3), (3, 5)]
    for _, lo, hi, gk, gpos, all_len in got:
        assert torch.equal(gk, wk[lo:hi]) and torch.equal(gpos, wpos[lo:hi])
        assert torch.equal(all_len, wlen)            # every rank ends up with every row's new length


def test_slices_and_errors():
    qs, kvs = shard.head_group_slices(32, 8, 128, rank=3, world=4)
    assert (qs.start, qs.stop, kvs.start, kvs.stop) == (3 * 8 * 128, 4 * 8 * 128, 3 * 2 * 128, 4 * 2 * 128)
    with pytest.raises(ValueError, match="shard by batch"):
        shard.head_group_slices(71, 1, 64, rank=0, world=2)          # Falcon MQA cannot split its single KV head
    parts = [shard.batch_slice(16, r, 3) for r in range(3)]
    assert [p.stop - p.start for p in parts] == [6, 5, 5] and parts[0].start == 0 and parts[-1].stop == 16
    with pytest.raises(ValueError):
        shard.shard_ffn_weights(torch.zeros(8, 20), torch.zeros(8, 20), torch.zeros(20, 8), None, 0, 2)


def _absent_worker(rank, world, port, ret):
    """Rank 1 joins the group and then never makes the collective (a stalled or dead peer); rank 0 must get an exception
    from the host-side watchdog, not a hang.  The failure is made on the host: no GPU is involved."""
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        if rank == 1:
            time.sleep(3.0)             # outlives rank 0's time limit, then leaves between steps
            ret[rank] = "absent"
            return
        t0 = time.monotonic()
        try:
            shard.all_reduce_checked(torch.ones(4), timeout_s=1.0)
            ret[rank] = "completed?!"
        except shard.CollectiveTimeout as e:
            ret[rank] = ("timeout", time.monotonic() - t0, str(e))
    finally:
        os._exit(0)                     # no orderly teardown with a peer that is not there


def test_all_reduce_with_an_absent_rank_raises_instead_of_hanging():
    port = _free_port()
    ret = mp.Manager().dict()
    procs = [mp.get_context("spawn").Process(target=_absent_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive(), "a rank hung"
    assert ret[1] == "absent"
    kind, waited, msg = ret[0]
    assert kind == "timeout" and 0.9 < waited < 8.0 and "did not complete" in msg
