"""Parity of the individual sm_100a kernels against fp32 references, through the C ABI."""
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import ATOL, RTOL, close, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from trinity_b200 import ops as o
    return o


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,cols", [(1, 64), (16, 4544), (300, 4096), (5, 8200), (3, 16384)])
def test_rmsnorm(ops, dt, rows, cols):
    g = torch.Generator().manual_seed(rows * 7 + cols)
    x = torch.randn(rows, cols, generator=g).to(dt)
    w = (1 + 0.02 * torch.randn(cols, generator=g)).to(dt)
    close(ops.rmsnorm(x.to(dev()), w.to(dev()), 1e-5), orc.rmsnorm(x, w, 1e-5), msg="weighted")
    inv = torch.zeros(rows, dtype=torch.float32, device=dev())
    y = ops.rmsnorm(x.to(dev()), None, 0.0, inv_rms=inv)
    close(y, orc.rmsnorm(x), msg="reference point (no weight, eps 0)")
    close(inv, torch.rsqrt(x.float().pow(2).mean(-1)), rtol=1e-4, atol=1e-6, msg="inv_rms")


def test_rmsnorm_rejects_bad_arguments(ops):
    from trinity_b200._lib import Tb200Error
    x = torch.zeros(4, 60, dtype=torch.bfloat16, device=dev())      # cols % 8 != 0
    with pytest.raises(Tb200Error):
        ops.rmsnorm(x)
    with pytest.raises(TypeError):
        ops.rmsnorm(torch.zeros(4, 64, dtype=torch.float64, device=dev()))


def _gemm_ref(a, b, b2=None, rs=None, res=None, act=0):
    r = a.float() @ b.float()
    if rs is not None:
        r = r * rs[:, None]
    if b2 is not None:
        u = a.float() @ b2.float()
        if rs is not None:
            u = u * rs[:, None]
        r = torch.nn.functional.silu(r) * u
    if act == 1:
        r = torch.nn.functional.gelu(r)
    if res is not None:
        r = r + res.float()
    return r


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K,opts", [
    (128, 256, 64, {}), (1, 8, 8, {}), (200, 328, 192, {}), (1000, 4544, 4544, {}), (257, 264, 4096, {}),
    (384, 512, 512, dict(rs=True, res=True)), (384, 1024, 520, dict(gelu=True)), (300, 640, 1024, dict(gated=True, rs=True)),
    (130, 136, 72, dict(gated=True)), (64, 4096, 2048, dict(split=4)), (64, 1024, 2048, dict(split=4, gated=True, rs=True)),
    (16, 512, 4096, dict(split=0, res=True)), (16, 512, 4096, dict(split=7, gelu=True, res=True)), (2100, 520, 136, {}),
    # either side of the 64-row tile (at most 64 rows: sixteen per epilogue warp; more: thirty-two)
    (63, 264, 128, dict(res=True, rs=True)), (65, 264, 128, dict(res=True, rs=True)), (33, 520, 1024, dict(gated=True, split=2)),
    (17, 256, 512, dict(gelu=True)), (49, 136, 200, dict(gated=True, rs=True)),
])
def test_gemm(ops, dt, M, N, K, opts):
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(dt).to(dev())
    b = (torch.randn(K, N, generator=g) * K ** -0.5).to(dt).to(dev())
    b2 = (torch.randn(K, N, generator=g) * K ** -0.5).to(dt).to(dev()) if opts.get("gated") else None
    rs = (torch.rand(M, generator=g) + 0.5).to(dev()) if opts.get("rs") else None
    res = torch.randn(M, N, generator=g).to(dt).to(dev()) if opts.get("res") else None
    act = 1 if opts.get("gelu") else 0
    out = torch.full((M, N), float("nan"), dtype=dt, device=dev())
    ops.gemm(a, b, b2=b2, row_scale=rs, residual=res, act=act, split_k=opts.get("split", 1), out=out)
    ops.device_status()
    close(out, _gemm_ref(a, b, b2, rs, res, act), msg=f"gemm {M}x{N}x{K} {opts}")


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K,opts", [
    (64, 4096, 14336, {}), (16, 4544, 4544, dict(res=True)), (128, 4096, 4096, dict(rs=True, gelu=True)),
    (100, 2048, 4104, dict(res=True, rs=True)), (64, 14336, 4096, dict(gated=True)), (16, 4544, 4544, dict(gated=True, rs=True)),
    (1, 8192, 2048, {}), (64, 1032, 8192, {}),
])
def test_gemm_few_rows_wide_weights(ops, dt, M, N, K, opts):
    """One row-tile of tokens against wide weights (the decode and 64-token shapes of the benchmark): with split_k = 0 the
    library cuts K into slices until the SMs are filled and sums the slices in a fixed order.  Run twice: same bits."""
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(dt).to(dev())
    b = (torch.randn(K, N, generator=g) * K ** -0.5).to(dt).to(dev())
    b2 = (torch.randn(K, N, generator=g) * K ** -0.5).to(dt).to(dev()) if opts.get("gated") else None
    rs = (torch.rand(M, generator=g) + 0.5).to(dev()) if opts.get("rs") else None
    res = torch.randn(M, N, generator=g).to(dt).to(dev()) if opts.get("res") else None
    act = 1 if opts.get("gelu") else 0
    ref = _gemm_ref(a, b, b2, rs, res, act)
    outs = []
    for _ in range(2):
        out = torch.full((M, N), float("nan"), dtype=dt, device=dev())
        ops.gemm(a, b, b2=b2, row_scale=rs, residual=res, act=act, split_k=0, out=out)
        ops.device_status()
        close(out, ref, msg=f"gemm {M}x{N}x{K} {opts}")
        outs.append(out)
    assert torch.equal(outs[0], outs[1]), "two runs of the same problem differ"


def test_gemm_is_deterministic(ops):
    g = torch.Generator().manual_seed(5)
    a = torch.randn(48, 4096, generator=g).to(torch.bfloat16).to(dev())
    b = (torch.randn(4096, 1024, generator=g) * 0.02).to(torch.bfloat16).to(dev())
    outs = [ops.gemm(a, b, split_k=0).clone() for _ in range(3)]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


@pytest.mark.parametrize("rows,n,k", [(1, 2, 1), (3, 17, 17), (8, 1040, 128), (4, 4096, 1024), (2, 16384, 1000), (5, 1000, 999)])
def test_topk_is_a_stable_descending_sort(ops, rows, n, k):
    g = torch.Generator().manual_seed(n)
    s = torch.randn(rows, n, generator=g)
    s = s.round(decimals=1)          # a grid of values: many exact ties
    got = ops.topk(s.to(dev()), k)
    assert torch.equal(got.cpu(), orc.stable_topk(s, k))


def test_topk_handles_zero_signs_and_rejects_oversize(ops):
    from trinity_b200._lib import Tb200Error
    s = torch.tensor([[0.0, -0.0, 0.0, 1.0, -0.0]])
    assert ops.topk(s.to(dev()), 5).cpu().tolist() == [[3, 0, 1, 2, 4]]
    with pytest.raises(Tb200Error):
        ops.topk(torch.zeros(1, 20000, device=dev()), 4)


# ------------------------------------------------------------------------------------------------- KV-cache eviction
def _evict_case(lead, L, kv_len, D, n_idx, keep_recent, dt, seed, junk=True):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(*lead, L, D, generator=g).to(dt)
    v = torch.randn(*lead, L, D, generator=g).to(dt)
    idx = torch.randint(0, max(kv_len, 1), (*lead, n_idx), generator=g, dtype=torch.int32)   # with duplicates
    if junk and n_idx >= 4:
        idx[..., 0] = -3
        idx[..., 1] = kv_len          # first invalid position
        idx[..., 2] = 2 ** 31 - 1
    return k, v, idx


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("lead,L,kv_len,D,n_idx,recent", [
    ((1,), 64, 64, 128, 16, 0),            # one CTA per row
    ((2, 3), 200, 137, 64, 40, 9),         # ragged: kv_len not a multiple of 32, recent window inside a bitmap word
    ((4, 8), 1040, 1040, 128, 256, 32),    # the reference's decode cache (P 1024 + M 16), GQA-sized rows
    ((71,), 1040, 1040, 64, 512, 0),       # Falcon heads
    ((2, 2), 4352, 4100, 128, 3000, 500),  # many chunks per row, keeps most of the cache
    ((3,), 96, 50, 128, 200, 0),           # more indices than positions: everything named survives once
    ((2,), 300, 300, 64, 0, 70),           # no index list at all: the recent window alone
])
def test_kv_compact_matches_oracle(ops, dt, lead, L, kv_len, D, n_idx, recent):
    k, v, idx = _evict_case(lead, L, kv_len, D, n_idx, recent, dt, seed=L + n_idx)
    rk, rv, rpos, rlen = orc.kv_compact(k, v, idx, kv_len, recent)
    max_keep = rpos.shape[-1]
    # destination rows longer than needed and pre-filled: positions beyond the kept count must stay untouched
    k_dst = torch.full((*lead, max_keep + 5, D), 7.0, dtype=dt, device=dev())
    v_dst = torch.full((*lead, max_keep + 5, D), -7.0, dtype=dt, device=dev())
    gk, gv, gpos, glen = ops.kv_compact(k.to(dev()), v.to(dev()), idx.to(dev()), kv_len, recent, k_dst=k_dst, v_dst=v_dst)
    ops.device_status()
    assert torch.equal(glen.cpu(), rlen) and torch.equal(gpos.cpu(), rpos)
    live = (torch.arange(max_keep + 5).expand(*lead, -1) < rlen.unsqueeze(-1)).unsqueeze(-1)
    pad = lambda t, fill: torch.cat([t, torch.zeros(*lead, 5, D, dtype=dt)], dim=-2).where(live, torch.tensor(fill, dtype=dt))
    assert torch.equal(gk.cpu(), pad(rk, 7.0)) and torch.equal(gv.cpu(), pad(rv, -7.0))


@pytest.mark.parametrize("lead,L,kv_len,D,n_idx,recent", [
    ((2, 3), 200, 137, 64, 40, 9), ((4, 8), 1040, 1040, 128, 256, 32), ((2, 2), 4352, 4100, 128, 3000, 500),
    ((3,), 96, 50, 128, 200, 0), ((2,), 300, 300, 64, 0, 70), ((1,), 512, 512, 128, 512, 0),
])
def test_kv_compact_in_place(ops, lead, L, kv_len, D, n_idx, recent):
    """Source and destination the same caches: packed prefix as the oracle's, everything behind it as it was."""
    k, v, idx = _evict_case(lead, L, kv_len, D, n_idx, recent, torch.bfloat16, seed=L * 3 + n_idx, junk=n_idx != 512)
    if n_idx == 512:
        idx = torch.arange(512, dtype=torch.int32).flip(0).expand(*lead, 512).contiguous()   # keep all: nothing moves
    rk, rv, rpos, rlen = orc.kv_compact(k, v, idx, kv_len, recent)
    kd, vd = k.to(dev()), v.to(dev())
    gk, gv, gpos, glen = ops.kv_compact(kd, vd, idx.to(dev()), kv_len, recent, k_dst=kd, v_dst=vd)
    ops.device_status()
    assert gk.data_ptr() == kd.data_ptr()
    assert torch.equal(glen.cpu(), rlen) and torch.equal(gpos.cpu(), rpos)
    live = (torch.arange(L).expand(*lead, -1) < rlen.unsqueeze(-1)).unsqueeze(-1)
    grow = lambda t: torch.cat([t, torch.zeros(*lead, L - t.shape[-2], D, dtype=t.dtype)], dim=-2)
    assert torch.equal(gk.cpu(), torch.where(live, grow(rk), k)) and torch.equal(gv.cpu(), torch.where(live, grow(rv), v))


def test_kv_compact_after_topk_keeps_the_best_keys(ops):
    """The chain the blocks feed: per-key scores -> top-k -> eviction; the kept set is the top-k set, in cache order."""
    g = torch.Generator().manual_seed(3)
    H, Lc, D, topk = 8, 1040, 128, 128
    scores = torch.randn(H, Lc, generator=g)
    k, v, _ = _evict_case((H,), Lc, Lc, D, 4, 0, torch.bfloat16, seed=4)
    idx = ops.topk(scores.to(dev()), topk)
    gk, gv, gpos, glen = ops.kv_compact(k.to(dev()), v.to(dev()), idx, Lc)
    assert glen.cpu().tolist() == [topk] * H
    want = torch.sort(orc.stable_topk(scores, topk).long(), dim=-1).values
    assert torch.equal(gpos.cpu().long(), want)
    assert torch.equal(gk.cpu(), torch.gather(k, 1, want.unsqueeze(-1).expand(-1, -1, D)))
    assert torch.equal(gv.cpu(), torch.gather(v, 1, want.unsqueeze(-1).expand(-1, -1, D)))


def test_kv_compact_full_size_properties(ops):
    """RoCo configuration size (B4, 32 heads, 4096+ keys, top-k 1024 + 64 recent): idempotence (evicting again with
    the identity list changes nothing), keep-all is a copy, and the run is bit-identical when repeated."""
    B, H, Lc, D, topk, recent = 4, 32, 4096, 128, 1024, 64
    g = torch.Generator(device=dev()).manual_seed(11)
    k = torch.randn(B, H, Lc, D, generator=g, device=dev()).to(torch.bfloat16)
    v = torch.randn(B, H, Lc, D, generator=g, device=dev()).to(torch.bfloat16)
    scores = torch.randn(B, H, Lc, generator=g, device=dev())
    idx = ops.topk(scores, topk)
    k1, v1, pos1, len1 = ops.kv_compact(k, v, idx, Lc, recent)
    k1b, v1b, pos1b, _ = ops.kv_compact(k, v, idx, Lc, recent)
    n = len1.long()
    assert int(n.min()) >= topk and int(n.max()) <= topk + recent
    valid = torch.arange(pos1.shape[-1], device=dev()).expand_as(pos1) < n.unsqueeze(-1)
    # destination positions beyond a row's count are left as they were (uninitialised here): compare the packed part
    assert torch.equal(k1[valid], k1b[valid]) and torch.equal(v1[valid], v1b[valid]) and torch.equal(pos1, pos1b)
    p = pos1.long().clamp_min(0)
    assert bool(((pos1 >= 0) == valid).all())
    assert bool((p[..., 1:] > p[..., :-1])[valid[..., 1:]].all())                      # strictly ascending
    assert bool((torch.gather(k, 2, p.unsqueeze(-1).expand(-1, -1, -1, D)) == k1)[valid].all())
    in_topk = torch.zeros(B, H, Lc, dtype=torch.bool, device=dev()).scatter_(2, idx.long(), True)
    in_topk[..., Lc - recent:] = True
    assert torch.equal(in_topk.sum(-1), n)
    # evicting the packed cache with the identity list keeps it as it is (rows share the smallest kept count)
    m = int(n.min())
    ident = torch.arange(m, dtype=torch.int32, device=dev()).expand(B, H, m).contiguous()
    k2, v2, pos2, len2 = ops.kv_compact(k1, v1, ident, m)
    assert torch.equal(k2, k1[..., :m, :]) and torch.equal(v2, v1[..., :m, :]) and bool((len2 == m).all())
    ops.device_status()


def test_kv_compact_rejects_bad_arguments(ops):
    from trinity_b200._lib import Tb200Error
    k, v, idx = (t.to(dev()) for t in _evict_case((2,), 64, 64, 128, 8, 0, torch.bfloat16, seed=1))
    with pytest.raises(Tb200Error):       # overlapping, but not the same caches: K packed into V's memory
        ops.kv_compact(k, v, idx, 64, k_dst=v, v_dst=torch.empty_like(v))
    buf = torch.zeros(3, 64, 128, dtype=k.dtype, device=dev())
    with pytest.raises(Tb200Error):       # destination rows start inside the source rows
        ops.kv_compact(buf[0:2], v, idx, 64, k_dst=buf[1:3], v_dst=torch.empty_like(v))
    with pytest.raises(Tb200Error):       # destination too short
        ops.kv_compact(k, v, idx, 64, k_dst=torch.empty(2, 4, 128, dtype=k.dtype, device=dev()), v_dst=torch.empty(2, 4, 128, dtype=k.dtype, device=dev()))
    with pytest.raises(Tb200Error):       # more valid positions than the cache holds
        ops.kv_compact(k, v, idx, 65)
    with pytest.raises(Tb200Error):       # head dimension
        ops.kv_compact(k[..., :32].contiguous(), v[..., :32].contiguous(), idx, 64)
    with pytest.raises(TypeError):
        ops.kv_compact(k, v, idx.long(), 64)
    # nothing to keep: a call that launches nothing and reports zero lengths
    _, _, pos, n = ops.kv_compact(k, v, idx[:, :0].contiguous(), 64)
    assert pos.shape == (2, 0) and n.cpu().tolist() == [0, 0]


def test_kv_compact_under_graph_replay(ops):
    """With caller-provided outputs the call allocates nothing: it can be captured and replayed like the blocks are."""
    k, v, idx = (t.to(dev()) for t in _evict_case((4, 8), 1040, 1040, 128, 256, 32, torch.bfloat16, seed=21))
    want = ops.kv_compact(k, v, idx, 1040, 32)                      # also the call outside capture (sets kernel attributes)
    outs = [torch.zeros_like(t) for t in want]
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            ops.kv_compact(k, v, idx, 1040, 32, k_dst=outs[0], v_dst=outs[1], kept_pos=outs[2], new_len=outs[3])
        for _ in range(3):
            graph.replay()
    torch.cuda.synchronize()
    ops.device_status()
    n = want[3].long()
    live = (torch.arange(want[2].shape[-1], device=dev()).expand_as(want[2]) < n.unsqueeze(-1))
    assert torch.equal(outs[3], want[3]) and torch.equal(outs[2], want[2])
    assert torch.equal(outs[0][live], want[0][live]) and torch.equal(outs[1][live], want[1][live])
