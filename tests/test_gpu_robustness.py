"""What happens around the kernels: a bounded device wait that runs out, and workspaces under CUDA-graph replay."""
import pytest
import torch

from oracle import oracle as orc
from trinity_b200 import _lib as L
from trinity_b200 import ops

from .gpu_util import close, dev

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_is_reported():
    """One CTA waits on an mbarrier that nothing arms, through the same mbar_wait / abort-flag code as the compute
    kernels, with a limit of 2e5 cycles (about 0.1 ms): the wait gives up, the kernel returns, the status call reports
    the timeout once and the device is healthy afterwards."""
    lib = L.load()
    ops.device_status()                                   # start clean
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.tb200_selftest_wait_timeout(200_000, stream) == 0
    with pytest.raises(L.Tb200Error) as e:
        ops.device_status()
    assert e.value.status == -5 and "device code 900" in str(e.value)
    assert ops.device_status() == 0                       # reading the word cleared it
    # the context is intact: a real kernel runs and is right
    x = torch.randn(8, 256, device=dev()).to(torch.bfloat16)
    close(ops.rmsnorm(x), orc.rmsnorm(x.cpu()), msg="rmsnorm after a reported timeout")
    assert ops.device_status() == 0


def test_wait_limit_reaches_the_kernels():
    """The host-set limit travels in the kernel parameters: with a generous but finite limit the blocks run as before."""
    lib = L.load()
    assert lib.tb200_set_wait_limit_cycles(500_000_000) == 0
    try:
        a = torch.randn(300, 512, device=dev()).to(torch.bfloat16)
        b = (torch.randn(512, 264, device=dev()) * 512 ** -0.5).to(torch.bfloat16)
        close(ops.gemm(a, b), a.float() @ b.float(), msg="gemm under a 5e8-cycle limit")
        assert ops.device_status() == 0
    finally:
        lib.tb200_set_wait_limit_cycles(4_000_000_000)


def test_graph_replay_survives_a_larger_eager_call():
    """A captured graph holds the address of the workspace it was captured with.  A later, larger eager call outgrows
    that buffer; the old one must stay alive (and unshared), or the replay would write partial sums into memory the
    allocator has handed to somebody else."""
    g = torch.Generator().manual_seed(3)
    M, N, K = 16, 1024, 4096                                # decode size: K is split, partial sums go to the workspace
    a = torch.randn(M, K, generator=g).to(torch.float16).to(dev())
    b = (torch.randn(K, N, generator=g) * K ** -0.5).to(torch.float16).to(dev())
    out = torch.zeros(M, N, dtype=torch.float16, device=dev())
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        ops.gemm(a, b, out=out)                             # sizes this stream's workspace
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            ops.gemm(a, b, out=out)
        # a larger call on the same stream: the buffer is replaced ...
        a2 = torch.randn(64, K, generator=g).to(torch.float16).to(dev())
        b2 = (torch.randn(K, 4096, generator=g) * K ** -0.5).to(torch.float16).to(dev())
        big = ops.gemm(a2, b2)
        # ... and fresh allocations may now land where a freed buffer would have been
        junk = [torch.full((1 << 20,), float("nan"), device=dev()) for _ in range(8)]
        out.zero_()
        graph.replay()
        side.synchronize()
    close(out, a.float() @ b.float(), msg="replayed graph after the workspace grew")
    close(big, a2.float() @ b2.float(), msg="the larger call")
    assert all(bool(torch.isnan(j).all()) for j in junk), "the replay wrote into memory it no longer owns"
    assert ops.device_status() == 0


def test_norm_weight_folded_into_the_projections():
    """(x * r * g) @ W = r * (x @ (diag(g) W)): the block with the folded weights (the default through ops) and with the
    materialised normalised activations agree with the oracle and with each other, and the folded path needs no room
    for a normalised copy of x."""
    import ctypes as C
    from .gpu_util import attention_case
    flags = L.ATTN_PRENORM | L.ATTN_CAUSAL
    try:
        ops.FoldedWeights.enabled = False
        plain, ref = attention_case(2, 300, 1024, 8, 2, 128, 20, flags, weights=True, seed=9)
        ops.FoldedWeights.enabled = True
        ops.FoldedWeights.clear()
        folded, _ = attention_case(2, 300, 1024, 8, 2, 128, 20, flags, weights=True, seed=9)
    finally:
        ops.FoldedWeights.enabled = True
    close(plain["O2"], ref["O2"], msg="O2, materialised norm")
    close(folded["O2"], ref["O2"], msg="O2, folded norm weight")
    close(folded["K_new"], ref["K_new"], msg="appended K rows, folded norm weight")
    close(folded["O2"], plain["O2"].float(), msg="folded against materialised")
    lib = L.load()
    a = L.AttnArgs(dtype=L.BF16, flags=flags, batch=2, seq=300, hidden=1024, n_q_heads=8, n_kv_heads=2, head_dim=128, past=20,
                   cache_len=320, sm_scale=1.0, tau=1.0, x=0x1000, wq=0x2000, wk=0x3000, wv=0x4000, k_cache=0x5000, v_cache=0x6000,
                   o2=0x7000, norm_weight=0x8000, aux_dtype=L.F32)
    unfolded_bytes = lib.tb200_attn_workspace_bytes(C.byref(a))
    a.flags = flags | L.ATTN_NORM_FOLDED
    assert unfolded_bytes - lib.tb200_attn_workspace_bytes(C.byref(a)) >= 2 * 300 * 1024 * 2 - 4096   # x_norm is gone


def test_ffn_block_with_a_weighted_norm():
    """The reference FFN block with a norm weight and eps (extension; the reference's norm has neither), folded into
    the gate / up projections."""
    g = torch.Generator().manual_seed(21)
    M, N, P = 200, 512, 1536
    rn = lambda *s: torch.randn(*s, generator=g)
    t = {"O2": rn(M, N), "X": rn(M, N), "WO": rn(N, N) * N ** -0.5, "WFF1a": rn(N, P) * N ** -0.5, "WFF1b": rn(N, P) * N ** -0.5,
         "WFF2": rn(P, N) * P ** -0.5, "g": 1 + 0.1 * rn(N)}
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    d = {k: v.to(dev()) for k, v in t.items()}
    ff2 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    ops.ffn_forward(d["X"], d["WFF1b"], d["WFF1a"], d["WFF2"], ff2, flags=L.FFN_NORM, o2=d["O2"], wo=d["WO"], norm_weight=d["g"], norm_eps=1e-5)
    ops.device_status()
    f = lambda k: t[k].float()
    ref = orc.ffn_block(f("O2"), f("WFF1b"), f("WFF1a"), f("WFF2"), wo=f("WO"), residual=f("X"), norm=True, norm_weight=f("g"), norm_eps=1e-5)
    close(ff2, ref["FF2"], rtol=3e-2, atol=3e-2 * float(ref["FF2"].abs().max()), msg="FF2")


def _layer_case(B, S, N, Hq, Hkv, D, P, inner, dt, flags):
    g = torch.Generator().manual_seed(11)
    rn = lambda *s: torch.randn(*s, generator=g)
    t = dict(x=rn(B, S, N), wq=rn(N, Hq * D) * 0.02, wk=rn(N, Hkv * D) * 0.02, wv=rn(N, Hkv * D) * 0.02,
             kc=rn(B, Hkv, P + S, D), vc=rn(B, Hkv, P + S, D), wo=rn(N, N) * 0.02, nw=1 + 0.02 * rn(N),
             wg=rn(N, inner) * 0.02, wu=rn(N, inner) * 0.02, wd=rn(inner, N) * 0.02)
    return {k: v.to(dt).to(dev()) for k, v in t.items()}


@pytest.mark.parametrize("B,S,N,Hq,Hkv,D,P,inner,dt", [
    (1, 16, 1024, 8, 2, 128, 1000, 2816, torch.float16),      # decode-sized: sliced projections, one-kernel attention
    (2, 200, 512, 8, 8, 64, 56, 1408, torch.bfloat16),        # prefill-sized: tile-parallel projections
])
def test_layer_call_equals_the_two_block_calls(B, S, N, Hq, Hkv, D, P, inner, dt):
    """tb200_layer_forward = tb200_attn_forward + tb200_ffn_forward, bit for bit, with chained launches on and off, in
    eager mode and replayed from a CUDA graph; and the pair agrees with the oracle."""
    lib = L.load()
    flags = L.ATTN_CAUSAL | L.ATTN_PRENORM
    t = _layer_case(B, S, N, Hq, Hkv, D, P, inner, dt, flags)

    def buffers():
        return dict(kc=t["kc"].clone(), vc=t["vc"].clone(), o2=torch.full((B, S, N), float("nan"), dtype=dt, device=dev()),
                    ff2=torch.full((B * S, N), float("nan"), dtype=dt, device=dev()))

    def attn_kw(b):
        return dict(tensors=(t["x"], t["wq"], t["wk"], t["wv"], b["kc"], b["vc"], b["o2"]), past=P, head_dim=D, flags=flags,
                    sm_scale=D ** -0.5, norm_weight=t["nw"], norm_eps=1e-5)

    def ffn_kw(b):
        return dict(tensors=(t["x"].view(B * S, N), t["wg"], t["wu"], t["wd"], b["ff2"]), act=L.FFN_SWIGLU, flags=L.FFN_NORM,
                    o2=b["o2"].view(B * S, N), wo=t["wo"], norm_weight=t["nw"], norm_eps=1e-5)

    def separate(b):
        a, f = attn_kw(b), ffn_kw(b)
        ops.attn_forward(*a.pop("tensors"), **a)
        ops.ffn_forward(*f.pop("tensors"), **f)

    results = []
    try:
        for chained in (0, 1):
            lib.tb200_set_chained_launch(chained)
            for run in (separate, lambda b: ops.layer_forward(attn_kw(b), ffn_kw(b))):
                b = buffers()
                run(b)
                assert ops.device_status() == 0
                results.append(b)
        lib.tb200_set_chained_launch(1)
        b = buffers()
        ops.layer_forward(attn_kw(b), ffn_kw(b))          # warm-up: workspaces and folded weights exist before capture
        torch.cuda.synchronize()
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                ops.layer_forward(attn_kw(b), ffn_kw(b))
        for name in ("o2", "ff2"):
            b[name].fill_(float("nan"))
        b["kc"].copy_(t["kc"]); b["vc"].copy_(t["vc"])
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        results.append(b)
    finally:
        lib.tb200_set_chained_launch(1)
    first = results[0]
    for other in results[1:]:
        for name in ("o2", "ff2", "kc", "vc"):
            assert torch.equal(first[name], other[name]), f"{name} differs between the ways of launching the same work"
    # against the oracle: the attention block, then the FFN block on its output
    f32 = lambda v: v.float().cpu()
    ref_a = orc.attention_block(f32(t["x"]), f32(t["wq"]), f32(t["wk"]), f32(t["wv"]), f32(t["kc"]), f32(t["vc"]), past=P, head_dim=D,
                                prenorm=True, norm_weight=f32(t["nw"]), norm_eps=1e-5, causal=True, sm_scale=D ** -0.5)
    close(first["o2"], ref_a["O2"], msg="O2 of the layer call")
    ref_f = orc.ffn_block(f32(first["o2"]).view(B * S, N), f32(t["wg"]), f32(t["wu"]), f32(t["wd"]), wo=f32(t["wo"]),
                          residual=f32(t["x"]).view(B * S, N), norm=True, norm_weight=f32(t["nw"]), norm_eps=1e-5)
    close(first["ff2"], ref_f["FF2"], msg="FF2 of the layer call")


def test_layer_call_refuses_blocks_that_do_not_fit_together():
    lib = L.load()
    t = _layer_case(1, 16, 256, 2, 2, 128, 0, 512, torch.bfloat16, 0)
    o2 = torch.empty(1, 16, 256, dtype=torch.bfloat16, device=dev())
    other = torch.empty(16, 256, dtype=torch.bfloat16, device=dev())
    ff2 = torch.empty(16, 256, dtype=torch.bfloat16, device=dev())
    attn = dict(tensors=(t["x"], t["wq"], t["wk"], t["wv"], t["kc"], t["vc"], o2), past=0, head_dim=128)
    with pytest.raises(L.Tb200Error):      # the FFN reads another tensor than the attention block writes
        ops.layer_forward(attn, dict(tensors=(t["x"].view(16, 256), t["wg"], t["wu"], t["wd"], ff2), o2=other, wo=t["wo"]))
    with pytest.raises(L.Tb200Error):      # an FFN without the output projection does not consume o2 at all
        ops.layer_forward(attn, dict(tensors=(t["x"].view(16, 256), t["wg"], t["wu"], t["wd"], ff2)))
    assert ops.device_status() == 0
