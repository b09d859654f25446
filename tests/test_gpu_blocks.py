"""Parity of the fused blocks: C ABI / generated module on the GPU against the oracle and against the
golden vectors made from the reference's own eager classes."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import ATOL, RTOL, attention_case, close, dev, close_but_for_rounding_outliers
from tests.test_codegen import FFN, KEYFORMER, PRENORM, ROCO, VANILLA

pytestmark = pytest.mark.gpu

from trinity_b200 import _lib as L  # noqa: E402

C, Pn, Q, KF, RC = L.ATTN_CAUSAL, L.ATTN_PRENORM, L.ATTN_QKNORM, L.ATTN_KEYFORMER, L.ATTN_ROCO


def check_common(got, ref, P):
    close(got["K_new"], ref["K_new"], msg="appended K rows")
    close(got["V_new"], ref["V_new"], msg="appended V rows")
    close(got["O2"], ref["O2"], msg="O2")
    # rows before `past` (and after past+S) of the caches are untouched
    assert torch.equal(got["K_cache"][:, :, :P].cpu(), got["K_cache_in"][:, :, :P])
    S = ref["O2"].shape[-2]
    assert torch.equal(got["V_cache"][:, :, P + S:].cpu(), got["V_cache_in"][:, :, P + S:])


@pytest.mark.parametrize("B,S,N,Hq,Hkv,D,P,flags,kw", [
    (1, 128, 256, 2, 2, 128, 0, 0, {}),
    (1, 16, 256, 2, 2, 128, 112, 0, {}),                         # decode shape: 16 new tokens on a cache
    (1, 16, 512, 8, 8, 64, 1024, 0, dict(dt=torch.float16)),     # the reference's Falcon-like point, fp16
    (1, 1, 256, 2, 1, 128, 0, 0, {}),                            # a single token, empty cache
    (1, 17, 256, 4, 2, 64, 1, C, {}),
    (2, 384, 512, 4, 2, 128, 0, C, {}),                          # GQA, causal, 3 tiles
    (2, 300, 512, 8, 1, 64, 37, C | Pn | Q, dict(weights=True)),  # MQA, ragged tails, all norms with weights
    (1, 200, 256, 2, 2, 128, 56, Pn, {}),                        # PreNorm reference point (no weight)
    (1, 130, 256, 2, 2, 128, 0, Q, {}),                          # QKNorm reference point
    (3, 129, 264, 3, 3, 64, 255, C | Q, dict(weights=True, cache_extra=40)),
    # decode-sized query blocks: the one-kernel path (K-slice sums finished in the kernel when the projection is sliced,
    # key shares merged inside a cluster)
    (2, 16, 512, 8, 2, 128, 1000, C, {}),                        # GQA, causal on a long cache, ragged last tile
    (1, 5, 256, 4, 4, 64, 63, C, dict(dt=torch.float16)),        # 5 tokens, the diagonal crosses a tile boundary
    (1, 16, 256, 4, 1, 64, 3, C | Pn | Q, dict(weights=True)),   # MQA, nearly empty cache, all norms
    (1, 1, 256, 2, 2, 128, 777, 0, dict(cache_extra=9)),         # one token, many shares
    (40, 3, 256, 16, 4, 128, 70, C, {}),                         # 640 heads in flight: one share per head, no merge
    (2, 9, 512, 4, 2, 128, 0, C, {}),                            # no cache at all
    (2, 16, 512, 8, 2, 128, 1000, C | Pn | Q, dict(weights=True)),   # sliced projection: q, k finished and normalised in the attention kernel
    (1, 13, 1024, 4, 4, 64, 300, Q, dict(weights=True, dt=torch.float16)),
    (3, 16, 512, 4, 1, 128, 2049, 0, dict(cache_extra=5)),       # MQA: four q heads share the appended rows; 8 shares of 257 keys
])
def test_attention_variants(B, S, N, Hq, Hkv, D, P, flags, kw):
    got, ref = attention_case(B, S, N, Hq, Hkv, D, P, flags, **kw)
    check_common(got, ref, P)


@pytest.mark.parametrize("B,S,N,Hq,Hkv,D,P,flags,kw", [
    (1, 256, 256, 4, 2, 128, 0, C | RC, dict(topk=64)),
    (1, 16, 256, 2, 2, 128, 240, RC, dict(topk=32)),
    (2, 200, 256, 4, 1, 64, 72, C | RC | Pn, dict(topk=100, weights=True)),
    (2, 256, 256, 4, 4, 64, 0, C | KF, dict(topk=64)),
    (1, 16, 256, 2, 2, 128, 240, KF, dict(tau=1.5, topk=32)),
    (1, 140, 256, 2, 2, 128, 20, C | KF | Q, dict(tau=1.0, topk=16, aux_dtype=torch.bfloat16)),
    (1, 131, 256, 2, 2, 64, 5, KF, dict(tau=1.5)),               # past+S not a multiple of 8
    (2, 12, 256, 8, 2, 128, 500, C | RC, dict(topk=50)),         # RoCo on a decode-sized block: its row statistic comes out of the merge of the key shares
])
def test_score_outputs_and_topk(B, S, N, Hq, Hkv, D, P, flags, kw):
    got, ref = attention_case(B, S, N, Hq, Hkv, D, P, flags, **kw)
    check_common(got, ref, P)
    for name in ("C_out", "C_out1", "C_out2"):
        if got[name] is not None:
            close(got[name], ref[name], msg=name)
    if flags & RC:   # a row-stochastic matrix: the column sums add up to the number of queries
        close(got["C_out1"].float().sum(-1), torch.full((B, Hq), float(S)), rtol=1e-3, atol=1e-2, msg="sum of column sums")
    if kw.get("topk") and kw.get("aux_dtype", torch.float32) == torch.float32:
        key = got["C_out"] if got["C_out"] is not None else got["C_out1"]
        assert torch.equal(got["topk_idx"].cpu(), orc.stable_topk(key.cpu(), kw["topk"])), "indices != stable sort of the emitted scores"


def test_attention_is_deterministic_and_overwrites():
    a, _ = attention_case(1, 200, 256, 4, 2, 128, 8, C | RC, topk=16, seed=9)
    b, _ = attention_case(1, 200, 256, 4, 2, 128, 8, C | RC, topk=16, seed=9)
    for name in ("O2", "C_out1", "C_out2", "topk_idx"):
        assert torch.equal(a[name], b[name]), name
    assert not torch.isnan(a["O2"].float()).any()


def test_attention_rejects_bad_arguments():
    from trinity_b200 import ops
    from trinity_b200._lib import Tb200Error
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev())
    with pytest.raises(Tb200Error):      # head_dim 32 has no kernel
        ops.attn_forward(z(4, 64), z(64, 64), z(64, 64), z(64, 64), z(2, 4, 32), z(2, 4, 32), z(4, 64), past=0, head_dim=32)
    with pytest.raises(Tb200Error):      # cache shorter than past + seq
        ops.attn_forward(z(4, 128), z(128, 128), z(128, 128), z(128, 128), z(2, 4, 64), z(2, 4, 64), z(4, 128), past=8, head_dim=64)
    with pytest.raises(ValueError):      # non-contiguous input
        ops.attn_forward(z(128, 4).t(), z(128, 128), z(128, 128), z(128, 128), z(2, 4, 64), z(2, 4, 64), z(4, 128), past=0, head_dim=64)


# ------------------------------------------------------------------ golden vectors through the generated module
def load_module(ir_text, constants):
    from trinity_b200.codegen import convert_ir_to_triton
    ns = {}
    exec(compile(convert_ir_to_triton(ir_text, None, constants), "<module>", "exec"), ns)
    return ns


CLASS_IR = {"Vanilla": VANILLA, "PreNorm": PRENORM, "KeyFormer": KEYFORMER, "RoCo": ROCO}


def run_module_attention(cls, inp, M, N, D, P, dt):
    """Call a generated module the way the reference harness does: positional tensors in TENSOR_PARAMS order, then
    the block sizes (convert_eval_rms.py:240-250)."""
    H = N // D
    m = load_module(CLASS_IR[cls], {"M": M, "D": D, "N": N, "P": P, "H": H})
    t = {k: v.to(dt).to(dev()) for k, v in inp.items()}
    t["O2"] = torch.zeros(M, N, dtype=dt, device=dev())
    for name in ("C_out", "C_out1", "C_out2"):
        t[name] = torch.zeros(H, P + M, dtype=dt, device=dev())
    args = [t[p] for p in m["TENSOR_PARAMS"]] + [32, 16][: len(m["BLOCK_PARAMS"])]
    assert m["forward"](*args) is None
    from trinity_b200 import ops
    ops.device_status()
    return t


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_small_golden_through_generated_module(golden_dir, tag):
    z = np.load(os.path.join(golden_dir, f"small_attn_{tag}.npz"))
    M, N, D, P = (int(v) for v in z["shape"])
    inp = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in_")}
    for cls in CLASS_IR:
        t = run_module_attention(cls, inp, M, N, D, P, torch.float16)
        close(t["O2"], torch.from_numpy(z[f"{cls}.O2"]), msg=f"{cls}.O2")
        for name in ("C_out", "C_out1", "C_out2"):
            if f"{cls}.{name}" in z.files:
                close(t[name], torch.from_numpy(z[f"{cls}.{name}"]), msg=f"{cls}.{name}")
        # the cache-append side effect of the emitted kernels (evaluation/vanilla/vanilla_falcon_benchmark28173.py:96-99)
        assert not torch.equal(t["K_cache"][:, P:].cpu(), inp["K_cache"][:, P:].to(torch.float16))


@pytest.mark.parametrize("model", ["llama", "falcon"])
def test_reference_shapes_against_golden(golden_dir, model):
    """The reference's own shapes (M16, P1024; Llama N4096 D128, Falcon N4544 D64) and its input distribution (seed 42,
    randn*0.01, fp16).  Tolerance: rtol 2e-2 with atol 2e-2 of the output's range -- the 16-bit-vs-fp32 bound, scaled
    because the un-normalised variants produce outputs of magnitude 0.006 at this input scale, for which the
    reference's own absolute 2e-3 (convert_eval_rms.py:387) would accept anything, while the PreNorm variants produce
    O(1) outputs for which the reference's own Triton path misses that same 2e-3."""
    from tests.golden.make_golden import fingerprint
    z = np.load(os.path.join(golden_dir, f"refshape_attn_{model}.npz"))
    M, N, D, P = (int(v) for v in z["shape"])
    inp = orc.ref_attention_inputs(M, N, D, P, seed=42)
    if not np.allclose(fingerprint(inp), z["fingerprint"], rtol=0, atol=0):
        pytest.skip("this torch build seeds different inputs than the one that made the fixture")
    from trinity_b200 import ops
    flagmap = {"Vanilla": 0, "PreNorm": Pn, "NormKeyFormer": Pn | KF, "KeyFormer": KF, "NormQKNorm": Pn | Q, "RoCo": RC}
    for cls in sorted({k.split(".")[0] for k in z.files if "." in k}):
        flags = flagmap[cls]
        t = {k: v.to(torch.float16).to(dev()) for k, v in inp.items()}
        H = N // D
        o2 = torch.zeros(M, N, dtype=torch.float16, device=dev())
        aux = {n: torch.zeros(H, P + M, dtype=torch.float32, device=dev()) for n in ("c_out", "c_out1", "c_out2")}
        ops.attn_forward(t["X"], t["WQ"], t["WK"], t["WV"], t["K_cache"], t["V_cache"], o2, past=P, head_dim=D, flags=flags,
                         sm_scale=1.0, tau=1.5, noise=t["noise"] if flags & KF else None,
                         c_out=aux["c_out"] if flags & KF else None, c_out1=aux["c_out1"] if flags & RC else None,
                         c_out2=aux["c_out2"] if flags & RC else None)
        ops.device_status()
        want = torch.from_numpy(z[f"{cls}.O2"])
        close(o2, want, rtol=2e-2, atol=2e-2 * float(want.abs().max()), msg=f"{cls}.O2")
        for name, key in (("C_out", "c_out"), ("C_out1", "c_out1"), ("C_out2", "c_out2")):
            if f"{cls}.{name}" in z.files:
                want = torch.from_numpy(z[f"{cls}.{name}"])
                close(aux[key], want, rtol=2e-2, atol=2e-2 * float(want.abs().max()), msg=f"{cls}.{name}")


# ------------------------------------------------------------------ FFN
def run_ffn(inp, dt, kind="ffn_llama"):
    M, N = inp["X"].shape
    P = inp["WFF1a"].shape[1]
    m = load_module(FFN if kind == "ffn_llama" else FFN.replace("(output FF2)", "(output O_FF_norm)"), {"M": M, "N": N, "P": P})
    t = {k: v.to(dt).to(dev()) for k, v in inp.items()}
    t.update(FF1=torch.zeros(M, P, dtype=dt, device=dev()), FF2=torch.zeros(M, N, dtype=dt, device=dev()),
             attn_O2=torch.zeros(M, N, dtype=dt, device=dev()), O_FF_norm=torch.zeros(M, N, dtype=dt, device=dev()))
    m["forward"](*[t[p] for p in m["TENSOR_PARAMS"]])
    from trinity_b200 import ops
    ops.device_status()
    return t


@pytest.mark.parametrize("tag", ["a", "b"])
def test_small_ffn_golden(golden_dir, tag):
    z = np.load(os.path.join(golden_dir, f"small_ffn_{tag}.npz"))
    inp = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in_")}
    t = run_ffn(inp, torch.bfloat16)
    ref = torch.from_numpy(z["SimpleFFN.FF2"])
    close(t["FF2"], ref, rtol=3e-2, atol=3e-2 * float(ref.abs().max()), msg="FF2")
    want = orc.ffn_block(inp["O2"], inp["WFF1b"], inp["WFF1a"], inp["WFF2"], wo=inp["WO"], residual=inp["X"], norm=True)
    close(t["attn_O2"], want["attn_O2"], msg="attn_O2")


def test_ffn_reference_shape_golden(golden_dir):
    """Llama FFN block at the reference's shape and input scale (convert_ffn_llama.py:86-99: randn.clamp*0.001, fp16)."""
    from tests.golden.make_golden import fingerprint
    z = np.load(os.path.join(golden_dir, "refshape_ffn_llama.npz"))
    M, N, P = (int(v) for v in z["shape"])
    inp = orc.ref_ffn_inputs(M, N, P, seed=42)
    if not np.allclose(fingerprint(inp), z["fingerprint"], rtol=0, atol=0):
        pytest.skip("this torch build seeds different inputs than the one that made the fixture")
    t = run_ffn(inp, torch.float16)
    ref = torch.from_numpy(z["SimpleFFN.FF2"])
    close(t["FF2"], ref, rtol=2e-2, atol=2e-2 * float(ref.abs().max()), msg="FF2")


def test_falcon_tail_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "small_ffn_falcon_tail.npz"))
    inp = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in_")}
    from trinity_b200 import ops
    dt = torch.bfloat16
    t = {k: v.to(dt).to(dev()) for k, v in inp.items()}
    M, N = inp["X"].shape
    ff2 = torch.zeros(M, N, dtype=dt, device=dev())
    out = torch.zeros(M, N, dtype=dt, device=dev())
    ops.ffn_forward(t["X"], t["WFF1b"], t["WFF1a"], t["WFF2"], ff2, flags=L.FFN_NORM | L.FFN_FALCON_TAIL, o2=t["O2"], wo=t["WO"],
                    tail_divisor=4544, o_ff_norm=out)
    ops.device_status()
    ref = torch.from_numpy(z["FalconTail.O_FF_norm"])
    close(out, ref, rtol=3e-2, atol=3e-2 * float(ref.abs().max()), msg="O_FF_norm")


@pytest.mark.parametrize("M,N,P,act,dt", [
    (64, 512, 1536, L.FFN_SWIGLU, torch.float16),      # weight-streaming regime (K split)
    (700, 520, 1032, L.FFN_SWIGLU, torch.bfloat16),    # large-M regime, ragged tiles
    (300, 584, 2336, L.FFN_GELU, torch.bfloat16),      # GELU MLP (Falcon-style 4x), unpinned in the reference
    (16, 584, 2336, L.FFN_GELU, torch.bfloat16),
])
def test_plain_mlp(M, N, P, act, dt):
    from trinity_b200 import ops
    t = orc.bench_ffn_inputs(M, N, P, seed=3, gated=act == L.FFN_SWIGLU)
    t = {k: v.to(dt) for k, v in t.items()}
    ff2 = torch.full((M, N), float("nan"), dtype=dt, device=dev())
    g = {k: v.to(dev()) for k, v in t.items()}
    ops.ffn_forward(g["X"], g["W_gate"], g.get("W_up"), g["W_down"], ff2, act=act)
    ops.device_status()
    ref = orc.ffn_block(t["X"].float(), t["W_gate"].float(), t["W_up"].float() if "W_up" in t else None, t["W_down"].float(),
                        act="swiglu" if act == L.FFN_SWIGLU else "gelu")["FF2"]
    close(ff2, ref, msg="FF2")


# ------------------------------------------------------------------ full-size checks by properties and samples
def test_full_size_prefill_properties():
    """Llama-3-8B prefill, batch 2 of the benchmark's 8, seq 2048: sequence 0 against the oracle, plus properties
    that need no oracle: batch independence and the RoCo column-sum identity."""
    from trinity_b200 import ops
    B, S, N, Hq, Hkv, D = 2, 2048, 4096, 32, 8, 128
    t = orc.bench_attention_inputs(B, S, N, Hq, Hkv, D, seed=0)
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    g = {k: v.to(dev()) for k, v in t.items()}
    kc = torch.zeros(B, Hkv, S, D, dtype=torch.bfloat16, device=dev())
    vc = torch.zeros_like(kc)
    o2 = torch.zeros(B, S, Hq * D, dtype=torch.bfloat16, device=dev())
    c1 = torch.zeros(B, Hq, S, dtype=torch.float32, device=dev())
    c2 = torch.zeros_like(c1)
    idx = torch.zeros(B, Hq, 1024, dtype=torch.int32, device=dev())
    ops.attn_forward(g["X"], g["WQ"], g["WK"], g["WV"], kc, vc, o2, past=0, head_dim=D, flags=C | RC, sm_scale=D ** -0.5,
                     c_out1=c1, c_out2=c2, topk=1024, topk_idx=idx)
    ops.device_status()
    ref = orc.attention_block(t["X"][:1].float(), t["WQ"].float(), t["WK"].float(), t["WV"].float(),
                              torch.zeros(1, Hkv, S, D), torch.zeros(1, Hkv, S, D), past=0, head_dim=D, causal=True,
                              sm_scale=D ** -0.5, roco=True)
    close(o2[:1], ref["O2"], msg="O2 of sequence 0")
    close(c1[:1], ref["C_out1"], msg="C_out1 of sequence 0")
    close(c1.sum(-1), torch.full((B, Hq), float(S)), rtol=1e-3, atol=0.5, msg="column sums add up to S")
    assert torch.equal(idx.cpu(), orc.stable_topk(c1.cpu(), 1024))
    # batch independence: sequence 1 alone gives the same bits as sequence 1 inside the batch
    o2b = torch.zeros(1, S, Hq * D, dtype=torch.bfloat16, device=dev())
    ops.attn_forward(g["X"][1:].contiguous(), g["WQ"], g["WK"], g["WV"], kc[1:].clone(), vc[1:].clone(), o2b, past=0,
                     head_dim=D, flags=C, sm_scale=D ** -0.5)
    assert torch.equal(o2b[0], o2[1])


def test_full_size_keyformer_properties():
    """Llama-3-8B KeyFormer, one sequence of the benchmark's batch at seq 2048 (256 work items for 148 persistent
    CTAs, a 268 MB noise tensor): everything against the oracle, plus the property that the per-key scores of a head add
    up to the number of queries (every perturbed softmax row sums to one)."""
    B, S, N, Hq, Hkv, D = 1, 2048, 4096, 32, 8, 128
    got, ref = attention_case(B, S, N, Hq, Hkv, D, 0, C | KF, topk=1024, tau=1.0, seed=7)
    close(got["O2"], ref["O2"], msg="O2")
    close(got["C_out"], ref["C_out"], msg="C_out")
    close(got["C_out"].sum(-1), torch.full((B, Hq), float(S)), rtol=1e-3, atol=0.5, msg="scores add up to S")
    assert torch.equal(got["topk_idx"].cpu(), orc.stable_topk(got["C_out"].float().cpu(), 1024))


@pytest.mark.parametrize("flags", [C | RC, C | KF, C | Pn | Q])
def test_falcon_shapes_multi_item(flags):
    """Falcon-7B geometry (hidden 4544, MQA 71/1, head_dim 64) at batch 2, seq 1024: 568 work items, so every
    persistent CTA walks several items of different lengths; against the oracle."""
    B, S, N, Hq, Hkv, D = 2, 1024, 4544, 71, 1, 64
    kw = dict(topk=256) if flags & (RC | KF) else dict(weights=True)
    got, ref = attention_case(B, S, N, Hq, Hkv, D, 0, flags, seed=11, **kw)
    close_but_for_rounding_outliers(got["O2"], ref["O2"], msg="O2")     # 9.3 million outputs
    close(got["K_new"], ref["K_new"], msg="appended K rows")
    if flags & RC:
        close(got["C_out1"], ref["C_out1"], msg="C_out1")
        close(got["C_out2"], ref["C_out2"], msg="C_out2")
        close(got["C_out1"].sum(-1), torch.full((B, Hq), float(S)), rtol=1e-3, atol=0.5, msg="column sums add up to S")
        assert torch.equal(got["topk_idx"].cpu(), orc.stable_topk(got["C_out1"].float().cpu(), 256))
    if flags & KF:
        close(got["C_out"], ref["C_out"], msg="C_out")
        close(got["C_out"].sum(-1), torch.full((B, Hq), float(S)), rtol=1e-3, atol=0.5, msg="scores add up to S")
        assert torch.equal(got["topk_idx"].cpu(), orc.stable_topk(got["C_out"].float().cpu(), 256))
