"""Parity at the shapes the benchmark numbers are quoted on: every configuration of the benchmark runs at its OWN
geometry on the GPU (full batch, full sequence length, BASELINE's input distributions: x ~ N(0,1), weights ~ N(0,0.02),
norm weights 1 + N(0,0.02)), and the fp32 oracle is evaluated on a sample of it -- a few (sequence, q head) pairs, which
the block computes independently of all others -- so that the CPU side stays within seconds.  What is compared per
sample: the head's slice of O2, the appended K / V rows of its KV head, the per-key outputs, and the top-k indices
(bit-exact against a stable sort of the scores the kernel emitted).  The reference's own end-to-end check is the
same comparison of O2 against its eager class (convert_eval_rms.py:386-414)."""
import pytest
import torch

from oracle import oracle as orc
from trinity_b200 import _lib as L
from trinity_b200 import ops
from trinity_b200.codegen import convert_ir_to_triton

from .gpu_util import RTOL, ATOL, close, close_but_for_rounding_outliers, dev

pytestmark = pytest.mark.gpu

C, Pn, Q, KF, RC = L.ATTN_CAUSAL, L.ATTN_PRENORM, L.ATTN_QKNORM, L.ATTN_KEYFORMER, L.ATTN_ROCO
BF = torch.bfloat16


def oracle_on_heads(t, b, heads, Hq, Hkv, D, *, flags, noise=None, tau=1.0, roco_stats=False):
    """The oracle on sequence ``b`` restricted to the q heads ``heads``: the weights' columns of those heads (and of
    their KV heads) are cut out, which turns the block into an MHA block with len(heads) heads -- the same arithmetic
    the full block does for them."""
    group = Hq // Hkv
    qcols = torch.cat([torch.arange(h * D, (h + 1) * D) for h in heads])
    kcols = torch.cat([torch.arange((h // group) * D, (h // group + 1) * D) for h in heads])
    S = t["X"].shape[1]
    f = lambda v: v.float()
    kw = {}
    if flags & Pn:
        kw.update(prenorm=True, norm_weight=f(t["norm_weight"]), norm_eps=1e-5)
    if flags & Q:
        kw.update(qknorm=True, q_norm_weight=f(t["q_norm_weight"]), k_norm_weight=f(t["k_norm_weight"]), qk_eps=1e-6)
    z = torch.zeros(len(heads), S, D)
    return orc.attention_block(f(t["X"][b]), f(t["WQ"][:, qcols]), f(t["WK"][:, kcols]), f(t["WV"][:, kcols]), z, z, past=0,
                               head_dim=D, causal=True, sm_scale=D ** -0.5, noise=None if noise is None else noise.float(), tau=tau,
                               roco=bool(flags & RC), **kw)


def run_block(B, S, N, Hq, Hkv, D, flags, *, topk=0, samples, through_module=True, roco_variance=False):
    t = orc.bench_attention_inputs(B, S, N, Hq, Hkv, D, seed=0, norm_weights=bool(flags & (Pn | Q)))
    t = {k: v.to(BF) for k, v in t.items()}
    g = {k: v.to(dev()) for k, v in t.items()}
    kc = torch.zeros(B, Hkv, S, D, dtype=BF, device=dev())
    vc = torch.zeros_like(kc)
    o2 = torch.full((B, S, Hq * D), float("nan"), dtype=BF, device=dev())
    named = {"X": g["X"], "WQ": g["WQ"], "WK": g["WK"], "WV": g["WV"], "K_cache": kc, "V_cache": vc, "O2": o2}
    extra = {}
    if flags & Pn:
        extra["norm_weight"] = g["norm_weight"]
    if flags & Q:
        extra.update(q_norm_weight=g["q_norm_weight"], k_norm_weight=g["k_norm_weight"])
    noise = None
    if flags & KF:   # Gumbel(0,1) noise made on the device (gigabytes at these shapes); the sampled heads' slices go to the oracle
        gen = torch.Generator(device=dev()).manual_seed(5)
        noise = torch.empty(B, Hq, S, S, dtype=BF, device=dev())
        for b in range(B):
            u = torch.rand(Hq, S, S, generator=gen, device=dev()).clamp_(1e-9, 1 - 1e-9)
            noise[b] = (-torch.log(-torch.log(u))).to(BF)
            del u
        named.update(noise=noise, C_out=torch.full((B, Hq, S), float("nan"), device=dev()))
    if flags & RC:
        named.update(C_out1=torch.full((B, Hq, S), float("nan"), device=dev()), C_out2=torch.full((B, Hq, S), float("nan"), device=dev()))
    if topk:
        extra["topk_idx"] = torch.full((B, Hq, topk), -1, dtype=torch.int32, device=dev())
    # the block runs through the generated module, as a user of the reference's operator API would call it
    kind = {0: "vanilla", Pn: "prenorm", Q: "qknorm", KF: "keyformer", RC: "roco"}[flags & ~C]
    ir = {"vanilla": "(store (output O2) (* (load (input X) (index fulltile)) (load (input WQ,WK,WV) (index fulltile))) (index fulltile))",
          "prenorm": "(seq (store (tensor X2) (rsum (sqr (load (input X) (index fulltile))) 1) (index fulltile)) (store (output O2) (* (load (input X) (index fulltile)) (load (input WQ,WK,WV) (index fulltile))) (index fulltile)))",
          "qknorm": "(seq (store (tensor Q_norm,K_norm) (load (input X) (index fulltile)) (index fulltile)) (store (output O2) (* (load (input X) (index fulltile)) (load (input WQ,WK,WV) (index fulltile))) (index fulltile)))",
          "keyformer": "(seq (store (output C_out) (load (input noise) (index fulltile)) (index fulltile)) (store (output O2) (* (load (input X) (index fulltile)) (load (input WQ,WK,WV) (index fulltile))) (index fulltile)))",
          "roco": "(seq (store (output C_out1) (load (input X) (index fulltile)) (index fulltile)) (seq (store (output C_out2) (load (input X) (index fulltile)) (index fulltile)) (store (output O2) (* (load (input X) (index fulltile)) (load (input WQ,WK,WV) (index fulltile))) (index fulltile))))"}[kind]
    ir = "(ploop 0 %d %d n (seq (store (input K_cache,V_cache) (load (input X) (index fulltile)) (index fulltile)) %s))" % (N, D, ir)
    constants = {"M": S, "D": D, "N": N, "P": 0, "H": Hq, "H_KV": Hkv, "CAUSAL": 1, "SM_SCALE": D ** -0.5, "NORM_EPS": 1e-5,
                 "QK_EPS": 1e-6, "TAU": 1.0, "TOPK": topk, "ROCO_VARIANCE": int(roco_variance)}
    ns = {}
    exec(compile(convert_ir_to_triton(ir, None, constants), "<generated module>", "exec"), ns)
    assert ns["KIND"] == kind, (ns["KIND"], kind)
    ns["forward"](*[named[p] for p in ns["TENSOR_PARAMS"]], **extra)
    ops.device_status()
    group = Hq // Hkv
    for b, heads in samples:
        nz = None if noise is None else noise[b, heads].cpu()
        ref = oracle_on_heads(t, b, heads, Hq, Hkv, D, flags=flags, noise=nz)
        for i, h in enumerate(heads):
            close_but_for_rounding_outliers(o2[b, :, h * D:(h + 1) * D], ref["O2"][:, i * D:(i + 1) * D], msg=f"O2 of sequence {b}, head {h}")
            close(kc[b, h // group], ref["K_new"][i], msg=f"appended K rows, sequence {b}, kv head {h // group}")
            close(vc[b, h // group], ref["V_new"][i], msg=f"appended V rows, sequence {b}, kv head {h // group}")
            if flags & KF:
                close(named["C_out"][b, h], ref["C_out"][i], msg=f"C_out of sequence {b}, head {h}")
            if flags & RC:
                close(named["C_out1"][b, h], ref["C_out1"][i], msg=f"C_out1 of sequence {b}, head {h}")
                if roco_variance:
                    close(named["C_out2"][b, h], ref["col_var"][i], rtol=RTOL, atol=1e-4, msg=f"column variance, sequence {b}, head {h}")
                else:
                    close(named["C_out2"][b, h], ref["C_out2"][i], msg=f"C_out2 of sequence {b}, head {h}")
    assert not torch.isnan(o2.float()).any(), "a part of O2 was never written"
    if topk:
        key = named["C_out"] if flags & KF else named["C_out1"]
        assert torch.equal(extra["topk_idx"].cpu(), orc.stable_topk(key.cpu(), topk)), "top-k differs from a stable sort of the emitted scores"
        close(key.sum(-1), torch.full((B, Hq), float(S)), rtol=1e-3, atol=0.5, msg="per-key scores add up to the number of queries")


def test_config2_llama_qknorm_prefill_b8_s2048():
    run_block(8, 2048, 4096, 32, 8, 128, C | Q, samples=[(0, [0, 21]), (7, [31])])


def test_config2_llama_vanilla_prefill_b8_s2048():
    run_block(8, 2048, 4096, 32, 8, 128, C, samples=[(3, [5]), (7, [30])])


def test_config3_llama_prenorm_b8_s4096():
    run_block(8, 4096, 4096, 32, 8, 128, C | Pn, samples=[(0, [0]), (7, [17, 31])])


@pytest.mark.parametrize("variance", [False, True])
def test_config4_llama_roco_b4_s4096(variance):
    run_block(4, 4096, 4096, 32, 8, 128, C | RC, topk=1024, samples=[(1, [2]), (3, [29])], roco_variance=variance)


def test_config4_llama_keyformer_b4_s4096():
    run_block(4, 4096, 4096, 32, 8, 128, C | KF, topk=1024, samples=[(0, [9]), (3, [31])])


@pytest.mark.parametrize("flags,topk", [(C, 0), (C | Pn, 0), (C | Q, 0), (C | RC, 1024), (C | KF, 1024)])
def test_config5_falcon_b16_s2048(flags, topk):
    run_block(16, 2048, 4544, 71, 1, 64, flags, topk=topk, samples=[(0, [0, 70]), (15, [35])])


def test_config5_falcon_gelu_ffn_32768_tokens():
    """GELU MLP 4544 -> 18176 -> 4544 on 16 x 2048 tokens; rows are independent, the oracle takes 96 of them."""
    M, N, P = 32768, 4544, 18176
    t = {k: v.to(BF) for k, v in orc.bench_ffn_inputs(M, N, P, seed=0, gated=False).items()}
    g = {k: v.to(dev()) for k, v in t.items()}
    ff2 = torch.full((M, N), float("nan"), dtype=BF, device=dev())
    ops.ffn_forward(g["X"], g["W_gate"], None, g["W_down"], ff2, act=L.FFN_GELU)
    ops.device_status()
    rows = torch.cat([torch.arange(0, 32), torch.arange(16000, 16032), torch.arange(M - 32, M)])
    ref = orc.ffn_block(t["X"][rows].float(), t["W_gate"].float(), None, t["W_down"].float(), act="gelu")["FF2"]
    close(ff2[rows.to(dev())], ref, msg="FF2 rows")
    assert not torch.isnan(ff2.float()).any()


def test_config1_llama_swiglu_ffn_m64_fp16():
    """Plain SwiGLU 4096 / 14336 on 64 tokens in fp16 (the configuration the reference itself can run on a CPU)."""
    M, N, P = 64, 4096, 14336
    t = {k: v.to(torch.float16) for k, v in orc.bench_ffn_inputs(M, N, P, seed=0, gated=True).items()}
    g = {k: v.to(dev()) for k, v in t.items()}
    ff2 = torch.full((M, N), float("nan"), dtype=torch.float16, device=dev())
    ops.ffn_forward(g["X"], g["W_gate"], g["W_up"], g["W_down"], ff2, act=L.FFN_SWIGLU)
    ops.device_status()
    ref = orc.ffn_block(t["X"].float(), t["W_gate"].float(), t["W_up"].float(), t["W_down"].float(), act="swiglu")["FF2"]
    close(ff2, ref, msg="FF2")
