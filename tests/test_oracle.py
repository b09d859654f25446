"""The fp32 oracle against the golden vectors made from the reference's eager classes."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.golden.make_golden import fingerprint

# class name -> oracle keywords at the reference parameter point (MHA, no mask, scale 1, tau 1.5)
CLASS_KW = {
    "Vanilla": {},
    "PreNorm": {"prenorm": True},
    "KeyFormer": {"keyformer": True},
    "NormKeyFormer": {"prenorm": True, "keyformer": True},
    "QKNorm": {"qknorm": True},
    "NormQKNorm": {"prenorm": True, "qknorm": True},
    "RoCo": {"roco": True},
    "NormRoCo": {"prenorm": True, "roco": True},
}


def run_oracle(inp, D, P, kw):
    kw = dict(kw)
    noise = inp["noise"] if kw.pop("keyformer", False) else None
    return orc.attention_block(inp["X"], inp["WQ"], inp["WK"], inp["WV"], inp["K_cache"], inp["V_cache"],
                               past=P, head_dim=D, noise=noise, **kw)


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_small_attention_matches_reference_classes(golden_dir, tag):
    z = np.load(os.path.join(golden_dir, f"small_attn_{tag}.npz"))
    M, N, D, P = (int(v) for v in z["shape"])
    inp = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in_")}
    for cls, kw in CLASS_KW.items():
        got = run_oracle(inp, D, P, kw)
        for name in ("O2", "C_out", "C_out1", "C_out2"):
            key = f"{cls}.{name}"
            if key in z.files:
                torch.testing.assert_close(got[name], torch.from_numpy(z[key]), rtol=1e-5, atol=1e-6, msg=key)


@pytest.mark.parametrize("model", ["llama", "falcon"])
def test_refshape_attention_matches_reference_classes(golden_dir, model):
    z = np.load(os.path.join(golden_dir, f"refshape_attn_{model}.npz"))
    M, N, D, P = (int(v) for v in z["shape"])
    inp = orc.ref_attention_inputs(M, N, D, P, seed=42)
    if not np.allclose(fingerprint(inp), z["fingerprint"], rtol=0, atol=0):
        pytest.skip("this torch build seeds different inputs than the one that made the fixture")
    for cls in sorted({k.split(".")[0] for k in z.files if "." in k}):
        got = run_oracle(inp, D, P, CLASS_KW[cls])
        for name in ("O2", "C_out", "C_out1", "C_out2"):
            key = f"{cls}.{name}"
            if key in z.files:
                torch.testing.assert_close(got[name], torch.from_numpy(z[key]), rtol=1e-4, atol=1e-6, msg=key)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_small_ffn_matches_simpleffn(golden_dir, tag):
    z = np.load(os.path.join(golden_dir, f"small_ffn_{tag}.npz"))
    inp = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in_")}
    got = orc.ffn_block(inp["O2"], inp["WFF1b"], inp["WFF1a"], inp["WFF2"], wo=inp["WO"], residual=inp["X"], norm=True)
    torch.testing.assert_close(got["FF2"], torch.from_numpy(z["SimpleFFN.FF2"]), rtol=1e-5, atol=1e-6)


def test_falcon_tail_matches_reference_body(golden_dir):
    z = np.load(os.path.join(golden_dir, "small_ffn_falcon_tail.npz"))
    inp = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in_")}
    got = orc.ffn_block(inp["O2"], inp["WFF1b"], inp["WFF1a"], inp["WFF2"], wo=inp["WO"], residual=inp["X"],
                        norm=True, falcon_tail=True, tail_divisor=4544)
    torch.testing.assert_close(got["O_FF_norm"], torch.from_numpy(z["FalconTail.O_FF_norm"]), rtol=1e-5, atol=1e-6)


def test_refshape_ffn_matches_simpleffn(golden_dir):
    z = np.load(os.path.join(golden_dir, "refshape_ffn_llama.npz"))
    M, N, P = (int(v) for v in z["shape"])
    inp = orc.ref_ffn_inputs(M, N, P, seed=42)
    if not np.allclose(fingerprint(inp), z["fingerprint"], rtol=0, atol=0):
        pytest.skip("this torch build seeds different inputs than the one that made the fixture")
    got = orc.ffn_block(inp["O2"], inp["WFF1b"], inp["WFF1a"], inp["WFF2"], wo=inp["WO"], residual=inp["X"], norm=True)
    torch.testing.assert_close(got["FF2"], torch.from_numpy(z["SimpleFFN.FF2"]), rtol=1e-4, atol=1e-7)


def test_extensions_collapse_to_reference_point():
    """GQA with group 1, a causal mask that hides nothing, unit weights and zero eps change nothing."""
    inp = orc.ref_attention_inputs(6, 128, 32, 10, seed=1, std=0.3)
    base = run_oracle(inp, 32, 10, {"prenorm": True, "qknorm": True, "roco": True})
    ext = run_oracle(inp, 32, 10, {"prenorm": True, "qknorm": True, "roco": True, "norm_weight": torch.ones(128),
                                   "q_norm_weight": torch.ones(32), "k_norm_weight": torch.ones(32),
                                   "norm_eps": 0.0, "qk_eps": 0.0, "sm_scale": 1.0})
    for name in ("O2", "C_out1", "C_out2"):
        torch.testing.assert_close(base[name], ext[name], rtol=0, atol=0)
    # batch axis == stacking independent calls
    xb = torch.stack([inp["X"], inp["X"] * 0.5])
    kc = torch.stack([inp["K_cache"]] * 2)
    vc = torch.stack([inp["V_cache"]] * 2)
    outb = orc.attention_block(xb, inp["WQ"], inp["WK"], inp["WV"], kc, vc, past=10, head_dim=32, causal=True, sm_scale=0.5)
    out1 = orc.attention_block(xb[1], inp["WQ"], inp["WK"], inp["WV"], kc[1], vc[1], past=10, head_dim=32, causal=True, sm_scale=0.5)
    torch.testing.assert_close(outb["O2"][1], out1["O2"], rtol=1e-6, atol=1e-7)


def test_causal_and_gqa_against_naive():
    g = torch.Generator().manual_seed(3)
    S, N, D, Hq, Hkv, P = 9, 64, 16, 4, 2, 5
    x = torch.randn(S, N, generator=g)
    wq = torch.randn(N, Hq * D, generator=g) * 0.2
    wk = torch.randn(N, Hkv * D, generator=g) * 0.2
    wv = torch.randn(N, Hkv * D, generator=g) * 0.2
    kc = torch.randn(Hkv, P + S, D, generator=g)
    vc = torch.randn(Hkv, P + S, D, generator=g)
    out = orc.attention_block(x, wq, wk, wv, kc, vc, past=P, head_dim=D, causal=True, sm_scale=D ** -0.5, roco=True, topk=4)
    q = (x @ wq).view(S, Hq, D)
    k = torch.cat([kc[:, :P], (x @ wk).view(S, Hkv, D).transpose(0, 1)], 1)
    v = torch.cat([vc[:, :P], (x @ wv).view(S, Hkv, D).transpose(0, 1)], 1)
    for i in range(S):
        for h in range(Hq):
            s = (k[h // 2, : P + i + 1] @ q[i, h]) * D ** -0.5
            p = torch.softmax(s, 0)
            torch.testing.assert_close(out["O2"][i, h * D:(h + 1) * D], p @ v[h // 2, : P + i + 1], rtol=1e-5, atol=1e-6)
    assert out["topk_idx"].shape == (Hq, 4) and out["topk_idx"].dtype == torch.int32
    # column sums of a row-stochastic matrix add up to the number of queries
    torch.testing.assert_close(out["C_out1"].sum(-1), torch.full((Hq,), float(S)), rtol=1e-5, atol=1e-5)


def test_stable_topk_ties_prefer_lower_index():
    s = torch.tensor([[1.0, 3.0, 3.0, 0.5, 3.0, 1.0]])
    assert orc.stable_topk(s, 5).tolist() == [[1, 2, 4, 0, 5]]


def test_kv_compact_known_answer():
    """Hand-checked case: duplicates once, out-of-range entries ignored, recent window united, ascending order."""
    k = torch.arange(2 * 10 * 4, dtype=torch.float32).reshape(2, 10, 4)     # rows 0/1, 10 positions (8 valid), D 4
    v = -k
    idx = torch.tensor([[5, 1, 5, 9, -1], [0, 0, 0, 0, 0]], dtype=torch.int32)
    k_out, v_out, kept, n = orc.kv_compact(k, v, idx, kv_len=8, keep_recent=2)
    assert kept.tolist() == [[1, 5, 6, 7, -1, -1, -1], [0, 6, 7, -1, -1, -1, -1]]
    assert n.tolist() == [4, 3]
    assert torch.equal(k_out[0, :4], k[0, [1, 5, 6, 7]]) and torch.equal(v_out[1, :3], v[1, [0, 6, 7]])
    assert not k_out[0, 4:].any() and not v_out[1, 3:].any()
    # keeping everything is the identity on the valid prefix
    k_all, _, kept_all, n_all = orc.kv_compact(k, v, torch.arange(8, dtype=torch.int32).flip(0).expand(2, 8), kv_len=8)
    assert torch.equal(k_all, k[:, :8]) and n_all.tolist() == [8, 8] and kept_all[0].tolist() == list(range(8))
