"""The generated-module boundary: convert_ir_to_triton returns module source with the reference's
metadata contract (TENSOR_PARAMS sorted, BLOCK_PARAMS, forward accepting trailing block sizes)."""
import pytest

from trinity_b200.codegen import convert_ir_to_triton, ir

# Minimal IRs in the reference grammar (codegen/IrParser.py), one per block family.
ATTN = ("(ploop 0 4096 128 n (seq (sloop 0 4096 tile_k k (store (tensor Q1,K1,V1) (+ (x (load (tensor Q1,K1,V1) (index fulltile (tile n))) 1) "
        "(* (load (input X) (index fulltile (tile k))) (load (input WQ,WK,WV) (index (tile k) (tile n))))) (index fulltile (tile n)))) "
        "(seq (store (input K_cache,V_cache) (load (tensor K,V) (index (elem n) fulltile fulltile)) (index (elem n) (const_tile 1024 16) fulltile)) "
        "(seq (sloop 0 1040 tile_p p (store (tensor C_exp) (exp (* (load (tensor Q) (index (elem n) fulltile fulltile)) "
        "(load (input K_cache) (index (elem n) (tile p) fulltile)))) (index (elem n) fulltile (tile p)))) %s"
        "(store (output O2) (load (tensor O) (index (elem n) fulltile fulltile)) (index fulltile (tile n)))))))")
VANILLA = ATTN % ""
PRENORM = VANILLA.replace("(seq (sloop 0 4096 tile_k k (store", "(seq (sloop 0 4096 tile_k k (seq (store (tensor X2) (rsum (sqr (load (input X) (index fulltile (tile k)))) 1) (index fulltile)) (store", 1).replace("(index fulltile (tile n)))) (seq (store (input K_cache", "(index fulltile (tile n))))) (seq (store (input K_cache", 1)
KEYFORMER = ATTN % "(seq (store (output C_out) (load (input noise) (index (elem n) fulltile fulltile)) (index (elem n) fulltile)) "
KEYFORMER = KEYFORMER[:-1] + "))"
ROCO = ATTN % "(seq (store (output C_out1) (load (tensor C_exp) (index (elem n) fulltile (tile p))) (index (elem n) fulltile)) (seq (store (output C_out2) (load (tensor C_exp) (index (elem n) fulltile (tile p))) (index (elem n) fulltile)) "
ROCO = ROCO[:-1] + ")))"
TWO_KERNELS = ("(seq (ploop 0 4096 128 n (store (tensor O) (* (load (input X) (index fulltile)) (load (input WQ,WK,WV) (index fulltile (tile n)))) (index (elem n) fulltile fulltile))) "
               "(ploop 0 4096 128 n (store (output O2) (load (tensor O) (index (elem n) fulltile fulltile)) (index fulltile (tile n)))))")
FFN = ("(seq (ploop 0 4096 tile_n n (store (tensor attn_O2) (+ (* (load (input O2) (index fulltile fulltile)) (load (input WO) (index fulltile (tile n)))) "
       "(load (input X) (index fulltile (tile n)))) (index fulltile (tile n)))) "
       "(seq (ploop 0 14336 tile_p p (store (tensor FF1) (x (* (load (tensor attn_O2) (index fulltile fulltile)) (load (input WFF1a) (index fulltile (tile p)))) "
       "(sigmoid (* (load (tensor attn_O2) (index fulltile fulltile)) (load (input WFF1b) (index fulltile (tile p)))))) (index fulltile (tile p)))) "
       "(ploop 0 4096 tile_n n (store (output FF2) (* (load (tensor FF1) (index fulltile fulltile)) (load (input WFF2) (index fulltile (tile n)))) (index fulltile (tile n))))))")
CONST = {"M": 16, "D": 128, "N": 4096, "P": 1024, "H": 32}


def load(src):
    ns = {}
    exec(compile(src, "<module>", "exec"), ns)
    return ns


@pytest.mark.parametrize("text,kind,extra", [
    (VANILLA, "vanilla", []), (PRENORM, "prenorm", []), (KEYFORMER, "keyformer", ["C_out", "noise"]),
    (ROCO, "roco", ["C_out1", "C_out2"]),
])
def test_attention_modules(text, kind, extra):
    s = ir.summarize(text)
    assert ir.classify(s) == kind
    m = load(convert_ir_to_triton(text, None, CONST))
    assert m["TENSOR_PARAMS"] == sorted(["K_cache", "O2", "V_cache", "WK", "WQ", "WV", "X"] + extra)
    assert m["BLOCK_PARAMS"] == ["block_k", "block_p"]
    assert m["KIND"] == kind and m["CONSTANTS"] == CONST
    import inspect
    sig = inspect.signature(m["forward"])
    assert list(sig.parameters) == m["TENSOR_PARAMS"] + m["BLOCK_PARAMS"] + m["OPTIONAL_TENSOR_PARAMS"]
    assert all(sig.parameters[b].default == 16 for b in m["BLOCK_PARAMS"])
    # tensors the reference's blocks do not have come last, keyword-only, default None: positional callers are unaffected
    assert all(sig.parameters[o].kind is inspect.Parameter.KEYWORD_ONLY and sig.parameters[o].default is None
               for o in m["OPTIONAL_TENSOR_PARAMS"])
    assert m["OPTIONAL_TENSOR_PARAMS"] == {"vanilla": [], "prenorm": ["norm_weight"], "keyformer": ["topk_idx"], "roco": ["topk_idx"]}[kind]


def test_cross_kernel_intermediate_becomes_a_parameter():
    m = load(convert_ir_to_triton(TWO_KERNELS, None, CONST))
    assert "O" in m["TENSOR_PARAMS"] and m["TENSOR_PARAMS"] == sorted(m["TENSOR_PARAMS"])
    assert m["BLOCK_PARAMS"] == []


def test_ffn_module():
    m = load(convert_ir_to_triton(FFN, None, {"M": 16, "N": 4096, "P": 14336}))
    assert m["KIND"] == "ffn_llama"
    assert m["TENSOR_PARAMS"] == ["FF1", "FF2", "O2", "WFF1a", "WFF1b", "WFF2", "WO", "X", "attn_O2"]
    assert m["BLOCK_PARAMS"] == ["block_n", "block_p"]


def test_errors_are_exceptions():
    with pytest.raises(ValueError):
        convert_ir_to_triton("(ploop 0 16 4 n (store (output Z) (load (input X) (index fulltile)) (index fulltile)))", None, {})
    with pytest.raises(ValueError):
        convert_ir_to_triton("(seq (store (output O2)", None, {})
    with pytest.raises(ValueError):
        convert_ir_to_triton("", None, {})


def test_parameter_lists_match_the_reference_generator(golden_dir):
    """IR candidates from the reference's own sweeps (evaluation/**/*.json) with the TENSOR_PARAMS / BLOCK_PARAMS its
    generator emitted for them (tests/golden/make_ir_fixtures.py): the replacement must declare the same lists, or the
    harness's positional call forward(*tensors) would bind the wrong tensors."""
    import json
    import os
    fixtures = json.load(open(os.path.join(golden_dir, "ir_modules.json")))
    assert len(fixtures) >= 20
    seen = set()
    for f in fixtures:
        m = load(convert_ir_to_triton(f["ir"], None, f["constants"]))
        assert m["TENSOR_PARAMS"] == f["tensor_params"], (f["family"], f["ir_id"])
        assert m["BLOCK_PARAMS"] == f["block_params"], (f["family"], f["ir_id"])
        assert m["KIND"].split("_prenorm")[0] in (f["family"], f["family"].replace("prenorm", "vanilla")) or m["KIND"] == f["family"]
        seen.add(f["family"])
    assert seen == {"vanilla", "prenorm", "qknorm", "keyformer", "roco", "ffn_llama", "ffn_falcon"}
