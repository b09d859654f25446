"""Record what the reference's code generator declares for a sample of its own IR candidates.

    python tests/golden/make_ir_fixtures.py --ref /path/to/Trinity

For a few candidates of every block family (the best recorded one plus a spread over the sweep) it runs the reference's
``convert_ir_to_triton`` (``codegen/convert_module.py:5-13``; pure Python, no GPU) on the IR text stored in
``evaluation/**/*.json`` and keeps the IR together with the ``TENSOR_PARAMS`` / ``BLOCK_PARAMS`` lines of the module it
emits.  ``tests/test_codegen.py`` checks the replacement generator against these.  ``--check-all`` runs both generators
over every stored candidate (about 14,500) and reports disagreements; nothing is written.
"""
import argparse
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

FAMILIES = {
    "vanilla": ("evaluation/vanilla/vanilla_llama.json", 28142),
    "prenorm": ("evaluation/prenorm/prenorm_llama.json", 579),
    "qknorm": ("evaluation/qknorm/qknorm_llama.json", 54735),
    "keyformer": ("evaluation/keyformer/keyformer_llama.json", 1813),
    "roco": ("evaluation/roco/roco_llama.json", 1753),
    "ffn_llama": ("evaluation/ffn/ffn_llama/benchmark_ffn_llama.json", 2248),
    "ffn_falcon": ("evaluation/ffn/ffn_falcon/benchmark_ffn_final.json", 428),
}


def params_of(text):
    tp = re.search(r"^TENSOR_PARAMS = (\[.*\])$", text, re.M)
    bp = re.search(r"^BLOCK_PARAMS = (\[.*\])$", text, re.M)
    if not tp or not bp:
        return None
    return json.loads(tp.group(1).replace("'", '"')), json.loads(bp.group(1).replace("'", '"'))


def check_all(ref_root, reference_generator):
    """Every candidate stored in evaluation/**/*.json through both generators; prints the counts and the first
    disagreement per file.  Minutes of pure Python; run where the reference is mounted."""
    import glob
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from trinity_b200.codegen import convert_ir_to_triton as replacement
    total = bad = 0
    for path in sorted(glob.glob(os.path.join(ref_root, "evaluation", "**", "*.json"), recursive=True)):
        rows = json.load(open(path))
        rows = [r for r in rows if isinstance(r, dict) and r.get("ir_expression")] if isinstance(rows, list) else []
        n = wrong = 0
        for r in rows:
            try:
                want = params_of(reference_generator(r["ir_expression"], None, r.get("tensor_config")))
            except Exception:
                continue                      # the reference generator itself rejects the candidate
            if want is None:
                continue
            n += 1
            try:
                got = params_of(replacement(r["ir_expression"], None, r.get("tensor_config")))
            except Exception as e:
                got = repr(e)
            if got != want:
                wrong += 1
                if wrong == 1:
                    print("  first disagreement:", r["ir_id"], want, got)
        if n:
            print(f"{os.path.relpath(path, ref_root)}: {n} candidates, {wrong} disagree")
        total, bad = total + n, bad + wrong
    print(f"total: {total} candidates, {bad} disagree")
    return bad


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="checkout of youngchan2/Trinity")
    ap.add_argument("--per-family", type=int, default=4)
    ap.add_argument("--check-all", action="store_true",
                    help="compare the replacement generator with the reference's on every stored candidate instead of writing fixtures")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.ref, "codegen"))
    from convert_module import convert_ir_to_triton  # the reference's
    if args.check_all:
        raise SystemExit(1 if check_all(args.ref, convert_ir_to_triton) else 0)

    out = []
    for family, (rel, best) in FAMILIES.items():
        rows = json.load(open(os.path.join(args.ref, rel)))
        rows = [r for r in rows if r.get("ir_expression") and not r.get("error")]
        picked = [r for r in rows if r["ir_id"] == best][:1]
        step = max(1, len(rows) // args.per_family)
        picked += [r for r in rows[::step] if r["ir_id"] != best][: args.per_family - len(picked)]
        for r in picked:
            shapes = None
            try:
                text = convert_ir_to_triton(r["ir_expression"], shapes, r["tensor_config"])
            except Exception as e:  # the reference generator needs the shape table for some candidates
                print("skip", family, r["ir_id"], type(e).__name__)
                continue
            tp = re.search(r"^TENSOR_PARAMS = (\[.*\])$", text, re.M)
            bp = re.search(r"^BLOCK_PARAMS = (\[.*\])$", text, re.M)
            if not tp or not bp:
                continue
            out.append({"family": family, "ir_id": r["ir_id"], "constants": r["tensor_config"], "ir": r["ir_expression"],
                        "tensor_params": json.loads(tp.group(1).replace("'", '"')),
                        "block_params": json.loads(bp.group(1).replace("'", '"'))})
    json.dump(out, open(os.path.join(HERE, "ir_modules.json"), "w"), indent=0)
    print("wrote", len(out), "fixtures")


if __name__ == "__main__":
    main()
