"""Record the tensor tables of the reference's sweep harnesses.

    python tests/golden/make_sweep_fixtures.py --ref /path/to/Trinity

Imports every ``benchmark/*_benchmark.py`` of the reference on the CPU (``torch.cuda.set_device`` and
``get_device_name`` made no-ops for the duration), builds its benchmark class for the model's tensor configuration
(``evaluation/llama_configs.json`` / ``falcon_configs.json``; the FFN harnesses take the hidden width from ``P``) and
keeps, per harness: the name -> shape table, which tensors it creates as zeros, and the largest magnitude of the random
ones.  ``tests/test_sweep.py`` checks ``trinity_b200.sweep.tensor_shapes`` and its zero lists against this file.
"""
import argparse
import importlib.util
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
HARNESSES = {  # file stem -> (family, model)
    "vanilla_llama": ("vanilla", "llama"), "vanilla_falcon": ("vanilla", "falcon"),
    "prenorm_llama": ("prenorm", "llama"), "prenorm_falcon": ("prenorm", "falcon"),
    "qknorm_llama": ("qknorm", "llama"), "qknorm_falcon": ("qknorm", "falcon"),
    "keyformer_llama": ("keyformer", "llama"), "keyformer_falcon": ("keyformer", "falcon"),
    "roco_llama": ("roco", "llama"), "roco_falcon": ("roco", "falcon"),
    "ffn_llama": ("ffn_llama", "llama"), "ffn_falcon": ("ffn_falcon", "falcon"),
}
# small stand-ins with the models' ratios, so that building the tables on a CPU stays cheap
CONFIGS = {"llama": {"M": 16, "D": 8, "N": 64, "P": 48, "H": 8}, "falcon": {"M": 16, "D": 4, "N": 44, "P": 24, "H": 11}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="checkout of youngchan2/Trinity")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    sys.path.insert(0, os.path.join(args.ref, "codegen"))  # the generator imports its siblings by bare name
    real = torch.cuda.set_device, torch.cuda.get_device_name
    torch.cuda.set_device = lambda *a, **k: None
    torch.cuda.get_device_name = lambda *a, **k: "cpu"
    import types
    for name in ("tensorrt", "flashinfer"):  # imported at module level by the Falcon FFN harness's baseline; never called here
        sys.modules.setdefault(name, types.ModuleType(name))
    out = []
    try:
        for stem, (family, model) in HARNESSES.items():
            path = os.path.join(args.ref, "benchmark", stem + "_benchmark.py")
            spec = importlib.util.spec_from_file_location("_trinity_ref_" + stem, path)
            mod = importlib.util.module_from_spec(spec)
            try:
                spec.loader.exec_module(mod)
            except ImportError as e:
                # benchmark/ffn_falcon_benchmark.py:18 imports a name its baseline module does not define; the table
                # does not depend on it, so retry with a placeholder module that answers any attribute
                print(stem, "import failed:", e, "- retrying with a placeholder baseline.ffn_ref")
                stub = types.ModuleType("baseline.ffn_ref")
                stub.__getattr__ = lambda name: type(name, (), {})
                sys.modules["baseline.ffn_ref"] = stub
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
            cls = next(v for k, v in vars(mod).items() if isinstance(v, type) and k.endswith("Benchmark") and hasattr(v, "create_test_tensors"))
            cfg = dict(CONFIGS[model])
            bench = cls(cfg)
            shapes = {k: list(v) if isinstance(v, tuple) else [v] for k, v in bench.tensor_shapes.items()}
            zeros = sorted(k for k, t in bench.tensors.items() if not bool(t.any()))
            amax = max(float(t.abs().max()) for k, t in bench.tensors.items() if k not in zeros)
            out.append({"harness": stem, "family": family, "config": cfg, "shapes": shapes, "zeros": zeros,
                        "dtype": str(next(iter(bench.tensors.values())).dtype), "input_abs_max": amax})
            print(stem, len(shapes), "tensors,", len(zeros), "zero-initialised, inputs within", amax)
    finally:
        torch.cuda.set_device, torch.cuda.get_device_name = real
    json.dump(out, open(os.path.join(HERE, "sweep_tables.json"), "w"), indent=0)


if __name__ == "__main__":
    main()
