"""Import the reference's own eager PyTorch classes on a CPU-only machine -- TEST INFRASTRUCTURE.

``baseline/ref_rms.py`` and ``baseline/ffn_ref.py`` of youngchan2/Trinity do two things at
import time that fail without a GPU and TensorRT: ``import tensorrt`` (``ref_rms.py:6``,
``ffn_ref.py:4``) and ``torch.cuda.set_device(torch.device('cpu'))`` (``ref_rms.py:24-25``).
This shim stubs the two third-party imports, makes ``set_device`` a no-op for the duration
of the import and switches the modules' global ``dtype`` to fp32, which turns the eager
classes into the fp32 reference.  It needs a checkout of the reference and is therefore
only used where one is mounted (golden-vector generation); nothing that runs on the GPU
machine imports it.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

import torch


def load_reference(ref_root: str):
    """Return ``(ref_rms, ffn_ref)`` modules loaded from ``<ref_root>/baseline`` in fp32 on CPU."""
    mods = []
    saved = {name: sys.modules.get(name) for name in ("tensorrt", "flashinfer")}
    real_set_device = torch.cuda.set_device
    try:
        for name in ("tensorrt", "flashinfer"):
            sys.modules[name] = types.ModuleType(name)
        torch.cuda.set_device = lambda *a, **k: None
        for fname in ("ref_rms", "ffn_ref"):
            path = os.path.join(ref_root, "baseline", fname + ".py")
            spec = importlib.util.spec_from_file_location("_trinity_ref_" + fname, path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.dtype = torch.float32
            mod.device = torch.device("cpu")
            mods.append(mod)
    finally:
        torch.cuda.set_device = real_set_device
        for name, old in saved.items():
            if old is None:
                sys.modules.pop(name, None)
            else:
                sys.modules[name] = old
    return tuple(mods)
