"""A reader for the tile IR -- enough to recognise WHICH fused block an IR describes and which tensors
its module takes; the IR is not compiled (the kernels are hand-written).

Grammar as parsed by the reference (``codegen/IrParser.py:13-19,49-135``): S-expressions;
``(ploop start end tile var body)``, ``(sloop start end tile var body)``, ``(seq a b)``,
``(store tref value index)``, ``(load tref index)`` with ``tref`` one of ``(input A[,B..])``,
``(output A)``, ``(tensor A[,B..])``; ``dummy`` leaves.  A symbolic tile ``tile_<v>`` becomes the
module's ``block_<v>`` parameter (``codegen/TritonGen.py:553-558``).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import List, Set, Union

Node = Union[str, List["Node"]]
_TOKEN = re.compile(r"\(|\)|[^\s()]+")


def parse(ir_code: str) -> Node:
    text = "\n".join(line.split(";", 1)[0] for line in ir_code.splitlines())
    tokens = _TOKEN.findall(text)
    if not tokens:
        raise ValueError("empty IR")
    pos = 0

    def read() -> Node:
        nonlocal pos
        if pos >= len(tokens):
            raise ValueError("unexpected end of IR")
        tok = tokens[pos]
        pos += 1
        if tok == "(":
            items: List[Node] = []
            while True:
                if pos >= len(tokens):
                    raise ValueError("unbalanced parentheses in IR")
                if tokens[pos] == ")":
                    pos += 1
                    return items
                items.append(read())
        if tok == ")":
            raise ValueError("unbalanced parentheses in IR")
        return tok

    root = read()
    if pos != len(tokens):
        raise ValueError("trailing tokens after the IR expression")
    return root


@dataclass
class KernelUse:
    stores: Set[str] = field(default_factory=set)
    loads: Set[str] = field(default_factory=set)
    store_index: dict = field(default_factory=dict)   # name -> set of index expressions it is stored with
    load_index: dict = field(default_factory=dict)    # name -> set of index expressions it is loaded with


@dataclass
class IrSummary:
    inputs: Set[str] = field(default_factory=set)
    outputs: Set[str] = field(default_factory=set)
    tensors: Set[str] = field(default_factory=set)
    block_params: Set[str] = field(default_factory=set)
    kernels: List[KernelUse] = field(default_factory=list)

    def cross_kernel(self) -> Set[str]:
        """Intermediates that live in HBM and are therefore module parameters: written by one kernel and read by
        another (``codegen/TritonGen.py:1018-1053``), or written and re-read inside one kernel through a different
        index expression (another tiling of the same tensor cannot stay in registers)."""
        out: Set[str] = set()
        for name in self.tensors:
            writers = {i for i, k in enumerate(self.kernels) if name in k.stores}
            readers = {i for i, k in enumerate(self.kernels) if name in k.loads}
            if writers and readers and (readers - writers or len(writers) > 1):
                out.add(name)
                continue
            for k in self.kernels:
                st, ld = k.store_index.get(name, set()), k.load_index.get(name, set())
                if st and ld and (ld - st):
                    out.add(name)
        return out


def _top_level_kernels(root: Node) -> List[Node]:
    """Each child of the root ``seq`` chain is one kernel (``codegen/TritonGen.py:458-541``)."""
    out: List[Node] = []

    def flatten(n: Node):
        if isinstance(n, list) and n and n[0] == "seq":
            for child in n[1:]:
                flatten(child)
        elif n != "dummy":
            out.append(n)

    flatten(root)
    return out


def summarize(ir_code: str) -> IrSummary:
    root = parse(ir_code)
    s = IrSummary()

    def names(tref: Node) -> List[str]:
        if not (isinstance(tref, list) and len(tref) >= 2 and tref[0] in ("input", "output", "tensor")):
            raise ValueError(f"malformed tensor reference: {tref!r}")
        got = [n for part in tref[1:] for n in str(part).split(",") if n]
        {"input": s.inputs, "output": s.outputs, "tensor": s.tensors}[tref[0]].update(got)
        return got

    def walk(n: Node, use: KernelUse):
        if not isinstance(n, list) or not n:
            return
        head = n[0]
        if head in ("ploop", "sloop"):
            if len(n) != 6:
                raise ValueError(f"malformed {head}")
            tile, var = n[3], n[4]
            if isinstance(tile, str) and not tile.isdigit():
                s.block_params.add(f"block_{var}")
            walk(n[5], use)
        elif head == "store":
            if len(n) != 4:
                raise ValueError("malformed store")
            got = names(n[1])
            use.stores.update(got)
            for name in got:
                use.store_index.setdefault(name, set()).add(repr(n[3]))
            walk(n[2], use)
        elif head == "load":
            got = names(n[1])
            use.loads.update(got)
            for name in got:
                use.load_index.setdefault(name, set()).add(repr(n[2]) if len(n) > 2 else "")
        else:
            for child in n[1:]:
                walk(child, use)

    for kernel in _top_level_kernels(root):
        use = KernelUse()
        walk(kernel, use)
        s.kernels.append(use)
    return s


def classify(s: IrSummary) -> str:
    """Block family by the tensor names an IR touches."""
    every = s.inputs | s.outputs | s.tensors
    if "O_FF_norm" in every:
        return "ffn_falcon"
    if "FF2" in every:
        return "ffn_llama"
    if "O2" not in s.outputs:
        raise ValueError("IR describes none of the fused blocks (no O2 / FF2 / O_FF_norm output)")
    kind = "vanilla"
    if "C_out" in every and "noise" in every:
        kind = "keyformer"
    elif "C_out1" in every or "C_out2" in every:
        kind = "roco"
    elif "Q_norm" in every or "K_norm" in every:
        kind = "qknorm"
    prenorm = "X2" in every or "X_norm" in every
    if kind == "vanilla":
        return "prenorm" if prenorm else "vanilla"
    return kind + ("_prenorm" if prenorm else "")
