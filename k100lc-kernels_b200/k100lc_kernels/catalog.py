"""Kernel directory: ``kernels(pattern)`` / ``info(name)`` over ``catalog.json``
(reference python/k100lc_kernels/catalog.py:14-25, schema docs/ABI.md:12-39).

``catalog.json`` is generated from the engine's own kernel table by ``make_catalog()``
(run ``python -m k100lc_kernels catalog``), and a test checks that the two agree.  Each
entry keeps the reference schema: ``lookup``, ``name``, ``args`` as ``(off, size,
kind)`` in a packed-by-natural-alignment kernarg layout, ``kernarg_size``,
``group_segment`` and ``private_segment`` (both 0: shared memory is sized by the
launcher here)."""
from __future__ import annotations

import json
import pathlib

CATALOG = pathlib.Path(__file__).resolve().parent / "catalog.json"


def load() -> list[dict]:
    return json.loads(CATALOG.read_text(encoding="utf-8"))["kernels"]


def kernels(pattern: str = "") -> list[dict]:
    return [k for k in load() if pattern in k["lookup"]]


def info(name: str) -> dict:
    for k in load():
        if name in (k["lookup"], k["name"]):
            return k
    raise KeyError(name)


def make_catalog(lib=None) -> dict:
    """Build the catalog dictionary from the library's kernel table (no GPU needed)."""
    from .runtime import load_library
    lib = load_library(lib)
    out = []
    for kid in range(lib.fm_kernel_count()):
        name = lib.fm_kernel_name(kid).decode()
        sig = lib.fm_kernel_sig(kid).decode()
        off, args = 0, []
        for ch in sig:
            size = 8 if ch == "p" else 4
            off = (off + size - 1) // size * size
            args.append({"off": off, "size": size, "kind": "global_buffer" if ch == "p" else "by_value",
                         "type": {"p": "pointer", "i": "i32", "f": "f32"}[ch]})
            off += size
        out.append({"lookup": name, "name": name, "args": args, "kernarg_size": (off + 7) // 8 * 8,
                    "group_segment": 0, "private_segment": 0})
    return {"version": 1, "target": "sm_100a", "kernels": out}
