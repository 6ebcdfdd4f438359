"""Small on-disk tile table keyed by shape (replaces the reference's compile-and-benchmark
autotuner, src/cute_prism/_autotune.py, and its compile-failure registry).

``tile_table.json`` holds a list of entries ``{"kernel", "dtype", "gate", "M", "N", "K", "gs",
"rs", "cfg"}``; ``M`` is matched by bucket (the entry with the largest ``M`` not above the call's
``M``), the other keys exactly; ``"*"`` matches anything.  ``cfg`` is the integer list handed to
the C ABI.  A miss returns ``None`` and the library's built-in default is used.
The path can be overridden with the environment variable ``PRISM_B200_TILE_TABLE``.
"""
from __future__ import annotations

import json
import os

import torch

_TABLE = None
_DT = {torch.float16: "fp16", torch.bfloat16: "bf16"}


def table_path() -> str:
    return os.environ.get("PRISM_B200_TILE_TABLE",
                          os.path.join(os.path.dirname(os.path.abspath(__file__)), "tile_table.json"))


def load(path: str | None = None):
    global _TABLE
    path = path or table_path()
    try:
        with open(path) as f:
            _TABLE = json.load(f)["entries"]
    except FileNotFoundError:
        _TABLE = []
    return _TABLE


def _match(v, want):
    return v == "*" or v == want


def lookup(kernel, dtype, gate, M, N, K, gs, rs):
    if _TABLE is None:
        load()
    best = None
    for e in _TABLE:
        if not (_match(e.get("kernel", "*"), kernel) and _match(e.get("dtype", "*"), _DT.get(dtype, str(dtype)))
                and _match(e.get("gate", "*"), gate) and _match(e.get("N", "*"), N) and _match(e.get("K", "*"), K)
                and _match(e.get("gs", "*"), gs) and _match(e.get("rs", "*"), rs)):
            continue
        m = e.get("M", 0)
        m = 0 if m == "*" else m
        if m <= M and (best is None or m >= best[0]):
            best = (m, e["cfg"])
    return None if best is None else list(best[1])
