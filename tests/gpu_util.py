"""Helpers for the GPU tier: a per-test buffer set on the session's ``Runtime``."""
from __future__ import annotations

import numpy as np


class Bufs:
    """Device buffers of one test case, freed together (the role of the reference's
    ``Ctx`` in tools/selftest_all.py:67-100)."""

    def __init__(self, rt):
        self.rt = rt
        self._ptrs: list[int] = []

    def put(self, data) -> int:
        data = np.ascontiguousarray(data)
        p = self.rt.alloc(max(data.nbytes, 4))
        self.rt.upload(p, data)
        self._ptrs.append(p)
        return p

    def zeros(self, count: int, dtype=np.float32, fill=0) -> int:
        return self.put(np.full(int(count), fill, dtype=dtype))

    def get(self, ptr: int, count: int, dtype=np.float32) -> np.ndarray:
        self.rt.sync()
        return self.rt.download(ptr, int(count), dtype)

    def close(self) -> None:
        for p in self._ptrs:
            self.rt.free(p)
        self._ptrs.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
