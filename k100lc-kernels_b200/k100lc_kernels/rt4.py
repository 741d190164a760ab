"""RT4 int4 weight files and the W4A8 / W4A4 launch recipes.

Mirror of the reference's python/k100lc_kernels/rt4.py: ``RT4File`` / ``RT4Tensor``
(rt4.py:62-190) read the single-file container — a ``.rt4`` blob plus a ``.rt4.json``
manifest ``{format: "RT4-v1", group, tensors: [{name, kind, shape, group, q_off, s_off,
nbytes}]}`` — and ``W4Runner`` (rt4.py:193-366) holds the kernel names, grids and
scratch buffers of the decode GEMV (M = 1..4) and the prefill GEMM.

Layout of an ``i4`` linear layer ``[N, K]`` with group 128:
  q region  N*K/2 bytes   signed int4, two per byte, low nibble = even k
  s region  N*(K/128)*2   f16 scales, ``w[n,k] = q[n,k] * s[n, k//128]``
"""
from __future__ import annotations

import dataclasses
import json
import mmap
import pathlib

import numpy as np

from .runtime import Runtime

GRP = 128            # weight scale group
SG = 32              # activation sub-group of the W4A4 path (quant_act4)
# kernel names by token count (reference rt4.py:38-41)
W4A8_KERNEL = {m: f"gemv_w4a8<{m},false,{1 if m == 1 else 2}>" for m in (1, 2, 3, 4)}
W4A4_KERNEL = {m: f"gemv_w4a4<{m}>" for m in (1, 2, 3, 4)}


def _div_magic(d: int, max_i: int) -> int:
    """``M`` with ``(i * M) >> 32 == i // d`` for all ``0 <= i < max_i``; the flat GEMM
    entry takes it for ABI compatibility (the B200 kernel divides directly)."""
    if d <= 1:
        raise ValueError("_div_magic needs d >= 2")
    m = (1 << 32) // d + 1
    if m >> 32:
        raise ValueError(f"_div_magic: d={d} is too large")
    i = np.arange(max_i, dtype=np.uint64)
    if ((i * np.uint64(m)) >> np.uint64(32) != i // np.uint64(d)).any():
        raise ValueError(f"_div_magic: d={d} is not exact below {max_i}")
    return int(m)


@dataclasses.dataclass(frozen=True)
class RT4Tensor:
    name: str
    kind: str
    shape: tuple[int, int]
    group: int
    q_off: int
    s_off: int
    nbytes: int

    @property
    def rows(self) -> int:
        return self.shape[0]

    @property
    def cols(self) -> int:
        return self.shape[1]

    @property
    def q_bytes(self) -> int:
        return self.rows * (self.cols // 2)

    @property
    def s_bytes(self) -> int:
        return self.rows * (self.cols // self.group) * 2


class RT4File:
    """Read-only, memory-mapped access to an RT4 file and its manifest."""

    def __init__(self, path):
        self.path = pathlib.Path(path)
        if self.path.suffix != ".rt4":
            raise ValueError(f"RT4File needs a .rt4 file: {self.path}")
        manifest = self.path.with_suffix(".rt4.json")
        if not manifest.is_file():
            manifest = self.path.with_suffix(".json")
            if not manifest.is_file():
                raise FileNotFoundError(f"manifest not found: {self.path.with_suffix('.rt4.json')}")
        self.manifest_path = manifest
        self.manifest = json.loads(manifest.read_text(encoding="utf-8"))
        if self.manifest.get("format") != "RT4-v1":
            raise ValueError(f"unsupported RT4 format: {self.manifest.get('format')}")
        self.group = int(self.manifest.get("group", GRP))
        self._index = {t["name"]: t for t in self.manifest["tensors"]}
        self._fh = open(self.path, "rb")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)

    def close(self) -> None:
        self._mm.close()
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def tensor(self, name: str) -> RT4Tensor:
        if name not in self._index:
            raise KeyError(f"no tensor {name} in {self.path.name}")
        t = self._index[name]
        return RT4Tensor(t["name"], t["kind"], tuple(t["shape"]), int(t.get("group", self.group)),
                         int(t["q_off"]), int(t["s_off"]), int(t["nbytes"]))

    def names(self, kind=None) -> list[str]:
        return [t["name"] for t in self.manifest["tensors"] if kind in (None, t["kind"])]

    def weight_bytes(self, t: RT4Tensor) -> tuple[bytes, bytes]:
        """``(packed int4 bytes, f16 scale bytes)`` of one layer."""
        if t.kind != "i4":
            raise ValueError(f"{t.name}: kind={t.kind}; the W4 paths take i4 tensors only")
        if t.cols % t.group or t.cols % 8:
            raise ValueError(f"{t.name}: K={t.cols} is not a multiple of {t.group}")
        return self._mm[t.q_off:t.q_off + t.q_bytes], self._mm[t.s_off:t.s_off + t.s_bytes]

    def upload_weight(self, rt: Runtime, t: RT4Tensor) -> tuple[int, int]:
        """Upload q and s; returns ``(wq_ptr, ws_ptr)``, owned by the caller."""
        q, s = self.weight_bytes(t)
        pq, ps = rt.alloc(len(q)), rt.alloc(len(s))
        rt.upload(pq, q)
        rt.upload(ps, s)
        return pq, ps

    def upload_weight_gemm(self, rt: Runtime, t: RT4Tensor) -> tuple[int, int]:
        """GEMM form: the same q region plus f32 scales transposed to ``[K/G, N]``."""
        q, s = self.weight_bytes(t)
        n, k = t.shape
        gf = np.ascontiguousarray(np.frombuffer(s, dtype=np.float16).astype(np.float32)
                                  .reshape(n, k // t.group).T)
        pq, ps = rt.alloc(len(q)), rt.alloc(gf.nbytes)
        rt.upload(pq, q)
        rt.upload(ps, gf)
        return pq, ps

    def dequant(self, t: RT4Tensor, rows=None, start: int = 0) -> np.ndarray:
        """Host dequantisation to f32 ``[rows, K]`` (whole layer by default)."""
        q, s = self.weight_bytes(t)
        rows = t.rows - start if rows is None else rows
        half, ng = t.cols // 2, t.cols // t.group
        raw = np.frombuffer(q, dtype=np.uint8)[start * half:(start + rows) * half].reshape(rows, half)
        vals = np.empty((rows, t.cols), dtype=np.int8)
        vals[:, 0::2] = (raw & 0xF).astype(np.int8)
        vals[:, 1::2] = (raw >> 4).astype(np.int8)
        vals = np.where(vals >= 8, vals - 16, vals)
        sc = np.frombuffer(s, dtype=np.float16)[start * ng:(start + rows) * ng].astype(np.float32)
        return (vals.reshape(rows, ng, t.group) * sc.reshape(rows, ng, 1)).reshape(rows, t.cols).astype(np.float32)


class W4Runner:
    """W4A8 / W4A4 decode GEMV (M = 1..4) and prefill GEMM on a ``Runtime``."""

    BM, BN, QG = 128, 64, 128      # GEMM granularity of the ABI: M % 128, N % 64, K % 128

    def __init__(self, rt: Runtime):
        self.rt = rt
        self._bufs: dict[tuple[str, int], int] = {}

    def _buf(self, name: str, nbytes: int) -> int:
        key = (name, int(nbytes))
        if key not in self._bufs:
            self._bufs[key] = self.rt.alloc(int(nbytes))
        return self._bufs[key]

    def close(self) -> None:
        for p in self._bufs.values():
            self.rt.free(p)
        self._bufs.clear()

    @staticmethod
    def _rows_of(x, x_dev, m, k):
        if x_dev is not None:
            if m is None:
                raise ValueError("x_dev needs m (the number of rows of x)")
            return None, int(m)
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim != 2 or x.shape[1] != k:
            raise ValueError(f"x has shape {x.shape}, expected [M,{k}]")
        return x, x.shape[0]

    FUSED_K = (5120, 6144)      # K of the one-token entries that quantise inside the GEMV (quant_gemv_w4a8 / _w4a4)

    def gemv_device(self, kind: str, wq: int, ws: int, x, n: int, k: int, threads: int = 256,
                    upload: bool = True, x_dev=None, y_dev=None, m=None, sync: bool = True, fused=None) -> int:
        """Activation quantiser + GEMV on the device; returns the device pointer of
        y ``[M,N]``.  ``x_dev`` chains layers without a host round trip; ``sync=False``
        leaves the work queued.  One W4A8 token at K = 5120 / 6144 is a single launch (the GEMV quantises x
        itself: same bits, one launch and the round trip of the codes less; 11.7 against 12.1 us for a
        17408 x 5120 layer); ``fused=False`` keeps the two launches of the reference's runner, ``fused=True``
        asks for the single launch on the W4A4 path as well (no faster there: every CTA repeats the
        quantiser's divisions)."""
        x, m = self._rows_of(x, x_dev, m, k)
        if m not in (1, 2, 3, 4):
            raise ValueError(f"the W4 GEMV takes M = 1..4 rows (got {m}); use the GEMM for prefill")
        if threads != 256:
            raise ValueError(f"the W4 GEMV needs threads=256 (4 rows per work-group); got {threads}")
        rt = self.rt
        px = int(x_dev) if x_dev is not None else self._buf("x", m * k * 4)
        py = int(y_dev) if y_dev is not None else self._buf("y", m * n * 4)
        if upload and x_dev is None:
            rt.upload(px, x)
        if kind not in ("w4a8", "w4a4"):
            raise ValueError(f"unknown W4 path {kind!r} (use 'w4a8' or 'w4a4')")
        one_launch = f"quant_gemv_{kind}"
        if fused is None:
            fused = kind == "w4a8" and m == 1 and k in self.FUSED_K and rt.has(one_launch)
        if fused:
            if m != 1 or k not in self.FUSED_K:
                raise ValueError(f"{one_launch} takes one token and K in {self.FUSED_K} (got M={m}, K={k})")
            rt.launch(one_launch, -(-n // 4), threads, [wq, ws, px, py, n, k])
        elif kind == "w4a8":
            if k % GRP:
                raise ValueError(f"W4A8 needs K to be a multiple of {GRP} (got {k})")
            half, ng4 = k // 2, (k // GRP) * 4
            ae, ao = self._buf("w4a8_ae", m * half), self._buf("w4a8_ao", m * half)
            asc, asu = self._buf("w4a8_asc", m * ng4), self._buf("w4a8_asu", m * ng4)
            # one 2-D launch, grid y = token row (the reference's runner issues one 1-D launch per row;
            # the kernel's own contract covers both)
            rt.launch2d("quant_act", k // GRP, m, 32, 1, [px, ae, ao, asc, asu, m, k])
            rows_per_wg = 4 * (1 if m == 1 else 2)
            rt.launch(W4A8_KERNEL[m], -(-n // rows_per_wg), threads, [wq, ws, ae, ao, asc, asu, py, n, k])
        elif kind == "w4a4":
            if k % SG:
                raise ValueError(f"W4A4 needs K to be a multiple of {SG} (got {k})")
            half, ns4 = k // 2, (k // SG) * 4
            aq, asc = self._buf("w4a4_aq", m * half), self._buf("w4a4_asc", m * ns4)
            rt.launch2d("quant_act4", k // SG, m, 32, 1, [px, aq, asc, m, k])
            rt.launch(W4A4_KERNEL[m], -(-n // 4), threads, [wq, ws, aq, asc, py, n, k])
        if sync:
            rt.sync()
        return py

    def gemv(self, kind: str, wq: int, ws: int, x: np.ndarray, n: int, k: int, threads: int = 256, fused=None) -> np.ndarray:
        """x ``[M,K]`` f32, M = 1..4 -> y ``[M,N]`` f32."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        py = self.gemv_device(kind, wq, ws, x, n, k, threads, fused=fused)
        return self.rt.download(py, x.shape[0] * n, np.float32).reshape(x.shape[0], n)

    def gemm_device(self, wq: int, wsc: int, x, n: int, k: int, threads: int = 256, upload: bool = True,
                    quantize: bool = True, x_dev=None, c_dev=None, m=None, sync: bool = True,
                    kind: str = "w4a4") -> int:
        """Prefill GEMM ``C[M,N] = A[M,K] . W[N,K]^T``: row quantiser then the flat GEMM.
        ``wq, wsc`` come from ``RT4File.upload_weight_gemm`` (f32 scales ``[K/128, N]``).
        ``kind="w4a8"`` selects int8 activations (an addition; the reference has W4A4
        only).  ``quantize=False`` re-uses the codes of a previous call."""
        x, m = self._rows_of(x, x_dev, m, k)
        if m % self.BM:
            raise ValueError(f"the GEMM needs M to be a multiple of {self.BM} (got {m})")
        if n % self.BN:
            raise ValueError(f"the GEMM needs N to be a multiple of {self.BN} (got {n})")
        if k % self.QG:
            raise ValueError(f"the GEMM needs K to be a multiple of {self.QG} (got {k})")
        if kind not in ("w4a4", "w4a8"):
            raise ValueError(f"unknown GEMM path {kind!r}")
        rt = self.rt
        px = int(x_dev) if x_dev is not None else self._buf("gx", m * k * 4)
        pasc = self._buf("gasc", (k // self.QG) * m * 4)
        pc = int(c_dev) if c_dev is not None else self._buf("gc", m * n * 4)
        if upload and x_dev is None:
            rt.upload(px, x)
        ng, nbn = k // self.QG, n // self.BN
        if kind == "w4a8":
            paq = self._buf("gaq8", m * k)
            if quantize:
                rt.launch("quant_rows_a8_k", m, 256, [paq, 0, pasc, 0, px, k, self.QG, m, k, 0])
            rt.launch("gemm_w4a8", nbn * (m // self.BM), threads, [paq, wq, pasc, wsc, pc, m, n, k])
        else:
            paq = self._buf("gaq", m * k // 2)
            if quantize:
                rt.launch("quant_rows_fast_k", m, 256, [paq, pasc, px, k, self.QG, m, k, 0, ng])
            grid = nbn * (m // self.BM)
            if nbn >= 2:
                rt.launch("gemm_w4a4_flat", grid, threads,
                          [paq, wq, pasc, wsc, pc, m, n, k, nbn, _div_magic(nbn, grid)])
            else:        # N == 64: the flat index algebra degenerates; 2-D entry, same kernel
                rt.launch2d("gemm_w4a4", nbn, m // self.BM, threads, 1, [paq, wq, pasc, wsc, pc, m, n, k])
        if sync:
            rt.sync()
        return pc

    def gemm(self, wq: int, wsc: int, x: np.ndarray, n: int, k: int, threads: int = 256,
             kind: str = "w4a4") -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        pc = self.gemm_device(wq, wsc, x, n, k, threads, kind=kind)
        return self.rt.download(pc, x.shape[0] * n, np.float32).reshape(x.shape[0], n)
