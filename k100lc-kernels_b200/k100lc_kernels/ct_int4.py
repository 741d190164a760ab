"""compressed-tensors INT4 checkpoints: safetensors reader for pack-quantised linear layers.

The host-side loader that feeds ``Int4Linear`` / ``DotLinear`` from a real checkpoint
(reference tools/ct_int4.py:61-184).  A layer ``<prefix>`` consists of three tensors:
``<prefix>.weight_packed`` (I32 ``[N, K/8]``, eight offset-binary codes per word, lowest k in
the lowest nibble), ``<prefix>.weight_scale`` (BF16 ``[N, K/128]``) and
``<prefix>.weight_shape`` (I64 ``[2] = (N, K)``).  Only the safetensors header is parsed up
front; rows are read with seek, so multi-GB files are never loaded whole.

A safetensors file is ``<u64 little-endian header length> <JSON header> <raw tensor bytes>``;
the header maps tensor names to ``{"dtype", "shape", "data_offsets": [begin, end]}`` relative
to the end of the header.  ``write_safetensors`` produces such files (used by the tests and
for exporting synthetic layers)."""
from __future__ import annotations

import json
import pathlib
import struct

import numpy as np

from .quant import GROUP, bf16_bits_to_f32, unpack_nibbles

_DTYPES = {"I32": np.int32, "I64": np.int64, "BF16": np.uint16, "F16": np.float16, "F32": np.float32,
           "U8": np.uint8, "I8": np.int8}


class SafeTensors:
    """Header of one ``.safetensors`` file plus ranged reads of its tensors."""

    def __init__(self, path):
        self.path = pathlib.Path(path)
        with open(self.path, "rb") as f:
            (self.header_len,) = struct.unpack("<Q", f.read(8))
            self.header = json.loads(f.read(self.header_len))
        self.header.pop("__metadata__", None)

    def __contains__(self, name: str) -> bool:
        return name in self.header

    def entry(self, name: str) -> dict:
        if name not in self.header:
            raise KeyError(f"{self.path.name} has no tensor {name}")
        return self.header[name]

    def read(self, name: str, begin: int = 0, nbytes: int | None = None) -> bytes:
        """``nbytes`` raw bytes of tensor ``name`` starting ``begin`` bytes into it."""
        lo, hi = self.entry(name)["data_offsets"]
        nbytes = hi - lo - begin if nbytes is None else nbytes
        if begin < 0 or nbytes < 0 or lo + begin + nbytes > hi:
            raise ValueError(f"{name}: range [{begin}, {begin + nbytes}) is outside the tensor ({hi - lo} bytes)")
        with open(self.path, "rb") as f:
            f.seek(8 + self.header_len + lo + begin)
            raw = f.read(nbytes)
        if len(raw) != nbytes:
            raise IOError(f"{name}: expected {nbytes} bytes, file ends after {len(raw)}")
        return raw

    def array(self, name: str) -> np.ndarray:
        e = self.entry(name)
        return np.frombuffer(self.read(name), dtype=_DTYPES[e["dtype"]]).reshape(e["shape"])


def write_safetensors(path, tensors: dict) -> None:
    """``tensors``: name -> (dtype string, ndarray).  BF16 arrays are passed as uint16 bit patterns."""
    header, blobs, off = {}, [], 0
    for name, (dtype, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


class CTInt4Layer:
    """One pack-quantised linear layer of a checkpoint directory (or of explicit files)."""

    def __init__(self, prefix: str, model_dir=None, files=None):
        self.prefix = prefix
        paths = [pathlib.Path(p) for p in files] if files else sorted(pathlib.Path(model_dir).glob("*.safetensors"))
        self._files = [SafeTensors(p) for p in paths if pathlib.Path(p).is_file()]
        if not self._files:
            raise FileNotFoundError(f"no safetensors file for {prefix} under {model_dir or files}")
        n, k = (int(v) for v in self._find("weight_shape").array(prefix + ".weight_shape"))
        if k % GROUP:
            raise ValueError(f"{prefix}: K={k} is not a multiple of {GROUP}")
        self.n, self.k, self.nbpr = n, k, k // GROUP
        for suffix, want in (("weight_packed", [n, k // 8]), ("weight_scale", [n, k // GROUP])):
            got = self._find(suffix).entry(f"{prefix}.{suffix}")["shape"]
            if list(got) != want:
                raise ValueError(f"{prefix}.{suffix}: shape {got} does not match weight_shape [{n},{k}]")

    def _find(self, suffix: str) -> SafeTensors:
        name = f"{self.prefix}.{suffix}"
        for st in self._files:
            if name in st:
                return st
        raise KeyError(f"{name} not found")

    def _rows(self, suffix: str, row0: int, nrows, row_bytes: int) -> bytes:
        nrows = self.n - row0 if nrows is None else nrows
        if row0 < 0 or nrows <= 0 or row0 + nrows > self.n:
            raise ValueError(f"{self.prefix}: rows [{row0},{row0 + nrows}) are outside N={self.n}")
        return self._find(suffix).read(f"{self.prefix}.{suffix}", row0 * row_bytes, nrows * row_bytes)

    def packed_rows(self, row0: int = 0, nrows=None) -> bytes:
        """Bytes of ``weight_packed`` for a run of rows: directly the ``w`` buffer of ``int4_dot_k``."""
        return self._rows("weight_packed", row0, nrows, self.k // 2)

    def scale_rows(self, row0: int = 0, nrows=None) -> bytes:
        """BF16 bytes of ``weight_scale`` for a run of rows: the scale table of ``int4_dot_k``."""
        return self._rows("weight_scale", row0, nrows, self.nbpr * 2)

    def dequant_rows(self, row0: int = 0, nrows=None) -> np.ndarray:
        """Host decode to f32 ``[rows, K]``: ``(code - 8) * scale``."""
        nrows = self.n - row0 if nrows is None else nrows
        codes = unpack_nibbles(np.frombuffer(self.packed_rows(row0, nrows), np.uint32).reshape(nrows, -1))
        s = bf16_bits_to_f32(np.frombuffer(self.scale_rows(row0, nrows), np.uint16)).reshape(nrows, self.nbpr)
        return (codes.astype(np.int32) - 8).astype(np.float32) * np.repeat(s, GROUP, axis=1)

    def linear(self, rt, path: str = "w4a8", ws=None, tag=None, **kw):
        """``Int4Linear`` for this layer on ``rt`` (weights uploaded once)."""
        from .model import Int4Linear
        return Int4Linear(rt, self.n, self.k, self.packed_rows(), self.scale_rows(), path, ws, tag or self.prefix, **kw)

    def __repr__(self) -> str:
        return f"CTInt4Layer({self.prefix}, N={self.n}, K={self.k}, {self.n * self.k / 2 / 1e6:.1f} MB packed)"
