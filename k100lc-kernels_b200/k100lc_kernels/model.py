"""Model-level operators for the weight-streaming quantized linear layer.

The classes keep the contract of the reference's python/k100lc_kernels/model.py:
weights are uploaded once at construction, intermediate buffers come from a
``Workspace`` keyed by tag, ``forward_device(x_dev, rows, sync=False, out_dev=None)``
chains device pointers without a host round trip and ``forward(x)`` is NumPy in /
NumPy out with a single sync (model.py:132-185, 206-310, 358-477).

In scope: ``Workspace``, ``run_sequence``, ``cdiv``, ``div_magic``, ``DotLinear`` for
the ``int4`` kind, ``RT4Linear``, ``Int4Linear`` and — an addition, the reference only
reaches NVFP4 through raw launches — ``NVFP4Linear``.  The reference's other operators
(norms, attention, MoE, RoPE, sampler ...) use kernels outside this path; their names
are exported so that imports keep working and raise ``NotImplementedError`` when used.
"""
from __future__ import annotations

import numpy as np

from .runtime import LaunchPlan, Runtime  # noqa: F401  (LaunchPlan re-exported like the reference)

__all__ = ["cdiv", "div_magic", "Workspace", "QUANT_SPECS", "DotLinear", "RT4Linear", "Int4Linear",
           "NVFP4Linear", "run_sequence"]


def cdiv(a: int, b: int) -> int:
    return -(-int(a) // int(b))


def div_magic(d: int, max_i: int) -> int:
    """Multiplier ``M`` with ``(i*M) >> 32 == i // d`` for ``0 <= i < max_i`` (reference
    model.py:110-129).  ``int4_dot_k`` takes three of them in its argument list."""
    d, max_i = int(d), int(max_i)
    if d <= 0:
        raise ValueError("div_magic: d must be positive")
    if max_i <= 0:
        return 0
    if d == 1:
        if max_i <= 1:
            return 0
        raise ValueError("div_magic: d=1 is only usable when the index is always 0")
    m = (1 << 32) // d + 1
    if m >> 32:
        raise ValueError(f"div_magic: d={d} is too large")
    i = np.arange(max_i, dtype=np.uint64)
    if ((i * np.uint64(m)) >> np.uint64(32) != i // np.uint64(d)).any():
        raise ValueError(f"div_magic: d={d} is not exact below {max_i}")
    return int(m)


class Workspace:
    """Device buffers re-used by key: ``buffer(key, nbytes)`` returns the same block for
    the same key and re-allocates only when it has to grow."""

    def __init__(self, rt: Runtime):
        self.rt = rt
        self._bufs: dict[str, tuple[int, int]] = {}

    def buffer(self, key: str, nbytes: int) -> int:
        have = self._bufs.get(key)
        if have and have[1] >= nbytes:
            return have[0]
        if have:
            self.rt.free(have[0])
        p = self.rt.alloc(int(nbytes))
        self._bufs[key] = (p, int(nbytes))
        return p

    def upload(self, key: str, data) -> int:
        n = len(data) if isinstance(data, (bytes, bytearray, memoryview)) else data.nbytes
        p = self.buffer(key, n)
        self.rt.upload(p, data)
        return p

    def size(self, key: str) -> int:
        return self._bufs.get(key, (0, 0))[1]

    def free(self) -> None:
        for p, _n in self._bufs.values():
            self.rt.free(p)
        self._bufs.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.free()


def run_sequence(rt: Runtime, ops, x_dev: int, sync: bool = True) -> int:
    """Queue a chain of device-pointer -> device-pointer operators and sync once."""
    for op in ops:
        x_dev = op(x_dev)
    if sync:
        rt.sync()
    return x_dev


# weight format -> kernel, block size and table pointers (only the INT4 entry of the
# reference's table, model.py:189-203, belongs to this path)
QUANT_SPECS: dict[str, dict] = {
    "int4": dict(kernel="int4_dot_k", elems=128, block_bytes=64, tables=("scale",)),
}


def _as_rows(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return x[None, :] if x.ndim == 1 else x


class DotLinear:
    """Native decode-and-dot linear layer (``int4_dot_k`` + ``reduce_blocks_k``): the
    W4A16 path.  Weights stay in the checkpoint's bytes; ``tables`` is
    ``(bf16_scale_bytes,)``.  One kernel pair per token row (reference model.py:260-277)."""

    def __init__(self, rt: Runtime, n: int, k: int, kind: str, weight_bytes, tables=(),
                 ws: Workspace | None = None, tag: str | None = None, ring: bool = True):
        if kind not in QUANT_SPECS:
            raise ValueError(f"unknown weight format {kind!r}; built here: {sorted(QUANT_SPECS)}")
        spec = QUANT_SPECS[kind]
        if k % spec["elems"]:
            raise ValueError(f"{kind}: K={k} is not a multiple of the block size {spec['elems']}")
        if len(tables) != len(spec["tables"]):
            raise ValueError(f"{kind} takes {len(spec['tables'])} table(s), got {len(tables)}")
        self.rt, self.n, self.k, self.kind, self.spec = rt, int(n), int(k), kind, spec
        self.nbpr = self.k // spec["elems"]
        self.tag = tag or f"dot_{kind}_{id(self):x}"
        self._own_ws = ws is None
        self.ws = ws or Workspace(rt)
        self.w = self.ws.upload(self.tag + ".w", weight_bytes)
        self.tables = [self.ws.upload(f"{self.tag}.t{i}", t) for i, t in enumerate(tables)]
        self.nblocks = self.n * self.nbpr
        self.partial = self.ws.buffer(self.tag + ".partial", self.nblocks * 4)
        self.ids = self.ws.upload(self.tag + ".ids", np.arange(self.n, dtype=np.uint32))
        self.m_nbpr = div_magic(self.nbpr, self.nblocks)
        self.m_rows = div_magic(self.n, self.n)
        self.ring = ring and rt.has("w4a16_decode_stream")

    def _argv(self, x_dev, rows_per_exp, magic_rpe, ids, stride, rows_per_w, magic_rpw):
        return ([self.w, int(x_dev), self.partial, self.nblocks, 64, self.nbpr, self.m_nbpr,
                 rows_per_exp, magic_rpe] + self.tables + [int(ids), stride, rows_per_w, magic_rpw])

    def _ring_table(self, x_dev: int, out: int, rows: int):
        """One validated layer-table entry per token row (same weights, its own x and y) for
        ``w4a16_decode_stream``; cached per (x, y, rows) because validating a table is a host round trip."""
        key = (int(x_dev), int(out), rows)
        if not hasattr(self, "_tables"):
            self._tables, self._status = {}, self.ws.buffer(self.tag + ".ring_status", 4)
            self.rt.memset(self._status, 0, 4)
        if key not in self._tables:
            slot = len(self._tables) % 8                     # eight table buffers of the workspace, reused in turn
            for k_old in [k for k, v in self._tables.items() if v[1] == slot]:
                del self._tables[k_old]
            dev = self.ws.buffer(f"{self.tag}.ring_table{slot}", 32 * max(rows, 4))
            self._tables[key] = (self.rt.stream_table(
                [(self.w, self.tables[0], int(x_dev) + r * self.k * 4, out + r * self.n * 4) for r in range(rows)],
                self.n, self.k, 0, dev=dev), slot)
        return self._tables[key][0]

    def forward_device(self, x_dev: int, rows: int, sync: bool = False, out_dev=None) -> int:
        out = int(out_dev) if out_dev is not None else self.ws.buffer(self.tag + ".out", rows * self.n * 4)
        stride = self.nbpr * self.spec["block_bytes"]
        if self.kind == "int4" and self.k == 5120 and self.ring and int(x_dev) % 16 == 0:
            # dense layout at K = 5120: the activation split and the bulk-copy ring, two launches for all rows
            # (the reference's dot + reduce pair per row, with its partial[N * 40] round trip, stays below)
            self.rt.launch("w4a16_decode_stream", 1, 1,
                           [self._ring_table(x_dev, out, rows), rows, self.n, self.k, 0, 0, 0, self._status, 0])
            if sync:
                self.rt.sync()
            return out
        for r in range(rows):
            self.rt.launch(self.spec["kernel"], cdiv(self.nblocks, 64), 64,
                           self._argv(int(x_dev) + r * self.k * 4, self.n, self.m_rows, self.ids, stride,
                                      self.n, self.m_rows))
            self.rt.launch("reduce_blocks_k", cdiv(self.n, 64), 64,
                           [self.partial, out + r * self.n * 4, self.n, self.nbpr])
        if sync:
            self.rt.sync()
        return out

    def forward_experts(self, x_dev: int, rows: int, ids_dev: int, stride_bytes: int, rows_per_exp: int,
                        rows_per_w: int, out_dev=None, sync: bool = False) -> int:
        """Expert-indexed form: weight group ``ids[row // rows_per_w]``, activation row
        ``row // rows_per_exp`` (reference model.py:279-298)."""
        out = int(out_dev) if out_dev is not None else self.ws.buffer(self.tag + ".out", self.n * 4)
        self.rt.launch(self.spec["kernel"], cdiv(self.nblocks, 64), 64,
                       self._argv(x_dev, rows_per_exp, div_magic(rows_per_exp, self.n), ids_dev, stride_bytes,
                                  rows_per_w, div_magic(rows_per_w, self.n)))
        self.rt.launch("reduce_blocks_k", cdiv(self.n, 64), 64, [self.partial, out, self.n, self.nbpr])
        if sync:
            self.rt.sync()
        return out

    def forward(self, x: np.ndarray, sync: bool = True):
        x = _as_rows(x)
        px = self.ws.upload(self.tag + ".x", x)
        out = self.forward_device(px, x.shape[0], sync=sync)
        if not sync:
            return out
        return self.rt.download(out, x.shape[0] * self.n, np.float32).reshape(x.shape[0], self.n)


def _gemv_w4a8_codes(rt, runner, tag, wq, ws_f16, codes, rows, n, k, out_dev, sync):
    from .rt4 import W4A8_KERNEL
    if rows not in (1, 2, 3, 4):
        raise ValueError(f"the W4A8 GEMV takes 1..4 rows of codes (got {rows})")
    ae, ao, asc, asu = (int(c) for c in codes)
    y = int(out_dev) if out_dev is not None else runner._buf(tag + ".ycodes", rows * n * 4)
    rows_per_wg = 4 * (1 if rows == 1 else 2)
    rt.launch(W4A8_KERNEL[rows], cdiv(n, rows_per_wg), 256, [wq, ws_f16, ae, ao, asc, asu, y, n, k])
    if sync:
        rt.sync()
    return y


class RT4Linear:
    """RT4 INT4 layer already on the device (``wq``, ``ws_scale`` pointers); W4A8 or W4A4
    decode for M = 1..4 (reference model.py:358-383)."""

    def __init__(self, rt: Runtime, n: int, k: int, wq: int, ws_scale: int, path: str = "w4a8",
                 runner=None, tag: str | None = None):
        from .rt4 import W4Runner
        self.rt, self.n, self.k = rt, int(n), int(k)
        self.wq, self.ws_scale, self.path = int(wq), int(ws_scale), path
        self.runner = runner or W4Runner(rt)
        self.tag = tag or f"rt4_{id(self):x}"

    def forward_device(self, x_dev: int, rows: int, sync: bool = False, out_dev=None) -> int:
        return self.runner.gemv_device(self.path, self.wq, self.ws_scale, None, self.n, self.k,
                                       x_dev=x_dev, m=rows, y_dev=out_dev, sync=sync)

    def forward_codes_device(self, codes, rows: int, out_dev=None, sync: bool = False) -> int:
        """W4A8 GEMV on activations that are already quantised: ``codes`` = (ae, ao, asc, asu) device
        pointers as ``quant_act`` / ``rmsnorm_quant_k`` / ``silu_mul_quant_k`` leave them (rows = 1..4)."""
        return _gemv_w4a8_codes(self.rt, self.runner, self.tag, self.wq, self.ws_scale, codes, rows, self.n, self.k,
                                out_dev, sync)

    def forward(self, x: np.ndarray) -> np.ndarray:
        return self.runner.gemv(self.path, self.wq, self.ws_scale, _as_rows(x), self.n, self.k)


class Int4Linear:
    """compressed-tensors INT4 layer with three paths (reference model.py:386-477):

    ``"w4a16"``  ``int4_dot_k`` on the checkpoint bytes (fp32 activations);
    ``"w4a8"``   ``quant_act`` + ``gemv_w4a8``;  ``"w4a4"``  ``quant_act4`` + ``gemv_w4a4``.

    For the last two the codes are converted once to RT4's two's-complement nibbles and
    the bf16 scales to f16 (GEMV) and to group-first f32 (GEMM).  Row counts that are a
    multiple of 128 go to the prefill GEMM — W4A4 as in the reference, or W4A8 when
    ``prefill="gemm_a8"`` — and other counts above 4 run the GEMV in chunks of 4."""

    def __init__(self, rt: Runtime, n: int, k: int, packed: bytes, scales_bf16: bytes, path: str = "w4a8",
                 ws: Workspace | None = None, tag: str | None = None, runner=None, prefill: str = "gemm"):
        from .quant import ct_int4_to_rt4, int4_scale_group_first_f32
        if path not in ("w4a16", "w4a8", "w4a4"):
            raise ValueError('path must be "w4a16", "w4a8" or "w4a4"')
        if prefill not in ("gemm", "gemm_a8", "gemv"):
            raise ValueError('prefill must be "gemm", "gemm_a8" or "gemv"')
        self.rt, self.n, self.k, self.path, self.prefill = rt, int(n), int(k), path, prefill
        self.tag = tag or f"int4_{path}_{id(self):x}"
        self._own_ws = ws is None
        self.ws = ws or Workspace(rt)
        self._dot = self._runner = None
        if path == "w4a16":
            self._dot = DotLinear(rt, n, k, "int4", packed, (scales_bf16,), self.ws, self.tag)
            return
        from .rt4 import W4Runner
        q, s16 = ct_int4_to_rt4(packed, scales_bf16)
        self.wq = self.ws.upload(self.tag + ".wq", q)
        self.ws_f16 = self.ws.upload(self.tag + ".ws", s16)
        self.wsc_gm = self.ws.upload(self.tag + ".wsc", int4_scale_group_first_f32(scales_bf16, self.n, self.k))
        self._runner = runner or W4Runner(rt)

    def forward_device(self, x_dev: int, rows: int, sync: bool = False, out_dev=None) -> int:
        if self._dot is not None:
            return self._dot.forward_device(x_dev, rows, sync=sync, out_dev=out_dev)
        y = int(out_dev) if out_dev is not None else self.ws.buffer(self.tag + ".y", rows * self.n * 4)
        run = self._runner
        if rows <= 4:
            return run.gemv_device(self.path, self.wq, self.ws_f16, None, self.n, self.k,
                                   x_dev=x_dev, y_dev=y, m=rows, sync=sync)
        if rows % 128 == 0 and self.n % 64 == 0 and self.prefill != "gemv":
            return run.gemm_device(self.wq, self.wsc_gm, None, self.n, self.k, x_dev=x_dev, c_dev=y, m=rows,
                                   sync=sync, kind="w4a8" if self.prefill == "gemm_a8" else "w4a4")
        for r0 in range(0, rows, 4):
            run.gemv_device(self.path, self.wq, self.ws_f16, None, self.n, self.k,
                            x_dev=int(x_dev) + r0 * self.k * 4, y_dev=y + r0 * self.n * 4,
                            m=min(4, rows - r0), sync=False)
        if sync:
            self.rt.sync()
        return y

    def forward_codes_device(self, codes, rows: int, out_dev=None, sync: bool = False) -> int:
        """W4A8 GEMV on activations that are already quantised (see ``RT4Linear.forward_codes_device``)."""
        if self.path != "w4a8":
            raise ValueError("pre-quantised int8 codes feed the W4A8 path only")
        return _gemv_w4a8_codes(self.rt, self._runner, self.tag, self.wq, self.ws_f16, codes, rows, self.n, self.k,
                                out_dev, sync)

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = _as_rows(x)
        px = self.ws.upload(self.tag + ".x", x)
        out = self.forward_device(px, x.shape[0], sync=True)
        return self.rt.download(out, x.shape[0] * self.n, np.float32).reshape(x.shape[0], self.n)


class NVFP4Linear:
    """NVFP4 layer: E2M1 codes ``[N,K/8]`` u32, E4M3 block scales ``[N,K/16]`` u8 and an
    f32 global scale; activations are quantised to int8 per 16-block by
    ``nvfp4_quant_act`` and multiplied by ``nvfp4_gemv<M,1>``.  The reference offers this
    path only as raw launches (docs/KERNEL_CALLING.md:637-646); the class follows the
    contract of ``Int4Linear``.  Row counts above 4 go to the prefill GEMM (``nvfp4_gemm_kernel``)."""

    def __init__(self, rt: Runtime, n: int, k: int, codes, block_scales, gscale: float,
                 ws: Workspace | None = None, tag: str | None = None):
        if k % 32:
            raise ValueError(f"NVFP4 needs K to be a multiple of 32 (got {k})")
        self.rt, self.n, self.k, self.gscale = rt, int(n), int(k), float(gscale)
        self.tag = tag or f"nvfp4_{id(self):x}"
        self._own_ws = ws is None
        self.ws = ws or Workspace(rt)
        self.wq = self.ws.upload(self.tag + ".wq", codes)
        self.wsb = self.ws.upload(self.tag + ".ws", block_scales)

    def _chunk(self, x_dev: int, m: int, y: int) -> None:
        k, half, nb4 = self.k, self.k // 2, (self.k // 16) * 4
        qa = self.ws.buffer(self.tag + ".qa", 4 * half)
        qb = self.ws.buffer(self.tag + ".qb", 4 * half)
        sc = self.ws.buffer(self.tag + ".sc", 4 * nb4)
        # one 2-D launch, grid y = token row
        self.rt.launch2d("nvfp4_quant_act", k // 16, m, 64, 1, [int(x_dev), qa, qb, sc, m, k])
        self.rt.launch(f"nvfp4_gemv<{m},1>", cdiv(self.n, 4), 256,
                       [self.wq, self.wsb, qa, qb, sc, y, self.n, k, self.gscale])

    def forward_device(self, x_dev: int, rows: int, sync: bool = False, out_dev=None) -> int:
        y = int(out_dev) if out_dev is not None else self.ws.buffer(self.tag + ".y", rows * self.n * 4)
        if rows > 4 and self.k % 128 == 0:
            # prefill: one quantiser launch over all rows, then the GEMM (the weights are streamed once)
            k, half, nb4 = self.k, self.k // 2, (self.k // 16) * 4
            qa = self.ws.buffer(self.tag + ".gqa", rows * half)
            qb = self.ws.buffer(self.tag + ".gqb", rows * half)
            sc = self.ws.buffer(self.tag + ".gsc", rows * nb4)
            self.rt.launch2d("nvfp4_quant_act", k // 16, rows, 64, 1, [int(x_dev), qa, qb, sc, rows, k])
            self.rt.launch2d("nvfp4_gemm_kernel", cdiv(self.n, 64), cdiv(rows, 64), 256, 1,
                             [self.wq, self.wsb, qa, qb, sc, y, rows, self.n, k, self.gscale])
            if sync:
                self.rt.sync()
            return y
        for r0 in range(0, rows, 4):
            self._chunk(int(x_dev) + r0 * self.k * 4, min(4, rows - r0), y + r0 * self.n * 4)
        if sync:
            self.rt.sync()
        return y

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = _as_rows(x)
        px = self.ws.upload(self.tag + ".x", x)
        out = self.forward_device(px, x.shape[0], sync=True)
        return self.rt.download(out, x.shape[0] * self.n, np.float32).reshape(x.shape[0], self.n)


class RMSNorm:
    """``y = x * rsqrt(mean(x^2) + eps) * w`` (reference model.py:480-524).  ``forward_device`` returns the
    normalised fp32 rows; ``forward_quant_device`` runs the norm and the W4A8 activation quantiser as one
    kernel (``rmsnorm_quant_k``, reference tools/gen_rmsnorm_quant.py) and returns the four ``quant_act``
    outputs, so the layer that follows needs no quantiser launch and the normalised row never reaches memory."""

    def __init__(self, rt: Runtime, dim: int, weight, eps: float = 1e-6, ws: Workspace | None = None,
                 tag: str | None = None):
        if dim % 64:
            raise ValueError(f"RMSNorm dim={dim} must be a multiple of 64")
        self.rt, self.dim, self.eps = rt, int(dim), float(eps)
        self.tag = tag or f"rms_{id(self):x}"
        self._own_ws = ws is None
        self.ws = ws or Workspace(rt)
        self.w = self.ws.upload(self.tag + ".w", np.ascontiguousarray(weight, dtype=np.float32))

    def forward_device(self, x_dev: int, rows: int, sync: bool = False) -> int:
        out = self.ws.buffer(self.tag + ".out", rows * self.dim * 4)
        self.rt.launch("rmsnorm_fast_k", rows, 64, [out, int(x_dev), self.w, self.dim, self.eps])
        if sync:
            self.rt.sync()
        return out

    def forward_quant_device(self, x_dev: int, rows: int, sync: bool = False):
        """-> (ae, ao, asc, asu) device pointers: what ``quant_act`` would leave for the normalised rows."""
        if self.dim % 128:
            raise ValueError("the fused norm + quantiser needs dim to be a multiple of 128")
        half, ng4 = rows * self.dim // 2, rows * (self.dim // 128) * 4
        bufs = [self.ws.buffer(f"{self.tag}.q{i}", n) for i, n in enumerate((half, half, ng4, ng4))]
        self.rt.launch("rmsnorm_quant_k", rows, 64, bufs + [int(x_dev), self.w, self.dim, self.eps])
        if sync:
            self.rt.sync()
        return tuple(bufs)

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = _as_rows(x)
        px = self.ws.upload(self.tag + ".x", x)
        out = self.forward_device(px, x.shape[0], sync=True)
        return self.rt.download(out, x.shape[0] * self.dim, np.float32).reshape(x.shape[0], self.dim)


class SwiGLU:
    """``y = silu(gate) * up`` (``silu_mul_k``, reference model.py:527-544)."""

    def __init__(self, rt: Runtime, ws: Workspace | None = None, tag: str = "swiglu"):
        self.rt, self.tag = rt, tag
        self._own_ws = ws is None
        self.ws = ws or Workspace(rt)

    def forward_device(self, gate_dev: int, up_dev: int, n: int, out_dev: int | None = None, sync: bool = False) -> int:
        out = int(out_dev) if out_dev is not None else self.ws.buffer(self.tag + ".out", n * 4)
        self.rt.launch("silu_mul_k", cdiv(n, 64), 64, [out, int(gate_dev), int(up_dev), n])
        if sync:
            self.rt.sync()
        return out


class MLP:
    """Gated MLP ``down(silu(gate(x)) * up(x))``, every kernel queued back to back (reference
    model.py:547-579).  When ``down`` is a W4A8 ``Int4Linear`` / ``RT4Linear`` and at most four rows are in
    flight, the gate and the quantiser of the down projection run as one kernel (``silu_mul_quant_k``): the
    reference fuses the gate into its f32 GEMV (model.py:1262-1266); with int8 activations the place to fuse
    it is the quantiser."""

    def __init__(self, rt: Runtime, gate, up, down, ws: Workspace | None = None, tag: str = "mlp", act: str = "silu"):
        if act != "silu":
            raise ValueError("MLP wraps the silu gate only")
        self.rt, self.tag = rt, tag
        self.gate, self.up, self.down = gate, up, down
        self.act = SwiGLU(rt, ws, tag + ".act")

    def _fused_down(self, rows: int) -> bool:
        return rows <= 4 and getattr(self.down, "path", None) == "w4a8" and hasattr(self.down, "forward_codes_device")

    def forward_device(self, x_dev: int, rows: int, sync: bool = False) -> int:
        h1 = self.gate.forward_device(x_dev, rows, sync=False)
        h2 = self.up.forward_device(x_dev, rows, sync=False)
        ffn = self.gate.n
        if self._fused_down(rows) and ffn % 128 == 0:
            ws = self.act.ws
            half, ng4 = rows * ffn // 2, rows * (ffn // 128) * 4
            codes = [ws.buffer(f"{self.tag}.q{i}", n) for i, n in enumerate((half, half, ng4, ng4))]
            self.rt.launch2d("silu_mul_quant_k", 1, rows, 64, 1, codes + [h1, h2, ffn])
            out = self.down.forward_codes_device(codes, rows)
        else:
            act = self.act.forward_device(h1, h2, rows * ffn, sync=False)
            out = self.down.forward_device(act, rows, sync=False)
        if sync:
            self.rt.sync()
        return out

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = _as_rows(x)
        ws = self.gate.ws
        px = ws.upload(self.tag + ".in.x", x)
        out = self.forward_device(px, x.shape[0], sync=True)
        return self.rt.download(out, x.shape[0] * self.down.n, np.float32).reshape(x.shape[0], self.down.n)


class MoECombine:
    """``y[r,:] = sum_e weights[r,e] * exp_out[e,r,:]`` (``moe_combine_k``, reference model.py:582-618).
    ``slot(e)`` is where expert e writes its ``[rows, dim]`` output."""

    def __init__(self, rt: Runtime, rows: int, dim: int, n_exp: int, ws: Workspace | None = None, tag: str = "moe"):
        self.rt, self.rows, self.dim, self.n_exp, self.tag = rt, int(rows), int(dim), int(n_exp), tag
        self._own_ws = ws is None
        self.ws = ws or Workspace(rt)
        self.exp_out = self.ws.buffer(tag + ".exp", rows * n_exp * dim * 4)
        self.weights = self.ws.buffer(tag + ".w", rows * n_exp * 4)
        self.out = self.ws.buffer(tag + ".out", rows * dim * 4)

    def slot(self, e: int) -> int:
        return self.exp_out + e * self.rows * self.dim * 4

    def forward_device(self, weights_dev: int | None = None, sync: bool = False) -> int:
        w = int(weights_dev) if weights_dev is not None else self.weights
        self.rt.launch("moe_combine_k", self.rows, 64, [self.out, self.exp_out, w, self.n_exp, self.rows, self.dim])
        if sync:
            self.rt.sync()
        return self.out

    def forward(self, exp_out: np.ndarray, weights: np.ndarray) -> np.ndarray:
        self.rt.upload(self.exp_out, np.ascontiguousarray(exp_out, dtype=np.float32))
        self.rt.upload(self.weights, np.ascontiguousarray(weights, dtype=np.float32))
        out = self.forward_device(sync=True)
        return self.rt.download(out, self.rows * self.dim, np.float32).reshape(self.rows, self.dim)


class MoEExperts:
    """Mixture-of-experts forward over token buckets (reference model.py:620-720): the host sorts the
    (token, expert) pairs of the router by expert, ``gather_rows_k`` copies each pair's input row into its
    expert's contiguous bucket, every non-empty expert runs its linear layer on its own bucket only — an
    ``Int4Linear`` / ``RT4Linear`` / ``NVFP4Linear`` / ``DotLinear`` streams its weights once for the whole
    bucket — and ``moe_combine_gather_k`` adds the weighted expert rows back per token."""

    def __init__(self, rt: Runtime, experts, rows: int, dim: int, out_dim: int, topk: int,
                 ws: Workspace | None = None, tag: str = "moe_experts"):
        if dim % 4 or out_dim % 4:
            raise ValueError(f"dim={dim} and out_dim={out_dim} must be multiples of 4 (128-bit row copies)")
        self.rt, self.experts = rt, list(experts)
        self.n_exp = len(self.experts)
        self.rows, self.dim, self.out_dim, self.topk = int(rows), int(dim), int(out_dim), int(topk)
        if topk > self.n_exp:
            raise ValueError(f"topk={topk} exceeds the number of experts {self.n_exp}")
        self.tag = tag
        self._own_ws = ws is None
        self.ws = ws or Workspace(rt)
        cap = self.rows * self.topk
        self.x_bucket = self.ws.buffer(tag + ".xb", cap * self.dim * 4)
        self.exp_bucket = self.ws.buffer(tag + ".eb", cap * self.out_dim * 4)
        self.idx = self.ws.buffer(tag + ".idx", cap * 4)
        self.base = self.ws.buffer(tag + ".base", cap * 4)
        self.weights = self.ws.buffer(tag + ".w", cap * 4)
        self.y = self.ws.buffer(tag + ".y", self.rows * self.out_dim * 4)

    def route(self, ids, weights):
        """-> ``(bucket_rows, base, weights, offsets)``: the token row of every bucket slot (buckets laid out
        expert after expert), the bucket slot of every (token, choice) pair (0 where the pair is unused —
        expert id out of range or weight 0, whose weight is then 0 as well), the f32 weights with the unused
        pairs zeroed, and the start of every expert's bucket."""
        ids = np.asarray(ids)
        w = np.array(weights, dtype=np.float32)
        if ids.shape != (self.rows, self.topk) or w.shape != ids.shape:
            raise ValueError(f"router output {ids.shape} does not match ({self.rows}, {self.topk})")
        valid = (ids >= 0) & (ids < self.n_exp) & (w != 0.0)
        w[~valid] = 0.0
        pair = np.flatnonzero(valid.reshape(-1))
        ex = ids.reshape(-1)[pair].astype(np.int64)
        order = np.argsort(ex, kind="stable")                    # bucket order: by expert, then by pair index
        counts = np.bincount(ex, minlength=self.n_exp)
        offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
        base = np.zeros(self.rows * self.topk, dtype=np.uint32)
        base[pair[order]] = np.arange(pair.size, dtype=np.uint32)
        bucket_rows = (pair[order] // self.topk).astype(np.uint32)
        return bucket_rows, base.reshape(self.rows, self.topk), w, offsets

    def forward_device(self, x_dev: int, rows: int, ids, weights, sync: bool = False) -> int:
        if rows != self.rows:
            raise ValueError(f"built for {self.rows} rows, got {rows}")
        bucket_rows, base, w, offsets = self.route(ids, weights)
        total = int(bucket_rows.size)
        if total:
            self.rt.upload(self.idx, bucket_rows)
            self.rt.launch("gather_rows_k", total, 64, [self.x_bucket, int(x_dev), self.idx, total, self.dim])
            for e, expert in enumerate(self.experts):
                lo, n = int(offsets[e]), int(offsets[e + 1] - offsets[e])
                if n:
                    expert.forward_device(self.x_bucket + lo * self.dim * 4, n,
                                          out_dev=self.exp_bucket + lo * self.out_dim * 4, sync=False)
        self.rt.upload(self.base, base)
        self.rt.upload(self.weights, w)
        # (with no pair in use every weight is 0 and the combine writes zeros; slot 0 of the bucket is read,
        # which is inside the buffer whatever it holds)
        if not total:
            self.rt.memset(self.exp_bucket, 0, self.out_dim * 4)
        self.rt.launch("moe_combine_gather_k", rows, 64,
                       [self.y, self.exp_bucket, self.weights, self.base, self.topk, rows, self.out_dim])
        if sync:
            self.rt.sync()
        return self.y

    def forward(self, x: np.ndarray, ids, weights) -> np.ndarray:
        x = _as_rows(x)
        px = self.ws.upload(self.tag + ".x", x)
        out = self.forward_device(px, x.shape[0], ids, weights, sync=True)
        return self.rt.download(out, x.shape[0] * self.out_dim, np.float32).reshape(x.shape[0], self.out_dim)


__all__ += ["RMSNorm", "SwiGLU", "MLP", "MoECombine", "MoEExperts"]


def _out_of_scope(name: str):
    def __init__(self, *a, **kw):
        raise NotImplementedError(
            f"{name} belongs to the reference's attention / sampling operators, which are outside the "
            "weight-streaming quantized linear-layer path built here")
    return type(name, (), {"__init__": __init__, "__doc__": f"Not built (outside the linear-layer path): {name}."})


for _n in ("F32Linear", "RoPE", "KVCache", "Sampler",
           "Attention", "FlashAttention", "TransformerLayer"):
    globals()[_n] = _out_of_scope(_n)
    __all__.append(_n)
