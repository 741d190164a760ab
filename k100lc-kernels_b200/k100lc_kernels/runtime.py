"""By-name kernel launch on a resident engine: the ``Runtime`` / ``LaunchPlan`` surface
of the reference package (python/k100lc_kernels/runtime.py) over ``libfm_engine.so``
built for B200.

Same public methods, argument meaning and error behaviour as the reference:
``alloc/free/upload/download/copy_dev/memset/launch/launch2d/launch_dyn/launch_any/
has/sync/batch`` (runtime.py:219-352) and ``LaunchPlan`` (runtime.py:50-103).  Device
pointers are plain Python integers, so byte offsets can be added to them.  There is no
CPU fallback: constructing a ``Runtime`` without the CUDA library or without a B200
raises.

Additions that the reference does not have are grouped at the end of the class
(``last_error``, device timers, pinned buffers, explicit graphs, the NCCL communicator).
"""
from __future__ import annotations

import ctypes
import json
import os
import pathlib
import struct

import numpy as np

PKG_DIR = pathlib.Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
DEFAULT_LIB = ROOT / "lib" / "libfm_engine.so"
# The reference loads its kernels from a code-object file and calls it ``hsaco``; here
# the kernels are linked into the library, and the argument names that library.
DEFAULT_HSACO = DEFAULT_LIB

_u64p = ctypes.POINTER(ctypes.c_uint64)
_u32p = ctypes.POINTER(ctypes.c_uint32)

_KIND_CODES = {"by_value": 0, "global_buffer": 0}


def _bits(value) -> int:
    """argv encoding (reference runtime.py:184-205): floats travel as their f32 bit
    pattern in the low four bytes, everything else as an integer."""
    if isinstance(value, (float, np.floating)):
        return struct.unpack("<I", struct.pack("<f", float(value)))[0]
    return int(value) & 0xFFFFFFFFFFFFFFFF


def load_library(path=None) -> ctypes.CDLL:
    """Open the engine and declare every symbol of ``include/fm_engine.h``."""
    path = pathlib.Path(path or os.environ.get("FM_ENGINE_LIB") or DEFAULT_LIB)
    if not path.is_file():
        raise RuntimeError(
            f"{path} not found: build it with `python {ROOT / 'build.py'}` "
            "(there is no CPU fallback for the kernels)")
    lib = ctypes.CDLL(str(path))
    c = ctypes
    sig = {
        "fm_init": (c.c_int, [c.c_char_p]),
        "fm_alloc": (c.c_void_p, [c.c_size_t]),
        "fm_free": (None, [c.c_void_p]),
        "fm_upload": (c.c_int, [c.c_void_p, c.c_void_p, c.c_size_t]),
        "fm_download": (c.c_int, [c.c_void_p, c.c_void_p, c.c_size_t]),
        "fm_copy": (c.c_int, [c.c_void_p, c.c_void_p, c.c_size_t]),
        "fm_memset": (c.c_int, [c.c_void_p, c.c_int, c.c_size_t]),
        "fm_sync": (c.c_int, []),
        "fm_launch": (c.c_int, [c.c_char_p, c.c_uint32, c.c_uint32, _u64p, c.c_int]),
        "fm_launch2d": (c.c_int, [c.c_char_p, c.c_uint32, c.c_uint32, c.c_uint32, c.c_uint32, _u64p, c.c_int]),
        "fm_launch_dyn": (c.c_int, [c.c_char_p, c.c_uint32, c.c_uint32, c.c_uint32, c.c_uint32, _u32p,
                                    c.c_uint32, c.c_uint32, c.c_uint32, c.c_uint32, _u64p, c.c_int]),
        "fm_has_kernel": (c.c_int, [c.c_char_p]),
        "fm_kernel_id": (c.c_int, [c.c_char_p]),
        "fm_launch_batch": (c.c_int, [_u64p, c.c_int]),
        "fm_last_error": (c.c_char_p, []),
        "fm_device_count": (c.c_int, []),
        "fm_set_device": (c.c_int, [c.c_int]),
        "fm_device_attr": (c.c_int, [c.c_int]),
        "fm_kernel_count": (c.c_int, []),
        "fm_kernel_name": (c.c_char_p, [c.c_int]),
        "fm_kernel_nargs": (c.c_int, [c.c_int]),
        "fm_kernel_sig": (c.c_char_p, [c.c_int]),
        "fm_launch_count": (c.c_ulonglong, []),
        "fm_host_alloc": (c.c_void_p, [c.c_size_t]),
        "fm_host_free": (None, [c.c_void_p]),
        "fm_upload_async": (c.c_int, [c.c_void_p, c.c_void_p, c.c_size_t]),
        "fm_download_async": (c.c_int, [c.c_void_p, c.c_void_p, c.c_size_t]),
        "fm_upload_beside": (c.c_int, [c.c_void_p, c.c_void_p, c.c_size_t]),
        "fm_upload_join": (c.c_int, []),
        "fm_copy_beside": (c.c_int, [c.c_void_p, c.c_void_p, c.c_size_t]),
        "fm_download_beside": (c.c_int, [c.c_void_p, c.c_size_t, c.c_void_p, c.c_size_t, c.c_size_t, c.c_size_t]),
        "fm_download_join": (c.c_int, [c.c_int]),
        "fm_stream_table_var": (c.c_int, [c.c_void_p, c.c_void_p, c.POINTER(c.c_uint64), c.c_int]),
        "fm_stream_rows": (c.c_int, [c.c_int, c.c_int, c.c_int, c.c_int, c.POINTER(c.c_int), c.POINTER(c.c_int)]),
        "fm_event_create": (c.c_int, []),
        "fm_event_record": (c.c_int, [c.c_int]),
        "fm_event_elapsed_ms": (c.c_float, [c.c_int, c.c_int]),
        "fm_graph_begin": (c.c_int, []),
        "fm_graph_end": (c.c_int, []),
        "fm_graph_launch": (c.c_int, [c.c_int]),
        "fm_graph_free": (c.c_int, [c.c_int]),
        "fm_comm_unique_id": (c.c_int, [c.c_void_p]),
        "fm_comm_init": (c.c_int, [c.c_void_p, c.c_int, c.c_int]),
        "fm_comm_rank": (c.c_int, []),
        "fm_comm_size": (c.c_int, []),
        "fm_allgather": (c.c_int, [c.c_void_p, c.c_void_p, c.c_size_t]),
        "fm_comm_destroy": (c.c_int, []),
        "fm_stream_table": (c.c_int, [c.c_void_p, _u64p, c.c_int, c.c_int, c.c_int, c.c_int]),
        "fm_gemm_status": (c.c_int, []),
        "fm_stream_status": (c.c_int, []),
        "fm_ipc_export": (c.c_int, [c.c_void_p, c.c_void_p, c.POINTER(c.c_ulonglong), c.POINTER(c.c_ulonglong)]),
        "fm_ipc_import": (c.c_void_p, [c.c_void_p, c.c_ulonglong]),
        "fm_stream_peers": (c.c_int, [c.c_void_p, _u64p, c.c_int, c.c_void_p, c.c_ulonglong]),
        "fm_w4a8_linear_static": (c.c_int, [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int,
                                            c.c_int, c.c_void_p, c.c_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)          # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


class _BatchScope:
    """``with rt.batch():`` — launches inside are recorded and handed to the engine as
    one plan on exit (reference runtime.py:30-47, 267-298)."""

    def __init__(self, rt: "Runtime"):
        self._rt = rt

    def __enter__(self):
        if self._rt._pending is not None:
            raise RuntimeError("batch() scopes do not nest")
        self._rt._pending = []
        return self

    def __exit__(self, exc_type, exc, tb):
        calls, self._rt._pending = self._rt._pending, None
        if exc_type is None and calls:
            LaunchPlan(self._rt, calls).run()
        return False


class LaunchPlan:
    """Record a list of launches once, replay it many times (reference
    runtime.py:50-103).  ``calls`` is ``[(kernel, grid, workgroup, argv), ...]``.  The
    flat ``uint64`` plan can be patched between runs with ``set_arg`` / ``set_grid``;
    the engine replays an unchanged plan as a CUDA graph and re-captures a patched one."""

    def __init__(self, rt: "Runtime", calls: list):
        self.rt = rt
        self.n = len(calls)
        words: list[int] = []
        self.starts: list[int] = []
        self._kids: list[int] = []
        for kernel, grid, wg, argv in calls:
            kid = rt._kernel_id(kernel)
            if kid < 0:
                raise RuntimeError(f"fm_kernel_id({kernel}) failed: no such kernel")
            self._kids.append(kid)
            words += [kid, int(grid), int(wg), len(argv)]
            self.starts.append(len(words))
            words += [_bits(v) for v in argv]
        self.buf = (ctypes.c_uint64 * max(1, len(words)))(*words)

    def set_arg(self, rec: int, idx: int, value) -> None:
        self.buf[self.starts[rec] + idx] = _bits(value)

    def set_grid(self, rec: int, grid: int) -> None:
        self.buf[self.starts[rec] - 3] = int(grid)

    @property
    def kernels(self) -> list:
        return [self.rt._names_by_id.get(k, "?") for k in self._kids]

    def run(self) -> int:
        got = self.rt._lib.fm_launch_batch(self.buf, self.n)
        if got != self.n:
            raise RuntimeError(f"fm_launch_batch enqueued {got}/{self.n} records: {self.rt.last_error()}")
        return got


# One engine per process, like the reference (runtime.py:106-123): a second Runtime that
# names another kernel image would silently keep running the first one, so it is refused.
_BOUND_IMAGE: pathlib.Path | None = None


class Runtime:
    """Resident engine: device buffers are allocated once and kernels are launched by
    name.  ``hsaco`` and ``lib`` both default to the in-tree ``libfm_engine.so``."""

    def __init__(self, hsaco=None, lib=None, catalog=None):
        global _BOUND_IMAGE
        image = pathlib.Path(os.environ.get("RT_HSACO") or hsaco or lib or os.environ.get("FM_ENGINE_LIB") or DEFAULT_HSACO)
        self._lib = load_library(lib or (image if image.suffix == ".so" else None))
        if _BOUND_IMAGE is not None and _BOUND_IMAGE.resolve() != image.resolve():
            raise RuntimeError(
                f"this process already runs the kernel image {_BOUND_IMAGE}; the engine is "
                f"process-global and would ignore {image}. Start a new process to switch images.")
        if self._lib.fm_init(str(image).encode()) != 0:
            raise RuntimeError(f"fm_init failed: {self.last_error()}")
        _BOUND_IMAGE = image
        self.hsaco = image
        self.catalog = self._read_catalog(catalog)
        self._enc: dict[str, bytes] = {}
        self._ids: dict[str, int] = {}
        self._names_by_id: dict[int, str] = {}
        self._pending: list | None = None
        self._argv = (ctypes.c_uint64 * 32)()

    # ---- helpers ---------------------------------------------------------------
    def _name(self, kernel: str) -> bytes:
        b = self._enc.get(kernel)
        if b is None:
            b = self._enc[kernel] = kernel.encode()
        return b

    def _kernel_id(self, kernel: str) -> int:
        kid = self._ids.get(kernel)
        if kid is None:
            kid = self._ids[kernel] = int(self._lib.fm_kernel_id(self._name(kernel)))
            self._names_by_id[kid] = kernel
        return kid

    def _pack(self, argv):
        n = len(argv)
        if n > len(self._argv):
            self._argv = (ctypes.c_uint64 * n)()
        buf = self._argv
        for i, v in enumerate(argv):
            buf[i] = _bits(v)
        return buf

    def _read_catalog(self, catalog):
        path = pathlib.Path(catalog) if catalog is not None else PKG_DIR / "catalog.json"
        if path.is_file():
            return json.loads(path.read_text(encoding="utf-8"))
        return {"kernels": []}

    def _fail(self, what: str):
        raise RuntimeError(f"{what} failed: {self.last_error()}")

    # ---- memory ----------------------------------------------------------------
    def alloc(self, nbytes: int) -> int:
        p = self._lib.fm_alloc(int(nbytes))
        if not p:
            raise MemoryError(f"fm_alloc({nbytes}) failed")
        return int(p)

    def free(self, ptr: int) -> None:
        self._lib.fm_free(ctypes.c_void_p(int(ptr)))

    def upload(self, ptr: int, data) -> None:
        if isinstance(data, np.ndarray):
            arr = np.ascontiguousarray(data)
            src, n = arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes
        else:
            raw = bytes(data)
            src, n = ctypes.cast(ctypes.c_char_p(raw), ctypes.c_void_p), len(raw)
        if self._lib.fm_upload(ctypes.c_void_p(int(ptr)), src, n) != 0:
            self._fail("fm_upload")

    def download(self, ptr: int, count: int, dtype) -> np.ndarray:
        dt = np.dtype(dtype)
        out = np.empty(int(count), dtype=dt)
        if self._lib.fm_download(out.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(int(ptr)),
                                 out.nbytes) != 0:
            self._fail("fm_download")
        return out

    def copy_dev(self, dst: int, src: int, nbytes: int) -> None:
        if self._lib.fm_copy(ctypes.c_void_p(int(dst)), ctypes.c_void_p(int(src)), int(nbytes)) != 0:
            self._fail("fm_copy")

    def memset(self, ptr: int, value: int, nbytes: int) -> None:
        if self._lib.fm_memset(ctypes.c_void_p(int(ptr)), int(value), int(nbytes)) != 0:
            self._fail("fm_memset")

    # ---- launches --------------------------------------------------------------
    def launch(self, kernel: str, grid: int, workgroup: int, argv: list) -> None:
        if self._pending is not None:
            self._pending.append((kernel, int(grid), int(workgroup), [_bits(v) for v in argv]))
            return
        rc = self._lib.fm_launch(self._name(kernel), int(grid), int(workgroup), self._pack(argv), len(argv))
        if rc != 0:
            raise RuntimeError(f"fm_launch({kernel}) failed rc={rc}: {self.last_error()}")

    def launch2d(self, kernel: str, gx: int, gy: int, wx: int, wy: int, argv: list) -> None:
        rc = self._lib.fm_launch2d(self._name(kernel), int(gx), int(gy), int(wx), int(wy),
                                   self._pack(argv), len(argv))
        if rc != 0:
            raise RuntimeError(f"fm_launch2d({kernel}) failed rc={rc}: {self.last_error()}")

    def batch(self) -> _BatchScope:
        return _BatchScope(self)

    def _find(self, kernel: str) -> dict:
        for k in self.catalog.get("kernels", []):
            if kernel in (k.get("lookup"), k.get("name")):
                return k
        raise KeyError(f"kernel {kernel} is not in the catalog")

    def launch_dyn(self, kernel: str, gx: int, gy: int, wx: int, wy: int, argv: list) -> None:
        """Launch through the catalog entry's argument layout (reference
        runtime.py:314-334)."""
        k = self._find(kernel)
        args = k["args"]
        layout = (ctypes.c_uint32 * (3 * len(args)))()
        for i, a in enumerate(args):
            layout[3 * i] = int(a.get("off", 0))
            layout[3 * i + 1] = int(a.get("size", 0))
            layout[3 * i + 2] = _KIND_CODES.get(str(a.get("kind", "by_value")), 1)
        rc = self._lib.fm_launch_dyn(str(k.get("lookup", kernel)).encode(), int(gx), int(gy), int(wx), int(wy),
                                     layout, len(args), int(k.get("group_segment", 0)),
                                     int(k.get("private_segment", 0)), int(k.get("kernarg_size", 0)),
                                     self._pack(argv), len(argv))
        if rc != 0:
            raise RuntimeError(f"fm_launch_dyn({kernel}) failed rc={rc}: {self.last_error()}")

    def launch_any(self, kernel: str, grid: int, workgroup: int, argv: list) -> None:
        try:
            self.launch_dyn(kernel, grid, 1, workgroup, 1, argv)
        except KeyError:
            self.launch(kernel, grid, workgroup, argv)

    def has(self, kernel: str) -> bool:
        return bool(self._lib.fm_has_kernel(kernel.encode()))

    def sync(self) -> None:
        if self._lib.fm_sync() != 0:
            self._fail("fm_sync")

    # ---- additions (not in the reference) --------------------------------------
    def last_error(self) -> str:
        msg = self._lib.fm_last_error()
        return msg.decode(errors="replace") if msg else ""

    def device_attr(self, what: str) -> int:
        return int(self._lib.fm_device_attr({"sm_count": 0, "l2_bytes": 1, "device": 2,
                                             "mem_mib": 3, "clock_khz": 4}[what]))

    def launch_count(self) -> int:
        return int(self._lib.fm_launch_count())

    def event(self) -> int:
        ev = self._lib.fm_event_create()
        if ev < 0:
            self._fail("fm_event_create")
        return ev

    def record(self, ev: int) -> None:
        if self._lib.fm_event_record(ev) != 0:
            self._fail("fm_event_record")

    def elapsed_ms(self, start: int, stop: int) -> float:
        ms = float(self._lib.fm_event_elapsed_ms(start, stop))
        if ms < 0:
            self._fail("fm_event_elapsed_ms")
        return ms

    def pinned(self, shape, dtype) -> np.ndarray:
        """A NumPy array backed by page-locked host memory; it lives as long as the process
        unless it is handed to ``free_pinned``."""
        dt = np.dtype(dtype)
        n = int(np.prod(shape)) * dt.itemsize
        p = self._lib.fm_host_alloc(max(n, 1))
        if not p:
            raise MemoryError(f"fm_host_alloc({n}) failed")
        raw = (ctypes.c_char * max(n, 1)).from_address(p)
        return np.frombuffer(raw, dtype=dt, count=int(np.prod(shape))).reshape(shape)

    def free_pinned(self, arr: np.ndarray) -> None:
        """Release a ``pinned`` array (the array must not be used afterwards).  Peer-offset arrays
        that name it as a receiver stop being valid."""
        self._lib.fm_host_free(ctypes.c_void_p(int(arr.ctypes.data)))

    def upload_async(self, ptr: int, arr: np.ndarray) -> None:
        if self._lib.fm_upload_async(ctypes.c_void_p(int(ptr)), arr.ctypes.data_as(ctypes.c_void_p),
                                     arr.nbytes) != 0:
            self._fail("fm_upload_async")

    def upload_beside(self, ptr: int, arr: np.ndarray) -> None:
        """Upload on the engine's second queue: starts when the work enqueued so far has finished, runs
        beside what is enqueued next; ``upload_join`` makes later launches wait for it."""
        if self._lib.fm_upload_beside(ctypes.c_void_p(int(ptr)), arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes) != 0:
            self._fail("fm_upload_beside")

    def copy_beside(self, dst: int, src: int, nbytes: int) -> None:
        """Device-to-device copy on the second queue (``dst`` may be a peer's imported allocation)."""
        if self._lib.fm_copy_beside(ctypes.c_void_p(int(dst)), ctypes.c_void_p(int(src)), int(nbytes)) != 0:
            self._fail("fm_copy_beside")

    def upload_join(self) -> None:
        if self._lib.fm_upload_join() != 0:
            self._fail("fm_upload_join")

    def download_beside(self, arr: np.ndarray, ptr: int, width: int | None = None, height: int = 1,
                        dpitch: int = 0, hpitch: int = 0, host_offset: int = 0) -> None:
        """Download on the engine's third queue: starts when the work enqueued so far has finished, runs beside
        what is enqueued next.  Plain form: all of ``arr``.  2-D form: ``height`` rows of ``width`` bytes, rows
        ``dpitch`` / ``hpitch`` bytes apart on the device / in ``arr``, starting ``host_offset`` bytes into ``arr``."""
        if width is None:
            width, height = arr.nbytes, 1
        elif host_offset + (height - 1) * hpitch + width > arr.nbytes:
            raise ValueError("download_beside: the rows do not fit the host array")
        if self._lib.fm_download_beside(ctypes.c_void_p(int(arr.ctypes.data) + int(host_offset)), int(hpitch),
                                        ctypes.c_void_p(int(ptr)), int(dpitch), int(width), int(height)) != 0:
            self._fail("fm_download_beside")

    def download_join(self, lag: int = 0) -> None:
        """Later launches wait for the ``download_beside`` issued ``lag`` calls before the latest."""
        if self._lib.fm_download_join(int(lag)) != 0:
            self._fail("fm_download_join")

    def download_async(self, arr: np.ndarray, ptr: int) -> None:
        if self._lib.fm_download_async(arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(int(ptr)),
                                       arr.nbytes) != 0:
            self._fail("fm_download_async")

    def graph_begin(self) -> None:
        if self._lib.fm_graph_begin() != 0:
            self._fail("fm_graph_begin")

    def graph_end(self) -> int:
        g = self._lib.fm_graph_end()
        if g < 0:
            self._fail("fm_graph_end")
        return g

    def graph_launch(self, graph: int) -> None:
        if self._lib.fm_graph_launch(graph) != 0:
            self._fail("fm_graph_launch")

    def graph_free(self, graph: int) -> None:
        self._lib.fm_graph_free(graph)

    def stream_table(self, layers, rows: int, k: int, row_base: int = 0, dev: int | None = None) -> int:
        """Validated device table for ``w4a8_decode_stream``: ``layers`` is a list of
        ``(wq, ws, x, y)`` device pointers; returns the table's device pointer (a fresh allocation of
        32 bytes per layer unless ``dev`` names a buffer of that size)."""
        flat = (ctypes.c_uint64 * (4 * len(layers)))(*[int(v) for lay in layers for v in lay])
        own = dev is None
        dev = self.alloc(32 * len(layers)) if own else int(dev)
        if self._lib.fm_stream_table(ctypes.c_void_p(dev), flat, len(layers), int(rows), int(k), int(row_base)) != 0:
            if own:
                self.free(dev)
            self._fail("fm_stream_table")
        return dev

    @staticmethod
    def layer_chunks(wq: int, ws: int, y: int, ae: int, ao: int, asc: int, asu: int, rows: int, k: int,
                     row_base: int = 0) -> list:
        """The entries of ``stream_table_var`` for one W4A8 weight matrix ``[rows, k]`` (k a multiple of 1024): one
        entry per 5120 k, the later ones adding to ``y``.  ``ae, ao, asc, asu`` are the outputs of ``quant_act`` for
        this matrix's input, in arrays padded with zeros to a multiple of 5120 k (2560-byte codes, 40 scales / sums
        per chunk)."""
        if k % 1024:
            raise ValueError("layer_chunks: K must be a multiple of 1024")
        out = []
        for c in range(-(-k // 5120)):
            kc = min(5120, k - 5120 * c)
            out.append((wq + c * 2560, ws + c * 80, 0, y, ae + c * 2560, ao + c * 2560, asc + c * 160, asu + c * 160,
                        rows, k // 2, (k // 128) * 2, kc // 2, (kc // 128) * 2, 1 if c else 0, row_base, c))
        return out

    def stream_table_var(self, entries) -> tuple[int, int]:
        """Validated layer table and shape array for ``w4a8_layers_stream``: ``entries`` is a list of 16-tuples as
        ``layer_chunks`` makes them.  Returns the two device pointers (fresh allocations: 32 and 64 bytes per entry)."""
        n = len(entries)
        flat = (ctypes.c_uint64 * (16 * n))(*[int(v) for ent in entries for v in ent])
        table, shapes = self.alloc(32 * n), self.alloc(64 * n)
        if self._lib.fm_stream_table_var(ctypes.c_void_p(table), ctypes.c_void_p(shapes), flat, n) != 0:
            self.free(table)
            self.free(shapes)
            self._fail("fm_stream_table_var")
        return table, shapes

    def stream_rows(self, rows: int, first: int, grid: int, cta: int) -> tuple[int, int]:
        """Rows ``[r0, r1)`` of a layer that CTA ``cta`` of ``grid`` computes where whole 16-row stages are dealt out
        (``first``: table index of the layer, or of the first chunk of its weight matrix)."""
        r0, r1 = ctypes.c_int(), ctypes.c_int()
        if self._lib.fm_stream_rows(int(rows), int(first), int(grid), int(cta), ctypes.byref(r0), ctypes.byref(r1)) != 0:
            self._fail("fm_stream_rows")
        return r0.value, r1.value

    def gemm_status(self) -> int:
        """Sync, then 0 or the code of a bounded wait that ran out in a GEMM kernel."""
        return int(self._lib.fm_gemm_status())

    def stream_status(self) -> int:
        """Sync, then 0 or the code of a bounded wait that ran out in a by-name GEMV that runs on the ring."""
        return int(self._lib.fm_stream_status())

    def ipc_export(self, ptr: int) -> tuple[bytes, int, int]:
        """(64-byte IPC handle, offset of ptr in its allocation, allocation size)."""
        h = ctypes.create_string_buffer(64)
        off, size = ctypes.c_ulonglong(), ctypes.c_ulonglong()
        if self._lib.fm_ipc_export(ctypes.c_void_p(int(ptr)), h, ctypes.byref(off), ctypes.byref(size)) != 0:
            self._fail("fm_ipc_export")
        return h.raw, int(off.value), int(size.value)

    def ipc_import(self, handle: bytes, size: int) -> int:
        p = self._lib.fm_ipc_import(ctypes.c_char_p(handle), int(size))
        if not p:
            self._fail("fm_ipc_import")
        return int(p)

    def stream_peers(self, peer_bases, local_base: int, span: int) -> int:
        """Validated device array of byte offsets (peer - local) for ``w4a8_decode_stream``."""
        n = len(peer_bases)
        dev = self.alloc(8 * n)
        arr = (ctypes.c_uint64 * n)(*[int(b) for b in peer_bases])
        if self._lib.fm_stream_peers(ctypes.c_void_p(dev), arr, n, ctypes.c_void_p(int(local_base)), int(span)) != 0:
            self.free(dev)
            self._fail("fm_stream_peers")
        return dev

    def comm_unique_id(self) -> bytes:
        buf = ctypes.create_string_buffer(128)
        if self._lib.fm_comm_unique_id(buf) != 0:
            self._fail("fm_comm_unique_id")
        return buf.raw

    def comm_init(self, uid: bytes, nranks: int, rank: int) -> None:
        if self._lib.fm_comm_init(ctypes.c_char_p(uid), int(nranks), int(rank)) != 0:
            self._fail("fm_comm_init")

    def allgather(self, recv: int, send: int, bytes_per_rank: int) -> None:
        if self._lib.fm_allgather(ctypes.c_void_p(int(recv)), ctypes.c_void_p(int(send)),
                                  int(bytes_per_rank)) != 0:
            self._fail("fm_allgather")

    def comm_destroy(self) -> None:
        self._lib.fm_comm_destroy()
