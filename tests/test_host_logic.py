"""CPU tier: host-side code of the package (no device): packers and converters against
the reference vectors, the catalog against the library's kernel table, every symbol of
include/fm_engine.h exported by the library, seeded generators, RT4 container round
trip, plan packing and argument validation."""
from __future__ import annotations

import ctypes
import json
import pathlib
import re

import numpy as np
import pytest

import cases
import w4_oracle as O
from k100lc_kernels import catalog, quant, synth
from k100lc_kernels.model import cdiv, div_magic
from k100lc_kernels.rt4 import RT4File, _div_magic
from k100lc_kernels.runtime import DEFAULT_LIB, _bits, load_library

ROOT = pathlib.Path(__file__).resolve().parents[1]


def test_host_quant_matches_reference(golden):
    arr, meta = golden
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((16, 256)) * 0.05).astype(np.float32)
    assert meta["host_quant"]["inputs_sha256"] == cases.digest(w)
    pk, sc = quant.pack_int4_group128(w)
    assert np.array_equal(np.frombuffer(pk, np.uint8), arr["host_quant.packed"])
    assert np.array_equal(np.frombuffer(sc, np.uint8), arr["host_quant.scales"])
    assert np.array_equal(quant.dequant_int4_group128(pk, sc, 16, 256), arr["host_quant.dequant"])
    q2, s2 = quant.ct_int4_to_rt4(pk, sc)
    assert np.array_equal(np.frombuffer(q2, np.uint8), arr["host_quant.rt4_q"])
    assert np.array_equal(np.frombuffer(s2, np.uint8), arr["host_quant.rt4_s"])
    assert np.array_equal(quant.int4_scale_group_first_f32(sc, 16, 256), arr["host_quant.gf"])
    # two's-complement conversion is value-preserving
    vals = O.int4_offset(np.frombuffer(pk, np.uint32).reshape(16, -1))
    assert np.array_equal(O.int4_twos(np.frombuffer(q2, np.uint32).reshape(16, -1)), vals)
    with pytest.raises(ValueError):
        quant.pack_int4_group128(np.zeros((4, 100), np.float32))


def test_nibble_and_fp_helpers():
    rng = np.random.default_rng(0)
    v = rng.integers(-8, 8, size=(5, 64))
    assert np.array_equal(quant.pack_nibbles(v), O.pack_nibbles(v))
    assert np.array_equal(quant.unpack_nibbles(quant.pack_nibbles(v)), (v & 0xF).astype(np.uint8))
    x = rng.standard_normal(4096).astype(np.float32)
    b = quant.f32_to_bf16_bits(x)
    assert np.abs(quant.bf16_bits_to_f32(b) / x - 1).max() < 2 ** -8
    assert np.array_equal(quant.e4m3_values().view(np.uint32), O.e4m3_decode(np.arange(256, dtype=np.uint8)).view(np.uint32))
    e = quant.f32_to_e4m3_bits(np.array([0.0625, 1.0, 1.0625, 3.9, 1000.0], np.float32))
    assert list(e) == [0x18, 0x38, 0x38, 0x48, 0x7E]      # tie 1.0625 -> even code, 1000 saturates at 448


def test_div_magic():
    for d, lim in ((40, 696320), (272, 4352), (17408, 17408), (3, 1000)):
        m = div_magic(d, lim) if d > 1 else 0
        i = np.arange(lim, dtype=np.uint64)
        assert np.array_equal((i * np.uint64(m)) >> np.uint64(32), i // np.uint64(d))
    assert _div_magic(272, 4352) == div_magic(272, 4352)
    assert div_magic(1, 1) == 0 and cdiv(7, 4) == 2
    with pytest.raises(ValueError):
        div_magic(1, 5)
    with pytest.raises(ValueError):
        _div_magic(1, 5)


def test_catalog_matches_library():
    """catalog.json is generated from the library's kernel table; they must not drift
    (the reference gates the same way: tools/check_all.sh:39-45)."""
    fresh = catalog.make_catalog()
    assert fresh == json.loads(catalog.CATALOG.read_text())
    names = [k["lookup"] for k in catalog.kernels()]
    for need in ("quant_act", "quant_act4", "nvfp4_quant_act", "quant_rows_fast_k", "quant_rows_k",
                 "gemv_w4a8<1,false,1>", "gemv_w4a8<4,false,2>", "gemv_w4a4<3>", "gemv_w4a4_r2_k",
                 "gemv_w4a4_r2_m3_k", "nvfp4_gemv<2,1>", "nvfp4_gemv_wide<4,2>", "int4_dot_k",
                 "reduce_blocks_k", "int4_dequant_k", "gemm_w4a4_flat", "gemm_w4a4", "gemm_w4a8"):
        assert need in names, need
    k = catalog.info("int4_dot_k")
    assert len(k["args"]) == 14 and k["kernarg_size"] == 80          # as in the reference catalog
    k = catalog.info("gemv_w4a8<1,false,1>")
    assert [a["off"] for a in k["args"]] == [0, 8, 16, 24, 32, 40, 48, 56, 60]
    with pytest.raises(KeyError):
        catalog.info("nope")


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "fm_engine.h").read_text()
    declared = sorted(set(re.findall(r"\b(fm_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) >= 35
    lib = ctypes.CDLL(str(DEFAULT_LIB))
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/fm_engine.h but not exported"
    lib = load_library()
    assert lib.fm_has_kernel(b"quant_act") == 1 and lib.fm_has_kernel(b"nope") == 0
    assert lib.fm_kernel_id(b"nope") == -1
    kid = lib.fm_kernel_id(b"gemv_w4a4<1>")
    assert lib.fm_kernel_name(kid) == b"gemv_w4a4<1>" and lib.fm_kernel_nargs(kid) == 7
    # argument validation that needs no device
    layout = (ctypes.c_uint32 * 6)(0, 8, 0, 8, 4, 0)
    argv = (ctypes.c_uint64 * 2)()
    assert lib.fm_launch_dyn(b"quant_act", 1, 1, 32, 1, layout, 2, 0, 0, 2048, argv, 2) == -3
    assert lib.fm_launch_dyn(b"quant_act", 1, 1, 32, 1, layout, 2, 0, 0, 64, argv, 1) == -2


def test_argv_bit_packing():
    assert _bits(1.0) == 0x3F800000 and _bits(np.float32(-2.0)) == 0xC0000000
    assert _bits(np.int32(7)) == 7 and _bits(2 ** 40 + 5) == 2 ** 40 + 5


def test_synth_is_deterministic_and_distributed_as_stated():
    a, b = synth.rt4_layer(64, 1024, 2, seed=1), synth.rt4_layer(64, 1024, 2, seed=1)
    assert all(np.array_equal(a[k], b[k]) for k in ("wq", "ws", "x"))
    assert a["w"].min() == -8 and a["w"].max() == 7 and a["ws"].dtype == np.float16
    assert np.array_equal(O.int4_twos(a["wq"]), a["w"])
    c = synth.w4a16_layer(32, 512, seed=0)
    assert np.array_equal(O.int4_offset(c["packed"]), c["w"]) and c["scale_bf16"].dtype == np.uint16
    f = synth.nvfp4_layer(32, 512, 1, seed=2)
    dec = quant.e4m3_values()[f["ws"]]
    assert dec.min() >= 2 ** -4 * 0.9 and dec.max() <= 4.0 and not (f["ws"] == 0x7F).any()
    g = synth.gemm_layer(64, 256, 128, seed=3)
    assert g["wsc_gf"].shape == (2, 64) and g["x"].shape == (128, 256)
    # stream blocks: the 8 row blocks of a layer are independent and reproducible
    b0, b0b, b1 = (synth.stream_layer_block(3, 0, 64, 256), synth.stream_layer_block(3, 0, 64, 256),
                   synth.stream_layer_block(3, 1, 64, 256))
    assert np.array_equal(b0["wq"], b0b["wq"]) and not np.array_equal(b0["wq"], b1["wq"])
    assert b0["wq"].shape == (8, 128) and b0["ws"].shape == (8, 2)
    assert not np.array_equal(synth.stream_layer_x(0, 256), synth.stream_layer_x(1, 256))


def test_rt4_file_roundtrip(tmp_path):
    """Write a two-tensor RT4 container and read it back through RT4File."""
    L = synth.rt4_layer(16, 256, 1, seed=9)
    q, s = L["wq"].tobytes(), L["ws"].tobytes()
    blob = q + s + b"\0" * 7
    (tmp_path / "m.rt4").write_bytes(blob)
    man = {"format": "RT4-v1", "group": 128, "tensors": [
        {"name": "l0.w", "kind": "i4", "shape": [16, 256], "group": 128, "q_off": 0, "s_off": len(q),
         "nbytes": len(q) + len(s)},
        {"name": "l0.norm", "kind": "f32", "shape": [1, 256], "q_off": 0, "s_off": 0, "nbytes": 0}]}
    (tmp_path / "m.rt4.json").write_text(json.dumps(man))
    with RT4File(tmp_path / "m.rt4") as f:
        assert f.names("i4") == ["l0.w"] and len(f.names()) == 2
        t = f.tensor("l0.w")
        assert (t.rows, t.cols, t.q_bytes, t.s_bytes) == (16, 256, 2048, 64)
        assert f.weight_bytes(t) == (q, s)
        want = L["w"].reshape(16, 2, 128).astype(np.float32) * L["ws"].astype(np.float32)[:, :, None]
        assert np.array_equal(f.dequant(t), want.reshape(16, 256))
        assert np.array_equal(f.dequant(t, rows=3, start=5), want.reshape(16, 256)[5:8])
        with pytest.raises(ValueError):
            f.weight_bytes(f.tensor("l0.norm"))
        with pytest.raises(KeyError):
            f.tensor("missing")
    with pytest.raises(ValueError):
        RT4File(tmp_path / "m.bin")
    (tmp_path / "bad.rt4").write_bytes(b"x")
    with pytest.raises(FileNotFoundError):
        RT4File(tmp_path / "bad.rt4")


def test_out_of_scope_operators_say_so():
    import k100lc_kernels as kk
    for name in ("Attention", "FlashAttention", "KVCache", "Sampler"):
        with pytest.raises(NotImplementedError):
            getattr(kk, name)()


def test_ct_int4_safetensors_reader(tmp_path):
    """A synthetic compressed-tensors checkpoint split over two files is read back row by row."""
    from k100lc_kernels.ct_int4 import CTInt4Layer, SafeTensors, write_safetensors
    rng = np.random.default_rng(3)
    n, k = 24, 256
    w = (rng.standard_normal((n, k)) * 0.03).astype(np.float32)
    packed, scales = quant.pack_int4_group128(w)
    pre = "model.layers.0.mlp.gate_proj"
    write_safetensors(tmp_path / "a.safetensors", {
        pre + ".weight_packed": ("I32", np.frombuffer(packed, np.int32).reshape(n, k // 8)),
        "other.bias": ("F32", np.zeros(7, np.float32))})
    write_safetensors(tmp_path / "b.safetensors", {
        pre + ".weight_scale": ("BF16", np.frombuffer(scales, np.uint16).reshape(n, k // 128)),
        pre + ".weight_shape": ("I64", np.array([n, k], np.int64))})
    lay = CTInt4Layer(pre, tmp_path)
    assert (lay.n, lay.k, lay.nbpr) == (n, k, 2) and "N=24" in repr(lay)
    assert lay.packed_rows() == packed and lay.scale_rows() == scales
    assert lay.packed_rows(5, 3) == packed[5 * k // 2: 8 * k // 2]
    assert np.array_equal(lay.dequant_rows(), quant.dequant_int4_group128(packed, scales, n, k))
    assert np.array_equal(lay.dequant_rows(20, 4), quant.dequant_int4_group128(packed, scales, n, k)[20:])
    st = SafeTensors(tmp_path / "a.safetensors")
    assert st.array("other.bias").shape == (7,) and pre + ".weight_packed" in st
    with pytest.raises(ValueError):
        lay.packed_rows(20, 9)
    with pytest.raises(KeyError):
        CTInt4Layer("missing.layer", tmp_path)
    with pytest.raises(ValueError):
        st.read("other.bias", 20, 20)


def test_int4_manifest_round_trip(tmp_path):
    """The manifest of a synthetic two-file checkpoint names every layer with absolute offsets that read back the
    layer's bytes, pins the file sizes, and aggregates the per-shape table."""
    from k100lc_kernels import int4_manifest as im
    from k100lc_kernels.ct_int4 import write_safetensors
    rng = np.random.default_rng(5)
    layers = {"model.layers.0.mlp.gate_proj": (24, 256), "model.layers.0.mlp.down_proj": (16, 384),
              "model.layers.1.mlp.gate_proj": (24, 256)}
    blobs = {}
    for i, (name, (n, k)) in enumerate(layers.items()):
        packed = rng.integers(0, 2**31, size=(n, k // 8)).astype(np.int32)
        scale = rng.integers(0, 2**16, size=(n, k // 128)).astype(np.uint16)
        blobs[name] = (packed, scale)
        t = {name + ".weight_packed": ("I32", packed), name + ".weight_scale": ("BF16", scale),
             name + ".weight_shape": ("I64", np.array([n, k], np.int64)), f"pad{i}": ("F32", np.zeros(3 + i, np.float32))}
        files = tmp_path / ("model-0000%d.safetensors" % (1 + i // 2))
        if files.exists():                                   # second layer of the same file: rewrite with both
            prev_name = list(layers)[i - 1]
            pp, ps = blobs[prev_name]
            t = {prev_name + ".weight_packed": ("I32", pp), prev_name + ".weight_scale": ("BF16", ps), **t}
        write_safetensors(files, t)
    rows = im.write_manifest(tmp_path, tmp_path / "m.tsv")
    assert [r.name for r in rows] == sorted(layers)
    back = im.read_manifest(tmp_path / "m.tsv", tmp_path)
    assert back == rows
    for r in back:
        packed, scale = blobs[r.name]
        p, s = im.read_layer(r, tmp_path)
        assert p == packed.tobytes() and s == scale.tobytes()
        p2, s2 = im.read_layer(r, tmp_path, 3, 5)
        assert p2 == packed[3:8].tobytes() and s2 == scale[3:8].tobytes()
    assert im.shape_table(rows)[0][:3] == (24, 256, 2)
    with open(tmp_path / "model-00001.safetensors", "ab") as f:   # a changed file voids the offsets
        f.write(b"x")
    with pytest.raises(ValueError, match="regenerate"):
        im.read_manifest(tmp_path / "m.tsv", tmp_path)


class _RecordingRuntime:
    """Stands in for Runtime where only the sequence of launches matters (no device)."""

    def __init__(self, kernels):
        self.kernels, self.launches, self._next = set(kernels), [], 4096

    def alloc(self, nbytes):
        self._next += 4096 + int(nbytes)
        return self._next

    def free(self, ptr):
        pass

    def has(self, name):
        return name in self.kernels

    def launch(self, name, grid, threads, argv):
        self.launches.append((name, grid, threads, len(argv)))

    def launch2d(self, name, gx, gy, wx, wy, argv):
        self.launches.append((name, (gx, gy), (wx, wy), len(argv)))

    def sync(self):
        pass


def test_runner_picks_the_one_launch_entry_only_where_it_applies():
    """W4Runner.gemv_device: one W4A8 token at K = 5120 / 6144 is the single launch quant_gemv_w4a8 when the library
    has it; every other case (more tokens, another K, W4A4, an older library, fused=False) keeps the reference's
    quantiser + GEMV pair; asking for the single launch on a shape it does not take is an error."""
    from k100lc_kernels.rt4 import W4Runner
    full = {"quant_gemv_w4a8", "quant_gemv_w4a4"}

    def names(kernels, kind, m, k, **kw):
        rt = _RecordingRuntime(kernels)
        W4Runner(rt).gemv_device(kind, 1, 2, None, 1000, k, x_dev=64, y_dev=128, m=m, sync=False, **kw)
        return [l[0] for l in rt.launches]

    assert names(full, "w4a8", 1, 5120) == ["quant_gemv_w4a8"]
    assert names(full, "w4a8", 1, 6144) == ["quant_gemv_w4a8"]
    assert names(full, "w4a8", 1, 5120, fused=False) == ["quant_act", "gemv_w4a8<1,false,1>"]
    assert names(set(), "w4a8", 1, 5120) == ["quant_act", "gemv_w4a8<1,false,1>"]
    assert names(full, "w4a8", 2, 5120) == ["quant_act", "gemv_w4a8<2,false,2>"]
    assert names(full, "w4a8", 1, 4096) == ["quant_act", "gemv_w4a8<1,false,1>"]
    assert names(full, "w4a4", 1, 5120) == ["quant_act4", "gemv_w4a4<1>"]
    assert names(full, "w4a4", 1, 5120, fused=True) == ["quant_gemv_w4a4"]
    with pytest.raises(ValueError, match="one token"):
        names(full, "w4a8", 3, 5120, fused=True)
    with pytest.raises(ValueError, match="one token"):
        names(full, "w4a8", 1, 1024, fused=True)
    with pytest.raises(ValueError, match="unknown W4 path"):
        names(full, "w8a8", 1, 5120)


def test_stage_split_deals_out_every_row_once():
    """fm_stream_rows (the function the stream kernels call with their own block index): for every layer the CTAs'
    ranges are disjoint and cover [0, rows); every range is whole 16-row stages except the end of the layer; stage
    counts of two CTAs differ by at most one; the chunks of a weight matrix (same `first`) are split alike; over a
    run of layers the extra stages are spread evenly over the CTAs."""
    lib = load_library()
    r0, r1 = ctypes.c_int(), ctypes.c_int()

    def split(rows, first, grid):
        out = []
        for cta in range(grid):
            assert lib.fm_stream_rows(rows, first, grid, cta, ctypes.byref(r0), ctypes.byref(r1)) == 0
            out.append((r0.value, r1.value))
        return out

    for rows, grid in ((17408, 148), (5120, 148), (2176, 148), (1024, 148), (7111, 148), (37, 37), (1, 1), (300, 148),
                       (8704, 132), (100000, 148), (16, 148), (17, 2)):
        for first in (0, 1, 2, 5, 77, 399, 655, 10_000):
            parts = split(rows, first, grid)
            covered = sorted(p for p in parts if p[1] > p[0])
            assert covered[0][0] == 0 and covered[-1][1] == rows
            assert all(a[1] == b[0] for a, b in zip(covered, covered[1:])), (rows, grid, first)
            assert all((a % 16 == 0 or a == rows) and (b % 16 == 0 or b == rows) for a, b in parts)   # (empty ranges sit at `rows`)
            stages = [-(-(b - a) // 16) for a, b in parts]
            assert max(stages) - min(stages) <= 1 and sum(stages) == -(-rows // 16)
            assert parts == split(rows, first, grid)                                    # the chunks of a matrix: same ranges
    # 400 layers of 17408 rows on 148 CTAs: 1088 stages per layer, 52 CTAs get one more than the others; over the
    # launch every CTA ends within a fraction of a per cent of the mean
    total = np.zeros(148, np.int64)
    for layer in range(400):
        total += np.array([-(-(b - a) // 16) for a, b in split(17408, layer, 148)])
    assert total.sum() == 400 * 1088 and (total.max() - total.min()) <= 0.01 * total.mean()
    # arguments out of range
    for bad in ((0, 0, 148, 0), (100, -1, 148, 0), (100, 0, 0, 0), (100, 0, 148, 148), (100, 0, 148, -1)):
        assert lib.fm_stream_rows(*bad, ctypes.byref(r0), ctypes.byref(r1)) == -1
