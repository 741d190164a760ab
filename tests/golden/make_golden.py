#!/usr/bin/env python3
"""Generate ``reference_vectors.npz`` / ``reference_vectors.json`` from the
reference project's own NumPy oracle.

Run where the reference checkout is mounted:

    python tests/golden/make_golden.py --reference /path/to/K100LC-kernels

The script imports the reference's ``tools/selftest_all.py``,
``tools/gen_int4_dot.py``, ``tools/gen_rmsnorm_quant.py`` and ``python/k100lc_kernels/quant.py`` (no device is
touched: the reference only opens its runtime inside ``main()``), feeds them the
seeded inputs of ``tests/cases.py`` and stores the outputs plus the SHA-256 of
the inputs.  The tests re-create the inputs from the same seeds, check the
digest, and compare ``oracle/w4_oracle.py`` against the stored outputs; the
fixtures therefore travel to machines where the reference does not exist.
"""
from __future__ import annotations

import argparse
import json
import pathlib
import sys

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import cases  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    ref_root = pathlib.Path(args.reference)
    sys.path.insert(0, str(ref_root / "tools"))
    sys.path.insert(0, str(ref_root / "python"))
    import selftest_all as st          # reference test oracle
    import gen_int4_dot as gid         # reference W4A16 host reference
    import gen_rmsnorm_quant as grq    # reference host check of the fused norm + quantiser
    from k100lc_kernels import quant as rq   # reference host pack/convert

    out: dict[str, np.ndarray] = {}
    meta: dict[str, dict] = {}

    def put(case: str, digest: str, **arrays):
        meta[case] = {"inputs_sha256": digest, "fields": sorted(arrays)}
        for k, v in arrays.items():
            out[f"{case}.{k}"] = np.ascontiguousarray(v)

    # ---- W4A4 / W4A8 GEMV (selftest seeds 60-63, plus M=2,3 which the reference
    #      functions support although its tests do not use them) ----
    for case, seed, m, kind in (("w4a4_m1", 60, 1, 4), ("w4a4_m4", 61, 4, 4),
                                ("w4a4_r2_m4", 62, 4, 4), ("w4a8_m1", 63, 1, 8),
                                ("w4a8_m2", 163, 2, 8), ("w4a8_m3", 164, 3, 8),
                                ("w4a8_m4", 165, 4, 8), ("w4a4_m2", 166, 2, 4),
                                ("w4a4_m3", 167, 3, 4)):
        wv, ws, x = cases.w4_case(seed, 256, 5120, m)
        if kind == 4:
            qa, asc = st.quant_act4_ref(x)
            y = st.w4_gemv_ref(st.pack_int4_lo(wv), ws, qa, asc, 5120, 32)
        else:
            qa, asc = st.quant_act_ref(x)
            y = st.w4_gemv_ref(st.pack_int4_lo(wv), ws, qa, asc, 5120, 128)
        put(case, cases.digest(wv, ws, x), y=y, asc=asc, qa=qa.astype(np.int8))

    # ---- quantisers, bit-exact (selftest seeds 70-73, 90) ----
    x = cases.normal_case(70, 32, 512)
    q, sc = st.quant_rows_ref(x, 512, 128)
    put("quant_rows_fast", cases.digest(x), q=q, sc=sc)
    x = cases.normal_case(73, 32, 512)
    q, sc = st.quant_rows_ref(x, 512, 128)
    put("quant_rows", cases.digest(x), q=q, sc=sc)
    x = cases.normal_case(71, 1, 5120)
    q, s = st.quant_act4_ref(x)
    put("quant_act4", cases.digest(x), packed=st.pack_int4_lo(q).view(np.uint8).reshape(-1), s=s)
    x = cases.normal_case(72, 1, 5120)
    q, s = st.quant_act_ref(x)
    put("quant_act", cases.digest(x), even=q[0, 0::2].astype(np.int8), odd=q[0, 1::2].astype(np.int8),
        s=s, gsum=q.reshape(1, 40, 128).sum(axis=2).astype(np.int32))
    x = cases.normal_case(90, 1, 5120, gain=3)
    a, b, s = st.nvfp4_quant_ref(x)
    put("nvfp4_quant", cases.digest(x), a=a, b=b, s=s)

    # ---- NVFP4 GEMV (selftest seed 202; plus a 3-token variant) ----
    for case, m in (("nvfp4_gemv", 1), ("nvfp4_gemv_m3", 3)):
        codes, ws, x = cases.nvfp4_case(202, 32, 512, m)
        wq = st.pack_nvfp4_codes(codes)
        a, b, s = st.nvfp4_quant_ref(x)
        gscale = float(np.float32(0.75))
        act = np.empty((m, 512), dtype=np.int32)
        act[:, 0::2], act[:, 1::2] = a, b
        rep = np.repeat(np.arange(512 // 16), 16)
        wvv = st.e2m1_decode(st.unpack_nvfp4_codes(wq, 512))
        y = ((wvv * st.e4m3_decode(ws)[:, rep]) @ (act.astype(np.float32) * s[:, rep]).T * gscale).T
        put(case, cases.digest(codes, ws, x), y=np.ascontiguousarray(y), wq=wq)
    put("fp4_tables", "-", e2m1=st.e2m1_decode(np.arange(16, dtype=np.uint8)),
        e4m3=st.e4m3_decode(np.arange(256, dtype=np.uint8)))

    # ---- W4A16 (selftest seeds 30, 40, 50) ----
    packed, scales = cases.int4_dequant_case()
    codes = np.empty((64, 128), dtype=np.int32)
    pk = packed.reshape(64, 16)
    for w in range(16):
        codes[:, w * 8:(w + 1) * 8] = ((pk[:, w][:, None] >> np.arange(0, 32, 4, dtype=np.uint32)) & 0xF)
    bf = (scales.astype(np.uint32) << 16).view(np.float32)
    put("int4_dequant", cases.digest(packed, scales),
        y=((codes - 8).astype(np.float32) * bf[:, None]).reshape(-1))
    part = cases.reduce_case()
    put("reduce_blocks", cases.digest(part), y=part.reshape(32, 5).sum(axis=1))
    packed, scales, x = cases.int4_dot_case()
    nbpr, rpe, nexp = 8, 6, 2
    ref = gid.ref_dot(packed.reshape(rpe * nexp, nbpr * 16), scales.reshape(rpe * nexp, nbpr), x,
                      rpe * nexp, nbpr, ids=list(range(nexp)), rows_per_exp=rpe, rows_per_w=rpe)
    put("int4_dot", cases.digest(packed, scales, x), partial=ref)

    # ---- host pack / convert (python/k100lc_kernels/quant.py) ----
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((16, 256)) * 0.05).astype(np.float32)
    pk, sc = rq.pack_int4_group128(w)
    q2, s2 = rq.ct_int4_to_rt4(pk, sc)
    put("host_quant", cases.digest(w), packed=np.frombuffer(pk, np.uint8), scales=np.frombuffer(sc, np.uint8),
        dequant=rq.dequant_int4_group128(pk, sc, 16, 256), rt4_q=np.frombuffer(q2, np.uint8),
        rt4_s=np.frombuffer(s2, np.uint8), gf=rq.int4_scale_group_first_f32(sc, 16, 256))

    # ---- W4A4 GEMM example (examples/python_w4a4_gemm.py:59-83) ----
    b, x = cases.gemm_case()
    m, k = x.shape
    xq = np.empty((m, k), dtype=np.float32)
    for r in range(m):
        for g in range(k // 128):
            blk = x[r, g * 128:(g + 1) * 128]
            s = max(np.abs(blk).max() / 7.0, 1e-30)
            xq[r, g * 128:(g + 1) * 128] = np.clip(np.rint(blk / s), -8, 7) * s
    put("gemm_w4a4", cases.digest(b, x), c=xq @ b.astype(np.float32).T)

    # ---- the operators either side of the layer: RMSNorm (+ quantiser) and the SiLU gate ----
    # (tools/gen_rmsnorm_quant.py:288-306 with the shapes of its self-test; tools/selftest_all.py:205-223, 266-279)
    for rows, dim in cases.RMSNORM_QUANT_SHAPES:
        x, w = cases.rmsnorm_case(rows, dim)
        q, s, asum = grq._ref(x, w, 1e-6)
        put(f"rmsnorm_quant_{rows}x{dim}", cases.digest(x, w), q=q.astype(np.int8), s=s, asum=asum)
    x, w = cases.rmsnorm_case(4, 256, seed=8, gain=1.0, plain_w=True)
    put("rmsnorm", cases.digest(x, w), y=(x / np.sqrt((x ** 2).mean(axis=1, keepdims=True) + 1e-5) * w).astype(np.float32))
    gate, up = cases.silu_case()
    put("silu_mul", cases.digest(gate, up), y=(st._silu(gate) * up).astype(np.float32))

    np.savez_compressed(HERE / "reference_vectors.npz", **out)
    (HERE / "reference_vectors.json").write_text(json.dumps(
        {"numpy": np.__version__, "generator": "tests/golden/make_golden.py",
         "reference": "Hong-agent/K100LC-kernels", "cases": meta}, indent=1))
    print(f"wrote {len(out)} arrays for {len(meta)} cases")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
