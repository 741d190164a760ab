"""Weight manifest of a compressed-tensors INT4 checkpoint: for every ``<name>.weight_packed`` /
``<name>.weight_scale`` pair, where its bytes sit in which file, so that a loader can stream the layers
into device memory in model order and hand them to ``int4_dot_k`` (or convert them once for the W4A8 /
W4A4 kernels) without parsing safetensors again.  Same role and columns as the reference's
tools/int4_engine_manifest.py:29-60 (absolute file offsets, sizes, N, K), extended by a file column so
that sharded checkpoints work; the first line pins every file's size, because absolute offsets are void
as soon as a file changes.

    python -m k100lc_kernels.int4_manifest --model-dir CKPT -o int4_manifest.tsv

Line format (tab separated):
    # source <file>:<bytes> [<file>:<bytes> ...]
    # name  file  packed_off  packed_bytes  scale_off  scale_bytes  N  K
"""
from __future__ import annotations

import argparse
import pathlib
from dataclasses import dataclass

from .ct_int4 import SafeTensors
from .quant import GROUP


@dataclass(frozen=True)
class ManifestRow:
    name: str
    file: str
    packed_off: int
    packed_bytes: int
    scale_off: int
    scale_bytes: int
    n: int
    k: int

    def line(self) -> str:
        return "\t".join(str(v) for v in (self.name, self.file, self.packed_off, self.packed_bytes, self.scale_off,
                                          self.scale_bytes, self.n, self.k))


def build_rows(model_dir) -> tuple[list[ManifestRow], dict[str, int]]:
    """All INT4 linear layers under ``model_dir`` (every ``*.safetensors`` file), sorted by name, and the
    size of every file that holds one."""
    model_dir = pathlib.Path(model_dir)
    rows, sizes = [], {}
    for path in sorted(model_dir.glob("*.safetensors")):
        st = SafeTensors(path)
        data0 = 8 + st.header_len
        for name in sorted(st.header):
            if not name.endswith(".weight_packed"):
                continue
            base = name[: -len(".weight_packed")]
            if base + ".weight_scale" not in st:
                raise KeyError(f"{base}: weight_scale is not in {path.name} (a layer must not straddle files)")
            p, s = st.entry(name), st.entry(base + ".weight_scale")
            n, k8 = (int(v) for v in p["shape"])
            k = k8 * 8
            if list(s["shape"]) != [n, k // GROUP] or k % GROUP:
                raise ValueError(f"{base}: scale shape {s['shape']} does not fit N={n}, K={k}")
            if p["data_offsets"][1] - p["data_offsets"][0] != n * k // 2 or s["data_offsets"][1] - s["data_offsets"][0] != n * (k // GROUP) * 2:
                raise ValueError(f"{base}: byte counts do not match the shapes")
            rows.append(ManifestRow(base, path.name, data0 + p["data_offsets"][0], n * k // 2, data0 + s["data_offsets"][0],
                                    n * (k // GROUP) * 2, n, k))
            sizes[path.name] = path.stat().st_size
    rows.sort(key=lambda r: r.name)
    return rows, sizes


def write_manifest(model_dir, out) -> list[ManifestRow]:
    rows, sizes = build_rows(model_dir)
    with open(out, "w", encoding="utf-8") as f:
        f.write("# source " + " ".join(f"{n}:{b}" for n, b in sorted(sizes.items())) + "\n")
        f.write("# name\tfile\tpacked_off\tpacked_bytes\tscale_off\tscale_bytes\tN\tK\n")
        for r in rows:
            f.write(r.line() + "\n")
    return rows


def read_manifest(path, model_dir=None) -> list[ManifestRow]:
    """Parse a manifest; with ``model_dir`` the recorded file sizes are checked against the files there."""
    rows, sizes = [], {}
    for line in pathlib.Path(path).read_text(encoding="utf-8").splitlines():
        if line.startswith("# source"):
            sizes = {n: int(b) for n, b in (item.rsplit(":", 1) for item in line.split()[2:])}
        elif line and not line.startswith("#"):
            name, file, *nums = line.split("\t")
            rows.append(ManifestRow(name, file, *(int(v) for v in nums)))
    if model_dir is not None:
        for name, size in sizes.items():
            have = (pathlib.Path(model_dir) / name).stat().st_size
            if have != size:
                raise ValueError(f"{name} is {have} bytes, the manifest was made for {size}: regenerate it")
    return rows


def read_layer(row: ManifestRow, model_dir, row0: int = 0, nrows: int | None = None) -> tuple[bytes, bytes]:
    """``(packed_bytes, scale_bf16_bytes)`` of rows ``[row0, row0 + nrows)`` of one manifest entry, read by seek."""
    nrows = row.n - row0 if nrows is None else nrows
    if row0 < 0 or nrows <= 0 or row0 + nrows > row.n:
        raise ValueError(f"{row.name}: rows [{row0},{row0 + nrows}) are outside N={row.n}")
    with open(pathlib.Path(model_dir) / row.file, "rb") as f:
        f.seek(row.packed_off + row0 * (row.k // 2))
        packed = f.read(nrows * (row.k // 2))
        f.seek(row.scale_off + row0 * (row.k // GROUP) * 2)
        scale = f.read(nrows * (row.k // GROUP) * 2)
    return packed, scale


def shape_table(rows) -> list[tuple[int, int, int, int]]:
    """``(N, K, layers, bytes)`` per distinct shape, largest share of bytes first — the per-layer-shape table of
    a checkpoint (the reference lists its 400-layer one in docs/INT4.md:170-181)."""
    agg: dict[tuple[int, int], list[int]] = {}
    for r in rows:
        a = agg.setdefault((r.n, r.k), [0, 0])
        a[0] += 1
        a[1] += r.packed_bytes + r.scale_bytes
    return sorted(((n, k, c, b) for (n, k), (c, b) in agg.items()), key=lambda t: -t[3])


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model-dir", type=pathlib.Path, required=True)
    ap.add_argument("-o", "--out", type=pathlib.Path, default=pathlib.Path("int4_manifest.tsv"))
    args = ap.parse_args()
    rows = write_manifest(args.model_dir, args.out)
    tot = sum(r.packed_bytes + r.scale_bytes for r in rows)
    print(f"{args.out}: {len(rows)} INT4 linear layers, {tot / 1e9:.3f} GB of codes and scales")
    for n, k, c, b in shape_table(rows):
        print(f"  {n:6d} x {k:<6d} {c:4d} layers {b / 1e9:8.3f} GB")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
