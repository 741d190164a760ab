"""``python -m k100lc_kernels list [PATTERN] | info NAME | catalog`` (reference
python/k100lc_kernels/__main__.py:8-25; ``catalog`` regenerates catalog.json)."""
from __future__ import annotations

import json
import sys

from .catalog import CATALOG, info, kernels, make_catalog


def main() -> int:
    args = sys.argv[1:]
    if not args or args[0] == "list":
        for k in kernels(args[1] if len(args) > 1 else ""):
            print(f"{k['lookup']:32s} args={len(k['args']):2d} kernarg={k['kernarg_size']:4d}")
        return 0
    if args[0] == "info" and len(args) > 1:
        print(json.dumps(info(args[1]), indent=2))
        return 0
    if args[0] == "catalog":
        CATALOG.write_text(json.dumps(make_catalog(), indent=1) + "\n", encoding="utf-8")
        print(f"wrote {CATALOG}")
        return 0
    print("usage: python -m k100lc_kernels [list [PATTERN] | info NAME | catalog]")
    return 2


if __name__ == "__main__":
    raise SystemExit(main())
