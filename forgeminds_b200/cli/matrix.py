"""Sweep ``bench`` over quantisation modes and print one comparison table.

    python -m forgeminds_b200.cli matrix --preset small --steps 10
"""
from __future__ import annotations

import sys

from . import bench

MODES = ("none", "fp8", "int8")


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    rows = []
    for mode in MODES:
        try:
            res = bench.main([*argv, "--quant", mode])
            rows.append((mode, res["quant_resolved"], res["tok_s"], res["step_ms_p50"], res.get("peak_mem_gb", "-")))
        except Exception as exc:       # a missing backend is a row of the table, not a crash
            rows.append((mode, f"unavailable: {str(exc)[:50]}", "-", "-", "-"))
    print(f"\n{'quant':8s} {'backend':40s} {'tok/s':>12s} {'p50 ms':>9s} {'mem GB':>8s}")
    for r in rows:
        print(f"{r[0]:8s} {str(r[1]):40s} {str(r[2]):>12s} {str(r[3]):>9s} {str(r[4]):>8s}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
