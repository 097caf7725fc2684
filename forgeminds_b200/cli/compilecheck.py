"""Offline compile check: every device kernel of the library, cross-compiled for sm_100a without a GPU.

``python -m forgeminds_b200.cli compilecheck [--force] [--json] [--max-spill BYTES]`` compiles each
``.cu`` file of ``forgeminds_b200/csrc`` with ``-Xptxas -v`` (a cached object is reused unless
``--force``), reads what the assembler printed for every entry function and fails (exit 1) when

* a translation unit does not compile,
* a kernel spills more than ``--max-spill`` bytes (default 512; kernels that spill less are listed as
  warnings: today those are the 256-thread-per-row RMSNorm variants for very wide rows and a few bytes in
  the widest GEMM and attention instantiations),
* a kernel's static shared memory exceeds the 227 KB a CTA of this part can have.

The reference's ``tools/offline_compile_check.py`` does the same job for its Triton kernels through
``triton.compile``; here the kernels are CUDA, so the compiler itself is the checker and the useful part is
the per-kernel resource table.
"""
from __future__ import annotations

import argparse
import json
import re
import subprocess
import sys

SMEM_LIMIT = 227 * 1024
_ENTRY = re.compile(r"Compiling entry function '([^']+)' for 'sm_100a'")
_SPILL = re.compile(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads")
_USED = re.compile(r"Used (\d+) registers(.*)")
_SMEM = re.compile(r"(\d+) bytes smem")
_BARS = re.compile(r"used (\d+) barriers")


def demangle(names):
    """Readable kernel names through ``c++filt`` when it is installed; the mangled name otherwise."""
    try:
        out = subprocess.run(["c++filt"], input="\n".join(names), capture_output=True, text=True, check=True).stdout
        pretty = out.strip("\n").split("\n")
        if len(pretty) == len(names):
            return [re.sub(r"\(.*", "", p).replace("void ", "") for p in pretty]
    except (OSError, subprocess.CalledProcessError):
        pass
    return list(names)


def parse_ptxas(text: str):
    """``[{name, registers, spill_stores, spill_loads, stack, smem, barriers}]`` from one ``-Xptxas -v`` log."""
    rows, cur = [], None
    for line in text.splitlines():
        m = _ENTRY.search(line)
        if m:
            cur = {"name": m.group(1), "registers": 0, "spill_stores": 0, "spill_loads": 0, "stack": 0, "smem": 0,
                   "barriers": 0}
            rows.append(cur)
            continue
        if cur is None:
            continue
        m = _SPILL.search(line)
        if m:
            cur["stack"], cur["spill_stores"], cur["spill_loads"] = (int(g) for g in m.groups())
            continue
        m = _USED.search(line)
        if m:
            cur["registers"] = int(m.group(1))
            s = _SMEM.search(m.group(2))
            b = _BARS.search(m.group(2))
            cur["smem"] = int(s.group(1)) if s else 0
            cur["barriers"] = int(b.group(1)) if b else 0
    return rows


def warnings(rows, max_spill: int = 512):
    return [f"{r['pretty']}: {r['spill_stores']} B spill stores, {r['spill_loads']} B spill loads"
            for r in rows if 0 < r["spill_stores"] + r["spill_loads"] <= max_spill]


def problems(rows, max_spill: int = 512):
    bad = []
    for r in rows:
        spill = r["spill_stores"] + r["spill_loads"]
        if spill > max_spill:
            bad.append(f"{r['pretty']}: {r['spill_stores']} B spill stores, {r['spill_loads']} B spill loads")
        if r["smem"] > SMEM_LIMIT:
            bad.append(f"{r['pretty']}: {r['smem']} B static shared memory (limit {SMEM_LIMIT})")
        if r["registers"] > 255:
            bad.append(f"{r['pretty']}: {r['registers']} registers")
    return bad


def collect(force: bool = False):
    """Build (or reuse) the objects, then read the assembler's report of every translation unit."""
    from ..csrc import build as B
    B.build(force=force)
    rows = []
    for log in sorted(B.OBJ.glob("*.log")):
        if ".dbg." in log.name or log.name.startswith(("link", "bindings")):
            continue
        found = parse_ptxas(log.read_text())
        for r in found:
            r["unit"] = log.stem
        rows += found
    for r, pretty in zip(rows, demangle([r["name"] for r in rows])):
        r["pretty"] = pretty
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="forgeminds_b200.cli compilecheck", description=__doc__.split("\n\n")[0])
    ap.add_argument("--force", action="store_true", help="recompile every translation unit")
    ap.add_argument("--json", action="store_true", help="print the table as JSON")
    ap.add_argument("--max-spill", type=int, default=512, help="accepted spill bytes per kernel")
    ap.add_argument("--top", type=int, default=0, help="only the N kernels with the most registers")
    a = ap.parse_args(argv)
    try:
        rows = collect(a.force)
    except RuntimeError as e:                      # a translation unit failed: the compiler's message is the report
        print(str(e)[-4000:], file=sys.stderr)
        return 1
    shown = sorted(rows, key=lambda r: -r["registers"])[: a.top] if a.top else rows
    if a.json:
        print(json.dumps(shown, indent=1))
    else:
        print(f"{'unit':<16}{'regs':>5}{'spill B':>9}{'stack':>7}{'smem B':>8}  kernel")
        for r in shown:
            print(f"{r['unit']:<16}{r['registers']:>5}{r['spill_stores'] + r['spill_loads']:>9}{r['stack']:>7}"
                  f"{r['smem']:>8}  {r['pretty'][:110]}")
        print(f"{len(rows)} kernels in {len({r['unit'] for r in rows})} translation units")
    bad = problems(rows, a.max_spill)
    if not a.json:
        for w in warnings(rows, a.max_spill):
            print("warn " + w, file=sys.stderr)
    for b in bad:
        print("FAIL " + b, file=sys.stderr)
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
