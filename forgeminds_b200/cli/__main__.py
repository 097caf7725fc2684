"""``python -m forgeminds_b200.cli {bench,kbench,gemmbench,matrix,audit,commbench,fusedprof,compilecheck,probe} [options]``"""
from __future__ import annotations

import sys

TOOLS = ("bench", "kbench", "gemmbench", "matrix", "audit", "commbench", "fusedprof", "compilecheck", "probe")


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help") or argv[0] not in TOOLS:
        print("usage: python -m forgeminds_b200.cli {bench|kbench|gemmbench|matrix|audit|commbench|fusedprof|compilecheck|probe} [options]\n"
              "  bench   training throughput of a GPT preset under any mesh / quant / offload setting\n"
              "  kbench  per-kernel timings against eager PyTorch\n"
              "  gemmbench  the linear-layer products of a GPT block against cuBLAS\n"
              "  matrix  sweep of bench over quantisation modes\n"
              "  audit   host reads, kernel launches and top kernels of one training step\n"
              "  commbench  peer-memory kernels against their NCCL formulations (run under torchrun)\n"
              "  fusedprof  single-rank forms of the fused compute + collective kernels, sized for a profiler capture\n"
              "  compilecheck  cross-compile every kernel for sm_100a (no GPU needed): registers, spills, shared memory\n"
              "  probe   every public kernel at awkward shapes against PyTorch, with the device status word")
        return 0 if argv and argv[0] in ("-h", "--help") else 2
    import importlib
    mod = importlib.import_module(f"forgeminds_b200.cli.{argv[0]}")
    out = mod.main(argv[1:])
    return out if isinstance(out, int) else 0


if __name__ == "__main__":
    raise SystemExit(main())
