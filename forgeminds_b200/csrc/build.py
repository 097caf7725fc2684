"""In-tree build of the native library for sm_100a.

``python -m forgeminds_b200.csrc.build`` compiles every ``.cu`` file in this directory with nvcc
(``-gencode arch=compute_100a,code=sm_100a``; cross-compiles without a GPU), the pybind11 binding
with g++, and links ``forgeminds_b200/_C.so``. Objects are cached by source hash under
``build/`` next to the sources, so a second call only rebuilds what changed.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
PKG = HERE.parent
OBJ = HERE / "build"
TARGET = PKG / "_C.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--use_fast_math",
              "-DFMB_BUILD"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wno-attributes", "-DFMB_WITH_ATTENTION"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _cuda_home() -> Path:
    return Path(_nvcc()).resolve().parent.parent


def _digest(paths, extra="") -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(Path(p).read_bytes())
    return h.hexdigest()[:16]


def _run(cmd, log_path=None):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path is not None:
        Path(log_path).write_text(" ".join(map(str, cmd)) + "\n" + proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError(f"command failed ({proc.returncode}): {' '.join(map(str, cmd))}\n{proc.stdout[-6000:]}")
    return proc.stdout


DEBUG_TARGET = PKG / "_C_debug.so"
DEBUG_SOURCES = ("comm", "moe_ep", "gemm_sm100")       # the translation units with peer-memory accesses


def build(verbose: bool = False, force: bool = False, debug_bounds: bool = False) -> Path:
    """``debug_bounds=True`` builds ``_C_debug.so`` instead: the same library with ``-DFMB_DEBUG_BOUNDS`` in the
    translation units that touch peer memory (every such access is checked against the registered buffers and
    skipped, with an error code in the status word, when it lies outside). ``FORGEMINDS_DEBUG_SO=1`` makes the
    package load that library."""
    import torch
    from torch.utils import cpp_extension as ce

    OBJ.mkdir(exist_ok=True)
    target = DEBUG_TARGET if debug_bounds else TARGET
    module = "_C_debug" if debug_bounds else "_C"
    headers = sorted(HERE.glob("*.cuh")) + sorted(HERE.glob("*.h"))
    hdr_sig = _digest(headers, " ".join(NVCC_FLAGS) + torch.__version__)
    cuda_inc = str(_cuda_home() / "include")
    jobs = []
    objects = []
    for src in sorted(HERE.glob("*.cu")):
        checked = debug_bounds and src.stem in DEBUG_SOURCES
        stem = src.stem + (".dbg" if checked else "")
        sig = _digest([src], hdr_sig)
        obj = OBJ / f"{stem}.{sig}.o"
        objects.append(obj)
        if obj.exists() and not force:
            continue
        for stale in OBJ.glob(f"{stem}.*.o"):
            if checked or ".dbg." not in stale.name:
                stale.unlink()
        extra = ["-DFMB_DEBUG_BOUNDS"] if checked else []
        jobs.append(([_nvcc(), *NVCC_FLAGS, *extra, "-I", str(HERE), "-c", str(src), "-o", str(obj)],
                     OBJ / f"{stem}.log"))
    torch_inc = [f"-I{p}" for p in ce.include_paths()]
    py_inc = f"-I{sysconfig.get_paths()['include']}"
    for src in sorted(HERE.glob("*.cpp")):
        named = src.stem == "bindings" and debug_bounds          # the module's init symbol carries its name
        stem = src.stem + (".dbg" if named else "")
        sig = _digest([src], hdr_sig)
        obj = OBJ / f"{stem}.{sig}.o"
        objects.append(obj)
        if obj.exists() and not force:
            continue
        for stale in OBJ.glob(f"{stem}.*.o"):
            if named or ".dbg." not in stale.name:
                stale.unlink()
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        jobs.append((["g++", *CXX_FLAGS, f"-D_GLIBCXX_USE_CXX11_ABI={abi}", f"-DTORCH_EXTENSION_NAME={module}",
                      "-DTORCH_API_INCLUDE_EXTENSION_H", f"-I{HERE}", f"-I{cuda_inc}", py_inc, *torch_inc,
                      "-c", str(src), "-o", str(obj)], OBJ / f"{stem}.log"))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for out in pool.map(lambda j: _run(*j), jobs):
                if verbose:
                    print(out)
    stamp = OBJ / ("link.dbg.sig" if debug_bounds else "link.sig")
    link_sig = _digest(objects)
    if force or jobs or not target.exists() or not stamp.exists() or stamp.read_text() != link_sig:
        lib_dirs = ce.library_paths()
        cuda_lib = str(_cuda_home() / "lib64")
        cmd = ["g++", "-shared", "-o", str(target), *map(str, objects)]
        for d in [*lib_dirs, cuda_lib]:
            cmd += [f"-L{d}", f"-Wl,-rpath,{d}"]
        cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
        _run(cmd, OBJ / ("link.dbg.log" if debug_bounds else "link.log"))
        stamp.write_text(link_sig)
    return target


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, as printed by ``-Xptxas -v`` at build time."""
    out = []
    for log in sorted(OBJ.glob("*.log")):
        out.append(f"== {log.name}\n{log.read_text()}")
    return "\n".join(out)


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv, debug_bounds="--debug-bounds" in sys.argv)
    print(path)
