"""In-tree native build: every ``csrc/**/*.cu`` is compiled for sm_100a with nvcc and linked
into ``_C/libhmf_b200_kernels.so``; ``csrc/runtime/*.cpp`` (host-only scheduler, block
manager, data packing) is compiled with g++ into ``_C/libhmf_b200_runtime.so``.

The libraries expose plain ``extern "C"`` entry points that the Python side binds with
``ctypes`` (see ``ops/_lib.py``), so no PyTorch header is needed at build time and a full
rebuild takes well under a minute on 8 cores.

Run ``python -m hybrid_model_factory_b200.build`` (or ``__graft_entry__.build()``).
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_C"
OBJ = OUT / "obj"

KERNEL_LIB = OUT / "libhmf_b200_kernels.so"
RUNTIME_LIB = OUT / "libhmf_b200_runtime.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "--expt-relaxed-constexpr", "--use_fast_math",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _digest(paths: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(str(p.relative_to(PKG)).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _headers() -> list[Path]:
    return sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.hpp")))


def _compile_one(src: Path, obj: Path, cmd: list[str], stamp: str, verbose: bool) -> tuple[Path, str]:
    stamp_file = obj.with_suffix(obj.suffix + ".stamp")
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        log = obj.with_suffix(".log")
        return obj, log.read_text() if log.exists() else ""
    proc = subprocess.run(cmd, capture_output=True, text=True)
    out = proc.stdout + proc.stderr
    if proc.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{out}")
    obj.with_suffix(".log").write_text(out)
    stamp_file.write_text(stamp)
    if verbose:
        print(f"[build] {src.relative_to(PKG)}")
    return obj, out


def build(verbose: bool = True, force: bool = False, jobs: int | None = None) -> dict[str, Path]:
    """Compile and link both native libraries; returns their paths."""
    OBJ.mkdir(parents=True, exist_ok=True)
    if force:
        for f in OBJ.glob("*"):
            f.unlink()
    nvcc = _nvcc()
    headers = _headers()
    hdr_digest = _digest(headers, "hdr")
    cu_srcs = sorted(CSRC.rglob("*.cu"))
    cpp_srcs = sorted((CSRC / "runtime").glob("*.cpp"))
    jobs = jobs or max(1, (os.cpu_count() or 2))
    tasks = []
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        for src in cu_srcs:
            obj = OBJ / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            stamp = _digest([src], hdr_digest + " ".join(NVCC_FLAGS))
            tasks.append(("cu", ex.submit(_compile_one, src, obj, cmd, stamp, verbose)))
        for src in cpp_srcs:
            obj = OBJ / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
            cmd = ["g++", *CXX_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            stamp = _digest([src], hdr_digest + " ".join(CXX_FLAGS))
            tasks.append(("cpp", ex.submit(_compile_one, src, obj, cmd, stamp, verbose)))
        results = [(kind, *t.result()) for kind, t in tasks]
    cu_objs = [str(o) for kind, o, _ in results if kind == "cu"]
    cpp_objs = [str(o) for kind, o, _ in results if kind == "cpp"]
    ptxas_log = "\n".join(out for kind, _, out in results if kind == "cu")
    (OUT / "ptxas.log").write_text(ptxas_log)
    if cu_objs:
        newest = max(Path(o).stat().st_mtime for o in cu_objs)
        if force or not KERNEL_LIB.exists() or KERNEL_LIB.stat().st_mtime < newest:
            cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
                   "-o", str(KERNEL_LIB), *cu_objs, "-cudart", "static"]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError(f"link failed: {' '.join(cmd)}\n{proc.stdout}{proc.stderr}")
            if verbose:
                print(f"[build] linked {KERNEL_LIB.relative_to(PKG)}")
    if cpp_objs:
        newest = max(Path(o).stat().st_mtime for o in cpp_objs)
        if force or not RUNTIME_LIB.exists() or RUNTIME_LIB.stat().st_mtime < newest:
            cmd = ["g++", "-shared", "-pthread", "-o", str(RUNTIME_LIB), *cpp_objs]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError(f"link failed: {' '.join(cmd)}\n{proc.stdout}{proc.stderr}")
            if verbose:
                print(f"[build] linked {RUNTIME_LIB.relative_to(PKG)}")
    return {"kernels": KERNEL_LIB, "runtime": RUNTIME_LIB}


def ptxas_summary() -> str:
    """Registers / spills / shared memory per kernel as reported by ``-Xptxas -v``."""
    log = OUT / "ptxas.log"
    return log.read_text() if log.exists() else ""


if __name__ == "__main__":
    build(verbose=True, force="--force" in sys.argv)
