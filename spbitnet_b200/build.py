"""Builds libspbitnet_b200.so in-tree with nvcc for sm_100a (no torch extension machinery).

`python -m spbitnet_b200.build` or `spbitnet_b200.build.build()`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libspbitnet_b200.so"
CLI = HERE / "spbitnet_infer"
SOURCES = ["core.cu", "gemv.cu", "gemv_batch_mma.cu", "gemv_mmasp.cu", "gemv_prepared.cu", "gemm.cu", "gemm_tcsp_ws.cu", "gemm_mmasp.cu", "unpack.cu",
           "decode_ops.cu", "attention.cu", "fused_ops.cu", "prefill.cu", "decode_persistent.cu", "engine.cu", "sharded.cu", "noalloc.cu", "pack.cu", "format_host.cpp",
           "tokenizer.cpp", "model_loader.cpp"]
COMPILE_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
                 "-Xcompiler", "-fPIC"]
LINK_FLAGS = ["-shared", "-gencode", "arch=compute_100a,code=sm_100a"]
OBJ = CSRC / "build"


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the sm_100a library cannot be built")


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [p for p in CSRC.glob("*") if p.is_file()] + [HERE.parent / "include" / "spbitnet_b200.h"]
    return any(p.stat().st_mtime > t for p in deps)


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> str:
    cmd = [nvcc, *COMPILE_FLAGS, "-c", "-o", str(obj), str(src)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    return res.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """One object file per source, compiled in parallel and only when the source or a header is newer than
    the object; then one link.  Objects live in csrc/build/ (not tracked)."""
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    headers = [p for p in CSRC.glob("*.cuh")] + [HERE.parent / "include" / "spbitnet_b200.h"]
    newest_header = max(p.stat().st_mtime for p in headers)
    jobs = []
    for src in sources():
        obj = OBJ / (src.name + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_header):
            jobs.append((src, obj))
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        logs = list(pool.map(lambda j: _compile_one(nvcc, j[0], j[1], verbose), jobs))
    if verbose:
        print("\n".join(logs))
    objs = [str(OBJ / (s.name + ".o")) for s in sources()]
    res = subprocess.run([nvcc, *LINK_FLAGS, "-o", str(LIB), *objs], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    # the command line (the reference's spbitnet_infer, src/main.cpp) on top of the library
    cli_src = CSRC / "cli_main.cpp"
    if force or not CLI.exists() or CLI.stat().st_mtime < max(cli_src.stat().st_mtime, LIB.stat().st_mtime):
        res = subprocess.run([nvcc, "-O2", "-std=c++17", "-o", str(CLI), str(cli_src), "-L", str(HERE), "-lspbitnet_b200",
                              "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"building spbitnet_infer failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
