"""Builds ``librlt_verify.so`` — the CUDA kernels and their C ABI — in-tree with nvcc.

    python -m vllm_rlt_b200.build            # build if sources are newer than the library
    python -m vllm_rlt_b200.build --force

The library targets sm_100a only and links the CUDA runtime statically, so it has no
dependency on PyTorch and can be bound from any host language through `include/rlt_verify.h`.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
INCLUDE = PACKAGE.parent / "include"
LIBRARY = PACKAGE / "librlt_verify.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--shared", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "-cudart", "static",
]


def nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found: the sm_100a kernels cannot be built")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    deps = list(CSRC.glob("*")) + list(INCLUDE.glob("*.h"))
    return any(p.stat().st_mtime > built for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIBRARY
    objects = []
    build_dir = PACKAGE / "build"
    build_dir.mkdir(exist_ok=True)
    compile_flags = [f for f in NVCC_FLAGS if f not in ("--shared",)]
    procs = []
    for src in sources():
        obj = build_dir / (src.stem + ".o")
        cmd = [nvcc(), *compile_flags, "-Xptxas", "-v", "-c", str(src), "-o", str(obj)]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(obj)
    log = []
    failed = False
    for src, obj, proc in procs:
        out, _ = proc.communicate()
        log.append(f"== {src.name}\n{out}")
        failed |= proc.returncode != 0
    (build_dir / "ptxas.log").write_text("\n".join(log))
    if verbose or failed:
        print("\n".join(log))
    if failed:
        raise RuntimeError("nvcc failed; see output above")
    link = [nvcc(), *NVCC_FLAGS, *map(str, objects), "-o", str(LIBRARY)]
    subprocess.run(link, check=True)
    return LIBRARY


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
