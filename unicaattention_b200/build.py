"""Builds libunica_b200.so (the C-ABI library, include/unica_b200.h) from csrc/*.cu with nvcc for sm_100a, in-tree.

    python -m unicaattention_b200.build [--force]

nvcc cross-compiles without a GPU.  The library links the CUDA runtime statically, so it needs nothing but the
driver at run time.
"""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libunica_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-cudart", "static"]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = [*sources(), *CSRC.glob("*.cuh"), *CSRC.glob("*.h"), HERE.parent / "include" / "unica_b200.h"]
    return any(p.stat().st_mtime > built for p in deps)


def build(force: bool = False, verbose: bool = False, defines: tuple[str, ...] = (), output: Path | None = None) -> Path:
    """Compile every .cu of csrc/ into objects (in build/) and link the shared library.  Returns its path.
    defines: extra -D flags (e.g. ("UNICA_TRACE",)) for a diagnostic build written to `output` instead of LIB."""
    if defines or output:
        return _build(HERE / "build" / ("-".join(defines) or "alt"), output or HERE / ("libunica_b200-" + "-".join(defines) + ".so"),
                      [f"-D{d}" for d in defines], verbose)
    if not force and not stale():
        return LIB
    return _build(HERE / "build", LIB, [], verbose)


def _build(objdir: Path, lib: Path, extra: list[str], verbose: bool) -> Path:
    objdir.mkdir(parents=True, exist_ok=True)
    objects = []
    procs = []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        cmd = ["nvcc", *ARCH_FLAGS, *NVCC_FLAGS, *extra, *(["-Xptxas", "-v"] if verbose else []), "-c", str(src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode:
            print(out)
        if proc.returncode:
            raise RuntimeError(f"nvcc failed on {src.name}")
    subprocess.run(["nvcc", *ARCH_FLAGS, "-shared", "-cudart", "static", "-o", str(lib), *objects], check=True)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
