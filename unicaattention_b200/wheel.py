"""Builds a wheel that ships the compiled library, for machines without nvcc (the reference's build_wheel.py:1-40 does
the same with its cubins).

    python -m unicaattention_b200.wheel [--out dist] [--no-build]

libunica_b200.so is compiled fresh from csrc/ (nvcc; no GPU needed), its sha256 is printed so that another machine can
check it loads the very same bytes, and the wheel holds the Python modules, the library and the C header, but no csrc/:
lib.library() then finds the file beside it and never looks for a compiler (the reference's shipped-binary lookup,
unica/cuda.py:55-61).  The library links the CUDA runtime statically and needs only the driver; it is sm_100a machine
code, so the wheel is tagged for Linux x86-64 and is of use on B200 only.
"""

from __future__ import annotations

import argparse
import base64
import hashlib
import zipfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
NAME, VERSION, TAG = "unicaattention_b200", "0.2.0", "py3-none-linux_x86_64"
SHIPPED_SUFFIXES = {".py"}


def files() -> list[tuple[Path, str]]:
    """(file, name inside the wheel) of everything that ships."""
    shipped = [(p, str(p.relative_to(ROOT))) for p in sorted(HERE.rglob("*")) if p.is_file() and p.suffix in SHIPPED_SUFFIXES
               and "csrc" not in p.relative_to(HERE).parts and "build" not in p.relative_to(HERE).parts]
    shipped.append((HERE / "libunica_b200.so", f"{NAME}/libunica_b200.so"))
    shipped.append((ROOT / "include" / "unica_b200.h", f"{NAME}/include/unica_b200.h"))
    return shipped


def record_line(name: str, data: bytes) -> str:
    digest = base64.urlsafe_b64encode(hashlib.sha256(data).digest()).rstrip(b"=").decode()
    return f"{name},sha256={digest},{len(data)}"


def build_wheel(out: Path, compile_library: bool = True) -> Path:
    if compile_library:
        from unicaattention_b200.build import build

        build(force=True)
    library = HERE / "libunica_b200.so"
    if not library.exists():
        raise SystemExit(f"{library} is missing: run without --no-build (needs nvcc)")
    print(f"{library.name}  sha256 {hashlib.sha256(library.read_bytes()).hexdigest()}")
    out.mkdir(parents=True, exist_ok=True)
    wheel = out / f"{NAME}-{VERSION}-{TAG}.whl"
    info = f"{NAME}-{VERSION}.dist-info"
    meta = {
        f"{info}/METADATA": f"Metadata-Version: 2.1\nName: {NAME}\nVersion: {VERSION}\nSummary: Quantized attention (INT8 / NVFP4) for B200\n"
                            "Requires-Python: >=3.10\nRequires-Dist: torch\n",
        f"{info}/WHEEL": f"Wheel-Version: 1.0\nGenerator: {NAME}.wheel\nRoot-Is-Purelib: false\nTag: {TAG}\n",
        f"{info}/top_level.txt": f"{NAME}\n",
    }
    record = []
    with zipfile.ZipFile(wheel, "w", zipfile.ZIP_DEFLATED) as z:
        for path, name in files():
            data = path.read_bytes()
            z.writestr(name, data)
            record.append(record_line(name, data))
        for name, text in meta.items():
            z.writestr(name, text)
            record.append(record_line(name, text.encode()))
        record.append(f"{info}/RECORD,,")
        z.writestr(f"{info}/RECORD", "\n".join(record) + "\n")
    names = zipfile.ZipFile(wheel).namelist()
    if any("/csrc/" in n for n in names) or f"{NAME}/libunica_b200.so" not in names:
        raise SystemExit(f"{wheel.name} is not what it should be: {names}")
    print(f"{wheel}: {len(names)} files")
    return wheel


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", type=Path, default=ROOT / "dist")
    ap.add_argument("--no-build", action="store_true", help="ship the library as it lies in the tree instead of compiling it afresh")
    args = ap.parse_args()
    build_wheel(args.out, not args.no_build)


if __name__ == "__main__":
    main()
