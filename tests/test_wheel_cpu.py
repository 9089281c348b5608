"""The wheel recipe: what it ships loads on a machine that has neither the sources nor a compiler (the reference's
build_wheel.py and its shipped-binary lookup, unica/cuda.py:55-61)."""

import os
import subprocess
import sys
import zipfile
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_the_wheel_loads_without_sources(tmp_path):
    from unicaattention_b200 import wheel

    if not (ROOT / "unicaattention_b200" / "libunica_b200.so").exists():
        pytest.skip("the library has not been built in this tree")
    built = wheel.build_wheel(tmp_path / "dist", compile_library=False)
    names = zipfile.ZipFile(built).namelist()
    assert "unicaattention_b200/libunica_b200.so" in names and "unicaattention_b200/include/unica_b200.h" in names
    assert "unicaattention_b200/comfyui/__init__.py" in names and not any("csrc" in n or n.endswith(".cu") for n in names)
    site = tmp_path / "site"
    zipfile.ZipFile(built).extractall(site)
    assert not (site / "unicaattention_b200" / "csrc").exists()
    # a fresh interpreter that can see only the unpacked wheel, with nvcc out of reach: importing and loading must not build
    code = ("import unicaattention_b200 as u, pathlib; from unicaattention_b200 import lib; l = lib.library(); "
            "assert pathlib.Path(u.__file__).parent.parent == pathlib.Path(r'%s'), u.__file__; "
            "assert l.unica_b200_version() >= 1; print(sorted(lib.SIGNATURES)[0])" % site)
    env = {**os.environ, "PYTHONPATH": str(site), "PATH": "/nonexistent"}
    env.pop("UNICA_B200_LIB", None)
    run = subprocess.run([sys.executable, "-c", code], cwd=tmp_path, env=env, capture_output=True, text=True)
    assert run.returncode == 0, run.stderr[-2000:]


def test_a_tree_without_library_or_sources_fails_loudly(tmp_path):
    """No CPU fallback: a package that has neither the library nor csrc/ to build it from raises on first use."""
    site = tmp_path / "site" / "unicaattention_b200"
    site.mkdir(parents=True)
    for path in (ROOT / "unicaattention_b200").glob("*.py"):
        (site / path.name).write_bytes(path.read_bytes())
    code = "from unicaattention_b200 import lib\ntry:\n    lib.library()\nexcept RuntimeError as e:\n    print('refused:', e)\nelse:\n    raise SystemExit('loaded?')"
    env = {**os.environ, "PYTHONPATH": str(tmp_path / "site")}
    env.pop("UNICA_B200_LIB", None)
    run = subprocess.run([sys.executable, "-c", code], cwd=tmp_path, env=env, capture_output=True, text=True)
    assert run.returncode == 0 and "refused:" in run.stdout, run.stdout + run.stderr[-2000:]
