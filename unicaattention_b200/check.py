"""Can this machine run the B200 kernels?  Same verdicts and call surface as the reference's unica/check.py
(`compatibility(found=None)`, `machine()`, OK / UNTESTED / UNSUPPORTED, a `Compatibility(status, reasons)` tuple),
re-targeted: libunica_b200.so holds sm_100a machine code, which only compute capability 10.0 loads.

The verdict is computed from a plain dict, so tests can describe machines that are not this one.
"""

from __future__ import annotations

import ctypes
import sys
from typing import Callable, NamedTuple

OK, UNTESTED, UNSUPPORTED = "ok", "untested", "unsupported"

# what the kernels need, and what they were measured on
NEEDS = {"capability": (10, 0), "driver": 12080}  # CUDA 12.8 is the first with tcgen05 for sm_100a
MEASURED = {"gpu": "NVIDIA B200", "driver": 13000, "torch": "2.11", "platforms": ("linux",)}

_HEADLINE = {OK: "tested on this machine", UNTESTED: "runs here, but untested", UNSUPPORTED: "cannot run here"}


class Compatibility(NamedTuple):
    status: str
    reasons: tuple[str, ...]

    def __str__(self) -> str:
        return "\n  - ".join([f"unica-b200: {_HEADLINE[self.status]}", *self.reasons])


def _cuda(version: int) -> str:
    return f"{version // 1000}.{version % 1000 // 10}"


def driver_version() -> int | None:
    """CUDA version the installed driver supports (1000 * major + 10 * minor); None when there is no driver."""
    try:
        out = ctypes.c_int()
        return out.value if ctypes.CDLL("libcuda.so.1").cuDriverGetVersion(ctypes.byref(out)) == 0 else None
    except OSError:
        return None


def machine() -> dict:
    """The facts compatibility() judges, read here.  GPU facts are None without CUDA."""
    import torch

    has_gpu = torch.cuda.is_available()
    return {
        "platform": sys.platform,
        "torch": torch.__version__,
        "torch_cuda": torch.version.cuda,
        "gpu": torch.cuda.get_device_name() if has_gpu else None,
        "capability": torch.cuda.get_device_capability() if has_gpu else None,
        "driver": driver_version(),
    }


def _blockers(m: dict) -> list[str]:
    """Reasons the library cannot run at all."""
    rules: list[tuple[Callable[[], bool], Callable[[], str]]] = [
        (lambda: m["driver"] is None, lambda: "no NVIDIA driver"),
        (lambda: m["driver"] is not None and m["driver"] < NEEDS["driver"],
         lambda: f"the driver supports CUDA {_cuda(m['driver'])}, the kernels need {_cuda(NEEDS['driver'])} or newer"),
        (lambda: m["torch_cuda"] is None, lambda: f"torch {m['torch']} is built without CUDA"),
        (lambda: m["torch_cuda"] is not None and m["capability"] is None, lambda: "torch sees no GPU"),
        (lambda: m["torch_cuda"] is not None and m["capability"] is not None and tuple(m["capability"]) != NEEDS["capability"],
         lambda: f"{m['gpu']} has compute capability {'.'.join(str(x) for x in m['capability'])}; the kernels are "
                 f"sm_100a code, which runs on {'.'.join(str(x) for x in NEEDS['capability'])} only (B200)"),
    ]
    return [say() for applies, say in rules if applies()]


def _caveats(m: dict) -> list[str]:
    """Reasons it runs but was not measured in this combination."""
    notes = []
    if m["driver"] is not None and NEEDS["driver"] <= m["driver"] < MEASURED["driver"]:
        notes.append(f"driver for CUDA {_cuda(m['driver'])}, older than the measured {_cuda(MEASURED['driver'])}")
    if m["capability"] is not None and tuple(m["capability"]) == NEEDS["capability"] and m["gpu"] != MEASURED["gpu"]:
        notes.append(f"{m['gpu']}: same compute capability, measured only on the {MEASURED['gpu']}")
    if not str(m["torch"]).startswith(MEASURED["torch"] + "."):
        notes.append(f"torch {m['torch']}, measured with {MEASURED['torch']}")
    if m["platform"] not in MEASURED["platforms"]:
        notes.append(f"platform {m['platform']}, measured on {', '.join(MEASURED['platforms'])}")
    return notes


def compatibility(found: dict | None = None) -> Compatibility:
    """OK, UNTESTED or UNSUPPORTED.  When it cannot run, only the blocking reasons are listed."""
    m = machine() if found is None else found
    blockers = _blockers(m)
    if blockers:
        return Compatibility(UNSUPPORTED, tuple(blockers))
    caveats = _caveats(m)
    return Compatibility(UNTESTED if caveats else OK, tuple(caveats))
