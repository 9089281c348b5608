"""python -m unicaattention_b200 [--shape B H N] [--json]: the library's self-test on this machine.

First the verdict of check.compatibility(); then, for every preset, one table row: the error against exact FP32
attention on seeded N(0, 1) inputs (with the limit a working kernel stays under), the time of a whole call split into
its quantization passes and its attention kernel, the effective TOPS and what fraction that is of the tensor-core
ceiling of the kernel's own tcgen05.mma mix as the peak micro-benchmark measures it on this GPU right now.  The
kernels' status word is read after every preset, so a pipeline time-out fails the run too.  Exit code 1 when the
machine cannot run the library or a preset is off (the role of the reference's `python -m unica`, unica/__main__.py).
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import sys

import torch

import unicaattention_b200 as unica
from unicaattention_b200 import peak, timing

# rel-L2 against FP32 on N(0, 1) inputs: the emulation's own error is 1.4 to 1.8 % (accurate) and about 19 % (fast, whose
# 4-bit P is at its worst on such inputs); a wrong tile, scale or lane lands near 100 % or at NaN
ERROR_LIMITS = {"per_token": 0.03, "per_channel": 0.03, "outliers": 0.03, "fast": 0.25}


@dataclasses.dataclass
class Row:
    preset: str
    rel_l2: float
    limit: float
    call_ms: float
    quantize_ms: float
    kernel_ms: float
    tops: float
    of_ceiling: float
    status: str

    @property
    def ok(self) -> bool:
        return self.status == "ok" and self.rel_l2 < self.limit  # False for NaN too


def exact_attention(q, k, v):
    """FP32 softmax(q k^T / sqrt(d)) v, a block of query rows at a time so that long shapes fit."""
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    kf, vf = k.float().transpose(-1, -2), v.float()
    for first in range(0, q.shape[2], 4096):
        rows = slice(first, first + 4096)
        out[:, :, rows] = torch.softmax(q[:, :, rows].float() @ kf * q.shape[-1] ** -0.5, -1) @ vf
    return out


def measure(name: str, q, k, v, exact, ceilings: dict[str, float]) -> Row:
    preset = unica.PRESETS[name]
    out = unica.attention(q, k, v, **preset).float()
    error = ((out - exact).norm() / exact.norm()).item()
    try:
        unica.check_status()
        status = "ok"
    except RuntimeError as gave_up:
        status = str(gave_up)
    inputs = unica.kernel_inputs(q, k, v, **preset)
    call = timing.median_ms(lambda: unica.attention(q, k, v, **preset))
    quantize = timing.median_ms(lambda: unica.kernel_inputs(q, k, v, **preset))
    kernel = timing.median_ms(lambda: unica.attention(q, k, v, inputs=inputs, **preset))
    batch, heads, n, d = q.shape
    tops = 4.0 * batch * heads * n * k.shape[2] * d / call / 1e9
    return Row(name, error, ERROR_LIMITS[name], call, quantize, kernel, tops, tops / ceilings["fast" if name == "fast" else "accurate"], status)


def main() -> int:
    ap = argparse.ArgumentParser(description="self-test of unicaattention_b200 on this machine")
    ap.add_argument("--shape", type=int, nargs=3, default=(1, 16, 4096), metavar=("BATCH", "HEADS", "TOKENS"))
    ap.add_argument("--presets", nargs="+", default=list(unica.PRESETS), choices=list(unica.PRESETS))
    ap.add_argument("--json", action="store_true", help="one JSON object instead of the table")
    args = ap.parse_args()
    verdict = unica.compatibility()
    if not args.json:
        print(verdict)
    if verdict.status == unica.UNSUPPORTED:
        return 1
    generator = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn((*args.shape, unica.HEAD_DIM), generator=generator).bfloat16().cuda() for _ in range(3))
    exact = exact_attention(q, k, v)
    mhz = torch.cuda.get_device_properties(0).clock_rate / 1e3 if hasattr(torch.cuda.get_device_properties(0), "clock_rate") else 1965.0
    ceilings = {mode: peak.attention_mix_tops(mode, mhz) for mode in ("accurate", "fast")}
    rows = [measure(name, q, k, v, exact, ceilings) for name in args.presets]
    if args.json:
        print(json.dumps({"compatibility": verdict.status, "shape": [*args.shape, unica.HEAD_DIM], "tensor_mix_ceiling_tops": ceilings,
                          "presets": [dataclasses.asdict(r) | {"ok": r.ok} for r in rows]}))
    else:
        print(f"{[*args.shape, unica.HEAD_DIM]} bf16 N(0,1); tensor ceiling of the tcgen05.mma mix at {mhz:.0f} MHz: "
              f"accurate {ceilings['accurate']:.0f}, fast {ceilings['fast']:.0f} TOPS")
        print(f"  {'preset':12} {'rel L2':>8} {'limit':>6} {'call':>9} {'quantize':>9} {'kernel':>9} {'eff. TOPS':>10} {'of ceiling':>10}")
        for r in rows:
            print(f"  {r.preset:12} {r.rel_l2:8.2%} {r.limit:6.0%} {r.call_ms:7.3f}ms {r.quantize_ms:7.3f}ms {r.kernel_ms:7.3f}ms "
                  f"{r.tops:10.0f} {r.of_ceiling:10.1%}  {'ok' if r.ok else 'FAILED: ' + (r.status if r.status != 'ok' else 'error above the limit')}")
    return 0 if all(r.ok for r in rows) else 1


if __name__ == "__main__":
    sys.exit(main())
