"""python -m unicaattention_b200: whether this machine can run the library, then every preset against exact attention on
random inputs with its time (the reference's `python -m unica`, unica/__main__.py).  Exit code 1 if it cannot run or a
preset is off."""

import statistics
import sys

import torch

import unicaattention_b200 as unica

SHAPE = (1, 16, 4096, 128)
# rel-L2 against FP32 a working kernel stays under on N(0, 1) inputs (the reference's limits, unica/__main__.py:13-16):
# a broken kernel lands near 100 % or NaN
ERROR_LIMITS = {"per_token": 0.03, "per_channel": 0.03, "outliers": 0.03, "fast": 0.25}


def time_ms(function, runs: int = 10) -> float:
    function()
    times = []
    for _ in range(runs):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        function()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    return statistics.median(times)


def main() -> int:
    status = unica.compatibility()
    print(status)
    if status.status == unica.UNSUPPORTED:
        return 1
    torch.manual_seed(0)
    q, k, v = (torch.randn(SHAPE, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    exact = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
    sdpa = time_ms(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v))
    print(f"{list(SHAPE)} bf16, PyTorch SDPA {sdpa:.2f} ms")
    failed = 0
    for name, preset in unica.PRESETS.items():
        try:
            error = ((unica.attention(q, k, v, **preset).float() - exact).norm() / exact.norm()).item()
            unica.check_status()
            ms = time_ms(lambda preset=preset: unica.attention(q, k, v, **preset))
        except NotImplementedError as missing:
            print(f"  {name:12} not built: {missing}")
            continue
        good = error < ERROR_LIMITS[name]  # also False for NaN
        failed += not good
        print(f"  {name:12} rel L2 {100 * error:5.2f} % (limit {100 * ERROR_LIMITS[name]:.0f} %)  {ms:6.2f} ms  {'ok' if good else 'FAILED'}")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
