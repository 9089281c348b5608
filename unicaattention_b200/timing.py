"""Timing helpers and side-by-side comparisons for the attention path.

    python -m unicaattention_b200.timing [per_channel per_token outliers fast] [--heads 40] [--tokens 32760]
    python -m unicaattention_b200.timing --pieces 40 20 10 5 [--heads 40] [--tokens 34020]

Run-to-run drift of a GPU is as large as many single optimisations, so two variants are only ever compared inside one
process, in alternating rounds (the reference's rule: bench/compare.py:1-7, bench/pieces_cost.py).  `alternate()` does
that for any set of callables; the command line uses it for the presets (whole call, quantization alone, kernel alone
on operands quantized beforehand) and for the cost of splitting a call by heads.
"""

from __future__ import annotations

import argparse
import statistics
from typing import Callable, Mapping

import torch


def event_times(function: Callable[[], object], runs: int = 10, warmup: int = 1) -> list[float]:
    """Milliseconds of each of `runs` calls, CUDA events on the current stream (the one the library launches on)."""
    for _ in range(warmup):
        function()
    times = []
    for _ in range(runs):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        function()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    return times


def median_ms(function: Callable[[], object], runs: int = 10, warmup: int = 1) -> float:
    return statistics.median(event_times(function, runs, warmup))


def alternate(arms: Mapping[str, Callable[[], object]], rounds: int = 4, runs: int = 5) -> dict[str, dict]:
    """Every arm timed `rounds` times (median of `runs` each), the arms taking turns and the order reversed on odd
    rounds so that none always runs on a warmer or cooler GPU.  Returns per arm: ms (median of its rounds), spread
    ((max - min) / median over the rounds) and vs_first (first arm's ms / this arm's)."""
    names = list(arms)
    samples: dict[str, list[float]] = {name: [] for name in names}
    for r in range(rounds):
        for name in names if r % 2 == 0 else reversed(names):
            samples[name].append(median_ms(arms[name], runs))
    first = statistics.median(samples[names[0]])
    return {name: {"ms": (ms := statistics.median(samples[name])), "spread": (max(samples[name]) - min(samples[name])) / ms,
                   "vs_first": first / ms, "rounds": samples[name]} for name in names}


def compare_presets(presets: list[str], heads: int, tokens: int, rounds: int, runs: int) -> dict[str, dict]:
    import unicaattention_b200 as unica

    torch.manual_seed(0)
    q, k, v = (torch.randn((1, heads, tokens, 128), device="cuda", dtype=torch.bfloat16) for _ in range(3))
    arms: dict[str, Callable[[], object]] = {}
    for name in presets:
        preset = unica.PRESETS[name]
        inputs = unica.kernel_inputs(q, k, v, **preset)
        arms[name] = lambda preset=preset: unica.attention(q, k, v, **preset)
        arms[name + " quantize"] = lambda preset=preset: unica.kernel_inputs(q, k, v, **preset)
        arms[name + " kernel"] = lambda preset=preset, inputs=inputs: unica.attention(q, k, v, inputs=inputs, **preset)
    result = alternate(arms, rounds, runs)
    unica.check_status()
    return result


def pieces_cost(pieces: list[int], heads: int, tokens: int, rounds: int, runs: int) -> dict[str, dict]:
    """What splitting a call by heads costs: the planner forced to `pieces` heads per call, fp16 input in ComfyUI's
    [batch, tokens, heads, 128] layout (bench/pieces_cost.py)."""
    import unicaattention_b200 as unica

    torch.manual_seed(0)
    q, k, v = (torch.randn(1, tokens, heads, 128, device="cuda", dtype=torch.float16).transpose(1, 2) for _ in range(3))
    real = unica.heads_per_call
    arms = {}
    for name in unica.PRESETS:
        for n in pieces:
            def run(name=name, n=n):
                unica.heads_per_call = lambda *args: n
                try:
                    return unica.attention(q, k, v, **unica.PRESETS[name])
                finally:
                    unica.heads_per_call = real
            arms[f"{name} {n} heads"] = run
    return alternate(arms, rounds, runs)


def main() -> None:
    import unicaattention_b200 as unica

    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("presets", nargs="*", default=list(unica.PRESETS))
    ap.add_argument("--heads", type=int, default=40)
    ap.add_argument("--tokens", type=int, default=32760)
    ap.add_argument("--rounds", type=int, default=4)
    ap.add_argument("--runs", type=int, default=5)
    ap.add_argument("--pieces", type=int, nargs="+", help="heads per call to force; compares the cost of head-splitting")
    args = ap.parse_args()
    ops = 4.0 * args.heads * args.tokens**2 * 128
    if args.pieces:
        result = pieces_cost(args.pieces, args.heads, args.tokens, args.rounds, args.runs)
    else:
        result = compare_presets(args.presets, args.heads, args.tokens, args.rounds, args.runs)
    print(f"1 x {args.heads} x {args.tokens} x 128, {args.rounds} alternating rounds x median of {args.runs}")
    width = max(map(len, result))
    for name, r in result.items():
        tops = "" if name.endswith("quantize") else f"  {ops / r['ms'] / 1e9:8.0f} eff. TOPS"
        print(f"  {name:{width}}  {r['ms']:8.3f} ms  spread {r['spread']:6.1%}  x{r['vs_first']:5.2f} of the first{tops}")


if __name__ == "__main__":
    main()
