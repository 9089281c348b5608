"""Benchmark of the quantized-attention forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--mode per_channel|per_token|outliers|fast] [--workload wan|hires|image|small]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...
    python bench.py --impl reference ...      # the CPU oracle port timed on the host cores, same config and metric

One step = one whole call `unica.attention(q, k, v, **preset)` (statistics + quantization + attention kernel) on the
named workload; with N > 1 the heads are sharded over the ranks and the step ends with the gather of the output heads.
Prints ONE JSON line (rank 0):

  value         effective TOPS = 4 * B * H * Nq * Nk * 128 / time (the reference's formula, bench/harness.py:69), whole
                job, inputs resident in HBM; ms_per_step is the ms/call of the same runs.  Headline: --mode on --workload
                (defaults: per_channel on wan = 1 x 40 x 32760 x 128)
  e2e           the same call fed from pinned host memory with the result copied back to it, every step
  roofline      the attention kernel alone (operands already quantized), CUDA events, against the tensor peak
  modes         the other presets on the same workload, measured in the same run (the reference reports its presets side
                by side: bench/signatures.py:27-100): ms/call, kernel ms, quantization ms, roofline fraction, accuracy
  configs       the other call signatures of the reference's README (image: 30 heads x 4128 tokens with uneven K channels
                and two outlier V tokens; hires: 40 heads x 118320 tokens with Q, K channel spread 2.3), accurate and fast
  cpu_baseline  the CPU oracle port on a bounded sample (1 head x 2048 queries x all keys), all host threads
Inputs are synthetic, seeded, generated per head on the CPU so each rank builds its own shard (the reference's
real-activation dumps are not available); their seeds and achieved statistics are in the line.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

WORKLOADS = {  # (batch, heads, tokens)
    "wan": (1, 40, 32760),  # the headline shape: WAN 2.2 self-attention, N(0,1) values
    "hires": (1, 40, 118320),  # the long hires-pass call: Q and K channels of uneven size (spread 2.3)
    "image": (1, 30, 4128),  # the image-model call: K channel spread 10.5, two V tokens 65x and 250x the rest
    "small": (1, 4, 1024),  # the reference emulator's own example, N(0,1)
}
MODES = ("per_channel", "per_token", "outliers", "fast")
PUBLISHED_RTX5080_TOPS = {"per_channel": 288.0}  # README.md:70-75: 76.3 ms on an RTX 5080, other hardware: not a baseline for B200
NOMINAL_PEAK_TOPS = {"per_channel": 4500.0, "per_token": 4500.0, "outliers": 4500.0, "fast": 9000.0}  # dense INT8 / NVFP4, datasheet
SPREAD = {"image": {1: 10.5}, "hires": {0: 2.3, 1: 2.3}}  # workload -> {tensor kind (0 q, 1 k, 2 v): max / median channel RMS}
V_OUTLIER_FACTORS = (65.0, 250.0)  # README.md:46: two V tokens of the image call, times the rest


def ops(batch, heads, nq, nk):
    return 4.0 * batch * heads * nq * nk * 128


def channel_factors(workload: str, kind: int, head: int) -> torch.Tensor | None:
    """Per-channel factors of tensor `kind` of one head: lognormal, then raised to the power that makes max / median
    exactly the workload's spread (the statistic the reference's node logs as channel_spread, comfyui/__init__.py:127-131)."""
    spread = SPREAD.get(workload, {}).get(kind)
    if spread is None:
        return None
    g = torch.Generator().manual_seed(7_000_003 * (kind + 1) + head)
    factors = torch.exp(0.6 * torch.randn(128, generator=g))
    have = (factors.max() / factors.median()).item()
    return factors ** (math.log(spread) / math.log(have))


def head_tensor(workload: str, kind: int, head: int, tokens: int) -> torch.Tensor:
    """Head `head` of q (0), k (1) or v (2) of a workload: bf16 [tokens, 128] from its own seed, on the CPU."""
    g = torch.Generator().manual_seed(1_000_003 * kind + head)
    x = torch.randn((tokens, 128), generator=g, dtype=torch.float32)
    factors = channel_factors(workload, kind, head)
    if factors is not None:
        x *= factors
    if workload == "image" and kind == 2:
        rows = torch.randperm(tokens, generator=torch.Generator().manual_seed(2_000_003 + head))[:2]
        for row, factor in zip(rows.tolist(), V_OUTLIER_FACTORS):
            x[row] *= factor
    return x.bfloat16()


def build_inputs(workload, batch, heads_slice, tokens, pin=True):
    out = []
    for kind in range(3):
        x = torch.empty((batch, len(heads_slice), tokens, 128), dtype=torch.bfloat16, pin_memory=pin)
        for i, h in enumerate(heads_slice):
            x[:, i] = head_tensor(workload, kind, h, tokens)
        out.append(x)
    return out


def channel_spread(x: torch.Tensor) -> float:
    """Largest channel RMS over the median channel's, per head, averaged (comfyui/__init__.py:127-131)."""
    rms = x.float().pow(2).mean(-2).sqrt()
    return (rms.amax(-1) / rms.median(-1).values).mean().item()


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 50 ms.  Started before the warm-up (the tool's own
    start-up takes driver locks for a few milliseconds: that must not fall into the timed region); `mark()` at the start of
    the timed region, and only the samples after it count."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.lines: list[str] = []
        self.first = 0
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        self.first = len(self.lines)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm, sm_max, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines[self.first:] or self.lines[-1:]:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                sm_max.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(mode: str, workload: str, tokens: int, sample_rows: int = 2048) -> dict:
    """The oracle port on one head x the first `sample_rows` queries x all keys, statistics over the whole head."""
    import oracle

    rows = min(sample_rows, tokens)
    oracle.threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count() or 1)  # all the host's cores
    q, k, v = (head_tensor(workload, kind, 0, tokens)[None] for kind in range(3))
    start = time.perf_counter()
    if mode == "fast":
        oracle.attention_fast(q, k, v, 512, recip=True, q_first=0, q_count=rows)
    else:
        oracle.attention_accurate(q, k, v, {"per_token": oracle.V_TOKEN, "outliers": oracle.V_OUTLIERS}.get(mode, oracle.V_CHANNEL), recip=True,
                                  q_first=0, q_count=rows)
    seconds = time.perf_counter() - start
    return {"value": ops(1, 1, rows, tokens) / seconds / 1e12, "unit": "TOPS", "cores": oracle.threads(), "kind": "port",
            "sample": f"1 head x first {rows} queries x all {tokens} keys (statistics and quantization of the whole head included), "
                      f"{seconds:.2f} s", "seconds": seconds}


def run_reference_arm(args, batch, heads, tokens):
    """--impl reference: the CPU port of the reference's emulation, all host threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times = []
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline(args.mode, args.workload, tokens, args.cpu_rows)
        if i >= args.warmup:
            times.append(base["seconds"])
    rows = min(args.cpu_rows, tokens)
    seconds = statistics.mean(times)
    value = ops(1, 1, rows, tokens) / seconds / 1e12
    base["value"] = value
    line = {"impl": "reference", "metric": metric_name(args.mode, batch, heads, tokens), "value": value, "unit": "TOPS",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype_of(args.mode), "data": "synthetic",
            "config": config_of(args, batch, heads, tokens), "cpu_baseline": {k: v for k, v in base.items() if k != "seconds"},
            "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference's CPU path for this operation is its PyTorch emulator; this times the C port of it "
                    "(oracle/) on a bounded sample per step; ms_per_step is that sample's time, not a whole call's"}
    print(json.dumps(line), flush=True)


def dtype_of(mode):
    return "nvfp4" if mode == "fast" else "int8"


def metric_name(mode, batch, heads, tokens):
    return f"eff. TOPS (ms/call in ms_per_step), {batch}x{heads}x{tokens}x128 bf16, {mode} (quant incl.)"


def config_of(args, batch, heads, tokens):
    return {"workload": f"{args.workload}: batch {batch}, heads {heads}, tokens {tokens}, head_dim 128, non-causal self-attention, "
                        f"mode {args.mode}", "l2": "inputs (3 x %.0f MB) larger than the 126 MB L2" % (batch * heads * tokens * 256 / 1e6),
            "sharding": f"heads over {args.gpus} GPU(s)" + (", gather of the output heads inside the step" if args.gpus > 1 else "")}


class Bench:
    """One process = one rank = one GPU."""

    def __init__(self, args):
        import unicaattention_b200 as unica
        from unicaattention_b200 import shard

        self.args, self.unica, self.shard = args, unica, shard
        self.gather_note = ("each attention kernel stores its output rows into every rank's copy over NVLink (peer stores), two barriers"
                            if args.gather == "peer" else "NCCL all-gathers of head groups on a side stream")
        self.rank, self.world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {self.world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
        torch.cuda.set_device(self.local)
        self.device = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.device)
            self.dist = dist
        try:
            self.peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        except (OSError, ValueError):
            self.peaks = {}

    # ------------------------------------------------------------------------------------------------------------ timing
    def barrier(self):
        torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, steps):
        """ms per step: CUDA events on the launching stream around `steps` calls, a barrier and a synchronize on both
        sides, the maximum over the ranks."""
        self.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        self.barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=self.device)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return ms.item() / steps

    # ------------------------------------------------------------------------------------------------------------ pieces
    def load(self, workload, heads=None, tokens=None):
        batch, all_heads, n = WORKLOADS[workload]
        all_heads, n = heads or all_heads, tokens or n
        mine = self.shard.head_slice(all_heads, self.rank, self.world)
        my_heads = list(range(mine.start, mine.stop))
        host = build_inputs(workload, batch, my_heads, n)
        dev = [x.to(self.device, non_blocking=True) for x in host]
        torch.cuda.synchronize()
        gathered = None
        if self.world > 1 and self.args.gather == "peer":
            try:  # the same outcome on every rank
                gathered = self.shard.SharedOutput(batch, all_heads, n)
            except RuntimeError as error:
                self.gather_note = f"NCCL all-gathers of head groups on a side stream (no shared output: {error})"
        if self.world > 1 and gathered is None:
            gathered = torch.empty((batch, all_heads, n, 128), dtype=torch.bfloat16, device=self.device)
        return {"workload": workload, "batch": batch, "heads": all_heads, "tokens": n, "my_heads": my_heads, "host": host, "dev": dev,
                "gathered": gathered}

    def step_fn(self, data, mode):
        unica, preset = self.unica, self.unica.PRESETS[mode]
        q, k, v = data["dev"]
        if self.world == 1:
            return lambda: unica.attention(q, k, v, **preset)
        gathered, heads = data["gathered"], data["heads"]
        return lambda: self.shard.attention_sharded(q, k, v, heads, out=gathered, **preset)

    def peak_of(self, mode):
        bf16 = self.peaks.get("bf16_tflops_sustained")
        factor = 4 if mode == "fast" else 2
        kind = "NVFP4 dense is four times" if mode == "fast" else "INT8 dense is twice"
        if bf16:
            return factor * bf16 * self.world, f"{factor} x MEASURED_PEAKS bf16_tflops_sustained ({kind} the bf16 rate; no measured entry of its own)"
        return factor * 1400.0 * self.world, f"{factor} x fallback sustained bf16 1.4 PFLOP/s"

    def accuracy(self, data, mode, rows=256):
        """Head 0 of this rank, the first `rows` queries against all keys: the kernel against the oracle's FP32 reference
        and against its emulation of the mode (outside every timed region)."""
        import oracle

        unica, preset = self.unica, self.unica.PRESETS[mode]
        q, k, v = (x[:, :1] for x in data["dev"])
        qs, ks, vs = (x[:, :1] for x in data["host"])
        rows = min(rows, data["tokens"])
        out = unica.attention(q, k, v, **preset)[0, 0, :rows].float().cpu().numpy()[None]
        ref = oracle.reference_fp32(qs, ks, vs, 0, rows)
        k_mean = (unica.rope_stats(k)[0] if mode == "fast" else unica.quantize_k(k)[2]).cpu()  # the mean the call itself takes away
        if mode == "fast":
            emu = oracle.attention_fast(qs, ks, vs, 512, recip=True, k_mean=k_mean, q_mean=unica.rope_stats(q, None, 512)[0].cpu(), q_count=rows)
        else:
            emu = oracle.attention_accurate(qs, ks, vs, {"per_token": oracle.V_TOKEN, "outliers": oracle.V_OUTLIERS}.get(mode, oracle.V_CHANNEL),
                                            recip=True, k_mean=k_mean, q_count=rows)
        return {"sample": f"head {data['my_heads'][0]}, first {rows} queries, all keys", "rel_l2_vs_fp32": oracle.rel_l2(out, ref),
                "emulation_rel_l2_vs_fp32": oracle.rel_l2(emu, ref), "rel_l2_vs_emulation": oracle.rel_l2(out, emu)}

    def measure(self, data, mode, steps, warmup, with_accuracy=True):
        """One preset on one workload: whole call, kernel alone, quantization alone, roofline fraction, accuracy sample."""
        from unicaattention_b200 import lib

        unica, preset = self.unica, self.unica.PRESETS[mode]
        q, k, v = data["dev"]
        step = self.step_fn(data, mode)
        for _ in range(warmup):
            step()
        unica.check_status(self.device)
        before = lib.launches
        ms_step = self.timed(step, steps)
        launches = lib.launches - before
        total_ops = ops(data["batch"], data["heads"], data["tokens"], data["tokens"])
        # Quantization alone.  Two untimed calls first: the operands are new allocations, and the first calls pay torch's
        # allocator going to the driver for them (milliseconds that a short timed loop would report as quantization).
        quantize = lambda: unica.kernel_inputs(q, k, v, **preset)  # noqa: E731
        for _ in range(2):
            quantize()
        ms_quant = self.timed(quantize, steps)
        inputs = quantize()
        kernel_only = lambda: unica.attention(q, k, v, inputs=inputs, **preset)  # noqa: E731
        for _ in range(2):
            kernel_only()
        ms_kernel = self.timed(kernel_only, steps)
        del inputs
        unica.check_status(self.device)
        peak, peak_source = self.peak_of(mode)
        achieved = total_ops / (ms_kernel * 1e-3) / 1e12  # all ranks run their share concurrently; max time over ranks
        tokens_total = data["batch"] * data["heads"] * data["tokens"]
        written = {"per_channel": 3 * 128, "per_token": 3 * 128 + 8, "outliers": 3 * 128, "fast": 72 + 72 + 82}[mode]
        result = {"ms_per_step": ms_step, "value": total_ops / (ms_step * 1e-3) / 1e12, "unit": "TOPS", "gpu_launches": launches,
                  "roofline": {"bound": "tensor", "kernel": "attention_fp4_kernel" if mode == "fast" else "attention_int8_kernel",
                               "achieved": achieved, "peak": peak, "unit": "TOP/s (x1e12)", "frac": achieved / peak, "ms_per_launch": ms_kernel,
                               "peak_source": peak_source, "frac_of_nominal": achieved / (NOMINAL_PEAK_TOPS[mode] * self.world)},
                  "quantization": {"ms": ms_quant, "algorithmic_gbs": (3 * 256 + written) * tokens_total / self.world / (ms_quant * 1e-3) / 1e9,
                                   "hbm_peak_gbs": self.peaks.get("hbm_gbs")},
                  "grid": unica.wave_plan(data["batch"] * len(data["my_heads"]), data["tokens"], preset.get("kernel", unica.DEFAULT_KERNEL), self.device)}
        if with_accuracy and self.rank == 0:
            result["accuracy"] = self.accuracy(data, mode)
        return result

    def e2e(self, data, mode, steps):
        """Host to host: every rank feeds its own heads from pinned host memory through the library's pipelined host call
        and copies its own heads of the result back; no gather on the device (the result is wanted in host memory)."""
        unica, preset = self.unica, self.unica.PRESETS[mode]
        qh, kh, vh = data["host"]
        out_host = torch.empty(qh.shape, dtype=torch.bfloat16, pin_memory=True)
        run = lambda: unica.attention_host(qh, kh, vh, out=out_host, device=self.device, **preset)  # noqa: E731
        run()
        ms = self.timed(run, max(1, min(steps, 5)))
        sizes = torch.tensor([sum(x.numel() * 2 for x in (qh, kh, vh)), out_host.numel() * 2], device=self.device, dtype=torch.float64)
        if self.world > 1:
            self.dist.all_reduce(sizes)
        total_ops = ops(data["batch"], data["heads"], data["tokens"], data["tokens"])
        return {"value": total_ops / (ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": ms, "h2d_bytes_per_step": int(sizes[0].item()),
                "d2h_bytes_per_step": int(sizes[1].item()),
                "how": "attention_host per rank on its own heads: copies in, kernels and copies out overlapped in head groups; job-wide bytes"}

    # -------------------------------------------------------------------------------------------------------------- run
    def run(self):
        args, unica = self.args, self.unica
        data = self.load(args.workload, args.heads, args.tokens)
        batch, heads, tokens = data["batch"], data["heads"], data["tokens"]
        if args.profile:
            step = self.step_fn(data, args.mode)
            for _ in range(1 + args.steps):
                step()
            unica.check_status(self.device)
            return
        sampler = ClockSampler(self.local) if self.rank == 0 else None
        step = self.step_fn(data, args.mode)
        for _ in range(args.warmup):
            step()
        if sampler:
            sampler.mark()
        head = self.measure(data, args.mode, args.steps, 0)
        clocks = sampler.stop() if sampler else None
        e2e = None if args.no_e2e else self.e2e(data, args.mode, args.steps)
        short = max(3, min(args.steps, 5))
        modes = {}
        if not args.no_modes:
            for mode in MODES:
                if mode != args.mode:
                    modes[mode] = self.measure(data, mode, short, 3)
        spreads = {"q": channel_spread(data["dev"][0]), "k": channel_spread(data["dev"][1])}
        del data, step
        torch.cuda.empty_cache()
        configs = {}
        if not args.no_configs:
            for workload in ("image", "hires"):
                if workload == args.workload:
                    continue  # (30 heads over 4 or 8 ranks: uneven slices, which both ways of gathering take)
                other = self.load(workload, None, args.hires_tokens if workload == "hires" else None)
                entry = {"shape": [other["batch"], other["heads"], other["tokens"], 128],
                         "inputs": {"q_channel_spread": channel_spread(other["dev"][0]), "k_channel_spread": channel_spread(other["dev"][1]),
                                    "v_max_over_median_token": (lambda a: (a.amax(-1) / a.median(-1).values).mean().item())(other["dev"][2].float().abs().amax(-1)),
                                    "seeds": "q/k/v head h: 1000003 * kind + h; channel factors: 7000003 * (kind + 1) + h; V outlier rows: 2000003 + h"}}
                for mode in (("per_channel", "per_token", "fast") if workload == "image" else ("per_channel", "fast")):
                    entry[mode] = self.measure(other, mode, 3, 3)
                configs[workload] = entry
                del other
                torch.cuda.empty_cache()
        if self.rank == 0:
            from unicaattention_b200 import peak as peak_bench

            mix = {m: peak_bench.attention_mix_tops(m, (clocks or {}).get("sm_max_mhz") or 1965.0) * self.world for m in ("accurate", "fast")}
            for name, entry in [(args.mode, head), *modes.items()]:
                entry["roofline"]["tensor_mix_microbench"] = mix["fast" if name == "fast" else "accurate"]
                entry["roofline"]["frac_of_tensor_mix_microbench"] = entry["roofline"]["achieved"] / entry["roofline"]["tensor_mix_microbench"]
            # DRAM traffic of the attention kernel per launch: one ncu capture on 40 heads x 8192 tokens scaled by heads x
            # tokens (every K/V tile comes from HBM once and is re-read from L2, so traffic grows with the token count)
            per_token_bytes = {"per_channel": 552.7, "fast": 441.9}.get(args.mode)
            head["roofline"]["traffic"] = per_token_bytes * batch * heads * tokens / self.world if per_token_bytes else None
            head["roofline"]["traffic_unit"] = "bytes per launch per GPU, derived: ncu dram bytes of a 40 x 8192 capture scaled by heads x tokens"
            line = {"metric": metric_name(args.mode, batch, heads, tokens), "value": head["value"], "unit": "TOPS", "n_gpus": self.world,
                    "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
                    "scaling": "strong", "vs_baseline": None, "dtype": dtype_of(args.mode), "data": "synthetic",
                    "config": config_of(args, batch, heads, tokens) | {"input_channel_spread": spreads} | ({"gather": self.gather_note} if self.world > 1 else {}), "clocks": clocks, "e2e": e2e,
                    "gpu_launches": head["gpu_launches"], "roofline": head["roofline"], "quantization": head["quantization"], "grid": head.get("grid"),
                    "accuracy": head.get("accuracy"), "modes": modes, "configs": configs,
                    "published_other_hardware": {"rtx5080_tops": PUBLISHED_RTX5080_TOPS.get(args.mode)}}
            if not args.no_cpu and self.world == 1:
                base = cpu_baseline(args.mode, args.workload, tokens, args.cpu_rows)
                line["cpu_baseline"] = {k_: v_ for k_, v_ in base.items() if k_ != "seconds"}
            print(json.dumps(line), flush=True)
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--mode", default="per_channel", choices=list(MODES))
    ap.add_argument("--workload", default="wan", choices=list(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=2048, help="query rows of the CPU baseline's sample")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-to-host leg")
    ap.add_argument("--no-modes", action="store_true", help="skip the other presets")
    ap.add_argument("--no-configs", action="store_true", help="skip the image and hires signatures")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="N > 1: output rows stored to every rank by the attention kernel (peer), or NCCL all-gathers of head groups")
    ap.add_argument("--heads", type=int, default=0, help="override the workload's head count (profiling on a small case)")
    ap.add_argument("--tokens", type=int, default=0, help="override the workload's token count (profiling on a small case)")
    ap.add_argument("--hires-tokens", type=int, default=0, help="override the hires signature's token count")
    ap.add_argument("--profile", action="store_true",
                    help="for captures under a profiler: one warm-up call and --steps calls, nothing else, no JSON line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not args.profile else args.warmup
    if args.impl == "reference":
        batch, heads, tokens = WORKLOADS[args.workload]
        return run_reference_arm(args, batch, args.heads or heads, args.tokens or tokens)
    Bench(args).run()


if __name__ == "__main__":
    main()
