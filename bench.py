"""Benchmark of the quantized-attention forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--mode per_channel|per_token|outliers|fast] [--workload wan|hires|image|small]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...
    python bench.py --impl reference ...      # the CPU oracle port timed on the host cores, same config and metric

One step = one whole call `unica.attention(q, k, v, **preset)` (statistics + quantization + attention kernel) on the
named workload; with N > 1 the heads are sharded over the ranks and the step ends with an NCCL all-gather of the
output heads.  Prints ONE JSON line (rank 0):

  value      effective TOPS = 4 * B * H * Nq * Nk * 128 / time (the reference's formula, bench/harness.py:69), whole job,
             inputs resident in HBM; ms_per_step is the ms/call of the same runs
  e2e        the same call fed from pinned host memory with the result copied back, every step
  roofline   the attention kernel alone (operands already quantized), timed with CUDA events, against the tensor peak
  cpu_baseline  the CPU oracle port on a bounded sample (1 head x 2048 queries x all keys), all host threads
Inputs are synthetic: seeded N(0,1) bf16 of the named shape, generated per head on the CPU so each rank builds its shard.
"""

from __future__ import annotations

import argparse
import json
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

WORKLOADS = {  # (batch, heads, tokens): BASELINE.json configs
    "wan": (1, 40, 32760),  # configs[1] / [2]: the headline shape
    "hires": (1, 40, 118320),  # configs[4]
    "image": (1, 30, 4128),  # configs[3] (shape only; N(0,1) values here)
    "small": (1, 4, 1024),  # configs[0]
}
PUBLISHED_RTX5080_TOPS = {"per_channel": 288.0}  # 76.3 ms on an RTX 5080, other hardware: not a baseline for B200
NOMINAL_PEAK_TOPS = {"per_channel": 4500.0, "per_token": 4500.0, "outliers": 4500.0, "fast": 9000.0}  # dense INT8 / NVFP4, datasheet


def ops(batch, heads, nq, nk):
    return 4.0 * batch * heads * nq * nk * 128


def head_tensor(kind: int, head: int, tokens: int) -> torch.Tensor:
    """Head `head` of q (0), k (1) or v (2): N(0,1) bf16 [tokens, 128] from its own seed, on the CPU."""
    g = torch.Generator().manual_seed(1_000_003 * kind + head)
    return torch.randn((tokens, 128), generator=g, dtype=torch.float32).bfloat16()


def build_inputs(batch, heads_slice, tokens, pin=True):
    out = []
    for kind in range(3):
        x = torch.empty((batch, len(heads_slice), tokens, 128), dtype=torch.bfloat16, pin_memory=pin)
        for i, h in enumerate(heads_slice):
            x[:, i] = head_tensor(kind, h, tokens)
        out.append(x)
    return out


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


def cpu_baseline(mode: str, tokens: int, sample_rows: int = 2048) -> dict:
    """The oracle port on one head x the first `sample_rows` queries x all keys, statistics over the whole head."""
    import oracle

    rows = min(sample_rows, tokens)
    oracle.threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count() or 1)  # all the host's cores
    q, k, v = (head_tensor(kind, 0, tokens)[None] for kind in range(3))
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
        base = cpu_baseline(args.mode, tokens, args.cpu_rows)
        if i >= args.warmup:
            times.append(base["seconds"])
    rows = min(args.cpu_rows, tokens)
    seconds = statistics.mean(times)
    value = ops(1, 1, rows, tokens) / seconds / 1e12
    base["value"] = value
    line = {"impl": "reference", "metric": metric_name(args, batch, heads, tokens), "value": value, "unit": "TOPS",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype_of(args.mode), "data": "synthetic",
            "config": config_of(args, batch, heads, tokens), "cpu_baseline": {k: v for k, v in base.items() if k != "seconds"},
            "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference's CPU path for this operation is its PyTorch emulator; this times the C port of it "
                    "(oracle/) on a bounded sample per step; ms_per_step is that sample's time, not a whole call's"}
    print(json.dumps(line), flush=True)


def dtype_of(mode):
    return "nvfp4" if mode == "fast" else "int8"


def metric_name(args, batch, heads, tokens):
    return f"eff. TOPS (ms/call in ms_per_step), {batch}x{heads}x{tokens}x128 bf16, {args.mode} (quant incl.)"


def config_of(args, batch, heads, tokens):
    return {"workload": f"{args.workload}: batch {batch}, heads {heads}, tokens {tokens}, head_dim 128, non-causal self-attention, "
                        f"mode {args.mode}", "l2": "inputs (3 x %.0f MB) larger than the 126 MB L2" % (batch * heads * tokens * 256 / 1e6),
            "sharding": f"heads over {args.gpus} GPU(s)" + (", NCCL all-gather of output heads inside the step" if args.gpus > 1 else "")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--mode", default="per_channel", choices=["per_channel", "per_token", "outliers", "fast"])
    ap.add_argument("--workload", default="wan", choices=list(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=2048, help="query rows of the CPU baseline's sample")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-to-host leg")
    ap.add_argument("--heads", type=int, default=0, help="override the workload's head count (profiling on a small case)")
    ap.add_argument("--tokens", type=int, default=0, help="override the workload's token count (profiling on a small case)")
    ap.add_argument("--profile", action="store_true",
                    help="for captures under a profiler: one warm-up call and --steps calls, nothing else, no JSON line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not args.profile else args.warmup
    batch, heads, tokens = WORKLOADS[args.workload]
    heads, tokens = args.heads or heads, args.tokens or tokens
    if args.impl == "reference":
        return run_reference_arm(args, batch, heads, tokens)

    import unicaattention_b200 as unica

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    from unicaattention_b200 import shard

    mine = shard.head_slice(heads, rank, world)
    my_heads = list(range(mine.start, mine.stop))
    preset = unica.PRESETS[args.mode]
    q_host, k_host, v_host = build_inputs(batch, my_heads, tokens)
    q, k, v = (x.to(device, non_blocking=True) for x in (q_host, k_host, v_host))
    gathered = torch.empty((batch, heads, tokens, 128), dtype=torch.bfloat16, device=device) if world > 1 else None

    def step(q, k, v):
        out = unica.attention(q, k, v, **preset)
        if world > 1:
            shard.gather_heads(out, gathered, heads, rank, world)
            return gathered
        return out

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps

    if args.profile:
        for _ in range(1 + args.steps):
            step(q, k, v)
        unica.check_status(device)
        return
    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(args.warmup):
        step(q, k, v)
    unica.check_status(device)
    if sampler:
        sampler.mark()
    ms_step = timed(lambda: step(q, k, v), args.steps)
    clocks = sampler.stop() if sampler else None
    total_ops = ops(batch, heads, tokens, tokens)
    value = total_ops / (ms_step * 1e-3) / 1e12

    # the attention kernel alone, operands already quantized (this rank's heads)
    inputs = unica.kernel_inputs(q, k, v, **preset)
    kernel_only = lambda: unica.attention(q, k, v, inputs=inputs, **preset)  # noqa: E731
    for _ in range(2):
        kernel_only()
    ms_kernel = timed(kernel_only, args.steps)
    ms_quant = timed(lambda: unica.kernel_inputs(q, k, v, **preset), args.steps)
    achieved = total_ops / (ms_kernel * 1e-3) / 1e12  # all ranks run their share concurrently; max time over ranks

    # end to end: pinned host inputs in, result out, every step
    e2e = None
    if not args.no_e2e:
        out_host = torch.empty((batch, len(my_heads) if world == 1 else heads, tokens, 128), dtype=torch.bfloat16, pin_memory=True)

        def e2e_step():
            if world == 1:  # the library's host-memory call: head groups, copies in and out overlapping the kernels
                unica.attention_host(q_host, k_host, v_host, out=out_host, device=device, **preset)
            else:
                qd, kd, vd = (x.to(device, non_blocking=True) for x in (q_host, k_host, v_host))
                out_host.copy_(step(qd, kd, vd), non_blocking=True)

        e2e_step()
        ms_e2e = timed(e2e_step, max(1, min(args.steps, 5)))
        e2e = {"value": total_ops / (ms_e2e * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": sum(x.numel() * 2 for x in (q_host, k_host, v_host)),
               "d2h_bytes_per_step": out_host.numel() * 2}
    unica.check_status(device)

    if rank == 0:
        import oracle

        peaks = {}
        try:
            peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        except (OSError, ValueError):
            pass
        bf16 = peaks.get("bf16_tflops_sustained")
        peak, peak_source = (2 * bf16 * world, "2 x MEASURED_PEAKS bf16_tflops_sustained (INT8 dense is twice the bf16 rate; no measured INT8 entry)") \
            if bf16 else (2 * 1400.0 * world, "2 x fallback sustained bf16 1.4 PFLOP/s")
        if args.mode == "fast":
            peak, peak_source = 2 * peak, peak_source.replace("2 x", "4 x").replace("INT8 dense is twice", "NVFP4 dense is four times")
        # accuracy on a bounded sample: head 0 of this rank, 256 query rows against all keys
        rows = min(256, tokens)
        out = unica.attention(q[:, :1], k[:, :1], v[:, :1], **preset)[0, 0, :rows].float().cpu().numpy()[None]
        qs, ks, vs = q_host[:, :1], k_host[:, :1], v_host[:, :1]
        ref = oracle.reference_fp32(qs, ks, vs, 0, rows)
        k_mean = unica.rope_stats(k[:, :1])[0].cpu()
        q_mean = unica.rope_stats(q[:, :1], None, 512)[0].cpu() if args.mode == "fast" else None
        emu = (oracle.attention_fast(qs, ks, vs, 512, recip=True, k_mean=k_mean, q_mean=q_mean, q_count=rows) if args.mode == "fast" else
               oracle.attention_accurate(qs, ks, vs, {"per_token": oracle.V_TOKEN, "outliers": oracle.V_OUTLIERS}.get(args.mode, oracle.V_CHANNEL), recip=True,
                                         k_mean=k_mean, q_count=rows))
        # this library's launches per call: statistics (2 per pass), quantizers, (outer scales, smoothing term), attention
        launches_per_step = {"per_channel": 8, "per_token": 6, "outliers": 8, "fast": 13}[args.mode]
        kernel_name = "attention_fp4_kernel" if args.mode == "fast" else "attention_int8_kernel"
        # bytes the quantization passes must move per head and token: bf16 read of Q, K, V + the operands written
        written = {"per_channel": 3 * 128, "per_token": 3 * 128 + 8, "outliers": 3 * 128, "fast": 72 + 72 + 82}[args.mode]
        reads = {"per_channel": 5 * 256, "per_token": 4 * 256, "outliers": 6 * 256, "fast": 7 * 256}[args.mode]  # statistics passes read again
        # DRAM traffic of the attention kernel per launch: ncu on 40 heads x 8192 tokens (profiles/), scaled by heads x tokens
        # (per channel: 125.99 MB read + 51.16 MB written; fast: 97.06 + 44.97 MB, the rest of the output still in L2)
        traffic_per_token = {"per_channel": 540.6, "fast": 433.4}.get(args.mode)
        traffic = traffic_per_token * batch * heads * tokens / world if traffic_per_token else None
        # what the tensor pipe alone sustains on one tile's tcgen05.mma mix, measured now by the micro-benchmark
        from unicaattention_b200 import peak as peak_bench
        mix_tops = peak_bench.attention_mix_tops("fast" if args.mode == "fast" else "accurate", clocks.get("sm_max_mhz") or 1965.0) * world
        line = {
            "metric": metric_name(args, batch, heads, tokens), "value": value, "unit": "TOPS", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": dtype_of(args.mode), "data": "synthetic", "config": config_of(args, batch, heads, tokens),
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "tensor", "kernel": kernel_name, "achieved": achieved, "peak": peak, "unit": "TOP/s (x1e12)",
                         "frac": achieved / peak, "traffic": traffic, "traffic_unit": "bytes per launch per GPU", "ms_per_launch": ms_kernel,
                         "peak_source": peak_source, "frac_of_nominal": achieved / (NOMINAL_PEAK_TOPS[args.mode] * world),
                         "tensor_mix_microbench": mix_tops, "frac_of_tensor_mix_microbench": achieved / mix_tops},
            "quantization": {"ms": ms_quant, "algorithmic_gbs": (3 * 256 + written) * batch * heads * tokens / world / (ms_quant * 1e-3) / 1e9,
                             "moved_gbs": (reads + written) * batch * heads * tokens / world / (ms_quant * 1e-3) / 1e9,
                             "hbm_peak_gbs": peaks.get("hbm_gbs")},
            "accuracy": {"sample": f"head {my_heads[0]}, first {rows} queries, all keys", "rel_l2_vs_fp32": oracle.rel_l2(out, ref),
                         "emulation_rel_l2_vs_fp32": oracle.rel_l2(emu, ref), "rel_l2_vs_emulation": oracle.rel_l2(out, emu)},
            "published_other_hardware": {"rtx5080_tops": PUBLISHED_RTX5080_TOPS.get(args.mode)},
        }
        if not args.no_cpu and world == 1:
            base = cpu_baseline(args.mode, tokens, args.cpu_rows)
            line["cpu_baseline"] = {k_: v_ for k_, v_ in base.items() if k_ != "seconds"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
