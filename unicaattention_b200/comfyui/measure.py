"""Measurement mode of the ComfyUI nodes: every n-th live self-attention call is run again, on its first few heads, by
every preset of the library and by exact FP32 attention, and one CSV row records the errors, the times and what the
inputs looked like (the reference's Measurement, comfyui/__init__.py:141-241, without its SageAttention columns).
Optionally the measured q, k, v are saved, which is how real-activation dumps for offline work come to exist.

Off (every = 0) it reads nothing and costs nothing: looking at the sampler's sigma is a device-to-host copy that would
stall the launch queue on every call.

An emulation column is filled only when an emulator is given: point UNICA_EMULATOR at a directory that holds the
reference project's bench/emulate.py and its `emulate(q, k, v, **config)` is run with the fast mode's configuration.
The library itself ships no emulator.
"""

from __future__ import annotations

import collections
import csv
import importlib.util
import logging
import os
import time
from pathlib import Path

import torch

import unicaattention_b200 as unica

log = logging.getLogger("UnicaAttention")
PRESET_COLUMNS = ("per_channel", "per_token", "outliers", "fast")
CSV_FIELDS = ["time", "tag", "node", "ran", "routes", "call", "step", "block", "batch", "tokens", "keys", "heads_measured",
              "unica_rel_l2", "unica_cos", "unica_ms", *(f"{name}_{what}" for name in PRESET_COLUMNS for what in ("rel_l2", "cos")),
              "emulated_fast_rel_l2", "q_channel_spread", "k_channel_spread", "v_offset", "q_offset"]
# the fast mode as the reference's emulator is configured for it (tests/test_fp4.py:24-25, 120-126)
EMULATED_FAST = dict(qk="nvfp4", p_fmt="nvfp4", v_fmt="nvfp4", p_local=False, sum_rounded=True, p_mul=1024.0, p_outer=1.0,
                     v_outer="channel", fp4_slots=True, smooth_q=512)


def output_dir() -> Path:
    """Where the CSV and the dumps go: UNICA_MEASURE_DIR, else ./unica_measure."""
    return Path(os.environ.get("UNICA_MEASURE_DIR", "unica_measure"))


def exact_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rows: int = 2048) -> torch.Tensor:
    """FP32 softmax(q k^T / sqrt(d)) v on [batch, heads, tokens, d], `rows` query rows at a time."""
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    kt, vf = k.float().transpose(-1, -2), v.float()
    for first in range(0, q.shape[2], rows):
        piece = slice(first, first + rows)
        out[:, :, piece] = torch.softmax(q[:, :, piece].float() @ kt * q.shape[-1] ** -0.5, -1) @ vf
    return out


def errors(out: torch.Tensor, exact: torch.Tensor) -> dict:
    out, exact = out.float().flatten(), exact.float().flatten()
    return {"rel_l2": ((out - exact).norm() / exact.norm()).item(), "cos": torch.nn.functional.cosine_similarity(out, exact, 0).item()}


def channel_spread(x: torch.Tensor) -> float:
    """Largest channel RMS over the median channel's, per head, averaged: 1 = even channels."""
    rms = x.float().pow(2).mean(-2).sqrt()
    return (rms.amax(-1) / rms.median(-1).values).mean().item()


def constant_share(x: torch.Tensor) -> float:
    """How much of x is a constant per channel: RMS of the channel means over RMS of x (0 = centred)."""
    x = x.float()
    return (x.mean(-2).pow(2).mean().sqrt() / x.pow(2).mean().sqrt()).item()


def emulator():
    """`emulate` of a reference checkout named by UNICA_EMULATOR, or None."""
    where = os.environ.get("UNICA_EMULATOR")
    path = Path(where) / "emulate.py" if where else None
    if path is None or not path.is_file():
        return None
    spec = importlib.util.spec_from_file_location("unica_measure_emulator", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module.emulate


class Measurement:
    """The state of one node's measurement: how often, how many heads, where the count stands."""

    def __init__(self, node: str) -> None:
        self.node, self.tag = node, ""
        self.every = self.heads = self.calls = 0
        self.step: int | None = 0
        self.block: int | None = None
        self.sigma: float | None = None
        self.numbered = False  # whether the model's calls carry a block index
        self.routes: collections.Counter = collections.Counter()  # "unica", or why a call went elsewhere

    def configure(self, every: int, heads: int, tag: str = "") -> None:
        self.every, self.heads, self.tag = every, heads, tag

    def route(self, reason: str | None, q: torch.Tensor, k: torch.Tensor) -> None:
        """Counts where a call went; the first call passed on for each reason is logged with its shapes."""
        key = reason or "unica"
        if reason is not None and not self.routes[key]:
            log.info("%s [%s]: passed on (%s), q %s, k %s", self.node, self.tag, reason, tuple(q.shape), tuple(k.shape))
        self.routes[key] += 1

    def due(self, options: dict | None = None) -> bool:
        """Advances the count and says whether this call is measured.  With ComfyUI's transformer_options (sigmas and a
        block index) the count is step * blocks + block + 1 inside one sampling run: the step advances when sigma
        falls and starts over when it rises, so every run measures the same (step, block) pairs.  Calls that carry sigmas
        but no block index are skipped once the model has been seen to number its blocks (context refiners), counted
        one by one if it never does; without options at all, a plain count."""
        if self.every == 0:
            return False
        options = options or {}
        block, sigmas = options.get("block_index"), options.get("sigmas")
        if sigmas is None or (block is None and not self.numbered):
            self.calls += 1
            self.step = self.block = None
        elif block is None:
            return False
        else:
            self.numbered = True
            sigma = float(sigmas.max())
            if self.sigma is None or self.step is None or sigma > self.sigma:
                self.step = 0
            elif sigma < self.sigma:
                self.step += 1
            self.sigma, self.block = sigma, block
            self.calls = self.step * options.get("total_blocks", 40) + block + 1
        return self.calls % self.every == 0

    def __call__(self, q, k, v, settings: dict, options: dict | None = None) -> None:
        """q, k, v [batch, tokens, heads, 128] of a call unica has just run with `settings`."""
        if self.due(options):
            self.measure(q, k, v, settings)

    def measure(self, q, k, v, settings: dict) -> dict:
        heads = min(self.heads or 1, q.shape[2])
        bhnd = [x[:, :, :heads].transpose(1, 2).to(torch.bfloat16).contiguous() for x in (q, k, v)]
        exact = exact_attention(*bhnd)
        ran = next((name for name, preset in unica.PRESETS.items() if preset == settings), "custom")
        row = {"time": time.strftime("%H:%M:%S"), "tag": self.tag, "node": self.node, "ran": ran,
               "routes": " ".join(f"{key}={n}" for key, n in sorted(self.routes.items())), "call": self.calls, "step": self.step,
               "block": self.block, "batch": q.shape[0], "tokens": q.shape[1], "keys": k.shape[1], "heads_measured": heads}
        on_gpu = bhnd[0].device.type == "cuda"
        if on_gpu:
            torch.cuda.synchronize(bhnd[0].device)
        start = time.perf_counter()
        mine = unica.attention(*bhnd, **settings)
        if on_gpu:
            torch.cuda.synchronize(bhnd[0].device)
        row["unica_ms"] = (time.perf_counter() - start) * 1e3
        for name, out in [("unica", mine), *((name, unica.attention(*bhnd, **unica.PRESETS[name])) for name in PRESET_COLUMNS)]:
            e = errors(out, exact)
            row[f"{name}_rel_l2"], row[f"{name}_cos"] = e["rel_l2"], e["cos"]
        emulate = emulator()
        if emulate is not None:
            row["emulated_fast_rel_l2"] = errors(emulate(*bhnd, **EMULATED_FAST), exact)["rel_l2"]
        row["q_channel_spread"], row["k_channel_spread"] = channel_spread(bhnd[0]), channel_spread(bhnd[1])
        row["v_offset"], row["q_offset"] = constant_share(bhnd[2]), constant_share(bhnd[0])
        folder = output_dir()
        folder.mkdir(parents=True, exist_ok=True)
        if (folder / "dumps.flag").exists():  # the measured q, k, v themselves, to take an error apart offline
            (folder / "dumps").mkdir(exist_ok=True)
            torch.save({"q": bhnd[0].cpu(), "k": bhnd[1].cpu(), "v": bhnd[2].cpu(), "row": row},
                       folder / "dumps" / f"{self.tag or self.node}_call{self.calls}_{time.monotonic_ns()}.pt")
        table = folder / "attention_errors.csv"
        new = not table.exists()
        with table.open("a", newline="") as f:
            writer = csv.DictWriter(f, fieldnames=CSV_FIELDS)
            if new:
                writer.writeheader()
            writer.writerow(row)
        log.info("%s call %d, %d tokens: rel L2 as run (%s) %.3f %%; %s; channel spread q %.2f k %.2f, v offset %.3f", self.node,
                 self.calls, q.shape[1], ran, 100 * row["unica_rel_l2"],
                 ", ".join(f"{name} {100 * row[f'{name}_rel_l2']:.3f} %" for name in PRESET_COLUMNS), row["q_channel_spread"],
                 row["k_channel_spread"], row["v_offset"])
        return row
