"""python -m unicaattention_b200.peak: measured per-SM ceilings of the instructions the attention kernels use, and the
tensor-core rate they imply for this GPU (the reference's bench/peak.py).  One block per SM."""

from __future__ import annotations

import ctypes

import torch

from unicaattention_b200 import lib

KINDS = {"i8": 0, "nvf4": 1, "ex2": 2, "fma.f32x2": 3, "fma.f32": 4, "prmt": 5, "cvt.f32.s32": 6, "cvt.u32.f32": 7}


def cycles(kind: str, n: int = 0, count: int = 4096, blocks: int | None = None) -> float:
    """Cycles per instruction (tensor kinds: per tcgen05.mma of 128 x n x K; others: per warp instruction per scheduler)."""
    blocks = blocks or torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    out = ctypes.c_double()
    lib.call("unica_b200_peak", KINDS[kind], n, count, blocks, ctypes.byref(out), lib.stream())
    return out.value


def tensor_tops(kind: str, n: int, sm_mhz: float, sms: int | None = None) -> float:
    """Dense rate of the whole GPU for one MMA shape, from its measured cycles, at the given SM clock."""
    sms = sms or torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    k = 32 if kind == "i8" else 64
    return 2.0 * 128 * n * k / cycles(kind, n) * sm_mhz * 1e6 * sms / 1e12


def attention_mix_tops(mode: str, sm_mhz: float) -> float:
    """The tensor ceiling of one attention tile's instruction mix at the given clock: accurate = 4 MMAs 128x64x32 (scores)
    + 2 MMAs 128x128x32 (P.V); fast = 2 MMAs 128x64x64 + 1 MMA 128x144x64 (the extra 16 columns are the denominator)."""
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    if mode == "fast":
        clk = 2 * cycles("nvf4", 64) + cycles("nvf4", 144)
    else:
        clk = 4 * cycles("i8", 64) + 2 * cycles("i8", 128)
    return 4.0 * 128 * 64 * 128 / clk * sm_mhz * 1e6 * sms / 1e12


def main() -> None:
    props = torch.cuda.get_device_properties(0)
    mhz = props.clock_rate / 1e3 if hasattr(props, "clock_rate") else 1965.0
    print(f"{props.name}, {props.multi_processor_count} SMs, rates at {mhz:.0f} MHz")
    for kind in ("i8", "nvf4"):
        for n in (64, 128, 144, 240):
            c = cycles(kind, n)
            k = 32 if kind == "i8" else 64
            print(f"  tcgen05.mma kind::{kind:5} 128x{n:3}x{k}: {c:7.1f} clk per MMA = {2 * 128 * n * k / c:8.0f} op/clk/SM "
                  f"= {2 * 128 * n * k / c * mhz * 1e6 * props.multi_processor_count / 1e12:7.0f} TOPS")
    for kind in ("ex2", "fma.f32x2", "fma.f32", "prmt", "cvt.f32.s32", "cvt.u32.f32"):
        print(f"  {kind:12} {cycles(kind, count=2000):5.2f} clk per warp instruction per scheduler")
    for mode in ("accurate", "fast"):
        print(f"  attention tile mix, {mode}: {attention_mix_tops(mode, mhz):.0f} TOPS")


if __name__ == "__main__":
    main()
