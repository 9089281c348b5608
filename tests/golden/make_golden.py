"""Generates tests/golden/golden.npz from the reference's own emulator (bench/emulate.py), imported from a checkout.

Run once where the reference checkout exists (it does not travel with the tests):

    python tests/golden/make_golden.py /path/to/reference

Everything is computed on CPU tensors, so scalar divisions are IEEE divisions (the oracle's recip=False form).  For each
case the file holds the inputs (bf16 bits; the seed-0 headline case is regenerated from its seed and only its checksum
is kept), the emulator's quantizer pieces (codes and scales) and the emulator's outputs for the contract
configurations, so that tests can pin the oracle without the reference being present.
"""

from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit(__doc__)
REF = Path(sys.argv[1])
sys.path.insert(0, str(REF / "bench"))
from emulate import FP4_SLOT_KEY, TODAY, block_scaled, emulate, errors, quant, reference, to_e2m1, to_fmt  # noqa: E402

FAST = TODAY | dict(p_fmt="nvfp4", v_fmt="nvfp4", p_local=False, p_mul=1024.0, p_outer=1.0, v_outer="channel",
                    fp4_slots=True, qk="nvfp4", smooth_q=512)
OUT = Path(__file__).resolve().parent / "golden.npz"


def bits(x: torch.Tensor) -> np.ndarray:
    return x.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def nvfp4_pieces(x: torch.Tensor, dim: int, outer):
    """The scale bytes, outer scale and dequantized values of block_scaled(x, "nvfp4", dim, outer), recomputed step by
    step the way emulate.py:98-113 does, so the oracle's bytes can be compared, not only its dequantized values."""
    xm = x.movedim(dim, -1)
    n = xm.shape[-1]
    blocks = torch.nn.functional.pad(xm, (0, -n % 16)).unflatten(-1, (-1, 16))
    amax = blocks.abs().amax(-1, keepdim=True)
    over = (-3, -2, -1) if outer is None else (-2, -1)
    o = (amax.amax(over, keepdim=True) / (6.0 * 448.0)).clamp_min(1e-30)
    sf = (amax / 6.0 / o).clamp(max=448.0).to(torch.float8_e4m3fn)
    return sf.view(torch.uint8)[..., 0].numpy(), o.numpy()


def slot_order(v: torch.Tensor) -> torch.Tensor:
    n = v.shape[-2]
    tiles = -(-n // 64)
    order = torch.arange(tiles * 64).view(tiles, -1)[:, FP4_SLOT_KEY].flatten()
    return torch.nn.functional.pad(v.float(), (0, 0, 0, tiles * 64 - n))[..., order, :]


def case(name: str, q, k, v, store_inputs: bool, rows: int | None, out: dict):
    """rows: keep only every (n // rows)-th query row of the outputs (None: all)."""
    qf, kf, vf = q.float(), k.float(), v.float()
    pre = name + "/"
    if store_inputs:
        out[pre + "q"], out[pre + "k"], out[pre + "v"] = bits(q), bits(k), bits(v)
    out[pre + "input_sha"] = np.array(sha(np.concatenate([bits(t).ravel() for t in (q, k, v)])))
    out[pre + "shape_q"], out[pre + "shape_k"] = np.array(q.shape), np.array(k.shape)

    # ---- quantizer pieces, as the reference's tests compose them (tests/test_quantize.py:22-46, tests/test_fp4.py:51-75)
    k_mean = kf.mean(-2)
    out[pre + "k_mean"] = k_mean.numpy()
    q8, sq = quant(qf, "int8", 128)
    k8, sk = quant(kf - k_mean[..., None, :], "int8", 64)
    out[pre + "q8_sha"], out[pre + "k8_sha"] = np.array(sha(q8.to(torch.int8).numpy())), np.array(sha(k8.to(torch.int8).numpy()))
    out[pre + "q_scale"], out[pre + "k_scale"] = sq[..., ::128, 0].numpy(), sk[..., ::64, 0].numpy()
    sv = (vf.abs().amax(-2, keepdim=True) / 127.0).clamp_min(1e-12)
    v8 = to_fmt(vf / sv, "int8")
    out[pre + "v8_sha"], out[pre + "v_scale"] = np.array(sha(v8.to(torch.int8).numpy())), sv[..., 0, :].numpy()
    s_tok = (vf.abs().amax(-1, keepdim=True) / 127.0).clamp_min(1e-12)
    v8t = to_fmt(vf / s_tok, "int8")
    out[pre + "v8t_sha"], out[pre + "v_tok_scale"] = np.array(sha(v8t.to(torch.int8).numpy())), s_tok[..., 0].numpy()
    # NVFP4: Q minus its 512-block means, K minus its mean, V along keys in slot order
    nq = q.shape[-2]
    blocks = torch.nn.functional.pad(qf, (0, 0, 0, -nq % 512)).unflatten(-2, (-1, 512))
    sizes = torch.full((blocks.shape[-3],), 512.0)
    sizes[-1] = nq - 512 * (blocks.shape[-3] - 1)
    q_mean = blocks.sum(-2) / sizes[:, None]
    out[pre + "q_mean"] = q_mean.numpy()
    qc = qf - q_mean.repeat_interleave(512, -2)[..., :nq, :]
    kc = kf - k_mean[..., None, :]
    for tag, x, dim, outer in (("q4", qc, -1, None), ("k4", kc, -1, None), ("v4", slot_order(v), -2, "channel")):
        deq = block_scaled(x, "nvfp4", dim, outer)
        sf, o = nvfp4_pieces(x, dim, outer)
        out[pre + tag + "_deq_sha"] = np.array(sha(deq.numpy()))
        out[pre + tag + "_sf_sha"] = np.array(sha(sf))
        out[pre + tag + "_outer"] = o.squeeze()

    # ---- outputs of the contract configurations
    ref = reference(q, k, v)
    sel = slice(None) if rows is None else slice(0, None, max(1, nq // rows))
    out[pre + "ref"] = ref[..., sel, :].numpy()
    for tag, cfg in (("per_channel", TODAY), ("per_token", TODAY | dict(v_token="float")),
                     ("outliers", TODAY | dict(v_outliers=8)), ("fast", FAST),
                     ("fast_unsmoothed", {k_: v_ for k_, v_ in FAST.items() if k_ != "smooth_q"})):
        o = emulate(q, k, v, **cfg)
        out[pre + "out_" + tag] = bits(o[..., sel, :].bfloat16())
        out[pre + "err_" + tag] = np.array(errors(o, ref)["rel_l2"])
        print(f"{name:10} {tag:16} rel-L2 vs FP32 {errors(o, ref)['rel_l2']:.4%}")


def main():
    out: dict = {}
    # BASELINE config 1: the reference's own recipe (bench/emulate.py:447-449) on the CPU
    torch.manual_seed(0)
    q, k, v = (torch.randn((1, 4, 1024, 128), dtype=torch.bfloat16) for _ in range(3))
    case("cfg1", q, k, v, store_inputs=False, rows=64, out=out)
    # cross-attention with ragged sizes (tests/test_attention.py:36-43 has (1, 2, 300, 77)), channels of unequal size
    g = torch.Generator().manual_seed(1)
    q = (torch.randn((1, 2, 300, 128), generator=g) * (torch.rand(128, generator=g) * 4)).bfloat16()
    k = (torch.randn((1, 2, 77, 128), generator=g) * (torch.rand(128, generator=g) * 4) + 0.5).bfloat16()
    v = (torch.randn((1, 2, 77, 128), generator=g) * (torch.rand(128, generator=g) * 4)).bfloat16()
    case("ragged", q, k, v, store_inputs=True, rows=None, out=out)
    # V outlier tokens 65x and 250x the rest (README.md:46; tests/test_v_token.py:23-29), drifting Q mean (tests/test_fp4.py:93-99)
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn((1, 2, 640, 128), generator=g) for _ in range(3))
    q = q + 3 * torch.randn((2, 1, 128), generator=g) + 4 * torch.linspace(0, 1, 640)[:, None] * torch.randn((2, 1, 128), generator=g)
    v[0, 0, 1] *= 65
    v[0, 1, 2] *= 250
    case("outlier", q.bfloat16(), k.bfloat16(), v.bfloat16(), store_inputs=True, rows=128, out=out)
    # known-answer vectors of the e2m1 rounding (tests/test_emulate.py:28-32)
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    out["e2m1/ties_in"], out["e2m1/ties_out"] = ties.numpy(), to_e2m1(ties).numpy()
    out["e2m1/sat_in"], out["e2m1/sat_out"] = np.array([7.0, 1e6, -9.0], np.float32), to_e2m1(torch.tensor([7.0, 1e6, -9.0])).numpy()
    out["e2m1/grid"] = to_e2m1(grid).numpy()
    xs = torch.linspace(-8, 8, 4097)
    out["e2m1/sweep_in"], out["e2m1/sweep_out"] = xs.numpy(), to_e2m1(xs).numpy()
    # e4m3 rounding as torch does it, over the range the scales use
    xs = torch.cat([torch.linspace(0, 448, 8193), torch.logspace(-12, 2.6, 4096, base=2.0)]).clamp(max=448.0)
    out["e4m3/in"], out["e4m3/bytes"] = xs.numpy(), xs.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    out["slot_key"] = FP4_SLOT_KEY.numpy()
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, OUT.stat().st_size // 1024, "KB, torch", torch.__version__)


if __name__ == "__main__":
    main()
