"""Generates tests/golden/golden_rope.npz: the reference's emulator (bench/emulate.py) on inputs rotated by its rope(),
the case of the reference's tests/test_rope.py (a WAN latent of 3 x 7 x 9 = 189 tokens, past a tile edge and a
statistics block), on CPU tensors.

    python tests/golden/make_golden_rope.py /path/to/reference

Holds the inputs (bf16 bits), the emulator's own table (to pin the restated table builder), the rotated statistics,
the quantizer pieces of the rotated tensors and the emulator's outputs for the accurate and fast contracts.
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
from emulate import TODAY, block_scaled, emulate, errors, quant, reference, rope, wan_rope_table  # noqa: E402

FAST = TODAY | dict(p_fmt="nvfp4", v_fmt="nvfp4", p_local=False, p_mul=1024.0, p_outer=1.0, v_outer="channel",
                    fp4_slots=True, qk="nvfp4")
OUT = Path(__file__).resolve().parent / "golden_rope.npz"
T, H, W, HEADS = 3, 7, 9, 3


def bits(x: torch.Tensor) -> np.ndarray:
    return x.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    out: dict = {}
    torch.manual_seed(0)
    shape = (1, T * H * W, HEADS, 128)  # ComfyUI's layout, read through a transpose (tests/test_rope.py:31-35)
    q, k, v = (torch.randn(shape).bfloat16().transpose(1, 2).contiguous() for _ in range(3))
    q = (q.float() + 2 * torch.randn(HEADS, 1, 128)).bfloat16()  # a Q mean for the smoothing to take out (test_rope.py:88)
    table = wan_rope_table(T, H, W, device="cpu")
    out["q"], out["k"], out["v"], out["table"] = bits(q), bits(k), bits(v), table.numpy()
    q_rot, k_rot = rope(q.float(), table), rope(k.float(), table)
    out["q_rot_sha"], out["k_rot_sha"] = np.array(sha(q_rot.numpy())), np.array(sha(k_rot.numpy()))
    out["k_low"], out["k_high"], out["k_mean"] = k_rot.amin(-2).numpy(), k_rot.amax(-2).numpy(), k_rot.mean(-2).numpy()
    k_mean = k_rot.mean(-2)
    k8, sk = quant(k_rot - k_mean[..., None, :], "int8", 64)
    q8, sq = quant(q_rot, "int8", 128)
    out["k8_sha"], out["k_scale"] = np.array(sha(k8.to(torch.int8).numpy())), sk[..., ::64, 0].numpy()
    out["q8_sha"], out["q_scale"] = np.array(sha(q8.to(torch.int8).numpy())), sq[..., ::128, 0].numpy()
    out["q4_deq_sha"] = np.array(sha(block_scaled(q_rot, "nvfp4", -1).numpy()))
    ref = reference(q_rot, k_rot, v)
    out["ref"] = ref.numpy()
    for tag, cfg in (("per_channel", TODAY), ("per_token", TODAY | dict(v_token="float")), ("fast", FAST | dict(smooth_q=256)),
                     ("fast_unsmoothed", FAST)):
        o = emulate(q_rot, k_rot, v, **cfg)
        out["out_" + tag] = bits(o.bfloat16())
        out["err_" + tag] = np.array(errors(o, ref)["rel_l2"])
        print(f"rope {tag:16} rel-L2 vs FP32 {errors(o, ref)['rel_l2']:.4%}")
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, OUT.stat().st_size // 1024, "KB, torch", torch.__version__)


if __name__ == "__main__":
    main()
