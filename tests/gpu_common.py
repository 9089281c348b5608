"""Helpers of the GPU parity tests: seeded inputs (built on the CPU, then moved), and views for the oracle."""

import numpy as np
import torch

import oracle

# the reference's edge shapes (its tests/test_attention.py:36-43): (batch, heads, n_queries, n_keys)
EDGE_SHAPES = [(1, 1, 64, 64), (1, 2, 1000, 1000), (2, 3, 129, 129), (1, 2, 1, 1), (1, 2, 300, 77), (1, 4, 4096, 4096)]


def randn_bf16(shape, seed, channel_scale=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    if channel_scale:  # channels of unequal size, as the reference's quantizer tests use
        x = x * (torch.rand(shape[-1], generator=g) * 4)
    return x.bfloat16()


def qkv(batch, heads, nq, nk, seed=0, channel_scale=False):
    q = randn_bf16((batch, heads, nq, 128), 3 * seed, channel_scale)
    k = randn_bf16((batch, heads, nk, 128), 3 * seed + 1, channel_scale)
    v = randn_bf16((batch, heads, nk, 128), 3 * seed + 2, channel_scale)
    return q, k, v


def np_heads(x: torch.Tensor) -> np.ndarray:
    """A [batch, heads, n, ...] tensor as numpy [batch * heads, n, ...]."""
    x = x.detach().float().cpu() if x.dtype == torch.bfloat16 else x.detach().cpu()
    return x.reshape(-1, *x.shape[2:]).numpy()


def out_heads(out: torch.Tensor) -> np.ndarray:
    return out.detach().float().cpu().reshape(-1, out.shape[2], 128).numpy()


rel_l2 = oracle.rel_l2
