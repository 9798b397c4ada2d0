"""Shared helpers of the Paluzen tests: small configurations whose sizes differ from one another (key heads
fewer than heads, value size unlike key size, rotation over part of a head or all of it or none, windows
that are neither a page nor a tile, several heads per key head, routed layers with and without groups and
identity experts, a layer without feed-forward, layers that repeat), random checkpoints, error measures."""
import numpy as np
import torch

from llmq_b200.paluzen import PaluzenLayer, PaluzenSpec, random_checkpoint

MOE = dict(ff="moe", ff_dim=40, n_experts=6, n_identity=2, top_k=2, n_groups=4, keep_groups=2)
MOE_ALL = dict(ff="moe", ff_dim=24, n_experts=3, n_identity=0, top_k=3, n_groups=1, keep_groups=1)
MOE_ONE = dict(ff="moe", ff_dim=56, n_experts=5, n_identity=1, top_k=1, n_groups=3, keep_groups=1)
DENSE = dict(ff="dense", ff_dim=120)


def lightning(heads=3, dim=16, vdim=24, decay=None, **ff):
    decay = decay or tuple(0.5 + 0.499 * h / max(heads - 1, 1) for h in range(heads))
    return PaluzenLayer(kind="lightning", heads=heads, dim=dim, vdim=vdim, decay=tuple(decay), **ff)


def parallel(heads=6, kv_heads=2, dim=24, vdim=40, window=21, rot_dims=12, rot_base=500.0, scale=0.3, left_scale=1.3,
             r_heads=3, r_dim=16, r_rank=5, right_scale=0.7, **ff):
    return PaluzenLayer(kind="parallel", heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, window=window,
                        rot_dims=rot_dims, rot_base=rot_base if rot_dims else 10000.0, scale=scale, left_scale=left_scale, r_heads=r_heads,
                        r_dim=r_dim, r_rank=r_rank, right_scale=right_scale, **ff)


def small_spec(width=96, vocab=211, layers=None, loop=(1, 3, 3), eps=1e-5, softcap=20.0):
    layers = layers or [
        lightning(**DENSE),
        parallel(**MOE),                                             # window 21: neither a page nor a tile
        lightning(heads=2, dim=40, vdim=8, **MOE_ONE),
        parallel(heads=3, kv_heads=3, dim=40, vdim=40, window=0, rot_dims=40, scale=0.15, r_heads=2, r_dim=40,
                 r_rank=3),                                          # every earlier key, whole head turned, no feed-forward
        parallel(heads=4, kv_heads=1, dim=16, vdim=8, window=33, rot_dims=0, r_heads=5, r_dim=8, r_rank=9, **MOE_ALL),
    ]
    return PaluzenSpec(width=width, vocab=vocab, base_layers=layers, loop=loop, rms_eps=eps, logit_softcap=softcap)


def checkpoint(spec, seed=0):
    """random bf16-representable weights (so the fp32 engine and the fp64 oracle read the same numbers)"""
    return random_checkpoint(spec, seed=seed, device="cpu")


def rel_err(got, want):
    """rms of the difference over the rms of the expected rows, worst row"""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    num = np.sqrt(((got - want) ** 2).mean(-1))
    den = np.sqrt((want ** 2).mean(-1)) + 1e-30
    return float((num / den).max())


def tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
