"""Shared helpers of the Kabavik tests: small configurations whose sizes differ from one another (key heads fewer
than heads or as many, value size unlike key size, rotation over part of a head or all of it or none, windows that
are neither a page nor a tile, kept first keys fewer and more than a window or a tile, borrowed keys under another
mask, layers without feed-forward, models without the per-layer token input), random checkpoints, error measures."""
import numpy as np
import torch

from llmq_b200.kabavik import KabavikLayer, KabavikSpec, random_checkpoint

DENSE = dict(ff="dense", ff_dim=72)


def attn(heads=6, kv_heads=2, dim=24, vdim=40, window=21, keep_first=3, rot_dims=12, rot_base=500.0, rot_factor=2.0,
         scale=0.3, kv_from=-1, **ff):
    return KabavikLayer(kind="attention", heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, window=window,
                        keep_first=keep_first, rot_dims=rot_dims, rot_base=rot_base if rot_dims else 10000.0,
                        rot_factor=rot_factor if rot_dims else 0.0, scale=scale, kv_from=kv_from, **ff)


def attn2(heads=4, kv_heads=2, dim=20, vdim=12, scale=0.25, softcap=4.0, coef=0.4, every=7, **ff):
    return KabavikLayer(kind="attention_2", heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale,
                        softcap=softcap, q_temp_coef=coef if every else 0.0, q_temp_every=every, **ff)


def latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, window=19, rot_base=100.0, factor=3.0, original=64.0,
           fast=8.0, slow=1.0, scale=0.2, **ff):
    return KabavikLayer(kind="latent_attention", heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank,
                        window=window, rot_dims=rot_dim, rot_base=rot_base, rot_factor=factor, rot_original=original,
                        rot_fast=fast if original else 0.0, rot_slow=slow if original else 0.0, scale=scale, **ff)


def small_spec(width=96, vocab=211, layers=None, eps=1e-5, mult=0.6, embed_scale=3.0, logit_scale=1.7, side_dim=10):
    layers = layers or [
        attn(**DENSE),                                                # window 21, three kept keys
        latent(**DENSE),
        attn2(**DENSE),
        attn(window=9, keep_first=0, kv_from=0),                      # layer 0's keys under another mask, no feed-forward
        latent(heads=2, dim=24, rot_dim=4, vdim=8, kv_rank=24, window=0, factor=0.0, original=0.0, **DENSE),
        attn(heads=3, kv_heads=3, dim=16, vdim=16, window=33, keep_first=40, rot_dims=16, rot_factor=0.0, **DENSE),
        attn(window=5, keep_first=1, kv_from=0, **DENSE),             # a second reader of layer 0's keys
    ]
    return KabavikSpec(width=width, vocab=vocab, layers=layers, rms_eps=eps, residual_mult=mult,
                       embed_scale=embed_scale, logit_scale=logit_scale, side_dim=side_dim)


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
