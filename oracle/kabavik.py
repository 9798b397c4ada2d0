"""Plain, slow restatement of the Kabavik decoder (test infrastructure only; the product never imports
it).  One function per mechanism, whole sequences at once, no cache, no batching: every position is
recomputed from the tokens, so a fault of the engine's pages, window edges, kept first tokens, shared
keys or portion handling cannot hide here.

Kabavik = layers over a residual stream x [T, width] with a norm on both sides of every sublayer:

    x <- x + m * Nb1(mixer(N1 x))      x <- x + m * Nb2(ff(N2 x))      x <- x + m * R(P (gelu(G x) * e_i)) * s

N = dynamic tanh, tanh(alpha v) * w + b (no statistics of the row); R(v) = v / sqrt(mean(v^2) + eps); e_i is
layer i's slice of a second embedding row of the token.  Mixers: `attention` (grouped-query, biases, RMS norm
over the whole query / key projection, half-split rotation of the leading dimensions with linearly scaled
frequencies, a sliding window that also keeps the first tokens, optionally the keys and values of an earlier
layer), `latent_attention` (keys and values from a normed latent plus one rotated key part shared by the heads,
interleaved rotation with YaRN-scaled frequencies, sliding window, a sigmoid gate per head), `attention_2`
(grouped-query, biases, per-head RMS norm of queries and keys, no rotation, a query temperature that grows with
the logarithm of the position, soft-capped scores, every earlier key).  Feed-forward: down(gelu(gate h) * up h).

`w` maps the checkpoint's tensor names to torch tensors, `cfg` is the parsed config.json; everything is
computed in `dtype`.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dynamic_tanh(x: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def base_frequencies(rot: dict) -> torch.Tensor:
    dims = int(rot["dims"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    return float(rot["base"]) ** (-2.0 * i / dims)


def linear_frequencies(rot: dict) -> torch.Tensor:
    """every frequency divided by the scaling factor (1 when no scaling is given)"""
    return base_frequencies(rot) / float((rot.get("scaling") or {}).get("factor", 1.0))


def yarn_frequencies(rot: dict):
    """frequencies blended between f and f / factor by a ramp over the pair index, and the factor by which
    sine and cosine grow"""
    f = base_frequencies(rot)
    sc = rot.get("scaling") or {}
    if "factor" not in sc:
        return f, 1.0
    dims, base, factor = int(rot["dims"]), float(rot["base"]), float(sc["factor"])
    if "original" not in sc:
        return f / factor, 1.0

    def at(turns):
        return dims * math.log(float(sc["original"]) / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(at(float(sc["fast"]))), 0)
    hi = min(math.ceil(at(float(sc["slow"]))), dims - 1)
    i = torch.arange(dims // 2, dtype=torch.float64)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def turn_half_split(x: torch.Tensor, freq: torch.Tensor, mag: float = 1.0) -> torch.Tensor:
    """x [T, heads, dim]: entry i is paired with entry i + n (n = len(freq)); entries from 2n on pass"""
    n = freq.numel()
    if n == 0:
        return x
    a = torch.arange(x.shape[0], dtype=torch.float64)[:, None] * freq[None, :]
    c, s = (torch.cos(a) * mag).to(x.dtype)[:, None, :], (torch.sin(a) * mag).to(x.dtype)[:, None, :]
    u, v = x[..., :n], x[..., n:2 * n]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * n:]], -1)


def turn_interleaved(x: torch.Tensor, freq: torch.Tensor, mag: float = 1.0) -> torch.Tensor:
    """x [T, heads, dim]: entry 2i is paired with entry 2i + 1; entries from 2 len(freq) on pass"""
    n = freq.numel()
    if n == 0:
        return x
    a = torch.arange(x.shape[0], dtype=torch.float64)[:, None] * freq[None, :]
    c, s = (torch.cos(a) * mag).to(x.dtype)[:, None, :], (torch.sin(a) * mag).to(x.dtype)[:, None, :]
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out = x.clone()
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return out


def visible(T: int, size: int = 0, keep_first: int = 0) -> torch.Tensor:
    """[T, T] bool: query i sees key j <= i when i - j < size or j < keep_first (size 0: every j <= i)"""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size > 0:
        ok = ok & ((i - j < size) | (j < keep_first))
    return ok


def softmax_attention(q, k, v, mask, scale, softcap=0.0):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; query head h reads key/value head h // (H / G)"""
    H, G = q.shape[1], k.shape[1]
    rep = H // G
    k = k.repeat_interleave(rep, 1)
    v = v.repeat_interleave(rep, 1)
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    if softcap > 0.0:
        s = softcap * torch.tanh(s / softcap)
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, -1)
    return torch.einsum("hij,jhd->ihd", p, v)


def _lin(h, w, name):
    y = h @ w[name].T
    return y + w[name + ".b"] if name + ".b" in w else y


def attention_keys(h, w, pre, mx, eps):
    """the keys (normed over the whole projection, turned) and values a layer of kind `attention` makes"""
    G, D, Dv = int(mx.get("kv_heads", mx["heads"])), int(mx["dim"]), int(mx.get("vdim", mx["dim"]))
    T = h.shape[0]
    k = rms(_lin(h, w, pre + "k"), eps) * w[pre + "k.norm"]
    v = _lin(h, w, pre + "v")
    rot = mx.get("rot")
    k = k.view(T, G, D)
    if rot:
        k = turn_half_split(k, linear_frequencies(rot))
    return k, v.view(T, G, Dv)


def attention(h, w, pre, mx, eps, shared=None):
    """`shared`: (keys, values) of the layer named by kv_from"""
    H, D = int(mx["heads"]), int(mx["dim"])
    T = h.shape[0]
    q = (rms(_lin(h, w, pre + "q"), eps) * w[pre + "q.norm"]).view(T, H, D)
    rot = mx.get("rot")
    if rot:
        q = turn_half_split(q, linear_frequencies(rot))
    k, v = shared if shared is not None else attention_keys(h, w, pre, mx, eps)
    mk = mx.get("mask") or {}
    o = softmax_attention(q, k, v, visible(T, int(mk.get("size") or 0), int(mk.get("keep_first") or 0)), float(mx["scale"]))
    return _lin(o.reshape(T, -1), w, pre + "o")


def attention_2(h, w, pre, mx, eps):
    H, G, D = int(mx["heads"]), int(mx.get("kv_heads", mx["heads"])), int(mx["dim"])
    Dv = int(mx.get("vdim", D))
    T = h.shape[0]
    q = rms(_lin(h, w, pre + "q").view(T, H, D), eps) * w[pre + "q.norm"]
    k = rms(_lin(h, w, pre + "k").view(T, G, D), eps) * w[pre + "k.norm"]
    v = _lin(h, w, pre + "v").view(T, G, Dv)
    qt = mx.get("q_temp")
    if qt:
        p = torch.arange(T, dtype=torch.float64)
        temp = 1.0 + float(qt["coef"]) * torch.log(torch.floor((p + 1.0) / float(qt["every"])) + 1.0)
        q = q * temp.to(q.dtype)[:, None, None]
    mk = mx.get("mask") or {}
    o = softmax_attention(q, k, v, visible(T, int(mk.get("size") or 0), int(mk.get("keep_first") or 0)), float(mx["scale"]),
                          float(mx.get("softcap") or 0.0))
    return _lin(o.reshape(T, -1), w, pre + "o")


def latent_attention(h, w, pre, mx, eps):
    H, D, P, Dv, R = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"]), int(mx["kv_rank"])
    T = h.shape[0]
    q = _lin(h, w, pre + "q").view(T, H, D + P)
    ckr = _lin(h, w, pre + "dkv")
    c = rms(ckr[:, :R], eps) * w[pre + "dkv.norm"]
    kr = ckr[:, R:].view(T, 1, P)
    rot = mx.get("rot")
    qr = q[..., D:]
    if rot:
        f, mag = yarn_frequencies(rot)
        qr, kr = turn_interleaved(qr, f, mag), turn_interleaved(kr, f, mag)
    ku = (c @ w[pre + "uk"].T).view(T, H, D)
    v = (c @ w[pre + "uv"].T).view(T, H, Dv)
    qq = torch.cat([q[..., :D], qr], -1)
    kk = torch.cat([ku, kr.expand(T, H, P)], -1)
    mk = mx.get("mask") or {}
    o = softmax_attention(qq, kk, v, visible(T, int(mk.get("size") or 0)), float(mx["scale"]))
    if pre + "g" in w:
        o = o * torch.sigmoid(_lin(h, w, pre + "g"))[:, :, None]
    return _lin(o.reshape(T, -1), w, pre + "o")


def feed_forward(h, w, pre, ml):
    if ml["kind"] != "dense":
        raise ValueError(f"unknown feed-forward kind {ml['kind']!r}")
    return (gelu_tanh(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def token_side(x, e, w, pre, eps):
    """e: the layer's slice of the tokens' second embedding rows"""
    y = (gelu_tanh(x @ w[pre + "gate"].T) * e) @ w[pre + "proj"].T
    return rms(y, eps) * w[pre + "norm"]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """logits [T, vocab]; `layers_out` receives the residual stream after every layer"""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float((cfg.get("norm") or {}).get("eps", 1e-6))
    m = float(cfg.get("residual_mult", 1.0))
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][ids] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    sd = int((cfg.get("token_side") or {}).get("dim") or 0)
    kept = {}
    for i, lc in enumerate(cfg["layers"]):
        p, mx, kind = f"l{i}.", lc["mixer"], lc["type"]
        h = dynamic_tanh(x, w, p + "norm1")
        if kind == "attention":
            src = mx.get("kv_from")
            if src is None:
                kept[i] = attention_keys(h, w, p + "mix.", mx, eps)
            y = attention(h, w, p + "mix.", mx, eps, kept[i if src is None else int(src)])
        elif kind == "attention_2":
            y = attention_2(h, w, p + "mix.", mx, eps)
        elif kind == "latent_attention":
            y = latent_attention(h, w, p + "mix.", mx, eps)
        else:
            raise ValueError(f"layer {i}: unknown layer type {kind!r}")
        x = x + m * dynamic_tanh(y, w, p + "norm1b")
        if lc.get("mlp"):
            x = x + m * dynamic_tanh(feed_forward(dynamic_tanh(x, w, p + "norm2"), w, p + "mlp.", lc["mlp"]), w, p + "norm2b")
        if sd:
            x = x + m * token_side(x, w["side.embed"][ids][:, i * sd:(i + 1) * sd], w, p + "side.", eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return (dynamic_tanh(x, w, "final.norm") @ w["head"].T) * float(cfg.get("logit_scale", 1.0))


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
