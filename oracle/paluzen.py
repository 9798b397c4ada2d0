"""Plain, slow restatement of the Paluzen decoder (test infrastructure only; the product never imports
it).  One function per mechanism, whole sequences at once, no cache, no state slots, no batching: every
position is recomputed from the tokens, so a fault of the engine's pages, slots, window edges or portion
handling cannot hide here.

Paluzen = sequential pre-norm layers over a residual stream x [T, width]:

    x <- x + mixer(token_shift(N(x) * norm1))        x <- x + ff(N(x) * norm2)

N(v) = v / sqrt(mean(v^2) + eps).  A range of layers may repeat with the same weights; each pass starts with
x <- W_in [x ; x0], x0 the embedding rows.  The logits are taken against the embedding table and soft-capped.

`w` maps the checkpoint's tensor names to torch tensors (any float dtype; everything is computed in the
dtype of `dtype`), `cfg` is the parsed config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def previous(h: torch.Tensor) -> torch.Tensor:
    """row t holds row t-1 of h; row 0 holds zeros"""
    return torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)


def token_shift(h: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return h + (previous(h) - h) * weight


def rotate_half_split(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, dim]: entry i < dims/2 of a head is paired with entry i + dims/2 and the pair is turned by
    the angle t * base^(-2i/dims); entries from dims on pass"""
    if dims == 0:
        return x
    T, half = x.shape[0], dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * f[None]
    c, s = torch.cos(ang).to(x.dtype)[:, None], torch.sin(ang).to(x.dtype)[:, None]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mx: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, D = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"]
    V = mx.get("vdim", D)
    rot = mx.get("rot") or {}
    q = rotate_half_split((h @ w[pre + "q"].T).view(T, H, D), int(rot.get("dims") or 0), float(rot.get("base", 1e4)))
    k = rotate_half_split((h @ w[pre + "k"].T).view(T, G, D), int(rot.get("dims") or 0), float(rot.get("base", 1e4)))
    v = (h @ w[pre + "v"].T).view(T, G, V)
    size = int((mx.get("mask") or {}).get("size") or 0)
    gate = torch.sigmoid(h @ w[pre + "g"].T)          # [T, H]
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        for i in range(T):
            lo = max(0, i - size + 1) if size else 0
            s = (k[lo:i + 1, g] @ q[i, hh]) * mx["scale"] * w[pre + "temp"][hh]
            out[i, hh] = torch.softmax(s, 0) @ v[lo:i + 1, g] * gate[i, hh]
    return out.reshape(T, H * V) @ w[pre + "o"].T


def decay_mix(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mx: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D = mx["heads"], mx["dim"]
    hp = previous(h)
    blend = {s: h + (hp - h) * w[pre + "mu." + s] for s in "rkvgw"}
    r = (blend["r"] @ w[pre + "r"].T).view(T, H, D)
    k = (blend["k"] @ w[pre + "k"].T).view(T, H, D)
    v = (blend["v"] @ w[pre + "v"].T).view(T, H, D)
    gate = F.silu(blend["g"] @ w[pre + "g"].T)
    dec = torch.exp(-torch.exp(torch.tanh(blend["w"] @ w[pre + "w1"].T) @ w[pre + "w2"].T + w[pre + "w0"])).view(T, H, D)
    u = w[pre + "u"].reshape(H, D)
    S = torch.zeros(H, D, D, dtype=h.dtype)
    out = torch.zeros(T, H, D, dtype=h.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = ((S + u[:, :, None] * kv) * r[t][:, :, None]).sum(1)
        S = dec[t][:, :, None] * S + kv
    return (rms(out, eps).reshape(T, H * D) * w[pre + "norm"] * gate) @ w[pre + "o"].T


def lightning(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mx: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D = mx["heads"], mx["dim"]
    V = mx.get("vdim", D)
    q = F.silu(h @ w[pre + "q"].T).view(T, H, D)
    k = F.silu(h @ w[pre + "k"].T).view(T, H, D)
    v = F.silu(h @ w[pre + "v"].T).view(T, H, V)
    lam = torch.tensor(mx["decay"], dtype=h.dtype)
    S = torch.zeros(H, D, V, dtype=h.dtype)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        S = lam[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = (S * q[t][:, :, None]).sum(1)
    o = rms(out.reshape(T, H * V), eps) * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.relu(z) ** 2


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, r: dict):
    """-> (chosen expert indices [T, top], their weights [T, top])"""
    total = r["experts"] + int(r.get("identity") or 0)
    g = r.get("groups") or {}
    count, keep = int(g.get("count") or 1), int(g.get("keep") or g.get("count") or 1)
    s = torch.softmax(h @ w[pre + "router"].T, -1)
    choice = s + w[pre + "correction"]
    T = h.shape[0]
    idx = torch.zeros(T, r["top"], dtype=torch.long)
    wt = torch.zeros(T, r["top"], dtype=h.dtype)
    per = total // count
    for t in range(T):
        best = sorted(range(count), key=lambda c: (-float(choice[t, c * per:(c + 1) * per].max()), c))[:keep]
        allowed = [e for e in range(total) if e // per in best]
        pick = sorted(allowed, key=lambda e: (-float(choice[t, e]), e))[:r["top"]]
        idx[t] = torch.tensor(pick)
        wt[t] = s[t, pick] / (s[t, pick].sum() + 1e-20)
    return idx, wt


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, ml: dict) -> torch.Tensor:
    if ml["kind"] == "dense":
        return relu_squared(h @ w[pre + "up"].T) @ w[pre + "down"].T
    r = ml["router"]
    idx, wt = route(h, w, pre, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            y = h[t] if e >= r["experts"] else relu_squared(h[t] @ w[f"{pre}e{e}.up"].T) @ w[f"{pre}e{e}.down"].T
            out[t] += wt[t, j] * y
    return out


def layer_runs(cfg: dict) -> List[tuple]:
    """(checkpoint layer, a pass begins here) for every layer run in order"""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(lp["start"])]
    for _ in range(lp.get("times", 1)):
        runs += [(i, i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, False) for i in range(lp["stop"], n)]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """logits [T, vocab] of every position; layers_out receives the residual stream after every layer run"""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)]
    x0 = x.clone()
    for i, begins in layer_runs(cfg):
        lc, p = cfg["layers"][i], f"l{i}."
        if begins:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T
        h = token_shift(rms(x, eps) * w[p + "norm1"], w[p + "shift"])
        mx = lc["mixer"]
        if lc["type"] == "lightning":
            x = x + lightning(h, w, p + "mix.", mx, eps)
        else:
            x = x + mx.get("left_scale", 1.0) * window_attention(h, w, p + "mix.left.", mx["left"]) \
                  + mx.get("right_scale", 1.0) * decay_mix(h, w, p + "mix.right.", mx["right"], eps)
        if lc.get("mlp"):
            x = x + feed_forward(rms(x, eps) * w[p + "norm2"], w, p + "mlp.", lc["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = (rms(x, eps) * w["final.norm"]) @ w["embed"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    out = list(prompt)
    for _ in range(n_new):
        out.append(int(forward(cfg, w, out)[-1].argmax()))
    return out[len(prompt):]
