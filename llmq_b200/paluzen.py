"""Host side of the Paluzen decoder: reading its config.json, mapping its checkpoint to the engine's
layered-model weights, and drawing random checkpoints for tests and benchmarks.

Paluzen is a stack of sequential pre-norm layers over an fp32 residual stream,

    x <- x + mixer(shift(norm1 x))        x <- x + ff(norm2 x)

with plain RMS norms.  `shift` blends every channel of the mixer's input with the previous token's normed
row (a per-channel weight; the previous row travels with the sequence).  Mixers: `lightning`, a linear
attention with a constant decay per head (SiLU on q, k, v, one RMS norm over the concatenated heads, a
sigmoid gate), and `parallel`, two mixers side by side whose outputs are summed with fixed scales —
a rotary grouped-query attention over a sliding window (half-split rotation of the leading dimensions, a
score temperature per head, one sigmoid gate number per head) and a time mixing with a data-dependent decay
per key channel (five blends of the input with its predecessor, a low-rank decay path, a bonus for the
current token, per-head RMS, SiLU gate).  Feed-forwards: squared-ReLU dense, or a top-k mixture of
squared-ReLU experts routed by softmax scores with a choice correction, group-limited choice and identity
experts.  A range of layers may run several times in a row with the same weights; every pass has its own
cache and state, and begins by re-injecting the embedding output (x <- W_in [x; x0]).  The output matrix is
the embedding table; logits are soft-capped.

The engine sees one layer per layer RUN: a repeated layer is listed once per pass, bound to the same device
tensors, with its own cache region and state.  Every size comes from config.json or a tensor's shape.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from . import lib as L
from .ramopel import checkpoint_shapes, load_checkpoint, save_checkpoint  # noqa: F401  (one file format)

ARCHITECTURE = "Paluzen"


@dataclass
class PaluzenLayer:
    kind: str                        # "lightning" | "parallel"
    # lightning: heads x (dim, dim, vdim) and one decay per head
    heads: int = 0
    dim: int = 0
    vdim: int = 0
    decay: Tuple[float, ...] = ()
    # parallel, left: sliding-window attention
    kv_heads: int = 0
    window: int = 0                  # 0 = every earlier key
    rot_dims: int = 0                # 0 = no rotation
    rot_base: float = 10000.0
    scale: float = 1.0
    left_scale: float = 1.0
    # parallel, right: decay mix (values as wide as keys)
    r_heads: int = 0
    r_dim: int = 0
    r_rank: int = 0                  # inner size of the decay path (from the tensor's shape)
    right_scale: float = 1.0
    # feed-forward
    ff: Optional[str] = None         # None | "dense" | "moe"
    ff_dim: int = 0
    n_experts: int = 0               # real experts
    n_identity: int = 0
    top_k: int = 0
    n_groups: int = 1
    keep_groups: int = 1
    # place in the stack
    src: int = 0                     # checkpoint layer whose tensors this run uses
    inject: bool = False             # a pass begins here: x <- W_in [x; x0]

    def desc(self) -> L.LayerDesc:
        ff = {None: L.FF_NONE, "dense": L.FF_RELU2, "moe": L.FF_MOE_GROUPED}[self.ff]
        common = dict(ff=ff, ff_dim=self.ff_dim, n_experts=self.n_experts, n_identity=self.n_identity,
                      top_k=self.top_k, n_groups=self.n_groups, keep_groups=self.keep_groups,
                      inject=int(self.inject), kv_from=-1)
        if self.kind == "lightning":
            return L.LayerDesc(mixer=L.MIXER_LIGHTNING, heads=self.heads, kv_heads=self.heads, dim=self.dim,
                               vdim=self.vdim, mix_scale=1.0, **common)
        return L.LayerDesc(mixer=L.MIXER_WINDOW_ATTN, heads=self.heads, kv_heads=self.kv_heads, dim=self.dim,
                           vdim=self.vdim, window=self.window, rot_dims=self.rot_dims, rot_base=self.rot_base,
                           attn_scale=self.scale, mix_scale=self.left_scale, side_mixer=L.MIXER_DECAY_MIX,
                           side_heads=self.r_heads, side_dim=self.r_dim, side_vdim=self.r_dim,
                           side_decay_rank=self.r_rank, side_scale=self.right_scale, **common)


def _layer_from_config(i: int, lc: dict, shapes) -> PaluzenLayer:
    mx, kind = lc["mixer"], lc["type"]
    if kind == "lightning":
        ly = PaluzenLayer(kind=kind, heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])),
                          decay=tuple(float(v) for v in mx["decay"]))
        if len(ly.decay) != ly.heads:
            raise ValueError(f"layer {i}: {len(ly.decay)} decays for {ly.heads} heads")
    elif kind == "parallel":
        le, ri = mx["left"], mx["right"]
        rot = le.get("rot") or {}
        rk = int(ri.get("rank", 0))
        if shapes is not None and f"l{i}.mix.right.w1" in shapes:
            rk = int(shapes[f"l{i}.mix.right.w1"][0])
        if rk <= 0:
            raise ValueError(f"layer {i}: the decay path's inner size comes from the tensor l{i}.mix.right.w1 "
                             "(or a 'rank' entry)")
        ly = PaluzenLayer(kind=kind, heads=int(le["heads"]), kv_heads=int(le.get("kv_heads", le["heads"])),
                          dim=int(le["dim"]), vdim=int(le.get("vdim", le["dim"])),
                          window=int((le.get("mask") or {}).get("size") or 0), rot_dims=int(rot.get("dims") or 0),
                          rot_base=float(rot.get("base", 10000.0)), scale=float(le["scale"]),
                          left_scale=float(mx.get("left_scale", 1.0)), r_heads=int(ri["heads"]), r_dim=int(ri["dim"]),
                          r_rank=rk, right_scale=float(mx.get("right_scale", 1.0)))
        if ly.heads % ly.kv_heads:
            raise ValueError(f"layer {i}: kv_heads ({ly.kv_heads}) must divide heads ({ly.heads})")
        if ly.rot_dims % 2 or ly.rot_dims > ly.dim:
            raise ValueError(f"layer {i}: rot.dims ({ly.rot_dims}) must be even and at most dim ({ly.dim})")
    else:
        raise ValueError(f"layer {i}: unknown layer type {kind!r}")
    ml = lc.get("mlp")
    if ml:
        if ml["kind"] == "dense":
            ly.ff, ly.ff_dim = "dense", int(ml["ff"])
        elif ml["kind"] == "moe":
            r = ml["router"]
            g = r.get("groups") or {}
            ly.ff, ly.ff_dim = "moe", int(ml["expert"]["ff"])
            ly.n_experts, ly.n_identity, ly.top_k = int(r["experts"]), int(r.get("identity") or 0), int(r["top"])
            ly.n_groups, ly.keep_groups = int(g.get("count") or 1), int(g.get("keep") or g.get("count") or 1)
            tot = ly.n_experts + ly.n_identity
            if tot % ly.n_groups or ly.keep_groups > ly.n_groups or ly.top_k > ly.keep_groups * (tot // ly.n_groups):
                raise ValueError(f"layer {i}: {ly.n_groups} groups must divide {tot} experts, keep at most that many, "
                                 f"and the kept groups must hold top = {ly.top_k} experts")
        else:
            raise ValueError(f"layer {i}: unknown feed-forward kind {ml['kind']!r}")
    return ly


@dataclass
class PaluzenSpec:
    """What `NativeModel` needs to know about a Paluzen checkpoint (the counterpart of `ModelSpec`).
    `layers` lists the layer RUNS in the order they execute; `base_layers` the checkpoint's layers."""
    width: int
    vocab: int
    base_layers: List[PaluzenLayer]
    loop: Optional[Tuple[int, int, int]] = None      # (start, stop, times): layers start..stop-1 run `times` times
    rms_eps: float = 1e-5
    logit_softcap: float = 0.0
    name: str = "paluzen"
    max_position_embeddings: int = 1 << 20   # positions are computed, not tabulated: the pool is the limit
    eos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    arch: str = "paluzen"
    layered: bool = field(default=True, repr=False)
    layers: List[PaluzenLayer] = field(default_factory=list, repr=False)

    def __post_init__(self):
        n = len(self.base_layers)
        for i, ly in enumerate(self.base_layers):
            ly.src, ly.inject = i, False
        if self.loop is None:
            self.layers = list(self.base_layers)
            return
        start, stop, times = self.loop
        if not (0 <= start < stop <= n and times >= 1):
            raise ValueError(f"loop {self.loop}: need 0 <= start < stop <= {n} layers and times >= 1")
        runs = list(self.base_layers[:start])
        for _ in range(times):
            for i in range(start, stop):
                runs.append(replace(self.base_layers[i], inject=(i == start)))
        self.layers = runs + list(self.base_layers[stop:])

    @property
    def hidden(self) -> int:
        return self.width

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    def config_extras(self) -> dict:
        """the fields of b200q_model_config that describe this design's layer form"""
        return dict(arch=L.ARCH_PALUZEN, layer_form=L.FORM_PRENORM, token_shift=1, logit_softcap=self.logit_softcap,
                    embed_scale=0.0)

    @staticmethod
    def from_config(cfg: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None,
                    name: str = "paluzen") -> "PaluzenSpec":
        """cfg: the parsed config.json; shapes: tensor name -> shape of the checkpoint, for the size that only
        a tensor gives (the inner size of the decay path)."""
        if cfg.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} config: architecture={cfg.get('architecture')!r}")
        layers = [_layer_from_config(i, lc, shapes) for i, lc in enumerate(cfg["layers"])]
        lp = cfg.get("loop")
        loop = (int(lp["start"]), int(lp["stop"]), int(lp.get("times", 1))) if lp else None
        return PaluzenSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), base_layers=layers, loop=loop,
                           rms_eps=float((cfg.get("norm") or {}).get("eps", 1e-5)),
                           logit_softcap=float(cfg.get("logit_softcap") or 0.0), name=name)

    def to_config(self) -> dict:
        out = []
        for ly in self.base_layers:
            if ly.kind == "lightning":
                mx = {"heads": ly.heads, "dim": ly.dim, "vdim": ly.vdim, "decay": list(ly.decay)}
            else:
                left = {"heads": ly.heads, "kv_heads": ly.kv_heads, "dim": ly.dim, "vdim": ly.vdim, "scale": ly.scale}
                if ly.window:
                    left["mask"] = {"size": ly.window}
                if ly.rot_dims:
                    left["rot"] = {"dims": ly.rot_dims, "base": ly.rot_base}
                mx = {"left": left, "right": {"heads": ly.r_heads, "dim": ly.r_dim, "rank": ly.r_rank},
                      "left_scale": ly.left_scale, "right_scale": ly.right_scale}
            ml = None
            if ly.ff == "dense":
                ml = {"kind": "dense", "ff": ly.ff_dim}
            elif ly.ff == "moe":
                ml = {"kind": "moe", "expert": {"ff": ly.ff_dim},
                      "router": {"experts": ly.n_experts, "identity": ly.n_identity, "top": ly.top_k,
                                 "groups": {"count": ly.n_groups, "keep": ly.keep_groups}}}
            out.append({"type": ly.kind, "mixer": mx, "mlp": ml})
        cfg = {"architecture": ARCHITECTURE, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.rms_eps},
               "logit_softcap": self.logit_softcap, "layers": out}
        if self.loop is not None:
            cfg["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return cfg

    def engine_weights(self, sd: Dict[str, torch.Tensor]) -> Iterable[Tuple[str, torch.Tensor]]:
        return engine_weights(self, sd)

    def random_checkpoint(self, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
        return random_checkpoint(self, seed, device)

    def weight_bytes_per_token(self, esize: int = 2, batch: int = 1) -> int:
        """matrix bytes one decode step of `batch` tokens touches (a repeated layer is read once per pass; a routed
        layer reads at most min(experts, batch * top_k) of its experts; embedding rows are read by row, the
        output matrix in full)"""
        W, n = self.width, self.vocab * self.width
        for ly in self.layers:
            if ly.inject:
                n += 2 * W * W
            if ly.kind == "lightning":
                n += W * (2 * ly.heads * ly.dim + 2 * ly.heads * ly.vdim) + W * ly.heads * ly.vdim
            else:
                hd, hv = ly.heads * ly.dim, ly.heads * ly.vdim
                n += W * (hd + ly.kv_heads * (ly.dim + ly.vdim) + ly.heads) + W * hv
                rd = ly.r_heads * ly.r_dim
                n += W * (4 * rd + ly.r_rank) + rd * ly.r_rank + W * rd
            if ly.ff == "dense":
                n += 2 * W * ly.ff_dim
            elif ly.ff == "moe":
                n += W * (ly.n_experts + ly.n_identity) + 2 * W * ly.ff_dim * min(ly.n_experts, batch * ly.top_k)
        return n * esize


# ---- checkpoint names -> engine names --------------------------------------------------------------
def _pad_rows(t: torch.Tensor, mult: int = 64) -> torch.Tensor:
    pad = -t.shape[0] % mult
    return torch.cat([t, t.new_zeros(pad, t.shape[1])], 0) if pad else t


def engine_weights(spec: PaluzenSpec, sd: Dict[str, torch.Tensor]) -> Iterable[Tuple[str, torch.Tensor]]:
    """Checkpoint tensors -> the layered engine's weights, one set of names per layer RUN.  2-D results are
    matrices (bound in the model's dtype); 1-D results are vectors and constants (bound as fp32 rows).  Runs of
    the same checkpoint layer yield the SAME tensor objects, which the model uploads once.  Fusions: the
    projections of a mixer that read the same input become one matrix (lightning: q, k, v, gate; window
    attention: q, k, v and the per-head gate rows, padded with zero rows to a multiple of 64; decay mix:
    r, k, v, gate stacked, each reading its own blend), the five blend weights become one row, the experts'
    matrices are stacked.  The output matrix is the embedding table."""
    yield "embed", sd["embed"]
    yield "final_norm", sd["final.norm"]
    yield "lm_head", sd["embed"]
    made: Dict[int, List[Tuple[str, torch.Tensor]]] = {}
    for run, ly in enumerate(spec.layers):
        if ly.src not in made:
            made[ly.src] = list(_layer_weights(spec, ly, sd))
        o = f"layers.{run}."
        if ly.inject:
            yield o + "inject", sd["loop.in"]
        for name, t in made[ly.src]:
            yield o + name, t


def _layer_weights(spec: PaluzenSpec, ly: PaluzenLayer, sd) -> Iterable[Tuple[str, torch.Tensor]]:
    p = f"l{ly.src}."
    yield "norm1", sd[p + "norm1"]
    yield "shift", sd[p + "shift"]
    m = p + "mix."
    if ly.kind == "lightning":
        yield "mix.proj", torch.cat([sd[m + "q"], sd[m + "k"], sd[m + "v"], sd[m + "g"]], 0)
        # a decay acts at every token of a sequence: rounded once, from the config's double
        yield "mix.decay", torch.tensor(ly.decay, dtype=torch.float64).to(torch.float32)
        yield "mix.out_norm", sd[m + "norm"]
        yield "mix.o", sd[m + "o"]
    else:
        le, ri = m + "left.", m + "right."
        yield "mix.proj", _pad_rows(torch.cat([sd[le + "q"], sd[le + "k"], sd[le + "v"], sd[le + "g"]], 0))
        yield "mix.temp", sd[le + "temp"]
        yield "mix.o", sd[le + "o"]
        yield "side.mu", torch.cat([sd[ri + "mu." + s] for s in "rkvgw"], 0)
        yield "side.proj", torch.cat([sd[ri + s] for s in "rkvg"], 0)
        yield "side.w1", sd[ri + "w1"]
        yield "side.w2", sd[ri + "w2"]
        yield "side.w0", sd[ri + "w0"]
        yield "side.bonus", sd[ri + "u"].reshape(-1)
        yield "side.out_norm", sd[ri + "norm"]
        yield "side.o", sd[ri + "o"]
    if ly.ff is not None:
        f = p + "mlp."
        yield "norm2", sd[p + "norm2"]
        if ly.ff == "dense":
            yield "mlp.up", sd[f + "up"]
            yield "mlp.down", sd[f + "down"]
        else:
            yield "mlp.router", sd[f + "router"]
            yield "mlp.router_bias", sd[f + "correction"]
            if ly.n_experts:
                yield "mlp.experts_up", torch.cat([sd[f"{f}e{e}.up"] for e in range(ly.n_experts)], 0)
                yield "mlp.experts_down", torch.cat([sd[f"{f}e{e}.down"] for e in range(ly.n_experts)], 0)


def random_checkpoint(spec: PaluzenSpec, seed: int = 0, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """A random checkpoint in the checkpoint's own names.  Matrices are Normal(0, 1/sqrt(fan_in)); norm weights,
    shift and blend weights, temperatures, decay offsets, bonuses and corrections are non-trivial values so that
    none of them is silently ignored."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = spec.width

    def mat(r, c, s=None):
        s = s if s is not None else c ** -0.5
        return (torch.randn(r, c, generator=g, device=device, dtype=torch.float32) * s).to(dtype)

    def vec(n, mean=0.0, s=0.1):
        return (mean + torch.randn(n, generator=g, device=device, dtype=torch.float32) * s).to(dtype)

    def uni(n, lo, hi):
        return (lo + (hi - lo) * torch.rand(n, generator=g, device=device, dtype=torch.float32)).to(dtype)

    sd = {"embed": mat(spec.vocab, W, 1.0), "final.norm": vec(W, 1.0)}
    if spec.loop is not None:
        sd["loop.in"] = mat(W, 2 * W, W ** -0.5)
    for i, ly in enumerate(spec.base_layers):
        p = f"l{i}."
        sd[p + "norm1"], sd[p + "shift"] = vec(W, 1.0), uni(W, 0.0, 1.0)
        m = p + "mix."
        if ly.kind == "lightning":
            hd, hv = ly.heads * ly.dim, ly.heads * ly.vdim
            sd[m + "q"], sd[m + "k"], sd[m + "v"], sd[m + "g"] = mat(hd, W), mat(hd, W), mat(hv, W), mat(hv, W)
            sd[m + "norm"], sd[m + "o"] = vec(hv, 1.0), mat(W, hv)
        else:
            le, ri = m + "left.", m + "right."
            hd, hv, gd, gv = ly.heads * ly.dim, ly.heads * ly.vdim, ly.kv_heads * ly.dim, ly.kv_heads * ly.vdim
            sd[le + "q"], sd[le + "k"], sd[le + "v"] = mat(hd, W), mat(gd, W), mat(gv, W)
            sd[le + "temp"], sd[le + "g"], sd[le + "o"] = uni(ly.heads, 0.5, 1.5), mat(ly.heads, W), mat(W, hv)
            rd = ly.r_heads * ly.r_dim
            for s in "rkvgw":
                sd[ri + "mu." + s] = uni(W, 0.0, 1.0)
            for s in "rkvg":
                sd[ri + s] = mat(rd, W)
            sd[ri + "w1"], sd[ri + "w2"] = mat(ly.r_rank, W), mat(rd, ly.r_rank)
            sd[ri + "w0"] = uni(rd, -4.0, 0.0)
            sd[ri + "u"] = vec(rd, 0.0, 0.5).reshape(ly.r_heads, ly.r_dim)
            sd[ri + "norm"], sd[ri + "o"] = vec(rd, 1.0), mat(W, rd)
        if ly.ff is not None:
            f = p + "mlp."
            sd[p + "norm2"] = vec(W, 1.0)
            if ly.ff == "dense":
                sd[f + "up"], sd[f + "down"] = mat(ly.ff_dim, W), mat(W, ly.ff_dim)
            else:
                tot = ly.n_experts + ly.n_identity
                sd[f + "router"] = mat(tot, W, 2.0 * W ** -0.5)
                sd[f + "correction"] = vec(tot, 0.0, 0.5 / tot)
                for e in range(ly.n_experts):
                    sd[f"{f}e{e}.up"], sd[f"{f}e{e}.down"] = mat(ly.ff_dim, W), mat(W, ly.ff_dim)
    return sd


def _cycle(width: int, vocab: int, n_layers: int, heads: int, kv_heads: int, dim: int, experts: int, top: int,
           ff: int, name: str, loop=None) -> PaluzenSpec:
    """layers in the order lightning, parallel, parallel, lightning, ... with a routed feed-forward in every layer
    but the first, whose feed-forward is dense"""
    lh = width // 128
    layers: List[PaluzenLayer] = []
    for i in range(n_layers):
        moe = dict(ff="moe", ff_dim=ff, n_experts=experts, n_identity=experts // 4, top_k=top, n_groups=4, keep_groups=2)
        if i == 0:
            moe = dict(ff="dense", ff_dim=4 * width)
        if i % 4 in (0, 3):
            decay = tuple(1.0 - 2.0 ** (-1.0 - 8.0 * h / max(lh - 1, 1)) for h in range(lh))
            layers.append(PaluzenLayer(kind="lightning", heads=lh, dim=64, vdim=128, decay=decay, **moe))
        else:
            layers.append(PaluzenLayer(kind="parallel", heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, window=2048,
                                       rot_dims=dim // 2, scale=dim ** -0.5, left_scale=1.0, r_heads=width // 64, r_dim=64,
                                       r_rank=64, right_scale=1.0, **moe))
    return PaluzenSpec(width=width, vocab=vocab, base_layers=layers, loop=loop, rms_eps=1e-5, logit_softcap=50.0, name=name)


# sizes that resemble a real model's layers (random weights; `random:<name>` as a model name)
BUILTIN_SPECS = {
    "paluzen-1b": _cycle(2048, 32768, 16, 16, 4, 128, 16, 4, 1536, "paluzen-1b"),
    "paluzen-3b": _cycle(3072, 32768, 24, 24, 8, 128, 32, 6, 2304, "paluzen-3b"),
}
