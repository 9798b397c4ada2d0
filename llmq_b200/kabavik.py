"""Host side of the Kabavik decoder: reading its config.json, mapping its checkpoint to the engine's
layered-model weights, and drawing random checkpoints for tests and benchmarks.

Kabavik is a stack of layers over an fp32 residual stream with a norm on BOTH sides of every sublayer and a
residual multiplier m,

    x <- x + m * Nb1(mixer(N1 x))      x <- x + m * Nb2(ff(N2 x))      x <- x + m * R(P (gelu(G x) * e_i)) * s

N = dynamic tanh, tanh(alpha v) * w + b, which needs no statistics of the row; R(v) = v / sqrt(mean(v^2) + eps);
e_i = layer i's columns of a second embedding row of the token (the per-layer token input).  Mixers:

  attention         grouped-query attention with biases, one RMS norm over the whole query (key) projection,
                    half-split rotation of the leading dimensions with linearly scaled frequencies, a sliding
                    window behind which the first tokens stay visible; a layer may read the keys and values an
                    earlier layer cached instead of making its own
  latent_attention  full-rank queries; keys and values from a normed latent plus one rotated key part shared by
                    the heads (only those two are cached); interleaved rotation with YaRN-scaled frequencies;
                    sliding window; one sigmoid gate number per head
  attention_2       grouped-query attention with biases, RMS norm per head on queries and keys, no rotation, a
                    query temperature 1 + c ln(floor((p + 1) / n) + 1) at position p, soft-capped scores, every
                    earlier key

Feed-forward: down(gelu_tanh(gate h) * up h).  Logits = head N(x) * logit_scale.  Every size comes from
config.json or a tensor's shape.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from . import lib as L
from .ramopel import checkpoint_shapes, load_checkpoint, save_checkpoint  # noqa: F401  (one file format)

ARCHITECTURE = "Kabavik"
KINDS = ("attention", "latent_attention", "attention_2")


@dataclass
class KabavikLayer:
    kind: str                        # one of KINDS
    heads: int = 0
    kv_heads: int = 0                # attention, attention_2
    dim: int = 0                     # per-head query / key size (latent attention: the unrotated part)
    vdim: int = 0
    rot_dim: int = 0                 # latent attention: the rotated part of a head
    kv_rank: int = 0                 # latent attention: size of the cached latent
    window: int = 0                  # 0 = every earlier key
    keep_first: int = 0              # attention: keys that stay visible behind the window
    rot_dims: int = 0                # rotated dimensions; 0 = no rotation
    rot_base: float = 10000.0
    rot_factor: float = 0.0          # 0 = unscaled frequencies
    rot_original: float = 0.0        # > 0: YaRN (with rot_fast, rot_slow)
    rot_fast: float = 0.0
    rot_slow: float = 0.0
    scale: float = 1.0
    softcap: float = 0.0             # attention_2
    q_temp_coef: float = 0.0         # attention_2
    q_temp_every: int = 0
    kv_from: int = -1                # attention: layer whose cached keys and values are read, -1 = own
    ff: Optional[str] = None         # None | "dense"
    ff_dim: int = 0

    def desc(self) -> L.LayerDesc:
        ff = dict(ff=L.FF_GEGLU if self.ff else L.FF_NONE, ff_dim=self.ff_dim)
        rot = dict(rot_dims=self.rot_dims, rot_base=self.rot_base, rot_factor=self.rot_factor,
                   rot_original=self.rot_original, rot_fast=self.rot_fast, rot_slow=self.rot_slow)
        if self.kind == "latent_attention":
            return L.LayerDesc(mixer=L.MIXER_LATENT_ATTN, heads=self.heads, dim=self.dim, rot_dim=self.rot_dim,
                               vdim=self.vdim, q_rank=0, kv_rank=self.kv_rank, kv_from=-1, window=self.window,
                               attn_scale=self.scale, head_gate=1, **rot, **ff)
        return L.LayerDesc(mixer=L.MIXER_WINDOW_ATTN, heads=self.heads, kv_heads=self.kv_heads, dim=self.dim,
                           vdim=self.vdim, kv_from=self.kv_from, window=self.window, keep_first=self.keep_first,
                           attn_scale=self.scale, softcap=self.softcap, q_temp_coef=self.q_temp_coef,
                           q_temp_every=self.q_temp_every, qk_norm=1 if self.kind == "attention" else 2, proj_bias=1,
                           bare=1, **rot, **ff)


def _rotation(i: int, mx: dict, limit: int) -> dict:
    rot = mx.get("rot") or {}
    dims = int(rot.get("dims") or 0)
    if dims % 2 or dims > limit:
        raise ValueError(f"layer {i}: rot.dims ({dims}) must be even and at most {limit}")
    sc = rot.get("scaling") or {}
    out = dict(rot_dims=dims, rot_base=float(rot.get("base", 10000.0)), rot_factor=float(sc.get("factor") or 0.0))
    if "original" in sc:
        out.update(rot_original=float(sc["original"]), rot_fast=float(sc["fast"]), rot_slow=float(sc["slow"]))
    return out


def _layer_from_config(i: int, lc: dict, layers: List[KabavikLayer]) -> KabavikLayer:
    mx, kind = lc["mixer"], lc["type"]
    mask = mx.get("mask") or {}
    if kind == "latent_attention":
        ly = KabavikLayer(kind=kind, heads=int(mx["heads"]), dim=int(mx["dim"]), rot_dim=int(mx.get("rot_dim") or 0),
                          vdim=int(mx.get("vdim", mx["dim"])), kv_rank=int(mx["kv_rank"]),
                          window=int(mask.get("size") or 0), scale=float(mx["scale"]),
                          **_rotation(i, mx, int(mx.get("rot_dim") or 0)))
    elif kind in ("attention", "attention_2"):
        ly = KabavikLayer(kind=kind, heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])),
                          dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])), window=int(mask.get("size") or 0),
                          keep_first=int(mask.get("keep_first") or 0), scale=float(mx["scale"]))
        if ly.heads % ly.kv_heads:
            raise ValueError(f"layer {i}: kv_heads ({ly.kv_heads}) must divide heads ({ly.heads})")
        if kind == "attention":
            for k, v in _rotation(i, mx, ly.dim).items():
                setattr(ly, k, v)
            src = mx.get("kv_from")
            if src is not None:
                src = int(src)
                o = layers[src] if 0 <= src < i else None
                if o is None or o.kind != "attention" or o.kv_from >= 0 or (o.kv_heads, o.dim, o.vdim) != (
                        ly.kv_heads, ly.dim, ly.vdim):
                    raise ValueError(f"layer {i}: kv_from={src} must name an earlier attention layer with keys and "
                                     "values of its own and the same sizes")
                ly.kv_from = src
        else:
            qt = mx.get("q_temp") or {}
            ly.softcap = float(mx.get("softcap") or 0.0)
            ly.q_temp_coef, ly.q_temp_every = float(qt.get("coef") or 0.0), int(qt.get("every") or 0)
    else:
        raise ValueError(f"layer {i}: unknown layer type {kind!r}")
    ml = lc.get("mlp")
    if ml:
        if ml["kind"] != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {ml['kind']!r}")
        ly.ff, ly.ff_dim = "dense", int(ml["ff"])
    return ly


def _layer_to_config(ly: KabavikLayer) -> dict:
    mx: dict = {"heads": ly.heads, "dim": ly.dim, "vdim": ly.vdim, "scale": ly.scale}
    mask = {}
    if ly.window:
        mask["size"] = ly.window
    if ly.keep_first:
        mask["keep_first"] = ly.keep_first
    if mask:
        mx["mask"] = mask
    if ly.rot_dims:
        rot: dict = {"dims": ly.rot_dims, "base": ly.rot_base}
        if ly.rot_factor:
            rot["scaling"] = {"factor": ly.rot_factor}
            if ly.rot_original:
                rot["scaling"].update(original=ly.rot_original, fast=ly.rot_fast, slow=ly.rot_slow)
        mx["rot"] = rot
    if ly.kind == "latent_attention":
        mx.update(rot_dim=ly.rot_dim, kv_rank=ly.kv_rank)
    else:
        mx["kv_heads"] = ly.kv_heads
        if ly.kv_from >= 0:
            mx["kv_from"] = ly.kv_from
        if ly.kind == "attention_2":
            if ly.softcap:
                mx["softcap"] = ly.softcap
            if ly.q_temp_every:
                mx["q_temp"] = {"coef": ly.q_temp_coef, "every": ly.q_temp_every}
    return {"type": ly.kind, "mixer": mx, "mlp": {"kind": "dense", "ff": ly.ff_dim} if ly.ff else None}


@dataclass
class KabavikSpec:
    """What `NativeModel` needs to know about a Kabavik checkpoint (the counterpart of `ModelSpec`)."""
    width: int
    vocab: int
    layers: List[KabavikLayer]
    rms_eps: float = 1e-6
    residual_mult: float = 1.0
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    side_dim: int = 0                        # columns of the second embedding table one layer reads; 0 = none
    name: str = "kabavik"
    max_position_embeddings: int = 1 << 20   # positions are computed, not tabulated: the pool is the limit
    eos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    arch: str = "kabavik"
    layered: bool = field(default=True, repr=False)

    @property
    def hidden(self) -> int:
        return self.width

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    def config_extras(self) -> dict:
        """the fields of b200q_model_config that describe this design's layer form"""
        return dict(arch=L.ARCH_KABAVIK, layer_form=L.FORM_SANDWICH, norm_kind=L.NORM_DYT,
                    residual_mult=self.residual_mult, side_dim=self.side_dim, logit_scale=self.logit_scale,
                    embed_scale=self.embed_scale)

    @staticmethod
    def from_config(cfg: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None,
                    name: str = "kabavik") -> "KabavikSpec":
        if cfg.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} config: architecture={cfg.get('architecture')!r}")
        layers: List[KabavikLayer] = []
        for i, lc in enumerate(cfg["layers"]):
            layers.append(_layer_from_config(i, lc, layers))
        return KabavikSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=layers,
                           rms_eps=float((cfg.get("norm") or {}).get("eps", 1e-6)),
                           residual_mult=float(cfg.get("residual_mult", 1.0)),
                           embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                           logit_scale=float(cfg.get("logit_scale", 1.0)),
                           side_dim=int((cfg.get("token_side") or {}).get("dim") or 0), name=name)

    def to_config(self) -> dict:
        cfg = {"architecture": ARCHITECTURE, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.rms_eps},
               "residual_mult": self.residual_mult, "embedding": {"scale": self.embed_scale},
               "logit_scale": self.logit_scale, "layers": [_layer_to_config(ly) for ly in self.layers]}
        if self.side_dim:
            cfg["token_side"] = {"dim": self.side_dim}
        return cfg

    def engine_weights(self, sd: Dict[str, torch.Tensor]) -> Iterable[Tuple[str, torch.Tensor]]:
        return engine_weights(self, sd)

    def random_checkpoint(self, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
        return random_checkpoint(self, seed, device)

    def weight_bytes_per_token(self, esize: int = 2, batch: int = 1) -> int:
        """matrix bytes one decode step touches (embedding rows are read by row, the output matrix in full)"""
        W, n = self.width, self.vocab * self.width
        for ly in self.layers:
            if ly.kind == "latent_attention":
                n += W * (ly.heads * (ly.dim + ly.rot_dim) + ly.kv_rank + ly.rot_dim + ly.heads)
                n += ly.heads * ly.kv_rank * (ly.dim + ly.vdim) + W * ly.heads * ly.vdim
            else:
                own = ly.kv_heads * (ly.dim + ly.vdim) if ly.kv_from < 0 else 0
                n += W * (ly.heads * ly.dim + own) + W * ly.heads * ly.vdim
            if ly.ff:
                n += 3 * W * ly.ff_dim
            n += 2 * W * self.side_dim
        return n * esize


# ---- checkpoint names -> engine names --------------------------------------------------------------
def _pad_rows(t: torch.Tensor, mult: int = 64) -> torch.Tensor:
    pad = -t.shape[0] % mult
    return torch.cat([t, t.new_zeros((pad,) + tuple(t.shape[1:]))], 0) if pad else t


GLU_BLOCK = 128


def _interleave(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[F, W], [F, W] -> [2F, W] with rows [256j, 256j + 128) = gate rows [128j, 128j + 128) and the next 128 the same
    rows of up: one 256-wide tile of the product carries both halves of 128 outputs, so the gated unit can be applied
    in the product's epilogue"""
    F, W = gate.shape
    return torch.stack([gate.view(F // GLU_BLOCK, GLU_BLOCK, W), up.view(F // GLU_BLOCK, GLU_BLOCK, W)], 1).reshape(2 * F, W)


def _dyt_row(sd, name: str) -> torch.Tensor:
    """a dynamic-tanh norm as the engine binds it: one row [w | b | alpha]"""
    return torch.cat([sd[name].reshape(-1).float(), sd[name + ".b"].reshape(-1).float(),
                      sd[name + ".alpha"].reshape(1).float()])


def engine_weights(spec: KabavikSpec, sd: Dict[str, torch.Tensor]) -> Iterable[Tuple[str, torch.Tensor]]:
    """Checkpoint tensors -> the layered engine's weights.  2-D results are matrices (bound in the model's dtype);
    1-D results are vectors and constants (bound as fp32 rows).  Fusions: the projections that read a mixer's input
    become one matrix with zero rows up to a multiple of 64 (attention: q, k, v — q alone when the keys and values
    are an earlier layer's; latent attention: q, the latent, the shared rotated key, the gate rows), their biases one
    row; gate and up of the feed-forward are stacked (interleaved in blocks of 128 rows when ff is a multiple of 128); each head's key up-projection is stored transposed (the engine
    carries the query into the latent space instead of expanding every cached latent into keys); a dynamic-tanh
    norm is one row [w | b | alpha]."""
    yield "embed", sd["embed"]
    yield "final_norm", _dyt_row(sd, "final.norm")
    yield "lm_head", sd["head"]
    if spec.side_dim:
        yield "tok_embed", sd["side.embed"]
    for i, ly in enumerate(spec.layers):
        p, o = f"l{i}.", f"layers.{i}."
        m = p + "mix."
        yield o + "norm1", _dyt_row(sd, p + "norm1")
        yield o + "norm1b", _dyt_row(sd, p + "norm1b")
        if ly.kind == "latent_attention":
            yield o + "mix.down", _pad_rows(torch.cat([sd[m + "q"], sd[m + "dkv"], sd[m + "g"]], 0))
            yield o + "mix.kv_norm", sd[m + "dkv.norm"]
            uk = sd[m + "uk"].reshape(ly.heads, ly.dim, ly.kv_rank)
            yield o + "mix.uk_t", uk.transpose(1, 2).reshape(ly.heads * ly.kv_rank, ly.dim)
            yield o + "mix.uv", sd[m + "uv"]
            yield o + "mix.o", sd[m + "o"]
        else:
            parts = ("q", "k", "v") if ly.kv_from < 0 else ("q",)
            yield o + "mix.proj", _pad_rows(torch.cat([sd[m + n] for n in parts], 0))
            yield o + "mix.proj_b", _pad_rows(torch.cat([sd[m + n + ".b"].float() for n in parts], 0))
            yield o + "mix.q_norm", sd[m + "q.norm"]
            if ly.kv_from < 0:
                yield o + "mix.k_norm", sd[m + "k.norm"]
            yield o + "mix.o", sd[m + "o"]
            yield o + "mix.o_b", sd[m + "o.b"]
        if ly.ff:
            f = p + "mlp."
            yield o + "norm2", _dyt_row(sd, p + "norm2")
            yield o + "norm2b", _dyt_row(sd, p + "norm2b")
            if ly.ff_dim % GLU_BLOCK == 0:
                yield o + "mlp.gate_up_il", _interleave(sd[f + "gate"], sd[f + "up"])
            else:
                yield o + "mlp.gate_up", torch.cat([sd[f + "gate"], sd[f + "up"]], 0)
            yield o + "mlp.down", sd[f + "down"]
        if spec.side_dim:
            yield o + "tok.gate", sd[p + "side.gate"]
            yield o + "tok.proj", sd[p + "side.proj"]
            yield o + "tok.norm", sd[p + "side.norm"]


def random_checkpoint(spec: KabavikSpec, seed: int = 0, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """A random checkpoint in the checkpoint's own names.  Matrices are Normal(0, 1/sqrt(fan_in)); norm weights,
    offsets, slopes and biases are non-trivial values so that none of them is silently ignored."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = spec.width

    def mat(r, c, s=None):
        s = s if s is not None else c ** -0.5
        return (torch.randn(r, c, generator=g, device=device, dtype=torch.float32) * s).to(dtype)

    def vec(n, mean=0.0, s=0.1):
        return (mean + torch.randn(n, generator=g, device=device, dtype=torch.float32) * s).to(dtype)

    def uni(lo, hi):
        return (lo + (hi - lo) * torch.rand((), generator=g, device=device, dtype=torch.float32)).to(dtype)

    sd: Dict[str, torch.Tensor] = {}

    def dyt(name, slope=(0.4, 1.2)):
        sd[name], sd[name + ".b"], sd[name + ".alpha"] = vec(W, 1.0), vec(W, 0.0, 0.05), uni(*slope)

    sd["embed"] = mat(spec.vocab, W, 1.0 / max(spec.embed_scale, 1e-6))
    if spec.side_dim:
        sd["side.embed"] = mat(spec.vocab, spec.n_layers * spec.side_dim, 1.0)
    for i, ly in enumerate(spec.layers):
        p = f"l{i}."
        m = p + "mix."
        dyt(p + "norm1")
        dyt(p + "norm1b")
        hv = ly.heads * ly.vdim
        if ly.kind == "latent_attention":
            qd = ly.dim + ly.rot_dim
            sd[m + "q"], sd[m + "dkv"] = mat(ly.heads * qd, W), mat(ly.kv_rank + ly.rot_dim, W)
            sd[m + "dkv.norm"] = vec(ly.kv_rank, 1.0)
            sd[m + "uk"], sd[m + "uv"] = mat(ly.heads * ly.dim, ly.kv_rank), mat(hv, ly.kv_rank)
            sd[m + "g"], sd[m + "o"] = mat(ly.heads, W), mat(W, hv)
        else:
            hd, gd, gv = ly.heads * ly.dim, ly.kv_heads * ly.dim, ly.kv_heads * ly.vdim
            sd[m + "q"], sd[m + "q.b"] = mat(hd, W), vec(hd)
            sd[m + "q.norm"] = vec(hd if ly.kind == "attention" else ly.dim, 1.0)
            if ly.kv_from < 0:
                sd[m + "k"], sd[m + "k.b"], sd[m + "v"], sd[m + "v.b"] = mat(gd, W), vec(gd), mat(gv, W), vec(gv)
                sd[m + "k.norm"] = vec(gd if ly.kind == "attention" else ly.dim, 1.0)
            sd[m + "o"], sd[m + "o.b"] = mat(W, hv), vec(W)
        if ly.ff:
            f = p + "mlp."
            dyt(p + "norm2")
            dyt(p + "norm2b")
            sd[f + "gate"], sd[f + "up"], sd[f + "down"] = mat(ly.ff_dim, W), mat(ly.ff_dim, W), mat(W, ly.ff_dim)
        if spec.side_dim:
            sd[p + "side.gate"], sd[p + "side.proj"] = mat(spec.side_dim, W), mat(W, spec.side_dim)
            sd[p + "side.norm"] = vec(W, 1.0)
    dyt("final.norm", (0.1, 0.3))
    sd["head"] = mat(spec.vocab, W)
    return sd


def _cycle(width: int, vocab: int, n_layers: int, heads: int, kv_heads: int, ff: int, name: str) -> KabavikSpec:
    """layers in the order latent_attention, attention_2, attention, attention (the keys and values of the one
    before it), ... with head sizes the tensor-core attention kernels take"""
    layers: List[KabavikLayer] = []
    for i in range(n_layers):
        common = dict(ff="dense", ff_dim=ff)
        if i % 4 == 0:
            layers.append(KabavikLayer(kind="latent_attention", heads=heads, dim=128, rot_dim=64, vdim=128, kv_rank=512,
                                       window=4096, rot_dims=64, rot_base=10000.0, rot_factor=4.0, rot_original=4096.0,
                                       rot_fast=32.0, rot_slow=1.0, scale=192 ** -0.5, **common))
        elif i % 4 == 1:
            layers.append(KabavikLayer(kind="attention_2", heads=heads, kv_heads=kv_heads, dim=128, vdim=128,
                                       scale=128 ** -0.5, softcap=30.0, q_temp_coef=0.2, q_temp_every=1024, **common))
        else:
            layers.append(KabavikLayer(kind="attention", heads=heads, kv_heads=kv_heads, dim=128, vdim=128, window=2048,
                                       keep_first=4, rot_dims=64, rot_base=500000.0, rot_factor=2.0, scale=128 ** -0.5,
                                       kv_from=i - 1 if i % 4 == 3 else -1, **common))
    return KabavikSpec(width=width, vocab=vocab, layers=layers, rms_eps=1e-6, residual_mult=0.5,
                       embed_scale=float(width) ** 0.5, logit_scale=0.5, side_dim=64, name=name)


# sizes that resemble a real model's layers (random weights; `random:<name>` as a model name)
BUILTIN_SPECS = {
    "kabavik-1b": _cycle(2048, 32768, 16, 16, 4, 6144, "kabavik-1b"),
    "kabavik-3b": _cycle(3072, 32768, 24, 24, 8, 8192, "kabavik-3b"),
}
