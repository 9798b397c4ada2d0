"""Host side of the Ramopel decoder: reading its config.json, mapping its checkpoint to the engine's
layered-model weights, and drawing random checkpoints for tests and benchmarks.

Ramopel is a stack of parallel layers  x <- x + mixer(norm1 x) + ff(norm2 x)  whose mixer is either
latent attention (low-rank queries and keys/values, one rotated key part shared by the heads, a sliding
window, optionally reading the cached latents of an earlier layer) or a generalized delta-rule
recurrence, and whose feed-forward is PolyNorm-dense, a top-k mixture of clamped gated experts with an
optional gated shared expert, or absent.  Every size comes from config.json or from a tensor's shape;
the native side (`b200q_model_create_layered`) takes the same information as one `b200q_layer_desc`
per layer, so other layered designs can reuse the mixers and feed-forwards with other constants.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from . import lib as L

ARCHITECTURE = "Ramopel"


@dataclass
class RamopelLayer:
    mixer: str                       # "latent_attention" | "general_delta"
    heads: int
    dim: int                         # attention: unrotated q/k dims per head; delta: key = value dims
    rot_dim: int = 0
    vdim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    kv_from: int = -1                # layer whose cached latents are read, -1 = own
    window: int = 0                  # 0 = every earlier key
    rot_dims: int = 0
    rot_base: float = 10000.0
    attn_scale: float = 1.0
    decay_rank: int = 0              # delta: inner size of the low-rank decay projection (from the tensor)
    ff: Optional[str] = None         # None | "dense" | "moe"
    ff_dim: int = 0
    n_experts: int = 0
    top_k: int = 0
    expert_limit: float = 0.0
    shared_dim: int = 0
    shared_limit: float = 0.0

    def desc(self) -> L.LayerDesc:
        return L.LayerDesc(
            mixer=L.MIXER_LATENT_ATTN if self.mixer == "latent_attention" else L.MIXER_GENERAL_DELTA,
            heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim, q_rank=self.q_rank,
            kv_rank=self.kv_rank, kv_from=self.kv_from, window=self.window, rot_dims=self.rot_dims,
            rot_base=self.rot_base, attn_scale=self.attn_scale, decay_rank=self.decay_rank,
            ff={None: L.FF_NONE, "dense": L.FF_POLYNORM, "moe": L.FF_MOE}[self.ff], ff_dim=self.ff_dim,
            n_experts=self.n_experts, top_k=self.top_k, expert_limit=self.expert_limit,
            shared_dim=self.shared_dim, shared_limit=self.shared_limit)


@dataclass
class RamopelSpec:
    """What `NativeModel` needs to know about a Ramopel checkpoint (the counterpart of `ModelSpec`)."""
    width: int
    vocab: int
    layers: List[RamopelLayer]
    rms_eps: float = 1e-5
    embed_scale: float = 1.0
    name: str = "ramopel"
    max_position_embeddings: int = 1 << 16   # positions are computed, not tabulated: the pool is the limit
    eos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    arch: str = "ramopel"
    layered: bool = field(default=True, repr=False)

    # the attributes the generic host code reads from any spec
    @property
    def hidden(self) -> int:
        return self.width

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    def config_extras(self) -> dict:
        """the fields of b200q_model_config that describe this design's layer form"""
        return dict(arch=L.ARCH_RAMOPEL, layer_form=L.FORM_PARALLEL, embed_scale=self.embed_scale)

    def engine_weights(self, sd: Dict[str, torch.Tensor]) -> Iterable[Tuple[str, torch.Tensor]]:
        return engine_weights(self, sd)

    def random_checkpoint(self, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
        return random_checkpoint(self, seed, device)

    @staticmethod
    def from_config(cfg: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None,
                    name: str = "ramopel") -> "RamopelSpec":
        """cfg: the parsed config.json; shapes: tensor name -> shape of the checkpoint, for the sizes that
        only a tensor gives (the rank of the decay projection)."""
        if cfg.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} config: architecture={cfg.get('architecture')!r}")
        layers: List[RamopelLayer] = []
        for i, lc in enumerate(cfg["layers"]):
            mx = lc["mixer"]
            if lc["type"] == "latent_attention":
                rot = mx.get("rot") or {}
                rot_dim = int(mx.get("rot_dim", 0))
                kv_from = mx.get("kv_from")
                ly = RamopelLayer(
                    mixer="latent_attention", heads=int(mx["heads"]), dim=int(mx["dim"]), rot_dim=rot_dim,
                    vdim=int(mx["vdim"]), q_rank=int(mx["q_rank"]), kv_rank=int(mx["kv_rank"]),
                    kv_from=-1 if kv_from is None else int(kv_from),
                    window=int((mx.get("mask") or {}).get("size", 0)),
                    rot_dims=int(rot.get("dims", rot_dim)), rot_base=float(rot.get("base", 10000.0)),
                    attn_scale=float(mx["scale"]))
            elif lc["type"] == "general_delta":
                rk = int(mx.get("decay_rank", 0))
                if shapes is not None and f"l{i}.mix.w1" in shapes:
                    rk = int(shapes[f"l{i}.mix.w1"][0])
                if rk <= 0:
                    raise ValueError(f"layer {i}: the decay projection's rank comes from the tensor l{i}.mix.w1")
                ly = RamopelLayer(mixer="general_delta", heads=int(mx["heads"]), dim=int(mx["dim"]), decay_rank=rk)
            else:
                raise ValueError(f"layer {i}: unknown layer type {lc['type']!r}")
            ml = lc.get("mlp")
            if ml:
                if ml["kind"] == "dense":
                    ly.ff, ly.ff_dim = "dense", int(ml["ff"])
                elif ml["kind"] == "moe":
                    ly.ff, ly.ff_dim = "moe", int(ml["expert"]["ff"])
                    ly.expert_limit = float(ml["expert"]["limit"])
                    ly.n_experts, ly.top_k = int(ml["router"]["experts"]), int(ml["router"]["top"])
                    sh = ml.get("shared")
                    if sh:
                        ly.shared_dim, ly.shared_limit = int(sh["ff"]), float(sh["limit"])
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {ml['kind']!r}")
            layers.append(ly)
        return RamopelSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=layers,
                           rms_eps=float(cfg["norm"]["eps"]),
                           embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)), name=name)

    def to_config(self) -> dict:
        out = []
        for ly in self.layers:
            if ly.mixer == "latent_attention":
                mx = {"heads": ly.heads, "dim": ly.dim, "rot_dim": ly.rot_dim, "vdim": ly.vdim, "q_rank": ly.q_rank,
                      "kv_rank": ly.kv_rank, "scale": ly.attn_scale,
                      "rot": {"base": ly.rot_base, "dims": ly.rot_dims}}
                if ly.window:
                    mx["mask"] = {"size": ly.window}
                if ly.kv_from >= 0:
                    mx["kv_from"] = ly.kv_from
            else:
                mx = {"heads": ly.heads, "dim": ly.dim}
            if ly.ff == "dense":
                ml = {"kind": "dense", "ff": ly.ff_dim}
            elif ly.ff == "moe":
                ml = {"kind": "moe", "expert": {"ff": ly.ff_dim, "limit": ly.expert_limit},
                      "router": {"experts": ly.n_experts, "top": ly.top_k}}
                if ly.shared_dim:
                    ml["shared"] = {"ff": ly.shared_dim, "limit": ly.shared_limit}
            else:
                ml = None
            out.append({"type": ly.mixer, "mixer": mx, "mlp": ml})
        return {"architecture": ARCHITECTURE, "width": self.width, "vocab": self.vocab,
                "norm": {"eps": self.rms_eps}, "embedding": {"scale": self.embed_scale}, "layers": out}

    def weight_bytes_per_token(self, esize: int = 2, batch: int = 1) -> int:
        """matrix bytes one decode step of `batch` tokens touches (a routed layer reads at most
        min(experts, batch * top_k) of its experts; the embedding table is read by row, the head in full)"""
        W, n = self.width, self.vocab * self.width
        for ly in self.layers:
            if ly.mixer == "latent_attention":
                own = ly.kv_rank + ly.rot_dim if ly.kv_from < 0 else 0
                n += W * (ly.q_rank + own) + ly.heads * (ly.dim + ly.rot_dim) * ly.q_rank
                n += ly.heads * ly.kv_rank * (ly.dim + ly.vdim) + W * ly.heads * ly.vdim
            else:
                hd = ly.heads * ly.dim
                n += W * (5 * hd + ly.decay_rank) + hd * ly.decay_rank + W * hd
            if ly.ff == "dense":
                n += 2 * W * ly.ff_dim
            elif ly.ff == "moe":
                n += (W * ly.n_experts + 3 * W * ly.ff_dim * min(ly.n_experts, batch * ly.top_k) + 3 * W * ly.shared_dim
                      + (W if ly.shared_dim else 0))
        return n * esize


# ---- checkpoint file -------------------------------------------------------------------------------
_ST_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32,
              "I64": torch.int64, "F64": torch.float64}


def read_safetensors_header(path: str) -> Tuple[dict, int]:
    """-> (header, offset of the data section).  The file is an 8-byte little-endian length, that many
    bytes of JSON (name -> dtype, shape, data_offsets) and the tensors' bytes."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
    header.pop("__metadata__", None)
    return header, 8 + n


def checkpoint_shapes(path: str) -> Dict[str, Tuple[int, ...]]:
    header, _ = read_safetensors_header(path)
    return {k: tuple(v["shape"]) for k, v in header.items()}


def load_checkpoint(path: str) -> Dict[str, torch.Tensor]:
    """every tensor of a safetensors file, in its stored dtype (host memory)"""
    import numpy as np

    header, base = read_safetensors_header(path)
    raw = np.fromfile(path, dtype=np.uint8)
    out: Dict[str, torch.Tensor] = {}
    for name, info in header.items():
        dt = _ST_DTYPES.get(info["dtype"])
        if dt is None:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
        lo, hi = info["data_offsets"]
        buf = torch.from_numpy(raw[base + lo: base + hi])
        out[name] = buf.view(dt).reshape(tuple(info["shape"])) if hi > lo else torch.empty(tuple(info["shape"]), dtype=dt)
    return out


# ---- checkpoint names -> engine names --------------------------------------------------------------
def engine_weights(spec: RamopelSpec, sd: Dict[str, torch.Tensor]) -> Iterable[Tuple[str, torch.Tensor]]:
    """Checkpoint tensors -> the layered engine's weights.  2-D results are matrices (bound in the model's
    dtype); 1-D results are vectors and constants (bound as fp32 rows).  Fusions: the two down-projections
    of a latent-attention layer become one matrix (query rows first), the five token projections and the
    decay's inner projection of a delta layer become one, gate and up of every expert are stacked, and
    each head's key up-projection is stored transposed (the engine carries the query into the latent
    space instead of expanding every cached latent into keys)."""
    yield "embed", sd["embed"]
    yield "final_norm", sd["final.norm"]
    yield "lm_head", sd["head"]
    for i, ly in enumerate(spec.layers):
        p, o = f"l{i}.", f"layers.{i}."
        yield o + "norm1", sd[p + "norm1"]
        if ly.ff is not None:
            yield o + "norm2", sd[p + "norm2"]
        m = p + "mix."
        if ly.mixer == "latent_attention":
            own = ly.kv_from < 0
            yield o + "mix.down", (torch.cat([sd[m + "dq"], sd[m + "dkv"]], 0) if own else sd[m + "dq"])
            yield o + "mix.q_norm", sd[m + "dq.norm"]
            if own:
                yield o + "mix.kv_norm", sd[m + "dkv.norm"]
            yield o + "mix.uq", sd[m + "uq"]
            uk = sd[m + "uk"].reshape(ly.heads, ly.dim, ly.kv_rank)
            yield o + "mix.uk_t", uk.transpose(1, 2).reshape(ly.heads * ly.kv_rank, ly.dim)
            yield o + "mix.uv", sd[m + "uv"]
            yield o + "mix.o", sd[m + "o"]
        else:
            yield o + "mix.proj", torch.cat([sd[m + n] for n in ("r", "k", "v", "g", "a", "w1")], 0)
            yield o + "mix.w2", sd[m + "w2"]
            yield o + "mix.w0", sd[m + "w0"]
            yield o + "mix.a_bias", sd[m + "a.b"]
            yield o + "mix.out_norm", sd[m + "norm"]
            yield o + "mix.o", sd[m + "o"]
        f = p + "mlp."
        if ly.ff == "dense":
            yield o + "mlp.up", sd[f + "up"]
            yield o + "mlp.act", sd[f + "act"]
            yield o + "mlp.down", sd[f + "down"]
        elif ly.ff == "moe":
            yield o + "mlp.router", sd[f + "router"]
            yield o + "mlp.router_bias", sd[f + "router.b"]
            yield o + "mlp.experts_gate_up", torch.cat(
                [t for e in range(ly.n_experts) for t in (sd[f"{f}e{e}.gate"], sd[f"{f}e{e}.up"])], 0)
            yield o + "mlp.experts_down", torch.cat([sd[f"{f}e{e}.down"] for e in range(ly.n_experts)], 0)
            if ly.shared_dim:
                yield o + "mlp.shared_gate_up", torch.cat([sd[f + "shared.gate"], sd[f + "shared.up"]], 0)
                yield o + "mlp.shared_down", sd[f + "shared.down"]
                yield o + "mlp.shared_gate", sd[f + "shared.sg"].reshape(1, -1)


def random_checkpoint(spec: RamopelSpec, seed: int = 0, device="cpu", std: Optional[float] = None,
                      dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """A random checkpoint in the checkpoint's own names.  Matrices are Normal(0, std or 1/sqrt(fan_in));
    norm offsets, biases and the PolyNorm constants are small non-zero values so that none of them is
    silently ignored."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = spec.width

    def mat(r, c, s=None):
        s = s if s is not None else (std if std is not None else c ** -0.5)
        return (torch.randn(r, c, generator=g, device=device, dtype=torch.float32) * s).to(dtype)

    def vec(n, mean=0.0, s=0.1):
        return (mean + torch.randn(n, generator=g, device=device, dtype=torch.float32) * s).to(dtype)

    sd = {"embed": mat(spec.vocab, W, 1.0), "final.norm": vec(W), "head": mat(spec.vocab, W)}
    for i, ly in enumerate(spec.layers):
        p = f"l{i}."
        sd[p + "norm1"] = vec(W)
        if ly.ff is not None:
            sd[p + "norm2"] = vec(W)
        m = p + "mix."
        if ly.mixer == "latent_attention":
            sd[m + "dq"] = mat(ly.q_rank, W)
            sd[m + "dq.norm"] = vec(ly.q_rank, 1.0)
            sd[m + "uq"] = mat(ly.heads * (ly.dim + ly.rot_dim), ly.q_rank)
            if ly.kv_from < 0:
                sd[m + "dkv"] = mat(ly.kv_rank + ly.rot_dim, W)
                sd[m + "dkv.norm"] = vec(ly.kv_rank, 1.0)
            sd[m + "uk"] = mat(ly.heads * ly.dim, ly.kv_rank)
            sd[m + "uv"] = mat(ly.heads * ly.vdim, ly.kv_rank)
            sd[m + "o"] = mat(W, ly.heads * ly.vdim)
        else:
            hd = ly.heads * ly.dim
            for n in ("r", "k", "v", "g", "a"):
                sd[m + n] = mat(hd, W)
            sd[m + "a.b"] = vec(hd)
            sd[m + "w1"] = mat(ly.decay_rank, W)
            sd[m + "w2"] = mat(hd, ly.decay_rank)
            sd[m + "w0"] = vec(hd, 0.0, 1.0)
            sd[m + "norm"] = vec(hd, 1.0)
            sd[m + "o"] = mat(W, hd)
        f = p + "mlp."
        if ly.ff == "dense":
            sd[f + "up"] = mat(ly.ff_dim, W)
            sd[f + "down"] = mat(W, ly.ff_dim)
            sd[f + "act"] = torch.tensor([0.6, 0.3, 0.15, 0.05], device=device).to(dtype) + vec(4, 0.0, 0.02)
        elif ly.ff == "moe":
            sd[f + "router"] = mat(ly.n_experts, W)
            sd[f + "router.b"] = vec(ly.n_experts)
            for e in range(ly.n_experts):
                sd[f"{f}e{e}.gate"] = mat(ly.ff_dim, W)
                sd[f"{f}e{e}.up"] = mat(ly.ff_dim, W)
                sd[f"{f}e{e}.down"] = mat(W, ly.ff_dim)
            if ly.shared_dim:
                sd[f + "shared.gate"] = mat(ly.shared_dim, W)
                sd[f + "shared.up"] = mat(ly.shared_dim, W)
                sd[f + "shared.down"] = mat(W, ly.shared_dim)
                sd[f + "shared.sg"] = mat(1, W)
    return sd


def save_checkpoint(path: str, sd: Dict[str, torch.Tensor]) -> None:
    """write `sd` as a safetensors file (the inverse of load_checkpoint)"""
    names = {v: k for k, v in _ST_DTYPES.items()}
    header, blobs, at = {}, [], 0
    for k, t in sd.items():
        # a tensor without axes (one scalar) is written through a one-element view and keeps its empty shape
        b = t.detach().cpu().contiguous().reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[k] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(b)]}
        blobs.append(b)
        at += len(b)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def _alternating(width: int, vocab: int, pairs: int, heads_attn: int, heads_delta: int, experts: int, top: int,
                 name: str) -> RamopelSpec:
    """`pairs` times (delta layer with a PolyNorm feed-forward, attention layer with a routed one); every
    second attention layer reads the latents of the one before it"""
    layers: List[RamopelLayer] = []
    for p in range(pairs):
        layers.append(RamopelLayer(mixer="general_delta", heads=heads_delta, dim=width // heads_delta, decay_rank=64,
                                   ff="dense", ff_dim=4 * width))
        layers.append(RamopelLayer(mixer="latent_attention", heads=heads_attn, dim=128, rot_dim=64, vdim=128,
                                   q_rank=width // 2, kv_rank=512, kv_from=(2 * p - 1) if p % 2 else -1, window=4096,
                                   rot_dims=64, rot_base=10000.0, attn_scale=192 ** -0.5, ff="moe", ff_dim=width // 2,
                                   n_experts=experts, top_k=top, expert_limit=7.0, shared_dim=width,
                                   shared_limit=7.0))
    return RamopelSpec(width=width, vocab=vocab, layers=layers, rms_eps=1e-5, embed_scale=1.0, name=name)


# sizes that resemble a real model's layers (random weights; `random:<name>` as a model name)
BUILTIN_SPECS = {
    "ramopel-1b": _alternating(2048, 32768, 8, 16, 32, 32, 4, "ramopel-1b"),
    "ramopel-3b": _alternating(3072, 32768, 12, 24, 48, 64, 6, "ramopel-3b"),
}
