"""CPU tests of the Kabavik host code: the config reader, the registry, the mapping of checkpoint tensors to engine
weights, the rotation-frequency table the engine uploads, and the oracle's own consistency (causality, window
confinement with kept first keys, rotations that depend on the distance only, borrowed keys)."""
import ctypes as C
import json
import math

import pytest
import torch

from llmq_b200 import kabavik as K
from llmq_b200 import lib as L
from oracle import kabavik as O
from tests.kabavik_util import DENSE, attn, attn2, checkpoint, latent, small_spec, tokens


def _with(cfg, path, value):
    bad = json.loads(json.dumps(cfg))
    at = bad
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    return bad


def test_config_round_trip_and_descriptions():
    spec = small_spec()
    cfg = json.loads(json.dumps(spec.to_config()))
    back = K.KabavikSpec.from_config(cfg)
    assert back.layers == spec.layers
    assert (back.width, back.vocab, back.rms_eps, back.residual_mult, back.embed_scale, back.logit_scale,
            back.side_dim) == (96, 211, 1e-5, 0.6, 3.0, 1.7, 10)
    assert back.layers[3].ff is None and back.layers[3].kv_from == 0 and back.layers[4].rot_original == 0.0
    with pytest.raises(ValueError):
        K.KabavikSpec.from_config({**cfg, "architecture": "Other"})
    for path, value in ((("layers", 0, "type"), "unknown"), (("layers", 0, "mixer", "kv_heads"), 4),
                        (("layers", 0, "mixer", "rot", "dims"), 13), (("layers", 0, "mixer", "rot", "dims"), 26),
                        (("layers", 1, "mixer", "rot", "dims"), 10), (("layers", 3, "mixer", "kv_from"), 1),
                        (("layers", 3, "mixer", "kv_from"), 3), (("layers", 6, "mixer", "kv_from"), 3),
                        (("layers", 3, "mixer", "dim"), 8), (("layers", 1, "mlp", "kind"), "other")):
        with pytest.raises(ValueError):
            K.KabavikSpec.from_config(_with(cfg, path, value))
    # what a config leaves out is off: no window, no kept keys, no rotation, no scaling, no token input
    bare = json.loads(json.dumps(cfg))
    del bare["token_side"], bare["layers"][0]["mixer"]["mask"], bare["layers"][0]["mixer"]["rot"]
    del bare["layers"][1]["mixer"]["rot"]["scaling"], bare["layers"][2]["mixer"]["q_temp"]
    sp = K.KabavikSpec.from_config(bare)
    assert sp.side_dim == 0 and (sp.layers[0].window, sp.layers[0].keep_first, sp.layers[0].rot_dims) == (0, 0, 0)
    assert (sp.layers[1].rot_factor, sp.layers[1].rot_original, sp.layers[1].rot_dims) == (0.0, 0.0, 8)
    assert sp.layers[2].q_temp_every == 0 and sp.layers[2].softcap == 4.0
    ex = spec.config_extras()
    assert (ex["arch"], ex["layer_form"], ex["norm_kind"], ex["side_dim"]) == (L.ARCH_KABAVIK, L.FORM_SANDWICH, L.NORM_DYT, 10)
    assert abs(ex["residual_mult"] - 0.6) < 1e-9 and abs(ex["logit_scale"] - 1.7) < 1e-9 and abs(ex["embed_scale"] - 3) < 1e-9
    d0, d1, d2, d3 = (spec.layers[i].desc() for i in range(4))
    assert (d0.mixer, d0.heads, d0.kv_heads, d0.dim, d0.vdim, d0.window, d0.keep_first, d0.rot_dims, d0.qk_norm,
            d0.proj_bias, d0.bare, d0.kv_from, d0.ff, d0.ff_dim) == \
        (L.MIXER_WINDOW_ATTN, 6, 2, 24, 40, 21, 3, 12, 1, 1, 1, -1, L.FF_GEGLU, 72)
    assert (d0.rot_factor, d0.rot_original) == (2.0, 0.0)
    assert (d1.mixer, d1.q_rank, d1.kv_rank, d1.rot_dim, d1.head_gate, d1.window, d1.rot_original, d1.rot_fast) == \
        (L.MIXER_LATENT_ATTN, 0, 40, 8, 1, 19, 64.0, 8.0)
    assert (d2.mixer, d2.qk_norm, d2.window, d2.rot_dims, d2.q_temp_every) == (L.MIXER_WINDOW_ATTN, 2, 0, 0, 7)
    assert abs(d2.softcap - 4.0) < 1e-6 and abs(d2.q_temp_coef - 0.4) < 1e-6
    assert (d3.kv_from, d3.window, d3.keep_first, d3.ff) == (0, 9, 0, L.FF_NONE)


def test_layer_description_matches_the_header(tmp_path):
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "t.c"
    src.write_text('#include "b200q.h"\n#include <stdio.h>\n#include <stddef.h>\n'
                   'int main(void){printf("%zu %zu %zu %zu\\n", sizeof(b200q_layer_desc), offsetof(b200q_layer_desc, '
                   'keep_first), offsetof(b200q_layer_desc, rot_factor), offsetof(b200q_model_config, norm_kind));'
                   'return 0;}\n')
    exe = tmp_path / "t"
    subprocess.run(["gcc", "-std=c99", "-I", os.path.join(root, "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    assert got == [C.sizeof(L.LayerDesc), L.LayerDesc.keep_first.offset, L.LayerDesc.rot_factor.offset,
                   L.ModelConfig.norm_kind.offset]


def test_resolve_model_picks_the_class_by_config(tmp_path):
    from llmq_b200.model import BUILTIN_SPECS, resolve_model
    spec = small_spec()
    sd = checkpoint(spec, 2)
    (tmp_path / "config.json").write_text(json.dumps(spec.to_config()))
    K.save_checkpoint(str(tmp_path / "model.safetensors"), sd)
    got, d = resolve_model(str(tmp_path))
    assert isinstance(got, K.KabavikSpec) and got.layers == spec.layers and d == str(tmp_path)
    assert BUILTIN_SPECS["kabavik-1b"].layered and resolve_model("random:kabavik-1b")[1] is None
    loaded = K.load_checkpoint(str(tmp_path / "model.safetensors"))
    assert set(loaded) == set(sd) and all(torch.equal(loaded[k], sd[k]) for k in sd)
    assert loaded["l0.norm1.alpha"].dim() == 0                           # a scalar travels as a tensor without axes


def test_engine_weights_shapes_and_fusions():
    spec = small_spec()
    sd = checkpoint(spec, 3)
    ew = dict(spec.engine_weights(sd))
    W = spec.width
    assert ew["tok_embed"].shape == (spec.vocab, 7 * 10) and ew["lm_head"] is sd["head"]
    n1 = ew["layers.0.norm1"]
    assert n1.shape == (2 * W + 1,) and n1.dtype == torch.float32
    assert torch.equal(n1[:W], sd["l0.norm1"].float()) and torch.equal(n1[W:2 * W], sd["l0.norm1.b"].float())
    assert float(n1[2 * W]) == float(sd["l0.norm1.alpha"])
    assert ew["final_norm"].shape == (2 * W + 1,)
    l0 = spec.layers[0]
    hd, gd, gv = l0.heads * l0.dim, l0.kv_heads * l0.dim, l0.kv_heads * l0.vdim
    proj, pb = ew["layers.0.mix.proj"], ew["layers.0.mix.proj_b"]
    rows = (hd + gd + gv + 63) // 64 * 64
    assert proj.shape == (rows, W) and pb.shape == (rows,) and pb.dtype == torch.float32
    assert torch.equal(proj[hd:hd + gd], sd["l0.mix.k"]) and torch.equal(pb[hd + gd:hd + gd + gv], sd["l0.mix.v.b"].float())
    assert float(proj[hd + gd + gv:].abs().max()) == 0.0 and float(pb[hd + gd + gv:].abs().max()) == 0.0
    assert ew["layers.0.mix.q_norm"].shape == (hd,) and ew["layers.0.mix.k_norm"].shape == (gd,)
    assert ew["layers.2.mix.q_norm"].shape == (spec.layers[2].dim,)       # per head: one weight row for all heads
    # a layer that reads another's keys projects queries only
    assert ew["layers.3.mix.proj"].shape == ((hd + 63) // 64 * 64, W) and "layers.3.mix.k_norm" not in ew
    assert "layers.3.norm2" not in ew and "layers.3.mlp.gate_up" not in ew and "layers.3.tok.gate" in ew
    l1 = spec.layers[1]
    nq, rp = l1.heads * (l1.dim + l1.rot_dim), l1.kv_rank + l1.rot_dim
    down = ew["layers.1.mix.down"]
    assert down.shape == ((nq + rp + l1.heads + 63) // 64 * 64, W)
    assert torch.equal(down[nq:nq + rp], sd["l1.mix.dkv"]) and torch.equal(down[nq + rp:nq + rp + l1.heads], sd["l1.mix.g"])
    ukt = ew["layers.1.mix.uk_t"]
    assert ukt.shape == (l1.heads * l1.kv_rank, l1.dim)
    assert torch.equal(ukt[l1.kv_rank:2 * l1.kv_rank].T, sd["l1.mix.uk"][l1.dim:2 * l1.dim])
    gu = ew["layers.0.mlp.gate_up"]
    assert gu.shape == (2 * 72, W) and torch.equal(gu[72:], sd["l0.mlp.up"])
    # a feed-forward whose size is a multiple of 128: gate and up rows alternate in blocks of 128
    sp2 = small_spec(layers=[attn2(ff="dense", ff_dim=256)], side_dim=0)
    sd2 = checkpoint(sp2, 4)
    ew2 = dict(sp2.engine_weights(sd2))
    il = ew2["layers.0.mlp.gate_up_il"]
    assert "layers.0.mlp.gate_up" not in ew2 and il.shape == (512, W)
    assert torch.equal(il[:128], sd2["l0.mlp.gate"][:128]) and torch.equal(il[128:256], sd2["l0.mlp.up"][:128])
    assert torch.equal(il[256:384], sd2["l0.mlp.gate"][128:]) and torch.equal(il[384:], sd2["l0.mlp.up"][128:])
    assert spec.weight_bytes_per_token() > 0


def test_rotation_frequencies_match_the_plain_form():
    lib = L.load()
    cases = [dict(dims=12, base=5000.0), dict(dims=20, base=80000.0, scaling={"factor": 2.5}),
             dict(dims=8, base=100.0, scaling={"factor": 3.0, "original": 64.0, "fast": 8.0, "slow": 1.0}),
             dict(dims=64, base=20000.0, scaling={"factor": 4.0, "original": 4096.0, "fast": 16.0, "slow": 2.0}),
             dict(dims=6, base=50.0, scaling={"factor": 1.5, "original": 16.0, "fast": 1.0, "slow": 1.0})]  # lo == hi
    for rot in cases:
        sc = rot.get("scaling") or {}
        if "original" in sc:
            want, mag = O.yarn_frequencies(rot)
        else:
            want, mag = O.linear_frequencies(rot), 1.0
        n = rot["dims"] // 2
        out = (C.c_double * n)()
        m = C.c_float()
        L.check(lib.b200q_rot_frequencies(rot["dims"], rot["base"], sc.get("factor", 0.0), sc.get("original", 0.0),
                                          sc.get("fast", 0.0), sc.get("slow", 0.0), C.addressof(out), C.addressof(m)))
        assert max(abs(out[i] - float(want[i])) / float(want[i]) for i in range(n)) < 1e-14
        assert abs(m.value - mag) < 1e-7
    assert lib.b200q_rot_frequencies(7, 100.0, 0.0, 0.0, 0.0, 0.0, None, None) != 0


def _changed(cfg, sd, n, at, vocab=50):
    a = tokens(n, vocab, 1)
    b = list(a)
    b[at] = (b[at] + 1) % vocab
    la, lb = O.forward(cfg, sd, a), O.forward(cfg, sd, b)
    return [i for i in range(n) if float((la[i] - lb[i]).abs().max()) > 1e-9]


def test_oracle_windows_kept_keys_and_borrowed_keys():
    def one(layer, **kw):
        spec = small_spec(width=64, vocab=50, layers=[layer], side_dim=0, **kw)
        return spec.to_config(), checkpoint(spec, 4)
    cfg, sd = one(attn(window=9, keep_first=3, **DENSE))
    assert _changed(cfg, sd, 40, 10) == list(range(10, 19))              # 10 .. 10 + 9 - 1 and no other
    assert _changed(cfg, sd, 40, 2) == list(range(2, 40))                # a kept key is seen for ever
    assert _changed(cfg, sd, 40, 3) == list(range(3, 12))                # the next one is not
    cfg, sd = one(latent(window=7))
    assert _changed(cfg, sd, 30, 5) == list(range(5, 12))
    cfg, sd = one(attn2())
    assert _changed(cfg, sd, 30, 5) == list(range(5, 30))
    # a reader of layer 0's keys under its own mask: those keys are made from the embedding alone, so a changed
    # token moves key 8 and nothing else, and the reader's window of 5 carries it 4 tokens on (keys of its own,
    # made from layer 0's output, would have carried it one further)
    spec = small_spec(width=64, vocab=50, layers=[attn(window=2, keep_first=0), attn(window=5, keep_first=0, kv_from=0)],
                      side_dim=0)
    sd = checkpoint(spec, 5)
    assert _changed(spec.to_config(), sd, 30, 8) == list(range(8, 13))
    # the per-layer token input reads the token itself: nothing else moves
    spec = small_spec(width=64, vocab=50, layers=[attn(window=1, keep_first=0)], side_dim=6)
    assert _changed(spec.to_config(), checkpoint(spec, 6), 20, 7) == [7]


def test_oracle_rotations_depend_on_the_distance_only():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(12, 2, 10, generator=g, dtype=torch.float64)
    x[:] = x[0]
    f = O.linear_frequencies({"dims": 6, "base": 100.0, "scaling": {"factor": 2.0}})
    for turn in (O.turn_half_split, O.turn_interleaved):
        r = turn(x, f)
        assert torch.allclose(r[..., 6:], x[..., 6:]) and torch.allclose(r[0], x[0])
        dots = torch.einsum("ihd,jhd->hij", r, r)
        for d in range(1, 5):
            diag = torch.diagonal(dots, offset=d, dim1=1, dim2=2)
            assert float((diag - diag[:, :1]).abs().max()) < 1e-9
        assert float((dots[:, 0, 1] - dots[:, 0, 2]).abs().max()) > 1e-3
    # pairs: half-split turns (0, 3), interleaved turns (0, 1)
    e = torch.zeros(2, 1, 6, dtype=torch.float64)
    e[:, 0, 0] = 1.0
    assert float(O.turn_half_split(e, f)[1, 0, 3].abs()) > 1e-3 and float(O.turn_half_split(e, f)[1, 0, 1].abs()) == 0.0
    assert float(O.turn_interleaved(e, f)[1, 0, 1].abs()) > 1e-3 and float(O.turn_interleaved(e, f)[1, 0, 3].abs()) == 0.0
    # the grown sine and cosine scale the turned part only
    r2 = O.turn_interleaved(x, f, 1.5)
    assert torch.allclose(r2[..., :6], 1.5 * O.turn_interleaved(x, f)[..., :6]) and torch.allclose(r2[..., 6:], x[..., 6:])


def test_oracle_query_temperature_and_soft_cap():
    p = torch.arange(30, dtype=torch.float64)
    want = 1.0 + 0.4 * torch.log(torch.floor((p + 1.0) / 7.0) + 1.0)
    assert float(want[5]) == 1.0 and abs(float(want[6]) - (1 + 0.4 * math.log(2.0))) < 1e-12
    q = torch.ones(1, 1, 4, dtype=torch.float64)
    k = torch.ones(1, 1, 4, dtype=torch.float64) * 100.0
    v = torch.ones(1, 1, 2, dtype=torch.float64)
    out = O.softmax_attention(q, k, v, O.visible(1), 1.0, softcap=5.0)
    assert torch.allclose(out, v)
