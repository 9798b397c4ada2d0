"""CPU tests of the Paluzen host code: the config reader, the registry, the expansion of repeated layers into
layer runs, the mapping of checkpoint tensors to engine weights, and the oracle's own consistency (causality,
window confinement, rotation that depends on the distance only, recurrences that can be cut and continued,
routing that respects groups and identity experts)."""
import json

import pytest
import torch

from llmq_b200 import lib as L
from llmq_b200 import paluzen as P
from oracle import paluzen as O
from tests.paluzen_util import DENSE, MOE, checkpoint, lightning, parallel, small_spec, tokens


def test_config_round_trip_and_layer_runs():
    spec = small_spec()
    cfg = json.loads(json.dumps(spec.to_config()))
    back = P.PaluzenSpec.from_config(cfg)
    assert back.layers == spec.layers and back.base_layers == spec.base_layers
    assert (back.width, back.vocab, back.rms_eps, back.logit_softcap, back.loop) == (96, 211, 1e-5, 20.0, (1, 3, 3))
    # layers 1 and 2 run three times between layer 0 and layers 3, 4; every pass begins with the re-injection
    assert [(ly.src, ly.inject) for ly in back.layers] == [(0, False), (1, True), (2, False), (1, True), (2, False),
                                                          (1, True), (2, False), (3, False), (4, False)]
    assert O.layer_runs(cfg) == [(ly.src, ly.inject) for ly in back.layers]
    assert back.base_layers[3].ff is None and back.base_layers[3].window == 0 and back.base_layers[4].rot_dims == 0
    with pytest.raises(ValueError):
        P.PaluzenSpec.from_config({**cfg, "architecture": "Other"})
    for path, value in ((("layers", 0, "type"), "unknown"), (("layers", 1, "mixer", "left", "kv_heads"), 4),
                        (("layers", 1, "mixer", "left", "rot", "dims"), 13), (("layers", 0, "mixer", "decay"), [0.5]),
                        (("layers", 1, "mlp", "router", "groups", "count"), 3), (("loop", "stop"), 9),
                        (("layers", 1, "mlp", "kind"), "other")):
        bad = json.loads(json.dumps(cfg))
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ValueError):
            P.PaluzenSpec.from_config(bad)
    nl = json.loads(json.dumps(cfg))
    del nl["loop"]
    assert [ly.src for ly in P.PaluzenSpec.from_config(nl).layers] == [0, 1, 2, 3, 4]
    no_rank = json.loads(json.dumps(cfg))
    del no_rank["layers"][1]["mixer"]["right"]["rank"]
    with pytest.raises(ValueError):
        P.PaluzenSpec.from_config(no_rank)                              # ... unless the tensor's shape gives it
    assert P.PaluzenSpec.from_config(no_rank, {"l1.mix.right.w1": (5, 96)}).layers == spec.layers
    ex = spec.config_extras()
    assert (ex["arch"], ex["layer_form"], ex["token_shift"], ex["logit_softcap"]) == (L.ARCH_PALUZEN, L.FORM_PRENORM, 1, 20.0)
    d0, d1 = spec.layers[0].desc(), spec.layers[1].desc()
    assert (d0.mixer, d0.heads, d0.dim, d0.vdim, d0.ff, d0.ff_dim, d0.inject, d0.side_mixer) == \
        (L.MIXER_LIGHTNING, 3, 16, 24, L.FF_RELU2, 120, 0, 0)
    assert (d1.mixer, d1.kv_heads, d1.window, d1.rot_dims, d1.side_mixer, d1.side_heads, d1.side_dim, d1.side_decay_rank,
            d1.ff, d1.n_experts, d1.n_identity, d1.n_groups, d1.keep_groups, d1.inject) == \
        (L.MIXER_WINDOW_ATTN, 2, 21, 12, L.MIXER_DECAY_MIX, 3, 16, 5, L.FF_MOE_GROUPED, 6, 2, 4, 2, 1)
    assert abs(d1.mix_scale - 1.3) < 1e-6 and abs(d1.side_scale - 0.7) < 1e-6


def test_resolve_model_picks_the_class_by_config(tmp_path):
    from llmq_b200.model import BUILTIN_SPECS, resolve_model
    spec = small_spec()
    sd = checkpoint(spec, 2)
    (tmp_path / "config.json").write_text(json.dumps(spec.to_config()))
    P.save_checkpoint(str(tmp_path / "model.safetensors"), sd)
    got, d = resolve_model(str(tmp_path))
    assert isinstance(got, P.PaluzenSpec) and got.layers == spec.layers and d == str(tmp_path)
    assert BUILTIN_SPECS["paluzen-1b"].layered and resolve_model("random:paluzen-1b")[1] is None
    loaded = P.load_checkpoint(str(tmp_path / "model.safetensors"))
    assert set(loaded) == set(sd) and all(torch.equal(loaded[k], sd[k]) for k in sd)


def test_engine_weights_shapes_fusions_and_sharing():
    spec = small_spec()
    sd = checkpoint(spec, 3)
    pairs = list(spec.engine_weights(sd))
    ew = dict(pairs)
    W = spec.width
    assert ew["lm_head"] is ew["embed"]                                  # tied: one upload
    l0, l1 = spec.base_layers[0], spec.base_layers[1]
    assert ew["layers.0.mix.proj"].shape == (2 * l0.heads * l0.dim + 2 * l0.heads * l0.vdim, W)
    assert ew["layers.0.mix.decay"].dtype == torch.float32 and ew["layers.0.mix.decay"].tolist() == \
        torch.tensor(l0.decay, dtype=torch.float64).float().tolist()
    n = l1.heads * l1.dim + l1.kv_heads * (l1.dim + l1.vdim) + l1.heads
    proj = ew["layers.1.mix.proj"]
    assert proj.shape == ((n + 63) // 64 * 64, W) and float(proj[n:].abs().max()) == 0.0
    assert torch.equal(proj[l1.heads * l1.dim + l1.kv_heads * (l1.dim + l1.vdim):n], sd["l1.mix.left.g"])
    assert ew["layers.1.side.mu"].shape == (5 * W,) and torch.equal(ew["layers.1.side.mu"][4 * W:], sd["l1.mix.right.mu.w"])
    rd = l1.r_heads * l1.r_dim
    assert ew["layers.1.side.proj"].shape == (4 * rd, W) and torch.equal(ew["layers.1.side.proj"][rd:2 * rd], sd["l1.mix.right.k"])
    assert ew["layers.1.side.bonus"].shape == (rd,)
    assert ew["layers.1.mlp.router"].shape == (8, W) and ew["layers.1.mlp.experts_up"].shape == (6 * 40, W)
    assert ew["layers.1.mlp.experts_down"].shape == (6 * W, 40)
    # a pass begins at runs 1, 3, 5 with the same matrix; runs of one layer share every tensor object
    assert ew["layers.1.inject"] is ew["layers.3.inject"] is ew["layers.5.inject"] and "layers.2.inject" not in ew
    for name in ("mix.proj", "side.proj", "mlp.experts_up", "norm1", "shift"):
        assert ew[f"layers.1.{name}"] is ew[f"layers.3.{name}"] is ew[f"layers.5.{name}"]
    assert "layers.7.norm2" not in ew and "layers.7.mlp.up" not in ew    # a layer without feed-forward
    assert len({id(t) for _, t in pairs}) < len(pairs)
    assert spec.weight_bytes_per_token() > 0 and spec.weight_bytes_per_token(batch=64) >= spec.weight_bytes_per_token()


def test_oracle_is_causal_and_confined_to_the_window():
    layers = [parallel(window=9, right_scale=0.0, **DENSE)]             # attention alone: the decay mix is switched off
    spec = small_spec(width=64, vocab=50, layers=layers, loop=None)
    sd = checkpoint(spec, 4)
    sd["l0.shift"].zero_()                                               # no token shift: the window is the only reach
    cfg = spec.to_config()
    a = tokens(40, 50, 1)
    b = list(a)
    b[10] = (b[10] + 1) % 50
    la, lb = O.forward(cfg, sd, a), O.forward(cfg, sd, b)
    changed = [i for i in range(40) if float((la[i] - lb[i]).abs().max()) > 1e-9]
    assert changed == list(range(10, 19))                               # positions 10 .. 10 + 9 - 1 and no other
    sd["l0.shift"].fill_(0.5)                                            # with the shift, the token before the window counts
    la, lb = O.forward(cfg, sd, a), O.forward(cfg, sd, b)
    changed = [i for i in range(40) if float((la[i] - lb[i]).abs().max()) > 1e-9]
    assert changed == list(range(10, 20))


def test_oracle_rotation_depends_on_the_distance_only():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(12, 2, 10, generator=g, dtype=torch.float64)
    x[:] = x[0]                                                          # the same vector at every position
    r = O.rotate_half_split(x, 6, 100.0)
    assert torch.allclose(r[..., 6:], x[..., 6:]) and torch.allclose(r[0], x[0])
    dots = torch.einsum("ihd,jhd->hij", r, r)
    for d in range(1, 5):
        diag = torch.diagonal(dots, offset=d, dim1=1, dim2=2)
        assert float((diag - diag[:, :1]).abs().max()) < 1e-9
    assert float((dots[:, 0, 1] - dots[:, 0, 2]).abs().max()) > 1e-3


def test_oracle_recurrences_can_be_cut_and_states_start_at_zero():
    layers = [lightning(**DENSE), parallel(left_scale=0.0, **MOE)]
    spec = small_spec(width=64, vocab=50, layers=layers, loop=(0, 2, 2))
    sd = checkpoint(spec, 6)
    cfg = spec.to_config()
    t = tokens(30, 50, 2)
    whole = O.forward(cfg, sd, t)
    assert float((O.forward(cfg, sd, t[:17]) - whole[:17]).abs().max()) < 1e-9    # a prefix never sees what follows
    other = O.forward(cfg, sd, t[5:])
    assert float((other[0] - whole[5]).abs().max()) > 1e-6                       # ... and the past matters


def test_oracle_routing_groups_identity_and_weights():
    g = torch.Generator().manual_seed(1)
    h = torch.randn(50, 16, generator=g, dtype=torch.float64)
    r = {"experts": 6, "identity": 2, "top": 3, "groups": {"count": 4, "keep": 2}}
    w = {"m.router": torch.randn(8, 16, generator=g, dtype=torch.float64),
         "m.correction": torch.randn(8, generator=g, dtype=torch.float64) * 0.3}
    idx, wt = O.route(h, w, "m.", r)
    s = torch.softmax(h @ w["m.router"].T, -1)
    for t in range(50):
        groups = {int(e) // 2 for e in idx[t]}
        assert len(groups) <= 2 and len(set(idx[t].tolist())) == 3
        assert abs(float(wt[t].sum()) - 1.0) < 1e-12
        assert torch.allclose(wt[t], s[t, idx[t]] / s[t, idx[t]].sum())           # weights ignore the correction
    assert int((idx >= 6).sum()) > 0                                              # identity experts are chosen too
    for e in range(6):
        w[f"m.e{e}.up"] = torch.zeros(4, 16, dtype=torch.float64)
        w[f"m.e{e}.down"] = torch.zeros(16, 4, dtype=torch.float64)
    out = O.feed_forward(h, w, "m.", {"kind": "moe", "router": r, "expert": {"ff": 4}})
    share = (wt * (idx >= 6)).sum(-1, keepdim=True)                               # with silent experts only identity speaks
    assert torch.allclose(out, share * h)
