"""GPU tests of the Kabavik path: the engine (scheduler, paged caches, kernels) against oracle/kabavik.py — a plain
fp64 restatement that recomputes every position from the tokens, with no cache and no batching.  The
configurations are small, differ from one another in every size, and are drawn here; the fp32 engine is held to a
tight bound, the bf16 engine to a rounding-sized one."""
import json
import math

import numpy as np
import pytest
import torch

from oracle import kabavik as O
from tests.kabavik_util import DENSE, attn, attn2, checkpoint, latent, rel_err, small_spec, tokens

pytestmark = pytest.mark.gpu
F32_TOL, BF16_TOL = 2e-4, 6e-2


def build(spec, sd, dtype=torch.float32, max_tokens=512, max_seqs=4, num_blocks=None):
    from llmq_b200.model import BLOCK_SIZE, Engine, NativeModel

    nb = num_blocks or (max_tokens // BLOCK_SIZE + max_seqs)
    model = NativeModel(spec, spec.engine_weights(sd), max_tokens=max_tokens, max_seqs=max_seqs,
                        max_model_len=max_tokens, num_blocks=nb, dtype=dtype, max_logit_rows=max_tokens)
    eng = Engine(model, max_num_seqs=max_seqs, max_num_batched_tokens=max_tokens, max_model_len=model.max_model_len)
    return model, eng


def oracle_logits(spec, sd, toks):
    return O.forward(spec.to_config(), sd, toks, torch.float64).numpy()


def replay_cut(eng, rid, toks, cuts):
    """feed toks to request rid in portions of the given sizes (the rest one by one); logits of every place"""
    out, at, cuts = [], 0, list(cuts)
    while at < len(toks):
        n = min(cuts.pop(0) if cuts else 1, len(toks) - at)
        out.append(eng.step_replay([(rid, toks[at:at + n], list(range(n)))]))
        at += n
    return np.concatenate(out)


def check_close(got, want, dtype, what=""):
    err = rel_err(got, want)
    assert err < (F32_TOL if dtype == torch.float32 else BF16_TOL), f"{what}: {err}"


def _ops():
    from llmq_b200 import lib as L
    return L, L.load()


# ---- every mechanism alone: a one-layer model around it --------------------------------------------------
ONE_LAYER = {
    "attention": [attn()],
    "attention_no_kept_keys_whole_head_turned": [attn(heads=3, kv_heads=3, dim=16, vdim=16, window=7, keep_first=0,
                                                      rot_dims=16, rot_factor=0.0)],
    "attention_more_kept_keys_than_window": [attn(heads=2, kv_heads=1, dim=40, vdim=8, window=4, keep_first=11)],
    "attention_one_key_window": [attn(window=1, keep_first=1, rot_dims=24)],
    "attention_every_key_no_rotation": [attn(heads=2, kv_heads=1, dim=72, vdim=24, window=0, keep_first=0, rot_dims=0)],
    "attention_many_heads_per_key": [attn(heads=18, kv_heads=2, dim=8, vdim=8, window=7, keep_first=2, rot_dims=2)],
    "attention_borrowed_keys": [attn(**DENSE), attn(window=6, keep_first=2, kv_from=0)],
    "attention_tile_sizes_kept_keys": [attn(heads=4, kv_heads=2, dim=64, vdim=64, window=20, keep_first=5, rot_dims=32)],
    "latent": [latent()],
    "latent_every_key_plain_frequencies": [latent(heads=2, dim=24, rot_dim=4, vdim=8, kv_rank=24, window=0, factor=0.0,
                                                  original=0.0)],
    "latent_linear_scaling_one_head": [latent(heads=1, dim=8, rot_dim=16, vdim=40, kv_rank=16, window=3, original=0.0)],
    "latent_tile_sizes": [latent(heads=5, dim=32, rot_dim=64, vdim=32, kv_rank=64, window=18)],
    "attention_2": [attn2()],
    "attention_2_temperature_every_token_no_cap": [attn2(heads=3, kv_heads=3, dim=16, vdim=16, softcap=0.0, every=1)],
    "attention_2_no_temperature_tight_cap": [attn2(heads=2, kv_heads=1, dim=24, vdim=40, softcap=0.5, every=0)],
    "attention_2_tile_sizes": [attn2(heads=4, kv_heads=1, dim=64, vdim=128, softcap=3.0, every=5)],
    "dense_and_token_input": [attn2(heads=1, kv_heads=1, dim=8, vdim=8, **DENSE)],
    "dense_gate_and_up_in_blocks": [attn2(heads=1, kv_heads=1, dim=8, vdim=8, ff="dense", ff_dim=256)],
}


@pytest.mark.parametrize("name", sorted(ONE_LAYER))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mechanism_alone(cuda, name, dtype):
    side = 0 if "attention" in name and "borrowed" not in name else 6
    spec = small_spec(width=80, vocab=97, layers=ONE_LAYER[name], side_dim=side,
                      mult=1.0 if "latent" in name else 0.6)
    sd = checkpoint(spec, seed=11)
    toks = tokens(45, spec.vocab, 5)
    model, eng = build(spec, sd, dtype)
    tap = torch.zeros(spec.n_layers, len(toks), spec.width, device=cuda)
    model.set_layer_tap(tap)
    got = eng.step_replay([(1, toks, list(range(len(toks))))])
    model.set_layer_tap(None)
    stream = []
    want = O.forward(spec.to_config(), sd, toks, torch.float64, stream)
    assert len(stream) == spec.n_layers
    check_close(tap.cpu().numpy()[-1], stream[-1].numpy(), dtype, name)
    check_close(got, want.numpy(), dtype, name)
    # the same tokens one by one through the cache
    again = replay_cut(eng, 2, toks, [])
    check_close(again, want.numpy(), dtype, name + " token by token")
    eng.close()
    model.close()


# ---- op level: made-up inputs that make a fault show ----------------------------------------------------
def _window_op(cuda, qs, keys, vals, window, keep_first, softcap, dtype, portions=None, block_size=16, shuffle_seed=0,
               companion=0):
    """run b200q_window_attn_ex for one sequence of T tokens whose keys and values lie in a paged cache with
    shuffled pages (unused places hold garbage).  portions: the token counts of successive steps (None = all at
    once); companion > 0 puts another sequence's single token first in every step."""
    L, lib = _ops()
    T, H, D = qs.shape
    G, V = keys.shape[1], vals.shape[2]
    tdt = torch.float32 if dtype == L.DTYPE_F32 else torch.bfloat16
    nb = (T + block_size - 1) // block_size
    pages = np.random.default_rng(shuffle_seed).permutation(nb + 4)[:nb + 1].astype(np.int32)
    cache = torch.full(((nb + 4) * block_size, G * (D + V)), 1e4, dtype=tdt, device=cuda)
    for t in range(T):
        cache[int(pages[t // block_size]) * block_size + t % block_size] = torch.cat(
            [keys[t].reshape(-1), vals[t].reshape(-1)]).to(tdt)
    other = int(pages[nb]) * block_size                        # the companion's only page: one key, value 1
    cache[other] = torch.cat([torch.zeros(G * D), torch.ones(G * V)]).to(tdt)
    bt = torch.zeros(2, nb, dtype=torch.int32)
    bt[0, 0] = int(pages[nb])
    bt[1] = torch.tensor(pages[:nb])
    bt = bt.to(cuda).contiguous()
    out = torch.zeros(T, H * V, dtype=tdt, device=cuda)
    qd = qs.to(cuda).float().contiguous()
    at = 0
    for n in (portions or [T]):
        n = min(n, T - at)
        if n <= 0:
            break
        c = 1 if companion else 0
        rows = c + n
        q_step = torch.zeros(rows, H, D, device=cuda)
        q_step[c:] = qd[at:at + n]
        row_seq = torch.tensor([0] * c + [1] * n, dtype=torch.int32, device=cuda)
        pos = torch.tensor([0] * c + list(range(at, at + n)), dtype=torch.int32, device=cuda)
        desc = torch.tensor(([[0, 1, 0, 0]] if c else []) + [[c, n, at, 1]], dtype=torch.int32, device=cuda)
        if not c:                                              # without a companion the sequence is row 0
            row_seq.zero_()
            desc[0, 3] = 0
        table = bt if c else bt[1:].contiguous()
        o_step = torch.zeros(rows, H * V, dtype=tdt, device=cuda)
        L.check(lib.b200q_window_attn_ex(q_step.data_ptr(), cache.data_ptr(), table.data_ptr(), nb, row_seq.data_ptr(),
                                         pos.data_ptr(), desc.data_ptr(), 1 + c, rows, H, G, D, V, block_size, window,
                                         keep_first, softcap, None, 0, o_step.data_ptr(), dtype, None))
        torch.cuda.synchronize()
        if c:
            assert torch.allclose(o_step[0].float(), torch.ones(H * V, device=cuda)), "the companion saw foreign keys"
        out[at:at + n] = o_step[c:]
        at += n
    return out.float().cpu().reshape(T, H, V)


def _standout(T, H, G, D, V, marks, seed):
    """small random queries and keys; at every marked position the key points along the (shared) query direction
    of its group and is large, so whoever sees it is dominated by it; the value of position j is j in every
    channel, so an output row names the keys it saw"""
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(G, D, generator=g)
    u = u / u.norm(dim=-1, keepdim=True)
    qs = 0.05 * torch.randn(T, H, D, generator=g) + 6.0 * u.repeat_interleave(H // G, 0)[None]
    keys = 0.3 * torch.randn(T, G, D, generator=g)
    for j in marks:
        keys[j] = 4.0 * u
    vals = torch.arange(T, dtype=torch.float32)[:, None, None].expand(T, G, V).clone()
    return qs, keys, vals


def _window_want(qs, keys, vals, window, keep_first, softcap):
    T, H, D = qs.shape
    G = keys.shape[1]
    out = torch.zeros(T, H, vals.shape[2], dtype=torch.float64)
    for h in range(H):
        for i in range(T):
            see = [j for j in range(i + 1) if not window or i - j < window or j < keep_first]
            s = keys[see, h // (H // G)].double() @ qs[i, h].double()
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            out[i, h] = torch.softmax(s, 0) @ vals[see, h // (H // G)].double()
    return out


WINDOW_CASES = [
    # (T, H, G, D, V, window, kept first keys, soft cap, marked keys)
    (150, 4, 2, 24, 40, 21, 3, 0.0, [2, 3, 20, 24, 47, 63, 64, 100]),       # the last kept key and the first that is not
    (200, 2, 1, 64, 64, 64, 6, 0.0, [5, 6, 15, 16, 63, 64, 127, 128, 135]),  # tile sizes: a window of one tile
    (300, 4, 2, 128, 128, 80, 1, 0.0, [0, 1, 79, 80, 83, 159, 160, 200]),    # head size 128, one kept key
    (260, 3, 3, 16, 8, 0, 0, 8.0, [5]),                                      # every earlier key, capped: one far back
    (230, 2, 2, 64, 128, 30, 70, 0.0, [63, 64, 69, 70, 99, 100, 130]),       # more kept keys than a tile or the window
    (90, 16, 1, 64, 128, 17, 2, 12.0, [0, 1, 2, 16, 17, 33, 50]),            # sixteen heads on one key head, capped
    (70, 24, 1, 128, 64, 19, 20, 0.0, [0, 18, 19, 20, 40]),                  # kept keys reach past the first window
    (140, 2, 1, 64, 64, 0, 0, 5.0, [7, 64, 100]),                            # tile sizes, every key, tightly capped
]


@pytest.mark.parametrize("case", range(len(WINDOW_CASES)))
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("how", ["whole", "portions", "single"])
def test_window_edges_kept_keys_pages_and_far_keys(cuda, case, dtype, how):
    """a key that dominates whoever sees it: it is seen up to window - 1 tokens later and not one more — unless it
    is one of the first keys, which stay — at page borders and tile borders alike, in a whole prompt, in portions
    of 1 to 70 tokens beside another sequence, and token by token"""
    L, _ = _ops()
    T, H, G, D, V, window, keep, cap, marks = WINDOW_CASES[case]
    qs, keys, vals = _standout(T, H, G, D, V, marks, seed=case)
    dt = L.DTYPE_F32 if dtype == "f32" else L.DTYPE_BF16
    if dtype == "bf16":                                        # what the cache can hold
        keys, vals = keys.bfloat16().float(), vals.bfloat16().float()
    want = _window_want(qs, keys, vals, window, keep, cap)
    portions = {"whole": None, "portions": [1, 2, 16, 3, 70, 17, 1, 1, 33, 64, 5] * 4, "single": [1] * T}[how]
    got = _window_op(cuda, qs, keys, vals, window, keep, cap, dt, portions, shuffle_seed=case, companion=how != "whole")
    tol = 2e-4 if dtype == "f32" else 2e-2
    assert float((got.double() - want).abs().max()) < tol * T
    # the marks do what they are meant to: the marked keys in sight share the weight, so an output row is the mean
    # of their positions — a key one token past the window is out of it, a kept first key never is
    if not cap:
        for i in range(T):
            seen = [m for m in marks if m <= i and (not window or i - m < window or m < keep)]
            if seen:
                assert abs(float(want[i, 0, 0]) - sum(seen) / len(seen)) < 0.5


def test_sums_norms_and_gated_units(cuda):
    """the elementwise kernels of the sandwich form against their formulas, both dtypes, a width that is and one
    that is not a multiple of four"""
    L, lib = _ops()
    g = torch.Generator().manual_seed(1)
    for W, T in ((52, 9), (37, 5)):
        x = torch.randn(T, W, generator=g) * 2
        y = torch.randn(T, W, generator=g) * 3
        bias = torch.randn(W, generator=g)
        dyt = lambda: torch.cat([torch.rand(W, generator=g) + 0.5, torch.randn(W, generator=g) * 0.1,
                                 torch.rand(1, generator=g) + 0.3])
        wa, wb, wr = dyt(), dyt(), torch.rand(W, generator=g) + 0.5

        def norm(kind, w, v):
            if kind == L.NORM_DYT:
                return torch.tanh(w[2 * W] * v) * w[:W] + w[W:2 * W]
            if kind == L.NORM_RMS:
                return v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5) * w[:W]
            return v

        for dtype, tdt, tol in ((L.DTYPE_F32, torch.float32, 1e-5), (L.DTYPE_BF16, torch.bfloat16, 2e-2)):
            yq = y.to(tdt).double()
            for post, pw in ((L.NORM_DYT, wa), (L.NORM_RMS, wr)):
                for nxt, nw in ((L.NORM_DYT, wb), (L.NORM_RMS, wr), (L.NORM_CAST, None), (L.NORM_NONE, None)):
                    for b in (None, bias):
                        xd, yd = x.to(cuda).clone(), y.to(cuda).to(tdt).contiguous()
                        out = torch.full((T, W), 7.0, dtype=tdt, device=cuda)
                        pwd, nwd = pw.to(cuda), nw.to(cuda) if nw is not None else None
                        bd = b.to(cuda) if b is not None else None
                        L.check(lib.b200q_sandwich_add(xd.data_ptr(), yd.data_ptr(), bd.data_ptr() if b is not None else None,
                                                       post, pwd.data_ptr(), 0.6, nxt, nwd.data_ptr() if nw is not None else None,
                                                       out.data_ptr(), T, W, 1e-5, dtype, None))
                        torch.cuda.synchronize()
                        xw = x.double() + 0.6 * norm(post, pw.double(), yq + (b.double() if b is not None else 0.0))
                        assert float((xd.cpu().double() - xw).abs().max()) < 1e-5
                        if nxt == L.NORM_NONE:
                            assert float(out.float().min()) == 7.0
                        else:
                            assert float((out.cpu().double() - norm(nxt, nw.double() if nw is not None else None, xw)).abs().max()) < tol
            rows = torch.tensor([3, 0, 3], dtype=torch.int32, device=cuda)
            for kind, w in ((L.NORM_DYT, wa), (L.NORM_RMS, wr), (L.NORM_CAST, None)):
                out = torch.zeros(3, W, dtype=tdt, device=cuda)
                wd = w.to(cuda) if w is not None else None
                xd = x.to(cuda)
                L.check(lib.b200q_row_norm(xd.data_ptr(), rows.data_ptr(), kind, wd.data_ptr() if w is not None else None,
                                           out.data_ptr(), 3, W, 1e-5, dtype, None))
                torch.cuda.synchronize()
                assert float((out.cpu().double() - norm(kind, w.double() if w is not None else None, x.double())[[3, 0, 3]]).abs().max()) < tol
            F = W - 1
            gu = torch.randn(T, 2 * F, generator=g).to(tdt)
            out = torch.zeros(T, F, dtype=tdt, device=cuda)
            gud = gu.to(cuda)                                   # every device buffer outlives the launch that reads it
            L.check(lib.b200q_gelu_glu(gud.data_ptr(), out.data_ptr(), T, F, dtype, None))
            torch.cuda.synchronize()
            assert float((out.cpu().double() - O.gelu_tanh(gu[:, :F].double()) * gu[:, F:].double()).abs().max()) < tol * 4
            # gate and up interleaved in blocks of 8 columns
            FB = 48
            gb = torch.randn(T, 2 * FB, generator=g).to(tdt)
            out = torch.zeros(T, FB, dtype=tdt, device=cuda)
            gbd = gb.to(cuda)
            L.check(lib.b200q_gelu_glu_ex(gbd.data_ptr(), out.data_ptr(), T, FB, 8, dtype, None))
            torch.cuda.synchronize()
            blocks = gb.double().view(T, FB // 8, 2, 8)
            want = (O.gelu_tanh(blocks[:, :, 0]) * blocks[:, :, 1]).reshape(T, FB)
            assert float((out.cpu().double() - want).abs().max()) < tol * 4
            assert lib.b200q_gelu_glu_ex(gbd.data_ptr(), out.data_ptr(), T, FB, 5, dtype, None) != 0
            # the per-layer token input's gate: columns 5 .. 5 + D of the token's table row; an id below zero names
            # a token that the step before sampled
            D, V = 6, 11
            table = torch.randn(V, 20, generator=g).to(tdt)
            gate = torch.randn(T, D + 2, generator=g).to(tdt)
            ids = torch.tensor([(3 * t) % V for t in range(T)], dtype=torch.int32)
            ids[2] = -1 - 1
            prev = torch.tensor([4, 9], dtype=torch.int32, device=cuda)
            out = torch.zeros(T, D, dtype=tdt, device=cuda)
            gd, idd, td = gate.to(cuda), ids.to(cuda), table.to(cuda)
            L.check(lib.b200q_token_side_gate(gd.data_ptr(), D + 2, idd.data_ptr(), prev.data_ptr(), td.data_ptr(), 20, 5,
                                              out.data_ptr(), T, D, dtype, None))
            torch.cuda.synchronize()
            real = ids.clone().long()
            real[2] = 9
            want = O.gelu_tanh(gate[:, :D].double()) * table[real][:, 5:5 + D].double()
            assert float((out.cpu().double() - want).abs().max()) < tol * 4
    v = torch.arange(10, dtype=torch.float32, device=cuda)
    L.check(lib.b200q_scale_f32(v.data_ptr(), 10, 2.5, None))
    torch.cuda.synchronize()
    assert v.cpu().tolist() == [2.5 * i for i in range(10)]


def test_query_and_key_preparation(cuda):
    """biases, the two query / key norms, scaled frequencies with grown sine and cosine, the query temperature at
    positions on both sides of its steps, and a layer that writes no keys — against the plain forms"""
    L, lib = _ops()
    g = torch.Generator().manual_seed(2)
    H, G, D, V, T = 4, 2, 12, 6, 7
    HD, GD, GV = H * D, G * D, G * V
    ld = HD + GD + GV + 3
    proj = torch.randn(T, ld, generator=g)
    bias = torch.randn(ld, generator=g) * 0.3
    pos = torch.tensor([0, 5, 6, 13, 14, 200, 1000], dtype=torch.int32)
    slots = torch.tensor([9, 3, 4, -1, 0, 7, 8], dtype=torch.int32)
    rot = {"dims": 8, "base": 50.0, "scaling": {"factor": 2.0}}
    freq = O.linear_frequencies(rot)
    for qk_norm, own, every, mag in ((1, True, 7, 1.0), (2, True, 0, 1.3), (2, False, 1, 1.0), (0, True, 3, 1.0)):
        wq = torch.rand(HD if qk_norm == 1 else D, generator=g) + 0.5
        wk = torch.rand(GD if qk_norm == 1 else D, generator=g) + 0.5
        q = (proj[:, :HD] + bias[:HD]).double()
        k = (proj[:, HD:HD + GD] + bias[HD:HD + GD]).double()
        v = (proj[:, HD + GD:HD + GD + GV] + bias[HD + GD:HD + GD + GV]).double()
        if qk_norm == 1:
            q, k = O.rms(q, 1e-5) * wq.double(), O.rms(k, 1e-5) * wk.double()
        q, k = q.view(T, H, D), k.view(T, G, D)
        if qk_norm == 2:
            q, k = O.rms(q, 1e-5) * wq.double(), O.rms(k, 1e-5) * wk.double()

        def turn(x):
            a = pos.double()[:, None] * freq[None, :]
            c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
            u, w = x[..., :4], x[..., 4:8]
            return torch.cat([u * c - w * s, w * c + u * s, x[..., 8:]], -1)

        temp = 1.0 + 0.4 * torch.log(torch.floor((pos.double() + 1.0) / every) + 1.0) if every else torch.ones(T, dtype=torch.float64)
        q_want = turn(q) * 0.3 * temp[:, None, None]
        k_want = turn(k)
        qs = torch.zeros(T, HD, device=cuda)
        cache = torch.full((10, GD + GV), 5.0, device=cuda)
        fd = freq.to(cuda)
        pd, bd = proj.to(cuda).contiguous(), bias.to(cuda)
        wqd, wkd, posd, slotd = wq.to(cuda), wk.to(cuda), pos.to(cuda), slots.to(cuda)
        L.check(lib.b200q_window_attn_prep_ex(pd.data_ptr(), ld, 0, HD if own else -1, HD + GD, bd.data_ptr(), H, G, D, V,
                                              qk_norm, wqd.data_ptr() if qk_norm else None,
                                              wkd.data_ptr() if qk_norm else None, 1e-5, 8, fd.data_ptr(), mag,
                                              posd.data_ptr(), slotd.data_ptr(), None, 0.3, 0.4, every,
                                              qs.data_ptr(), cache.data_ptr() if own else None, T, L.DTYPE_F32, None))
        torch.cuda.synchronize()
        assert float((qs.cpu().double().view(T, H, D) - q_want).abs().max()) < 1e-5
        if own:
            for t in range(T):
                if slots[t] >= 0:
                    row = cache[int(slots[t])].cpu().double()
                    assert float((row[:GD] - k_want[t].reshape(-1)).abs().max()) < 1e-5
                    assert float((row[GD:] - v[t]).abs().max()) < 1e-5
            assert float(cache[1].min()) == 5.0 and float(cache[2].max()) == 5.0   # places no token names are untouched


LATENT_CASES = [
    # (T, H, latent size, rotated size, window, marked keys)
    (150, 3, 40, 8, 19, [0, 18, 19, 47, 63, 64, 100]),          # sizes no tile takes
    (200, 5, 64, 64, 64, [0, 15, 16, 63, 64, 127, 128, 135]),   # tile sizes, a window of one tile
    (250, 9, 128, 64, 80, [3, 79, 80, 83, 159, 160, 200]),      # more heads than one tile has rows
    (256, 2, 128, 16, 0, [5]),                                  # every earlier key: one far back among hundreds
    (120, 20, 256, 64, 33, [0, 32, 33, 64, 65, 97]),
]


@pytest.mark.parametrize("case", range(len(LATENT_CASES)))
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("how", ["whole", "portions", "single"])
def test_latent_window_edges_pages_far_keys_and_gates(cuda, case, dtype, how):
    """latent attention over a paged cache of [latent | rotated key] rows: a marked row dominates whoever sees it
    and the first latent channel holds the row's position (the query ignores that channel), so an output names
    the rows it saw; every head's output is scaled by the sigmoid of its gate number"""
    L, lib = _ops()
    T, H, R, P, window, marks = LATENT_CASES[case]
    RP, bs = R + P, 16
    g = torch.Generator().manual_seed(case)
    u = torch.randn(RP, generator=g)
    u[0] = 0.0
    u = u / u.norm()
    qa = 0.05 * torch.randn(T, H, RP, generator=g) + 6.0 * u
    qa[..., 0] = 0.0
    rows = 0.3 * torch.randn(T, RP, generator=g)
    for j in marks:
        rows[j] = 4.0 * u
    rows[:, 0] = torch.arange(T, dtype=torch.float32)
    gate = torch.randn(T, H + 3, generator=g)
    dt, tdt = (L.DTYPE_F32, torch.float32) if dtype == "f32" else (L.DTYPE_BF16, torch.bfloat16)
    rows, gate = rows.to(tdt).float(), gate.to(tdt).float()
    want = torch.zeros(T, H, R, dtype=torch.float64)
    for i in range(T):
        lo = max(0, i - window + 1) if window else 0
        s = torch.einsum("hr,jr->hj", qa[i].double(), rows[lo:i + 1].double()) * 0.9
        want[i] = (torch.softmax(s, -1) @ rows[lo:i + 1, :R].double()) * torch.sigmoid(gate[i, :H].double())[:, None]
    nb = (T + bs - 1) // bs
    pages = np.random.default_rng(case).permutation(nb + 4)[:nb + 1].astype(np.int32)
    cache = torch.full(((nb + 4) * bs, RP), 1e4, dtype=tdt, device=cuda)
    for t in range(T):
        cache[int(pages[t // bs]) * bs + t % bs] = rows[t].to(tdt)
    cache[int(pages[nb]) * bs] = torch.ones(RP).to(tdt)         # the companion's only row
    bt = torch.zeros(2, nb, dtype=torch.int32)
    bt[0, 0] = int(pages[nb])
    bt[1] = torch.tensor(pages[:nb])
    bt = bt.to(cuda).contiguous()
    got = torch.zeros(T, H * R, dtype=tdt, device=cuda)
    portions = {"whole": [T], "portions": [1, 2, 16, 3, 70, 17, 1, 1, 33, 64, 5] * 4, "single": [1] * T}[how]
    c = 0 if how == "whole" else 1
    at = 0
    for n in portions:
        n = min(n, T - at)
        if n <= 0:
            break
        q_step = torch.zeros(c + n, H, RP, device=cuda)
        q_step[c:] = qa[at:at + n].to(cuda)
        g_step = torch.zeros(c + n, H + 3, dtype=tdt, device=cuda)
        g_step[c:] = gate[at:at + n].to(tdt).to(cuda)
        row_seq = torch.tensor([0] * c + [c] * n, dtype=torch.int32, device=cuda)
        pos = torch.tensor([0] * c + list(range(at, at + n)), dtype=torch.int32, device=cuda)
        table = bt if c else bt[1:].contiguous()
        o_step = torch.zeros(c + n, H * R, dtype=tdt, device=cuda)
        L.check(lib.b200q_latent_attn_ex(q_step.data_ptr(), cache.data_ptr(), table.data_ptr(), nb, row_seq.data_ptr(),
                                         pos.data_ptr(), c + n, H, R, P, bs, window, 0.9, g_step.data_ptr(), H + 3,
                                         o_step.data_ptr(), dt, None))
        torch.cuda.synchronize()
        if c:                                                   # one row of ones, gate 0: every channel a half
            assert torch.allclose(o_step[0].float(), torch.full((H * R,), 0.5, device=cuda)), "the companion saw foreign rows"
        got[at:at + n] = o_step[c:]
        at += n
    tol = 2e-4 if dtype == "f32" else 2e-2
    assert float((got.float().cpu().double().view(T, H, R) - want).abs().max()) < tol * T
    for i in range(T):                                          # the marks do what they are meant to
        seen = [m for m in marks if m <= i and (not window or i - m < window)]
        if seen:
            mean = float(want[i, 0, 0] / torch.sigmoid(gate[i, 0].double()))
            assert abs(mean - sum(seen) / len(seen)) < 0.5


# ---- whole models ------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def small():
    spec = small_spec()
    sd = checkpoint(spec, seed=21)
    return spec, sd


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_every_layer(cuda, small, dtype):
    spec, sd = small
    toks = tokens(70, spec.vocab, 1)
    model, eng = build(spec, sd, dtype)
    tap = torch.zeros(spec.n_layers, len(toks), spec.width, device=cuda)
    model.set_layer_tap(tap)
    got = eng.step_replay([(1, toks, list(range(len(toks))))])
    model.set_layer_tap(None)
    stream = []
    want = O.forward(spec.to_config(), sd, toks, torch.float64, stream)
    for i in range(spec.n_layers):
        check_close(tap[i].cpu().numpy(), stream[i].numpy(), dtype, f"layer {i}")
    check_close(got, want.numpy(), dtype)
    eng.close()
    model.close()


@pytest.mark.parametrize("cuts", [[], [1, 1], [2, 2, 2, 3, 5], [16, 16, 1, 15], [20, 2, 21], [21, 21, 2], [64], [7, 90]])
def test_portions_and_token_by_token(cuda, small, cuts):
    """a prompt cut into portions (down to two tokens, across page and window edges and the kept first keys) and
    then decoded token by token gives the logits of the whole prompt; [] = every token alone from the first"""
    spec, sd = small
    toks = tokens(100, spec.vocab, 2)
    want = oracle_logits(spec, sd, toks)
    model, eng = build(spec, sd)
    got = replay_cut(eng, 1, toks, cuts)
    assert rel_err(got, want) < F32_TOL
    eng.close()
    model.close()


def test_long_decoding_past_windows_pages_and_temperature_steps(cuda, small):
    spec, sd = small
    toks = tokens(330, spec.vocab, 3)
    want = oracle_logits(spec, sd, toks)
    for dtype in (torch.float32, torch.bfloat16):
        model, eng = build(spec, sd, dtype)
        got = replay_cut(eng, 1, toks, [3])
        check_close(got, want, dtype)
        eng.close()
        model.close()


def _tile_spec():
    """head sizes and latents the tensor-core attention kernels take, with kept keys, a cap, borrowed keys"""
    layers = [attn(heads=4, kv_heads=2, dim=64, vdim=64, window=24, keep_first=3, rot_dims=32, ff="dense", ff_dim=128),
              latent(heads=3, dim=32, rot_dim=64, vdim=32, kv_rank=64, window=20, ff="dense", ff_dim=64),
              attn2(heads=2, kv_heads=1, dim=128, vdim=64, softcap=5.0, every=16, ff="dense", ff_dim=64),
              attn(heads=8, kv_heads=2, dim=64, vdim=64, window=17, keep_first=20, rot_dims=32, kv_from=0)]
    return small_spec(width=128, vocab=256, layers=layers, side_dim=8)


@pytest.mark.parametrize("which,dtype", [("small", torch.float32), ("tiles", torch.float32), ("tiles", torch.bfloat16)])
def test_mixed_batches_pages_reused(cuda, small, which, dtype):
    """up to three live requests in a pool too small for all of them: portions of some beside single tokens of
    others, requests that sit a step out, finished requests whose pages go to the next one (the pool starts
    dirty).  Every request must come out as if it had run alone."""
    spec, sd = small if which == "small" else (_tile_spec(), None)
    sd = sd or checkpoint(spec, seed=31)
    rng = np.random.default_rng(7)
    lens = [37, 5, 64, 18, 1, 49, 33, 2, 80]
    reqs = {i: tokens(n, spec.vocab, 100 + i) for i, n in enumerate(lens)}
    want = {i: oracle_logits(spec, sd, t) for i, t in reqs.items()}
    model, eng = build(spec, sd, dtype, max_tokens=160, max_seqs=3, num_blocks=13)   # 208 token places for 289 tokens
    model.kv.view(torch.int16).fill_(0x4E4E)                                  # large values in either dtype
    got = {i: [] for i in reqs}
    at = {i: 0 for i in reqs}
    waiting, live = list(reqs), []
    while waiting or live:
        while waiting and len(live) < 3:
            need = sum((len(reqs[i]) + 15) // 16 for i in live) + (len(reqs[waiting[0]]) + 15) // 16
            if need > 13:
                break
            live.append(waiting.pop(0))
        entries, done = [], []
        for i in live:
            if len(live) > 1 and rng.random() < 0.2:
                continue                                                       # sits this step out
            left = len(reqs[i]) - at[i]
            n = min(left, int(rng.choice([1, 1, 2, 3, 9, 16, 40])))
            entries.append((i, reqs[i][at[i]:at[i] + n], list(range(n))))
        if not entries:
            continue
        out = eng.step_replay(entries)
        row = 0
        for i, t, w in entries:
            got[i].append(out[row:row + len(w)])
            row += len(w)
            at[i] += len(t)
            if at[i] == len(reqs[i]):
                done.append(i)
        for i in done:
            eng.abort(i)
            live.remove(i)
    for i in reqs:
        check_close(np.concatenate(got[i]), want[i], dtype, f"request {i}")
    assert eng.stats().free_blocks == 13
    eng.close()
    model.close()


def test_other_sizes_power_of_two_everything(cuda):
    """sizes the tensor-core paths take (multiples of 64; head sizes 64 and 128; latents of 64 and 128), in bf16
    and fp32; multipliers of one, no token input, a first layer that is not latent attention"""
    layers = [attn(heads=4, kv_heads=1, dim=64, vdim=64, window=64, keep_first=4, rot_dims=64, ff="dense", ff_dim=256),
              latent(heads=4, dim=64, rot_dim=64, vdim=64, kv_rank=64, window=40, ff="dense", ff_dim=128),
              attn2(heads=2, kv_heads=2, dim=128, vdim=128, softcap=6.0, every=64, ff="dense", ff_dim=128),
              attn(heads=8, kv_heads=1, dim=64, vdim=64, window=30, keep_first=70, rot_dims=64, kv_from=0),
              latent(heads=2, dim=128, rot_dim=64, vdim=128, kv_rank=128, window=100, original=0.0, ff="dense", ff_dim=64)]
    spec = small_spec(width=128, vocab=256, layers=layers, mult=1.0, embed_scale=1.0, logit_scale=1.0, side_dim=0)
    sd = checkpoint(spec, seed=5)
    toks = tokens(150, spec.vocab, 8)
    want = oracle_logits(spec, sd, toks)
    for dtype in (torch.float32, torch.bfloat16):
        model, eng = build(spec, sd, dtype)
        got = replay_cut(eng, 1, toks, [130, 2, 9])
        check_close(got, want, dtype)
        eng.close()
        model.close()


def test_long_portions_take_the_product_with_the_gated_unit_in_its_epilogue(cuda):
    """portions of 512 tokens and more run gate / up through the fused product (bf16, sizes in blocks of 128), shorter
    ones through the plain product and the elementwise kernel over the same interleaved rows: one prompt whole, cut
    in two long portions, and cut short"""
    layers = [attn(heads=2, kv_heads=1, dim=64, vdim=64, window=200, keep_first=3, rot_dims=32, ff="dense", ff_dim=256),
              latent(heads=2, dim=32, rot_dim=32, vdim=64, kv_rank=64, window=300, ff="dense", ff_dim=128)]
    spec = small_spec(width=128, vocab=256, layers=layers, side_dim=8)
    sd = checkpoint(spec, seed=9)
    toks = tokens(1100, spec.vocab, 4)
    want = oracle_logits(spec, sd, toks)
    for dtype in (torch.float32, torch.bfloat16):
        model, eng = build(spec, sd, dtype, max_tokens=1152)
        for rid, cuts in ((1, [1100]), (2, [520, 580]), (3, [300, 511, 289])):
            got = replay_cut(eng, rid, toks, cuts)
            eng.abort(rid)
            check_close(got, want, dtype, str(cuts))
        eng.close()
        model.close()


# ---- generation through the engine's own scheduler, sampler and model directory reader ----------------
def _generate(eng, prompts, n_new):
    for i, p in enumerate(prompts):
        eng.add_request(i, p, n_new, ignore_eos=True)
    outs = {i: [] for i in range(len(prompts))}
    while eng.has_work():
        ids, toks, _ = eng.step()
        for i, t in zip(ids.tolist(), toks.tolist()):
            outs[i].append(t)
    return outs


def test_greedy_generation_from_a_model_directory(cuda, small, tmp_path):
    """config.json + model.safetensors on disk -> resolve_model -> NativeModel -> Engine.add_request/step:
    chunked prefill under a small token budget, continuous batching of unequal requests, decode-only steps,
    more requests than may be live at once"""
    from llmq_b200.kabavik import save_checkpoint
    from llmq_b200.model import Engine, NativeModel, checkpoint_engine_weights, resolve_model

    spec, sd = small
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(spec.to_config()))
    save_checkpoint(str(d / "model.safetensors"), sd)
    spec2, model_dir = resolve_model(str(d))
    assert spec2.layers == spec.layers and spec2.layered and spec2.arch == "kabavik"
    prompts = [tokens(n, spec.vocab, 40 + n) for n in (3, 41, 1, 26, 17, 9)]
    n_new = 24
    model = NativeModel(spec2, checkpoint_engine_weights(spec2, model_dir), max_tokens=32, max_seqs=4,
                        max_model_len=128, num_blocks=24, dtype=torch.float32)
    eng = Engine(model, max_num_seqs=4, max_num_batched_tokens=32)
    outs = _generate(eng, prompts, n_new)
    for i, p in enumerate(prompts):
        assert outs[i] == O.greedy(spec.to_config(), sd, p, n_new), f"request {i}"
    eng.close()
    model.close()


def test_greedy_generation_bf16_matches_its_own_replay(cuda, small):
    """bf16 serving: what the scheduler generates is what a replay of the same tokens predicts (sampling, async
    stepping and graphs change nothing)"""
    spec, sd = small
    prompts = [tokens(n, spec.vocab, 60 + n) for n in (12, 30)]
    model, eng = build(spec, sd, torch.bfloat16, max_tokens=64)
    outs = _generate(eng, prompts, 20)
    fresh_model, fresh = build(spec, sd, torch.bfloat16, max_tokens=64)
    for i, p in enumerate(prompts):
        full = p + outs[i]
        lg = eng.step_replay([(100 + i, full, list(range(len(full))))])
        eng.abort(100 + i)
        again = fresh.step_replay([(1, full, list(range(len(full))))])
        fresh.abort(1)
        assert rel_err(lg, again) < 1e-6
        top2 = np.sort(lg[len(p) - 1:-1], -1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 0.05 * np.abs(lg).max()         # skip near-ties of bf16 rounding
        pred = lg[len(p) - 1:-1].argmax(-1)
        assert (pred[clear] == np.asarray(outs[i])[clear]).all()
    fresh.close()
    fresh_model.close()
    eng.close()
    model.close()
