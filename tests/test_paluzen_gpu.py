"""GPU tests of the Paluzen path: the engine (scheduler, paged key/value cache, state slots, kernels) against
oracle/paluzen.py — a plain fp64 restatement that recomputes every position from the tokens, with no cache,
no state and no batching.  The configurations are small, differ from one another in every size, and are
drawn here; the fp32 engine is held to a tight bound, the bf16 engine to a rounding-sized one."""
import json

import numpy as np
import pytest
import torch

from oracle import paluzen as O
from tests.paluzen_util import (DENSE, MOE, MOE_ALL, MOE_ONE, checkpoint, lightning, parallel, rel_err, small_spec,
                                tokens)

pytestmark = pytest.mark.gpu
F32_TOL, BF16_TOL = 2e-4, 8e-2


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
    """fp32: every row within the tight bound.  bf16: a router may settle a near-tie the other way on a few
    rows (another expert answers there), so nine rows in ten within the rounding-sized bound"""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    rows = np.sqrt(((got - want) ** 2).mean(-1)) / (np.sqrt((want ** 2).mean(-1)) + 1e-30)
    if dtype == torch.float32:
        assert rows.max() < F32_TOL, what
    else:
        assert np.quantile(rows, 0.9) < BF16_TOL, what


def _ops():
    from llmq_b200 import lib as L
    return L, L.load()


# ---- every mechanism alone: a one-layer model around it --------------------------------------------------
ONE_LAYER = {
    "lightning": ([lightning()], None),
    "lightning_wide_keys": ([lightning(heads=2, dim=72, vdim=8, decay=(1.0, 0.25))], None),
    "lightning_one_head_odd": ([lightning(heads=1, dim=7, vdim=33, decay=(0.9,))], None),
    "window_and_decay_mix": ([parallel()], None),
    "window_one_key": ([parallel(window=1, rot_dims=24, r_heads=1, r_dim=72, r_rank=1)], None),
    "window_many_heads_per_key": ([parallel(heads=18, kv_heads=2, dim=8, vdim=8, window=7, rot_dims=2)], None),
    "no_window_no_rotation": ([parallel(heads=2, kv_heads=1, dim=72, vdim=24, window=0, rot_dims=0)], None),
    "dense": ([lightning(heads=1, dim=8, vdim=8, decay=(0.5,), **DENSE)], None),
    "experts_groups_identity": ([lightning(heads=1, dim=8, vdim=8, decay=(0.5,), **MOE)], None),
    "experts_one": ([lightning(heads=1, dim=8, vdim=8, decay=(0.5,), **MOE_ONE)], None),
    "experts_all_chosen": ([lightning(heads=1, dim=8, vdim=8, decay=(0.5,), **MOE_ALL)], None),
    "experts_identity_only": ([lightning(heads=1, dim=8, vdim=8, decay=(0.5,), ff="moe", ff_dim=8, n_experts=0,
                                         n_identity=4, top_k=2, n_groups=2, keep_groups=2)], None),
    "one_layer_five_passes": ([lightning(**MOE)], (0, 1, 5)),
    "one_pass_is_still_injected": ([parallel(**DENSE)], (0, 1, 1)),
}


@pytest.mark.parametrize("name", sorted(ONE_LAYER))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mechanism_alone(cuda, name, dtype):
    layers, loop = ONE_LAYER[name]
    spec = small_spec(width=80, vocab=97, layers=layers, loop=loop, softcap=0.0 if "dense" in name else 15.0)
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
    eng.close()
    model.close()


# ---- op level: made-up inputs that make a fault show ----------------------------------------------------
def _window_op(cuda, qs, keys, vals, window, dtype, portions=None, block_size=16, shuffle_seed=0, companion=0):
    """run b200q_window_attn for one sequence of T tokens whose keys and values lie in a paged cache with
    shuffled pages (unused places hold garbage); no gate.  portions: the token counts of successive steps
    (None = all at once); companion > 0 puts another sequence's single token first in every step."""
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
        L.check(lib.b200q_window_attn(q_step.data_ptr(), cache.data_ptr(), table.data_ptr(), nb, row_seq.data_ptr(),
                                      pos.data_ptr(), desc.data_ptr(), 1 + c, rows, H, G, D, V, block_size, window, None,
                                      0, o_step.data_ptr(), dtype, None))
        torch.cuda.synchronize()
        if c:
            assert torch.allclose(o_step[0].float(), torch.ones(H * V, device=cuda)), "the companion saw foreign keys"
        out[at:at + n] = o_step[c:]
        at += n
    return out.float().cpu().reshape(T, H, V)


def _standout(T, H, G, D, V, marks, seed):
    """small random queries and keys; at every marked position the key points along the (shared) query
    direction of its group and is large, so whoever sees it is dominated by it; the value of position j is j
    in every channel, so an output row names the keys it saw"""
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(G, D, generator=g)
    u = u / u.norm(dim=-1, keepdim=True)
    qs = 0.05 * torch.randn(T, H, D, generator=g) + 6.0 * u.repeat_interleave(H // G, 0)[None]
    keys = 0.3 * torch.randn(T, G, D, generator=g)
    for j in marks:
        keys[j] = 4.0 * u
    vals = torch.arange(T, dtype=torch.float32)[:, None, None].expand(T, G, V).clone()
    return qs, keys, vals


def _window_want(qs, keys, vals, window):
    T, H, D = qs.shape
    G = keys.shape[1]
    out = torch.zeros(T, H, vals.shape[2], dtype=torch.float64)
    for h in range(H):
        for i in range(T):
            lo = max(0, i - window + 1) if window else 0
            s = keys[lo:i + 1, h // (H // G)].double() @ qs[i, h].double()
            out[i, h] = torch.softmax(s, 0) @ vals[lo:i + 1, h // (H // G)].double()
    return out


WINDOW_CASES = [
    # (T, H, G, D, V, window, marked keys)
    (150, 4, 2, 24, 40, 21, [0, 20, 21, 47, 63, 64, 100]),        # window edges off pages and tiles
    (200, 2, 1, 64, 64, 64, [0, 15, 16, 63, 64, 127, 128, 135]),   # a window of one tile, pages at its edges
    (300, 4, 2, 128, 128, 80, [3, 79, 80, 83, 159, 160, 200]),     # head size 128, window 80
    (260, 3, 3, 16, 8, 0, [5]),                                    # every earlier key: one far back among hundreds
    (90, 16, 1, 64, 128, 17, [0, 16, 17, 33, 50]),                 # sixteen heads on one key head, values wider than keys
    (70, 24, 1, 128, 64, 19, [0, 18, 19, 40]),                     # more heads per key head than a decode tile has rows
]


@pytest.mark.parametrize("case", range(len(WINDOW_CASES)))
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("how", ["whole", "portions", "single"])
def test_window_edges_pages_and_far_keys(cuda, case, dtype, how):
    """a key that dominates whoever sees it: it is seen up to window - 1 tokens later and not one more, at page
    borders and tile borders alike, in a whole prompt, in portions of 1 to 70 tokens beside another sequence, and
    token by token"""
    L, _ = _ops()
    T, H, G, D, V, window, marks = WINDOW_CASES[case]
    qs, keys, vals = _standout(T, H, G, D, V, marks, seed=case)
    dt = L.DTYPE_F32 if dtype == "f32" else L.DTYPE_BF16
    if dtype == "bf16":                                        # what the cache can hold
        keys, vals = keys.bfloat16().float(), vals.bfloat16().float()
    want = _window_want(qs, keys, vals, window)
    portions = {"whole": None, "portions": [1, 2, 16, 3, 70, 17, 1, 1, 33, 64, 5] * 4, "single": [1] * T}[how]
    got = _window_op(cuda, qs, keys, vals, window, dt, portions, shuffle_seed=case, companion=how != "whole")
    tol = 2e-4 if dtype == "f32" else 2e-2
    assert float((got.double() - want).abs().max()) < tol * T
    # the marks do what they are meant to: one token past the window the marked key is gone
    for j in marks:
        last = j + window - 1 if window else T - 1
        if last < T and not any(j < m <= last for m in marks):
            assert abs(float(want[last, 0, 0]) - j) < 0.5
        if window and last + 1 < T and not any(j < m <= last + 1 for m in marks):
            assert abs(float(want[last + 1, 0, 0]) - j) > 0.5


def test_decay_attention_continues_from_its_slot(cuda):
    """both forms of the decayed state: a sequence fed in portions of 1, 2, 7 and 9 tokens beside another
    sequence's token equals the sequence at once; its first portion ignores what the slot held"""
    L, lib = _ops()
    g = torch.Generator().manual_seed(3)
    T, H, D = 40, 3, 12
    for vec, V in ((False, 20), (True, D)):
        q, k, v = (torch.randn(T, H * n, generator=g) for n in (D, D, V))
        w = torch.rand(T, H * D, generator=g) * 0.5 + 0.5
        bonus = torch.randn(H * D, generator=g)
        lam = torch.tensor([0.9, 0.5, 1.0])
        S = torch.zeros(H, D, V, dtype=torch.float64)
        want = torch.zeros(T, H, V, dtype=torch.float64)
        for t in range(T):
            kv = k[t].view(H, D, 1).double() * v[t].view(H, 1, V).double()
            if vec:
                want[t] = ((S + bonus.view(H, D, 1).double() * kv) * q[t].view(H, D, 1).double()).sum(1)
                S = w[t].view(H, D, 1).double() * S + kv
            else:
                S = lam.view(H, 1, 1).double() * S + kv
                want[t] = (S * q[t].view(H, D, 1).double()).sum(1)
        qkv = torch.cat([q, k, v], 1).to(cuda).contiguous()
        ld = qkv.shape[1]
        slot_stride = H * D * V + 8
        state = torch.full((3, slot_stride), 7.0, device=cuda)
        got = torch.zeros(T, H * V, device=cuda)
        wd, bd, lamd = w.to(cuda).contiguous(), bonus.to(cuda), lam.to(cuda)
        at = 0
        for n in [1, 2, 7, 9, 1, 20]:
            # the sequence is the second of the step (slot 2); the first is another sequence's token in slot 0
            desc = torch.tensor([[0, 1, 5, 0], [1, n, at, 2]], dtype=torch.int32, device=cuda)
            step = torch.zeros(1 + n, ld, device=cuda)
            step[1:] = qkv[at:at + n]
            wstep = torch.ones(1 + n, H * D, device=cuda)
            wstep[1:] = wd[at:at + n]
            raw = torch.zeros(1 + n, H * V, device=cuda)
            L.check(lib.b200q_decay_attn(step.data_ptr(), ld, 0, H * D, 2 * H * D, None if vec else lamd.data_ptr(),
                                         wstep.data_ptr() if vec else None, H * D, bd.data_ptr() if vec else None,
                                         state.data_ptr(), slot_stride, desc.data_ptr(), 2, H, D, V, raw.data_ptr(), None))
            got[at:at + n] = raw[1:]
            at += n
        torch.cuda.synchronize()
        assert float((got.cpu().double().view(T, H, V) - want).abs().max()) < 1e-4 * float(want.abs().max())
        assert float(state[1].min()) == 7.0                     # an unused slot is untouched


def test_shifted_norm_carries_the_previous_row(cuda):
    """norm + token shift over portions of 1, 2 and more tokens of two interleaved sequences equals the whole"""
    L, lib = _ops()
    g = torch.Generator().manual_seed(5)
    W, T = 50, 23
    xs = [torch.randn(T, W, generator=g) * 3 for _ in range(2)]
    wn, sh = torch.rand(W, generator=g) + 0.5, torch.rand(W, generator=g)
    want = [O.token_shift(O.rms(x.double(), 1e-5) * wn.double(), sh.double()) for x in xs]
    state = torch.full((4, W + 4), 9.0, device=cuda)
    carry = torch.zeros(4, W, device=cuda)
    wd, sd = wn.to(cuda), sh.to(cuda)
    got = [torch.zeros(T, W), torch.zeros(T, W)]
    at = [0, 0]
    for na, nb in [(1, 2), (2, 1), (1, 1), (5, 0), (0, 3), (14, 16)]:
        parts = [(s, n) for s, n in ((0, na), (1, nb)) if n > 0]
        rows = sum(n for _, n in parts)
        x = torch.cat([xs[s][at[s]:at[s] + n] for s, n in parts]).to(cuda).contiguous()
        desc, row_seq, r0 = [], [], 0
        for i, (s, n) in enumerate(parts):
            desc.append([r0, n, at[s], 3 - s])                 # sequence s lives in slot 3 - s
            row_seq += [i] * n
            r0 += n
        desc = torch.tensor(desc, dtype=torch.int32, device=cuda)
        row_seq = torch.tensor(row_seq, dtype=torch.int32, device=cuda)
        y = torch.zeros(rows, W, device=cuda)
        L.check(lib.b200q_rmsnorm_shift(x.data_ptr(), None, wd.data_ptr(), sd.data_ptr(), state.data_ptr(), W + 4,
                                        desc.data_ptr(), row_seq.data_ptr(), len(parts), carry.data_ptr(), None,
                                        y.data_ptr(), rows, W, 1e-5, L.DTYPE_F32, None))
        L.check(lib.b200q_store_carry(carry.data_ptr(), 0, state.data_ptr(), W + 4, desc.data_ptr(), len(parts), W, 1, None))
        torch.cuda.synchronize()
        r0 = 0
        for s, n in parts:
            got[s][at[s]:at[s] + n] = y[r0:r0 + n].cpu()
            r0 += n
            at[s] += n
    for s in range(2):
        assert float((got[s].double() - want[s]).abs().max()) < 1e-5


def test_grouped_routing_ties_negative_scores_and_masked_groups(cuda):
    """made-up logits and corrections: the correction decides the choice but not the weights; an expert outside
    the kept groups loses even to a negative choice score; ties go to the lowest index"""
    L, lib = _ops()
    E, top, groups, keep = 12, 3, 4, 2
    logits = torch.zeros(5, E)
    corr = torch.zeros(E)
    logits[0, 7] = 3.0                                          # group 2 wins; its three experts are chosen first
    logits[1] = torch.linspace(0, 1.1, E)                       # ascending: groups 3 and 2 are kept
    corr_case = corr.clone()
    corr_case[0] = 0.5                                          # row 2: the correction lifts expert 0 (group 0) ...
    logits[3, 4] = 2.0                                          # row 3: all equal but one
    rows = [(logits, corr), (logits, corr_case), (logits, torch.full((E,), -5.0))]
    for lg, cr in rows:
        w = {"r.router": torch.eye(E, dtype=torch.float64), "r.correction": cr.double()}
        idx_w, wt_w = O.route(lg.double(), w, "r.", {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}})
        T = lg.shape[0]
        idx = torch.zeros(T, top, dtype=torch.int32, device=cuda)
        wts = torch.zeros(T, top, device=cuda)
        aux = [torch.zeros(T * top + E + 2, dtype=torch.int32, device=cuda) for _ in range(3)]
        lgd, crd = lg.to(cuda).contiguous(), cr.to(cuda).contiguous()
        L.check(lib.b200q_moe_route_grouped(lgd.data_ptr(), crd.data_ptr(), T, E, E, top,
                                            groups, keep, idx.data_ptr(), wts.data_ptr(), aux[0].data_ptr(),
                                            aux[1].data_ptr(), aux[2].data_ptr(), None, None, None))
        torch.cuda.synchronize()
        assert idx.cpu().tolist() == idx_w.tolist()
        assert float((wts.cpu().double() - wt_w).abs().max()) < 1e-6
        off = aux[0].cpu().tolist()[:E + 1]
        assert off[0] == 0 and off[E] == T * top and all(a <= b for a, b in zip(off, off[1:]))


# ---- whole models ------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def small():
    spec = small_spec()
    sd = checkpoint(spec, seed=21)
    return spec, sd


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_every_layer_run(cuda, small, dtype):
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
        check_close(tap[i].cpu().numpy(), stream[i].numpy(), dtype, f"layer run {i}")
    check_close(got, want.numpy(), dtype)
    eng.close()
    model.close()


@pytest.mark.parametrize("cuts", [[], [1, 1], [2, 2, 2, 3, 5], [16, 16, 1, 15], [20, 2, 21], [21, 21, 2], [64], [7, 90]])
def test_portions_and_token_by_token(cuda, small, cuts):
    """a prompt cut into portions (down to two tokens, across page and window edges) and then decoded token by
    token gives the logits of the whole prompt; [] = every token alone from the first"""
    spec, sd = small
    toks = tokens(100, spec.vocab, 2)
    want = oracle_logits(spec, sd, toks)
    model, eng = build(spec, sd)
    got = replay_cut(eng, 1, toks, cuts)
    assert rel_err(got, want) < F32_TOL
    eng.close()
    model.close()


def test_long_decoding_past_windows_and_pages(cuda, small):
    spec, sd = small
    toks = tokens(330, spec.vocab, 3)
    want = oracle_logits(spec, sd, toks)
    for dtype in (torch.float32, torch.bfloat16):
        model, eng = build(spec, sd, dtype)
        got = replay_cut(eng, 1, toks, [3])
        check_close(got, want, dtype)
        eng.close()
        model.close()


def test_mixed_batches_pages_and_slots_reused(cuda, small):
    """up to three live requests in a pool too small for all of them: portions of some beside single tokens of
    others, requests that sit a step out, finished requests whose pages and state slot go to the next one
    (pool and slots start dirty).  Every request must come out as if it had run alone."""
    spec, sd = small
    rng = np.random.default_rng(7)
    lens = [37, 5, 64, 18, 1, 49, 33, 2, 80]
    reqs = {i: tokens(n, spec.vocab, 100 + i) for i, n in enumerate(lens)}
    want = {i: oracle_logits(spec, sd, t) for i, t in reqs.items()}
    model, eng = build(spec, sd, max_tokens=160, max_seqs=3, num_blocks=13)   # 208 token places for 289 tokens
    model.state.fill_(3.0)
    model.kv.view(torch.float32).fill_(1e3)
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
        assert rel_err(np.concatenate(got[i]), want[i]) < F32_TOL, f"request {i}"
    assert eng.stats().free_blocks == 13
    eng.close()
    model.close()


def test_other_sizes_power_of_two_everything(cuda):
    """sizes the tensor-core paths take (multiples of 64; head sizes 64 and 128), in bf16 and fp32, without a loop"""
    layers = [lightning(heads=2, dim=64, vdim=128, ff="moe", ff_dim=128, n_experts=7, n_identity=1, top_k=2, n_groups=2,
                        keep_groups=1),
              parallel(heads=4, kv_heads=1, dim=64, vdim=64, window=64, rot_dims=64, r_heads=2, r_dim=64, r_rank=64,
                       ff="dense", ff_dim=256),
              parallel(heads=2, kv_heads=2, dim=128, vdim=128, window=40, rot_dims=32, r_heads=4, r_dim=32, r_rank=64,
                       ff="moe", ff_dim=64, n_experts=4, n_identity=0, top_k=4, n_groups=1, keep_groups=1)]
    spec = small_spec(width=128, vocab=256, layers=layers, loop=None)
    sd = checkpoint(spec, seed=5)
    toks = tokens(150, spec.vocab, 8)
    want = oracle_logits(spec, sd, toks)
    for dtype in (torch.float32, torch.bfloat16):
        model, eng = build(spec, sd, dtype)
        got = replay_cut(eng, 1, toks, [130, 2, 9])
        check_close(got, want, dtype)
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
    chunked prefill under a small token budget, continuous batching of unequal requests, decode-only steps
    (replayed from CUDA graphs), more requests than state slots"""
    from llmq_b200.model import Engine, NativeModel, checkpoint_engine_weights, resolve_model
    from llmq_b200.paluzen import save_checkpoint

    spec, sd = small
    d = tmp_path / "model"
    d.mkdir()
    cfg = spec.to_config()
    for lc in cfg["layers"]:                                    # the inner size of the decay path comes from the tensor
        if lc["type"] == "parallel":
            del lc["mixer"]["right"]["rank"]
    (d / "config.json").write_text(json.dumps(cfg))
    save_checkpoint(str(d / "model.safetensors"), sd)
    spec2, model_dir = resolve_model(str(d))
    assert spec2.layers == spec.layers and spec2.layered and spec2.arch == "paluzen"
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
    """bf16 serving: what the scheduler generates is what a replay of the same tokens predicts (sampling,
    async stepping and graphs change nothing)"""
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
