"""Bigerax on the GPU against the plain implementation (tests/plain_bigerax.py): each mechanism alone, then whole
models under every way of cutting, decoding from the first token, slots and pages used again, generation through the
engine's own entry point, and the replay program."""
import numpy as np
import pytest
import torch

import bigerax_util as bu
import plain_bigerax as pb
import replay_util as ru
from conftest import random_tokens

pytestmark = pytest.mark.gpu

DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# relative root-mean-square error of a logits row against float64: fp32 sums of a few hundred terms; bfloat16 rounds the
# activations to 8 bits between kernels
ROW_TOL = {"float32": 3e-5, "bfloat16": 4e-2}


def rel_rms(got, want):
    d = np.asarray(got, dtype=np.float64) - want
    return np.sqrt((d * d).mean(axis=-1)) / max(np.sqrt((want * want).mean()), 1e-9)


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype)


def bf16_round(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


# ---- mechanisms alone ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("d,groups", [(64, 1), (60, 3), (256, 8), (512, 32), (4096, 2), (96, 96), (2048, 4), (8192, 1), (768, 3)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_group_norm_chain(d, groups, dtype):
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(d + groups)
    n, eps = 7, 1e-5
    res0 = rng.randn(n, d) * 3
    branch = bf16_round(rng.randn(n, d) * np.linspace(0.1, 5, d)) if dtype == "bfloat16" else rng.randn(n, d) * np.linspace(0.1, 5, d)
    w1, w2 = bf16_round(1 + 0.2 * rng.randn(d)), bf16_round(1 + 0.2 * rng.randn(d))
    tol = 2e-5 if dtype == "float32" else 1e-2             # groups of one element are sensitive near zero
    # norm the branch, add, norm the sum
    residual = dev(res0)
    out = torch.empty((n, d), dtype=DT[dtype], device=DEV)
    ops.group_norm_chain(residual, dev(branch, DT[dtype]), dev(w1, DT[dtype]), dev(w2, DT[dtype]), groups, eps, out)
    want_res = res0.astype(np.float32).astype(np.float64) + pb.group_rmsnorm(branch, w1, groups, eps)
    assert np.abs(residual.cpu().numpy() - want_res).max() <= 2e-6 * np.abs(want_res).max() + 1e-6
    want = pb.group_rmsnorm(want_res, w2, groups, eps)
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()
    # add only; norm only, of gathered rows
    residual = dev(res0)
    ops.group_norm_chain(residual, dev(branch, DT[dtype]), dev(w1, DT[dtype]), None, groups, eps)
    assert np.abs(residual.cpu().numpy() - want_res).max() <= 2e-6 * np.abs(want_res).max() + 1e-6
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out = torch.empty((3, d), dtype=DT[dtype], device=DEV)
    ops.group_norm_chain(residual, None, None, dev(w2, DT[dtype]), groups, eps, out, rows)
    assert np.abs(out.float().cpu().numpy() - want[[5, 0, 5]]).max() <= tol * np.abs(want).max()
    # a group of a row is normed by its own mean square: scaling one group changes nothing outside it
    if groups > 1:
        res2 = res0.copy()
        res2[:, : d // groups] *= 100.0
        a, b = torch.empty((n, d), dtype=DT[dtype], device=DEV), torch.empty((n, d), dtype=DT[dtype], device=DEV)
        ops.group_norm_chain(dev(res0), None, None, dev(w2, DT[dtype]), groups, eps, a)
        ops.group_norm_chain(dev(res2), None, None, dev(w2, DT[dtype]), groups, eps, b)
        assert torch.equal(a[:, d // groups:], b[:, d // groups:])


@pytest.mark.parametrize("d,mp,mc", [(24, 29, 13), (20, -7, 5), (7, 1, 1), (24, 2 ** 40 + 3, 2 ** 35 + 1)])
def test_bigram_embedding_carries_the_previous_token_in_its_slot(d, mp, mc):
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(3)
    V, B = 50, 13
    table, pairs = bf16_round(rng.randn(V, d)), bf16_round(rng.randn(B + 1, d))
    state = torch.full((4,), 7, dtype=torch.int32, device=DEV)          # what an earlier user of the slots left behind

    def step(entries):
        """entries: (slot, first position, tokens)"""
        ids = np.concatenate([t for _, _, t in entries]).astype(np.int32)
        pos = np.concatenate([np.arange(p, p + len(t)) for _, p, t in entries]).astype(np.int32)
        req = np.concatenate([np.full(len(t), r) for r, (_, _, t) in enumerate(entries)]).astype(np.int32)
        starts = np.cumsum([0] + [len(t) for _, _, t in entries])[:-1]
        meta = np.stack([starts, [len(t) for _, _, t in entries], np.zeros(len(entries)), [s for s, _, _ in entries]], 1).astype(np.int32)
        out = torch.empty((len(ids), d), dtype=torch.float32, device=DEV)
        ops.embedding_bigram(dev(ids, torch.int32), dev(pos, torch.int32), dev(req, torch.int32), dev(meta, torch.int32),
                             dev(meta[:, 3].copy(), torch.int32), state, dev(table, torch.bfloat16), dev(pairs, torch.bfloat16), out, B, mp, mc)
        return out.cpu().numpy()

    a, b = rng.randint(0, V, 40), rng.randint(0, V, 9)
    want_a = pb.bigram_embedding(list(a), table, pairs, B, mp, mc)
    want_b = pb.bigram_embedding(list(b), table, pairs, B, mp, mc)
    # a in portions of 5, 1, 2, 32 in slot 2, b beside it in slot 0 in portions of 1, 8
    got1 = step([(2, 0, a[:5]), (0, 0, b[:1])])
    got2 = step([(0, 1, b[1:]), (2, 5, a[5:6])])
    got3 = step([(2, 6, a[6:8])])
    got4 = step([(2, 8, a[8:])])
    got_a = np.concatenate([got1[:5], got2[8:], got3, got4])
    got_b = np.concatenate([got1[5:], got2[:8]])
    assert np.abs(got_a - want_a).max() < 1e-6 and np.abs(got_b - want_b).max() < 1e-6
    # a new request in a used slot starts with the extra row, whatever the slot holds
    got = step([(2, 0, b[:3])])
    assert np.abs(got - want_b[:3]).max() < 1e-6
    # the first row is the table's last, not a hashed one
    assert np.allclose(got[0], table[b[0]] + pairs[B])


def _paged(k, v, page_size, rng, dtype):
    """Keys [T, G, dk] and values [T, G, dv] of one request scattered over shuffled pages; returns pools and the table."""
    T, G, dk = k.shape
    dv = v.shape[2]
    n_pages = (T + page_size - 1) // page_size
    order = rng.permutation(n_pages + 3)[:n_pages]
    kp = torch.zeros((n_pages + 3, G, page_size, dk), dtype=dtype, device=DEV)
    vp = torch.zeros((n_pages + 3, G, page_size, dv), dtype=dtype, device=DEV)
    for t in range(T):
        kp[order[t // page_size], :, t % page_size] = dev(k[t], dtype)
        vp[order[t // page_size], :, t % page_size] = dev(v[t], dtype)
    return kp, vp, torch.tensor(order[None, :].astype(np.int32), device=DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,window,page", [(4, 2, 24, 16, 19, 16), (3, 3, 9, 7, 40, 8), (8, 1, 64, 64, 0, 16), (4, 4, 96, 64, 33, 32),
                                                   (2, 1, 128, 128, 130, 16), (2, 2, 16, 200, 5, 16), (16, 1, 32, 96, 100, 16),
                                                   (6, 2, 128, 64, 0, 64)])
@pytest.mark.parametrize("kernels", ["tcgen05", "mma", "plain"])
def test_sink_attention_against_the_plain_one(H, G, dk, dv, window, page, dtype, kernels, monkeypatch):
    from mimirmind_b200.kernels import attention
    if dtype == "float32" and kernels != "plain":
        pytest.skip("the 32-bit path has one kernel")
    if kernels == "tcgen05" and not (dk == dv and dk in (64, 128)):
        pytest.skip("the tcgen05 prefill kernel takes equal key and value sizes of 64 or 128")
    monkeypatch.setattr(attention, "USE_SINK_MMA", kernels != "plain")
    monkeypatch.setattr(attention, "USE_SINK_TCGEN05", kernels == "tcgen05")
    monkeypatch.setattr(attention, "USE_SINK_TMA_DECODE", kernels == "tcgen05")
    from mimirmind_b200.parts.base import LayerCache
    rng = np.random.RandomState(H * 100 + dk)
    T, scale = 300, 0.37 / np.sqrt(dk) * 4
    q, k, v = bf16_round(rng.randn(T, H, dk)), bf16_round(rng.randn(T, G, dk)), bf16_round(rng.randn(T, G, dv))
    want = pb.window_sink_attention(q, k, v, scale, window)
    kp, vp, table = _paged(k, v, page, rng, DT[dtype])
    tol = 2e-5 if dtype == "float32" else 1.5e-2

    class Ctx:
        pass

    def run(lo, hi):
        """queries lo..hi-1 as one portion (keys up to hi-1 are cached)"""
        ctx = Ctx()
        ctx.positions = torch.arange(lo, hi, dtype=torch.int32, device=DEV)
        ctx.token_req = torch.zeros(hi - lo, dtype=torch.int32, device=DEV)
        ctx.max_q_len, ctx.max_kv_len, ctx.n_requests, ctx.q_start, ctx.q_len, ctx.kv_len = hi - lo, hi, 1, [0], [hi - lo], [hi]
        ctx.derived, ctx.plans = {}, {}
        cache = LayerCache(arrays={"k": kp, "v": vp}, block_table=table, page_size=page)
        out = torch.empty((hi - lo, H * dv), dtype=DT[dtype], device=DEV)
        attention.paged_sink_attention(dev(q[lo:hi].reshape(hi - lo, H * dk), DT[dtype]), cache, out, ctx, H, G, dk, dv, window, scale, True)
        return out.float().cpu().numpy().reshape(hi - lo, H, dv)

    whole = run(0, T)
    assert np.abs(whole - want).max() <= tol * np.abs(want).max(), "whole prompt"
    for lo, hi in ((0, 1), (1, 3), (17, 130), (130, 300), (299, 300), (150, 151)):
        got = run(lo, hi)
        assert np.abs(got - want[lo:hi]).max() <= tol * np.abs(want).max(), f"portion {lo}..{hi}"
    # without the sink the weights sum to one: a constant value comes back unchanged; with it, less than that
    ones = torch.ones_like(vp)
    for sink, check in ((False, lambda o: np.allclose(o, 1.0, atol=1e-2)), (True, lambda o: (o < 1.0 - 1e-4).all() if dtype == "float32" else (o.max() <= 1.0 and o.min() < 0.9))):
        ctx = Ctx()
        ctx.positions = torch.arange(0, 40, dtype=torch.int32, device=DEV)
        ctx.token_req = torch.zeros(40, dtype=torch.int32, device=DEV)
        ctx.max_q_len, ctx.max_kv_len, ctx.n_requests, ctx.q_start, ctx.q_len, ctx.kv_len = 40, 40, 1, [0], [40], [40]
        ctx.derived, ctx.plans = {}, {}
        out = torch.empty((40, H * dv), dtype=DT[dtype], device=DEV)
        attention.paged_sink_attention(dev(q[:40].reshape(40, H * dk), DT[dtype]), LayerCache(arrays={"k": kp, "v": ones}, block_table=table, page_size=page),
                                       out, ctx, H, G, dk, dv, window, scale, sink)
        assert check(out.float().cpu().numpy())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,page", [(40, 16), (64, 16), (17, 8), (0, 16), (65, 32)])
@pytest.mark.parametrize("dk,dv", [(32, 8), (32, 32), (64, 64)])
def test_one_key_that_stands_out_is_seen_exactly_inside_the_window(window, page, dtype, dk, dv):
    """Every key is orthogonal to the query but one, whose score stands out by far and whose value is a marker: the
    output shows the marker exactly when that key is inside the window, in a prompt and for a single decoded token, with
    the key at a page's border, far back, and just inside and just outside the window."""
    from mimirmind_b200.kernels import attention
    from mimirmind_b200.parts.base import LayerCache
    H, G = 4, 2                     # bfloat16: values of 8 run the fp32-arithmetic kernel, 32 the mma.sync kernels, 64/64 tcgen05
    T = 400
    rng = np.random.RandomState(window + page)

    class Ctx:
        pass

    for query in (399, 256, 255, 64, 40, 17, 16, 1, 0):
        spots = {query, query - 1, 0, 15, 16, 17, query - window + 1, query - window, query - window - 1, (query // page) * page,
                 (query // page) * page - 1, query - 200, (query // 64) * 64, (query // 64) * 64 - 1}
        for spot in sorted(s for s in spots if 0 <= s <= query):
            k = rng.randn(T, G, dk) * 0.01
            k[:, :, 0] = 0.0
            v = rng.randn(T, G, dv) * 0.01
            q = np.zeros((T, H, dk))
            q[:, :, 0] = 30.0
            k[spot, :, 0] = 1.0
            v[spot] = 5.0
            kp, vp, table = _paged(k, v, page, rng, DT[dtype])
            inside = window == 0 or query - spot < window
            for lo in (query, max(0, query - 50)):                        # decoded alone; the last of a portion
                ctx = Ctx()
                ctx.positions = torch.arange(lo, query + 1, dtype=torch.int32, device=DEV)
                ctx.token_req = torch.zeros(query + 1 - lo, dtype=torch.int32, device=DEV)
                n = query + 1 - lo
                ctx.max_q_len, ctx.max_kv_len, ctx.n_requests, ctx.q_start, ctx.q_len, ctx.kv_len = n, query + 1, 1, [0], [n], [query + 1]
                ctx.derived, ctx.plans = {}, {}
                out = torch.empty((n, H * dv), dtype=DT[dtype], device=DEV)
                attention.paged_sink_attention(dev(q[lo:query + 1].reshape(n, H * dk), DT[dtype]), LayerCache(arrays={"k": kp, "v": vp}, block_table=table, page_size=page),
                                               out, ctx, H, G, dk, dv, window, 1.0, True)
                last = out[-1].float().cpu().numpy()
                if inside:
                    assert (last > 4.9).all(), f"query {query}, key {spot}, window {window}, from {lo}: the key was not seen"
                else:
                    assert (np.abs(last) < 0.1).all(), f"query {query}, key {spot}, window {window}, from {lo}: a key outside the window was seen"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,rots", [(3, 2, 10, 6, ((10, 10000.0), (4, 250000.0), (0, 1.0))),
                                            (4, 2, 32, 16, ((32, 10000.0), (8, 250000.0), (0, 1.0))),      # 16-byte chunks
                                            (2, 1, 96, 32, ((64, 300.0), (12, 10000.0)))])
def test_pair_rotation_value_mixing_and_cache_write_sizes(H, G, dk, dv, rots, dtype):
    _pair_rotation_case(H, G, dk, dv, rots, dtype)


def _pair_rotation_case(H, G, dk, dv, rots, dtype):
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(9)
    page, n = 8, 21
    for rot_dims, base in rots:
        start = 1000
        positions = np.arange(start, start + n)
        qkv = bf16_round(rng.randn(n, (H + G) * dk + G * dv))
        v_first = bf16_round(rng.randn(n, G * dv))
        lam = 0.3
        inv_freq = (base ** (-2.0 * np.arange(max(1, rot_dims // 2)) / max(1, rot_dims))).astype(np.float32)
        n_pages = (start + n) // page + 1
        table = torch.arange(n_pages, dtype=torch.int32, device=DEV).flip(0).view(1, -1).contiguous()
        kp = torch.zeros((n_pages, G, page, dk), dtype=DT[dtype], device=DEV)
        vp = torch.zeros((n_pages, G, page, dv), dtype=DT[dtype], device=DEV)
        q_out = torch.empty((n, H * dk), dtype=DT[dtype], device=DEV)
        vf = dev(v_first, DT[dtype])
        d_pos, d_req = dev(positions, torch.int32), torch.zeros(n, dtype=torch.int32, device=DEV)
        rot = ops.rope_pairs_table(d_pos, dev(inv_freq), rot_dims) if rot_dims else None
        slots = ops.slot_mapping(d_pos, d_req, table, page)
        ops.qkv_pairs_post(dev(qkv, DT[dtype]), q_out, kp, vp, vf, rot, slots, page, H, G, dk, dv, rot_dims, 2, lam)
        q = qkv[:, :H * dk].reshape(n, H, dk)
        k = qkv[:, H * dk:(H + G) * dk].reshape(n, G, dk)
        v = qkv[:, (H + G) * dk:].reshape(n, G, dv)
        want_q = pb.rotate_pairs(q, positions, rot_dims, base) if rot_dims else q
        want_k = pb.rotate_pairs(k, positions, rot_dims, base) if rot_dims else k
        want_v = (1 - lam) * v + lam * v_first.reshape(n, G, dv)
        tol = 3e-4 if dtype == "float32" else 2e-2      # fp32 angles at positions around a thousand
        assert np.abs(q_out.float().cpu().numpy().reshape(n, H, dk) - want_q).max() < tol * 4
        pages = (n_pages - 1 - positions // page)
        got_k = kp.float().cpu().numpy()[pages, :, positions % page]
        got_v = vp.float().cpu().numpy()[pages, :, positions % page]
        assert np.abs(got_k - want_k).max() < tol * 4 and np.abs(got_v - want_v).max() < tol
        # a source layer hands its values on unchanged
        out = torch.zeros((n, G * dv), dtype=DT[dtype], device=DEV)
        ops.qkv_pairs_post(dev(qkv, DT[dtype]), q_out, kp, vp, out, rot, slots, page, H, G, dk, dv, rot_dims, 1, 0.0)
        assert np.array_equal(out.float().cpu().numpy(), qkv[:, (H + G) * dk:].astype(np.float32))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mingru_walk_and_chunked_scan(dtype):
    from mimirmind_b200.kernels import ops
    from mimirmind_b200.parts import mingru as part
    rng = np.random.RandomState(4)
    W = 70
    lens = [300, 1, 65, 128]
    starts = np.cumsum([0] + lens)[:-1]
    n = sum(lens)
    a = rng.randn(n, 3 * W).astype(np.float32) * 2
    bias = rng.randn(2 * W).astype(np.float32)
    ab = a.astype(np.float64).copy()
    ab[:, :2 * W] += bias                                                # what the recurrence sees
    slots = np.array([3, 0, 2, 1], dtype=np.int32)
    first_pos = [0, 5, 0, 77]                                            # two requests go on from a state, two start
    state0 = rng.randn(4, W).astype(np.float32)
    want_y, want_state = np.zeros((n, W)), state0.astype(np.float64).copy()
    for r, (s, ln) in enumerate(zip(starts, lens)):
        init = np.zeros(W) if first_pos[r] == 0 else state0[slots[r]].astype(np.float64)
        z, u, g = pb.sigmoid(ab[s:s + ln, :W]), ab[s:s + ln, W:2 * W], ab[s:s + ln, 2 * W:]
        S, last = pb.mingru_scan(z, u, init)
        want_y[s:s + ln] = S * (g * pb.sigmoid(g))
        want_state[slots[r]] = last
    positions = np.concatenate([np.arange(p, p + ln) for p, ln in zip(first_pos, lens)]).astype(np.int32)
    meta = np.stack([starts, lens, np.zeros(4), slots], 1).astype(np.int32)
    tol = 3e-6 if dtype == "float32" else 1e-2
    state_tol = 3e-6 if dtype == "float32" else 3e-5          # bfloat16 runs take the hardware's exponential and reciprocal
    # the walk
    state = dev(state0)
    y = torch.empty((n, W), dtype=DT[dtype], device=DEV)
    ops.mingru_walk(dev(a), y, state, dev(meta, torch.int32), dev(slots, torch.int32), dev(positions, torch.int32), 4, dev(bias))
    assert np.abs(y.float().cpu().numpy() - want_y).max() <= tol * np.abs(want_y).max()
    assert np.abs(state.cpu().numpy() - want_state).max() <= state_tol * np.abs(want_state).max()
    # the scan over chunks

    class Ctx:
        q_start, q_len, derived, token_ids = list(starts), lens, {}, dev(positions, torch.int32)

    chunk_meta, req_chunks = part.MinGRU._chunks(Ctx)
    assert chunk_meta.shape[0] == sum(-(-ln // part.CHUNK) for ln in lens)
    state = dev(state0)
    y2 = torch.empty((n, W), dtype=DT[dtype], device=DEV)
    ops.mingru_chunked(dev(a), y2, state, chunk_meta, req_chunks, dev(slots, torch.int32), dev(positions, torch.int32), dev(bias))
    assert np.abs(y2.float().cpu().numpy() - want_y).max() <= tol * np.abs(want_y).max()
    assert np.abs(state.cpu().numpy() - want_state).max() <= state_tol * np.abs(want_state).max()
    # one token per request without a request table (a decode batch): request r is token r
    state = dev(state0)
    a1 = a[:4]
    y3 = torch.empty((4, W), dtype=DT[dtype], device=DEV)
    ops.mingru_walk(dev(a1), y3, state, None, dev(slots, torch.int32), dev(np.array([3, 0, 9, 1], dtype=np.int32), torch.int32), 4)
    for r in range(4):
        init = np.zeros(W) if r == 1 else state0[slots[r]].astype(np.float64)
        S, last = pb.mingru_scan(pb.sigmoid(a1[r:r + 1, :W].astype(np.float64)), a1[r:r + 1, W:2 * W].astype(np.float64), init)
        assert np.abs(state.cpu().numpy()[slots[r]] - last).max() < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_bias_and_activation(dtype):
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(0)
    want_fn = {"relu2": pb.relu_squared, "relu": lambda z: np.maximum(z, 0), "silu": lambda z: z * pb.sigmoid(z),
               "gelu_tanh": lambda z: 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3)))}
    for f in (33, 64):
        x, b = bf16_round(rng.randn(5, f) * 2), bf16_round(rng.randn(f))
        for act, fn in want_fn.items():
            got = ops.bias_act(dev(x, DT[dtype]), dev(b, DT[dtype]), act).float().cpu().numpy()
            want = fn(x + b)
            assert np.abs(got - want).max() <= (1e-6 if dtype == "float32" else 8e-3) * max(1.0, np.abs(want).max()), act


@pytest.mark.parametrize("m,n,k", [(300, 512, 256), (2048, 1024, 512), (384, 264, 64), (5, 512, 256)])
@pytest.mark.parametrize("activation", ["relu2", "gelu_tanh", "silu", "relu"])
def test_products_with_bias_and_activation_in_their_epilogue(m, n, k, activation):
    """The tcgen05 product (single CTAs and CTA pairs) and the weight-streaming product with the activation in their
    epilogue against the float64 formula."""
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(m + n)
    x, w, b = bf16_round(rng.randn(m, k)), bf16_round(rng.randn(n, k) / np.sqrt(k)), bf16_round(rng.randn(n))
    fn = {"relu2": pb.relu_squared, "relu": lambda z: np.maximum(z, 0), "silu": lambda z: z * pb.sigmoid(z),
          "gelu_tanh": lambda z: 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3)))}[activation]
    want = fn(x @ w.T + b)
    tol = 1e-2 * max(1.0, np.abs(want).max())
    dx, dw, db = dev(x, torch.bfloat16), dev(w, torch.bfloat16), dev(b, torch.bfloat16)
    if m <= 8:
        got = ops.gemv_bf16_act(dx, dw, db, activation).float().cpu().numpy()
        assert np.abs(got - want).max() <= tol
        return
    for pair in (False, True):
        got = ops.gemm_tcgen05_act(dx, dw, db, activation, pair=pair).float().cpu().numpy()
        assert np.abs(got - want).max() <= tol, f"pair={pair}"
    got = ops.gemm_tcgen05_act(dx, dw, None, activation).float().cpu().numpy()
    assert np.abs(got - fn(x @ w.T)).max() <= tol
    ops.check_tcgen05_errors(dx.device)


# ---- whole models -------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    cache = {}

    def get(name):
        if name not in cache:
            folder = bu.write_model(str(tmp_path_factory.mktemp(f"bigerax_{name}")), bu.CONFIGS[name], seed=len(cache) + 11)
            cache[name] = (folder,) + pb.load_folder(folder)
        return cache[name]

    return get


def check_rows(trace, outputs, reqs, ref, dtype, what):
    got = ru.collect(trace, outputs)
    for rid, toks in reqs.items():
        rows = np.stack([got[(rid, p)] for p in range(len(toks))])
        err = rel_rms(rows, ref[rid])
        assert err.max() <= ROW_TOL[dtype], (f"{what} {dtype} request {rid}: error {err.max():.3g} at position {int(err.argmax())} of {len(toks)}, "
                                             f"first position above the bound: {int(np.argmax(err > ROW_TOL[dtype]))}")
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("P", 16), ("Q", 16), ("R", 8), ("P", 32), ("S", 16)])
def test_every_way_of_cutting_matches_the_plain_implementation(name, page_size, dtype, models):
    folder, cfg, w = models(name)
    reqs = {f"{name}{i}": random_tokens(cfg["vocab"], n, 100 * i + n) for i, n in enumerate(bu.LENGTHS[name])}
    ref = {rid: pb.forward(cfg, w, t) for rid, t in reqs.items()}
    results = {}
    t = ru.Trace()
    for rid, toks in reqs.items():
        ru.whole(t, rid, toks)
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    results["whole"] = check_rows(t, out, reqs, ref, dtype, "whole")
    t = ru.Trace()
    for rid, toks in reqs.items():
        ru.tail_one_by_one(t, rid, toks, 80)                             # longer than every window: it passes over decoded tokens
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    results["tail"] = check_rows(t, out, reqs, ref, dtype, "tail one by one")
    t = ru.Trace()
    for i, (rid, toks) in enumerate(reqs.items()):
        ru.chunks(t, rid, toks, [[17, 7, 5, 3, 2], [2, 64, 3, 31], [33, 2, 2, 16], [2]][i % 4])
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    results["chunks"] = check_rows(t, out, reqs, ref, dtype, "portions")
    t = ru.Trace()
    twice = dict(reqs)
    twice.update({rid + "x": toks for rid, toks in reqs.items()})
    ru.mixed(t, twice, seed=len(name) + page_size)
    out, runner = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    ref2 = dict(ref)
    ref2.update({rid + "x": ref[rid] for rid in reqs})
    results["mixed"] = check_rows(t, out, twice, ref2, dtype, "mixed")
    assert runner.manager.reuses() > 0, "the pool was large enough that no page was used again"
    for g in runner.manager.groups:
        assert runner.manager.free_pages(g) == runner.manager.total_pages(g)
    if dtype == "float32":
        # the 32-bit kernels sum in an order fixed by position: cutting changes nothing at all
        for mode in ("tail", "chunks", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(results[mode][key], row), f"{mode}: {key} differs from the whole run"


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("R", "bfloat16")])
def test_decoding_from_the_first_token(name, dtype, models):
    folder, cfg, w = models(name)
    toks = random_tokens(cfg["vocab"], 200, 5)
    t = ru.Trace()
    ru.chunks(t, "d", toks, [1])
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens())
    check_rows(t, out, {"d": toks}, {"d": pb.forward(cfg, w, toks)}, dtype, "decode from the first token")


def test_a_slot_used_again_starts_clean(models):
    """Two state slots, five requests one after the other and in pairs: a request never sees what the slot's last
    user left (the recurrent state, the previous token)."""
    from mimirmind_b200.engine.loader import load_model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    folder, cfg, w = models("P")
    model, _ = load_model(folder, "float32")
    runner = ModelRunner(model, page_size=16, num_pages=12, max_requests=2)
    reqs = [random_tokens(cfg["vocab"], n, n) for n in (60, 3, 90, 31, 64)]
    ref = [pb.forward(cfg, w, t) for t in reqs]
    assert runner.add_request(0) and runner.add_request(1) and not runner.add_request(2)
    got0 = runner.step([StepEntry(0, reqs[0][:50], [49]), StepEntry(1, reqs[1], [2])]).cpu().numpy()
    runner.release(1)
    assert runner.add_request(2)
    got1 = runner.step([StepEntry(2, reqs[2][:7], [6]), StepEntry(0, reqs[0][50:], [9])]).cpu().numpy()
    runner.release(0)
    assert runner.add_request(3)
    got2 = runner.step([StepEntry(3, reqs[3], [30]), StepEntry(2, reqs[2][7:], [82])]).cpu().numpy()
    runner.release(2), runner.release(3)
    assert runner.add_request(4)
    got3 = runner.step([StepEntry(4, reqs[4], [0, 63])]).cpu().numpy()
    for got, want in ((got0[0], ref[0][49]), (got0[1], ref[1][2]), (got1[0], ref[2][6]), (got1[1], ref[0][59]), (got2[0], ref[3][30]),
                      (got2[1], ref[2][89]), (got3[0], ref[4][0]), (got3[1], ref[4][63])):
        assert rel_rms(got, want) <= ROW_TOL["float32"]


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("Q", "bfloat16")])
def test_greedy_generation_through_the_engine(name, dtype, models):
    """Engine.generate (scheduler, prompt portions, captured decode steps) picks the plain implementation's tokens."""
    from mimirmind_b200 import Engine
    folder, cfg, w = models(name)
    prompts = [random_tokens(cfg["vocab"], n, 40 + n) for n in (5, 17, 33, 64)]
    eng = Engine.from_folder(folder, dtype=dtype, page_size=16, cache_tokens=1024, max_context=512, token_budget=48, max_active=4)
    res = eng.generate(prompts, max_new_tokens=24)
    margin = 1e-4 if dtype == "float32" else 0.12
    exact = 0
    for p, r in zip(prompts, res):
        assert r.stats.generated_tokens == 24 and r.stats.finish_reason == "length"
        toks = list(p)
        for i, tok in enumerate(r.tokens):
            row = pb.forward(cfg, w, toks)[-1]
            best = int(np.argmax(row))
            assert row[tok] >= row[best] - margin, f"token {i}: engine chose {tok} ({row[tok]:.4f}), plain {best} ({row[best]:.4f})"
            exact += tok == best
            toks.append(tok)
    assert exact >= (96 if dtype == "float32" else 80)
    assert eng.runner.manager.free_pages() == eng.runner.manager.total_pages()
    # a second run over the same engine (slots and pages used again) gives the same tokens
    again = eng.generate(prompts, max_new_tokens=24)
    if dtype == "float32":
        assert [r.tokens for r in again] == [r.tokens for r in res]


def test_the_replay_program_on_this_design(models, tmp_path):
    folder, cfg, w = models("R")
    reqs = {f"r{i}": random_tokens(cfg["vocab"], n, 11 + i) for i, n in enumerate([3, 90, 41, 150])}
    ref = {rid: pb.forward(cfg, w, t) for rid, t in reqs.items()}
    t = ru.Trace()
    ru.mixed(t, reqs, seed=3)
    t.step([("last", [1, 2, 3], [])], end=["last"])
    out = ru.run_program(folder, "bfloat16", t, t.max_live_tokens(), str(tmp_path / "out"), cfg["vocab"])
    check_rows(t, out, reqs, ref, "bfloat16", "program")


def test_the_command_line_generates_with_this_design(models, tmp_path):
    """bin/mimirmind: random-weights mode writes a Bigerax folder from its config.json, smoke generates from it and from
    a test model; the greedy tokens of the test model are the plain implementation's."""
    import json
    import os
    import subprocess
    import sys
    from conftest import ROOT
    folder, cfg, w = models("S")
    exe = [sys.executable, os.path.join(ROOT, "bin", "mimirmind")]
    conf = {"defaultModel": "m", "models": [{"id": "m", "path": folder}], "runtime": {"dtype": "float32", "maxContextTokens": 256, "cacheTokens": 512}}
    (tmp_path / "config.json").write_text(json.dumps(conf))
    out = subprocess.run(exe + ["smoke", "--config", str(tmp_path / "config.json"), "--prompt", "5 17 3 150", "--max-new", "6"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    got = [int(t) for t in lines[0].split()]
    assert len(got) == 6 and lines[1] == "generated 6"
    toks = [5, 17, 3, 150]
    for tok in got:
        row = pb.forward(cfg, w, toks)[-1]
        assert row[tok] >= row.max() - 1e-4
        toks.append(tok)
    (tmp_path / "mc.json").write_text(json.dumps(bu.CONFIGS["R"]))
    rw = subprocess.run(exe + ["random-weights", "--model-config", str(tmp_path / "mc.json"), "--seed", "9", "--out", str(tmp_path / "rw"),
                               "--dtype", "bfloat16"], capture_output=True, text=True, timeout=300)
    assert rw.returncode == 0, rw.stderr
    conf["models"][0]["path"] = str(tmp_path / "rw")
    conf["runtime"]["dtype"] = "bfloat16"
    (tmp_path / "config2.json").write_text(json.dumps(conf))
    out = subprocess.run(exe + ["smoke", "--config", str(tmp_path / "config2.json"), "--prompt", "1 2 3", "--max-new", "4"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert out.stdout.strip().splitlines()[1] == "generated 4"


def test_prompt_steps_with_the_feed_forwards_fused_epilogue(models, monkeypatch):
    """The width from which a prompt's up product takes bias and activation as its epilogue is lowered so that a small
    model runs it: same logits as the plain implementation."""
    from mimirmind_b200.parts import mlp
    monkeypatch.setattr(mlp, "FUSED_UP_MIN_HIDDEN", 0)
    folder, cfg, w = models("Q")
    reqs = {"f0": random_tokens(cfg["vocab"], 300, 1), "f1": random_tokens(cfg["vocab"], 257, 2)}
    ref = {rid: pb.forward(cfg, w, t) for rid, t in reqs.items()}
    t = ru.Trace()
    for rid, toks in reqs.items():
        ru.whole(t, rid, toks)
    out, _ = ru.run_in_process(folder, "bfloat16", t, t.max_live_tokens())
    check_rows(t, out, reqs, ref, "bfloat16", "fused feed-forward epilogue")
