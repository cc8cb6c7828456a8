"""The kernels of the state mixers and of the window attention with pooled blocks, each alone against the plain
implementation's function for the same mechanism, on packed batches of unequal sequences, over several steps (the
state, the previous rows and the pooled rows come from the step before), on slots and pages in no particular order,
at sizes that fill a lane's registers unevenly.  Inputs are made so that one far key decides the result: a key that
is seen, not seen, or seen through its block changes the output by much more than any tolerance."""
import numpy as np
import pytest
import torch

import plain_sagizen as plain
from edgelm_b200.csrc import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def f32(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=DEV).contiguous()


def packed(lengths):
    tok0 = np.concatenate([[0], np.cumsum(lengths)])
    tok_seq = np.repeat(np.arange(len(lengths)), lengths)
    return i32(tok0), i32(tok_seq)


def steps_of(total, cuts):
    """Per step the (start, count) of every sequence: sequence s of length total[s] is fed in pieces of cuts[s]."""
    n_steps = max(len(c) for c in cuts)
    at = [0] * len(total)
    out = []
    for k in range(n_steps):
        step = []
        for s, c in enumerate(cuts):
            n = c[k] if k < len(c) else 0
            step.append((at[s], n))
            at[s] += n
        out.append(step)
    assert at == list(total)
    return out


@pytest.mark.parametrize("N,P,H,G", [(40, 12, 3, 3), (16, 8, 4, 2), (70, 5, 2, 1), (200, 3, 1, 1)])
def test_state_space_scan_over_steps(N, P, H, G):
    g = np.random.default_rng(N)
    total, cuts, slots = [43, 6, 1], [[5, 1, 37], [2, 4], [1]], [4, 0, 2]
    inner, C = H * P, H * P + 2 * G * N
    xbc = [g.normal(size=(n, C)) for n in total]
    dtr = [g.normal(size=(n, H)) for n in total]
    dt_bias, A_log, D = g.uniform(-1, 0.5, H), g.uniform(-4, -1, H), g.normal(size=H)
    want = [plain.ssm_recurrence(x[:, :inner].reshape(-1, H, P), x[:, inner:inner + G * N].reshape(-1, G, N), x[:, inner + G * N:].reshape(-1, G, N),
                                 plain.softplus(d + dt_bias), A_log, D, G).reshape(-1, inner) for x, d in zip(xbc, dtr)]
    state = torch.zeros(6, H, P, N, device=DEV)
    state[1].fill_(float("nan"))      # a slot of nobody: never read
    got = [np.zeros_like(w) for w in want]
    for step in steps_of(total, cuts):
        live = [(s, a, n) for s, (a, n) in enumerate(step) if n]
        tok0, _ = packed([n for _, _, n in live])
        x = f32(np.concatenate([xbc[s][a:a + n] for s, a, n in live]))
        u = f32(np.concatenate([dtr[s][a:a + n] for s, a, n in live]))
        y = torch.full((x.shape[0], inner), float("nan"), device=DEV)
        ops.ssm_scan(x, u, 0, f32(dt_bias), f32(A_log), f32(D), state, y, tok0, i32([slots[s] for s, _, _ in live]), len(live), H, G, N, P)
        y = y.cpu().numpy()
        at = 0
        for s, a, n in live:
            got[s][a:a + n] = y[at:at + n]
            at += n
    for w, o in zip(want, got):
        assert np.abs(o - w).max() < 2e-5 * max(1.0, np.abs(w).max())


@pytest.mark.parametrize("K,H", [(40, 2), (16, 3), (70, 1), (130, 1)])
def test_decayed_outer_product_scan_over_steps(K, H):
    g = np.random.default_rng(K)
    total, cuts, slots = [50, 3, 9], [[1, 2, 47], [3], [4, 4, 1]], [1, 3, 0]
    r, k, v = [[g.normal(size=(n, H, K)) * 0.5 for n in total] for _ in range(3)]
    w = [g.uniform(0.8, 0.999, size=(n, H, K)) for n in total]
    u = g.uniform(0, 1, size=(H, K))
    want = [plain.wkv_recurrence(r[s], k[s], v[s], w[s], u).reshape(-1, H * K) for s in range(3)]
    state = torch.zeros(5, H, K, K, device=DEV)
    got = [np.zeros_like(x) for x in want]
    for step in steps_of(total, cuts):
        live = [(s, a, n) for s, (a, n) in enumerate(step) if n]
        tok0, _ = packed([n for _, _, n in live])
        cat = lambda src: f32(np.concatenate([src[s][a:a + n].reshape(n, H * K) for s, a, n in live]))
        o = torch.full((int(tok0[-1]), H * K), float("nan"), device=DEV)
        ops.wkv_scan(cat(r), cat(k), cat(v), cat(w), f32(u), state, o, tok0, i32([slots[s] for s, _, _ in live]), len(live), H, K)
        o = o.cpu().numpy()
        at = 0
        for s, a, n in live:
            got[s][a:a + n] = o[at:at + n]
            at += n
    for x, o in zip(want, got):
        assert np.abs(o - x).max() < 2e-5 * max(1.0, np.abs(x).max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_blend_convolution_and_norms(dtype):
    g = np.random.default_rng(5)
    lengths, slots, D = [4, 1, 2], [2, 0, 1], 24
    tok0, tok_seq = packed(lengths)
    seqslot = i32(slots)
    x = g.normal(size=(7, D))
    prev = g.normal(size=(3, D))          # the state rows: what the step before left
    mu = g.uniform(0, 1, size=(5, D))
    state = f32(prev)
    out = torch.empty(5, 7, D, dtype=dtype, device=DEV)
    xin = f32(x).to(dtype)
    ops.shift_mix(xin, state, f32(mu), out, tok_seq, tok0, seqslot)
    xr = xin.float().cpu().numpy().astype(np.float64)
    before = np.concatenate([np.concatenate([prev[slots[s]][None].astype(np.float32), xr[a:b - 1]]) for s, (a, b) in enumerate(zip(tok0.tolist(), tok0.tolist()[1:]))])
    want = xr[None] + (before - xr)[None] * mu[:, None].astype(np.float32)
    tol = 1e-6 if dtype == torch.float32 else 2e-2
    assert np.abs(out.float().cpu().numpy() - want).max() < tol
    ops.save_last_rows(xin, state, tok0, seqslot, 3)
    assert np.array_equal(state.cpu().numpy()[slots], xr[[3, 4, 6]].astype(np.float32))
    # convolution: taps 4, steps of 4, 1 and 2 tokens on top of a tail of 3 rows
    C, taps = 10, 4
    u = g.normal(size=(7, C + 3))
    w, b = g.normal(size=(C, taps)), g.normal(size=C)
    tail = g.normal(size=(3, taps - 1, C))
    cstate = f32(tail)
    y = torch.empty(7, C, device=DEV)
    ops.conv_silu(f32(u), 2, f32(w), f32(b), cstate, y, tok_seq, tok0, seqslot, 3)
    for s, (a, e) in enumerate(zip(tok0.tolist(), tok0.tolist()[1:])):
        full = np.concatenate([tail[slots[s]], u[a:e, 2:2 + C]])
        ref = plain.causal_conv_silu(full, w, b)[taps - 1:]
        assert np.abs(y[a:e].cpu().numpy() - ref).max() < 1e-5
        assert np.allclose(cstate[slots[s]].cpu().numpy(), full[-(taps - 1):], atol=1e-6)
    # gated group norm, both orders; the norm on a sublayer's output with the residual sum
    yv, gate, wn = g.normal(size=(7, 24)), g.normal(size=(7, 30)), g.uniform(0.5, 1.5, 24)
    for first in (True, False):
        o = torch.empty(7, 24, dtype=dtype, device=DEV)
        ops.gated_group_norm(f32(yv), f32(gate)[:, 3:27], f32(wn), o, 3, 1e-4, first)
        gt = plain.silu(gate[:, 3:27])
        ref = plain.unit_rms((yv * gt).reshape(7, 3, 8), 1e-4).reshape(7, 24) * wn if first else plain.unit_rms(yv.reshape(7, 3, 8), 1e-4).reshape(7, 24) * wn * gt
        assert np.abs(o.float().cpu().numpy() - ref).max() < (1e-5 if dtype == torch.float32 else 3e-2)
    xs, y1, y2 = g.normal(size=(7, 24)), g.normal(size=(7, 24)), g.normal(size=(7, 24))
    xd, cast = f32(xs), torch.empty(7, 24, dtype=dtype, device=DEV)
    ops.rmsnorm_add(xd, f32(y1), f32(wn), 1e-3, a=1.2, y2=f32(y2), b=0.7, cast=cast)
    ref = xs + plain.rmsnorm(1.2 * y1 + 0.7 * y2, wn, 1e-3)
    assert np.abs(xd.cpu().numpy() - ref).max() < 1e-5 and np.abs(cast.float().cpu().numpy() - ref).max() < (1e-5 if dtype == torch.float32 else 3e-2)
    a = g.normal(size=(7, 6))
    w2, w0 = g.normal(size=(24, 6)), g.uniform(-4, -1, 24)
    dec = torch.empty(7, 24, device=DEV)
    w2d = f32(w2).to(dtype)
    ops.lowrank_decay(f32(a), w2d, f32(w0), dec)
    ref = np.exp(-np.exp(np.tanh(a) @ w2d.float().cpu().numpy().astype(np.float64).T + w0))
    assert np.abs(dec.cpu().numpy() - ref).max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,pool,dk,dv,H,G", [(9, 4, 20, 12, 4, 2), (3, 7, 40, 72, 2, 1), (70, 64, 16, 16, 3, 3), (5, 1, 33, 8, 2, 2)])
def test_window_attention_with_pooled_blocks(dtype, window, pool, dk, dv, H, G):
    """Two sequences side by side through prompt pieces and single tokens.  In the first, key 37 (its block too) is far
    larger than every other along the direction all queries point in: where it is seen it takes almost all the weight."""
    g = np.random.default_rng(window * 100 + pool)
    PAGE = 64
    total = [150, 70]
    cuts = [[41] + [1] * 19 + [90], [1, 2, 3] + [1] * 17 + [47]]
    q = [g.normal(size=(n, H, dk)) * 0.3 for n in total]
    k = [g.normal(size=(n, G, dk)) * 0.3 for n in total]
    v = [g.normal(size=(n, G, dv)) for n in total]
    q[0][:, :, 0] += 3.0
    k[0][37, :, 0] += 12.0
    scale = 0.5
    rnd = lambda a: f32(a).to(dtype).float().cpu().numpy().astype(np.float64)     # what the cache holds
    want = [plain.pooled_window_attention(rnd(q[s]), rnd(k[s]), rnd(v[s]), scale, window, pool).reshape(total[s], H * dv) for s in range(2)]
    w0 = want[0].reshape(150, H, dv)
    seen_as_token, unseen, seen_as_block = 37 + window - 1, 37 + window, (37 // pool) * pool + pool - 1 + window
    if seen_as_block > unseen:     # (the block is complete and behind the window later than the token leaves it)
        assert np.abs(w0[seen_as_token] - w0[unseen]).max() > 0.3 and np.abs(w0[seen_as_block] - w0[seen_as_block - 1]).max() > 0.05
    n_pages, R = 8, -(-PAGE // pool)
    kc = torch.full((n_pages, G, PAGE, dk), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full((n_pages, G, PAGE, dv), float("nan"), dtype=dtype, device=DEV)
    pk = torch.full((n_pages, G, R, dk), float("nan"), device=DEV)
    pv = torch.full((n_pages, G, R, dv), float("nan"), device=DEV)
    table = i32([[5, 2, 7, -1], [0, 6, -1, -1]])
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = [np.zeros_like(w) for w in want]
    got_tiled = [np.zeros_like(w) for w in want]
    for step in steps_of(total, cuts):
        live = [(s, a, n) for s, (a, n) in enumerate(step) if n]
        T = sum(n for _, _, n in live)
        tok_pos = i32(np.concatenate([np.arange(a, a + n) for _, a, n in live]))
        tok_seq = i32(np.concatenate([np.full(n, s) for s, _, n in live]))     # rows of the page table: here the sequences themselves
        qkv = f32(np.concatenate([np.concatenate([q[s][a:a + n].reshape(n, -1), k[s][a:a + n].reshape(n, -1), v[s][a:a + n].reshape(n, -1)], 1) for s, a, n in live]))
        qd = torch.empty(T, H * dk, dtype=dtype, device=DEV)
        ops.qk_rope_norm_append(qkv, None, qd, tok_pos, tok_seq, table, kc, vc, H, G, dk, dv, 0, None, 0.0, False, err)
        ops.pool_blocks(tok_pos, tok_seq, table, kc, vc, pk, pv, T, G, dk, dv, pool, err)
        out = torch.full((T, H * dv), float("nan"), dtype=dtype, device=DEV)
        ops.pooled_window_attn(qd, out, kc, vc, pk, pv, tok_pos, tok_seq, table, H, G, dk, dv, scale, window, pool)
        # the prompt kernel on the same step: runs of at most 32 / (H / G) tokens, 32 rows a block
        from edgelm_b200.engine.batch import make_tiles
        tile_tokens = max(1, 32 // (H // G))
        assert [s for s, _, _ in live] == list(range(len(live)))      # (a tile's sequence index is its row of the page table)
        cols = make_tiles([n for _, _, n in live], [a for _, a, _ in live], tile_tokens)
        out_t = torch.full((T, H * dv), float("nan"), dtype=dtype, device=DEV)
        ops.pooled_window_attn_tiled(qd, out_t, kc, vc, pk, pv, table, i32(cols[0]), i32(cols[1]), i32(cols[2]), i32(cols[3]), len(cols[0]),
                                     tile_tokens, H, G, dk, dv, scale, window, pool)
        out, out_t = out.float().cpu().numpy(), out_t.float().cpu().numpy()
        at = 0
        for s, a, n in live:
            got[s][a:a + n] = out[at:at + n]
            got_tiled[s][a:a + n] = out_t[at:at + n]
            at += n
    assert int(err.item()) == 0
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for w, o, ot in zip(want, got, got_tiled):
        assert np.isfinite(o).all() and np.abs(o - w).max() < tol * max(1.0, np.abs(w).max())
        assert np.isfinite(ot).all() and np.abs(ot - w).max() < tol * max(1.0, np.abs(w).max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_bias_and_unit_norm(dtype):
    g = np.random.default_rng(9)
    H, G, dk, dv, rot, eps = 3, 1, 20, 6, 12, 1e-4
    pos = np.array([0, 1, 63, 64, 1000, 250000])
    T = len(pos)
    qkv = g.normal(size=(T, (H + G) * dk + G * dv))
    bias = g.normal(size=qkv.shape[1])
    freq = 1e4 ** (-2.0 * np.arange(rot // 2) / rot) / 3.0
    n_pages = 250000 // 64 + 1
    kc = torch.zeros((n_pages, G, 64, dk), dtype=dtype, device=DEV)
    vc = torch.zeros((n_pages, G, 64, dv), dtype=dtype, device=DEV)
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(1, -1)
    qd = torch.empty(T, H * dk, dtype=dtype, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.qk_rope_norm_append(f32(qkv), f32(bias), qd, i32(pos), i32(np.zeros(T)), table, kc, vc, H, G, dk, dv, rot,
                            torch.tensor(freq, dtype=torch.float64, device=DEV), eps, True, err)
    x = qkv.astype(np.float32).astype(np.float64) + bias.astype(np.float32)
    qk = plain.unit_rms(plain.rotate_partial(x[:, :(H + G) * dk].reshape(T, H + G, dk), pos, rot, 1e4, 3.0), eps)
    tol = 3e-6 if dtype == torch.float32 else 2e-2
    assert np.abs(qd.float().cpu().numpy().reshape(T, H, dk) - qk[:, :H]).max() < tol
    for i, p in enumerate(pos):
        assert np.abs(kc[p // 64, 0, p % 64].float().cpu().numpy() - qk[i, H]).max() < tol
        assert np.abs(vc[p // 64, 0, p % 64].float().cpu().numpy() - x[i, (H + G) * dk:]).max() < tol
    assert int(err.item()) == 0
