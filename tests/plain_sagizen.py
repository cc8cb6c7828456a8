"""A plain, slow implementation of the Sagizen decoder in NumPy float64: one function per mechanism, whole
sequences at a time, no cache and no state (every token is recomputed from the sequence's start).  It shares no
code with the library; the GPU tests compare the library with it.

Notation: x [T, D] the residual stream, h the mixer's input, eps the norm's epsilon.
  layer:        h_t = x_t + (x_(t-1) - x_t) * shift;  x += norm1(mixer(h));  x += norm2(ff(x))      (norm on the OUTPUT)
  norm(y):      y / sqrt(mean(y^2) + eps) * w
"""
import json
import os

import numpy as np

from plain_llama import read_safetensors

f64 = np.float64


# ----------------------------------------------------------------------------- small functions
def silu(z):
    return z / (1.0 + np.exp(-z))


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rmsnorm(x, w, eps):
    return unit_rms(x, eps) * w


def previous_rows(h):
    """Row t holds h[t - 1]; zeros for the first token."""
    return np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)


def token_shift(h, mu):
    """h + (h' - h) * mu with h' the previous token's h."""
    return h + (previous_rows(h) - h) * mu


# ----------------------------------------------------------------------------- state-space mixer
def causal_conv_silu(x, w, b):
    """x [T, C], w [C, taps] (last column: the current token), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), f64), x], axis=0)
    out = np.zeros((T, C), f64)
    for j in range(taps):
        out += padded[j:j + T] * w[:, j]
    return silu(out + b)


def ssm_recurrence(x, B, C, dt, A_log, D, groups):
    """x [T, H, P], B and C [T, G, N], dt [T, H] (after softplus).  S_t = exp(-exp(A_log) dt) S + dt B x^T; y = S^T C + D x."""
    T, H, P = x.shape
    N = B.shape[2]
    y = np.zeros((T, H, P), f64)
    for h in range(H):
        g = h // (H // groups)
        S = np.zeros((N, P), f64)
        a = -np.exp(A_log[h])
        for t in range(T):
            S = np.exp(a * dt[t, h]) * S + dt[t, h] * np.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * x[t, h]
    return y


def mamba2_mixer(W, p, m, h, eps):
    T = h.shape[0]
    H, P, N, G, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * P
    u = h @ W[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = causal_conv_silu(xbc, W[p + "conv"], W[p + "conv.b"])
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    y = ssm_recurrence(x, B, C, softplus(dt + W[p + "dt_bias"]), W[p + "A_log"], W[p + "D"], G)
    y = y.reshape(T, inner) * silu(z)                                   # the gate comes before the norm
    y = unit_rms(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


# ----------------------------------------------------------------------------- attention with a window and pooled blocks
def rotate_partial(x, positions, dims, base, factor):
    """x [T, heads, d]: the first `dims` dimensions rotated, i paired with i + dims/2, angle p * base^(-2i/dims) / factor."""
    if not dims:
        return x
    half = dims // 2
    f = base ** (-2.0 * np.arange(half, dtype=f64) / dims) / factor
    ang = np.asarray(positions, f64)[:, None] * f[None]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def visible(i, window, pool):
    """What position i sees: the token positions, and the indices of the pooled blocks."""
    tokens = [j for j in range(i + 1) if 0 <= i - j < window]
    blocks = []
    if pool:
        b = 0
        while b * pool + pool - 1 <= i - window:
            blocks.append(b)
            b += 1
    return tokens, blocks


def pooled_window_attention(q, k, v, scale, window, pool):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]; one softmax over the window's tokens and the seen blocks."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), f64)
    for i in range(T):
        tokens, blocks = visible(i, window, pool)
        for h in range(H):
            g = h // (H // G)
            ks = [k[j, g] for j in tokens] + [k[b * pool:(b + 1) * pool, g].mean(0) for b in blocks]
            vs = [v[j, g] for j in tokens] + [v[b * pool:(b + 1) * pool, g].mean(0) for b in blocks]
            s = np.array(ks) @ q[i, h] * scale
            w = np.exp(s - s.max())
            out[i, h] = (w / w.sum()) @ np.array(vs)
    return out


def left_mixer(W, p, m, h, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, dk)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, dk)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_partial(q, range(T), rot["dims"], rot["base"], factor)
        k = rotate_partial(k, range(T), rot["dims"], rot["base"], factor)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    o = pooled_window_attention(q, k, v, m["scale"], m["mask"]["size"], m["mask"].get("pool"))
    return o.reshape(T, H * dv) @ W[p + "o"].T


# ----------------------------------------------------------------------------- time mix with a matrix state
def decay_from_lowrank(x, w1, w2, w0):
    return np.exp(-np.exp(np.tanh(x @ w1.T) @ w2.T + w0))


def wkv_recurrence(r, k, v, w, u):
    """r, k, v, w [T, H, K], u [H, K]: o_t = (S + diag(u) k v^T)^T r; S = diag(w) S + k v^T."""
    T, H, K = r.shape
    o = np.zeros((T, H, K), f64)
    for h in range(H):
        S = np.zeros((K, K), f64)
        for t in range(T):
            kv = np.outer(k[t, h], v[t, h])
            o[t, h] = (S + u[h][:, None] * kv).T @ r[t, h]
            S = w[t, h][:, None] * S + kv
    return o


def right_mixer(W, p, m, h, eps):
    T = h.shape[0]
    H, K = m["heads"], m["dim"]
    blend = {s: token_shift(h, W[p + "mu." + s]) for s in "rkvgw"}
    r, k, v = [(blend[s] @ W[p + s].T).reshape(T, H, K) for s in "rkv"]
    gate = silu(blend["g"] @ W[p + "g"].T)
    w = decay_from_lowrank(blend["w"], W[p + "w1"], W[p + "w2"], W[p + "w0"]).reshape(T, H, K)
    o = unit_rms(wkv_recurrence(r, k, v, w, W[p + "u"]), eps).reshape(T, H * K)
    return (o * W[p + "norm"] * gate) @ W[p + "o"].T


# ----------------------------------------------------------------------------- the model
def dense_ff(W, p, h):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of the whole sequence."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    layers = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = token_shift(x, W[p + "shift"])
        m = L["mixer"]
        if L["type"] == "mamba2":
            y = mamba2_mixer(W, p + "mix.", m, h, eps)
        else:
            y = m["left_scale"] * left_mixer(W, p + "mix.left.", m["left"], h, eps) + \
                m["right_scale"] * right_mixer(W, p + "mix.right.", m["right"], h, eps)
        x = x + rmsnorm(y, W[p + "norm1"], eps)
        if L.get("mlp"):
            x = x + rmsnorm(dense_ff(W, p + "mlp.", x), W[p + "norm2"], eps)
        layers.append(x.copy())
    logits = rmsnorm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, layers) if return_layers else logits


def generate_greedy(cfg, W, prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        t = int(forward(cfg, W, seq)[-1].argmax())
        out.append(t)
        seq.append(t)
    return out


def read_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    W = {}
    for fn in sorted(os.listdir(model_dir)):
        if fn.endswith(".safetensors"):
            W.update({k: np.asarray(v, f64) for k, v in read_safetensors(os.path.join(model_dir, fn)).items()})
    return cfg, W
