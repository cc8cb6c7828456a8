"""A plain, slow implementation of the Vosulorn decoder in NumPy float64: one function per mechanism, whole
sequences at a time, no cache and no state (every token is recomputed from the sequence's start).  It shares no
code with the library; the GPU tests compare the library with it.

Notation: x [T, D] the residual stream, eps the norm's epsilon.
  layer:   x += mixer(norm1(x));  x += ff(norm2(x))  (a layer may have no ff);   norm(y) = y / sqrt(mean(y^2) + eps) * w
  mixers:  "delta" (gated delta rule with short convolutions), "attention" (grouped heads, partly rotated with
           neighbouring pairs, chunked mask, a sink in the softmax), "latent_attention" (keys and values expanded from a
           shared low-rank latent, one rotated key part for all heads, optionally read from an earlier layer)
  ff:      a mixture of experts: the `top` largest router logits choose, their softmax weighs
"""
import json
import os

import numpy as np

from plain_llama import read_safetensors

f64 = np.float64


# ----------------------------------------------------------------------------- small functions
def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def rmsnorm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def embed(table, ids, scale):
    return table[np.asarray(ids)] * scale


# ----------------------------------------------------------------------------- rotation
def frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with `scaling` {factor, low, high, original}: wavelengths under
    original/high keep f, those over original/low get f/factor, the ones between are blended linearly in original/l."""
    i = np.arange(dims // 2, dtype=f64)
    f = np.power(f64(base), -2.0 * i / dims)
    if scaling:
        fac, lo, hi, orig = (f64(scaling[k]) for k in ("factor", "low", "high", "original"))
        wl = 2.0 * np.pi / f
        s = (orig / wl - lo) / (hi - lo)
        mid = (1.0 - s) * f / fac + s * f
        f = np.where(wl < orig / hi, f, np.where(wl > orig / lo, f / fac, mid))
    return f


def rotate(x, pos, freq, interleaved):
    """x [T, heads, d]: the first 2 len(freq) dimensions of every head are rotated by pos * freq; pairs are
    (2i, 2i + 1) if `interleaved`, else (i, i + len(freq))."""
    n = len(freq)
    ang = np.asarray(pos, dtype=f64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    if interleaved:
        a, b = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
        out[..., 0:2 * n:2], out[..., 1:2 * n:2] = a * c - b * s, b * c + a * s
    else:
        a, b = x[..., :n], x[..., n:2 * n]
        out[..., :n], out[..., n:2 * n] = a * c - b * s, b * c + a * s
    return out


# ----------------------------------------------------------------------------- attention cores
def masked_softmax_attention(q, k, v, scale, chunk=None, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e].  Token i sees j <= i, with `chunk` only those of its own
    chunk of positions.  `sink` [H]: one more term exp(sink_h) in the denominator, without key or value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), f64)
    idx = np.arange(T)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        seen = idx[None, :] <= idx[:, None]
        if chunk:
            seen &= (idx[None, :] // chunk) == (idx[:, None] // chunk)
        s = np.where(seen, s, -np.inf)
        m = s.max(-1, keepdims=True)
        if sink is not None:
            m = np.maximum(m, sink[h])
        p = np.exp(s - m)
        den = p.sum(-1, keepdims=True)
        if sink is not None:
            den = den + np.exp(sink[h] - m)
        out[:, h] = (p / den) @ v[:, g]
    return out


def attention_mixer(W, p, m, h, eps):
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, d)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, d)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, e)
    rot = m.get("rot")
    if rot:
        f = frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate(q, np.arange(T), f, True), rotate(k, np.arange(T), f, True)
    mask = m.get("mask") or {}
    a = masked_softmax_attention(q, k, v, m["scale"], chunk=mask.get("size"), sink=W.get(p + "sink"))
    return a.reshape(T, H * e) @ W[p + "o"].T + W[p + "o.b"]


def latent_kv(W, p, m, h, eps):
    """The latent c [T, rank] (normed) and the rotated key part [T, rot_dim] that a latent-attention layer keeps."""
    T = h.shape[0]
    r, rd = m["kv_rank"], m["rot_dim"]
    ckr = h @ W[p + "dkv"].T
    c = rmsnorm(ckr[:, :r], W[p + "dkv.norm"], eps)
    f = frequencies(rd, m["rot"]["base"], m["rot"].get("scaling"))
    kr = rotate(ckr[:, None, r:], np.arange(T), f, False)[:, 0]
    return c, kr


def latent_attention_mixer(W, p, m, h, eps, kv):
    """`kv`: (c, rotated key part) of this layer or of the layer it reads."""
    T = h.shape[0]
    H, d, rd, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = kv
    q = (h @ W[p + "q"].T).reshape(T, H, d + rd)
    f = frequencies(rd, m["rot"]["base"], m["rot"].get("scaling"))
    qr = rotate(q[..., d:], np.arange(T), f, False)
    kn = (c @ W[p + "uk"].T).reshape(T, H, d)
    v = (c @ W[p + "uv"].T).reshape(T, H, e)
    qq = np.concatenate([q[..., :d], qr], axis=-1)
    kk = np.concatenate([kn, np.broadcast_to(kr[:, None, :], (T, H, rd))], axis=-1)
    a = masked_softmax_attention(qq, kk, v, m["scale"])
    return a.reshape(T, H * e) @ W[p + "o"].T


# ----------------------------------------------------------------------------- gated delta rule
def causal_conv_silu(x, w):
    """x [T, C], w [C, taps] (last column: the current token), zeros before the start, no bias."""
    T, C = x.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), f64), x], axis=0)
    out = np.zeros((T, C), f64)
    for j in range(taps):
        out += padded[j:j + T] * w[:, j]
    return silu(out)


def unit_vectors(x):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)


def delta_recurrence(q, k, v, beta, g):
    """q, k [T, H, d], v [T, H, e], beta and g [T, H].  Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q (the read-out sees the token's own write)."""
    T, H, d = q.shape
    o = np.zeros_like(v)
    for h in range(H):
        S = np.zeros((d, v.shape[2]), f64)
        for t in range(T):
            S = g[t, h] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, h])
            S = S + np.outer(k[t, h], u)
            o[t, h] = S.T @ q[t, h]
    return o


def delta_mixer(W, p, m, h, eps):
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ W[p + "q"].T, W[p + "q.conv"]).reshape(T, G, d)
    k = causal_conv_silu(h @ W[p + "k"].T, W[p + "k.conv"]).reshape(T, G, d)
    v = causal_conv_silu(h @ W[p + "v"].T, W[p + "v.conv"]).reshape(T, H, e)
    q, k = unit_vectors(q) * d ** -0.5, unit_vectors(k)
    rep = H // G
    q, k = np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1)       # head h uses q/k head h // rep
    beta = sigmoid(h @ W[p + "b"].T)
    g = np.exp(-np.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    o = delta_recurrence(q, k, v, beta, g)
    o = o / np.sqrt((o * o).mean(-1, keepdims=True) + eps) * W[p + "norm"]
    o = o.reshape(T, H * e) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# ----------------------------------------------------------------------------- feed-forward
def router(W, p, r, h):
    """Chosen experts [T, top] (largest logits first) and their weights (softmax over the chosen logits)."""
    z = h @ W[p + "router"].T + W[p + "router.b"]
    order = np.argsort(-z, axis=-1, kind="stable")[:, :r["top"]]
    zc = np.take_along_axis(z, order, axis=-1)
    w = np.exp(zc - zc.max(-1, keepdims=True))
    return order, w / w.sum(-1, keepdims=True)


def expert(W, p, h):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def moe(W, p, mlp, h):
    chosen, weights = router(W, p, mlp["router"], h)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            out[t] += w * expert(W, f"{p}e{e}.", h[t:t + 1])[0]
    return out


# ----------------------------------------------------------------------------- the model
def forward(cfg, W, ids, layers_out=None):
    """Logits [T, vocab] of one sequence from its start.  `layers_out`: a list that receives x after every layer."""
    eps = cfg["norm"]["eps"]
    x = embed(W["embed"], ids, cfg["embedding"]["scale"])
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = rmsnorm(x, W[p + "norm1"], eps)
        if L["type"] == "delta":
            y = delta_mixer(W, p + "mix.", m, h, eps)
        elif L["type"] == "attention":
            y = attention_mixer(W, p + "mix.", m, h, eps)
        elif L["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_kv(W, p + "mix.", m, h, eps)
            y = latent_attention_mixer(W, p + "mix.", m, h, eps, kept[m["kv_from"] if m.get("kv_from") is not None else i])
        else:
            raise ValueError(L["type"])
        x = x + y
        if L.get("mlp") is not None:
            x = x + moe(W, p + "mlp.", L["mlp"], rmsnorm(x, W[p + "norm2"], eps))
        if layers_out is not None:
            layers_out.append(x.copy())
    return rmsnorm(x, W["final.norm"], eps) @ W["head"].T


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    W = {k: np.asarray(v, dtype=f64) for k, v in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, W
