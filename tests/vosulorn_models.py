"""Small Vosulorn configurations and model folders for the tests.

Weights are drawn so that nothing hides: decays close to 1 (a state remembers tens of tokens), step sizes around a half,
norms' weights around 1, sinks of the size of a typical score, router matrices large enough for the choice of experts to
change from token to token, matrices wide enough for logits of order 1.  The folders are written in bfloat16 (what a
float32 engine widens exactly), so the plain implementation and the library compute from the same numbers.
"""
import json
import os

import numpy as np
import torch


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def delta(heads, kv_heads, dim, vdim, conv, mlp):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, scale, rot, chunk, mlp):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        m["rot"] = rot
    if chunk:
        m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, rank, scale, base, mlp, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


# Sizes differ in everything from layer to layer and between the two: grouped, multi-query and one key head per query
# head; value heads wider and narrower than key heads; chunks shorter than, equal to and longer than a page of 64;
# rotation of a part of a head and of all of it, with and without stretched wavelengths; delta-rule states of 8, 16, 40
# and 70 rows and of more than 32 columns; 1, 2, 3 and 4 taps; one expert of two, all of five, three of six; layers
# without a feed-forward; a latent read by a later layer with other head counts and sizes.
CFG_A = {"architecture": "Vosulorn", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0}, "layers": [
    delta(4, 2, 16, 24, 4, moe(4, 2, 40)),
    latent(4, 16, 8, 24, 32, 0.2, 10000.0, moe(4, 2, 40)),
    attention(6, 2, 16, 8, 0.3, {"base": 500.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}, 7, None),
    delta(3, 3, 40, 12, 2, moe(3, 1, 56)),
    latent(2, 24, 8, 16, 32, 0.15, 10000.0, moe(5, 5, 16), kv_from=1),
    attention(2, 1, 24, 24, 0.25, {"base": 90.0, "dims": 24}, None, moe(4, 2, 40)),
]}
CFG_B = {"architecture": "Vosulorn", "vocab": 97, "width": 50, "norm": {"eps": 3e-4}, "embedding": {"scale": 0.5}, "layers": [
    attention(3, 3, 10, 14, 0.4, {"base": 77.0, "dims": 6}, 70, moe(2, 1, 30)),
    delta(2, 1, 70, 40, 1, None),
    latent(5, 10, 4, 6, 20, 0.3, 300.0, moe(6, 3, 24)),
    latent(1, 12, 4, 30, 20, 0.35, 300.0, moe(6, 3, 24), kv_from=2),
    delta(6, 2, 8, 8, 3, moe(2, 2, 10)),
    attention(4, 2, 32, 32, 0.17, {"base": 1000.0, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 2.0, "original": 16}}, 64, moe(3, 2, 20)),
]}
CONFIGS = {"a": CFG_A, "b": CFG_B}


def tensors_for(cfg, seed):
    g = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, rows, cols, gain=1.0):
        W[name] = g.normal(0.0, gain / np.sqrt(cols), size=(rows, cols))

    def vec(name, n, lo, hi):
        W[name] = g.uniform(lo, hi, size=(n,))

    W["embed"] = g.normal(0.0, 0.7 / cfg["embedding"]["scale"], size=(V, D))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", D, 0.6, 1.4)
        if L["type"] == "delta":
            H, G, d, e, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for s, n in (("q", G * d), ("k", G * d), ("v", H * e)):
                mat(p + "mix." + s, n, D, 1.5)
                W[p + "mix." + s + ".conv"] = g.normal(0.0, 0.6, size=(n, taps)) + (np.arange(taps) == taps - 1) * 0.8
            mat(p + "mix.b", H, D, 1.5)
            mat(p + "mix.a", H, D, 1.0)
            vec(p + "mix.A_log", H, -4.0, -2.0)
            vec(p + "mix.dt_bias", H, -1.0, 0.5)
            mat(p + "mix.g", H * e, D, 1.5)
            vec(p + "mix.norm", e, 0.6, 1.4)
            mat(p + "mix.o", D, H * e)
        elif L["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for s, n in (("q", H * d), ("k", G * d), ("v", G * e)):
                mat(p + "mix." + s, n, D, 2.0)
                vec(p + "mix." + s + ".b", n, -0.5, 0.5)
            mat(p + "mix.o", D, H * e)
            vec(p + "mix.o.b", D, -0.3, 0.3)
            vec(p + "mix.sink", H, -1.0, 2.0)
        else:
            H, d, rd, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            mat(p + "mix.q", H * (d + rd), D, 2.0)
            if m.get("kv_from") is None:
                mat(p + "mix.dkv", r + rd, D, 2.0)
                vec(p + "mix.dkv.norm", r, 0.6, 1.4)
            mat(p + "mix.uk", H * d, r, 1.5)
            mat(p + "mix.uv", H * e, r, 1.5)
            mat(p + "mix.o", D, H * e)
        if L.get("mlp"):
            E, ff = L["mlp"]["router"]["experts"], L["mlp"]["expert"]["ff"]
            vec(p + "norm2", D, 0.6, 1.4)
            mat(p + "mlp.router", E, D, 3.0)
            vec(p + "mlp.router.b", E, -0.5, 0.5)
            for e_ in range(E):
                mat(f"{p}mlp.e{e_}.gate", ff, D, 1.5)
                mat(f"{p}mlp.e{e_}.up", ff, D, 1.5)
                mat(f"{p}mlp.e{e_}.down", D, ff)
    vec("final.norm", D, 0.6, 1.4)
    mat("head", V, D, 2.0)
    return W


def write_dir(path, cfg, seed, overrides=None):
    """config.json and model.safetensors (bfloat16) for `cfg`; `overrides`: name -> array put in place of the drawn one."""
    from edgelm_b200.weights import write_file
    os.makedirs(path, exist_ok=True)
    W = tensors_for(cfg, seed)
    for k, v in (overrides or {}).items():
        assert k in W and np.shape(v) == W[k].shape, k
        W[k] = np.asarray(v)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(path, "model.safetensors"), {k: torch.tensor(v, dtype=torch.float32).to(torch.bfloat16) for k, v in W.items()})
    return path


def tokens(cfg, n, salt):
    return [int(t) for t in np.random.default_rng(9000 + salt).integers(0, cfg["vocab"], size=n)]
