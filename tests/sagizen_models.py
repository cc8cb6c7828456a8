"""Small Sagizen configurations and model folders for the tests.

Weights are drawn so that nothing hides: decays close to 1 (a state remembers tens of tokens), blends anywhere
between a token and the one before it, norms' weights around 1, matrices wide enough for logits of order 1.
The folders are written in bfloat16 (what a float32 engine widens exactly), so the plain implementation and the
library compute from the same numbers.
"""
import json
import os

import numpy as np
import torch


def mamba(heads, vdim, state, groups, conv, norm_groups, ff):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def parallel(heads, kv_heads, dim, vdim, size, pool, rot, scale, r_heads, r_dim, ls, rs, ff):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size, "pool": pool}, "scale": scale}
    if rot:
        left["rot"] = rot
    return {"type": "parallel", "mixer": {"left": left, "left_scale": ls, "right": {"heads": r_heads, "dim": r_dim}, "right_scale": rs},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


# Sizes differ in everything from layer to layer and between the two: grouped, multi-query and one key head per query
# head; value heads wider and narrower than key heads; windows shorter and longer than a pooled block; blocks that
# do and do not divide a page of 64; rotation of a part of a head and of all of it, with and without scaled positions;
# states of 16, 40 and 70 rows (one, two and three registers a lane); 1, 2, 3 and 4 taps; layers without a feed-forward.
CFG_A = {"architecture": "Sagizen", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "layers": [
    mamba(4, 8, 16, 2, 4, 2, 96),
    parallel(4, 2, 16, 24, 7, 3, {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0}}, 0.3, 2, 32, 0.7, 1.3, None),
    mamba(3, 12, 40, 3, 2, 1, 80),
    parallel(3, 3, 24, 8, 70, 64, {"base": 500.0, "dims": 24}, 0.25, 4, 16, 1.0, 0.5, 48),
]}
CFG_B = {"architecture": "Sagizen", "vocab": 97, "width": 50, "norm": {"eps": 3e-4}, "layers": [
    parallel(6, 1, 10, 14, 4, 9, {"base": 77.0, "dims": 6, "scaling": {"factor": 1.5}}, 0.4, 5, 10, 1.5, 0.25, 70),
    mamba(6, 6, 70, 1, 3, 3, None),
    mamba(2, 24, 8, 2, 1, 2, 30),
    parallel(2, 2, 32, 32, 33, 5, None, 0.2, 1, 40, 0.9, 1.1, 64),
]}
DECAY_RANK = {"a": 24, "b": 5}     # the rank of the decay's projection is a size that only the tensors' shapes give
CONFIGS = {"a": CFG_A, "b": CFG_B}


def tensors_for(cfg, seed, decay_rank):
    g = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, rows, cols, gain=1.0):
        W[name] = g.normal(0.0, gain / np.sqrt(cols), size=(rows, cols))

    def vec(name, n, lo, hi):
        W[name] = g.uniform(lo, hi, size=(n,))

    W["embed"] = g.normal(0.0, 0.7, size=(V, D))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", D, 0.6, 1.4)
        vec(p + "shift", D, 0.0, 1.0)
        if L["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, C = H * P, H * P + 2 * G * N
            mat(p + "mix.in", 2 * inner + 2 * G * N + H, D, 1.5)
            W[p + "mix.conv"] = g.normal(0.0, 0.6, size=(C, m["conv"]))
            vec(p + "mix.conv.b", C, -0.2, 0.2)
            vec(p + "mix.dt_bias", H, -1.0, 0.5)
            vec(p + "mix.A_log", H, -4.0, -2.0)
            vec(p + "mix.D", H, 0.5, 1.5)
            vec(p + "mix.norm", inner, 0.6, 1.4)
            mat(p + "mix.o", D, inner)
        else:
            l, r = m["left"], m["right"]
            for s, n in (("q", l["heads"] * l["dim"]), ("k", l["kv_heads"] * l["dim"]), ("v", l["kv_heads"] * l["vdim"])):
                mat(p + "mix.left." + s, n, D, 1.5)
                vec(p + "mix.left." + s + ".b", n, -0.5, 0.5)
            mat(p + "mix.left.o", D, l["heads"] * l["vdim"])
            inner = r["heads"] * r["dim"]
            for s in "rkvgw":
                vec(p + "mix.right.mu." + s, D, 0.0, 1.0)
            for s in "rkvg":
                mat(p + "mix.right." + s, inner, D, 1.2)
            mat(p + "mix.right.w1", decay_rank, D)
            mat(p + "mix.right.w2", inner, decay_rank)
            vec(p + "mix.right.w0", inner, -5.0, -2.0)
            W[p + "mix.right.u"] = g.uniform(0.0, 1.0, size=(r["heads"], r["dim"]))
            vec(p + "mix.right.norm", inner, 0.6, 1.4)
            mat(p + "mix.right.o", D, inner)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            vec(p + "norm2", D, 0.6, 1.4)
            mat(p + "mlp.gate", ff, D, 1.5)
            mat(p + "mlp.up", ff, D, 1.5)
            mat(p + "mlp.down", D, ff)
    vec("final.norm", D, 0.6, 1.4)
    mat("head", V, D, 2.0)
    return W


def write_dir(path, cfg, seed, decay_rank=24, overrides=None):
    """config.json and model.safetensors (bfloat16) for `cfg`; `overrides`: name -> array put in place of the drawn one."""
    from edgelm_b200.weights import write_file
    os.makedirs(path, exist_ok=True)
    W = tensors_for(cfg, seed, decay_rank)
    for k, v in (overrides or {}).items():
        assert k in W and np.shape(v) == W[k].shape, k
        W[k] = np.asarray(v)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(path, "model.safetensors"), {k: torch.tensor(v, dtype=torch.float32).to(torch.bfloat16) for k, v in W.items()})
    return path


def tokens(cfg, n, salt):
    return [int(t) for t in np.random.default_rng(7000 + salt).integers(0, cfg["vocab"], size=n)]
