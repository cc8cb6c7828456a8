"""Host-side parts of the Sagizen decoder: the configuration reader and its plan, the tensor names and shapes, what
the layers keep in the cache, and the plain implementation's own mechanisms against brute force."""
import copy

import numpy as np
import pytest
import torch

import plain_sagizen as plain
import sagizen_models as M
from edgelm_b200.cache import CompositeEntry, SequenceCache
from edgelm_b200.config import ConfigError, config_class_for
from edgelm_b200.engine.model import DecoderModel
from edgelm_b200.parts import KVNeed, NeedSet, StateNeed


@pytest.mark.parametrize("name", ["a", "b"])
def test_plan_names_every_tensor_with_its_shape(name):
    cfg = M.CONFIGS[name]
    conf = config_class_for(cfg).from_dict(cfg)
    assert type(conf).__name__ == "SagizenConfig"
    W = M.tensors_for(cfg, 0, M.DECAY_RANK[name])
    conf = conf.shape_given_sizes({k: v.shape for k, v in W.items()})      # the decay's rank comes from a tensor's shape
    want = DecoderModel(conf.plan(), torch.float32).expected_weights()
    assert {k: tuple(v) for k, v in want.items()} == {k: tuple(v.shape) for k, v in W.items()}
    again = config_class_for(conf.to_dict()).from_dict(conf.to_dict())
    assert again.plan() == conf.plan()


def test_refusals():
    for change, text in ((lambda c: c["layers"][0].update(type="conv"), "not part of this architecture"),
                         (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "kind 'experts'"),
                         (lambda c: c["layers"][0]["mixer"].pop("state"), "'state' is missing"),
                         (lambda c: c.pop("norm"), "'norm'"),
                         (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "multiple")):
        cfg = copy.deepcopy(M.CFG_A)
        change(cfg)
        with pytest.raises(ConfigError, match=text):
            DecoderModel(config_class_for(cfg).from_dict(cfg).plan(), torch.float32)


def test_what_the_layers_keep():
    cfg = M.CFG_A
    model = DecoderModel(config_class_for(cfg).from_dict(cfg).plan(), torch.bfloat16)
    needs = model.cache_needs()
    m0 = dict(needs[0].items)
    assert m0["shift"] == StateNeed((64,))
    assert dict(m0["mixer"].items) == {"conv": StateNeed((3, 4 * 8 + 2 * 2 * 16)), "ssm": StateNeed((4, 8, 16))}
    p1 = dict(dict(needs[1].items)["mixer"].items)
    assert p1["left"] == KVNeed(2, 16, None, v_head_dim=24, pool=3)
    assert dict(p1["right"].items) == {"last": StateNeed((64,)), "wkv": StateNeed((2, 32, 32))}
    cache = SequenceCache(needs, max_tokens=256, max_positions=1 << 20)
    assert all(isinstance(e, CompositeEntry) for e in cache.entries)
    assert len(cache.kv_groups) == 2 and {g.pooled_rows for g in cache.kv_groups} == {22, 1}     # ceil(64 / 3), ceil(64 / 64)
    assert cache.entries[0]["shift"].group is cache.entries[1]["shift"].group                     # equal needs share a group
    assert cache.entries[1]["mixer"]["right"]["last"].group is cache.entries[0]["shift"].group
    s = cache.open()
    cache.reserve(s, 130)
    cache.advance(s, 130)
    cache.check()
    cache.close(s)
    cache.check()


def test_needset_drops_nothing_kept():
    n = NeedSet.of(a=None, b=StateNeed((3,)))
    assert n.items == (("b", StateNeed((3,))),)


def test_plain_visibility_rule():
    """Position i sees the last `window` tokens and the blocks wholly before the window; a token that left the window
    is unseen until its block is complete AND wholly behind the window."""
    for window, pool in ((7, 3), (4, 9), (33, 5), (5, 5), (1, 1)):
        for i in range(60):
            tokens, blocks = plain.visible(i, window, pool)
            assert tokens == list(range(max(0, i - window + 1), i + 1))
            assert blocks == [b for b in range(i // pool + 1) if b * pool + pool - 1 <= i - window]
    tokens, blocks = plain.visible(10, 4, 3)        # window 7..10; blocks 0 (0-2) and 1 (3-5) are seen, token 6 is not
    assert tokens == [7, 8, 9, 10] and blocks == [0, 1]


def test_plain_recurrences_against_closed_forms():
    g = np.random.default_rng(0)
    T, H, P, N = 9, 2, 3, 4
    x, B, C = g.normal(size=(T, H, P)), g.normal(size=(T, 1, N)), g.normal(size=(T, 1, N))
    dt, A_log, D = g.uniform(0.1, 1.0, size=(T, H)), g.normal(size=H), g.normal(size=H)
    y = plain.ssm_recurrence(x, B, C, dt, A_log, D, 1)
    for h in range(H):      # y_t = sum_{s<=t} exp(-exp(A) (dt_{s+1} + .. + dt_t)) dt_s (C_t . B_s) x_s + D x_t
        for t in range(T):
            acc = D[h] * x[t, h]
            for s in range(t + 1):
                acc = acc + np.exp(-np.exp(A_log[h]) * dt[s + 1:t + 1, h].sum()) * dt[s, h] * (C[t, 0] @ B[s, 0]) * x[s, h]
            assert np.allclose(y[t, h], acc)
    K = 3
    r, k, v, w = g.normal(size=(T, 1, K)), g.normal(size=(T, 1, K)), g.normal(size=(T, 1, K)), g.uniform(0.5, 1.0, size=(T, 1, K))
    u = g.normal(size=(1, K))
    o = plain.wkv_recurrence(r, k, v, w, u)
    for t in range(T):      # o_t = sum_{s<t} (r_t * prod_{s<q<t} w_q . k_s) v_s + (r_t * u . k_t) v_t
        acc = (r[t, 0] * u[0] @ k[t, 0]) * v[t, 0]
        for s in range(t):
            acc = acc + ((r[t, 0] * w[s + 1:t, 0].prod(0)) @ k[s, 0]) * v[s, 0]
        assert np.allclose(o[t, 0], acc)
    xs = g.normal(size=(6, 2))
    cw, cb = g.normal(size=(2, 3)), g.normal(size=2)
    out = plain.causal_conv_silu(xs, cw, cb)
    z = cb + cw[:, 2] * xs[4] + cw[:, 1] * xs[3] + cw[:, 0] * xs[2]
    assert np.allclose(out[4], z / (1 + np.exp(-z)))
    assert np.allclose(out[0], plain.silu(cb + cw[:, 2] * xs[0]))
