"""Host-side parts of the Vosulorn decoder: the configuration reader and its plan, the tensor names and shapes, what the
layers keep in the cache (a latent without value rows, read by a later layer), the stretched frequencies, and the plain
implementation's own mechanisms against brute force."""
import copy

import numpy as np
import pytest
import torch

import plain_vosulorn as plain
import vosulorn_models as M
from edgelm_b200.cache import CompositeEntry, SequenceCache
from edgelm_b200.config import ConfigError, config_class_for
from edgelm_b200.engine.model import DecoderModel
from edgelm_b200.parts import KVNeed, StateNeed
from edgelm_b200.parts.rope import rotary_frequencies


@pytest.mark.parametrize("name", ["a", "b"])
def test_plan_names_every_tensor_with_its_shape(name):
    cfg = M.CONFIGS[name]
    conf = config_class_for(cfg).from_dict(cfg)
    assert type(conf).__name__ == "VosulornConfig"
    W = M.tensors_for(cfg, 0)
    want = DecoderModel(conf.plan(), torch.float32).expected_weights()
    assert {k: tuple(v) for k, v in want.items()} == {k: tuple(v.shape) for k, v in W.items()}
    again = config_class_for(conf.to_dict()).from_dict(conf.to_dict())
    assert again.plan() == conf.plan()


def test_the_plan_reads_every_constant():
    plan = config_class_for(M.CFG_A).from_dict(M.CFG_A).plan()
    assert plan.embedding["scale"] == 4.0 and plan.hidden_size == 64 and plan.vocab_size == 211
    assert [e.reads_cache_of for e in plan.schedule] == [None, None, None, None, 1, None]
    att, att2 = plan.layers[2].mixer, plan.layers[5].mixer
    assert att.kind == "masked_attention" and att["mask"] == {"kind": "chunk", "size": 7} and att["rot_pairs"] == "interleaved"
    assert att["rot_dims"] == 8 and att["rot_scaling"]["original"] == 64 and att["scale"] == 0.3 and att["v_head_dim"] == 8
    assert att2["mask"] is None and att2["rot_scaling"] is None and att2["num_kv_heads"] == 1
    assert plan.layers[2].ffn is None and plan.layers[0].ffn["experts"] == 4 and plan.layers[4].ffn["top"] == 5
    lat = plan.layers[4].mixer
    assert lat["reads_cache"] and lat["kv_rank"] == 32 and lat["rot_dim"] == 8 and plan.layers[1].mixer["reads_cache"] is False
    assert plan.layers[3].mixer["conv"] == 2 and plan.layers[3].mixer["kv_heads"] == 3


def test_refusals():
    for change, text in ((lambda c: c["layers"][0].update(type="conv"), "not part of this architecture"),
                         (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind 'dense'"),
                         (lambda c: c["layers"][0]["mixer"].pop("conv"), "'conv' is missing"),
                         (lambda c: c.pop("norm"), "'norm'"),
                         (lambda c: c["layers"][2]["mixer"].update(kv_heads=4), "multiple"),
                         (lambda c: c["layers"][4]["mixer"].update(kv_from=0), "kv_from 0"),
                         (lambda c: c["layers"][4]["mixer"].update(kv_from=5), "kv_from 5"),
                         (lambda c: c["layers"][4]["mixer"].update(kv_rank=16), "differ"),
                         (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4), "rot_dim"),
                         (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "9 of 4")):
        cfg = copy.deepcopy(M.CFG_A)
        change(cfg)
        with pytest.raises(ConfigError, match=text):
            DecoderModel(config_class_for(cfg).from_dict(cfg).plan(), torch.float32)


def test_what_the_layers_keep():
    model = DecoderModel(config_class_for(M.CFG_A).from_dict(M.CFG_A).plan(), torch.bfloat16)
    needs = model.cache_needs()
    assert dict(needs[0].items) == {"conv": StateNeed((3, 2 * 2 * 16 + 4 * 24)), "delta": StateNeed((4, 24, 16))}
    assert needs[1] == KVNeed(1, 32 + 8, None, v_head_dim=32, values_in_keys=True)
    assert needs[2] == KVNeed(2, 16, None, v_head_dim=8)
    assert needs[4] is None                                   # reads what layer 1 keeps
    one_tap = DecoderModel(config_class_for(M.CFG_B).from_dict(M.CFG_B).plan(), torch.float32).cache_needs()[1]
    assert dict(one_tap.items) == {"delta": StateNeed((2, 40, 70))}      # a convolution of one tap keeps no input
    cache = SequenceCache(needs, max_tokens=256, max_positions=1 << 20)
    assert isinstance(cache.entries[0], CompositeEntry) and cache.entries[4] is None
    latent_group = cache.entries[1].group
    assert latent_group.need.values_in_keys and latent_group.bytes_per_token(2) == 40 * 2
    s = cache.open()
    cache.reserve(s, 130)
    cache.advance(s, 130)
    cache.check()
    assert all(g.n_held[s] == 3 for g in cache.kv_groups)
    cache.close(s)
    cache.check()


def test_stretched_frequencies():
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    f = rotary_frequencies(16, 50.0, sc).numpy()
    plain_f = 50.0 ** (-2.0 * np.arange(8) / 16)
    wl = 2 * np.pi / plain_f
    assert (wl < 16).any() and (wl > 64).any() and ((wl >= 16) & (wl <= 64)).any()         # all three bands occur
    for fi, pi_, l in zip(f, plain_f, wl):
        if l < 16:
            assert fi == pi_
        elif l > 64:
            assert np.isclose(fi, pi_ / 4.0, rtol=1e-15)
        else:
            s = (64 / l - 1.0) / 3.0
            assert np.isclose(fi, (1 - s) * pi_ / 4 + s * pi_, rtol=1e-14) and pi_ / 4 <= fi <= pi_
    assert np.allclose(f, plain.frequencies(16, 50.0, sc), rtol=1e-14)
    assert np.allclose(rotary_frequencies(6, 77.0).numpy(), plain.frequencies(6, 77.0), rtol=1e-15)
    assert np.allclose(rotary_frequencies(6, 77.0, 2.0).numpy(), plain.frequencies(6, 77.0) / 2.0, rtol=1e-15)


def test_plain_mechanisms_against_brute_force():
    g = np.random.default_rng(1)
    # the delta rule after one token: S = k u^T with u = beta v, o = (q . k) beta v
    q, k, v = g.normal(size=(1, 1, 5)), g.normal(size=(1, 1, 5)), g.normal(size=(1, 1, 3))
    o = plain.delta_recurrence(q, k, v, np.array([[0.7]]), np.array([[0.9]]))
    assert np.allclose(o[0, 0], (q[0, 0] @ k[0, 0]) * 0.7 * v[0, 0])
    # with beta = 1 and a unit key, the state returns exactly v for that key (the write replaces what was there)
    T = 6
    k = plain.unit_vectors(g.normal(size=(T, 1, 4))) * (1 + 1e-6 / 2)
    v = g.normal(size=(T, 1, 3))
    o = plain.delta_recurrence(k, k, v, np.ones((T, 1)), np.full((T, 1), 0.8))
    assert np.allclose(o, v, atol=1e-5)
    # chunked attention with a sink: row i, by hand
    q, k, v = g.normal(size=(9, 2, 4)), g.normal(size=(9, 1, 4)), g.normal(size=(9, 1, 3))
    sink = np.array([0.3, -0.2])
    out = plain.masked_softmax_attention(q, k, v, 0.5, chunk=4, sink=sink)
    i, h = 6, 1
    s = np.array([q[i, h] @ k[j, 0] * 0.5 for j in (4, 5, 6)])
    w = np.exp(s) / (np.exp(s).sum() + np.exp(sink[h]))
    assert np.allclose(out[i, h], w @ v[4:7, 0])
    assert np.allclose(plain.masked_softmax_attention(q, k, v, 0.5, chunk=4, sink=sink)[4], plain.masked_softmax_attention(q[4:5], k[4:5], v[4:5], 0.5, sink=sink)[0])
    # neighbouring and half-split pairs rotate the same numbers, differently placed
    x = g.normal(size=(3, 1, 8))
    f = plain.frequencies(8, 100.0)
    a, b = plain.rotate(x, [0, 5, 9], f, True), plain.rotate(x[..., [0, 2, 4, 6, 1, 3, 5, 7]], [0, 5, 9], f, False)
    assert np.allclose(a[..., [0, 2, 4, 6, 1, 3, 5, 7]], b) and np.allclose(a[0], x[0])
    # the router: the largest logits first, weights over the chosen only
    W = {"router": np.eye(4), "router.b": np.zeros(4)}
    ch, w = plain.router(W, "", {"top": 2}, np.array([[0.1, 2.0, -1.0, 1.0]]))
    assert ch.tolist() == [[1, 3]] and np.allclose(w, [[np.e / (1 + np.e), 1 / (1 + np.e)]])
