"""The Vosulorn decoder through the engine against the plain implementation (tests/plain_vosulorn.py), in float32 and
bfloat16, cut in every way the engine allows: whole prompts, a long tail decoded token by token, pieces down to one and
two tokens, unequal batches on slots and pages that are used again, steps cut by the engine itself, greedy generation
through the package's entry point, the command line and the trace replay.  Two configurations that differ in every size
(tests/vosulorn_models.py), and one whose weights make a single far key decide the logits."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers as H
import plain_vosulorn as plain
import vosulorn_models as M

pytestmark = pytest.mark.gpu

NAMES = ["a", "b"]
DTYPES = ["float32", "bfloat16"]
TOL = {"float32": 5e-5, "bfloat16": 6e-2}
# bfloat16: in these narrow models a router's best logits are now and then closer than the bfloat16 rounding of the
# router's input, and a token that takes another expert differs by that expert's whole output, as does every later token
# that reads a state or a key it left.  So the bfloat16 runs use the same configurations with every expert chosen (the
# router's weights stay in play, its choice does not); the choice itself is tested in float32 here and, in both types,
# on the kernels alone (tests/test_vosulorn_kernels_gpu.py).  These models' matrices are drawn large so that logits are of
# order 1 at a width of 50, which makes their softmaxes peaked: a key's bfloat16 rounding moves a score by a tenth, and
# single rows by several times the usual error.  The typical row must be close and no row far off; a kernel that read or
# wrote the wrong thing in bfloat16 would move most rows by the logits' own size.
BF16_TYPICAL, BF16_WORST = 4e-2, 0.5


def every_expert(cfg):
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        if layer.get("mlp"):
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return cfg


CONFIGS = {"a": M.CFG_A, "b": M.CFG_B, "a_all": every_expert(M.CFG_A), "b_all": every_expert(M.CFG_B)}


def model_for(name, dtype):
    return name + "_all" if dtype == "bfloat16" else name


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("vosulorn")
    return {n: M.write_dir(str(tmp / n), CONFIGS[n], seed=21 + i % 2) for i, n in enumerate(CONFIGS)}


class Oracle:
    def __init__(self, d):
        self.cfg, self.W = plain.load(d)
        self.memo = {}

    def logits(self, toks):
        key = tuple(toks)
        if key not in self.memo:
            self.memo[key] = plain.forward(self.cfg, self.W, list(toks))
        return self.memo[key]


@pytest.fixture(scope="module")
def oracles(dirs):
    return {n: Oracle(d) for n, d in dirs.items()}


_engines = {}


def engine_for(dirs, name, dtype, max_tokens=1536, **kw):
    from edgelm_b200.engine.engine import Engine
    key = (dirs[name], dtype, max_tokens, tuple(sorted(kw.items())))
    if key not in _engines:
        _engines[key] = Engine.from_dir(dirs[name], dtype=dtype, max_tokens=max_tokens, **kw)
    return _engines[key]


def close(got, want, dtype, what=""):
    err = H.rel_err(got, want)
    if dtype == "bfloat16":
        rows = np.abs(np.asarray(got, np.float64) - want).max(-1) / max(1.0, np.abs(want).max())
        assert err < BF16_WORST and (len(rows) < 8 or np.median(rows) < BF16_TYPICAL), (what, err, float(np.median(rows)))
        return
    assert err < TOL[dtype], (what, err)
    if dtype == "float32":
        share, n = H.decisive_agreement(got, want, gap=0.01)
        assert share == 1.0, (what, share, n)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(dirs, oracles, name, dtype):
    """Lengths around everything that has an edge: one token, two, a chunk, a page of 64, several pages."""
    name = model_for(name, dtype)
    eng = engine_for(dirs, name, dtype)
    for i, n in enumerate((1, 2, 6, 7, 8, 33, 64, 65, 70, 71, 130, 200)):
        toks = M.tokens(CONFIGS[name], n, i)
        close(H.run_whole(eng, toks), oracles[name].logits(toks), dtype, n)
    eng.cache.check()
    eng.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_long_decoding(dirs, oracles, name, dtype):
    """A prompt in one step and 130 tokens one by one: the delta rule's states and the convolutions' tails are carried,
    the latent's rows are read by two layers, over page borders and past every chunk edge; and from the very first
    token on (a prompt of one token)."""
    name = model_for(name, dtype)
    eng = engine_for(dirs, name, dtype)
    toks = M.tokens(CONFIGS[name], 200, 20)
    close(H.run_tail_one_by_one(eng, toks, 130), oracles[name].logits(toks), dtype, "tail 130")
    toks = M.tokens(CONFIGS[name], 80, 21)
    close(H.run_tail_one_by_one(eng, toks, 79), oracles[name].logits(toks), dtype, "all but one decoded")
    eng.cache.check()
    eng.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_pieces_of_a_prompt(dirs, oracles, name, dtype):
    """One stream in pieces of many sizes, down to one and two tokens (shorter than a convolution's tail), with cuts
    inside chunks and at their edges."""
    name = model_for(name, dtype)
    from edgelm_b200.engine.engine import StepEntry
    eng = engine_for(dirs, name, dtype)
    toks = M.tokens(CONFIGS[name], 230, 30)
    want = oracles[name].logits(toks)
    for cuts in ((2, 3, 64, 1, 37, 2, 2, 1, 70, 48), (1, 1, 2, 60, 66, 100), (129, 2, 99), (7, 7, 56, 70, 90)):
        assert sum(cuts) == len(toks)
        slot = eng.open(1)[0]
        rows, at = [], 0
        for c in cuts:
            rows.append(eng.step([StepEntry(slot, toks[at:at + c], list(range(c)))]).cpu().numpy())
            at += c
        eng.close([slot])
        close(np.concatenate(rows, 0), want, dtype, cuts)
    eng.cache.check()
    eng.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_on_reused_slots(dirs, oracles, name, dtype):
    """Requests of unequal lengths in batches of three, decoded together; shorter ones leave earlier; the next batch
    takes the slots and pages just given back (their states must start from zero again).  Every request's logits
    equal those it has alone."""
    name = model_for(name, dtype)
    eng = engine_for(dirs, name, dtype, max_tokens=768)
    cfg = CONFIGS[name]
    requests = [M.tokens(cfg, n, 40 + i) for i, n in enumerate((150, 31, 1, 97, 64, 140, 2, 75, 66))]
    got = H.run_batches(eng, requests, batch_size=3, decode_tail=25)
    for r, g in zip(requests, got):
        close(g, oracles[name].logits(r), dtype, len(r))
    got = H.run_batches(eng, requests[::-1], batch_size=4, decode_tail=3)
    for r, g in zip(requests[::-1], got):
        close(g, oracles[name].logits(r), dtype, len(r))
    eng.check_device_errors()


@pytest.mark.parametrize("name", NAMES)
def test_steps_cut_by_the_engine(dirs, oracles, name):
    """An engine that runs at most 64 tokens at a time cuts a step of three prompts into consecutive smaller ones."""
    from edgelm_b200.engine.engine import StepEntry
    eng = engine_for(dirs, name, "float32", max_tokens=768, max_step_tokens=64)
    cfg = CONFIGS[name]
    requests = [M.tokens(cfg, n, 60 + i) for i, n in enumerate((150, 70, 33))]
    slots = eng.open(3)
    lg = eng.step([StepEntry(s, r, list(range(len(r)))) for s, r in zip(slots, requests)]).cpu().numpy()
    eng.close(slots)
    at = 0
    for r in requests:
        close(lg[at:at + len(r)], oracles[name].logits(r), "float32", len(r))
        at += len(r)
    eng.cache.check()
    eng.check_device_errors()


def test_a_far_key_decides(tmp_path):
    """One layer of chunked attention and one of latent attention whose queries and keys are scaled up, so that the
    softmax of most tokens rests on one far key: a key lost at a page border, a chunk that starts one token off, a sink
    left out or a latent row read from the wrong place moves the logits by their own size, in prompts and in decoding."""
    from edgelm_b200.engine.engine import Engine
    cfg = {"architecture": "Vosulorn", "vocab": 120, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "layers": [
        M.attention(8, 1, 16, 16, 0.25, {"base": 5000.0, "dims": 8}, 96, None),     # (eight heads to a key head: decoding shares the staged keys)
        M.latent(8, 16, 8, 12, 24, 0.25, 5000.0, M.moe(3, 2, 20)),
        M.latent(2, 8, 8, 20, 24, 0.3, 5000.0, None, kv_from=1)]}
    W = M.tensors_for(cfg, 77)
    for name in ("l0.mix.q", "l0.mix.k", "l1.mix.q", "l1.mix.dkv", "l2.mix.q"):
        W[name] = W[name] * 4.0
    d = M.write_dir(str(tmp_path / "far"), cfg, 77, overrides={k: W[k] for k in ("l0.mix.q", "l0.mix.k", "l1.mix.q", "l1.mix.dkv", "l2.mix.q")})
    pcfg, PW = plain.load(d)
    eng = Engine.from_dir(d, dtype="float32", max_tokens=1024)
    toks = M.tokens(cfg, 300, 5)
    want = plain.forward(pcfg, PW, toks)
    # scores sixteen times the usual size carry sixteen times the rounding error into the exponentials: the tolerance is
    # wider than elsewhere, and still a thousand times under what a lost key costs
    assert np.abs(want).max() > 1.0
    assert H.rel_err(H.run_whole(eng, toks), want) < 1e-3
    assert H.rel_err(H.run_tail_one_by_one(eng, toks, 110), want) < 1e-3
    eng.cache.check()
    eng.check_device_errors()


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_entry_point(dirs, oracles, name):
    """`edgelm_b200.generate`: the generation loop, its batches, the sampler and the captured decode graphs."""
    import edgelm_b200
    cfg = CONFIGS[name]
    prompts = [M.tokens(cfg, n, 80 + i) for i, n in enumerate((9, 1, 70, 30, 3))]
    got = edgelm_b200.generate(dirs[name], prompts, n=24, dtype="float32", ctx=128, slots=3, stop=[], ignore_eos=True)
    o = oracles[name]
    for p, g in zip(prompts, got):
        seq = list(p)
        for t in g:     # the library's choice is the plain implementation's, or as good as it within float32 rounding
            lg = plain.forward(o.cfg, o.W, seq)[-1]
            assert lg[t] >= lg.max() - 1e-3, (len(p), len(seq))
            seq.append(t)
        assert len(g) == 24


def test_info_and_trace_replay_commands(dirs, tmp_path):
    """The command line describes the model from its parts, and bin/trace_run replays a trace of it."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-m", "edgelm_b200", "info", "-m", dirs["a"]], cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert "gated_delta" in out.stdout and "masked_attention" in out.stdout and "latent_attention" in out.stdout and "moe" in out.stdout
    cfg = M.CONFIGS["a"]
    ra, rb = M.tokens(cfg, 70, 90), M.tokens(cfg, 9, 91)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": ra[:60], "want": [0, 59]}, {"id": "y", "tokens": rb[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": [ra[60]], "want": [0]}, {"id": "y", "tokens": [rb[8]], "want": [0]}], "end": ["y"]}]
    steps += [{"step": 2 + i, "entries": [{"id": "x", "tokens": [ra[61 + i]], "want": [0] if i % 2 else []}], "end": ["x"] if i == 8 else []} for i in range(9)]
    outdir = tmp_path / "out"
    run = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", dirs["a"], "--dtype", "float32", "--out", str(outdir), "--max-tokens", "256"],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", cwd=root, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr
    assert [l for l in run.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(11)]
    pcfg, W = plain.load(dirs["a"])
    wa, wb = plain.forward(pcfg, W, ra), plain.forward(pcfg, W, rb)
    s0 = np.fromfile(outdir / "0.f32", dtype="<f4").reshape(3, -1)
    assert H.rel_err(s0, np.stack([wa[0], wa[59], wb[7]])) < TOL["float32"]
    s1 = np.fromfile(outdir / "1.f32", dtype="<f4").reshape(2, -1)
    assert H.rel_err(s1, np.stack([wa[60], wb[8]])) < TOL["float32"]
    assert not (outdir / "2.f32").exists()
    s3 = np.fromfile(outdir / "3.f32", dtype="<f4").reshape(1, -1)
    assert H.rel_err(s3, wa[62:63]) < TOL["float32"]
