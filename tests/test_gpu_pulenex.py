"""Whole Pulenex models with random weights through the engine, against the plain implementation: whole prompts, a prompt
and then single tokens, portions of several sizes, batches of unequal requests, slots and cache blocks that are used again,
long decoding, and greedy generation through the library's entry point and scheduler."""
import numpy as np
import pytest
import torch

import helpers
import pulenex_models
from plain import pulenex_plain as plain

pytestmark = pytest.mark.gpu
NAMES = ["odd", "even", "bare"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: pulenex_models.make_model_dir(str(tmp_path_factory.mktemp("pulenex_" + n)), n) for n in NAMES}


@pytest.fixture(scope="module")
def oracles(folders):
    return {n: plain.read_model(folders[n]) for n in folders}


@pytest.fixture(scope="module")
def engines(folders):
    from hymt2sharp_b200.engine.engine import Engine
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = Engine(folders[name], dtype=dtype, max_tokens=4096)
        return made[(name, dtype)]
    return get


def _vocab(name):
    return pulenex_models.CONFIGS[name]["config"]["vocab"]


def _reference(oracles, name, tokens):
    cfg, w = oracles[name]
    return plain.forward(cfg, w, tokens).numpy()


FACTOR = {"float32": 4.0, "bfloat16": 2.5}
BF16_MEDIAN, BF16_FAR, BF16_FAR_SHARE = 0.08, 0.35, 0.1


def _assert_rows(got, ref, dtype, what):
    """32-bit: every row within the shared tolerance; this is the sharp comparison, and a wrong or missing key, slot, state or
    block shows in it.  bfloat16: the mixers with a state divide every head's output by its root mean square, which enlarges
    the rounding of the bfloat16 products wherever that output is a sum of a few terms that cancel, and the state carries a
    token's error to every token behind it; so the rows are held to a distribution: a row's error is the root mean square of
    the difference of the logits (mean taken off) over that of the plain logits; its median over the rows stays under
    BF16_MEDIAN, and at most BF16_FAR_SHARE of the rows (or one) lie beyond BF16_FAR."""
    if dtype == "float32":
        return helpers.assert_close(got, ref, dtype, what, factor=FACTOR[dtype])
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape and np.isfinite(got).all(), f"{what}: shape {got.shape} vs {ref.shape}, or non-finite values"
    g, r = got - got.mean(1, keepdims=True), ref - ref.mean(1, keepdims=True)
    e = np.sqrt(((g - r) ** 2).mean(1)) / np.sqrt((r ** 2).mean())
    far = np.flatnonzero(e > BF16_FAR)
    assert len(far) <= max(1, int(BF16_FAR_SHARE * len(e))), f"{what}: rows {far.tolist()} of {len(e)} are off by more than {BF16_FAR}"
    if len(e) >= 8:
        assert np.median(e) <= BF16_MEDIAN, f"{what}: the median error of a row is {np.median(e):.3f}"


def _run(engine, requests, cuts):
    """cuts[step][request] tokens per step (0: rests); every token's logits are asked for.  Returns per request [n, vocab]."""
    from hymt2sharp_b200.engine.engine import StepEntry
    slots = engine.alloc_slots(len(requests))
    at = [0] * len(requests)
    rows = [[] for _ in requests]
    for step in cuts:
        live = [(i, n) for i, n in enumerate(step) if n]
        out = engine.step([StepEntry(slots[i], requests[i][at[i]:at[i] + n], list(range(n))) for i, n in live]).cpu().numpy()
        o = 0
        for i, n in live:
            rows[i].append(out[o:o + n]); o += n; at[i] += n
    engine.check()
    engine.free_slots(slots)
    engine.cache.book.audit()
    assert all(a == len(r) for a, r in zip(at, requests))
    return [np.concatenate(r) for r in rows]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_against_plain(name, dtype, engines, oracles):
    """Among them a prompt that crosses several chunks, windows and cache blocks, and prompts of one and two tokens."""
    eng = engines(name, dtype)
    reqs = [helpers.random_tokens(_vocab(name), n, 40 + n) for n in (260, 1, 2, 67)]
    got = _run(eng, reqs, [[len(r) for r in reqs]])
    for r, g in zip(reqs, got):
        _assert_rows(g, _reference(oracles, name, r), dtype, f"{name} whole prompt of {len(r)}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_cuts_batches_and_reused_slots_agree(name, dtype, engines, oracles):
    """The logits of a position depend neither on how its tokens were cut into steps, nor on what else was in the batch,
    nor on which slot, state row and blocks the sequence got."""
    eng = engines(name, dtype)
    V = _vocab(name)
    reqs = [helpers.random_tokens(V, n, 7 + n) for n in (140, 33, 5)]
    refs = [_reference(oracles, name, r) for r in reqs]
    schedules = {
        "each alone": None,
        "one batch": [[140, 33, 5]],
        "token by token after a short start": [[2, 1, 1]] + [[1, 1, 1]] * 4 + [[1, 1, 0]] * 28 + [[1, 0, 0]] * 106,
        "portions of 2, 3, 64 and the rest": [[2, 2, 2], [3, 3, 3], [64, 28, 0], [71, 0, 0]],
        "a prompt, then decoding together": [[100, 20, 2]] + [[1, 1, 1]] * 3 + [[1, 1, 0]] * 10 + [[1, 0, 0]] * 27,
    }
    for what, cuts in schedules.items():
        if cuts is None:
            got = [_run(eng, [r], [[len(r)]])[0] for r in reqs]
        else:
            got = _run(eng, reqs, cuts)
        for r, g, ref in zip(reqs, got, refs):
            _assert_rows(g, ref, dtype, f"{name} {what} ({len(r)} tokens)")
    # slots, state rows and blocks that another, longer request held before
    _run(eng, [helpers.random_tokens(V, 300, 1)], [[300]])
    again = _run(eng, [reqs[1]], [[20], [13]])[0]
    _assert_rows(again, refs[1], dtype, f"{name} a slot used again")


@pytest.mark.parametrize("name", NAMES)
def test_cuts_do_not_show_in_float32_beyond_rounding(name, engines):
    eng = engines(name, "float32")
    toks = helpers.random_tokens(_vocab(name), 300, 77)
    whole = _run(eng, [toks], [[300]])[0]
    cut = _run(eng, [toks, toks[:40]], [[258, 40]] + [[1, 0]] * 42)[0]
    assert np.abs(whole - cut).max() <= 4e-5 * np.abs(whole).max()


@pytest.mark.parametrize("name", NAMES)
def test_long_decoding_in_float32(name, engines, oracles):
    """300 single-token steps after a prompt of 30: across block borders, past every window and through many chunks, in a cache
    and a state area whose rows were poisoned."""
    eng = engines(name, "float32")
    for s in eng.cache.storage:
        s.fill_(float("nan"))
    eng.cache.state.fill_(255)
    toks = helpers.random_tokens(_vocab(name), 330, 5)
    got = _run(eng, [toks], [[30]] + [[1]] * 300)[0]
    helpers.assert_close(got, _reference(oracles, name, toks), "float32", f"{name} long decoding", factor=4.0)


def test_a_model_with_state_is_reset_but_not_cut(engines):
    from hymt2sharp_b200.engine.engine import EngineError, StepEntry
    eng = engines("odd", "float32")
    slot = eng.alloc_slots(1)[0]
    toks = helpers.random_tokens(_vocab("odd"), 20, 3)
    first = eng.step([StepEntry(slot, toks, [19])]).cpu().numpy()
    with pytest.raises(EngineError, match="reset"):
        eng.truncate(slot, 10)
    eng.reset(slot)
    again = eng.step([StepEntry(slot, toks, [19])]).cpu().numpy()
    eng.free_slots([slot])
    assert np.array_equal(first, again)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_entry_point(name, dtype, folders, oracles):
    """hymt2sharp_b200.load(...).generate(...): unequal prompts in one batch, the decode steps replayed from a CUDA graph.  In
    32-bit the tokens are the plain implementation's; in bfloat16 every generated token must be one that the plain logits
    rank (nearly) first."""
    import hymt2sharp_b200
    cfg, w = oracles[name]
    engine = hymt2sharp_b200.load(folders[name], dtype=dtype, max_tokens=2048)
    assert engine.model.graph_safe
    prompts = [helpers.random_tokens(_vocab(name), n, 90 + n) for n in (21, 3, 70)]
    out = engine.generate(prompts, max_new_tokens=12)
    assert [len(r.tokens) for r in out.results] == [12, 12, 12] and out.stats.decode_steps == 11
    low = 0
    for p, r in zip(prompts, out.results):
        if dtype == "float32":
            assert r.tokens == plain.greedy(cfg, w, p, 12)
        else:
            toks = list(p)
            for t in r.tokens:
                logits = plain.forward(cfg, w, toks)[-1]
                low += float(logits[t]) < float(logits.max()) - 0.15 * float(logits.max() - logits.min())
                toks.append(t)
    assert low <= 2, f"{low} of 36 generated tokens rank low in the plain logits"
    again = engine.generate(prompts, max_new_tokens=12)
    assert [r.tokens for r in again.results] == [r.tokens for r in out.results]
    engine.cache.book.audit()


def test_trace_replay_of_a_batch(folders, oracles):
    """bin/trace_run on a schedule with unequal requests that start together and are decoded together."""
    for name, dtype in (("odd", "float32"), ("even", "bfloat16")):
        V = _vocab(name)
        reqs = {"a": helpers.random_tokens(V, 50, 1), "b": helpers.random_tokens(V, 9, 2), "c": helpers.random_tokens(V, 70, 3)}
        tb = helpers.TraceBuilder()
        tb.batch([("a", reqs["a"], 6), ("b", reqs["b"], 3), ("c", reqs["c"], 0)])
        tb.whole("d", reqs["b"], key="b")
        got = tb.collect(helpers.run_trace(folders[name], dtype, tb.steps, 256, V))
        for key, toks in reqs.items():
            ref = _reference(oracles, name, toks)
            places = sorted(got[key])
            for k in range(max(len(got[key][p]) for p in places)):      # (a request that ran twice has two rows a place)
                at = [p for p in places if len(got[key][p]) > k]
                _assert_rows(np.stack([got[key][p][k] for p in at]), ref[at], dtype, f"trace {key}")


def test_command_line_runs_the_design(folders, oracles, capsys, tmp_path):
    """python -m hymt2sharp_b200 on a Pulenex folder, and --random from a configuration file of the design."""
    import json
    from hymt2sharp_b200 import cli
    cfg, w = oracles["odd"]
    assert cli.main(["--model", folders["odd"], "--dtype", "float32", "--prompt", "5 17 3 60", "--max-tokens", "5"]) == 0
    out = capsys.readouterr().out
    assert "arch=Pulenex layers=5 hidden=46 mixers=parallelx2,latent_attentionx2,retentionx1 vocab=103" in out
    want = plain.greedy(cfg, w, [5, 17, 3, 60], 6)
    assert "Assistant: " + ",".join(map(str, want)) in out
    (tmp_path / "c.json").write_text(json.dumps(pulenex_models.CONFIGS["even"]["config"]))
    assert cli.main(["--model", str(tmp_path / "m"), "--random", str(tmp_path / "c.json"), "--weights-seed", "3", "--sigma", "0.05",
                     "--prompt", "1 2 3", "--max-tokens", "3"]) == 0
    assert "arch=Pulenex layers=6 hidden=128" in capsys.readouterr().out
