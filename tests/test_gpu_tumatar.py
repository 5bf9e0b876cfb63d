"""The Tumatar design through the engine against the plain implementation (tests/plain_tumatar.py): whole
prompts, prompts then token by token, prompts in portions down to two tokens, unequal batches with slots and
pages used again, sequences that end at, before and behind a page border, the first tokens, long decoding,
greedy generation through ``Engine.generate``, and a replay through ``bin/trace_run``; in float32 and in
bfloat16, at four configurations that differ in every size.  The recurrences are made to remember for
hundreds of tokens and the routers' choice scores are all negative (tests/tumatar_cases.py: long_memory)."""
import json
import os

import numpy as np
import pytest
import torch

import plain_tumatar as P
import tumatar_cases as TC
from helpers import random_tokens

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _act(dn):
    return None if dn == "float32" else torch.bfloat16


class Zoo:
    """Engines and plain logits, made once per (configuration, type)."""

    def __init__(self):
        self.made = {}

    def get(self, name, dn):
        key = (name, dn)
        if key not in self.made:
            eng, cfg, w = TC.build(TC.for_type(TC.config(name), dn), 11, dn)
            reqs = [random_tokens(n, cfg["vocab"], 500 + n) for n in (1, 2, 63, 64, 65, 130, 201)]
            want = [P.forward(cfg, w, r, act=_act(dn)) for r in reqs]
            self.made[key] = (eng, cfg, w, reqs, want)
        return self.made[key]


@pytest.fixture(scope="module")
def zoo():
    return Zoo()


CASES = [(n, d) for n in ("A", "B", "C", "D") for d in DTYPES]


@pytest.mark.parametrize("name,dn", CASES)
def test_whole_prompts_and_the_first_tokens(zoo, name, dn):
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    for r, wl in zip(reqs, want):          # lengths 1 and 2: the first tokens; 63, 64, 65: around a page border
        s = eng.alloc_slot()
        got = eng.step([(s, r)], [list(range(len(r)))]).clone()
        eng.free_slot(s)
        TC.rows_close(got, wl, dn, f"{name} whole, {len(r)} tokens")
    eng.cache.slots.check()


@pytest.mark.parametrize("name,dn", CASES)
def test_prompt_then_token_by_token(zoo, name, dn):
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    for r, wl, first in ((reqs[4], want[4], 1), (reqs[5], want[5], 60), (reqs[6], want[6], 127)):
        s = eng.alloc_slot()
        rows = [eng.step([(s, r[:first])], [list(range(first))]).clone()]
        rows += [eng.step([(s, [t])]).clone() for t in r[first:]]          # the decode graph, across page borders
        eng.free_slot(s)
        TC.rows_close(torch.cat(rows), wl, dn, f"{name} {first} tokens then one by one")


@pytest.mark.parametrize("name,dn", CASES)
def test_prompts_in_portions(zoo, name, dn):
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    for r, wl, cuts in ((reqs[6], want[6], [2, 2, 3, 57, 2, 64, 1, 33, 37]), (reqs[5], want[5], [64, 2, 62, 2]),
                        (reqs[4], want[4], [17, 48])):
        assert sum(cuts) == len(r)
        s = eng.alloc_slot()
        rows, at = [], 0
        for n in cuts:
            rows.append(eng.step([(s, r[at:at + n])], [list(range(n))]).clone())
            at += n
        eng.free_slot(s)
        TC.rows_close(torch.cat(rows), wl, dn, f"{name} in portions {cuts}")


@pytest.mark.parametrize("name,dn", CASES)
def test_unequal_batches_with_slots_and_pages_used_again(zoo, name, dn):
    from test_gpu_model import run_batches
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    # batch after batch in the same few slots: a slot's state and a page's rows are what the last user left
    got = run_batches(eng, reqs, [[6, 0, 3], [5, 1], [2, 4]], [150 if len(r) > 150 else max(1, len(r) - k)
                                                              for r, k in zip(reqs, (0, 1, 3, 0, 32, 30, 0))])
    for i, wl in enumerate(want):
        TC.rows_close(got[i], wl, dn, f"{name} batched, request {i}")
    eng.cache.slots.check()
    assert eng.cache.slots.slots.n_held == 0


@pytest.mark.parametrize("dn", DTYPES)
def test_a_state_that_is_lost_would_show(zoo, dn):
    """The check of the checks: with the recurrences made to remember, zeroing the state of a sequence between
    two steps changes the logits far beyond the tolerance (so the comparisons above do see the state)."""
    eng, cfg, w, reqs, want = zoo.get("A", dn)
    r, wl = reqs[5], want[5]
    s = eng.alloc_slot()
    eng.step([(s, r[:100])])
    for st in eng.cache.states.values():
        st[s].zero_()
    got = eng.step([(s, r[100:])], [list(range(len(r) - 100))]).clone()
    eng.free_slot(s)
    with pytest.raises(AssertionError):
        TC.rows_close(got, wl[100:], dn, "state zeroed")


@pytest.mark.parametrize("dn", DTYPES)
def test_a_far_key_among_hundreds(dn):
    """One score is made to stand out.  The query latent reads only the first half of the residual stream and
    the key/value latent only the second half, through the same matrices, and the last token's first half is
    the first token's second half: the last query equals the first key, its score there is |k|^2 against
    scores of random sign everywhere else, so the last row is the first position's value.  The first position
    lies hundreds of tokens and several pages back; without it the row is another one altogether."""
    cfg = TC.config("C")
    cfg["loop"] = None
    cfg["layers"] = [cfg["layers"][1]]
    cfg["layers"][0]["mixer"].update(q_rank=64, kv_rank=64, scale=1.0)
    half = cfg["width"] // 2

    def tweak(w):
        p = "l0.mix."
        w[p + "dq"][:, half:] = 0
        w[p + "dkv"][:, :half] = 0
        w[p + "dkv"][:, half:] = w[p + "dq"][:, :half]
        w[p + "dkv.norm"].copy_(w[p + "dq.norm"])
        w[p + "uq"].copy_(w[p + "uk"])
        w["l0.norm1"].fill_(1.0)
        w["embed"][5, :half] = w["embed"][7, half:]

    eng, cfg, w = TC.build(cfg, 3, dn, tweak=tweak)
    toks = [7] + [t if t not in (5, 7) else 6 for t in random_tokens(298, cfg["vocab"], 9)] + [5]
    want = P.forward(cfg, w, toks, act=_act(dn))
    without = P.forward(cfg, w, toks[1:], act=_act(dn))
    assert (want[-1] - without[-1]).abs().max() > 0.2 * want[-1].abs().max()      # the far key matters
    for first in (290, len(toks)):              # the last token decoded alone, and as the end of the prompt
        s = eng.alloc_slot()
        rows = [eng.step([(s, toks[:first])], [list(range(first))]).clone()]
        rows += [eng.step([(s, [t])]).clone() for t in toks[first:]]
        eng.free_slot(s)
        got = torch.cat(rows)
        if dn == "float32":
            TC.rows_close(got, want, dn, "far key")
        TC.rows_close(got[-1:], want[-1:], dn, "far key, last row")


@pytest.mark.parametrize("name,dn", [("B", "float32"), ("C", "bfloat16")])
def test_long_decoding(zoo, name, dn):
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    r, wl = reqs[6], want[6]
    s = eng.alloc_slot()
    rows = [eng.step([(s, r[:3])], [[0, 1, 2]]).clone()] + [eng.step([(s, [t])]).clone() for t in r[3:]]
    eng.free_slot(s)
    TC.rows_close(torch.cat(rows), wl, dn, f"{name} decoded for {len(r) - 3} tokens")


@pytest.mark.parametrize("dn", DTYPES)
def test_float32_logits_do_not_depend_on_the_schedule(zoo, dn):
    if dn != "float32":
        pytest.skip("the bfloat16 kernels of prompts and of decode steps differ")
    eng, cfg, w, reqs, want = zoo.get("A", dn)
    r = reqs[5]
    s = eng.alloc_slot()
    whole = eng.step([(s, r)], [list(range(len(r)))]).clone()
    eng.free_slot(s)
    s, other = eng.alloc_slot(), eng.alloc_slot()
    a = eng.step([(other, reqs[3]), (s, r[:70])], [[], list(range(70))]).clone()
    b = torch.cat([eng.step([(other, [1]), (s, [t])], [[], [0]]).clone() for t in r[70:]])
    eng.free_slot(s); eng.free_slot(other)
    assert (torch.cat([a, b]) - whole).abs().max().item() <= 2e-5 * whole.abs().max().item()


@pytest.mark.parametrize("name,dn", [("A", "float32"), ("B", "bfloat16")])
def test_greedy_generation_through_the_entry_point(name, dn):
    from ziglm_b200 import GenerationOptions, SamplerParams
    eng, cfg, w = TC.build(TC.for_type(TC.config(name), dn), 5, dn, std=0.3)       # large weights: well separated logits
    prompts = [random_tokens(n, cfg["vocab"], 70 + n) for n in (3, 40, 9)]
    results, stats = eng.generate(prompts, GenerationOptions(max_tokens=8, ignore_eos=True,
                                                             sampler=SamplerParams(greedy=True)))
    for p, r in zip(prompts, results):
        seq = list(p)
        assert len(r.tokens) == 8
        for tok in r.tokens:
            # the generated token is the plain implementation's best one; in bfloat16 it may be one that the
            # plain logits put within a twentieth of their spread of the best (then the sequence goes on with it)
            row = P.forward(cfg, w, seq, act=_act(dn))[-1]
            slack = 0.0 if dn == "float32" else 0.05 * row.std().item()
            assert row.max().item() - row[tok].item() <= slack, f"token {tok} after {len(seq)} tokens"
            seq.append(tok)
    assert stats.completion_tokens == 24


def test_replay_from_a_folder(tmp_path):
    """A folder written by the library, loaded by name of the architecture and replayed by ``bin/trace_run``."""
    from safetensors.torch import load_file
    from test_gpu_replay import Replay
    from ziglm_b200 import config_from_dict, write_random_model
    cfg = TC.config("C")
    folder = str(tmp_path / "model")
    write_random_model(folder, config_from_dict(cfg), 8, dtype=torch.bfloat16, std=0.12, norm_jitter=0.1, device="cuda")
    w = load_file(os.path.join(folder, "model.safetensors"))
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "Tumatar"
    reqs = [random_tokens(n, cfg["vocab"], 30 + n) for n in (70, 9)]
    for dn in DTYPES:
        want = [P.forward(cfg, w, r, act=_act(dn)) for r in reqs]
        rp = Replay(folder, dn, str(tmp_path / ("logits_" + dn)), max_tokens=256)
        try:
            first = rp.step([{"id": "a", "tokens": reqs[0][:40], "want": list(range(40))},
                             {"id": "b", "tokens": reqs[1][:5], "want": [0, 4]}])
            TC.rows_close(first, torch.cat([want[0][:40], want[1][[0, 4]]]), dn, "replay, first step")
            for i in range(4):
                got = rp.step([{"id": "a", "tokens": [reqs[0][40 + i]], "want": [0]},
                               {"id": "b", "tokens": [reqs[1][5 + i]], "want": [0]}], end=["b"] if i == 3 else [])
                TC.rows_close(got, torch.stack([want[0][40 + i], want[1][5 + i]]), dn, f"replay, step {i + 1}")
            for i in range(44, 70):
                got = rp.step([{"id": "a", "tokens": [reqs[0][i]], "want": [0]}], end=["a"] if i == 69 else [])
                TC.rows_close(got, want[0][i:i + 1], dn, f"replay, token {i}")
        finally:
            rp.close()


@pytest.mark.parametrize("kind", ["rglru", "latent_attention"])
def test_a_model_of_one_kind_of_mixer(kind):
    """Only recurrences (no cache group at all: nothing but state is kept) and only attention (no state): the
    same layer three times in a row through a loop of one layer."""
    cfg = TC.config("B")
    layer = [l for l in cfg["layers"] if l["type"] == kind][0]
    cfg["layers"] = [layer]
    cfg["loop"] = {"start": 0, "stop": 1, "times": 3}
    eng, cfg, w = TC.build(cfg, 21, "float32")
    assert (len(eng.cache.groups) == 0) == (kind == "rglru") and (len(eng.cache.states) == 0) == (kind != "rglru")
    r = random_tokens(90, cfg["vocab"], 77)
    want = P.forward(cfg, w, r)
    s = eng.alloc_slot()
    rows = [eng.step([(s, r[:70])], [list(range(70))]).clone()] + [eng.step([(s, [t])]).clone() for t in r[70:]]
    eng.free_slot(s)
    TC.rows_close(torch.cat(rows), want, "float32", f"only {kind}")
