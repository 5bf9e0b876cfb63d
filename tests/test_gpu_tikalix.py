"""The Tikalix design through the engine against the plain implementation (tests/plain_tikalix.py): whole prompts,
prompts then token by token, prompts in portions down to two tokens, unequal batches with slots and pages used
again, sequences that end at, before and behind a page border, the first tokens, long decoding, a far key made to
stand out, a soft cap and a gate that show, greedy generation through ``Engine.generate``, and a replay through
``bin/trace_run``; in float32 and in bfloat16, at three configurations that differ in every size."""
import json
import os

import pytest
import torch

import tikalix_cases as TC
from helpers import random_tokens

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


class Zoo:
    """Engines and plain logits, made once per (configuration, type)."""

    def __init__(self):
        self.made = {}

    def get(self, name, dn):
        key = (name, dn)
        if key not in self.made:
            eng, cfg, w = TC.build(TC.for_type(TC.config(name), dn), 11, dn)
            reqs = [random_tokens(n, cfg["vocab"], 500 + n) for n in (1, 2, 63, 64, 65, 130, 201)]
            plain = TC.plain(cfg, w, dn)
            want = [plain.forward(r) for r in reqs]
            self.made[key] = (eng, cfg, w, reqs, want)
        return self.made[key]


@pytest.fixture(scope="module")
def zoo():
    return Zoo()


CASES = [(n, d) for n in ("A", "B", "C") for d in DTYPES]


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
    # batch after batch in the same few slots: a page's rows are what the last user left
    got = run_batches(eng, reqs, [[6, 0, 3], [5, 1], [2, 4]], [150 if len(r) > 150 else max(1, len(r) - k)
                                                              for r, k in zip(reqs, (0, 1, 3, 0, 32, 30, 0))])
    for i, wl in enumerate(want):
        TC.rows_close(got[i], wl, dn, f"{name} batched, request {i}")
    eng.cache.slots.check()
    assert eng.cache.slots.slots.n_held == 0


def _far_key_model(dn, softcap):
    """One layer whose query and key are made from different halves of the residual stream through the same matrix,
    and an embedding in which the last token's first half is the first token's second half: after the unit norm the
    last query equals the first key (the rotation is kept off the dimensions that carry them), so its score at the
    first position is dim * scale against scores of random sign elsewhere."""
    cfg = TC.config("B")
    cfg["layers"] = [cfg["layers"][1]]
    cfg["layers"][0]["mlp"] = None
    m = cfg["layers"][0]["mixer"]
    m.update(heads=2, kv_heads=1, dim=64, vdim=64, scale=0.25, softcap=softcap)
    m["rot"] = {"dims": 2, "base": 10000.0}
    half = cfg["width"] // 2

    def tweak(w):
        p = "l0.mix."
        w[p + "q"][:, half:] = 0
        w[p + "k"][:, :half] = 0
        w[p + "k"][:, half:] = w[p + "q"][:64, :half]
        w[p + "q"][64:, :half] = w[p + "q"][:64, :half]
        for n in ("q.b", "k.b"):
            w[p + n].zero_()
        # the two rotated dimensions carry nothing
        for n in ("q", "k"):
            rows = w[p + n].view(-1, 64, w[p + n].shape[1])
            rows[:, 0] = 0
            rows[:, 1] = 0
        w["embed"][5, :half] = w["embed"][7, half:]

    return cfg, tweak


@pytest.mark.parametrize("dn", DTYPES)
@pytest.mark.parametrize("softcap", [None, 6.0])
def test_a_far_key_among_hundreds(dn, softcap):
    """The first position lies hundreds of tokens and several pages back.  Without a cap the last row is nearly the
    first position's value; with a cap of 6 the standing-out score of 16 becomes 6 tanh(16/6) = 5.9 and the other
    keys keep a share, so a cap that is left out (or applied before the factor on the scores) shows as well."""
    cfg, tweak = _far_key_model(dn, softcap)
    eng, cfg, w = TC.build(cfg, 3, dn, tweak=tweak)
    toks = [7] + [t if t not in (5, 7) else 6 for t in random_tokens(298, cfg["vocab"], 9)] + [5]
    plain = TC.plain(cfg, w, dn)
    want = plain.forward(toks)
    without = plain.forward(toks[1:])
    assert (want[-1] - without[-1]).abs().max() > (0.1 if softcap else 0.2) * want[-1].abs().max()      # the far key matters
    other = {**cfg, "layers": [{**cfg["layers"][0], "mixer": {**cfg["layers"][0]["mixer"],
                                                                "softcap": None if softcap else 6.0}}]}
    uncapped = TC.plain(other, w, dn).forward(toks)
    assert (want[-1] - uncapped[-1]).abs().max() > 0.05 * want[-1].abs().max()    # and so does the cap
    for first in (290, len(toks)):              # the last token decoded alone, and as the end of the prompt
        s = eng.alloc_slot()
        rows = [eng.step([(s, toks[:first])], [list(range(first))]).clone()]
        rows += [eng.step([(s, [t])]).clone() for t in toks[first:]]
        eng.free_slot(s)
        got = torch.cat(rows)
        if dn == "float32":
            TC.rows_close(got, want, dn, "far key")
        TC.rows_close(got[-1:], want[-1:], dn, "far key, last row")


@pytest.mark.parametrize("name,dn", [("A", "float32"), ("B", "bfloat16"), ("C", "bfloat16")])
def test_long_decoding(zoo, name, dn):
    eng, cfg, w, reqs, want = zoo.get(name, dn)
    r, wl = reqs[6], want[6]
    s = eng.alloc_slot()
    rows = [eng.step([(s, r[:3])], [[0, 1, 2]]).clone()] + [eng.step([(s, [t])]).clone() for t in r[3:]]
    eng.free_slot(s)
    TC.rows_close(torch.cat(rows), wl, dn, f"{name} decoded for {len(r) - 3} tokens")


@pytest.mark.parametrize("name", ["A", "C"])
def test_float32_logits_do_not_depend_on_the_schedule(zoo, name):
    eng, cfg, w, reqs, want = zoo.get(name, "float32")
    r = reqs[5]
    s = eng.alloc_slot()
    whole = eng.step([(s, r)], [list(range(len(r)))]).clone()
    eng.free_slot(s)
    s, other = eng.alloc_slot(), eng.alloc_slot()
    a = eng.step([(other, reqs[3]), (s, r[:70])], [[], list(range(70))]).clone()
    b = torch.cat([eng.step([(other, [1]), (s, [t])], [[], [0]]).clone() for t in r[70:]])
    eng.free_slot(s); eng.free_slot(other)
    assert (torch.cat([a, b]) - whole).abs().max().item() <= 2e-5 * whole.abs().max().item()


@pytest.mark.parametrize("dn", DTYPES)
def test_every_option_left_out(dn):
    """No cap, no stretching, no shared expert, no feed-forward in the last layer, multiplier and embedding scale of
    one, one key/value head per query head, the whole head rotated."""
    cfg = {"architecture": "Tikalix", "vocab": 120, "width": 64, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
           "residual_mult": 1.0,
           "layers": [{"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.2,
                                                      "softcap": None, "rot": {"dims": 32, "base": 100.0, "scaling": None}},
                       "mlp": {"kind": "moe", "expert": {"ff": 40, "limit": 2.0}, "router": {"experts": 5, "top": 2}}},
                      {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 16, "scale": 0.3,
                                                      "rot": {"dims": 16, "base": 100.0}}, "mlp": None}]}
    eng, cfg, w = TC.build(cfg, 17, dn)
    r = random_tokens(100, cfg["vocab"], 5)
    want = TC.plain(cfg, w, dn).forward(r)
    s = eng.alloc_slot()
    rows = [eng.step([(s, r[:80])], [list(range(80))]).clone()] + [eng.step([(s, [t])]).clone() for t in r[80:]]
    eng.free_slot(s)
    TC.rows_close(torch.cat(rows), want, dn, "options left out")


@pytest.mark.parametrize("name,dn", [("A", "float32"), ("B", "bfloat16")])
def test_greedy_generation_through_the_entry_point(name, dn):
    from ziglm_b200 import GenerationOptions, SamplerParams
    eng, cfg, w = TC.build(TC.for_type(TC.config(name), dn), 5, dn, std=0.3)       # large weights: well separated logits
    prompts = [random_tokens(n, cfg["vocab"], 70 + n) for n in (3, 40, 9)]
    results, stats = eng.generate(prompts, GenerationOptions(max_tokens=8, ignore_eos=True,
                                                             sampler=SamplerParams(greedy=True)))
    plain = TC.plain(cfg, w, dn)
    for p, r in zip(prompts, results):
        seq = list(p)
        assert len(r.tokens) == 8
        for tok in r.tokens:
            # the generated token is the plain implementation's best one; in bfloat16 it may be one that the
            # plain logits put within a twentieth of their spread of the best (then the sequence goes on with it)
            row = plain.forward(seq)[-1]
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
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "Tikalix"
    reqs = [random_tokens(n, cfg["vocab"], 30 + n) for n in (70, 9)]
    for dn in DTYPES:
        plain = TC.plain(cfg, w, dn)
        want = [plain.forward(r) for r in reqs]
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


def test_replay_of_many_requests_whose_last_pages_are_nearly_empty(tmp_path):
    """``--max-tokens`` counts tokens, the cache hands out pages of 64: six requests of 66 to 71 tokens in one batch
    hold 411 tokens but twelve pages, and decode on together until the shorter ones have ended."""
    from safetensors.torch import load_file
    from test_gpu_replay import Replay
    from ziglm_b200 import config_from_dict, write_random_model
    cfg = TC.config("A")
    folder = str(tmp_path / "model")
    write_random_model(folder, config_from_dict(cfg), 9, dtype=torch.bfloat16, std=0.12, norm_jitter=0.1, device="cuda")
    w = load_file(os.path.join(folder, "model.safetensors"))
    reqs = [random_tokens(66 + i, cfg["vocab"], 90 + i) for i in range(6)]
    plain = TC.plain(cfg, w, "float32")
    want = [plain.forward(r) for r in reqs]
    rp = Replay(folder, "float32", str(tmp_path / "logits"), max_tokens=sum(len(r) for r in reqs))
    try:
        first = rp.step([{"id": str(i), "tokens": r[:60], "want": [0, 59]} for i, r in enumerate(reqs)])
        TC.rows_close(first, torch.cat([wl[[0, 59]] for wl in want]), "float32", "replay of six, first step")
        for p in range(60, 71):
            live = [i for i, r in enumerate(reqs) if len(r) > p]
            got = rp.step([{"id": str(i), "tokens": [reqs[i][p]], "want": [0]} for i in live],
                          end=[str(i) for i in live if len(reqs[i]) == p + 1])
            TC.rows_close(got, torch.stack([want[i][p] for i in live]), "float32", f"replay of six, position {p}")
    finally:
        rp.close()
