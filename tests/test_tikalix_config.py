"""Tikalix without a GPU: the configuration reader and its refusals, the layout it produces, the frequency table
against the plain implementation's and against values worked out by hand, and the plain implementation's own
parts (router, soft cap, rotation) on cases whose answer is known."""
import math

import pytest
import torch

import plain_tikalix as P
import tikalix_cases as TC
from ziglm_b200 import ConfigError, config_from_dict
from ziglm_b200.engine.model import declare_parameters
from ziglm_b200.parts.rope import inverse_frequencies


def test_layout_and_names():
    conf = config_from_dict(TC.config("A"))
    spec = conf.model_spec()
    assert spec.architecture == "Tikalix" and spec.head_name == "head" and spec.embedding_scale == 3.0
    assert [l.block for l in spec.layers] == ["postnorm"] * 3
    assert spec.layers[1].ffn is None and spec.layers[0].ffn.kind == "mlp" and spec.layers[2].ffn.kind == "moe"
    names = declare_parameters(spec)
    for n, shape in (("embed", (211, 96)), ("head", (211, 96)), ("final.norm", (96,)), ("l0.norm1", (96,)),
                     ("l0.mix.q", (144, 96)), ("l0.mix.q.b", (144,)), ("l0.mix.k", (48, 96)), ("l0.mix.v", (80, 96)),
                     ("l0.mix.v.b", (80,)), ("l0.mix.g", (240, 96)), ("l0.mix.o", (96, 240)), ("l0.mlp.up", (136, 96)),
                     ("l0.mlp.down", (96, 136)), ("l2.mlp.router", (6, 96)), ("l2.mlp.e5.gate", (40, 96)),
                     ("l2.mlp.e0.down", (96, 40)), ("l2.mlp.shared.up", (24, 96)), ("l2.mlp.shared.down", (96, 24))):
        assert tuple(names[n].shape) == shape, n
    assert "l1.norm2" not in names and "l1.mlp.up" not in names and "l0.mix.g.b" not in names
    m = spec.layers[0].mixer
    assert (m.n_heads, m.n_kv_heads, m.head_dim, m.options["value_dim"], m.scale, m.options["softcap"]) == (6, 2, 24, 40, 0.3, 4.0)
    assert spec.layers[1].mixer.options["softcap"] is None and spec.layers[1].mixer.position.scaling is None
    assert conf.to_dict() == TC.config("A")


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), 0, "vocab"), (("residual_mult",), None, "residual_mult"), (("layers", 0, "type"), "mamba", "type"),
    (("layers", 0, "mixer", "heads"), 5, "kv_heads"), (("layers", 0, "mixer", "rot", "dims"), 15, "rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 26, "rot.dims"), (("layers", 0, "mixer", "softcap"), "x", "softcap"),
    (("layers", 0, "mixer", "rot", "scaling", "factor"), None, "factor"), (("layers", 0, "mlp", "kind"), "glu", "kind"),
    (("layers", 2, "mlp", "router", "top"), 7, "router"), (("layers", 2, "mlp", "expert", "limit"), -1.0, "limit"),
    (("layers", 2, "mlp", "shared", "ff"), 0, "shared"), (("norm",), 3, "norm"),
])
def test_refusals_name_the_key(path, value, word):
    cfg = TC.config("A")
    d = cfg
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)


def test_frequencies_by_hand_and_against_the_library():
    # 8 pairs, base 100, original 64: the pair at which a frequency makes r turns over 64 positions is
    # 16 ln(64 / (2 pi r)) / (2 ln 100); fast 8 -> 0.42 -> 0, slow 0.5 -> 5.24 -> 6: ramp i / 6
    rot = TC.config("A")["layers"][0]["mixer"]["rot"]
    f, amp = P.rotary_frequencies(rot)
    base = [100.0 ** (-2 * i / 16) for i in range(8)]
    for i in range(8):
        ramp = min(i / 6.0, 1.0)
        assert f[i].item() == pytest.approx(base[i] * (1 - ramp) + base[i] / 4 * ramp, rel=1e-12)
    assert amp == pytest.approx(0.1 * math.log(4.0) + 1.0)
    # a table of one pair whose ramp has no width: lo = hi, the pair lies on it
    f1, _ = P.rotary_frequencies({"dims": 2, "base": 7.0, "scaling": {"factor": 1.5, "original": 32, "fast": 4.0, "slow": 1.0}})
    assert f1.tolist() == [1.0]
    # ends that cross (a short original length pushes hi below lo): the ramp is a step at lo
    crossing = {"dims": 8, "base": 4.0, "scaling": {"factor": 2.0, "original": 7, "fast": 0.01, "slow": 1.0}}
    fx, _ = P.rotary_frequencies(crossing)
    pair = lambda t: 8 * math.log(7 / (2 * math.pi * t)) / (2 * math.log(4.0))
    lo, hi = max(math.floor(pair(0.01)), 0), min(math.ceil(pair(1.0)), 7)
    assert hi < lo
    assert fx.tolist() == pytest.approx([4.0 ** (-2 * i / 8) * (0.5 if i > lo else 1.0) for i in range(4)])
    cfg = TC.config("A")
    cfg["layers"][0]["mixer"]["rot"] = crossing
    cfg["layers"][0]["mixer"]["dim"] = 24
    pos = config_from_dict(cfg).model_spec().layers[0].mixer.position
    assert torch.allclose(inverse_frequencies(pos.rotary_dim, pos.theta, pos.scaling).double(), fx, rtol=1e-6, atol=0)
    for name in ("A", "B", "C"):
        conf = config_from_dict(TC.config(name))
        for layer, ls in zip(TC.config(name)["layers"], conf.model_spec().layers):
            want, amp = P.rotary_frequencies(layer["mixer"]["rot"])
            pos = ls.mixer.position
            got = inverse_frequencies(pos.rotary_dim, pos.theta, pos.scaling)
            assert torch.allclose(got.double(), want, rtol=1e-6, atol=0)
            assert (pos.scaling or {}).get("attention_factor", 1.0) == pytest.approx(amp)


def test_plain_router_and_cap():
    p = P.Plain()
    h = torch.eye(4)
    router = torch.tensor([[1.0, 0, 0, 5], [3.0, 0, 0, 5], [2.0, 0, 0, -9], [0.0, 0, 0, 5.5]])
    ids, wts = P.route(p, h[[0, 3]], router, 2)
    assert ids.tolist() == [[1, 2], [3, 0]] or ids.tolist() == [[1, 2], [3, 1]]
    assert wts[0].tolist() == pytest.approx([math.e / (1 + math.e), 1 / (1 + math.e)])
    assert ids[1, 0].item() == 3 and wts[1, 0].item() == pytest.approx(1 / (1 + math.exp(-0.5)))
    assert P.soft_cap(torch.tensor([100.0, -100.0, 0.1]), 2.0).tolist() == pytest.approx([2.0, -2.0, 2 * math.tanh(0.05)])
    assert P.soft_cap(torch.tensor([100.0]), None).item() == 100.0


def test_plain_rotation_turns_pairs_half_a_head_apart():
    x = torch.zeros(1, 1, 6)
    x[0, 0, 0] = 1.0
    x[0, 0, 5] = 7.0
    y = P.rotate(x.clone(), torch.tensor([3]), {"dims": 4, "base": 10.0})
    # pair (0, 2) turns by 3 * 1, pair (1, 3) by 3 * 10^-0.5; dimensions 4 and 5 pass
    assert y[0, 0].tolist() == pytest.approx([math.cos(3.0), 0.0, math.sin(3.0), 0.0, 0.0, 7.0], abs=1e-6)


def test_prefill_equals_decoding_in_the_plain_implementation():
    cfg = TC.config("C")
    conf = config_from_dict(cfg)
    from ziglm_b200.weights import random_tensors
    w = dict(random_tensors(declare_parameters(conf.model_spec()), 3, torch.float32, torch.device("cpu"), std=0.12, norm_jitter=0.3))
    m = P.PlainTikalix(cfg, w)
    toks = list(range(1, 30))
    whole = m.forward(toks)
    st = m.new_state()
    rows = [m.forward(toks[:20], st, 0)] + [m.forward([t], st, 20 + i) for i, t in enumerate(toks[20:])]
    assert (torch.cat(rows) - whole).abs().max() < 1e-4


def test_shapes_for_random_models():
    from ziglm_b200.config import shape
    for name in ("tikalix-1b", "tikalix-8b"):
        conf = config_from_dict(shape(name))
        spec = conf.model_spec()
        assert spec.layers[0].mixer.kind == "capped_attention"
        assert {l.ffn.kind for l in spec.layers} == {"mlp", "moe"}
