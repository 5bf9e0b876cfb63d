"""The Tumatar configuration without a GPU: reading config.json, the layout it gives (schedule of a repeated
run, hooks, tensor names and shapes), refusals that name the key, and the plain implementation's own pieces."""
import copy

import pytest
import torch

import plain_tumatar as P
import tumatar_cases as TC
from ziglm_b200 import ConfigError, config_from_dict
from ziglm_b200.engine.model import declare_parameters


def test_layout_of_a_repeated_run():
    conf = config_from_dict(TC.config("A"))
    spec = conf.model_spec()
    assert spec.architecture == "Tumatar" and spec.head_name is None and spec.embedding_scale == 3.0
    assert spec.schedule == (0, 1, 2, 1, 2, 3)
    assert sorted(spec.place_hooks) == [1, 3] and [spec.place_hooks[p].options["row"] for p in (1, 3)] == [0, 1]
    assert spec.logits_hook.kind == "scale" and spec.logits_hook.options["factor"] == 0.5
    assert spec.layers[1].ffn is None and spec.layers[1].ffn_norm is None and spec.layers[0].ffn.kind == "moe"
    assert [(li, t) for li, t in conf.running_order()] == [(li, t) for li, t in P.running_order(TC.config("A"))]
    decl = declare_parameters(spec)
    assert decl["loop.step"].shape == (2, 96) and decl["embed"].shape == (211, 96) and decl["final.norm"].shape == (96,)
    assert decl["l0.mix.uk"].shape == (72, 44) and decl["l0.mix.uv"].shape == (48, 44) and decl["l0.mix.g"].shape == (48, 96)
    assert decl["l0.mix.dq.norm"].shape == (40,) and decl["l0.mlp.correction"].shape == (8,)
    assert decl["l0.mlp.e7.down"].shape == (96, 40) and "l0.mlp.e8.down" not in decl
    assert decl["l1.mix.ra"].shape == (4, 16, 16) and decl["l1.mix.conv"].shape == (64, 3) and decl["l1.mix.lam"].shape == (64,)
    assert "l1.norm2" not in decl and "l1.norm1b" in decl and decl["l2.mlp.gate"].shape == (136, 96)
    assert conf.to_dict() == TC.config("A")


def test_no_repeated_run_and_a_whole_stack_repeated():
    b = config_from_dict(TC.config("B")).model_spec()
    assert b.schedule == (0, 1, 2) and not b.place_hooks and b.logits_hook is None
    assert "loop.step" not in declare_parameters(b)
    c = config_from_dict(TC.config("C")).model_spec()
    assert c.schedule == (0, 1, 0, 1, 0, 1) and sorted(c.place_hooks) == [0, 2, 4]
    assert declare_parameters(c)["loop.step"].shape == (3, 64)


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "mamba", "type"), (("layers", 0, "mixer", "heads"), 0, "heads"),
    (("layers", 1, "mixer", "blocks"), 5, "blocks"), (("layers", 2, "mlp", "kind"), "sparse", "kind"),
    (("layers", 0, "mlp", "router", "groups", "count"), 3, "groups"), (("loop", "stop"), 9, "loop"),
    (("norm", "eps"), "small", "eps"), (("vocab",), None, "vocab"), (("layers", 2, "mlp", "limit"), -1.0, "limit"),
])
def test_refusals_name_the_key(path, value, word):
    cfg = TC.config("A")
    at = cfg
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


def test_plain_router_masks_groups_with_minus_infinity():
    # experts 0..3 in two groups; every choice score is negative; group 1 is the better one
    z = torch.tensor([-3.0, -2.5, -1.0, -1.2])
    chosen, weights = P.route(z, torch.tensor([-1.0] * 4), top=2, n_groups=2, keep=1)
    assert chosen == [2, 3] and weights == [pytest.approx(torch.sigmoid(z[2]).item()), pytest.approx(torch.sigmoid(z[3]).item())]
    # the correction decides the choice and stays out of the weight
    chosen, weights = P.route(torch.zeros(4), torch.tensor([0.0, 0.3, 0.1, 0.2]), top=1, n_groups=1, keep=1)
    assert chosen == [1] and weights == [0.5]


def test_plain_convolution_and_recurrence():
    x = torch.arange(12.0).view(6, 2)
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])           # channel 0: the current token; channel 1: two back
    u = P.causal_conv(x, taps, torch.zeros(2))
    assert u[:, 0].tolist() == x[:, 0].tolist() and u[:, 1].tolist() == [0.0, 0.0] + x[:4, 1].tolist()
    assert torch.allclose(P.gelu_tanh(torch.tensor([0.0, 3.0])), torch.tensor([0.0, 2.9964]), atol=1e-4)
