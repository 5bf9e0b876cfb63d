"""Small Tumatar configurations for the tests, and how a model with tensors the test controls is built.

The configurations differ from one another in every size and option: heads that share nothing with powers of
two, value sizes other than the key size, latents of 44, 64, 128 and 320 elements (64 and 128 are what the
tensor-core attention takes in bfloat16; 320 is above the 256 of a usual head; 44 is no multiple of 8), a recurrence with one block
and one tap (sizes that make parts of the formulas trivial), layers without a feed-forward, experts without
groups, a repeated run of layers, and none.
"""
from __future__ import annotations

import copy
from typing import Callable, Dict, Optional

import torch


def _moe(ff, experts, top, count, keep):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top,
                                                            "groups": {"count": count, "keep": keep}}}


def _lat(heads, dim, vdim, q_rank, kv_rank, scale):
    return {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}


# a repeated run (layers 1 and 2, twice), a layer without a feed-forward, experts in groups, one block / one tap
CFG_A = {
    "architecture": "Tumatar", "vocab": 211, "width": 96, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "logit_scale": 0.5, "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        {"type": "latent_attention", "mixer": _lat(3, 24, 16, 40, 44, 0.2), "mlp": _moe(40, 8, 2, 4, 2)},
        {"type": "rglru", "mixer": {"width": 64, "blocks": 4, "conv": 3}, "mlp": None},
        {"type": "latent_attention", "mixer": _lat(4, 16, 32, 24, 64, 0.25),
         "mlp": {"kind": "dense", "ff": 136, "limit": 0.75}},
        {"type": "rglru", "mixer": {"width": 80, "blocks": 1, "conv": 1}, "mlp": _moe(24, 6, 1, 1, 1)},
    ],
}
# no repeated run; the latent the tensor-core kernels take at head size 128; factors on the scores that make the
# softmax sharp (score differences of a few units), so that a query picks out few keys, anywhere in its past
CFG_B = {
    "architecture": "Tumatar", "vocab": 300, "width": 128, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "logit_scale": 1.0, "loop": None,
    "layers": [
        {"type": "rglru", "mixer": {"width": 96, "blocks": 3, "conv": 4}, "mlp": {"kind": "dense", "ff": 200, "limit": 2.0}},
        {"type": "latent_attention", "mixer": _lat(5, 32, 24, 56, 128, 0.5), "mlp": _moe(64, 9, 3, 3, 2)},
        {"type": "latent_attention", "mixer": _lat(2, 40, 40, 32, 320, 0.3), "mlp": None},
    ],
}
# the whole stack repeated three times, one layer of each kind
CFG_C = {
    "architecture": "Tumatar", "vocab": 97, "width": 64, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6},
    "logit_scale": 2.0, "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        {"type": "rglru", "mixer": {"width": 64, "blocks": 2, "conv": 2}, "mlp": _moe(32, 4, 2, 2, 1)},
        {"type": "latent_attention", "mixer": _lat(2, 32, 32, 16, 64, 1.0), "mlp": {"kind": "dense", "ff": 96, "limit": 1.5}},
    ],
}
# more heads than the tensor-core attention takes on one key/value head (they go through it 16 at a time), and
# sizes that are no multiple of 8 anywhere (head 12, value 6, query latent 20, 42 channels in blocks of 14): the
# kernels that move sixteen bytes at a time step aside for the ones that take any size
CFG_D = {
    "architecture": "Tumatar", "vocab": 150, "width": 64, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
    "logit_scale": 1.0,
    "layers": [
        {"type": "latent_attention", "mixer": _lat(20, 12, 6, 20, 64, 0.5), "mlp": {"kind": "dense", "ff": 76, "limit": 3.0}},
        {"type": "rglru", "mixer": {"width": 42, "blocks": 3, "conv": 5}, "mlp": _moe(20, 3, 2, 1, 1)},
    ],
}
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def for_type(cfg: dict, dn: str) -> dict:
    """In bfloat16 the factors on the scores are a quarter: with a sharp softmax a rounding that moves a score
    moves the residual stream enough for routers further up to send many tokens to other experts, in the plain
    implementation's own bfloat16 roundings too, and a comparison row by row then says nothing.  float32 keeps the
    sharp scores."""
    if dn == "bfloat16":
        for layer in cfg["layers"]:
            if layer["type"] == "latent_attention":
                layer["mixer"]["scale"] *= 0.25
    return cfg


def long_memory(w: Dict[str, torch.Tensor]) -> None:
    """Make every recurrence remember: lam far below zero gives decays close to 1, so a state that is lost,
    zeroed or taken from another sequence shows hundreds of tokens later.  And push every correction of a router
    below -1, so that all choice scores are negative (a masked group must count as minus infinity, not as 0)."""
    for name, t in w.items():
        if name.endswith(".mix.lam"):
            t.copy_(t.float().mul(0.5).sub(5.0).to(t.dtype))
        if name.endswith(".mlp.correction"):
            t.copy_(t.float().sub(1.5).to(t.dtype))


def build(cfg: dict, seed: int, dn: str, tweak: Optional[Callable] = long_memory, std: float = 0.12, **options):
    """(engine, config dictionary, tensors on the CPU) of a model with random weights, changed by ``tweak``."""
    from ziglm_b200 import config_from_dict
    from ziglm_b200.engine.engine import Engine, EngineOptions
    from ziglm_b200.engine.model import Model, declare_parameters
    from ziglm_b200.weights import random_tensors
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dn]
    conf = config_from_dict(cfg)
    spec = conf.model_spec()
    dev = torch.device("cuda:0")
    w = dict(random_tensors(declare_parameters(spec), seed, dtype, dev, std=std, norm_jitter=0.1))
    if tweak is not None:
        tweak(w)
    model = Model(spec, dtype, dev)
    model.bind(w)
    opts = dict(dtype=dn, max_tokens=1024, max_batch=4, max_seq_len=512)
    opts.update(options)
    eng = Engine(conf, model, EngineOptions(**opts))
    return eng, cfg, {k: v.detach().cpu() for k, v in w.items()}


def rows_close(got: torch.Tensor, want: torch.Tensor, dn: str, what: str = "") -> None:
    """Row by row: the difference of the logits (mean taken off, root mean square over the vocabulary) relative
    to the root mean square of the row.  float32: every row within 3e-5.  bfloat16: all rows but one in twenty-five (or two)
    within 0.04 (a router's close call may send a token to another expert, which with one expert a token changes
    the whole feed-forward's output), and those within 1."""
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    d = got - want
    d = d - d.mean(dim=1, keepdim=True)
    ref = want - want.mean(dim=1, keepdim=True)
    err = d.pow(2).mean(dim=1).sqrt() / ref.pow(2).mean(dim=1).sqrt().clamp_min(1e-6)
    assert torch.isfinite(err).all(), f"{what}: a row is not finite"
    if dn == "float32":
        assert err.max().item() < 3e-5, f"{what}: row {int(err.argmax())} differs by {err.max().item():.3g}"
    else:
        over = int((err > 0.04).sum())
        assert err.max().item() < 1.0 and over <= max(2, got.shape[0] // 25), \
            f"{what}: {over} of {got.shape[0]} rows differ, the worst (row {int(err.argmax())}) by {err.max().item():.3g}"
