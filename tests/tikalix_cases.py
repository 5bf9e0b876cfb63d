"""Small Tikalix configurations for the tests, and how a model with tensors the test controls is built.

The configurations differ from one another in every size and option: group sizes 1, 2, 3 and 5; key sizes above,
below and equal to the value size; heads of 64 and 128 (what the tensor-core attention takes in bfloat16) and
heads that are no multiple of 8; rotation over the whole head, over a part of it and over two dimensions; YaRN
stretching with ramps that lie inside, at the edge of and outside the table, and none; soft caps that bite, that
barely do, and none; layers without a feed-forward; experts with and without a shared one, one expert a token,
all experts a token; a residual multiplier of one and an embedding scale of one.
"""
from __future__ import annotations

import copy
from typing import Callable, Dict, Optional

import torch


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _att(heads, kv, dim, vdim, scale, softcap, rot):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if softcap != "absent":
        m["softcap"] = softcap
    return m


def _moe(ff, limit, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


# groups of 3 and 1; value heads larger and smaller than key heads; part of the head rotated; a cap that bites
CFG_A = {
    "architecture": "Tikalix", "vocab": 211, "width": 96, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "residual_mult": 0.5,
    "layers": [
        {"type": "attention", "mixer": _att(6, 2, 24, 40, 0.3, 4.0, _rot(16, 100.0, (4.0, 64, 8.0, 0.5))),
         "mlp": {"kind": "dense", "ff": 136}},
        {"type": "attention", "mixer": _att(3, 3, 32, 16, 0.2, None, _rot(32, 10000.0)), "mlp": None},
        {"type": "attention", "mixer": _att(4, 1, 16, 16, 0.5, 50.0, _rot(2, 7.0, (1.5, 32, 4.0, 1.0))),
         "mlp": _moe(40, 0.75, 6, 2, (24, 2.0))},
    ],
}
# the head sizes of the tensor-core kernels (64 and 128, keys and values alike), with and without a cap
CFG_B = {
    "architecture": "Tikalix", "vocab": 300, "width": 128, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "residual_mult": 1.0,
    "layers": [
        {"type": "attention", "mixer": _att(4, 2, 64, 64, 0.25, 20.0, _rot(64, 10000.0, (8.0, 128, 32.0, 1.0))),
         "mlp": _moe(64, 3.0, 9, 3)},
        {"type": "attention", "mixer": _att(2, 1, 128, 128, 0.4, "absent", _rot(64, 500.0)),
         "mlp": {"kind": "dense", "ff": 200}},
        {"type": "attention", "mixer": _att(5, 5, 64, 56, 0.3, 8.0, _rot(48, 1000.0, (2.0, 4096, 32.0, 1.0))),
         "mlp": _moe(32, 1.0, 4, 4, (48, 0.5))},
    ],
}
# sizes that are no multiple of 8 anywhere, a group of 5, one expert a token
CFG_C = {
    "architecture": "Tikalix", "vocab": 97, "width": 60, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6},
    "residual_mult": 0.25,
    "layers": [
        {"type": "attention", "mixer": _att(5, 1, 12, 6, 0.6, 2.0, _rot(6, 50.0, (3.0, 16, 2.0, 0.25))),
         "mlp": _moe(20, 1.5, 3, 1, (12, 1.0))},
        {"type": "attention", "mixer": _att(2, 2, 20, 28, 0.2, 25.0, _rot(20, 3000.0)),
         "mlp": {"kind": "dense", "ff": 76}},
    ],
}
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def for_type(cfg: dict, dn: str) -> dict:
    """In bfloat16 the factors on the scores are halved: with a sharp softmax a rounding that moves a score moves the
    residual stream enough for routers further up to send tokens to other experts, in the plain implementation's own
    bfloat16 roundings too, and a comparison row by row then says little.  float32 keeps the sharp scores."""
    if dn == "bfloat16":
        for layer in cfg["layers"]:
            layer["mixer"]["scale"] *= 0.5
    return cfg


def lively(w: Dict[str, torch.Tensor]) -> None:
    """Biases of the size of the projections' outputs (a lost bias shows), and routers with larger weights (logits
    well apart: a close call of the router is rare)."""
    for name, t in w.items():
        if name.endswith(".b"):
            t.copy_((t.float() * 3.0).to(t.dtype))
        if name.endswith(".mlp.router"):
            t.copy_((t.float() * 4.0).to(t.dtype))


def build(cfg: dict, seed: int, dn: str, tweak: Optional[Callable] = lively, std: float = 0.12, **options):
    """(engine, config dictionary, tensors on the CPU) of a model with random weights, changed by ``tweak``."""
    from ziglm_b200 import config_from_dict
    from ziglm_b200.engine.engine import Engine, EngineOptions
    from ziglm_b200.engine.model import Model, declare_parameters
    from ziglm_b200.weights import random_tensors
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dn]
    conf = config_from_dict(cfg)
    spec = conf.model_spec()
    dev = torch.device("cuda:0")
    w = dict(random_tensors(declare_parameters(spec), seed, dtype, dev, std=std, norm_jitter=0.3))
    if tweak is not None:
        tweak(w)
    model = Model(spec, dtype, dev)
    model.bind(w)
    opts = dict(dtype=dn, max_tokens=1024, max_batch=4, max_seq_len=512)
    opts.update(options)
    eng = Engine(conf, model, EngineOptions(**opts))
    return eng, cfg, {k: v.detach().cpu() for k, v in w.items()}


def plain(cfg: dict, w: Dict[str, torch.Tensor], dn: str):
    import plain_tikalix
    return plain_tikalix.PlainTikalix(cfg, w, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dn])


def rows_close(got: torch.Tensor, want: torch.Tensor, dn: str, what: str = "") -> None:
    """Row by row: the difference of the logits (mean taken off, root mean square over the vocabulary) relative
    to the root mean square of the row.  float32: every row within 3e-5.  bfloat16: all rows but one in fifteen
    (or two) within 0.04 (a router's close call may send a token to another expert), and those within 1."""
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
        assert err.max().item() < 1.0 and over <= max(2, got.shape[0] // 15), \
            f"{what}: {over} of {got.shape[0]} rows differ, the worst (row {int(err.argmax())}) by {err.max().item():.3g}"
