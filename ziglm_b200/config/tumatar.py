"""Typed configuration of the Tumatar decoder, read from config.json.

The design: every layer is ``x += post(mixer(pre(x)))`` followed, where the layer
has a feed-forward, by ``x += post(ff(pre(x)))``, all four norms RMS norms.  The
mixer is either attention through a low-rank latent (no positions, sigmoid output
gate) or a gated linear recurrence behind a short causal convolution; the
feed-forward is either a dense gated one with clamped inputs or a mixture of
experts routed by sigmoid scores within the best groups of experts.  A run of
consecutive layers may be passed through several times with the same weights,
each pass keeping its own cache or state and starting with a learned vector
added to the residual stream.  The embedding is scaled, the head is the
embedding table, the logits are scaled.

config.json keys
----------------
architecture            "Tumatar"
vocab, width            sizes of the embedding table
embedding.scale         factor on the embedded tokens
norm.eps                epsilon of every norm
layers[i].type          "latent_attention" or "rglru"
layers[i].mixer         latent_attention: heads, dim (query/key size per head), vdim (value size per head),
                        q_rank, kv_rank (sizes of the two latents), scale (factor on the scores);
                        rglru: width (channels), blocks (parts of the block-diagonal gates), conv (taps)
layers[i].mlp           null, or kind "dense" with ff and limit, or kind "moe" with expert.ff and
                        router.experts / router.top / router.groups.count / router.groups.keep
loop                    null/absent, or start, stop, times: layers start..stop-1 run ``times`` times in a row
logit_scale             factor on the logits

Every size and constant is read from here; nothing is inferred from tensor shapes (the loader checks the
shapes against this configuration).  Tensor names: ``embed``, ``final.norm``, ``loop.step`` and, under
``l<i>.``, ``norm1``, ``norm1b``, ``norm2``, ``norm2b``, ``mix.*`` and ``mlp.*``.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .common import ConfigError, architecture_name
from .spec import FeedForwardSpec, HookSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec

# Constants the design fixes.
GATE_SLOPE = 1.702          # dense feed-forward: gate * sigmoid(GATE_SLOPE * gate)
DECAY_RATE = 8.0            # recurrence: log a = -DECAY_RATE * r * softplus(lam)
GROUP_BEST = 2              # a group of experts is scored by the sum of this many of its best choice scores


def _obj(d: Mapping[str, Any], key: str, where: str, optional: bool = False) -> Optional[Mapping[str, Any]]:
    v = d.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}'{key}' must be an object, found {v!r}")
    return v


def _int(d: Mapping[str, Any], key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: {where}'{key}' must be an integer, found {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: {where}'{key}' must be >= {minimum}, found {v}")
    return v


def _num(d: Mapping[str, Any], key: str, where: str, positive: bool = True) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"config.json: {where}'{key}' must be a finite number, found {v!r}")
    if positive and float(v) <= 0.0:
        raise ConfigError(f"config.json: {where}'{key}' must be positive, found {v}")
    return float(v)


@dataclass(frozen=True)
class TumatarConfig:
    ARCHITECTURE = "Tumatar"

    raw: Mapping[str, Any]          # the checked dictionary, as it was read
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    logit_scale: float
    layers: Tuple[Mapping[str, Any], ...]
    loop: Optional[Tuple[int, int, int]]      # start, stop, times

    @property
    def architecture(self) -> str:
        return self.ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def eos_token_ids(self) -> Tuple[int, ...]:
        return ()

    # -------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "TumatarConfig":
        if architecture_name(d) != cls.ARCHITECTURE:
            raise ConfigError(f"config.json names the architecture {architecture_name(d)!r}, not {cls.ARCHITECTURE!r}")
        vocab = _int(d, "vocab", "")
        width = _int(d, "width", "")
        emb = _obj(d, "embedding", "")
        norm = _obj(d, "norm", "")
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = layer.get("type")
            m = _obj(layer, "mixer", where)
            if kind == "latent_attention":
                for k in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
                    _int(m, k, where + "mixer.")
                _num(m, "scale", where + "mixer.")
            elif kind == "rglru":
                w, b = _int(m, "width", where + "mixer."), _int(m, "blocks", where + "mixer.")
                _int(m, "conv", where + "mixer.")
                if w % b:
                    raise ConfigError(f"config.json: {where}mixer.width {w} is not a multiple of its blocks {b}")
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not known (latent_attention, rglru)")
            mlp = _obj(layer, "mlp", where, optional=True)
            if mlp is not None:
                fk = mlp.get("kind")
                if fk == "dense":
                    _int(mlp, "ff", where + "mlp.")
                    _num(mlp, "limit", where + "mlp.")
                elif fk == "moe":
                    _int(_obj(mlp, "expert", where + "mlp."), "ff", where + "mlp.expert.")
                    r = _obj(mlp, "router", where + "mlp.")
                    E, top = _int(r, "experts", where + "mlp.router."), _int(r, "top", where + "mlp.router.")
                    g = _obj(r, "groups", where + "mlp.router.")
                    count, keep = _int(g, "count", where + "mlp.router.groups."), _int(g, "keep", where + "mlp.router.groups.")
                    if E % count or keep > count or top > keep * (E // count):
                        raise ConfigError(f"config.json: {where}mlp.router: {E} experts in {count} groups of which {keep} "
                                          f"are kept cannot give {top} experts a token")
                else:
                    raise ConfigError(f"config.json: {where}mlp.kind {fk!r} is not known (dense, moe)")
            checked.append(copy.deepcopy(dict(layer)))
        loop = _obj(d, "loop", "", optional=True)
        loop_t = None
        if loop is not None:
            start, stop = _int(loop, "start", "loop.", 0), _int(loop, "stop", "loop.")
            times = _int(loop, "times", "loop.")
            if not 0 <= start < stop <= len(checked):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(checked)} layers")
            loop_t = (start, stop, times)
        return cls(raw=copy.deepcopy(dict(d)), vocab=vocab, width=width,
                   embedding_scale=_num(emb, "scale", "embedding."), eps=_num(norm, "eps", "norm."),
                   logit_scale=_num(d, "logit_scale", ""), layers=tuple(checked), loop=loop_t)

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(dict(self.raw))

    # ------------------------------------------------------------------ layout
    def running_order(self) -> Tuple[Tuple[int, Optional[int]], ...]:
        """(layer, pass number at the first layer of a pass of the repeated run or None) in running order."""
        n = len(self.layers)
        if self.loop is None:
            return tuple((i, None) for i in range(n))
        start, stop, times = self.loop
        order = [(i, None) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None) for i in range(start, stop)]
        order += [(i, None) for i in range(stop, n)]
        return tuple(order)

    def model_spec(self) -> ModelSpec:
        d, eps = self.width, self.eps
        norm = NormSpec("rmsnorm", d, eps)
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            names = {"mixer_norm.weight": "norm1", "mixer_post_norm.weight": "norm1b"}
            if layer["type"] == "latent_attention":
                mixer = MixerSpec(kind="latent_attention", width=d, n_heads=m["heads"], n_kv_heads=1, head_dim=m["dim"],
                                  scale=float(m["scale"]),
                                  options={"value_dim": m["vdim"], "q_rank": m["q_rank"], "kv_rank": m["kv_rank"],
                                           "norm_eps": eps, "gate": "sigmoid"})
                for local, name in (("dq.weight", "dq"), ("dq_norm.weight", "dq.norm"), ("uq.weight", "uq"),
                                    ("dkv.weight", "dkv"), ("dkv_norm.weight", "dkv.norm"), ("uk.weight", "uk"),
                                    ("uv.weight", "uv"), ("g.weight", "g"), ("o.weight", "o")):
                    names["mixer." + local] = "mix." + name
            else:
                mixer = MixerSpec(kind="rglru", width=d,
                                  options={"channels": m["width"], "blocks": m["blocks"], "taps": m["conv"],
                                           "decay_rate": DECAY_RATE})
                for local, name in (("y.weight", "y"), ("y.bias", "y.b"), ("x.weight", "x"), ("x.bias", "x.b"),
                                    ("conv.weight", "conv"), ("conv.bias", "conv.b"), ("ra.weight", "ra"),
                                    ("ra.bias", "ra.b"), ("ri.weight", "ri"), ("ri.bias", "ri.b"), ("lam", "lam"),
                                    ("o.weight", "o")):
                    names["mixer." + local] = "mix." + name
            mlp = layer.get("mlp")
            ffn = ffn_norm = None
            options: Dict[str, Any] = {"mixer_post_norm": norm}
            if mlp is not None:
                ffn_norm = norm
                options["ffn_post_norm"] = norm
                names["ffn_norm.weight"] = "norm2"
                names["ffn_post_norm.weight"] = "norm2b"
                if mlp["kind"] == "dense":
                    ffn = FeedForwardSpec(kind="gated_mlp", width=d, intermediate=mlp["ff"], activation="swish_clamped",
                                          options={"limit": float(mlp["limit"]), "slope": GATE_SLOPE})
                    for part in ("gate", "up", "down"):
                        names[f"ffn.{part}.weight"] = f"mlp.{part}"
                else:
                    r = mlp["router"]
                    E = r["experts"]
                    ffn = FeedForwardSpec(kind="moe", width=d, intermediate=mlp["expert"]["ff"], activation="silu",
                                          options={"experts": E, "top": r["top"], "groups": r["groups"]["count"],
                                                   "keep_groups": r["groups"]["keep"], "group_best": GROUP_BEST,
                                                   "score": "sigmoid", "correction": True, "renormalize": False})
                    names["ffn.router.weight"] = "mlp.router"
                    names["ffn.correction"] = "mlp.correction"
                    for e in range(E):
                        for part in ("gate", "up", "down"):
                            names[f"ffn.e{e}.{part}.weight"] = f"mlp.e{e}.{part}"
            layers.append(LayerSpec(block="sandwich", prefix=f"l{i}.", mixer_norm=norm, mixer=mixer, ffn_norm=ffn_norm,
                                    ffn=ffn, names=names, options=options))
        order = self.running_order()
        place_hooks = {}
        n_passes = 0
        for place, (_, pass_no) in enumerate(order):
            if pass_no is not None:
                n_passes = max(n_passes, pass_no + 1)
                place_hooks[place] = HookSpec("add_row", {"rows": n_passes, "row": pass_no, "width": d},
                                              {"table": "loop.step"})
        # every hook declares the whole table
        place_hooks = {p: HookSpec(h.kind, {**h.options, "rows": n_passes}, h.names) for p, h in place_hooks.items()}
        return ModelSpec(
            architecture=self.ARCHITECTURE, width=d, vocab_size=self.vocab, layers=tuple(layers),
            schedule=tuple(li for li, _ in order), final_norm=norm, embedding_name="embed",
            final_norm_name="final.norm", head_name=None, embedding_scale=self.embedding_scale, max_positions=0,
            logits_hook=HookSpec("scale", {"factor": self.logit_scale}) if self.logit_scale != 1.0 else None,
            place_hooks=place_hooks)
