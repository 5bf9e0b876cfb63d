"""Typed configuration of the Tikalix decoder, read from config.json.

The design: the sublayers read the residual stream itself and a norm stands behind each of them,
``x += m * norm(mixer(x))`` and then, where the layer has a feed-forward, ``x += m * norm(ff(x))`` with one
multiplier m for the whole model; every norm is an RMS norm whose stored weight is its gain minus one.  The
mixer is causal grouped-query attention with biased q/k/v projections, rotary positions over the first part of
each head (optionally stretched by the YaRN rule, whose amplitude multiplies the cosines and sines), a unit RMS
norm of every rotated query and key head, scores with a factor from the configuration and a tanh soft cap, keys
and values of different sizes, and a sigmoid gate (a projection of the mixer's input) on the concatenated heads
before the output projection.  The feed-forward is a dense one with the squared relu, or a mixture of experts:
the ``top`` largest router logits choose the experts, their weights are the softmax over the chosen logits
alone, every expert is a gated feed-forward with a clamped gate and up and a sloped sigmoid, and an optional
shared expert of the same form runs for every token.  The embedding is scaled; the head is a matrix of its own.

config.json keys
----------------
architecture            "Tikalix"
vocab, width            sizes of the embedding table
embedding.scale         factor on the embedded tokens
norm.eps                epsilon of every norm (also of the unit norm of queries and keys)
residual_mult           m
layers[i].type          "attention"
layers[i].mixer         heads, kv_heads, dim (query/key size per head), vdim (value size per head), scale (factor on
                        the scores), softcap (absent or null: none), rot.dims, rot.base, rot.scaling (absent or
                        null: none; else factor, original, fast, slow)
layers[i].mlp           null, or kind "dense" with ff, or kind "moe" with expert.ff, expert.limit, router.experts,
                        router.top and optionally shared.ff, shared.limit

Every size and constant is read from here; nothing is inferred from tensor shapes (the loader checks the shapes
against this configuration).  Tensor names: ``embed``, ``head``, ``final.norm`` and, under ``l<i>.``, ``norm1``,
``norm2``, ``mix.{q,k,v}`` with ``.b`` biases, ``mix.g``, ``mix.o``, ``mlp.up``/``mlp.down`` (dense),
``mlp.router``, ``mlp.e<j>.{gate,up,down}`` and ``mlp.shared.{gate,up,down}`` (experts).
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .common import ConfigError, architecture_name
from .spec import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
from .tumatar import _int, _num, _obj

# Constants the design fixes.
GATE_SLOPE = 1.702          # experts: gate * sigmoid(GATE_SLOPE * gate)
YARN_AMPLITUDE = 0.1        # cosines and sines are multiplied by YARN_AMPLITUDE * ln(factor) + 1
RAMP_FLOOR = 0.001          # the least width of the ramp between kept and stretched frequencies


def _optional_num(d: Mapping[str, Any], key: str, where: str) -> Optional[float]:
    return None if d.get(key) is None else _num(d, key, where)


@dataclass(frozen=True)
class TikalixConfig:
    ARCHITECTURE = "Tikalix"

    raw: Mapping[str, Any]          # the checked dictionary, as it was read
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    residual_mult: float
    layers: Tuple[Mapping[str, Any], ...]

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
    def from_dict(cls, d: Mapping[str, Any]) -> "TikalixConfig":
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
            if kind != "attention":
                raise ConfigError(f"config.json: {where}type {kind!r} is not known (attention)")
            m = _obj(layer, "mixer", where)
            mw = where + "mixer."
            H, G = _int(m, "heads", mw), _int(m, "kv_heads", mw)
            if H % G:
                raise ConfigError(f"config.json: {mw}heads {H} is not a multiple of kv_heads {G}")
            D = _int(m, "dim", mw)
            _int(m, "vdim", mw)
            _num(m, "scale", mw)
            _optional_num(m, "softcap", mw)
            rot = _obj(m, "rot", mw)
            R = _int(rot, "dims", mw + "rot.")
            if R % 2 or R > D:
                raise ConfigError(f"config.json: {mw}rot.dims {R} must be even and at most dim {D}")
            base = _num(rot, "base", mw + "rot.")
            if base == 1.0:
                raise ConfigError(f"config.json: {mw}rot.base must differ from 1")
            sc = _obj(rot, "scaling", mw + "rot.", optional=True)
            if sc is not None:
                for k in ("factor", "original", "fast", "slow"):
                    _num(sc, k, mw + "rot.scaling.")
            mlp = _obj(layer, "mlp", where, optional=True)
            if mlp is not None:
                fw = where + "mlp."
                fk = mlp.get("kind")
                if fk == "dense":
                    _int(mlp, "ff", fw)
                elif fk == "moe":
                    ex = _obj(mlp, "expert", fw)
                    _int(ex, "ff", fw + "expert.")
                    _num(ex, "limit", fw + "expert.")
                    r = _obj(mlp, "router", fw)
                    E, top = _int(r, "experts", fw + "router."), _int(r, "top", fw + "router.")
                    if top > E:
                        raise ConfigError(f"config.json: {fw}router: {E} experts cannot give {top} a token")
                    sh = _obj(mlp, "shared", fw, optional=True)
                    if sh is not None:
                        _int(sh, "ff", fw + "shared.")
                        _num(sh, "limit", fw + "shared.")
                else:
                    raise ConfigError(f"config.json: {fw}kind {fk!r} is not known (dense, moe)")
            checked.append(copy.deepcopy(dict(layer)))
        return cls(raw=copy.deepcopy(dict(d)), vocab=vocab, width=width,
                   embedding_scale=_num(emb, "scale", "embedding."), eps=_num(norm, "eps", "norm."),
                   residual_mult=_num(d, "residual_mult", ""), layers=tuple(checked))

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(dict(self.raw))

    # ------------------------------------------------------------------ layout
    @staticmethod
    def _position(rot: Mapping[str, Any]) -> PositionSpec:
        sc = rot.get("scaling")
        scaling = None
        if sc is not None:
            factor = float(sc["factor"])
            scaling = {"rope_type": "yarn", "factor": factor, "original_max_position_embeddings": float(sc["original"]),
                       "beta_fast": float(sc["fast"]), "beta_slow": float(sc["slow"]),
                       "attention_factor": YARN_AMPLITUDE * math.log(factor) + 1.0, "min_ramp_width": RAMP_FLOOR}
        # the amplitude belongs to the cosines and sines: a unit norm follows the rotation, and only part of a head
        # may be rotated, so it cannot be moved into the factor on the scores
        return PositionSpec(kind="rope", rotary_dim=int(rot["dims"]), theta=float(rot["base"]), scaling=scaling,
                            options={"amplitude_in_table": True})

    def model_spec(self) -> ModelSpec:
        d, eps = self.width, self.eps
        norm = NormSpec("rmsnorm", d, eps, options={"unit_offset": True})
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            names = {"mixer_post_norm.weight": "norm1", "mixer.g.weight": "mix.g", "mixer.o.weight": "mix.o"}
            for p in ("q", "k", "v"):
                names[f"mixer.{p}.weight"] = f"mix.{p}"
                names[f"mixer.{p}.bias"] = f"mix.{p}.b"
            mixer = MixerSpec(kind="capped_attention", width=d, n_heads=m["heads"], n_kv_heads=m["kv_heads"],
                              head_dim=m["dim"], bias=True, scale=float(m["scale"]), position=self._position(m["rot"]),
                              options={"value_dim": m["vdim"], "qk_norm_eps": eps,
                                       "softcap": None if m.get("softcap") is None else float(m["softcap"]),
                                       "gate": "sigmoid"})
            mlp = layer.get("mlp")
            ffn = None
            options: Dict[str, Any] = {"mixer_post_norm": norm, "residual_mult": self.residual_mult}
            if mlp is not None:
                options["ffn_post_norm"] = norm
                names["ffn_post_norm.weight"] = "norm2"
                if mlp["kind"] == "dense":
                    ffn = FeedForwardSpec(kind="mlp", width=d, intermediate=mlp["ff"], activation="relu2")
                    names["ffn.up.weight"] = "mlp.up"
                    names["ffn.down.weight"] = "mlp.down"
                else:
                    r, ex, sh = mlp["router"], mlp["expert"], mlp.get("shared")
                    E = r["experts"]
                    opts: Dict[str, Any] = {"experts": E, "top": r["top"], "score": "softmax_chosen",
                                            "limit": float(ex["limit"]), "slope": GATE_SLOPE}
                    if sh is not None:
                        opts["shared"] = FeedForwardSpec(kind="gated_mlp", width=d, intermediate=sh["ff"],
                                                         activation="swish_clamped",
                                                         options={"limit": float(sh["limit"]), "slope": GATE_SLOPE})
                        for part in ("gate", "up", "down"):
                            names[f"ffn.shared.{part}.weight"] = f"mlp.shared.{part}"
                    ffn = FeedForwardSpec(kind="moe", width=d, intermediate=ex["ff"], activation="swish_clamped",
                                          options=opts)
                    names["ffn.router.weight"] = "mlp.router"
                    for e in range(E):
                        for part in ("gate", "up", "down"):
                            names[f"ffn.e{e}.{part}.weight"] = f"mlp.e{e}.{part}"
            layers.append(LayerSpec(block="postnorm", prefix=f"l{i}.", mixer_norm=None, mixer=mixer, ffn_norm=None,
                                    ffn=ffn, names=names, options=options))
        return ModelSpec(
            architecture=self.ARCHITECTURE, width=d, vocab_size=self.vocab, layers=tuple(layers),
            schedule=tuple(range(len(layers))), final_norm=norm, embedding_name="embed",
            final_norm_name="final.norm", head_name="head", embedding_scale=self.embedding_scale, max_positions=0)
