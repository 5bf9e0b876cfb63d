"""A plain, slow statement of the Tikalix decoder in PyTorch on the CPU: the oracle of the tests.

One function per mechanism, written from the design's equations and sharing no code with the library's product
path.  ``dtype`` float32 computes everything in float32 (float64 with ``wide=True``); bfloat16 rounds where the
library may: the operands and results of the projections and the activations between them, while positions,
angles, scores, softmax, norms, router and the residual stream stay float32.

Notation: d model width, H query heads, G key/value heads, D query/key size, V value size, R rotated dimensions,
T tokens of one sequence, m the residual multiplier.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Mapping, Optional

import torch

GATE_SLOPE = 1.702
YARN_AMPLITUDE = 0.1


class Plain:
    """How numbers are held: ``act`` is the type of projections' inputs and outputs, ``acc`` the type of
    everything the design computes in 32-bit (float64 stands in for it when a tighter oracle is wanted)."""

    def __init__(self, dtype: torch.dtype = torch.float32, wide: bool = False):
        self.act = dtype
        self.acc = torch.float64 if wide else torch.float32

    def linear(self, x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
        """y = W x (+ b): operands rounded to ``act``, summed in ``acc``, result rounded to ``act``."""
        y = x.to(self.act).to(self.acc) @ w.to(self.act).to(self.acc).t()
        if b is not None:
            y = y + b.to(self.act).to(self.acc)
        return y.to(self.act).to(self.acc)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the gain minus one."""
    return rms_unit(x, eps) * (1.0 + w.to(x.dtype))


def rotary_frequencies(rot: Mapping[str, Any]):
    """(frequency per pair [R/2] in float64, amplitude): YaRN-stretched when ``rot['scaling']`` is given."""
    R, base = int(rot["dims"]), float(rot["base"])
    half = R // 2
    f = [base ** (-2.0 * i / R) for i in range(half)]
    s = rot.get("scaling")
    if not s:
        return torch.tensor(f, dtype=torch.float64), 1.0
    factor, orig = float(s["factor"]), float(s["original"])

    def pair_of(turns: float) -> float:
        return R * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(s["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(s["slow"]))), R - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64), YARN_AMPLITUDE * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Mapping[str, Any]) -> torch.Tensor:
    """x: [T, heads, D]; the first R dimensions of every head are turned, pair (i, i + R/2)."""
    R = int(rot["dims"])
    half = R // 2
    freq, amp = rotary_frequencies(rot)
    # the angle is formed in 32-bit from a 32-bit frequency, as position * frequency
    ang = positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]
    ang = ang.to(x.dtype)
    c, s = (torch.cos(ang) * amp)[:, None, :], (torch.sin(ang) * amp)[:, None, :]
    u, v = x[..., :half], x[..., half:R]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., R:]], dim=-1)


def soft_cap(s: torch.Tensor, cap: Optional[float]) -> torch.Tensor:
    return s if not cap else cap * torch.tanh(s / cap)


def attention_mixer(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping[str, Any], eps: float,
                    past: Optional[Dict[str, torch.Tensor]] = None, first_position: int = 0):
    """Causal grouped-query attention of one sequence.  ``h`` [T, d] are the rows of the step; ``past`` holds the
    keys and values of the positions before ``first_position`` (and receives the new ones)."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = p.linear(h, w["q"], w["q.b"]).view(T, H, D)
    k = p.linear(h, w["k"], w["k.b"]).view(T, G, D)
    v = p.linear(h, w["v"], w["v.b"]).view(T, G, V)
    pos = torch.arange(first_position, first_position + T)
    q = rms_unit(rotate(q, pos, m["rot"]), eps)
    k = rms_unit(rotate(k, pos, m["rot"]), eps)
    if p.act != torch.float32:
        # what the library keeps in its cache and feeds its score product is rounded once, after the unit norm
        q, k = q.to(p.act).to(p.acc), k.to(p.act).to(p.acc)
    if past is not None:
        if "k" in past:
            k = torch.cat([past["k"], k], dim=0)
            v = torch.cat([past["v"], v], dim=0)
        past["k"], past["v"] = k, v
    n_keys = k.shape[0]
    out = torch.zeros(T, H, V, dtype=p.acc)
    key_pos = torch.arange(n_keys)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head, :] @ k[:, g, :].t()) * float(m["scale"])
        s = soft_cap(s, m.get("softcap"))
        s = s.masked_fill(key_pos[None, :] > pos[:, None], float("-inf"))
        out[:, head, :] = torch.softmax(s, dim=-1) @ v[:, g, :]
    out = out.reshape(T, H * V).to(p.act).to(p.acc)
    gate = torch.sigmoid(p.linear(h, w["g"]))
    return p.linear(out * gate, w["o"])


def relu_squared_ff(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor]) -> torch.Tensor:
    a = torch.relu(p.linear(h, w["up"]))
    return p.linear(a * a, w["down"])


def clamped_expert(p: Plain, h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
                   limit: float) -> torch.Tensor:
    g = p.linear(h, gate).clamp(max=limit)
    u = p.linear(h, up).clamp(min=-limit, max=limit)
    return p.linear(g * torch.sigmoid(GATE_SLOPE * g) * (u + 1.0), down)


def route(p: Plain, h: torch.Tensor, router: torch.Tensor, top: int):
    """(chosen experts [T, top] by falling logit, their weights: the softmax over the chosen logits alone)."""
    z = h.to(p.act).to(p.acc) @ router.to(p.act).to(p.acc).t()
    best, ids = torch.topk(z, top, dim=-1)
    return ids, torch.softmax(best, dim=-1)


def experts_ff(p: Plain, h: torch.Tensor, w: Mapping[str, torch.Tensor], mlp: Mapping[str, Any]) -> torch.Tensor:
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    limit = float(mlp["expert"]["limit"])
    ids, weights = route(p, h, w["router"], top)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=p.acc)
    for e in range(E):
        rows, slot = (ids == e).nonzero(as_tuple=True)
        if rows.numel():
            y = clamped_expert(p, h[rows], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)
            out.index_add_(0, rows, y * weights[rows, slot][:, None])
    shared = mlp.get("shared")
    if shared:
        out = out + clamped_expert(p, h, w["shared.gate"], w["shared.up"], w["shared.down"], float(shared["limit"]))
    return out


def _sub(tensors: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


class PlainTikalix:
    """The whole model over one sequence at a time, with keys and values kept between calls."""

    def __init__(self, config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor],
                 dtype: torch.dtype = torch.float32, wide: bool = False):
        self.c = config
        self.p = Plain(dtype, wide)
        self.w = {k: (v if v.dtype in (torch.int32, torch.int64) else v.to(self.p.acc)) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.m = float(config["residual_mult"])

    def new_state(self) -> List[Dict[str, torch.Tensor]]:
        return [{} for _ in self.c["layers"]]

    def forward(self, tokens: List[int], state: Optional[List[Dict[str, torch.Tensor]]] = None,
                first_position: int = 0, layers_out: Optional[list] = None) -> torch.Tensor:
        """Logits [T, vocab] of the given tokens, which follow ``first_position`` tokens held in ``state``."""
        c, p, w = self.c, self.p, self.w
        x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float(c["embedding"]["scale"])
        for i, layer in enumerate(c["layers"]):
            lw = _sub(w, f"l{i}.")
            if layer["type"] != "attention":
                raise ValueError(f"layer type {layer['type']!r} is not part of the design")
            y = attention_mixer(p, x, _sub(lw, "mix."), layer["mixer"], self.eps,
                                None if state is None else state[i], first_position)
            x = x + self.m * norm_around_zero(y, lw["norm1"], self.eps)
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp["kind"] == "dense":
                    y = relu_squared_ff(p, x, _sub(lw, "mlp."))
                elif mlp["kind"] == "moe":
                    y = experts_ff(p, x, _sub(lw, "mlp."), mlp)
                else:
                    raise ValueError(f"feed-forward kind {mlp['kind']!r} is not part of the design")
                x = x + self.m * norm_around_zero(y, lw["norm2"], self.eps)
            if layers_out is not None:
                layers_out.append(x.clone())
        h = norm_around_zero(x, w["final.norm"], self.eps)
        return (h.to(p.act).to(p.acc) @ w["head"].to(p.act).to(p.acc).t()).to(torch.float32)
