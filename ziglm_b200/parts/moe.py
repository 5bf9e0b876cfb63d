"""Mixture of experts: a router picks ``top`` of E small gated feed-forwards for every token.

    z = W_r h (float32)              score = sigmoid(z) (or softmax)         choice = score + correction
    the experts form ``groups`` equal groups of neighbours, a group is scored by the sum of its ``group_best``
    best choice scores, and only experts of the ``keep_groups`` best groups can be chosen;
    out = sum over the chosen e of score_e * W_down[e] (act(W_gate[e] h) * (W_up[e] h))
(the weights are divided by their sum only with ``renormalize``).  Options of the spec: ``experts``, ``top``,
``groups``, ``keep_groups``, ``group_best``, ``score`` ("sigmoid" or "softmax"), ``correction`` (whether a
learned offset per expert enters the choice), ``renormalize``.

The (token, choice) pairs are grouped by expert on the device (nothing is read back, so a decode step stays a
replayable graph), the experts' products run over the groups, each pair's result lands in a float32 row of its
own, and a token's rows are summed in the order of its choices.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import FeedForwardSpec
from .base import ParamDecl, Part, register_feed_forward
from .linear import Linear


class MixtureOfExperts(Part):
    can_overwrite = True

    def __init__(self, spec: FeedForwardSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        o = spec.options
        self.n_experts, self.top = int(o["experts"]), int(o["top"])
        self.groups, self.keep_groups = int(o.get("groups", 1)), int(o.get("keep_groups", o.get("groups", 1)))
        self.group_best = int(o.get("group_best", 2))
        if o.get("score", "sigmoid") not in ("sigmoid", "softmax"):
            raise ValueError(f"moe: router score {o.get('score')!r} is not known (sigmoid, softmax)")
        self.softmax = o.get("score", "sigmoid") == "softmax"
        self.renormalize = bool(o.get("renormalize", False))
        if spec.activation != "silu":
            raise ValueError(f"moe: expert activation {spec.activation!r} is not known (silu)")
        E, G = self.n_experts, self.groups
        if E % G or not 1 <= self.keep_groups <= G or not 1 <= self.top <= self.keep_groups * (E // G):
            raise ValueError(f"moe: {E} experts in {G} groups of which {self.keep_groups} are kept cannot give "
                             f"{self.top} experts a token")
        self.ff = spec.intermediate
        self.router: Optional[torch.Tensor] = None
        self.correction: Optional[torch.Tensor] = None
        self.gate_up: Optional[torch.Tensor] = None     # [E, 2 ff, d]
        self.down: Optional[torch.Tensor] = None        # [E, d, ff]

    @classmethod
    def declare(cls, spec: FeedForwardSpec) -> Dict[str, ParamDecl]:
        o = spec.options
        E, ff, d = int(o["experts"]), spec.intermediate, spec.width
        p = {"router.weight": ParamDecl((E, d))}
        if o.get("correction", False):
            p["correction"] = ParamDecl((E,))
        for e in range(E):
            p[f"e{e}.gate.weight"] = ParamDecl((ff, d))
            p[f"e{e}.up.weight"] = ParamDecl((ff, d))
            p[f"e{e}.down.weight"] = ParamDecl((d, ff))
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        E = self.n_experts
        self.router = tensors["router.weight"].contiguous()
        self.correction = tensors["correction"].float().contiguous() if "correction" in tensors else None
        mats = [tensors[f"e{e}.{n}.weight"] for e in range(E) for n in ("gate", "up", "down")]
        wide = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
        self.gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate.weight"].to(wide), tensors[f"e{e}.up.weight"].to(wide)], dim=0)
                                    for e in range(E)]).contiguous()
        self.down = torch.stack([tensors[f"e{e}.down.weight"].to(wide) for e in range(E)]).contiguous()

    def kernel_libraries(self) -> Tuple[str, ...]:
        return ("moe", "gemm_generic")

    def forward(self, step, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True):
        T, d = residual.shape
        E, top, ff = self.n_experts, self.top, self.ff
        P = T * top
        ws = step.ws
        z = ws.buf("moe_logits", (T, E), torch.float32)
        kernels.gemm_generic(h, self.router, z)
        ids = ws.buf("moe_ids", (T, top), torch.int32)
        weights = ws.buf("moe_weights", (T, top), torch.float32)
        kernels.moe_route(z, self.correction, top, self.groups, self.keep_groups, self.group_best, ids, weights,
                          softmax_scores=self.softmax, renormalize=self.renormalize)
        max_tiles = kernels.moe_max_tiles(P, E)
        offs = ws.buf("moe_offs", (E + 1,), torch.int32)
        order = ws.buf("moe_order", (P,), torch.int32)
        tile_expert = ws.buf("moe_tile_expert", (max_tiles,), torch.int32)
        tile_row = ws.buf("moe_tile_row", (max_tiles,), torch.int32)
        n_tiles = ws.buf("moe_n_tiles", (1,), torch.int32)
        kernels.moe_group(ids.view(-1), E, offs, order, tile_expert, tile_row, n_tiles)
        groups = (offs, order, tile_expert, tile_row, n_tiles)
        act = ws.buf("moe_act", (P, ff), self.dtype)
        kernels.moe_grouped(h, self.gate_up, act, True, P, top, *groups)
        y = ws.buf("moe_y", (P, d), torch.float32)
        kernels.moe_grouped(act, self.down, y, False, P, top, *groups)
        kernels.moe_combine(y, weights, residual, accumulate)
        return None


register_feed_forward("moe", MixtureOfExperts)
