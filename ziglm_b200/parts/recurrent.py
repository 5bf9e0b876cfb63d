"""A recurrent mixer: a real-gated linear recurrence behind a short causal convolution, beside a gelu branch.

For the normed input h, with C channels in B equal blocks and a convolution of K taps:
    y_t = gelu_tanh(W_y h_t + b_y)                x_t = W_x h_t + b_x
    u_t = conv(x)_t                               (per channel, K taps, zeros before the start, no activation)
    r_t = sigmoid(A_b u_t[b] + a_b)               i_t = sigmoid(I_b u_t[b] + i_b)      (block b of the channels)
    a_t = exp(-rate * r_t * softplus(lam))        S_t = a_t S_{t-1} + sqrt(1 - a_t^2) i_t u_t,  S = 0 at the start
    out = W_o (S_t * y_t)
A sequence carries [K, C] float32 from step to step (``StateNeed``): its last K-1 inputs x and S.  The two
branches are one matrix product; the two gate matrices of a block are one block-diagonal product whose float32
result goes through the sigmoid in its epilogue; gates, decay and state are float32 in both precisions.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import MixerSpec
from .base import KVNeed, LayerIO, ParamDecl, Part, StateNeed, register_mixer
from .linear import Linear


class GatedLinearRecurrence(Part):
    can_overwrite = True

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        o = spec.options
        self.channels, self.blocks, self.taps = int(o["channels"]), int(o["blocks"]), int(o["taps"])
        self.rate = float(o["decay_rate"])
        if self.channels % self.blocks:
            raise ValueError(f"rglru: {self.channels} channels cannot form {self.blocks} equal blocks")
        self.in_proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.conv_w = self.conv_b = self.gate_w = self.gate_b = self.lam = None

    @classmethod
    def declare(cls, spec: MixerSpec) -> Dict[str, ParamDecl]:
        o = spec.options
        C, B, K, d = int(o["channels"]), int(o["blocks"]), int(o["taps"]), spec.width
        n = C // B
        return {"y.weight": ParamDecl((C, d)), "y.bias": ParamDecl((C,)), "x.weight": ParamDecl((C, d)),
                "x.bias": ParamDecl((C,)), "conv.weight": ParamDecl((C, K)), "conv.bias": ParamDecl((C,)),
                "ra.weight": ParamDecl((B, n, n)), "ra.bias": ParamDecl((B, n)), "ri.weight": ParamDecl((B, n, n)),
                "ri.bias": ParamDecl((B, n)), "lam": ParamDecl((C,)), "o.weight": ParamDecl((d, C))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        ws = [tensors["y.weight"], tensors["x.weight"]]
        wide = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        bs = [tensors["y.bias"], tensors["x.bias"]]
        bwide = torch.float32 if any(b.dtype == torch.float32 for b in bs) else bs[0].dtype
        self.in_proj = Linear(torch.cat([w.to(wide) for w in ws], dim=0), torch.cat([b.to(bwide) for b in bs], dim=0))
        self.o = Linear(tensors["o.weight"])
        self.conv_w = tensors["conv.weight"].float().t().contiguous()          # [taps, channels]: a row per tap
        self.conv_b = tensors["conv.bias"].float().contiguous()
        gw = [tensors["ra.weight"], tensors["ri.weight"]]
        gwide = torch.float32 if any(w.dtype == torch.float32 for w in gw) else gw[0].dtype
        self.gate_w = torch.cat([w.to(gwide) for w in gw], dim=1).contiguous()           # [B, 2n, n]
        self.gate_b = torch.cat([tensors["ra.bias"].float(), tensors["ri.bias"].float()], dim=1).reshape(-1).contiguous()
        self.lam = tensors["lam"].float().contiguous()

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs = ("recurrent", "block_linear")
        for lin in (self.in_proj, self.o):
            if lin is not None:
                libs += lin.libraries(self.dtype)
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        return None

    def state_needs(self) -> Optional[StateNeed]:
        return StateNeed((self.taps, self.channels), torch.float32)

    def forward(self, step, io: LayerIO, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True):
        T, C = residual.shape[0], self.channels
        proj = step.ws.buf("rec_proj", (T, 2 * C), self.dtype)
        self.in_proj(h, proj)
        y, x = proj[:, :C], proj[:, C:]
        u = step.ws.buf("rec_u", (T, C), self.dtype)
        kernels.causal_conv(x, self.conv_w, self.conv_b, io.state, step, u)
        gates = step.ws.buf("rec_gates", (T, 2 * C), torch.float32)
        kernels.block_linear(u, self.gate_w, gates, bias=self.gate_b, epilogue="sigmoid")
        out = step.ws.buf("rec_out", (T, C), self.dtype)
        kernels.gated_scan(u, gates, C // self.blocks, y, x, self.lam, self.rate, io.state, step, out)
        self.o(out, residual, accumulate=accumulate)
        return None


register_mixer("rglru", GatedLinearRecurrence)
