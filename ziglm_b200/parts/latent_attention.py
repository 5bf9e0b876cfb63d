"""Attention through a low-rank latent, without positions, with a sigmoid gate on the heads' outputs.

For the normed input h of a layer with H heads of query/key size D, value size V and latent sizes Rq, R:
    c_q = norm(W_dq h)            q  = W_uq c_q                       [H, D]
    c   = norm(W_dkv h)           k_j = W_uk c_j,  v_j = W_uv c_j      [H, D], [H, V]   (j: a position)
    s_ij = (q_i . k_j) * scale, j <= i; p = softmax_j(s);  o_i = sum_j p_ij v_j
    out = W_o (o * sigmoid(W_g h))
Only the latent c is kept per position: one vector of R elements that is key and value at once
(``KVNeed(values_are_keys=True)``).  The products with W_uk and W_uv are moved to the other side of the
attention, head by head:
    q'_i = W_uk[h]^T q_i  (an R-vector per head),   s_ij = (q'_i . c_j) * scale,
    l_i  = sum_j p_ij c_j (an R-vector per head),   o_i  = W_uv[h] l_i,
so the attention itself is the library's attention of H query heads over one key/value head of size R
whose keys and values are the same pages, and the two per-head products are block-diagonal products.
The three projections of h (W_dq, W_dkv, W_g) are one matrix product with a float32 result: the norms of the
two latents and the gate's sigmoid read it in float32.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import MixerSpec, NormSpec
from .base import KVNeed, LayerIO, ParamDecl, Part, StateNeed, norm_class, register_mixer
from .linear import Linear


class LatentAttention(Part):
    can_overwrite = True

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        o = spec.options
        self.n_heads, self.dim = spec.n_heads, spec.head_dim
        self.value_dim, self.q_rank, self.kv_rank = int(o["value_dim"]), int(o["q_rank"]), int(o["kv_rank"])
        if spec.scale is None:
            raise ValueError("latent_attention: the spec must give the factor on the scores")
        self.scale = float(spec.scale)
        if o.get("gate", "sigmoid") != "sigmoid":
            raise ValueError(f"latent_attention: output gate {o.get('gate')!r} is not known (sigmoid)")
        # the attention kernels take head sizes that are multiples of 8: a latent of another size is kept with
        # zeros behind it (they add nothing to a score and their part of the result is not read)
        self.kept = -(-self.kv_rank // 8) * 8
        if self.kept > 512:
            raise ValueError(f"latent_attention: a key/value latent of {self.kv_rank} elements is not supported (at most 512)")
        eps = float(o["norm_eps"])
        norm_kind = o.get("norm", "rmsnorm")
        self.q_norm = norm_class(norm_kind)(NormSpec(norm_kind, self.q_rank, eps), dtype, device)
        self.kv_norm = norm_class(norm_kind)(NormSpec(norm_kind, self.kv_rank, eps), dtype, device)
        self.down: Optional[Linear] = None       # [W_dq; W_dkv; W_g]
        self.uq: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.uk_t: Optional[torch.Tensor] = None  # [H, R, D]: W_uk of each head, transposed
        self.uv: Optional[torch.Tensor] = None    # [H, V, R]

    @classmethod
    def declare(cls, spec: MixerSpec) -> Dict[str, ParamDecl]:
        o = spec.options
        H, D, V, Rq, R, d = spec.n_heads, spec.head_dim, int(o["value_dim"]), int(o["q_rank"]), int(o["kv_rank"]), spec.width
        return {"dq.weight": ParamDecl((Rq, d)), "dq_norm.weight": ParamDecl((Rq,), init="ones"),
                "uq.weight": ParamDecl((H * D, Rq)),
                "dkv.weight": ParamDecl((R, d)), "dkv_norm.weight": ParamDecl((R,), init="ones"),
                "uk.weight": ParamDecl((H * D, R)), "uv.weight": ParamDecl((H * V, R)),
                "g.weight": ParamDecl((H * V, d)), "o.weight": ParamDecl((d, H * V))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        H, D, V, R = self.n_heads, self.dim, self.value_dim, self.kv_rank
        ws = [tensors["dq.weight"], tensors["dkv.weight"], tensors["g.weight"]]
        wide = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.down = Linear(torch.cat([w.to(wide) for w in ws], dim=0))
        self.uq = Linear(tensors["uq.weight"])
        self.o = Linear(tensors["o.weight"])
        self.q_norm.bind({"weight": tensors["dq_norm.weight"]})
        self.kv_norm.bind({"weight": tensors["dkv_norm.weight"]})
        uk_t = tensors["uk.weight"].view(H, D, R).transpose(1, 2)
        uv = tensors["uv.weight"].view(H, V, R)
        if self.kept != R:
            pad = self.kept - R
            uk_t = torch.cat([uk_t, uk_t.new_zeros(H, pad, D)], dim=1)
            uv = torch.cat([uv, uv.new_zeros(H, V, pad)], dim=2)
        self.uk_t = uk_t.contiguous()
        self.uv = uv.contiguous()

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs = ("elementwise", "block_linear", "attention")
        libs += kernels.fast_attention_libraries(self.dtype, self.kept, min(self.n_heads, self.HEADS_AT_ONCE), 1)
        for lin in (self.down, self.uq, self.o):
            if lin is not None:
                libs += lin.libraries(self.dtype)
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        return KVNeed(1, self.kept, None, values_are_keys=True)

    def state_needs(self) -> Optional[StateNeed]:
        return None

    def forward(self, step, io: LayerIO, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True):
        T = residual.shape[0]
        H, D, V, Rq, Rn, R = self.n_heads, self.dim, self.value_dim, self.q_rank, self.kv_rank, self.kept
        proj = step.ws.buf("lat_proj", (T, Rq + Rn + H * V), torch.float32)
        self.down(h, proj)
        cq = step.ws.buf("lat_cq", (T, Rq), self.dtype)
        self.q_norm.forward_rows(proj[:, :Rq], cq)
        # a row of ``qc``: the H queries in the latent's space, then the token's latent (the one key/value head)
        qc = step.ws.buf("lat_qc", (T, (H + 1) * R), self.dtype)
        self.kv_norm.forward_rows(proj[:, Rq:Rq + Rn], qc[:, H * R:H * R + Rn])
        if R != Rn:
            qc[:, H * R + Rn:].zero_()
        q = step.ws.buf("lat_q", (T, H * D), self.dtype)
        self.uq(cq, q)
        kernels.block_linear(q, self.uk_t, qc[:, :H * R])
        kernels.rope_store(qc, H, 1, R, 0, None, step.positions, step.seq_of_token, io.block_table, io.k_pages, None,
                           io.page_size, keys_only=True)
        heads = step.ws.buf("lat_heads", (T, H * V), self.dtype)
        gate = proj[:, Rq + Rn:]
        # all heads read the one key/value head; the tensor-core kernels take up to 16 query heads a key/value head,
        # so more heads go through them 16 at a time (the queries are a column slice of the rows, the latent pages
        # are the same)
        n = self.HEADS_AT_ONCE if (H > self.HEADS_AT_ONCE and kernels.fast_attention_libraries(
            self.dtype, R, self.HEADS_AT_ONCE, 1)) else H
        for h0 in range(0, H, n):
            h1 = min(H, h0 + n)
            mixed = step.ws.buf("lat_mixed", (T, (h1 - h0) * R), self.dtype)
            kernels.attention(step, qc[:, h0 * R:h1 * R], mixed, h1 - h0, 1, R, self.scale, None, io)
            kernels.block_linear(mixed, self.uv[h0:h1], heads[:, h0 * V:h1 * V], epilogue="sigmoid_gate",
                                 gate=gate[:, h0 * V:h1 * V])
        self.o(heads, residual, accumulate=accumulate)
        return None

    HEADS_AT_ONCE = 16


register_mixer("latent_attention", LatentAttention)
