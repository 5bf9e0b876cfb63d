"""Grouped-query attention with the options of newer decoders, each of which may be left out.

For the rows h the mixer reads, H query heads, G key/value heads, query/key size D and value size V:
    q = W_q h + b_q,  k = W_k h + b_k,  v = W_v h + b_v
    q, k <- rotate(q, k; position)              the first ``rotary_dim`` dimensions of a head, pairs (i, i + R/2);
                                                cosines and sines times the encoding's amplitude
    q, k <- q / rms(q), k / rms(k)              per head over D, no weight        (``qk_norm_eps``; None: left out)
    s_ij = (q_i . k_j) * scale;  s <- c tanh(s / c)                               (``softcap`` c; None: left out)
    p = softmax over j <= i;  o_i = sum_j p_ij v_j
    out = W_o (concat(o) * sigmoid(W_g h))                                       (``gate`` "sigmoid"; None: left out)
``value_dim`` V may differ from ``head_dim`` D.  The four projections of h are one matrix product over the
concatenated weight [q; k; v; g].

Keys and values share the cache's head size: both are kept with max(D, V) elements a head (rounded up to a
multiple of 8), the shorter of the two with zeros behind it, which add nothing to a score and whose part of the
result is zero.  The padding is built into the weights when they are bound (zero rows of W_k or W_v, zero columns
of W_o), so every kernel sees one head size; the unit norm divides by the true D.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import MixerSpec
from .base import KVNeed, LayerIO, ParamDecl, Part, StateNeed, position_class, register_mixer
from .linear import Linear


def _pad_heads(w: torch.Tensor, heads: int, size: int, padded: int) -> torch.Tensor:
    """[heads * size, ...] -> [heads * padded, ...] with zero rows behind every head."""
    if size == padded:
        return w
    rest = tuple(w.shape[1:])
    out = w.new_zeros((heads, padded) + rest)
    out[:, :size] = w.reshape((heads, size) + rest)
    return out.reshape((heads * padded,) + rest)


class CappedAttention(Part):
    can_overwrite = True

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        o = spec.options
        if spec.n_heads <= 0 or spec.n_kv_heads <= 0 or spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"attention: {spec.n_heads} heads cannot share {spec.n_kv_heads} key/value heads")
        if spec.scale is None:
            raise ValueError("capped_attention: the spec must give the factor on the scores")
        if spec.window is not None or spec.cache_from is not None:
            raise ValueError("capped_attention: windows and shared caches are not part of this mixer")
        self.n_heads, self.n_kv, self.dim = spec.n_heads, spec.n_kv_heads, spec.head_dim
        self.value_dim = int(o.get("value_dim", spec.head_dim))
        self.scale = float(spec.scale)
        self.softcap = float(o["softcap"]) if o.get("softcap") else 0.0
        self.norm_eps = None if o.get("qk_norm_eps") is None else float(o["qk_norm_eps"])
        if o.get("gate") not in (None, "sigmoid"):
            raise ValueError(f"capped_attention: output gate {o.get('gate')!r} is not known (sigmoid)")
        self.gated = o.get("gate") == "sigmoid"
        self.kept = self.kept_head_size(self.dim, self.value_dim, dtype)
        if self.kept > 512:
            raise ValueError(f"capped_attention: heads of {max(self.dim, self.value_dim)} elements are not supported (at most 512)")
        self.position = position_class(spec.position.kind)(spec.position, dtype, device)
        self.proj: Optional[Linear] = None      # [q; k; v; g] with every head padded to ``kept``
        self.o: Optional[Linear] = None

    @staticmethod
    def kept_head_size(dim: int, value_dim: int, dtype: torch.dtype) -> int:
        """The one head size keys, values and queries are held with: the larger of the two, as a multiple of 8; in
        bfloat16 the next size the tensor-core attention kernels take (64, 128) when that is at most a quarter more."""
        kept = -(-max(dim, value_dim) // 8) * 8
        if dtype == torch.bfloat16:
            for fast in (64, 128):
                if kept <= fast and fast * 4 <= kept * 5:
                    return fast
        return kept

    @classmethod
    def declare(cls, spec: MixerSpec) -> Dict[str, ParamDecl]:
        H, G, D, d = spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.width
        V = int(spec.options.get("value_dim", D))
        p = {"q.weight": ParamDecl((H * D, d)), "k.weight": ParamDecl((G * D, d)), "v.weight": ParamDecl((G * V, d)),
             "o.weight": ParamDecl((d, H * V))}
        if spec.bias:
            p.update({"q.bias": ParamDecl((H * D,)), "k.bias": ParamDecl((G * D,)), "v.bias": ParamDecl((G * V,))})
        if spec.options.get("gate") == "sigmoid":
            p["g.weight"] = ParamDecl((H * V, d))
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        H, G, D, V, P = self.n_heads, self.n_kv, self.dim, self.value_dim, self.kept
        parts = [("q", H, D), ("k", G, D), ("v", G, V)] + ([("g", H, V)] if self.gated else [])
        ws = [tensors[f"{n}.weight"] for n, _, _ in parts]
        wide = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        weight = torch.cat([_pad_heads(w.to(wide), heads, size, P) for w, (_, heads, size) in zip(ws, parts)], dim=0)
        bias = None
        if self.spec.bias:
            bs = []
            for n, heads, size in parts:
                b = tensors.get(f"{n}.bias")
                b = b if b is not None else ws[0].new_zeros(heads * size)
                bs.append(_pad_heads(b.to(torch.float32), heads, size, P))
            bias = torch.cat(bs, dim=0)
        self.proj = Linear(weight, bias)
        w_o = tensors["o.weight"]
        if V != P:
            w_o = _pad_heads(w_o.t().contiguous(), H, V, P).t().contiguous()
        self.o = Linear(w_o)

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs = ("attention", "elementwise")
        libs += kernels.fast_attention_libraries(self.dtype, self.kept, self.n_heads, self.n_kv, softcap=self.softcap)
        for lin in (self.proj, self.o):
            if lin is not None:
                libs += lin.libraries(self.dtype)
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        return KVNeed(self.n_kv, self.kept, None)

    def state_needs(self) -> Optional[StateNeed]:
        return None

    def forward(self, step, io: LayerIO, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True):
        T = residual.shape[0]
        H, G, P = self.n_heads, self.n_kv, self.kept
        width = (H + 2 * G + (H if self.gated else 0)) * P
        proj = step.ws.buf("cattn_proj", (T, width), self.dtype)
        self.proj(h, proj)
        table = self.position.rotary_table()
        inv_freq, rot = table if table is not None else (None, 0)
        amplitude = float(getattr(self.position, "amplitude", 1.0))
        kernels.rope_norm_store(proj, H, G, P, rot, inv_freq, amplitude, self.dim if self.norm_eps is not None else 0,
                                self.norm_eps or 0.0, step.positions, step.seq_of_token, io.block_table,
                                io.k_pages if io.writes_cache else None, io.v_pages if io.writes_cache else None,
                                io.page_size)
        out = step.ws.buf("attn_out", (T, H * P), self.dtype)
        gate = proj[:, (H + 2 * G) * P:] if self.gated else None
        # the flat decode kernel multiplies by the gate's sigmoid as it stores; behind the others a kernel does
        if not kernels.attention(step, proj, out, H, G, P, self.scale, None, io, softcap=self.softcap, gate=gate) and self.gated:
            kernels.sigmoid_mul(out, gate, out)
        self.o(out, residual, accumulate=accumulate)
        return None


register_mixer("capped_attention", CappedAttention)
