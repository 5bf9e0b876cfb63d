"""A plain, slow implementation of the Tumatar decoder for the tests to compare against.

Whole sequences, no cache, no batching, one function per mechanism, PyTorch on
the CPU in float32.  It shares no code with ``ziglm_b200``: it reads the raw
config.json dictionary and the tensors under the names they have in the weight
file.

The design in short.  A stack of layers, each ``x += post1(mixer(pre1(x)))`` and,
if the layer has a feed-forward, ``x += post2(ff(pre2(x)))`` with four RMS
norms; a run of consecutive layers may be passed through several times with the
same weights, each pass with a learned vector added to x before its first layer.
Two mixers: attention through a low-rank latent without positions and with a
sigmoid output gate, and a gated linear recurrence behind a short causal
convolution.  Two feed-forwards: a dense one with clamped gate/up and a
mixture of experts whose router scores are sigmoids, chosen within the best
groups of experts.  The head is the embedding table.

``act`` is the type activations are rounded to where the engine stores them in
that type (None: nothing is rounded).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

GATE_SLOPE = 1.702          # the dense feed-forward's gate is g * sigmoid(GATE_SLOPE * g)
DECAY_RATE = 8.0            # log a = -DECAY_RATE * r * softplus(lam)


def _round(t: torch.Tensor, act: Optional[torch.dtype]) -> torch.Tensor:
    return t if act is None else t.to(act).to(torch.float32)


def _f(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32)


# ------------------------------------------------------------------ small parts
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * w, row by row."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * _f(weight)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x @ _f(weight).t()
    return y if bias is None else y + _f(bias)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------- latent attention
def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                     act: Optional[torch.dtype] = None) -> torch.Tensor:
    """Queries and keys/values both come through a normed low-rank latent; only the key/value latent would
    have to be kept.  No positions enter.  score_ij = q_i . k_j * scale for j <= i, softmax, heads gated by
    sigmoid(W_g h), then W_o."""
    T = h.shape[0]
    H, dq, dv = m["heads"], m["dim"], m["vdim"]
    cq = _round(rms_norm(linear(h, w[p + "dq"]), w[p + "dq.norm"], eps), act)
    q = _round(linear(cq, w[p + "uq"]), act).view(T, H, dq)
    c = _round(rms_norm(linear(h, w[p + "dkv"]), w[p + "dkv.norm"], eps), act)
    k = _round(linear(c, w[p + "uk"]), act).view(T, H, dq)
    v = _round(linear(c, w[p + "uv"]), act).view(T, H, dv)
    out = torch.zeros(T, H, dv)
    for i in range(T):
        for a in range(H):
            s = (k[: i + 1, a] @ q[i, a]) * float(m["scale"])
            pr = torch.softmax(s, dim=0)
            out[i, a] = pr @ v[: i + 1, a]
    out = _round(out, act).reshape(T, H * dv)
    gate = torch.sigmoid(linear(h, w[p + "g"]))
    return linear(_round(out * gate, act), w[p + "o"])


# ----------------------------------------------------------- gated recurrence
def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """u_t[c] = b[c] + sum_j taps[c, K-1-j] x_{t-j}[c]; the last column multiplies the current token; zeros
    before the start."""
    T, C = x.shape
    K = taps.shape[1]
    kf = _f(taps)
    out = torch.zeros(T, C)
    for t in range(T):
        acc = _f(bias).clone()
        for j in range(K):
            if t - j >= 0:
                acc = acc + kf[:, K - 1 - j] * x[t - j]
        out[t] = acc
    return out


def block_gate(u: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """sigmoid of a block-diagonal product: part b of u (equal parts) goes through the square matrix weight[b]."""
    B, n, _ = weight.shape
    T = u.shape[0]
    parts = u.view(T, B, n)
    z = torch.stack([parts[:, b] @ _f(weight[b]).t() + _f(bias[b]) for b in range(B)], dim=1)
    return torch.sigmoid(z).reshape(T, B * n)


def rglru(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, act: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = gelu(W_y h + b); u = conv(W_x h + b); r, i = block gates of u; a = exp(-c r softplus(lam));
    S_t = a S_{t-1} + sqrt(1 - a^2) i u from S = 0; out = W_o (S y)."""
    y = _round(gelu_tanh(linear(h, w[p + "y"], w[p + "y.b"])), act)
    xb = _round(linear(h, w[p + "x"], w[p + "x.b"]), act)
    u = _round(causal_conv(xb, w[p + "conv"], w[p + "conv.b"]), act)
    r = block_gate(u, w[p + "ra"], w[p + "ra.b"])
    i = block_gate(u, w[p + "ri"], w[p + "ri.b"])
    log_a = -DECAY_RATE * r * torch.nn.functional.softplus(_f(w[p + "lam"]))
    a = torch.exp(log_a)
    b = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(u.shape[1])
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        S = a[t] * S + b[t]
        out[t] = S
    return linear(_round(out * y, act), w[p + "o"])


# -------------------------------------------------------------- feed-forwards
def clamped_glu(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, limit: float,
                act: Optional[torch.dtype] = None) -> torch.Tensor:
    """g = min(W_g h, L); u = clamp(W_u h, -L, L); out = W_d (g sigmoid(GATE_SLOPE g) (u + 1))."""
    g = torch.clamp(_round(linear(h, w[p + "gate"]), act), max=limit)
    u = torch.clamp(_round(linear(h, w[p + "up"]), act), min=-limit, max=limit)
    y = g * torch.sigmoid(GATE_SLOPE * g) * (u + 1.0)
    return linear(_round(y, act), w[p + "down"])


def route(z: torch.Tensor, correction: torch.Tensor, top: int, n_groups: int, keep: int):
    """For one token: router logits z [E] -> (chosen experts, their weights).  s = sigmoid(z); experts are
    chosen by s + correction, within the ``keep`` groups (of E / n_groups neighbours) whose two best choice
    scores sum highest; the weights are s itself, not renormalised."""
    E = z.numel()
    s = torch.sigmoid(z)
    choice = s + _f(correction)
    size = E // n_groups
    group_score = []
    for g in range(n_groups):
        part = sorted(choice[g * size:(g + 1) * size].tolist(), reverse=True)
        group_score.append(sum(part[:2]))
    best = sorted(range(n_groups), key=lambda g: (-group_score[g], g))[:keep]
    allowed = [e for e in range(E) if e // size in best]
    chosen = sorted(allowed, key=lambda e: (-float(choice[e]), e))[:top]
    return chosen, [float(s[e]) for e in chosen]


def expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, act: Optional[torch.dtype] = None) -> torch.Tensor:
    g = _round(linear(h, w[p + "gate"]), act)
    u = _round(linear(h, w[p + "up"]), act)
    return linear(_round(g * torch.sigmoid(g) * u, act), w[p + "down"])


def moe(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict, act: Optional[torch.dtype] = None) -> torch.Tensor:
    r = mlp["router"]
    z = linear(h, w[p + "router"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0])
    for t in range(h.shape[0]):
        chosen, weights = route(z[t], w[p + "correction"], r["top"], r["groups"]["count"], r["groups"]["keep"])
        for e, g in zip(chosen, weights):
            out[t] += g * expert(h[t:t + 1], w, f"{p}e{e}.", act)[0]
    return out


# ---------------------------------------------------------------------- model
def running_order(cfg: dict):
    """(layer index, pass number or None) in the order the layers run; the pass number is given at the first
    layer of each pass of the repeated run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    lo, hi, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(lo)]
    for t in range(times):
        order += [(i, t if i == lo else None) for i in range(lo, hi)]
    order += [(i, None) for i in range(hi, n)]
    return order


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], act: Optional[torch.dtype] = None,
            layers_out: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``layers_out`` collects the residual stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = _f(w["embed"])[list(tokens)] * float(cfg["embedding"]["scale"])
    for li, pass_no in running_order(cfg):
        layer = cfg["layers"][li]
        p = f"l{li}."
        if pass_no is not None:
            x = x + _f(w["loop.step"][pass_no])
        h = _round(rms_norm(x, w[p + "norm1"], eps), act)
        if layer["type"] == "latent_attention":
            m = latent_attention(h, w, p + "mix.", layer["mixer"], eps, act)
        elif layer["type"] == "rglru":
            m = rglru(h, w, p + "mix.", layer["mixer"], act)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(m, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = _round(rms_norm(x, w[p + "norm2"], eps), act)
            if mlp["kind"] == "dense":
                f = clamped_glu(h, w, p + "mlp.", float(mlp["limit"]), act)
            elif mlp["kind"] == "moe":
                f = moe(h, w, p + "mlp.", mlp, act)
            else:
                raise ValueError(mlp["kind"])
            x = x + rms_norm(f, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = _round(rms_norm(x, w["final.norm"], eps), act)
    return linear(h, w["embed"]) * float(cfg["logit_scale"])
