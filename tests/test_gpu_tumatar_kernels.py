"""Each mechanism of the Tumatar design alone: the kernel (or the part) against the plain function that states
its formula (tests/plain_tumatar.py), at sizes that are no multiple of a tile, with strided rows, several
sequences in a step, state carried over steps, and inputs made so that a fault shows."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_tumatar as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _r(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _step(new_lens, slots):
    cu = [0]
    seq = []
    for b, n in enumerate(new_lens):
        cu.append(cu[-1] + n)
        seq += [b] * n
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(seq_of_token=i32(seq), cu_seqlens=i32(cu), slots=i32(slots), n_seqs=len(new_lens),
                           max_new=max(new_lens), n_tokens=cu[-1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,B,N,K", [(1, 3, 16, 24), (37, 5, 70, 33), (130, 2, 64, 128)])
def test_block_diagonal_product(dtype, T, B, N, K):
    from ziglm_b200 import kernels
    wide = _r(T, B * K + 8, seed=1, dtype=dtype)
    x = wide[:, 8:]                                   # rows with a stride of their own
    w = _r(B, N, K, seed=2, scale=0.2, dtype=dtype)
    bias = _r(B * N, seed=3)
    gate = _r(T, B * N + 4, seed=4)[:, 4:]
    ref = torch.einsum("tbk,bnk->tbn", x.float().view(T, B, K), w.float()).reshape(T, B * N)
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    out = torch.empty(T, B * N + 16, dtype=dtype, device=DEV)[:, 16:]
    kernels.block_linear(x, w, out)
    torch.testing.assert_close(out.float(), ref, **tol)
    out32 = torch.empty(T, B * N, dtype=torch.float32, device=DEV)
    if dtype == torch.bfloat16 or True:
        kernels.block_linear(x, w, out32, bias=bias, epilogue="sigmoid")
        torch.testing.assert_close(out32, torch.sigmoid(ref + bias), atol=2e-5 if dtype == torch.float32 else 2e-3, rtol=1e-3)
    kernels.block_linear(x, w, out, epilogue="sigmoid_gate", gate=gate)
    torch.testing.assert_close(out.float(), ref.to(dtype).float() * torch.sigmoid(gate), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,K,blocks", [(40, 4, 5), (96, 1, 1), (64, 3, 2)])
def test_convolution_and_recurrence_over_steps(dtype, C, K, blocks):
    """Three sequences of unequal lengths in slots 3, 0, 2, each run in portions (one of them token by token);
    the state carries the convolution's inputs and S over the steps.  Decays close to 1: S remembers."""
    from ziglm_b200 import kernels
    lens = [50, 7, 33]
    slots = [3, 0, 2]
    n = C // blocks
    taps, cb = _r(C, K, seed=1, scale=0.5), _r(C, seed=2, scale=0.1)
    gw = _r(blocks, 2 * n, n, seed=3, scale=0.3, dtype=dtype)
    ra, ri = gw[:, :n].contiguous(), gw[:, n:].contiguous()
    gb = _r(blocks, 2 * n, seed=4, scale=0.2)
    lam = _r(C, seed=5) - 4.0
    xs = [_r(L, C, seed=10 + i, dtype=dtype) for i, L in enumerate(lens)]
    ys = [_r(L, C, seed=20 + i, dtype=dtype) for i, L in enumerate(lens)]
    want = []
    rnd = (lambda t: t.to(dtype).float())
    for x, y in zip(xs, ys):
        u = rnd(P.causal_conv(x.float().cpu(), taps.cpu(), cb.cpu()))
        r = P.block_gate(u, ra.cpu(), gb[:, :n].cpu())
        i = P.block_gate(u, ri.cpu(), gb[:, n:].cpu())
        a = torch.exp(-8.0 * r * torch.nn.functional.softplus(lam.cpu()))
        S, rows = torch.zeros(C), []
        for t in range(x.shape[0]):
            S = a[t] * S + torch.sqrt(1 - a[t] ** 2) * i[t] * u[t]
            rows.append(S * P.gelu_tanh(y[t].float().cpu()))
        want.append(torch.stack(rows))
    state = _r(4, K, C, seed=6)                       # whatever the slots' last users left
    for s in slots:
        state[s].zero_()
    portions = [[20, 1, 29], [1] * 7, [2, 30, 1]]
    got = [[] for _ in lens]
    used = [0, 0, 0]
    for step_no in range(max(len(p) for p in portions)):
        live = [b for b in range(3) if step_no < len(portions[b])]
        new = [portions[b][step_no] for b in live]
        st = _step(new, [slots[b] for b in live])
        x = torch.cat([xs[b][used[b]:used[b] + n_] for b, n_ in zip(live, new)])
        y = torch.cat([ys[b][used[b]:used[b] + n_] for b, n_ in zip(live, new)])
        proj = torch.cat([y, x], dim=1).contiguous()  # as the part lays them out: [y | x]
        u = torch.empty(st.n_tokens, C, dtype=dtype, device=DEV)
        kernels.causal_conv(proj[:, C:], taps.t().contiguous(), cb, state, st, u)
        gates = torch.empty(st.n_tokens, 2 * C, dtype=torch.float32, device=DEV)
        kernels.block_linear(u, gw, gates, bias=gb.reshape(-1).contiguous(), epilogue="sigmoid")
        out = torch.empty_like(u)
        kernels.gated_scan(u, gates, n, proj[:, :C], proj[:, C:], lam, 8.0, state, st, out)
        at = 0
        for b, n_ in zip(live, new):
            got[b].append(out[at:at + n_].float().cpu())
            at += n_
            used[b] += n_
    tol = dict(atol=2e-5, rtol=2e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    for b in range(3):
        torch.testing.assert_close(torch.cat(got[b]), want[b], **tol)
    assert state[1].abs().sum().item() > 0 and (state[1] == _r(4, K, C, seed=6)[1]).all()     # a slot of no sequence is untouched


def test_long_scan_in_chunks_equals_token_by_token():
    """A step of 700 tokens is cut into chunks whose maps are composed; the same tokens one by one give the same."""
    from ziglm_b200 import kernels
    C, K, L = 48, 2, 700
    taps, cb, lam = _r(C, K, seed=1), _r(C, seed=2), _r(C, seed=3) - 5.0
    gw, gb = _r(1, 2 * C, C, seed=4, scale=0.1), _r(2 * C, seed=5)
    proj = _r(L, 2 * C, seed=6)
    outs = []
    for cuts in ([L], [1] * L):
        state = torch.zeros(1, K, C, device=DEV)
        rows, at = [], 0
        for n in cuts:
            st = _step([n], [0])
            pr = proj[at:at + n].contiguous()
            u = torch.empty(n, C, device=DEV)
            kernels.causal_conv(pr[:, C:], taps.t().contiguous(), cb, state, st, u)
            gates = torch.empty(n, 2 * C, device=DEV)
            kernels.block_linear(u, gw, gates, bias=gb, epilogue="sigmoid")
            out = torch.empty_like(u)
            kernels.gated_scan(u, gates, C, pr[:, :C], pr[:, C:], lam, 8.0, state, st, out)
            rows.append(out.clone())
            at += n
        outs.append(torch.cat(rows))
    torch.testing.assert_close(outs[0], outs[1], atol=2e-5, rtol=2e-4)


@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 4, 2), (15, 3, 3, 1), (6, 1, 1, 1), (64, 6, 8, 3), (5, 5, 1, 1)])
def test_router(E, top, groups, keep):
    from ziglm_b200 import kernels
    T = 50
    z = _r(T, E, seed=E, scale=2.0)
    corr = _r(E, seed=1, scale=0.3) - 2.0             # every choice score is negative
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
    kernels.moe_route(z, corr, top, groups, keep, 2, ids, wts)
    for t in range(T):
        chosen, weights = P.route(z[t].cpu(), corr.cpu(), top, groups, keep)
        assert ids[t].tolist() == chosen, f"token {t}"
        torch.testing.assert_close(wts[t].cpu(), torch.tensor(weights), atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 5, 200])
def test_mixture_of_experts_part(dtype, T):
    """The part as the block calls it, on a hand-made step: every expert gets some tokens, some get none (T = 1)."""
    from ziglm_b200.config.spec import FeedForwardSpec
    from ziglm_b200.engine.workspace import Workspace
    from ziglm_b200.parts import feed_forward_class
    d, ff, E = 72, 40, 6             # T = 1, 5: the streaming kernel; 200: tiles (float32), tensor cores (bfloat16)
    spec = FeedForwardSpec("moe", d, ff, "silu", options={"experts": E, "top": 2, "groups": 3, "keep_groups": 2,
                                                           "group_best": 2, "score": "sigmoid", "correction": True})
    cls = feed_forward_class("moe")
    w = {name: _r(*decl.shape, seed=i, scale=0.2, dtype=dtype) for i, (name, decl) in enumerate(cls.declare(spec).items())}
    part = cls(spec, dtype, torch.device(DEV))
    part.bind(w)
    from ziglm_b200 import kernels
    kernels.require(part.kernel_libraries())
    h = _r(T, d, seed=99, dtype=dtype)
    plain_w = {"m." + k.replace(".weight", ""): v.cpu() for k, v in w.items()}
    mlp = {"router": {"top": 2, "groups": {"count": 3, "keep": 2}}}
    want = P.moe(h.float().cpu(), plain_w, "m.", mlp, act=None if dtype == torch.float32 else dtype)
    step = SimpleNamespace(ws=Workspace(torch.device(DEV)))
    out = torch.full((T, d), 7.0, device=DEV)
    part.forward(step, h, out, accumulate=False)
    # bfloat16: the tensor-core product applies the activation to its float32 sums, the plain one to rounded ones
    tol = dict(atol=1e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=6e-2, rtol=5e-2)
    torch.testing.assert_close(out.cpu(), want, **tol)
    part.forward(step, h, out, accumulate=True)
    torch.testing.assert_close(out.cpu(), 2 * want, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_activation_and_the_norm_that_adds(dtype):
    from ziglm_b200 import kernels
    T, I = 9, 50
    gu = _r(T, 2 * I, seed=1, scale=2.0, dtype=dtype)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    kernels.gated_act(gu, out, "swish_clamped", limit=0.8, slope=1.702)
    g = gu[:, :I].float().clamp(max=0.8)
    u = gu[:, I:].float().clamp(-0.8, 0.8)
    torch.testing.assert_close(out.float(), (g * torch.sigmoid(1.702 * g) * (u + 1)).to(dtype).float(), atol=1e-6, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5)
    x = _r(T, 3 * I, seed=2)
    wt = _r(I, seed=3, dtype=dtype) + 1.0
    res = _r(T, I, seed=4)
    want = res + P.rms_norm(x[:, I:2 * I].cpu(), wt.cpu(), 1e-5).to(DEV)
    kernels.rmsnorm_rows(x[:, I:2 * I], wt, res, 1e-5, add=True)
    torch.testing.assert_close(res, want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,d", [(1, 24), (37, 200), (5, 4096)])
def test_norm_sum_norm_in_one_kernel(dtype, T, d):
    """x += norm1(branch); h = norm2(x) against the two norms taken one after the other."""
    from ziglm_b200 import kernels
    branch, x = _r(T, d, seed=1, scale=3.0), _r(T, d, seed=2)
    w1, w2 = _r(d, seed=3, dtype=dtype) + 1.0, _r(d, seed=4, dtype=dtype) + 1.0
    want_x = x.cpu() + P.rms_norm(branch.cpu(), w1.cpu(), 1e-5)
    want_h = P.rms_norm(want_x, w2.cpu(), 1e-6)
    h = torch.empty(T, d, dtype=dtype, device=DEV)
    assert kernels.norm_add_norm(branch, w1, 1e-5, x, w2, 1e-6, h)
    torch.testing.assert_close(x.cpu(), want_x, atol=1e-5, rtol=1e-5)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(h.float().cpu(), want_h, **tol)
    assert not kernels.norm_add_norm(_r(2, 20000, seed=5), _r(20000, seed=6, dtype=dtype), 1e-5, _r(2, 20000, seed=7),
                                     _r(20000, seed=8, dtype=dtype), 1e-5, torch.empty(2, 20000, dtype=dtype, device=DEV))


@pytest.mark.parametrize("dtype,R,H", [(torch.float32, 320, 2), (torch.float32, 40, 3), (torch.bfloat16, 128, 7),
                                       (torch.bfloat16, 64, 16), (torch.bfloat16, 200, 4)])
def test_attention_over_a_latent_that_is_key_and_value(dtype, R, H):
    """One vector per position is key and value (one set of pages); prompts of two sequences with shuffled pages,
    then a decoded token each.  Latents of 64 and 128 take the tensor-core kernels in bfloat16."""
    from ziglm_b200 import kernels
    from ziglm_b200.engine.workspace import Workspace
    from ziglm_b200.parts.base import LayerIO
    kernels.require(("attention",) + kernels.fast_attention_libraries(dtype, R, H, 1))
    lens, page = [150, 70], 64
    pages = torch.zeros(8, 1, page, R, dtype=dtype, device=DEV)
    table = torch.tensor([[5, 2, 7], [1, 6, -1]], dtype=torch.int32, device=DEV)
    cs = [_r(L + 1, R, seed=i, dtype=dtype) for i, L in enumerate(lens)]
    qs = [_r(L + 1, H * R, seed=7 + i, scale=0.3, dtype=dtype) for i, L in enumerate(lens)]
    scale = 1.0 / math.sqrt(R)

    def plain(q, c):
        out = torch.zeros(q.shape[0], H, R)
        qh, cf = q.float().cpu().view(-1, H, R), c.float().cpu()
        for i in range(q.shape[0]):
            pr = torch.softmax((cf[: i + 1] @ qh[i].t()) * scale, dim=0)       # [i+1, H]
            out[i] = pr.t() @ cf[: i + 1]
        return out.reshape(q.shape[0], H * R)

    want = [plain(q, c) for q, c in zip(qs, cs)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    for decode in (False, True):
        new = [1, 1] if decode else lens
        past = lens if decode else [0, 0]
        qc = torch.cat([torch.cat([q[p:p + n], c[p:p + n]], dim=1) for q, c, p, n in zip(qs, cs, past, new)]).contiguous()
        T = qc.shape[0]
        cu = [0, new[0], new[0] + new[1]]
        step = SimpleNamespace(
            n_tokens=T, n_seqs=2, single_token=decode, max_new=max(new), max_total=max(p + n for p, n in zip(past, new)),
            positions=i32([p + i for p, n in zip(past, new) for i in range(n)]),
            seq_of_token=i32([b for b, n in enumerate(new) for _ in range(n)]), cu_seqlens=i32(cu), past_lens=i32(past),
            total_lens=i32([p + n for p, n in zip(past, new)]), ws=Workspace(torch.device(DEV)))
        io = LayerIO(k_pages=pages, v_pages=pages, block_table=table, page_size=page)
        kernels.rope_store(qc, H, 1, R, 0, None, step.positions, step.seq_of_token, table, pages, None, page, keys_only=True)
        out = torch.empty(T, H * R, dtype=dtype, device=DEV)
        kernels.attention(step, qc, out, H, 1, R, scale, None, io)
        ref = torch.cat([w[p:p + n] for w, p, n in zip(want, past, new)])
        tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(out.float().cpu(), ref, **tol)


@pytest.mark.parametrize("T,I,K", [(3, 40, 64), (70, 136, 96), (300, 256, 128)])
def test_gated_product_with_the_clamped_activation_in_its_epilogue(T, I, K):
    """The tensor-core gated product (rows of the weight alternate gate and up) against the formula."""
    from ziglm_b200 import kernels
    kernels.require(("gemm_tc",))
    x = _r(T, K, seed=1, dtype=torch.bfloat16)
    gate, up = _r(I, K, seed=2, scale=0.3, dtype=torch.bfloat16), _r(I, K, seed=3, scale=0.3, dtype=torch.bfloat16)
    w = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()
    out = torch.empty(T, I, dtype=torch.bfloat16, device=DEV)
    assert kernels.gemm_tc_swish_clamped(x, w, out, 0.9, 1.702)
    g = (x.float() @ gate.float().t()).clamp(max=0.9)
    u = (x.float() @ up.float().t()).clamp(-0.9, 0.9)
    torch.testing.assert_close(out.float(), g * torch.sigmoid(1.702 * g) * (u + 1), atol=2e-2, rtol=2e-2)
