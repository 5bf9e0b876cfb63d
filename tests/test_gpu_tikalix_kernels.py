"""Each mechanism of the Tikalix design alone: the kernel (or the part) against the plain function that states its
formula (tests/plain_tikalix.py), at sizes that are no multiple of a tile, with strided rows, several sequences in
a step, shuffled pages, prompts and decoded tokens, and inputs made so that a fault shows."""
from types import SimpleNamespace

import pytest
import torch

import plain_tikalix as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _r(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _tol(dtype, f32=(1e-5, 1e-5), bf16=(2e-2, 2e-2)):
    a, r = f32 if dtype == torch.float32 else bf16
    return dict(atol=a, rtol=r)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,rot,norm_dim,scaling", [
    (6, 2, 40, 16, 24, (4.0, 64, 8.0, 0.5)),       # heads kept with zeros behind them: the norm divides by 24
    (4, 4, 64, 64, 64, None), (5, 1, 16, 2, 12, (1.5, 32, 4.0, 1.0)), (2, 1, 128, 64, 0, (8.0, 128, 32.0, 1.0)),
])
def test_rotation_unit_norm_and_cache_write(dtype, H, G, hd, rot, norm_dim, scaling):
    """Two sequences (a prompt of 70 after 3 cached tokens, one decoded token at position 130) with shuffled pages;
    rows that are wider than the heads (a gate behind them); norm_dim 0: no norm."""
    from ziglm_b200 import kernels
    kernels.require(("attention",))
    eps, page = 1e-5, 64
    positions = list(range(3, 73)) + [130]
    seq = [0] * 70 + [1]
    T = len(positions)
    width = (H + 2 * G) * hd
    rows = _r(T, width + 24, seed=hd, dtype=dtype)
    x = rows[:, :width].view(T, H + 2 * G, hd)
    if norm_dim and norm_dim < hd:
        x[:, :H + G, norm_dim:] = 0                     # what lies behind the true head is zero, as the weights make it
    before = rows.clone()
    rotd = {"dims": rot, "base": 100.0}
    if scaling:
        rotd["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    freq, amp = P.rotary_frequencies(rotd)
    qk = before[:, :(H + G) * hd].float().cpu().view(T, H + G, hd)
    turned = P.rotate(qk, torch.tensor(positions), rotd)
    if norm_dim:
        turned = turned / torch.sqrt((turned[..., :norm_dim] ** 2).mean(-1, keepdim=True) + eps)
    k_pages = torch.full((5, G, page, hd), 9.0, dtype=dtype, device=DEV)
    v_pages = torch.full((5, G, page, hd), 9.0, dtype=dtype, device=DEV)
    table = _i32([[4, 1, -1], [0, 3, 2]])
    kernels.rope_norm_store(rows, H, G, hd, rot, freq.float().to(DEV), amp, norm_dim, eps, _i32(positions), _i32(seq),
                            table, k_pages, v_pages, page)
    tol = _tol(dtype, (2e-5, 2e-5), (1e-2, 1e-2))
    torch.testing.assert_close(rows[:, :(H + G) * hd].float().cpu().view(T, H + G, hd), turned, **tol)
    assert torch.equal(rows[:, (H + G) * hd:], before[:, (H + G) * hd:])          # values and the rest are left alone
    tb = table.cpu()
    for t, (pos, b) in enumerate(zip(positions, seq)):
        pg = tb[b, pos // page].item()
        torch.testing.assert_close(k_pages[pg, :, pos % page].float().cpu(), turned[t, H:], **tol)
        assert torch.equal(v_pages[pg, :, pos % page], before[t, (H + G) * hd:width].view(G, hd))
    assert (k_pages == 9.0).sum().item() == (5 * page - T) * G * hd               # nothing else was written


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,cap", [(6, 2, 40, 3.0), (4, 1, 64, 20.0), (5, 5, 24, 0.5), (3, 1, 128, None), (8, 2, 128, 5.0),
                                        (2, 2, 64, 1.5)])
def test_attention_with_a_soft_cap(dtype, H, G, hd, cap):
    """Prompts of two sequences (one continued) and then a decoded token each, against the formula; the queries are
    large enough for the cap to bite."""
    from ziglm_b200 import kernels
    from ziglm_b200.engine.workspace import Workspace
    from ziglm_b200.parts.base import LayerIO
    kernels.require(("attention",) + kernels.fast_attention_libraries(dtype, hd, H, G, softcap=cap or 0.0))
    lens, page, scale = [300, 70], 64, 0.7
    ks = [_r(L + 1, G, hd, seed=i, dtype=dtype) for i, L in enumerate(lens)]
    vs = [_r(L + 1, G, hd, seed=3 + i, dtype=dtype) for i, L in enumerate(lens)]
    qs = [_r(L + 1, H, hd, seed=7 + i, scale=0.6, dtype=dtype) for i, L in enumerate(lens)]
    k_pages = torch.zeros(9, G, page, hd, dtype=dtype, device=DEV)
    v_pages = torch.zeros(9, G, page, hd, dtype=dtype, device=DEV)
    table = _i32([[5, 2, 7, 0, 8], [1, 6, -1, -1, -1]])

    def plain(q, k, v):
        out = torch.zeros(q.shape[0], H, hd)
        q, k, v = q.float().cpu(), k.float().cpu(), v.float().cpu()
        for h in range(H):
            g = h // (H // G)
            s = P.soft_cap((q[:, h] @ k[:, g].t()) * scale, cap)
            s = s.masked_fill(torch.triu(torch.ones_like(s, dtype=torch.bool), 1), float("-inf"))
            out[:, h] = torch.softmax(s, -1) @ v[:, g]
        return out.reshape(q.shape[0], H * hd)

    want = [plain(q, k, v) for q, k, v in zip(qs, ks, vs)]
    for b, (k, v) in enumerate(zip(ks, vs)):
        for pos in range(k.shape[0]):
            pg = table[b, pos // page].item()
            k_pages[pg, :, pos % page] = k[pos]
            v_pages[pg, :, pos % page] = v[pos]
    for new, past in ((lens, [0, 0]), ([100, 30], [200, 40]), ([1, 1], lens)):
        q = torch.cat([x[p:p + n].reshape(n, H * hd) for x, p, n in zip(qs, past, new)]).contiguous()
        T = q.shape[0]
        step = SimpleNamespace(
            n_tokens=T, n_seqs=2, single_token=new == [1, 1], max_new=max(new), max_total=max(p + n for p, n in zip(past, new)),
            positions=_i32([p + i for p, n in zip(past, new) for i in range(n)]),
            seq_of_token=_i32([b for b, n in enumerate(new) for _ in range(n)]), cu_seqlens=_i32([0, new[0], new[0] + new[1]]),
            past_lens=_i32(past), total_lens=_i32([p + n for p, n in zip(past, new)]), ws=Workspace(torch.device(DEV)))
        io = LayerIO(k_pages=k_pages, v_pages=v_pages, block_table=table, page_size=page)
        out = torch.empty(T, H * hd, dtype=dtype, device=DEV)
        kernels.attention(step, q, out, H, G, hd, scale, None, io, softcap=cap or 0.0)
        ref = torch.cat([w[p:p + n] for w, p, n in zip(want, past, new)])
        torch.testing.assert_close(out.float().cpu(), ref, **_tol(dtype, (2e-5, 1e-4), (2e-2, 2e-2)))
        # a gate on the heads' outputs (a column slice of wider rows): the flat decode kernel multiplies by its
        # sigmoid as it stores and says so; the others leave the output as it is
        gate = _r(T, H * hd + 16, seed=11, scale=2.0, dtype=dtype)[:, 16:]
        out.fill_(7.0)
        applied = kernels.attention(step, q, out, H, G, hd, scale, None, io, softcap=cap or 0.0, gate=gate)
        assert applied == (dtype == torch.bfloat16 and hd in (64, 128) and new == [1, 1])
        gated = ref * torch.sigmoid(gate.float().cpu()) if applied else ref
        torch.testing.assert_close(out.float().cpu(), gated, **_tol(dtype, (2e-5, 1e-4), (2e-2, 2e-2)))
    if cap:
        s = (qs[0][:, 0].float() @ ks[0][:, 0].float().t()) * scale
        assert (s.abs() > cap / 4).float().mean().item() > 0.01       # the cap does bend scores in this test


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_norm_behind_a_sublayer_and_squared_relu(dtype):
    from ziglm_b200 import kernels
    kernels.require(("elementwise",))
    T = 9
    for n in (50, 64):                                             # 64: sixteen bytes a thread in bfloat16
        wide = _r(T, 3 * n + 8, seed=1, scale=2.0, dtype=dtype)
        a, g = wide[:, :n], wide[:, 2 * n + 8:]
        want = (a.float() * torch.sigmoid(g.float())).to(dtype)
        rest = wide[:, n:].clone()
        kernels.sigmoid_mul(a, g, a)                               # in place, strided rows
        torch.testing.assert_close(a.float(), want.float(), **_tol(dtype, (1e-6, 1e-6), (1e-6, 1e-2)))
        assert torch.equal(wide[:, n:], rest)
    n = 50
    x = _r(T, n, seed=2, scale=3.0, dtype=dtype)
    y = torch.empty_like(x)
    kernels.unary_act(x, y, "relu2")
    torch.testing.assert_close(y.float(), (torch.relu(x.float()) ** 2).to(dtype).float(), atol=0, rtol=0)
    # x += m * branch / rms(branch) * (1 + w), and the new rows in the storage type
    for d in (50, 96, 321):
        branch, res = _r(T, d, seed=3, scale=5.0), _r(T, d, seed=4)
        w = _r(d, seed=5, scale=0.3, dtype=dtype)
        want = res.cpu() + 0.3 * P.norm_around_zero(branch.cpu(), w.float().cpu(), 1e-5)
        rows = torch.empty(T, d, dtype=dtype, device=DEV)
        kernels.norm_add_scaled(branch, w, 1e-5, 0.3, res, rows, weight_offset=1.0)
        torch.testing.assert_close(res.cpu(), want, atol=2e-6, rtol=1e-5)
        assert torch.equal(rows, res.to(dtype))
        kernels.norm_add_scaled(branch, w, 1e-5, 0.3, res, None, weight_offset=1.0)
        torch.testing.assert_close(res.cpu(), want + 0.3 * P.norm_around_zero(branch.cpu(), w.float().cpu(), 1e-5), atol=4e-6, rtol=1e-5)


@pytest.mark.parametrize("T,N,K", [(3, 40, 64), (70, 136, 96), (300, 256, 128)])
def test_product_with_the_squared_relu_in_its_epilogue(T, N, K):
    from ziglm_b200 import kernels
    kernels.require(kernels.fast_gemm_libraries())
    x = _r(T, K, seed=1, dtype=torch.bfloat16)
    w = _r(N, K, seed=2, scale=0.2, dtype=torch.bfloat16)
    bias = _r(N, seed=3)
    out = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    assert kernels.gemm_tc_unary(x, w, out, "relu2", bias=bias)
    want = torch.relu(x.float() @ w.float().t() + bias) ** 2
    torch.testing.assert_close(out.float(), want, atol=2e-2, rtol=2e-2)
    assert (out == 0).float().mean().item() > 0.2                 # the relu did cut


@pytest.mark.parametrize("E,top", [(8, 3), (5, 1), (4, 4), (70, 6)])
def test_router_softmax_over_the_chosen(E, top):
    from ziglm_b200 import kernels
    kernels.require(("moe",))
    T, d = 50, 40
    h = _r(T, d, seed=E)
    router = _r(E, d, seed=1, scale=0.5)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
    want_ids, want_w = P.route(P.Plain(), h.cpu(), router.cpu(), top)
    for z in (None, (h @ router.t()).contiguous()):               # the product taken inside, and given
        kernels.moe_route(z, None, top, 1, 1, 2, ids, wts, softmax_scores=2, h=h if z is None else None,
                          router=router if z is None else None)
        assert torch.equal(ids.cpu().long(), want_ids)
        torch.testing.assert_close(wts.cpu(), want_w, atol=1e-6, rtol=1e-5)
    assert torch.allclose(wts.sum(1), torch.ones(T, device=DEV), atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 5, 200])
@pytest.mark.parametrize("shared", [False, True])
def test_mixture_of_experts_part(dtype, T, shared):
    """The part as the block calls it, on a hand-made step (T = 1, 5: the streaming kernel; 200: tiles in float32,
    tensor cores in bfloat16), with limits below the spread of gate and up so that every clamp is taken."""
    from ziglm_b200.config.spec import FeedForwardSpec
    from ziglm_b200.engine.workspace import Workspace
    from ziglm_b200.parts import feed_forward_class
    from ziglm_b200 import kernels
    d, ff, E, top = 72, 40, 6, 3
    opts = {"experts": E, "top": top, "score": "softmax_chosen", "limit": 0.6, "slope": P.GATE_SLOPE}
    mlp = {"expert": {"ff": ff, "limit": 0.6}, "router": {"experts": E, "top": top}}
    if shared:
        opts["shared"] = FeedForwardSpec("gated_mlp", d, 24, "swish_clamped", options={"limit": 0.4, "slope": P.GATE_SLOPE})
        mlp["shared"] = {"ff": 24, "limit": 0.4}
    spec = FeedForwardSpec("moe", d, ff, "swish_clamped", options=opts)
    cls = feed_forward_class("moe")
    w = {name: _r(*decl.shape, seed=i, scale=0.2, dtype=dtype) for i, (name, decl) in enumerate(cls.declare(spec).items())}
    assert ("shared.gate.weight" in w) == shared
    part = cls(spec, dtype, torch.device(DEV))
    part.bind(w)
    kernels.require(part.kernel_libraries())
    h = _r(T, d, seed=99, dtype=dtype)
    plain_w = {k.replace(".weight", ""): v.float().cpu() for k, v in w.items()}
    want = P.experts_ff(P.Plain(dtype), h.float().cpu(), plain_w, mlp)
    step = SimpleNamespace(ws=Workspace(torch.device(DEV)))
    out = torch.full((T, d), 7.0, device=DEV)
    part.forward(step, h, out, accumulate=False)
    tol = dict(atol=1e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=6e-2, rtol=5e-2)
    torch.testing.assert_close(out.cpu(), want, **tol)
    part.forward(step, h, out, accumulate=True)
    torch.testing.assert_close(out.cpu(), 2 * want, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 40, 200])
def test_feed_forward_with_the_squared_relu(dtype, T):
    from ziglm_b200.config.spec import FeedForwardSpec
    from ziglm_b200.engine.workspace import Workspace
    from ziglm_b200.parts import feed_forward_class
    from ziglm_b200 import kernels
    d, ff = 72, 136
    spec = FeedForwardSpec("mlp", d, ff, "relu2")
    cls = feed_forward_class("mlp")
    w = {name: _r(*decl.shape, seed=i, scale=0.2, dtype=dtype) for i, (name, decl) in enumerate(cls.declare(spec).items())}
    part = cls(spec, dtype, torch.device(DEV))
    part.bind(w)
    kernels.require(part.kernel_libraries())
    h = _r(T, d, seed=9, dtype=dtype)
    want = P.relu_squared_ff(P.Plain(dtype), h.float().cpu(), {k.replace(".weight", ""): v.float().cpu() for k, v in w.items()})
    step = SimpleNamespace(ws=Workspace(torch.device(DEV)))
    out = torch.full((T, d), 7.0, device=DEV)
    part.forward(step, h, out, accumulate=False)
    # bfloat16: the squares are rounded once in the product's epilogue and twice in the plain form; the sums over
    # 136 of them differ by a hundredth of the outputs' spread
    tol = dict(atol=1e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=0.02 * want.abs().max().item(), rtol=5e-2)
    torch.testing.assert_close(out.cpu(), want, **tol)
    part.forward(step, h, out, accumulate=True)
    torch.testing.assert_close(out.cpu(), 2 * want, **tol)
