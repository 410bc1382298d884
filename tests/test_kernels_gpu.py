"""CUDA kernels against the plain-PyTorch fp32/fp64 statements of the same
operators (values and gradients).  Needs a B200; run with `-m gpu`."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _close(a, b, atol, rtol, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert torch.allclose(a, b, atol=atol, rtol=rtol), f"{what}: max err {err:.3e} (ref max {ref:.3e})"


def _tol(dtype):
    return (2e-5, 2e-4) if dtype == torch.float32 else (3e-2, 3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [256, 1000, 4096])
def test_rms_and_layer_norm(dtype, D):
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(0)
    x = torch.randn(3, 37, D, device=_dev(), dtype=dtype)
    w = (torch.randn(D, device=_dev()) * 0.1).to(dtype)
    b = (torch.randn(D, device=_dev()) * 0.1).to(dtype)
    g = torch.randn_like(x)
    atol, rtol = _tol(dtype)
    for kind in ("rms", "rms_noaffine", "layer"):
        xs = [x.clone().requires_grad_(), x.clone().requires_grad_()]
        ws = [w.clone().requires_grad_(), w.clone().requires_grad_()]
        bs = [b.clone().requires_grad_(), b.clone().requires_grad_()]
        outs = []
        for i, mod in enumerate((ops, reference)):
            if kind == "rms":
                y = mod.rms_norm(xs[i], ws[i], 1e-5, 1.0)
            elif kind == "rms_noaffine":
                y = mod.rms_norm(xs[i], None, 1e-5, 0.0)
            else:
                y = mod.layer_norm(xs[i], ws[i], bs[i], 1e-5, 1.0)
            y.backward(g)
            outs.append(y)
        _close(outs[0], outs[1], atol, rtol, f"{kind} y")
        _close(xs[0].grad, xs[1].grad, atol * 4, rtol, f"{kind} dx")
        if kind != "rms_noaffine":
            _close(ws[0].grad, ws[1].grad, atol * 40, rtol * 3, f"{kind} dw")
        if kind == "layer":
            _close(bs[0].grad, bs[1].grad, atol * 40, rtol * 3, f"{kind} db")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,L,H,G,masked", [(2, 70, 64, 8, True), (1, 1, 128, 32, False),
                                            (2, 1030, 256, 4, False), (1, 300, 96, 96, True),
                                            (1, 16500, 32, 4, True)])   # the last: longer than the one-CTA scan covers
def test_timestep_norm(dtype, B, L, H, G, masked):
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(1)
    dev = _dev()
    x = torch.randn(B, L, H, device=dev, dtype=dtype) * 1.5 + 0.3
    pc = torch.tensor([5, 0][:B], device=dev, dtype=torch.int64) if G != H else torch.full((B,), 4, device=dev)
    pm = (torch.randn(B, G, device=dev) * 0.2).to(dtype)
    pv = (torch.rand(B, G, device=dev) + 0.5).to(dtype)
    gamma = (torch.randn(H, device=dev) * 0.1).to(dtype)
    beta = (torch.randn(H, device=dev) * 0.1).to(dtype)
    mask = None
    if masked:
        mask = torch.zeros(B, L, dtype=torch.bool, device=dev)
        mask[0, L - L // 4:] = True
        if L > 4:
            mask[-1, 3] = True
    gy = torch.randn_like(x)
    gm = torch.randn(B, G, device=dev).to(dtype)
    gv = torch.randn(B, G, device=dev).to(dtype)
    res = []
    for mod in (ops, reference):
        leaves = [t.clone().requires_grad_() for t in (x, pm, pv, gamma, beta)]
        y, c, m, v = mod.timestep_norm(leaves[0], pc, leaves[1], leaves[2], leaves[3], leaves[4], mask, G,
                                       1e-5, 1.0)
        (y.float() * gy.float()).sum().add((m.float() * gm.float()).sum()).add((v.float() * gv.float()).sum()).backward()
        res.append((y, c, m, v, [t.grad for t in leaves]))
    atol, rtol = _tol(dtype)
    (y0, c0, m0, v0, g0), (y1, c1, m1, v1, g1) = res
    assert torch.equal(c0, c1)
    _close(y0, y1, atol * 2, rtol, "y")
    _close(m0, m1, atol, rtol, "mean")
    _close(v0, v1, atol, rtol, "var")
    names = ["dx", "dprev_mean", "dprev_var", "dgamma", "dbeta"]
    scale = [4, 20, 20, 60, 60]
    for n, s, a, b in zip(names, scale, g0, g1):
        _close(a, b, atol * s, rtol * 3, n)


def _cema_coeffs(D, N, dev):
    alpha = torch.sigmoid(torch.randn(D, N, 1, device=dev))
    delta = torch.sigmoid(torch.randn(D, N, 1, device=dev))
    theta = torch.sigmoid(torch.randn(D, 1, 1, device=dev)) * (2 * math.pi / N) * \
        torch.arange(1, N + 1, device=dev).view(1, N, 1)
    p = alpha
    q = torch.polar(1.0 - alpha * delta, theta)
    gamma = torch.view_as_complex(torch.randn(D, N, 2, device=dev)) * math.sqrt(1.0 / N)
    omega = torch.randn(D, 1, device=dev) * 0.3
    return p, q, gamma, omega


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,L,D,N,with_h", [(2, 37, 24, 16, True), (1, 300, 40, 16, True),
                                            (2, 260, 16, 4, False), (1, 1, 32, 16, True),
                                            (2, 513, 8, 8, True), (1, 1024, 256, 16, True),
                                            (1, 200, 136, 32, True), (2, 129, 128, 16, False)])
def test_cema(dtype, B, L, D, N, with_h):
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(2)
    dev = _dev()
    x = (torch.randn(B, L, D, device=dev)).to(dtype)
    p, q, gamma, omega = _cema_coeffs(D, N, dev)
    hx = torch.view_as_complex(torch.randn(B, D, N, 2, device=dev)) if with_h else None
    gy = torch.randn_like(x)
    gh = torch.view_as_complex(torch.randn(B, D, N, 2, device=dev))
    res = []
    for mod in (ops, reference):
        leaves = [t.clone().requires_grad_() for t in (x, p, q, gamma, omega)]
        h_in = None if hx is None else hx.clone().requires_grad_()
        y, h = mod.cema(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], h_in, True)
        loss = (y.float() * gy.float()).sum() + (torch.view_as_real(h) * torch.view_as_real(gh)).sum()
        loss.backward()
        res.append((y, h, [t.grad for t in leaves] + ([h_in.grad] if h_in is not None else [])))
    atol, rtol = (1e-4, 1e-3) if dtype == torch.float32 else (4e-2, 4e-2)
    (y0, h0, g0), (y1, h1, g1) = res
    _close(y0, y1, atol, rtol, "y")
    _close(torch.view_as_real(h0), torch.view_as_real(h1), 1e-3, 1e-2, "h_last")
    names = ["dx", "dp", "dq", "dgamma", "domega", "dhx"]
    for n, a, b in zip(names, g0, g1):
        if a.is_complex():
            a, b = torch.view_as_real(a), torch.view_as_real(b)
        big = b.float().abs().max().item() + 1.0
        tol = (2e-3 if dtype == torch.float32 else 6e-2) * big
        _close(a, b, tol, rtol, n)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_elementwise(dtype):
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(3)
    dev = _dev()
    atol, rtol = _tol(dtype)
    a = torch.randn(5, 33, 96, device=dev, dtype=dtype)
    b = torch.randn_like(a)
    g = torch.randn_like(a)
    outs = []
    for mod in (ops, reference):
        aa, bb = a.clone().requires_grad_(), b.clone().requires_grad_()
        y = mod.swiglu(aa, bb)
        y.backward(g)
        outs.append((y, aa.grad, bb.grad))
    for u, v in zip(*outs):
        _close(u, v, atol, rtol, "swiglu")
    # rotary
    x = torch.randn(2, 16, 3, 64, device=dev, dtype=dtype)
    ang = torch.outer(torch.arange(16, device=dev).float(), torch.rand(32, device=dev))
    fc = torch.polar(torch.ones_like(ang), ang)
    for conj in (False, True):
        _close(ops.rotary(x, fc, conj), reference.rotary(x, fc, conj), atol, rtol, "rotary")
    gx = torch.randn_like(x)
    xr = x.clone().requires_grad_()
    ops.rotary(xr, fc).backward(gx)
    xr2 = x.clone().requires_grad_()
    reference.rotary(xr2, fc).backward(gx)
    _close(xr.grad, xr2.grad, atol, rtol, "rotary grad")


def test_cross_entropy_and_adamw():
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(4)
    dev = _dev()
    logits = torch.randn(50, 1000, device=dev) * 3
    tgt = torch.randint(0, 1000, (50,), device=dev)
    tgt[7] = -100
    g = torch.rand(50, device=dev)
    outs = []
    for mod in (ops, reference):
        l = logits.clone().requires_grad_()
        loss = mod.cross_entropy(l, tgt)
        loss.backward(g)
        outs.append((loss, l.grad))
    _close(outs[0][0], outs[1][0], 1e-4, 1e-4, "ce")
    _close(outs[0][1], outs[1][1], 1e-5, 1e-3, "ce grad")

    n = 4096 + 64
    state = [torch.randn(n, device=dev) for _ in range(2)]
    grad = torch.randn(n, device=dev)
    for gdtype in (torch.float32, torch.bfloat16):
        ps = [state[0].clone(), state[0].clone()]
        ms = [torch.zeros(n, device=dev), torch.zeros(n, device=dev)]
        vs = [torch.zeros(n, device=dev), torch.zeros(n, device=dev)]
        lows = [torch.empty(n, device=dev, dtype=torch.bfloat16) for _ in range(2)]
        for step in (1, 2, 3):
            for i, mod in enumerate((ops, reference)):
                mod.adamw_step(ps[i], grad.to(gdtype), ms[i], vs[i], lr=1e-2, beta1=0.9, beta2=0.98, eps=1e-8,
                               weight_decay=0.1, step=step, grad_scale=0.5, low=lows[i])
        _close(ps[0], ps[1], 1e-5, 1e-4, "adamw p")
        _close(ms[0], ms[1], 1e-6, 1e-4, "adamw m")
        _close(vs[0], vs[1], 1e-6, 1e-4, "adamw v")
        _close(lows[0], lows[1], 1e-2, 1e-2, "adamw low")
    acc = torch.zeros((), dtype=torch.float64, device=dev)
    ops.sum_squares(grad.bfloat16(), acc)
    assert abs(acc.item() - grad.bfloat16().double().pow(2).sum().item()) < 1e-3 * acc.item()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (304, 264, 136), (4096, 1024, 4096), (512, 11264, 4096)])
@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_tcgen05_gemm(M, N, K, layout):
    """C = A B^T for K-major / MN-major operand layouts against fp32 matmul of the same bf16 inputs."""
    from megalodon_b200.ops import cuda_ops
    torch.manual_seed(5)
    dev = _dev()
    A = torch.randn(M, K, device=dev).bfloat16()
    Bm = torch.randn(N, K, device=dev).bfloat16()
    ref = A.float() @ Bm.float().t()
    if layout == "nt":
        out, _ = cuda_ops.gemm(A, Bm)
    elif layout == "nn":          # B stored [K, N]
        out, _ = cuda_ops.gemm(A, Bm.t().contiguous(), b_mn=True)
    else:                          # A stored [K, M], B stored [K, N]
        out, _ = cuda_ops.gemm(A.t().contiguous(), Bm.t().contiguous(), a_mn=True, b_mn=True)
    torch.cuda.synchronize()
    cuda_ops.check_kernel_errors()
    # entries are ~ sqrt(K) in magnitude; the only rounding is the final one to bf16 (2^-8 relative),
    # so the bound is relative to the result's scale, not a fixed 2e-2 sqrt(K)
    _rel_close(out, ref, K, f"gemm {layout}")


def test_tcgen05_gemm_epilogue_and_linear_grad():
    from megalodon_b200 import ops
    from megalodon_b200.ops import cuda_ops
    torch.manual_seed(6)
    dev = _dev()
    x = torch.randn(3, 100, 256, device=dev).bfloat16()
    w = (torch.randn(384, 256, device=dev) * 0.05).bfloat16()
    b = torch.randn(384, device=dev).bfloat16()
    g = torch.randn(3, 100, 384, device=dev).bfloat16()
    for act in (None, "silu"):
        xs = [x.clone().requires_grad_(), x.float().clone().requires_grad_()]
        ws = [w.clone().requires_grad_(), w.float().clone().requires_grad_()]
        bs = [b.clone().requires_grad_(), b.float().clone().requires_grad_()]
        y0 = ops.linear(xs[0], ws[0], bs[0], act)
        y0.backward(g)
        y1 = torch.nn.functional.linear(xs[1], ws[1], bs[1])
        y1 = torch.nn.functional.silu(y1) if act else y1
        y1.backward(g.float())
        cuda_ops.check_kernel_errors()
        _close(y0, y1, 5e-2, 3e-2, f"linear {act}")
        _close(xs[0].grad, xs[1].grad, 5e-2, 3e-2, f"linear dx {act}")
        _close(ws[0].grad, ws[1].grad, 0.3, 3e-2, f"linear dw {act}")
        _close(bs[0].grad, bs[1].grad, 0.3, 3e-2, f"linear db {act}")


def test_tiny_model_trains_on_gpu():
    from megalodon_b200.config import ModelConf, OptimConf
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.modules.losses import cross_entropy
    from megalodon_b200.optim import build_optimizer
    from megalodon_b200.utils import clip_grad_norm_, set_random_seed
    from megalodon_b200.ops import cuda_ops
    cfg = ModelConf(num_layers=2, model_dim=256, num_heads=2, z_dim=128, value_dim=512, ffn_hidden_dim=512,
                    cema_ndim=16, chunk_size=128, vocab_size=512, swiglu=True, norm_num_groups=16,
                    efficient_attn="fused", layerwise_ckpt=True)
    losses = {}
    for dtype in ("bf16",):
        set_random_seed(0)
        model = build_model(cfg, dtype, False, True)
        opt, sched = build_optimizer(model, OptimConf(lr=3e-3, warmup=2), 20, dtype)
        g = torch.Generator().manual_seed(0)
        toks = torch.randint(0, 512, (2, 257), generator=g).cuda()
        x, y = toks[:, :-1], toks[:, 1:]
        curve = []
        for _ in range(8):
            pred, _ = model(x)
            loss = cross_entropy(pred, y).mean()
            loss.backward()
            model.grad_all_reduce()
            clip_grad_norm_(model, 1.0)
            opt.step(); sched.step(); opt.zero_grad()
            curve.append(loss.item())
        cuda_ops.check_kernel_errors()
        losses[dtype] = curve
    c = losses["bf16"]
    assert all(math.isfinite(v) for v in c), c
    assert abs(c[0] - math.log(512)) < 0.5, c
    assert c[-1] < c[0] - 0.1, c


@pytest.mark.parametrize("B,L1,L2,H,dk,dv,causal", [
    (2, 256, 256, 2, 64, 128, True),      # square causal: triangular tile structure
    (1, 640, 640, 4, 256, 512, True),     # several 128-blocks, 7B head dims scaled down in dv
    (2, 1, 100, 2, 64, 128, False),       # single-token decode against a cache
    (1, 24, 152, 1, 32, 64, True),        # prompt remainder against a cache (L1 < L2)
])
def test_attention_matches_reference(B, L1, L2, H, dk, dv, causal):
    from megalodon_b200 import ops
    from megalodon_b200.ops import cuda_ops, reference
    _attention_case(ops, cuda_ops, reference, B, L1, L2, H, dk, dv, causal)
    cuda_ops.set_fused_attention_softmax(False)          # the stand-alone softmax kernels
    try:
        _attention_case(ops, cuda_ops, reference, B, L1, L2, H, dk, dv, causal)
    finally:
        cuda_ops.set_fused_attention_softmax(True)


def _attention_case(ops, cuda_ops, reference, B, L1, L2, H, dk, dv, causal):
    torch.manual_seed(8)
    dev = _dev()
    q = (torch.randn(B, L1, H, dk, device=dev) * 0.3).bfloat16()
    k = (torch.randn(B, L2, H, dk, device=dev) * 0.3).bfloat16()
    v = torch.randn(B, L2, H, dv, device=dev).bfloat16()
    g = torch.randn(B, L1, H, dv, device=dev).bfloat16()
    res = []
    for mod, cast in ((ops, lambda t: t), (reference, lambda t: t.float())):
        qq, kk, vv = (cast(t).clone().requires_grad_() for t in (q, k, v))
        o = mod.attention(qq, kk, vv, 0.7, 0.0, causal, True)
        o.backward(cast(g))
        res.append((o, qq.grad, kk.grad, vv.grad))
    cuda_ops.check_kernel_errors()
    for name, a, b in zip(("o", "dq", "dk", "dv"), *res):
        scale = b.float().abs().max().item() + 1e-3
        _close(a, b, 3e-2 * scale, 5e-2, f"attention {name}")


def test_attention_softmax_op():
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(9)
    dev = _dev()
    x = torch.randn(2, 3, 40, 72, device=dev)
    g = torch.randn_like(x)
    for causal in (True, False):
        outs = []
        for mod in (ops, reference):
            xx = x.clone().requires_grad_()
            y = mod.attention_softmax(xx, 0.0, causal, True)
            y.backward(g)
            outs.append((y, xx.grad))
        _close(outs[0][0], outs[1][0], 1e-5, 1e-4, "softmax")
        _close(outs[0][1], outs[1][1], 1e-5, 1e-3, "softmax grad")
    # DropKey: rows still sum to one, roughly p of the visible keys are removed
    y = ops.attention_softmax(x, 0.5, False, True)
    assert torch.allclose(y.sum(-1), torch.ones_like(y.sum(-1)), atol=1e-4)
    frac = (y == 0).float().mean().item()
    assert 0.4 < frac < 0.6, frac


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("groups,length_last,masked", [(None, False, False), (None, True, True), (4, False, True),
                                                       (8, True, False)])
def test_sequence_norm(dtype, groups, length_last, masked):
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(10)
    dev = _dev()
    B, L, H = 3, 150, 64
    x = torch.randn(B, L, H, device=dev) * 2 + 0.5
    if length_last:
        x = x.transpose(1, 2).contiguous()
    x = x.to(dtype)
    gamma = (torch.randn(H, device=dev) * 0.3 + 1).to(dtype)
    beta = (torch.randn(H, device=dev) * 0.3).to(dtype)
    mask = None
    if masked:
        mask = torch.zeros(B, L, dtype=torch.bool, device=dev)
        mask[0, 100:] = True
        mask[2, 7] = True
    g = torch.randn_like(x)
    res = []
    for mod in (ops, reference):
        leaves = [t.clone().requires_grad_() for t in (x, gamma, beta)]
        y = mod.sequence_norm(leaves[0], leaves[1], leaves[2], mask, groups, 1e-5, length_last)
        y.backward(g)
        res.append((y, [t.grad for t in leaves]))
    atol, rtol = (1e-4, 1e-3) if dtype == torch.float32 else (4e-2, 4e-2)
    _close(res[0][0], res[1][0], atol, rtol, "seqnorm y")
    for n, s, a, b in zip(("dx", "dgamma", "dbeta"), (4, 60, 60), res[0][1], res[1][1]):
        _close(a, b, atol * s, rtol * 3, f"seqnorm {n}")


def test_ema_parameters_hidden_and_dropout():
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(11)
    dev = _dev()
    B, D, N, L = 2, 12, 16, 200
    p, q, gamma, _ = _cema_coeffs(D, N, dev)
    hx = torch.view_as_complex(torch.randn(B, D, N, 2, device=dev))
    gk = torch.randn(D, L, device=dev)
    gb = torch.randn(B, D, L, device=dev)
    res = []
    for mod in (ops, reference):
        leaves = [t.clone().requires_grad_() for t in (p, q, gamma, hx)]
        k, b = mod.ema_parameters(leaves[0], leaves[1], leaves[2], leaves[3], L)
        ((k * gk).sum() + (b * gb).sum()).backward()
        res.append((k, b, [t.grad for t in leaves]))
    _close(res[0][0], res[1][0], 2e-4, 2e-3, "ema k")
    _close(res[0][1], res[1][1], 2e-4, 2e-3, "ema b")
    for n, a, b_ in zip(("dp", "dq", "dgamma", "dh"), res[0][2], res[1][2]):
        if a.is_complex():
            a, b_ = torch.view_as_real(a), torch.view_as_real(b_)
        _close(a, b_, 2e-3 * (b_.abs().max().item() + 1), 5e-3, f"ema {n}")
    # ema_hidden
    x = torch.randn(B, D, L, device=dev)
    gh = torch.view_as_complex(torch.randn(B, D, N, 2, device=dev))
    res = []
    for mod in (ops, reference):
        leaves = [t.clone().requires_grad_() for t in (x, p, q, hx)]
        h = mod.ema_hidden(leaves[0], leaves[1], leaves[2], leaves[3])
        (torch.view_as_real(h) * torch.view_as_real(gh)).sum().backward()
        res.append((h, [t.grad for t in leaves]))
    _close(torch.view_as_real(res[0][0]), torch.view_as_real(res[1][0]), 1e-3, 1e-2, "ema_hidden h")
    for n, a, b_ in zip(("dx", "dp", "dq", "dh"), res[0][1], res[1][1]):
        if a.is_complex():
            a, b_ = torch.view_as_real(a), torch.view_as_real(b_)
        _close(a, b_, 2e-3 * (b_.abs().max().item() + 1), 1e-2, f"ema_hidden {n}")
    # dropout: keeps ~1-p of the entries, scales them, and backward applies the same mask
    t = torch.randn(1 << 16, device=dev).requires_grad_()
    y = ops.memory_efficient_dropout(t, 0.25, True)
    kept = (y != 0)
    assert 0.72 < kept.float().mean().item() < 0.78
    assert torch.allclose(y[kept], t.detach()[kept] / 0.75, rtol=1e-5)
    y.backward(torch.ones_like(y))
    assert torch.equal(t.grad != 0, kept)


def test_decode_session_cuda_graph_matches_cache_path():
    """Graph-replayed decoding gives the logits of the regular cache path (bf16, chunk boundary crossed)."""
    from megalodon_b200.config import ModelConf
    from megalodon_b200.decoding import DecodeSession
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.utils import init_cache, set_random_seed
    from megalodon_b200.ops import cuda_ops
    cfg = ModelConf(num_layers=2, model_dim=256, num_heads=2, z_dim=128, value_dim=512, ffn_hidden_dim=512,
                    cema_ndim=16, chunk_size=128, vocab_size=512, swiglu=True, norm_num_groups=16,
                    efficient_attn="fused")
    set_random_seed(0)
    model = build_model(cfg, "bf16", False, False)
    model.eval()
    inner = model._wrapped
    B = 2
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 512, (B, 128 + 120), generator=g).cuda()
    with torch.no_grad():
        cache = init_cache(B, inner, torch.bfloat16, device=prompt.device)
        _, cache = model(prompt[:, :128], cache=cache)
        logits, cache = model(prompt[:, 128:], cache=cache)
        sess = DecodeSession(model, B, torch.bfloat16)
        sess.load_cache(cache)
        tok = logits[:, -1].argmax(-1)
        worst = 0.0
        for i in range(20):                       # position 120 -> 140: crosses the chunk boundary at 128
            ref, cache = model(tok.view(B, 1), cache=cache)
            got = sess.step(tok)
            worst = max(worst, (ref[:, -1] - got).abs().max().item())
            tok = ref[:, -1].argmax(-1)           # both paths follow the reference tokens
        assert sess._graph is not None, "the step was never captured"
        cuda_ops.check_kernel_errors()
    assert worst < 0.15, worst


@pytest.mark.parametrize("M,N,K", [(1, 272, 136), (3, 1024, 4096), (16, 530, 264)])
@pytest.mark.parametrize("act", [None, "silu"])
def test_small_m_linear(M, N, K, act):
    """Few-row linear (decode path) against an fp32 reference."""
    from megalodon_b200.ops import cuda_ops
    torch.manual_seed(11)
    dev = _dev()
    x = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
    b = torch.randn(N, device=dev).bfloat16()
    for out_dtype in (torch.bfloat16, torch.float32):
        y, _ = cuda_ops.gemm(x, w, b, act, out_dtype=out_dtype)
        ref = x.float() @ w.float().t() + b.float()
        if act:
            ref = torch.nn.functional.silu(ref)
        assert y.dtype == out_dtype and y.shape == (M, N)
        _close(y, ref, 3e-2, 2e-2, f"small-m linear {M}x{N}x{K} {act} {out_dtype}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,D,L", [(2, 8, 37), (1, 16, 300), (2, 4, 4096), (2, 4, 8192), (1, 4, 12000), (2, 3, 16384)])
def test_fftconv_native(dtype, B, D, L):
    """Shared-memory FFT convolution (forward and both gradients) and rfft against torch.fft."""
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(12)
    dev = _dev()
    x = torch.randn(B, D, L, device=dev).to(dtype)
    k = torch.randn(D, L, device=dev) * torch.exp(-torch.arange(L, device=dev) / 50.0)
    g = torch.randn(B, D, L, device=dev).to(dtype)
    outs = []
    for mod in (ops, reference):
        xs, ks = x.clone().requires_grad_(), k.clone().requires_grad_()
        y = mod.fftconv(xs, ks)
        y.backward(g)
        outs.append((y, xs.grad, ks.grad))
    (y0, dx0, dk0), (y1, dx1, dk1) = outs
    atol, rtol = (2e-3, 2e-3) if dtype == torch.float32 else (8e-2, 5e-2)
    _close(y0, y1, atol, rtol, "fftconv y")
    _close(dx0, dx1, atol, rtol, "fftconv dx")
    _close(dk0, dk1, atol * (10 if dtype != torch.float32 else 1) * max(1.0, dk1.abs().max().item()), rtol, "fftconv dk")
    for flip in (False, True):
        f0 = torch.view_as_real(ops.rfft(x, flip))
        f1 = torch.view_as_real(reference.rfft(x, flip))
        _close(f0, f1, 5e-3 * max(1.0, f1.abs().max().item()), 2e-3, f"rfft flip={flip}")


@pytest.mark.parametrize("L", [33, 500, 4096])
def test_packed_real_transforms_match_the_plain_ones(L):
    """The half-size (packed) transforms that rows above 8192 samples need, forced on short rows and
    compared with the full-size kernels and with torch.fft."""
    from megalodon_b200.ops._ext import require
    ext = require()
    torch.manual_seed(18)
    dev = _dev()
    x = torch.randn(3, 5, L, device=dev)
    k = torch.randn(5, L, device=dev) * torch.exp(-torch.arange(L, device=dev) / 40.0)
    for flip in (False, True):
        plain = ext.rfft_rows(x, flip, 0)
        packed = ext.rfft_rows(x, flip, 1)
        scale = plain.abs().max().item()
        assert (plain - packed).abs().max().item() < 2e-5 * scale * math.log2(L + 2)
    kf = ext.rfft_rows(k, False, 0)
    n2 = 2 * (kf.shape[-2] - 1)
    want = torch.fft.irfft(torch.fft.rfft(x, n=n2) * torch.fft.rfft(k, n=n2), n=n2)[..., :L]
    for conj in (False, True):
        y0 = ext.fftconv_apply(x, kf, conj, 0)
        y1 = ext.fftconv_apply(x, kf, conj, 1)
        assert (y0 - y1).abs().max().item() < 1e-4 * max(1.0, y0.abs().max().item())
        if not conj:
            assert (y1 - want).abs().max().item() < 1e-3 * max(1.0, want.abs().max().item())
    spec = ext.rfft_rows(x, False, 0)
    back0 = ext.irfft_rows(spec, L, 0)
    back1 = ext.irfft_rows(spec, L, 1)
    assert (back0 - x).abs().max().item() < 1e-4 and (back1 - x).abs().max().item() < 1e-4


def test_reduce_scatter_adamw_kernel_two_local_ranks():
    """The fused reduce-scatter + AdamW kernel on one GPU: the two 'ranks' are two staging buffers
    in local memory, each rank's shard is checked against the AdamW formula on the summed gradient."""
    from megalodon_b200.ops._ext import require
    from megalodon_b200.ops.cuda_ops import _DT
    ext = require()
    torch.manual_seed(13)
    dev = _dev()
    world, shard_n = 2, 4096 + 64
    stage = [torch.randn(world * shard_n, device=dev).bfloat16() for _ in range(world)]
    bufs = torch.tensor([t.data_ptr() for t in stage], dtype=torch.int64, device=dev)
    lr, b1, b2, eps, wd, step, scale = 3e-3, 0.9, 0.95, 1e-8, 0.1, 3, 0.5
    for rank in range(world):
        p = torch.randn(shard_n, device=dev)
        m = torch.randn(shard_n, device=dev) * 0.1
        v = torch.rand(shard_n, device=dev) * 0.1
        low = torch.empty(shard_n, device=dev, dtype=torch.bfloat16)
        sumsq = torch.zeros((), device=dev, dtype=torch.float64)
        g = scale * sum(t.float()[rank * shard_n:(rank + 1) * shard_n] for t in stage)
        m_ref = b1 * m + (1 - b1) * g
        v_ref = b2 * v + (1 - b2) * g * g
        p_ref = p * (1 - lr * wd) - (lr / (1 - b1 ** step)) * m_ref / (v_ref.sqrt() / (1 - b2 ** step) ** 0.5 + eps)
        ext.reduce_scatter_adamw(bufs, rank, _DT[torch.bfloat16], scale, p, m, v, low, sumsq, lr, b1, b2, eps, wd, step)
        torch.cuda.synchronize()
        _close(p, p_ref, 1e-5, 1e-5, "p")
        _close(m, m_ref, 1e-6, 1e-5, "m")
        _close(v, v_ref, 1e-6, 1e-5, "v")
        _close(low, p_ref, 2e-2, 1e-2, "low")
        assert abs(sumsq.item() - (g.double() ** 2).sum().item()) < 1e-3 * (g.double() ** 2).sum().item()


def test_generate_with_decode_session_on_gpu():
    """`generate()` on a CUDA model takes the graph-replayed session after the prompt; it must run and
    agree with the growing-cache path on the first token (later ones can diverge on bf16 near-ties; the
    logits themselves are compared in test_decode_session_cuda_graph_matches_cache_path)."""
    from megalodon_b200.config import ModelConf
    from megalodon_b200.generation import generate
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.utils import set_random_seed
    cfg = ModelConf(num_layers=2, model_dim=256, num_heads=2, z_dim=128, value_dim=512, ffn_hidden_dim=512,
                    cema_ndim=16, chunk_size=128, vocab_size=512, swiglu=True, norm_num_groups=16,
                    efficient_attn="fused")
    set_random_seed(0)
    model = build_model(cfg, "bf16", False, False)

    class Tok:
        bos_id, eos_id, pad_id, n_words = 1, 2, 0, 512

        def encode(self, s, bos, eos):
            return ([self.bos_id] if bos else []) + [3 + (ord(ch) % 200) for ch in s]

    prompt = ["the quick brown fox jumps over the lazy dog " * 3]
    a = generate(model, "bf16", Tok(), prompt=prompt, max_gen_len=24, use_decode_session=False)
    b = generate(model, "bf16", Tok(), prompt=prompt, max_gen_len=24)
    assert len(a) == len(b) == 1 and len(a[0]) == len(b[0]) == 24
    assert a[0][0] == b[0][0], (a, b)
    agree = sum(int(x == y) for x, y in zip(a[0], b[0]))
    assert agree >= 1


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_reduce_scatter_sumsq_kernel_local_ranks(world, out_dtype):
    """The peer-memory reduce-scatter kernel with every 'rank' a local buffer: sum, scale, cast, squared
    norm and the accumulate mode for 2, 4 and 8 ranks."""
    from megalodon_b200.ops._ext import require
    from megalodon_b200.ops.cuda_ops import _DT
    ext = require()
    torch.manual_seed(14)
    dev = _dev()
    shard_n = 2048 + 64
    stage = [torch.randn(world * shard_n, device=dev).bfloat16() for _ in range(world)]
    bufs = torch.tensor([t.data_ptr() for t in stage], dtype=torch.int64, device=dev)
    scale = 1.0 / world
    for rank in (0, world - 1):
        ref = scale * sum(t.float()[rank * shard_n:(rank + 1) * shard_n] for t in stage)
        out = torch.empty(shard_n, device=dev, dtype=out_dtype)
        sumsq = torch.zeros((), device=dev, dtype=torch.float64)
        ext.reduce_scatter_sumsq(bufs, rank, _DT[torch.bfloat16], scale, out, sumsq, False)
        _close(out, ref, 2e-2 if out_dtype == torch.bfloat16 else 1e-5, 1e-2, f"reduce-scatter world={world}")
        want = (out.double() ** 2).sum().item() if out_dtype == torch.float32 else (ref.double() ** 2).sum().item()
        assert abs(sumsq.item() - want) < 2e-2 * want
        prev = out.clone()
        ext.reduce_scatter_sumsq(bufs, rank, _DT[torch.bfloat16], scale, out, None, True)     # out += ...
        _close(out, prev.float() + ref, 4e-2 if out_dtype == torch.bfloat16 else 1e-5, 2e-2, "accumulate")


def _pieces(world, numels):
    """Piece table of per-parameter sharding for parameters of the given sizes (fsdp.py layout)."""
    rows, off = [], 0
    for n in numels:
        piece = -(-n // (world * 64)) * 64
        rows.append([off // world, piece, off])
        off += piece * world
    return rows, off


@pytest.mark.parametrize("world", [2, 4, 8])
def test_per_parameter_sharding_kernels_local_ranks(world):
    """Gather-by-pull into the natural layout and the reduce-scatter with a piece table, every 'rank' a
    local buffer, against index arithmetic in PyTorch."""
    from megalodon_b200.ops._ext import require
    from megalodon_b200.ops.cuda_ops import _DT
    ext = require()
    torch.manual_seed(15)
    dev = _dev()
    rows, total = _pieces(world, [4096 * 24, 130, 64 * world, 7000, 8 * 1024 * 3])
    table = torch.tensor(rows, dtype=torch.int64, device=dev)
    S = total // world
    # all-gather: shard r holds piece r of every parameter
    full_ref = torch.randn(total, device=dev).bfloat16()
    shards = [torch.empty(S, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    for so, piece, off in rows:
        for r in range(world):
            shards[r][so:so + piece] = full_ref[off + r * piece:off + (r + 1) * piece]
    ptrs = torch.tensor([t.data_ptr() for t in shards], dtype=torch.int64, device=dev)
    full = torch.zeros(total, device=dev, dtype=torch.bfloat16)
    ext.gather_pull(full, ptrs, table, total)
    assert torch.equal(full, full_ref)
    full32 = torch.zeros(total, device=dev, dtype=torch.float32)
    shards32 = [s.float() for s in shards]
    ptrs32 = torch.tensor([t.data_ptr() for t in shards32], dtype=torch.int64, device=dev)
    ext.gather_pull(full32, ptrs32, table, total)
    # a subset of the parameters (the others are gathered elsewhere) leaves the rest of the buffer alone
    some = torch.tensor([rows[1], rows[3]], dtype=torch.int64, device=dev)
    part = torch.full((total,), -7.0, device=dev, dtype=torch.bfloat16)
    ext.gather_pull(part, ptrs, some, world * (rows[1][1] + rows[3][1]))
    want = torch.full((total,), -7.0, device=dev, dtype=torch.bfloat16)
    for so, piece, off in (rows[1], rows[3]):
        want[off:off + world * piece] = full_ref[off:off + world * piece]
    assert torch.equal(part, want)
    assert torch.equal(full32, full_ref.float())
    # reduce-scatter: staged gradients in natural order, rank r receives piece r of every parameter
    stage = [torch.randn(total, device=dev).bfloat16() for _ in range(world)]
    bufs = torch.tensor([t.data_ptr() for t in stage], dtype=torch.int64, device=dev)
    summed = sum(t.float() for t in stage) / world
    for rank in (0, world // 2, world - 1):
        ref = torch.empty(S, device=dev)
        for so, piece, off in rows:
            ref[so:so + piece] = summed[off + rank * piece:off + (rank + 1) * piece]
        out = torch.empty(S, device=dev, dtype=torch.float32)
        sumsq = torch.zeros((), device=dev, dtype=torch.float64)
        ext.reduce_scatter_sumsq(bufs, rank, _DT[torch.bfloat16], 1.0 / world, out, sumsq, False, None, table)
        _close(out, ref, 1e-5, 1e-5, f"reduce-scatter with piece table, world={world} rank={rank}")
        assert abs(sumsq.item() - (ref.double() ** 2).sum().item()) < 1e-3 * (ref.double() ** 2).sum().item()


@pytest.mark.parametrize("world,M,N,K", [(2, 512, 512, 256), (4, 384, 1024, 512), (8, 1024, 2048, 1024),
                                         (8, 4096, 1024, 4096)])
def test_gemm_that_gathers_its_weight_local_ranks(world, M, N, K):
    """The GEMM whose copy warps gather the row-sharded weight while it runs: every 'rank' is a local
    buffer here.  The product must equal x w^T and the full weight must be complete afterwards."""
    from megalodon_b200.ops import cuda_ops
    torch.manual_seed(16)
    dev = _dev()
    x = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(N, K, device=dev) / K ** 0.5).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    rows = N // world
    blocks = [w[r * rows:(r + 1) * rows].clone() for r in range(world)]
    ref = x.float() @ w.float().t() + bias.float()
    for rank in (0, world - 1):
        full = torch.full((N, K), float("nan"), device=dev, dtype=torch.bfloat16)
        y, _ = cuda_ops.gemm(x, full, bias, None, b_gather=([b.data_ptr() for b in blocks], rank))
        torch.cuda.synchronize()
        assert torch.equal(full, w), "gathered weight incomplete"
        _close(y, ref, 3e-2, 2e-2, f"gathering GEMM world={world} rank={rank}")
        cuda_ops.check_kernel_errors()
    # second use of the same scratch flags, SiLU epilogue with pre-activation
    full = torch.zeros(N, K, device=dev, dtype=torch.bfloat16)
    y, pre = cuda_ops.gemm(x, full, bias, "silu", want_preact=True, b_gather=([b.data_ptr() for b in blocks], 1))
    _close(pre, ref, 3e-2, 2e-2, "pre-activation")
    _close(y, torch.nn.functional.silu(ref), 3e-2, 2e-2, "silu")
    cuda_ops.check_kernel_errors()


@pytest.mark.parametrize("fused", [True, False])
def test_attention_at_the_7b_shape(fused):
    """One 4096-token chunk with the 7B head geometry (4 heads, d_qk 256, d_v 2048), causal: the fused
    softmax epilogues (and the stand-alone softmax kernels) against fp32 PyTorch, forward and backward.
    Logits are made large enough (|s| up to ~15) that a wrong row maximum would overflow or flush rows."""
    from megalodon_b200.ops import cuda_ops, reference
    torch.manual_seed(17)
    dev = _dev()
    B, L, H, dk, dv = 1, 4096, 4, 256, 2048
    q = (torch.randn(B, L, H, dk, device=dev) * 0.25).bfloat16()
    k = (torch.randn(B, L, H, dk, device=dev) * 0.25).bfloat16()
    v = torch.randn(B, L, H, dv, device=dev).bfloat16()
    g = torch.randn(B, L, H, dv, device=dev).bfloat16()
    cuda_ops.set_fused_attention_softmax(fused)
    try:
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        o = cuda_ops.attention(qq, kk, vv, 1.0, 0.0, True, True)
        o.backward(g)
    finally:
        cuda_ops.set_fused_attention_softmax(True)
    cuda_ops.check_kernel_errors()
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    oref = reference.attention(qr, kr, vr, 1.0, 0.0, True, True)
    oref.backward(g.float())
    for name, a, b in (("o", o, oref), ("dq", qq.grad, qr.grad), ("dk", kk.grad, kr.grad), ("dv", vv.grad, vr.grad)):
        rel = (a.float() - b).norm() / b.norm()
        assert rel < 2e-2, f"{name}: relative error {rel:.4f}"
        assert torch.isfinite(a.float()).all(), name


def test_cema_at_the_7b_shape():
    """L = 4096, D = 4096, N = 16 in bf16 with an incoming state: the shape the segment planner and the
    tiled kernels see in training.  Features are independent, so the fp32 restatement runs on slices."""
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(21)
    dev = _dev()
    B, L, D, N = 1, 4096, 4096, 16
    x = torch.randn(B, L, D, device=dev).bfloat16()
    p, q, gamma, omega = _cema_coeffs(D, N, dev)
    hx = torch.view_as_complex(torch.randn(B, D, N, 2, device=dev))
    gy = torch.randn_like(x)
    gh = torch.view_as_complex(torch.randn(B, D, N, 2, device=dev))
    leaves = [t.clone().requires_grad_() for t in (x, p, q, gamma, omega, hx)]
    y, h = ops.cema(*leaves[:5], leaves[5], True)
    ((y.float() * gy.float()).sum() + (torch.view_as_real(h) * torch.view_as_real(gh)).sum()).backward()
    for d0 in (0, 1987, D - 64):
        sl = slice(d0, d0 + 64)
        ref_leaves = [t[..., sl].float().clone().requires_grad_() if t is x else t[sl].clone().requires_grad_()
                      for t in (x, p, q, gamma, omega)]
        h_in = hx[:, sl].clone().requires_grad_()
        yr, hr = reference.cema(*ref_leaves, h_in, True)
        ((yr * gy[..., sl].float()).sum() + (torch.view_as_real(hr) * torch.view_as_real(gh[:, sl])).sum()).backward()
        _close(y[..., sl], yr, 6e-2, 4e-2, f"y[{d0}]")
        _close(torch.view_as_real(h[:, sl]), torch.view_as_real(hr), 2e-2, 2e-2, f"h_last[{d0}]")
        got = [leaves[0].grad[..., sl]] + [t.grad[sl] for t in leaves[1:5]] + [leaves[5].grad[:, sl]]
        want = [t.grad for t in ref_leaves] + [h_in.grad]
        for n, a, b in zip(["dx", "dp", "dq", "dgamma", "domega", "dhx"], got, want):
            if a.is_complex():
                a, b = torch.view_as_real(a), torch.view_as_real(b)
            rel = (a.float() - b.float()).norm() / (b.float().norm() + 1e-6)
            assert rel < 3e-2, f"{n}[{d0}]: relative error {rel:.4f}"


def test_timestep_norm_at_the_7b_shape():
    """L = 4096, H = 4096, 64 groups in bf16 with carried statistics; groups are independent, so the
    fp32 restatement runs on two of them."""
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(22)
    dev = _dev()
    B, L, H, G = 1, 4096, 4096, 64
    per = H // G
    x = (torch.randn(B, L, H, device=dev) * 1.5 + 0.3).bfloat16()
    pc = torch.full((B,), 8192, device=dev, dtype=torch.int64)
    pm = (torch.randn(B, G, device=dev) * 0.2).bfloat16()
    pv = (torch.rand(B, G, device=dev) + 0.5).bfloat16()
    gamma = (torch.randn(H, device=dev) * 0.1).bfloat16()
    beta = (torch.randn(H, device=dev) * 0.1).bfloat16()
    gy = torch.randn_like(x)
    gm = torch.randn(B, G, device=dev).bfloat16()
    gv = torch.randn(B, G, device=dev).bfloat16()
    leaves = [t.clone().requires_grad_() for t in (x, pm, pv, gamma, beta)]
    y, c, m, v = ops.timestep_norm(leaves[0], pc, leaves[1], leaves[2], leaves[3], leaves[4], None, G, 1e-5, 1.0)
    ((y.float() * gy.float()).sum() + (m.float() * gm.float()).sum() + (v.float() * gv.float()).sum()).backward()
    assert int(c[0]) == 8192 + L
    for g0 in (0, 37):
        fs, gs = slice(g0 * per, (g0 + 2) * per), slice(g0, g0 + 2)
        ref = [x[..., fs].float().clone().requires_grad_(), pm[:, gs].float().clone().requires_grad_(),
               pv[:, gs].float().clone().requires_grad_(), gamma[fs].float().clone().requires_grad_(),
               beta[fs].float().clone().requires_grad_()]
        yr, cr, mr, vr = reference.timestep_norm(ref[0], pc, ref[1], ref[2], ref[3], ref[4], None, 2, 1e-5, 1.0)
        ((yr * gy[..., fs].float()).sum() + (mr * gm[:, gs].float()).sum() + (vr * gv[:, gs].float()).sum()).backward()
        _close(y[..., fs], yr, 6e-2, 4e-2, f"y group {g0}")
        _close(m[:, gs], mr, 2e-2, 2e-2, "mean")
        _close(v[:, gs], vr, 2e-2, 2e-2, "var")
        got = [leaves[0].grad[..., fs], leaves[1].grad[:, gs], leaves[2].grad[:, gs], leaves[3].grad[fs], leaves[4].grad[fs]]
        for n, a, b in zip(["dx", "dprev_mean", "dprev_var", "dgamma", "dbeta"], got, [t.grad for t in ref]):
            rel = (a.float() - b.float()).norm() / (b.float().norm() + 1e-6)
            assert rel < 4e-2, f"{n} group {g0}: relative error {rel:.4f}"


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_tcgen05_gemm_causal_modes_batched_and_accumulating(mode):
    """The triangular tile structures of the attention products, called directly: batched 3-D operands
    (strided head views), the result compared where the mode defines it, then the accumulating epilogue."""
    from megalodon_b200.ops import cuda_ops
    torch.manual_seed(23)
    dev = _dev()
    Bt, L, d = 3, 640, 128
    tri = torch.tril(torch.ones(L, L, device=dev))
    if mode == 1:       # S = Q K^T, tiles above the diagonal are left unwritten
        q = torch.randn(L, Bt, d, device=dev).bfloat16().permute(1, 0, 2)         # strided batch views
        k = torch.randn(L, Bt, d, device=dev).bfloat16().permute(1, 0, 2)
        out = torch.zeros(Bt, L, L, device=dev, dtype=torch.bfloat16)
        cuda_ops.gemm(q, k, out=out, mode=1, alpha=0.5)
        ref = 0.5 * q.float() @ k.float().transpose(1, 2)
        _rel_close(out.float() * tri, ref * tri, d, "mode 1")
    else:
        a = (torch.randn(Bt, L, L, device=dev) * tri).bfloat16()                  # lower-triangular A
        v = torch.randn(L, Bt, d, device=dev).bfloat16().permute(1, 0, 2)
        out = torch.randn(Bt, L, d, device=dev).bfloat16()
        base = out.float().clone()
        if mode == 2:   # O = A V with A lower-triangular: contraction stops at the tile's last row
            cuda_ops.gemm(a, v, b_mn=True, out=out, mode=2)
            ref = a.float() @ v.float()
            _rel_close(out, ref, L, "mode 2")
            cuda_ops.gemm(a, v, b_mn=True, out=out, mode=2, accumulate=True)
            _rel_close(out, 2 * ref, L, "mode 2 accumulate", extra=ref.abs().max().item() * 8e-3)
        else:           # dV = A^T G with A lower-triangular: contraction starts at the tile's first row
            cuda_ops.gemm(a, v, a_mn=True, b_mn=True, out=out, mode=3)
            ref = a.float().transpose(1, 2) @ v.float()
            _rel_close(out, ref, L, "mode 3")
        del base
    cuda_ops.check_kernel_errors()


def _rel_close(got, want, K, what, extra=0.0):
    """Error bound of a bf16-input, fp32-accumulated product rounded to bf16: relative to the typical
    magnitude sqrt(K) |a| |b| of an entry, at bf16 epsilon."""
    got, want = got.float(), want.float()
    scale = want.abs().max().item()
    err = (got - want).abs().max().item()
    assert err <= 2 ** -7 * scale + extra + 1e-6, f"{what}: max error {err:.4g} against magnitude {scale:.4g}"


def test_table_driven_kernels_skip_and_record_a_bad_index():
    """A piece table that points outside the buffers must not become an out-of-bounds access: the kernel
    checks every index it computes, records the first bad one and skips the access."""
    from megalodon_b200.ops._ext import require
    from megalodon_b200.parallel.symm import describe_abort
    ext = require()
    dev = _dev()
    world = 2
    rows, total = _pieces(world, [4096, 1024])
    S = total // world
    shards = [torch.ones(S, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    ptrs = torch.tensor([t.data_ptr() for t in shards], dtype=torch.int64, device=dev)
    full = torch.zeros(total, device=dev, dtype=torch.bfloat16)
    abort = torch.zeros(16, dtype=torch.int32, device=dev)
    bad = [list(r) for r in rows]
    bad[1][2] = total + 4096                      # natural offset of the second parameter far outside `full`
    ext.gather_pull(full, ptrs, torch.tensor(bad, dtype=torch.int64, device=dev), total, abort, S)
    torch.cuda.synchronize()
    words = abort.tolist()
    assert words[0] == 30, words
    assert "natural index" in describe_abort(words) and "skipped" in describe_abort(words)
    assert bool((full[:rows[0][1] * world] == 1).all())          # the good parameter was still gathered
    # a healthy table leaves the record alone
    abort.zero_()
    ext.gather_pull(full, ptrs, torch.tensor(rows, dtype=torch.int64, device=dev), total, abort, S)
    torch.cuda.synchronize()
    assert abort[0].item() == 0 and bool((full == 1).all())


def test_linear_add_epilogue():
    """x w^T + b + addend with the addition in the GEMM epilogue, values and all four gradients."""
    from megalodon_b200 import ops
    torch.manual_seed(24)
    dev = _dev()
    x = torch.randn(2, 300, 256, device=dev).bfloat16()
    w = (torch.randn(384, 256, device=dev) * 0.05).bfloat16()
    b = torch.randn(384, device=dev).bfloat16()
    r = torch.randn(2, 300, 384, device=dev).bfloat16()
    g = torch.randn(2, 300, 384, device=dev).bfloat16()
    for bias in (b, None):
        a = [t.clone().requires_grad_() for t in (x, w, r)] + ([bias.clone().requires_grad_()] if bias is not None else [None])
        f = [t.float().clone().requires_grad_() for t in (x, w, r)] + ([bias.float().clone().requires_grad_()] if bias is not None else [None])
        y0 = ops.linear_add(a[0], a[1], a[3], a[2])
        y0.backward(g)
        y1 = torch.nn.functional.linear(f[0], f[1], f[3]) + f[2]
        y1.backward(g.float())
        _close(y0, y1, 5e-2, 3e-2, "linear_add")
        for n, p, q in zip(["dx", "dw", "dr", "db"], a, f):
            if p is not None:
                rel = (p.grad.float() - q.grad).norm() / (q.grad.norm() + 1e-6)
                assert rel < 2e-2, (n, rel)


@pytest.mark.parametrize("B,L,H,dh,P,wdtype", [(2, 256, 2, 64, 256, torch.bfloat16), (1, 1024, 4, 256, 512, torch.float32),
                                              (3, 1, 4, 32, 1, torch.bfloat16), (2, 40, 1, 16, 40, torch.float32)])
def test_fused_qk_affine_rotary(B, L, H, dh, P, wdtype):
    """q, k = rotary(z (gamma + 1) / sqrt(d) + beta) in one kernel against the composition of the separate
    operators in fp32, with the gradients w.r.t. z, gamma and beta."""
    from megalodon_b200 import ops
    torch.manual_seed(25)
    dev = _dev()
    S = H * dh
    z = torch.randn(B, L, S, device=dev).bfloat16()
    gamma = (torch.randn(2, S, device=dev) * 0.2).to(wdtype)
    beta = (torch.randn(2, S, device=dev) * 0.2).to(wdtype)
    ang = torch.outer(torch.arange(P, device=dev, dtype=torch.float32) + 3, torch.rand(dh // 2, device=dev))
    freqs = torch.polar(torch.ones_like(ang), ang)
    gq, gk = torch.randn(B, L, S, device=dev).bfloat16(), torch.randn(B, L, S, device=dev).bfloat16()
    a = [t.clone().requires_grad_() for t in (z, gamma, beta)]
    q0, k0 = ops.qk_rotary(a[0], a[1], a[2], freqs, dh)
    (q0.float() * gq.float()).sum().add((k0.float() * gk.float()).sum()).backward()
    f = [t.float().clone().requires_grad_() for t in (z, gamma, beta)]
    q1, k1 = ops.qk_rotary(f[0], f[1], f[2], freqs, dh)            # fp32 input takes the composed path
    (q1 * gq.float()).sum().add((k1 * gk.float()).sum()).backward()
    _close(q0, q1, 3e-2, 2e-2, "q")
    _close(k0, k1, 3e-2, 2e-2, "k")
    for n, p, r in zip(["dz", "dgamma", "dbeta"], a, f):
        rel = (p.grad.float() - r.grad).norm() / (r.grad.norm() + 1e-6)
        assert rel < 2e-2, (n, rel.item())


@pytest.mark.parametrize("B,H,C,dk,dv,pos", [(1, 4, 4096, 256, 2048, 0), (4, 4, 4096, 256, 2048, 1234),
                                             (16, 2, 512, 64, 192, 511), (2, 1, 100, 32, 40, 57)])
def test_decode_attention_reads_only_the_filled_slots(B, H, C, dk, dv, pos):
    """The decode-step attention kernel against fp32 PyTorch; slots beyond `pos` hold NaNs, which a kernel
    that touched them would propagate."""
    from megalodon_b200 import ops
    torch.manual_seed(26)
    dev = _dev()
    q = (torch.randn(B, H, dk, device=dev) * 0.3).bfloat16()
    kb = (torch.randn(B, H, C, dk, device=dev) * 0.3).bfloat16()
    vb = torch.randn(B, H, C, dv, device=dev).bfloat16()
    kb[:, :, pos + 1:] = float("nan")
    vb[:, :, pos + 1:] = float("nan")
    p = torch.tensor([pos], device=dev, dtype=torch.int64)
    out = ops.decode_attention(q, kb, vb, p, 0.9)
    s = torch.einsum("bhd,bhcd->bhc", q.float(), kb[:, :, :pos + 1].float()) * 0.9
    ref = torch.einsum("bhc,bhcd->bhd", torch.softmax(s, -1), vb[:, :, :pos + 1].float())
    assert torch.isfinite(out.float()).all()
    _close(out, ref, 2e-2, 2e-2, "decode attention")


@pytest.mark.parametrize("kind", ["rms", "layer"])
def test_norm_backward_weight_gradients_with_more_rows_than_ctas(kind):
    """2048 rows of 4096: every CTA of the backward kernel walks several rows and leaves one row of partial
    column sums in the workspace, which the finishing kernel adds up."""
    from megalodon_b200 import ops
    from megalodon_b200.ops import reference
    torch.manual_seed(5)
    dev = _dev()
    x = torch.randn(1, 2048, 4096, device=dev).bfloat16()
    w = (torch.randn(4096, device=dev) * 0.1).bfloat16()
    b = (torch.randn(4096, device=dev) * 0.1).bfloat16()
    g = torch.randn_like(x)
    got = []
    for mod, dt in ((ops, torch.bfloat16), (reference, torch.float32)):
        xs, ws, bs = (t.to(dt).clone().requires_grad_() for t in (x, w, b))
        y = mod.rms_norm(xs, ws, 1e-5, 1.0) if kind == "rms" else mod.layer_norm(xs, ws, bs, 1e-5, 1.0)
        y.backward(g.to(dt))
        got.append((xs.grad, ws.grad, bs.grad))
    for name, a, r in zip(("dx", "dw", "db"), got[0], got[1]):
        if a is None:
            assert name == "db" and kind == "rms"
            continue
        rel = (a.float() - r).norm() / r.norm()
        assert rel < 2e-2, f"{kind} {name}: relative error {rel:.4f}"


def test_attention_backward_with_recomputed_probabilities_matches_kept_ones():
    from megalodon_b200.ops import cuda_ops
    torch.manual_seed(11)
    dev = _dev()
    B, L, H, dk, dv = 2, 512, 2, 64, 256
    q = (torch.randn(B, L, H, dk, device=dev) / dk ** 0.5).bfloat16()
    k = torch.randn(B, L, H, dk, device=dev).bfloat16()
    v = torch.randn(B, L, H, dv, device=dev).bfloat16()
    g = torch.randn(B, L, H, dv, device=dev).bfloat16()
    res = []
    try:
        for recompute in (False, True):
            cuda_ops.set_attention_recompute_scores(recompute)
            leaves = [t.clone().requires_grad_() for t in (q, k, v)]
            out = cuda_ops.attention(leaves[0], leaves[1], leaves[2], 1.0, 0.0, True, True)
            out.backward(g)
            res.append([out] + [t.grad for t in leaves])
    finally:
        cuda_ops.set_attention_recompute_scores(False)
    for name, a, b in zip(("out", "dq", "dk", "dv"), res[0], res[1]):
        assert torch.equal(a, b), f"{name} differs: {(a.float() - b.float()).abs().max().item()}"


@pytest.mark.parametrize("M,N", [(4096, 8192), (300, 1024), (37, 264), (5, 16384)])
def test_bias_gradient_column_sums(M, N):
    """The bias gradient of the linear layers: fp32 column sums of a bf16 matrix through per-CTA partial rows
    (the last shape is wider than the kernel covers and takes the library reduction)."""
    from megalodon_b200.ops import cuda_ops
    torch.manual_seed(2)
    g = torch.randn(M, N, device=_dev()).bfloat16()
    got = cuda_ops._bias_grad(g)
    ref = g.double().sum(0)
    assert got.dtype == torch.float32 and got.shape == (N,)
    err = (got.double() - ref).abs().max().item()
    assert err < 1e-3 * max(1.0, M ** 0.5), err
