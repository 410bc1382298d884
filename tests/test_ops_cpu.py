"""C++ host implementations (csrc/cpu_ops.cpp) against the PyTorch statements of the same operators."""
import pytest
import torch

from megalodon_b200 import ops
from megalodon_b200.ops import _ext, reference

needs_ext = pytest.mark.skipif(not _ext.have_ext(), reason="extension not built")


@needs_ext
@pytest.mark.parametrize("B,L,H,G,masked", [(2, 70, 64, 8, True), (1, 1, 32, 32, False), (3, 33, 48, 4, False)])
def test_cpu_timestep_norm_forward(B, L, H, G, masked):
    torch.manual_seed(0)
    x = torch.randn(B, L, H)
    cnt = torch.randint(0, 5, (B,))
    cnt[0] = 0
    pm, pv = torch.randn(B, G) * 0.1, torch.rand(B, G) + 0.5
    gm, bt = torch.randn(H) * 0.1, torch.randn(H) * 0.1
    mask = None
    if masked:
        mask = torch.zeros(B, L, dtype=torch.bool)
        mask[-1, L - 7:] = True
    with torch.no_grad():
        got = ops.timestep_norm(x, cnt, pm, pv, gm, bt, mask, G, 1e-5, 1.0)
        ref = reference.timestep_norm(x, cnt, pm, pv, gm, bt, mask, G, 1e-5, 1.0)
    for a, b in zip(got, ref):
        assert a.dtype == b.dtype and a.shape == b.shape
        assert torch.allclose(a.double(), b.double(), atol=1e-5, rtol=1e-5)


@needs_ext
@pytest.mark.parametrize("with_h", [True, False])
def test_cpu_cema_forward(with_h):
    torch.manual_seed(1)
    B, L, D, N = 2, 37, 24, 16
    x = torch.randn(B, L, D)
    alpha, delta = torch.rand(D, N) * 0.5 + 0.1, torch.rand(D, N) * 0.5 + 0.1
    q = torch.polar(1 - alpha * delta, torch.rand(D, N) * 3)
    gamma = torch.view_as_complex(torch.randn(D, N, 2)) * 0.25
    omega = torch.randn(D)
    hx = torch.view_as_complex(torch.randn(B, D, N, 2)) if with_h else None
    with torch.no_grad():
        y0, h0 = ops.cema(x, alpha, q, gamma, omega, hx, True)
        y1, h1 = reference.cema_scan(x, alpha, q, gamma, omega, hx)
    assert torch.allclose(y0, y1, atol=1e-4, rtol=1e-4)
    assert torch.allclose(torch.view_as_real(h0), torch.view_as_real(h1), atol=1e-4, rtol=1e-4)


@needs_ext
def test_cpu_ops_leave_autograd_to_pytorch():
    """With gradients required the dispatcher must not take the forward-only C++ path."""
    x = torch.randn(1, 5, 8, requires_grad=True)
    cnt, pm, pv = torch.zeros(1, dtype=torch.long), torch.zeros(1, 2), torch.ones(1, 2)
    y = ops.timestep_norm(x, cnt, pm, pv, torch.zeros(8), torch.zeros(8), None, 2, 1e-5, 1.0)[0]
    y.sum().backward()
    assert x.grad is not None


@needs_ext
@pytest.mark.parametrize("groups,length_last,masked", [(None, False, False), (None, True, True), (4, False, True),
                                                       (4, True, False)])
def test_cpu_sequence_norm_forward(groups, length_last, masked):
    torch.manual_seed(2)
    B, L, H = 2, 19, 16
    x = torch.randn(B, H, L) if length_last else torch.randn(B, L, H)
    gamma, beta = torch.randn(H), torch.randn(H)
    mask = None
    if masked:
        mask = torch.zeros(B, L, dtype=torch.bool)
        mask[0, 15:] = True
    with torch.no_grad():
        got = ops.sequence_norm(x, gamma, beta, mask, groups, 1e-5, length_last)
        ref = reference.sequence_norm(x, gamma, beta, mask, groups, 1e-5, length_last)
    assert got.shape == ref.shape and torch.allclose(got, ref, atol=1e-5, rtol=1e-5)


@needs_ext
@pytest.mark.parametrize("with_h", [True, False])
def test_cpu_ema_parameters_and_hidden_forward(with_h):
    torch.manual_seed(3)
    B, L, D, N = 2, 23, 6, 4
    alpha, delta = torch.rand(D, N) * 0.5 + 0.1, torch.rand(D, N) * 0.5 + 0.1
    q = torch.polar(1 - alpha * delta, torch.rand(D, N) * 3)
    gamma = torch.view_as_complex(torch.randn(D, N, 2)) * 0.25
    hx = torch.view_as_complex(torch.randn(B, D, N, 2)) if with_h else None
    x = torch.randn(B, D, L)
    with torch.no_grad():
        k0, b0 = ops.ema_parameters(alpha, q, gamma, hx, L)
        k1, b1 = reference.ema_parameters(alpha, q, gamma, hx, L)
        h0 = ops.ema_hidden(x, alpha, q, hx)
        h1 = reference.ema_hidden(x, alpha, q, hx)
    assert torch.allclose(k0, k1, atol=1e-5, rtol=1e-5)
    assert (b0 is None) == (b1 is None)
    if b0 is not None:
        assert torch.allclose(b0, b1, atol=1e-5, rtol=1e-5)
    assert torch.allclose(torch.view_as_real(h0), torch.view_as_real(h1), atol=1e-5, rtol=1e-5)


# ---------------------------------------------------------------------------- C++ backward passes
def _c():
    return _ext.require()


@needs_ext
@pytest.mark.parametrize("B,L,H,G,masked", [(2, 70, 64, 8, True), (1, 5, 32, 32, False), (3, 33, 48, 4, False)])
def test_cpu_timestep_norm_backward(B, L, H, G, masked):
    torch.manual_seed(3)
    x = torch.randn(B, L, H)
    cnt = torch.randint(0, 5, (B,))
    cnt[0] = 0
    pm, pv = torch.randn(B, G) * 0.1, torch.rand(B, G) + 0.5
    gm, bt = torch.randn(H) * 0.1, torch.randn(H) * 0.1
    mask = None
    if masked:
        mask = torch.zeros(B, L, dtype=torch.bool)
        mask[-1, L - 7:] = True
        mask[0, 2] = True
    gy, gmean, gvar = torch.randn(B, L, H), torch.randn(B, G), torch.randn(B, G)
    leaves = [t.clone().requires_grad_() for t in (x, pm, pv, gm, bt)]
    y, _, m, v = reference.timestep_norm(leaves[0], cnt, leaves[1], leaves[2], leaves[3], leaves[4], mask, G, 1e-5, 1.0)
    ((y * gy).sum() + (m * gmean).sum() + (v * gvar).sum()).backward()
    got = _c().cpu_timestep_norm_bwd(gy, gmean, gvar, x, cnt, pm, pv, gm, 1.0, mask, G, 1e-5)
    for name, a, b in zip(["dx", "dprev_mean", "dprev_var", "dgamma", "dbeta"], got, [t.grad for t in leaves]):
        assert torch.allclose(a.double(), b.double(), atol=2e-4, rtol=2e-4), (name, (a - b).abs().max())


@needs_ext
@pytest.mark.parametrize("G,length_last,masked", [(0, False, True), (0, True, False), (4, False, False), (8, True, True)])
def test_cpu_sequence_norm_backward(G, length_last, masked):
    torch.manual_seed(4)
    B, L, H = 3, 41, 32
    x = torch.randn(B, L, H) * 2 + 0.5
    if length_last:
        x = x.transpose(1, 2).contiguous()
    gm, bt = torch.randn(H) * 0.3 + 1, torch.randn(H) * 0.3
    mask = None
    if masked:
        mask = torch.zeros(B, L, dtype=torch.bool)
        mask[1, L - 9:] = True
    gy = torch.randn_like(x)
    leaves = [t.clone().requires_grad_() for t in (x, gm, bt)]
    y = reference.sequence_norm(leaves[0], leaves[1], leaves[2], mask, G or None, 1e-5, length_last)
    (y * gy).sum().backward()
    got = _c().cpu_sequence_norm_bwd(gy, x, gm, mask, G, 1e-5, length_last)
    for name, a, b in zip(["dx", "dgamma", "dbeta"], got, [t.grad for t in leaves]):
        assert torch.allclose(a.double(), b.double(), atol=2e-4, rtol=2e-4), (name, (a - b).abs().max())


def _ema_coeffs(D, N):
    alpha, delta = torch.rand(D, N) * 0.5 + 0.1, torch.rand(D, N) * 0.5 + 0.1
    q = torch.polar(1 - alpha * delta, torch.rand(D, N) * 3)
    gamma = torch.view_as_complex(torch.randn(D, N, 2)) * 0.25
    return alpha, q, gamma


@needs_ext
@pytest.mark.parametrize("with_h", [True, False])
def test_cpu_ema_parameters_backward(with_h):
    torch.manual_seed(5)
    B, D, N, L = 2, 6, 4, 29
    p, q, gamma = _ema_coeffs(D, N)
    hx = torch.view_as_complex(torch.randn(B, D, N, 2)) if with_h else None
    dk, db = torch.randn(D, L), torch.randn(B, D, L)
    leaves = [t.clone().requires_grad_() for t in (p, q, gamma)] + ([hx.clone().requires_grad_()] if with_h else [])
    k, b = reference.ema_parameters(leaves[0], leaves[1], leaves[2], leaves[3] if with_h else None, L)
    loss = (k * dk).sum() + ((b * db).sum() if with_h else 0.0)
    loss.backward()
    got = _c().cpu_ema_parameters_bwd(dk, db if with_h else None, p, q, gamma, hx)
    for name, a, b_ in zip(["dp", "dq", "dgamma", "dh"], got, [t.grad for t in leaves]):
        a2 = torch.view_as_real(a) if a.is_complex() else a
        b2 = torch.view_as_real(b_) if b_.is_complex() else b_
        assert torch.allclose(a2.double(), b2.double(), atol=2e-4, rtol=2e-4), (name, (a2 - b2).abs().max())


@needs_ext
@pytest.mark.parametrize("with_h", [True, False])
def test_cpu_ema_hidden_backward(with_h):
    torch.manual_seed(6)
    B, D, N, L = 2, 5, 4, 23
    p, q, _ = _ema_coeffs(D, N)
    x = torch.randn(B, D, L)
    hx = torch.view_as_complex(torch.randn(B, D, N, 2)) if with_h else None
    g = torch.view_as_complex(torch.randn(B, D, N, 2))
    leaves = [t.clone().requires_grad_() for t in (x, p, q)] + ([hx.clone().requires_grad_()] if with_h else [])
    h = reference.ema_hidden(leaves[0], leaves[1], leaves[2], leaves[3] if with_h else None)
    h.backward(g)
    got = _c().cpu_ema_hidden_bwd(g, x, p, q, hx)
    for name, a, b_ in zip(["dx", "dp", "dq", "dh"], got, [t.grad for t in leaves]):
        a2 = torch.view_as_real(a) if a.is_complex() else a
        b2 = torch.view_as_real(b_) if b_.is_complex() else b_
        assert torch.allclose(a2.double(), b2.double(), atol=2e-4, rtol=2e-4), (name, (a2 - b2).abs().max())


# ---------------------------------------------------------------------------- autograd over the C++ host code
@needs_ext
def test_cpu_autograd_runs_native_forward_and_backward():
    """fp32 host tensors with gradients go through `ops/cpu_native.py` (C++ forward and backward); values
    and gradients equal autograd through the PyTorch statements of `ops/reference.py`."""
    from megalodon_b200 import ops
    from megalodon_b200.ops import cpu_native

    def close(a, b, what):
        a2 = torch.view_as_real(a) if a.is_complex() else a
        b2 = torch.view_as_real(b) if b.is_complex() else b
        assert torch.allclose(a2.double(), b2.double(), atol=3e-4, rtol=3e-4), (what, (a2 - b2).abs().max())

    torch.manual_seed(7)
    B, L, H, G = 2, 37, 32, 8
    x = torch.randn(B, L, H)
    cnt = torch.tensor([0, 3])
    pm, pv = torch.randn(B, G) * 0.1, torch.rand(B, G) + 0.5
    gm, bt = torch.randn(H) * 0.1, torch.randn(H) * 0.1
    mask = torch.zeros(B, L, dtype=torch.bool)
    mask[1, 30:] = True
    gy, gmean, gvar = torch.randn(B, L, H), torch.randn(B, G), torch.randn(B, G)
    res = []
    for fn in (reference.timestep_norm, ops.timestep_norm):
        lv = [t.clone().requires_grad_() for t in (x, pm, pv, gm, bt)]
        y, c, m, v = fn(lv[0], cnt, lv[1], lv[2], lv[3], lv[4], mask, G, 1e-5, 1.0)
        ((y * gy).sum() + (m * gmean).sum() + (v * gvar).sum()).backward()
        res.append([y, m, v] + [t.grad for t in lv])
    assert res[1][0].grad_fn is not None and "TimestepNorm" in type(res[1][0].grad_fn).__name__
    for i, (a, b) in enumerate(zip(*res)):
        close(a, b, f"timestep_norm {i}")

    D, N, Lk = 6, 4, 29
    p, q, gamma = _ema_coeffs(D, N)
    hx = torch.view_as_complex(torch.randn(B, D, N, 2))
    dk, db = torch.randn(D, Lk), torch.randn(B, D, Lk)
    xx, g = torch.randn(B, D, Lk), torch.view_as_complex(torch.randn(B, D, N, 2))
    res = []
    for mod in (reference, ops):
        lv = [t.clone().requires_grad_() for t in (p, q, gamma, hx, xx)]
        k, b = mod.ema_parameters(lv[0], lv[1], lv[2], lv[3], Lk)
        h = mod.ema_hidden(lv[4], lv[0], lv[1], lv[3])
        ((k * dk).sum() + (b * db).sum()).backward(retain_graph=True)
        h.backward(g)
        res.append([k, b, h] + [t.grad for t in lv])
    for i, (a, b_) in enumerate(zip(*res)):
        close(a, b_, f"ema {i}")
    assert cpu_native is not None


@needs_ext
@pytest.mark.parametrize("with_h", [True, False])
def test_cpu_cema_layer_native_autograd(with_h):
    """The fused complex-EMA layer on the host: C++ forward and backward against autograd through the
    explicit recurrence of `reference.cema_scan` (values, every gradient, the last state and its gradient)."""
    from megalodon_b200 import ops
    torch.manual_seed(8)
    B, L, D, N = 2, 45, 6, 4
    p, q, gamma = _ema_coeffs(D, N)
    p, q, gamma = p.view(D, N, 1), q.view(D, N, 1), gamma.view(D, N, 1)
    omega = torch.randn(D, 1)
    x = torch.randn(B, L, D)
    hx = torch.view_as_complex(torch.randn(B, D, N, 2)) if with_h else None
    gy, gh = torch.randn(B, L, D), torch.view_as_complex(torch.randn(B, D, N, 2))
    res = []
    for native in (False, True):
        lv = [t.clone().requires_grad_() for t in (x, p, q, gamma, omega)] + ([hx.clone().requires_grad_()] if with_h else [])
        h0 = lv[5] if with_h else None
        if native:
            y, h = ops.cema(lv[0], lv[1], lv[2], lv[3], lv[4], h0, True)
            assert "Cema" in type(y.grad_fn).__name__
        else:
            y, h = reference.cema_scan(lv[0], lv[1], lv[2], lv[3], lv[4], h0)
        ((y * gy).sum() + (torch.view_as_real(h) * torch.view_as_real(gh)).sum()).backward()
        res.append([y, h] + [t.grad for t in lv])
    names = ["y", "h", "dx", "dp", "dq", "dgamma", "domega", "dhx"]
    for name, a, b in zip(names, *res):
        a2 = torch.view_as_real(a) if a.is_complex() else a
        b2 = torch.view_as_real(b) if b.is_complex() else b
        assert torch.allclose(a2.double(), b2.double(), atol=3e-4, rtol=3e-4), (name, (a2 - b2).abs().max())
