"""The fused batch norm + ReLU + dropout (csrc/norm_act.cu) against the three torch modules the
reference applies after every hidden conv (hiscache/history_model.py:141-143): forward, running
statistics, all three gradients; row masks; dropout regenerated identically in the backward."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(x, w, b, rm, rv, mask=None, keep=None, p=0.0):
    """fp64 reference with the same semantics; keep: 0/1 dropout mask or None."""
    x = x.double()
    rows = x if mask is None else x[mask]
    mean, var = rows.mean(0), rows.var(0, unbiased=False)
    n = rows.shape[0]
    rm2 = 0.9 * rm.double() + 0.1 * mean
    rv2 = 0.9 * rv.double() + 0.1 * var * n / max(n - 1, 1)
    y = F.relu((x - mean) / torch.sqrt(var + 1e-5) * w.double() + b.double())
    if keep is not None:
        y = y * keep.double() / (1.0 - p)
    if mask is not None:
        y = y * mask.double().unsqueeze(1)
    return y, rm2, rv2


@pytest.mark.parametrize("n,feat", [(1, 8), (37, 100), (5000, 256), (16411, 256), (700, 1024), (3, 4)])
@pytest.mark.parametrize("masked", [False, True])
def test_norm_act_matches_torch(backend, n, feat, masked):
    g = torch.Generator(device=DEV).manual_seed(n + feat)
    x = (torch.randn(n, feat, generator=g, device=DEV) * 1.7 + 0.3).requires_grad_(True)
    w = (torch.rand(feat, generator=g, device=DEV) + 0.5).requires_grad_(True)
    b = (torch.randn(feat, generator=g, device=DEV) * 0.2).requires_grad_(True)
    rm, rv = torch.zeros(feat, device=DEV), torch.ones(feat, device=DEV)
    mask = (torch.rand(n, generator=g, device=DEV) < 0.7) if masked else None
    if masked and int(mask.sum()) < 2:
        mask[:2] = True
        mask = mask[:n]
    state = torch.zeros(4, dtype=torch.int64, device=DEV)
    y = backend.norm_act(x, w, b, state, valid=mask, running_mean=rm, running_var=rv, p=0.0)
    gy = torch.randn(n, feat, generator=g, device=DEV)
    y.backward(gy)
    xr, wr, br = (t.detach().double().requires_grad_(True) for t in (x, w, b))
    yr, rm_r, rv_r = _ref(xr, wr, br, torch.zeros(feat, device=DEV), torch.ones(feat, device=DEV), mask)
    yr.backward(gy.double())
    tol = dict(rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(y.detach().double(), yr.detach(), **tol)
    if n > 1:
        torch.testing.assert_close(rm.double(), rm_r.detach(), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(rv.double(), rv_r.detach(), rtol=1e-4, atol=1e-6)
        # batch-norm gradients cancel heavily: compare against the gradient's own scale
        scale = float(xr.grad.abs().max()) + 1e-12
        assert float((x.grad.double() - xr.grad).abs().max()) < 2e-4 * scale + 1e-6
        torch.testing.assert_close(w.grad.double(), wr.grad, rtol=2e-4, atol=2e-4 * float(wr.grad.abs().max()) + 1e-6)
        torch.testing.assert_close(b.grad.double(), br.grad, rtol=2e-4, atol=2e-4 * float(br.grad.abs().max()) + 1e-6)
    if masked:
        assert float(y.detach()[~mask].abs().sum()) == 0.0
        assert float(x.grad[~mask].abs().sum()) == 0.0
    assert int(state[0]) == 0          # no dropout: the step counter does not move


def test_norm_act_dropout_is_regenerated_in_backward(backend):
    n, feat, p = 4000, 256, 0.5
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn(n, feat, generator=g, device=DEV).requires_grad_(True)
    w = torch.ones(feat, device=DEV, requires_grad=True)
    b = torch.full((feat,), 0.5, device=DEV, requires_grad=True)     # most pre-activations positive
    state = torch.zeros(4, dtype=torch.int64, device=DEV)
    y0 = backend.norm_act(x, w, b, state, p=0.0).detach()
    ys = []
    for step in range(2):
        y = backend.norm_act(x, w, b, state, p=p, seed=1234)
        keep = (y.detach() != 0) | (y0 == 0)
        frac = float(keep[y0 > 0].float().mean())
        assert abs(frac - (1 - p)) < 0.01, frac                       # 1e6 draws: sigma 5e-4
        torch.testing.assert_close(y.detach()[keep], (y0 / (1 - p))[keep], rtol=1e-6, atol=1e-7)
        gy = torch.randn(n, feat, generator=g, device=DEV)
        x.grad = w.grad = b.grad = None
        y.backward(gy)
        xr, wr, br = (t.detach().double().requires_grad_(True) for t in (x, w, b))
        yr, _, _ = _ref(xr, wr, br, torch.zeros(feat, device=DEV), torch.ones(feat, device=DEV), None, keep, p)
        yr.backward(gy.double())
        scale = float(xr.grad.abs().max())
        assert float((x.grad.double() - xr.grad).abs().max()) < 2e-4 * scale
        torch.testing.assert_close(b.grad.double(), br.grad, rtol=2e-4, atol=2e-4 * float(br.grad.abs().max()))
        ys.append(y.detach().clone())
        assert int(state[0]) == step + 1
    # another step, another mask; the same (seed, step) gives the same mask
    assert not torch.equal(ys[0] != 0, ys[1] != 0)
    state2 = torch.zeros(4, dtype=torch.int64, device=DEV)
    assert torch.equal(backend.norm_act(x, w, b, state2, p=p, seed=1234).detach(), ys[0])


def test_fused_layer_trains_like_the_torch_modules(backend):
    """FusedNormAct.act with dropout 0 against BatchNorm1d -> relu on the same data, a few steps of
    SGD: same parameters, same running statistics, interchangeable state dicts."""
    from hiscache.history_model import FusedNormAct
    torch.manual_seed(0)
    fused = FusedNormAct(64).to(DEV).train()
    plain = torch.nn.BatchNorm1d(64).to(DEV).train()
    plain.load_state_dict(fused.state_dict())
    of, op = torch.optim.SGD(fused.parameters(), lr=0.1), torch.optim.SGD(plain.parameters(), lr=0.1)
    for _ in range(5):
        x = torch.randn(300, 64, device=DEV) * 2 + 1
        t = torch.randn(300, 64, device=DEV)
        for m, o, f in ((fused, of, lambda v: fused.act(v, None, 0.0)), (plain, op, lambda v: F.relu(plain(v)))):
            o.zero_grad()
            ((f(x) - t) ** 2).mean().backward()
            o.step()
    for (k, a), (_, b_) in zip(fused.state_dict().items(), plain.state_dict().items()):
        torch.testing.assert_close(a.float(), b_.float(), rtol=1e-4, atol=1e-5, msg=k)
    fused.eval()
    plain.eval()
    x = torch.randn(50, 64, device=DEV)
    torch.testing.assert_close(fused.act(x, None, 0.5), F.relu(plain(x)), rtol=1e-5, atol=1e-6)
