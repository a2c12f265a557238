"""Final residual add + RMSNorm in front of the head (solution/body/norm_rope.py:83-162).

CPU: the oracle restatement against golden vectors made by the reference's own Triton kernels
(tests/golden/make_golden_norm.py). GPU: the CUDA kernels against the golden vectors and the
oracle, and the fused norm -> head -> loss chain against the oracle's chain."""

import os

import numpy as np
import pytest
import torch

from oracle import head_oracle as ho

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "final_norm.npz")
CASES = ("h1536", "h96", "nodelta")


def _half(raw):
    return torch.from_numpy(raw.view(np.int16)).view(torch.float16)


def _case(d, tag):
    c = {k[len(tag) + 1:]: v for k, v in d.items() if k.startswith(tag + "_")}
    out = {"r_in": torch.from_numpy(c["r_in"]), "gamma": torch.from_numpy(c["gamma"]),
           "dy": torch.from_numpy(c["dy"]), "eps": float(c["eps"]),
           "delta": _half(c["delta"]) if int(c["with_delta"]) else None,
           "dr_out": torch.from_numpy(c["dr_out"]) if int(c["with_dr_out"]) else None,
           "r_out": torch.from_numpy(c["r_out"]), "y": _half(c["y"]),
           "rstd": torch.from_numpy(c["rstd"]), "dr": torch.from_numpy(c["dr"]),
           "ddelta": _half(c["ddelta"]) if int(c["with_delta"]) else None}
    return out


def _close16(got, want, ulps=1.0):
    """16-bit outputs may differ by one rounding step where the fp32 value sits on a boundary."""
    g, w = got.float(), want.float()
    tol = ulps * torch.maximum(w.abs() * 2.0 ** -10, torch.full_like(w, 2.0 ** -24))
    assert bool(((g - w).abs() <= tol).all()), float(((g - w).abs() - tol).max())


@pytest.mark.parametrize("tag", CASES)
def test_oracle_norm_matches_reference_kernels(tag):
    c = _case(dict(np.load(GOLDEN)), tag)
    r_out, y, rstd = ho.final_norm_forward(c["r_in"], c["delta"], c["gamma"], c["eps"])
    assert torch.equal(r_out, c["r_out"])
    np.testing.assert_allclose(rstd.numpy(), c["rstd"].numpy(), rtol=2e-6)
    _close16(y, c["y"])
    dr, ddelta = ho.final_norm_backward(c["dy"], c["r_out"], c["rstd"], c["gamma"], c["dr_out"],
                                        torch.float16 if c["delta"] is not None else None)
    scale = float(c["dr"].abs().max())
    np.testing.assert_allclose(dr.numpy(), c["dr"].numpy(), rtol=1e-4, atol=1e-6 * scale)
    if c["ddelta"] is not None:
        _close16(ddelta, c["ddelta"], ulps=2.0)
    # the all-zero row and the zero-gradient row
    assert abs(float(rstd[1]) - c["eps"] ** -0.5) < 1e-2
    assert float(dr[2].abs().max()) == (0.0 if c["dr_out"] is None else float(c["dr_out"][2].abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("tag", CASES)
def test_cuda_norm_matches_reference_kernels(tag):
    from esep_soup_kernels_b200.head import final_norm_backward, final_norm_forward

    c = _case(dict(np.load(GOLDEN)), tag)
    dev = torch.device("cuda", 0)
    cu = lambda t: None if t is None else t.to(dev)
    r_out, y, rstd = final_norm_forward(cu(c["r_in"]), cu(c["delta"]), cu(c["gamma"]), c["eps"],
                                        torch.float16)
    assert torch.equal(r_out.cpu(), c["r_out"])
    np.testing.assert_allclose(rstd.cpu().numpy(), c["rstd"].numpy(), rtol=2e-6)
    _close16(y.cpu(), c["y"])
    dr, ddelta = final_norm_backward(cu(c["dy"]), cu(c["r_out"]), cu(c["rstd"]), cu(c["gamma"]),
                                     cu(c["dr_out"]),
                                     torch.float16 if c["delta"] is not None else None)
    scale = float(c["dr"].abs().max())
    np.testing.assert_allclose(dr.cpu().numpy(), c["dr"].numpy(), rtol=1e-4, atol=1e-6 * scale)
    if c["ddelta"] is not None:
        _close16(ddelta.cpu(), c["ddelta"], ulps=2.0)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,n,h", [(torch.bfloat16, 300, 1536), (torch.float16, 513, 3584),
                                       (torch.float16, 7, 8192), (torch.bfloat16, 1, 4)])
def test_cuda_norm_matches_oracle_on_other_shapes(dtype, n, h):
    from esep_soup_kernels_b200.head import final_norm_backward, final_norm_forward

    g = torch.Generator().manual_seed(h + n)
    r_in = torch.randn(n, h, generator=g) * 2.0
    delta = torch.randn(n, h, generator=g).to(dtype)
    gamma = torch.rand(h, generator=g) + 0.5
    dy = torch.randn(n, h, generator=g) * 1e-3
    dr_out = torch.randn(n, h, generator=g) * 1e-3
    dev = torch.device("cuda", 0)
    r_out, y, rstd = final_norm_forward(r_in.to(dev), delta.to(dev), gamma.to(dev), 1e-6, dtype)
    o_r, o_y, o_rstd = ho.final_norm_forward(r_in, delta, gamma, 1e-6, dtype)
    assert torch.equal(r_out.cpu(), o_r)
    np.testing.assert_allclose(rstd.cpu().numpy(), o_rstd.numpy(), rtol=2e-6)
    ulp = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
    assert float(((y.cpu().float() - o_y.float()).abs() / o_y.float().abs().clamp_min(1e-3)).max()) <= ulp
    dr, ddelta = final_norm_backward(dy.to(dev), r_out, rstd, gamma.to(dev), dr_out.to(dev), dtype)
    o_dr, _ = ho.final_norm_backward(dy, o_r, o_rstd, gamma, dr_out, dtype)
    np.testing.assert_allclose(dr.cpu().numpy(), o_dr.numpy(), rtol=1e-4,
                               atol=1e-6 * float(o_dr.abs().max()))
    assert ddelta.dtype == dtype
    assert float((ddelta.cpu().float() - dr.cpu()).abs().max()) <= ulp * float(dr.abs().max())


@pytest.mark.gpu
def test_bad_norm_arguments_are_rejected():
    from esep_soup_kernels_b200.head import final_norm_forward

    dev = torch.device("cuda", 0)
    with pytest.raises(AssertionError):
        final_norm_forward(torch.zeros(4, 6, device=dev), None, torch.ones(6, device=dev))       # h % 4
    with pytest.raises(AssertionError):
        final_norm_forward(torch.zeros(4, 8, device=dev).half(), None, torch.ones(8, device=dev))  # r_in fp32
    r_out, y, rstd = final_norm_forward(torch.zeros(0, 8, device=dev), None, torch.ones(8, device=dev))
    assert y.shape == (0, 8) and rstd.shape == (0,)


@pytest.mark.gpu
def test_fused_norm_head_matches_the_oracle_chain():
    """norm -> head -> loss in one call: loss / stats against the oracle's norm followed by its
    full-vocabulary cross-entropy, gradients of r_in and delta against autograd through the same
    chain in fp32. Tolerances as for the head alone: loss 1e-3 rel, gradient 2e-2 rel."""
    from esep_soup_kernels_b200.head import fused_norm_linear_ce

    g = torch.Generator().manual_seed(5)
    n, h, v = 333, 256, 5003
    r_in = torch.randn(n, h, generator=g) * 2.0
    delta = torch.randn(n, h, generator=g).half()
    gamma = torch.rand(h, generator=g) + 0.5
    w = (torch.randn(v, h, generator=g) * 0.1).half()
    t = torch.randint(0, v, (n,), generator=g)
    t[::5] = -100
    cew = torch.rand(n, generator=g) / n
    dev = torch.device("cuda", 0)
    r_d = r_in.to(dev).requires_grad_(True)
    d_d = delta.to(dev).requires_grad_(True)
    loss, stats = fused_norm_linear_ce(r_d, d_d, gamma.to(dev), w.to(dev), t.to(dev), cew.to(dev))
    (loss * 3.0).backward()

    # oracle chain with autograd in fp32 (the 16-bit rounding of y is kept, as the head sees it)
    r_ref = r_in.clone().requires_grad_(True)
    d_ref = delta.float().requires_grad_(True)
    r = r_ref + d_ref
    xhat = r * torch.rsqrt((r * r).mean(-1, keepdim=True) + 1e-6)
    y = gamma * xhat
    y16 = y + (y.half().float() - y).detach()          # straight-through rounding
    logits = y16 @ w.float().T
    valid = t >= 0
    ce = torch.nn.functional.cross_entropy(logits, t.clamp_min(0), reduction="none")
    ref_loss = (cew * ce * valid).sum()
    (ref_loss * 3.0).backward()

    np.testing.assert_allclose(float(loss.detach()), float(ref_loss.detach()), rtol=1e-3)
    np.testing.assert_allclose(stats["lse"].cpu().numpy(),
                               torch.logsumexp(logits, -1).detach().numpy(), rtol=1e-3, atol=1e-3)
    assert float((stats["argmax"].cpu() == logits.argmax(-1)).float().mean()) > 0.99
    gr, gd = r_d.grad.cpu(), d_d.grad.cpu().float()
    assert gd.dtype == torch.float32 and d_d.grad.dtype == torch.float16
    rel = lambda a, b: float((a - b).norm() / b.norm())
    assert rel(gr, r_ref.grad) < 2e-2
    assert rel(gd, d_ref.grad) < 2e-2
    dead = ~valid
    assert float(gr[dead].abs().max()) == 0.0

    # no-grad path and empty input
    with torch.no_grad():
        loss2, _ = fused_norm_linear_ce(r_in.to(dev), delta.to(dev), gamma.to(dev), w.to(dev),
                                        t.to(dev), cew.to(dev))
    assert not loss2.requires_grad and float(loss2) == float(loss.detach())
    l0, s0 = fused_norm_linear_ce(r_in[:0].to(dev), None, gamma.to(dev), w.to(dev), t[:0].to(dev),
                                  cew[:0].to(dev))
    assert float(l0) == 0.0 and s0["argmax"].dtype == torch.int64
