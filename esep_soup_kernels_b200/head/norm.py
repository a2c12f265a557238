"""The step either side of the LM head: final residual add + RMSNorm, fused with the head.

Mirrors, for the final norm of the packed forward (solution/body/packed.py:833), the reference's
`add_rmsnorm(r_in, delta, weight, eps, out_dtype)` (solution/body/norm_rope.py:289-306, kernels
:83-109 and :116-162):

    r_out = r_in + delta                         fp32
    y     = weight * (r_out * rsqrt(mean(r_out^2) + eps))     fp32 math, stored 16-bit

`final_norm_forward` / `final_norm_backward` are the two kernels; `fused_norm_linear_ce` chains
norm -> head -> loss and, in the backward, feeds the head's fp32 dHidden straight into the norm
backward (the reference rounds it to x.dtype first, head/op.py:143-145, and the norm kernel
upcasts it again). The norm weight is treated as frozen, as in the reference (norm_rope.py:296).
All device work goes through the C library; there is no other implementation behind it.
"""

import torch

from . import _lib
from .op import _DTYPES, _KEYS, _forward, _ptr, _stream


def _check_rows(t, n, h, dtype, name):
    assert t.shape == (n, h) and t.dtype == dtype and t.is_cuda, f"{name}: expected [{n}, {h}] {dtype}"
    return t.contiguous()


def final_norm_forward(r_in, delta, weight, eps=1e-6, out_dtype=None):
    """Returns (r_out fp32 [n, h], y 16-bit [n, h], rstd fp32 [n]). delta None: r_out is r_in.

    out_dtype defaults to delta's dtype (fp16 when there is no delta)."""
    assert r_in.dim() == 2 and r_in.is_cuda and r_in.dtype == torch.float32, "r_in: fp32 [n, h] on a GPU"
    n, h = r_in.shape
    if out_dtype is None:
        out_dtype = delta.dtype if delta is not None else torch.float16
    assert out_dtype in _DTYPES, "y must be fp16 or bf16"
    assert h % 4 == 0 and h <= 8192, "hidden size must be a multiple of 4, at most 8192"
    r_in = r_in.contiguous()
    gamma = _check_rows(weight.detach().to(torch.float32).reshape(1, h), 1, h, torch.float32, "weight")
    dev = r_in.device
    if delta is not None:
        delta = _check_rows(delta, n, h, out_dtype, "delta")
        r_out = torch.empty_like(r_in)
    else:
        r_out = r_in
    y = torch.empty(n, h, device=dev, dtype=out_dtype)
    rstd = torch.empty(n, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        code = _lib.load().esep_head_norm_forward(
            _ptr(r_in), _ptr(delta) if delta is not None else None, _ptr(gamma), n, h, float(eps),
            _DTYPES[out_dtype], _ptr(r_out) if delta is not None else None, _ptr(y), _ptr(rstd),
            _stream(dev))
    _lib.check("esep_head_norm_forward", code)
    return r_out, y, rstd


def final_norm_backward(dy, r_out, rstd, weight, dr_out=None, delta_dtype=None):
    """Returns (dr fp32 [n, h], ddelta in delta_dtype or None) from the fp32 gradient dy of y."""
    n, h = r_out.shape
    dev = r_out.device
    dy = _check_rows(dy, n, h, torch.float32, "dy")
    r_out = _check_rows(r_out, n, h, torch.float32, "r_out")
    gamma = weight.detach().to(torch.float32).reshape(h).contiguous()
    assert rstd.shape == (n,) and rstd.dtype == torch.float32
    if dr_out is not None:
        dr_out = _check_rows(dr_out, n, h, torch.float32, "dr_out")
    assert delta_dtype is None or delta_dtype in _DTYPES
    dr = torch.empty(n, h, device=dev, dtype=torch.float32)
    ddelta = torch.empty(n, h, device=dev, dtype=delta_dtype) if delta_dtype is not None else None
    with torch.cuda.device(dev):
        code = _lib.load().esep_head_norm_backward(
            _ptr(dy), _ptr(r_out), _ptr(rstd.contiguous()), _ptr(gamma),
            _ptr(dr_out) if dr_out is not None else None, n, h,
            _DTYPES[delta_dtype if delta_dtype is not None else torch.float16], _ptr(dr),
            _ptr(ddelta) if ddelta is not None else None, _stream(dev))
    _lib.check("esep_head_norm_backward", code)
    return dr, ddelta


class _NormHead(torch.autograd.Function):
    """norm -> head -> loss. The forward also runs the head's backward sweep and the norm backward
    (both linear in grad_loss), so the backward is one scale, as in the reference's head
    (head/op.py:131-145); what is saved is d loss / d r_out-before-the-norm, not dHidden."""

    @staticmethod
    def forward(ctx, r_in, delta, norm_weight, w16, target, ce_weight, eps):
        r_out, y, rstd = final_norm_forward(r_in, delta, norm_weight, eps, w16.dtype)
        loss, stats, dx, _ = _forward(y, w16, target, ce_weight, True)
        dr, _ = final_norm_backward(dx, r_out, rstd, norm_weight)
        ctx.save_for_backward(dr)
        ctx.delta_dtype = delta.dtype if delta is not None else None
        ctx.set_materialize_grads(False)   # no zero tensors for the outputs without gradient
        ctx.mark_non_differentiable(*stats)
        return (loss, *stats)

    @staticmethod
    def backward(ctx, grad_loss, *unused):
        (dr,) = ctx.saved_tensors
        g = dr * grad_loss
        d_delta = g.to(ctx.delta_dtype) if ctx.delta_dtype is not None and ctx.needs_input_grad[1] else None
        return (g if ctx.needs_input_grad[0] else None), d_delta, None, None, None, None, None


def fused_norm_linear_ce(r_in, delta, norm_weight, w16, target, ce_weight, eps=1e-6,
                         need_grad=None):
    """loss, stats of `fused_linear_ce(add_rmsnorm(r_in, delta, norm_weight)[1], w16, ...)`.

    r_in: fp32 [n, h] residual stream rows that feed the head; delta: 16-bit [n, h] (the last
    layer's output still to be added) or None; gradients flow to r_in (fp32) and delta (its
    dtype). need_grad=None: grad mode is on and r_in or delta requires grad."""
    assert w16.dtype in _DTYPES and w16.dim() == 2 and r_in.dim() == 2
    assert r_in.shape[1] == w16.shape[1], "shape mismatch"
    assert delta is None or delta.dtype == w16.dtype, "delta must have the head weight's dtype"
    if need_grad is None:
        need_grad = torch.is_grad_enabled() and (
            r_in.requires_grad or (delta is not None and delta.requires_grad))
    w16 = w16.contiguous()
    target = target.to(torch.int64)
    if not r_in.shape[0]:
        z = torch.zeros(0, device=r_in.device, dtype=torch.float32)
        loss = r_in.sum() * 0.0 if need_grad else z.sum()
        return loss, dict(zip(_KEYS, (z, z, z, z, z.long())))
    if need_grad:
        loss, *stats = _NormHead.apply(r_in, delta, norm_weight, w16, target, ce_weight, float(eps))
    else:
        with torch.no_grad():
            _, y, _ = final_norm_forward(r_in, delta, norm_weight, eps, w16.dtype)
            loss, stats, _, _ = _forward(y, w16, target, ce_weight, False)
    return loss, dict(zip(_KEYS, stats))


__all__ = ["final_norm_forward", "final_norm_backward", "fused_norm_linear_ce"]

