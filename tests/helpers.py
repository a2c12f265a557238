"""Shared checks for the GPU parity tests: CUDA path vs the CPU oracle on the same tensors."""

import numpy as np
import torch

from oracle import head_oracle as ho

# Tolerances of the parity contract: loss and entropy 1e-3 relative, dHidden 2e-2 relative,
# argmax exact except ties. Per-row statistics get the same 1e-3 with a 1e-3 absolute floor
# (lse and entropy are O(10); target logits can be near 0).
LOSS_RTOL = 1e-3
ROW_RTOL, ROW_ATOL = 1e-3, 1e-3
DX_FRO_RTOL = 1e-2       # the reference's own bound, solution/test_head.py:111-112
DX_MAX_RTOL = 2e-2       # solution/test_head.py:113-114
ARGMAX_LOGIT_ATOL = 2e-3  # "tie": our index's fp32 logit equals the row maximum up to rounding


def run_op(x, w, target, ce_weight, need_grad=True, device="cuda"):
    from esep_soup_kernels_b200.head import fused_linear_ce, last_device_status

    xd = x.to(device).requires_grad_(need_grad)
    loss, stats = fused_linear_ce(xd, w.to(device), target.to(device), ce_weight.to(device))
    dx = None
    if need_grad:
        loss.backward()
        dx = xd.grad
    assert last_device_status(device) == 0
    return loss, stats, dx


def check_against_oracle(x, w, target, ce_weight, loss, stats, dx, rows=None, tie_pairs=None):
    """`rows`: optional index tensor; the oracle then runs on that subset only (rows are
    independent) and loss is not compared."""
    v = w.shape[0]
    if rows is not None:
        xs, ts, cs = x[rows], target[rows], ce_weight[rows]
        stats = {k: s[rows.to(s.device)] for k, s in stats.items()}
        dx = dx[rows.to(dx.device)] if dx is not None else None
    else:
        xs, ts, cs = x, target, ce_weight
    x16 = xs.to(w.dtype)  # the op casts fp32 x to the weight's 16-bit type (reference op.py:109)
    ref = ho.full_vocab_reference(x16, w, ts, cs, want_dx=dx is not None, want_rounded=False)
    cpu = {k: s.detach().cpu() for k, s in stats.items()}
    if rows is None:
        np.testing.assert_allclose(float(loss.detach()), float(ref["loss"]), rtol=LOSS_RTOL, atol=1e-5)
    assert torch.isfinite(cpu["lse"]).all() and torch.isfinite(cpu["entropy"]).all()
    torch.testing.assert_close(cpu["lse"], ref["lse"], rtol=ROW_RTOL, atol=ROW_ATOL)
    torch.testing.assert_close(cpu["entropy"], ref["ent"], rtol=ROW_RTOL, atol=ROW_ATOL)
    torch.testing.assert_close(cpu["target_logit"], ref["tlogit"], rtol=ROW_RTOL, atol=ROW_ATOL)
    valid = (ts >= 0) & (ts < v)
    ref_ce = torch.where(valid, ref["lse"] - ref["tlogit"], torch.zeros(()))
    torch.testing.assert_close(cpu["ce"], ref_ce, rtol=ROW_RTOL, atol=ROW_ATOL)
    assert (cpu["ce"][~valid] == 0).all() and (cpu["target_logit"][~valid] == 0).all()
    # argmax: exact except ties -> the fp32 logit at our index must equal the row maximum
    assert cpu["argmax"].dtype == torch.int64
    assert ((cpu["argmax"] >= 0) & (cpu["argmax"] < v)).all()
    ours_at = (x16.float() * w.float()[cpu["argmax"]]).sum(-1)
    torch.testing.assert_close(ours_at, ref["maxlogit"], rtol=0, atol=ARGMAX_LOGIT_ATOL)
    mism = (cpu["argmax"] != ref["argmax"])
    assert mism.float().mean() < 0.01, "argmax differs from the oracle on more than 1 % of rows"
    if tie_pairs:
        lookup = {int(r): i for i, r in enumerate(rows.tolist())} if rows is not None else None
        for r, j1, j2 in tie_pairs:
            if lookup is not None:
                if r not in lookup:
                    continue
                r = lookup[r]
            assert int(cpu["argmax"][r]) == min(j1, j2), "tie must resolve to the lowest index"
    if dx is not None:
        dxc = dx.detach().float().cpu()
        assert dx.dtype == x.dtype and dxc.shape == xs.shape
        zero_rows = (cs == 0) | ~valid
        if zero_rows.any():
            assert dxc[zero_rows].abs().max().item() == 0.0
        ref_dx = ref["dx"]
        denom = ref_dx.norm().item()
        if denom > 0:
            err = (dxc - ref_dx).norm().item() / denom
            assert err < DX_FRO_RTOL, f"dX relative error {err:.3e}"
            mx = (dxc - ref_dx).abs().max().item() / ref_dx.abs().max().item()
            assert mx < DX_MAX_RTOL, f"dX max error {mx:.3e}"
    return ref
