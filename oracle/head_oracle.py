"""CPU oracle for the fused LM-head path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, the algorithm of the reference's chunked LM head so that the CUDA
kernels can be checked against it. Only tests/, __graft_entry__.smoke() and the cpu_baseline /
reference legs of bench.py may import it; the product package never does, and fails loudly when
its CUDA library is missing.

Parity pin: tests/golden/*.npz hold outputs of the REFERENCE's own code (its Triton row kernel and
op._forward run under TRITON_INTERPRET=1 on CPU tensors, and the _reference function of its unit
test) on seeded inputs; tests/test_oracle.py checks every function below against them. The
fixtures are produced by tests/golden/make_golden.py.

What is restated (paths are inside the reference project):
  full_vocab_reference    solution/test_head.py:12-51   plain fp32 full-vocabulary cross-entropy
  row_softmax_pass1       solution/head/kernels.py:46-82 online max / sum-exp / entropy / argmax
  row_softmax_pass2       solution/head/kernels.py:84-93 g = (softmax - onehot) * G_SCALE
  chunked_op              solution/head/op.py:68-128     chunk loop, live-first permutation, dX
  merge_records           solution/head/kernels.py:70-81 merge of partial (m, s, t, idx) records
  partial_record          the same statistics over a vocabulary shard (vocab-parallel mode)
  step_from_logits        solution/head/patch.py:562-579 per-token loss / entropy / accuracy from logits
  final_norm_forward      solution/body/norm_rope.py:83-109  residual add + RMSNorm in front of the head
  final_norm_backward     solution/body/norm_rope.py:116-162 its backward from the fp32 residual
(the two norm functions are pinned by tests/golden/final_norm.npz, produced by
tests/golden/make_golden_norm.py from the reference's Triton kernels)
"""

import numpy as np
import torch

NEG_BIG = -1.0e30          # solution/head/kernels.py:34
G_SCALE = 1024.0           # solution/head/op.py:39
ROW_BV = 2048              # solution/head/op.py:42
CHUNK_ROWS = 256           # solution/head/op.py:37
IGNORE_INDEX = -100


def _as16(t, dtype):
    return t.to(dtype)


# ---------------------------------------------------------------------------------------------
# solution/test_head.py:12-51  (_reference): the PyTorch full-vocabulary cross-entropy, the parity oracle.
# ---------------------------------------------------------------------------------------------
def full_vocab_reference(x, w, target, ce_weight, rows_per_step=256, want_dx=True,
                         want_rounded=True):
    """fp32 logits = x.float() @ w.float().T, log_softmax, NLL with ignored rows, dX by autograd.

    x [N,H] and w [V,H] are taken at their stored precision (16-bit values upcast exactly).
    Returns a dict of CPU tensors: loss (float64 0-dim), lse, tlogit, ent, maxlogit, argmax, dx,
    and lse16 / tlogit16 / ent16 computed from logits rounded to w.dtype (what a 16-bit GEMM
    output gives, test_head.py:38-45)."""
    w32 = w.float()
    v = w.shape[0]
    keys = ["lse", "tlogit", "ent", "maxlogit", "argmax"]
    if want_dx:
        keys.append("dx")
    if want_rounded:
        keys += ["lse16", "tlogit16", "ent16"]
    outs = {k: [] for k in keys}
    loss = torch.zeros((), dtype=torch.float64)
    for r0 in range(0, x.shape[0], rows_per_step):
        xs = x[r0:r0 + rows_per_step].float().requires_grad_(want_dx)
        ts = target[r0:r0 + rows_per_step]
        cs = ce_weight[r0:r0 + rows_per_step].float()
        logits = xs @ w32.T
        logp = torch.log_softmax(logits, dim=-1)
        valid = (ts >= 0) & (ts < v)
        safe_t = torch.where(valid, ts, torch.zeros_like(ts))
        nll = -logp.gather(1, safe_t[:, None])[:, 0]
        part = (torch.where(valid, cs, torch.zeros_like(cs)) * nll).sum()
        if want_dx:
            (dxs,) = torch.autograd.grad(part, xs)
            outs["dx"].append(dxs)
        with torch.no_grad():
            lse = torch.logsumexp(logits, dim=-1)
            outs["lse"].append(lse)
            outs["tlogit"].append(torch.where(valid, logits.gather(1, safe_t[:, None])[:, 0],
                                              torch.zeros_like(lse)))
            outs["ent"].append(-(logp.exp() * logp).sum(-1))
            mx = logits.max(-1)
            outs["maxlogit"].append(mx.values)
            outs["argmax"].append(mx.indices)
            if want_rounded:
                z16 = logits.to(w.dtype).float()
                lp16 = torch.log_softmax(z16, dim=-1)
                outs["lse16"].append(torch.logsumexp(z16, dim=-1))
                outs["tlogit16"].append(torch.where(valid, z16.gather(1, safe_t[:, None])[:, 0],
                                                    torch.zeros_like(lse)))
                outs["ent16"].append(-(lp16.exp() * lp16).sum(-1))
        loss += part.detach().double()
    res = {k: torch.cat(vs) for k, vs in outs.items()}
    res["loss"] = loss
    return res


# ---------------------------------------------------------------------------------------------
# solution/head/kernels.py:46-82: pass 1 of the row kernel, lane-parallel exactly as written.
# ---------------------------------------------------------------------------------------------
def row_softmax_pass1(z_row, tgt, bv=ROW_BV):
    """z_row: 1-D float32 numpy array (the 16-bit logits upcast). Returns (lse, entropy, argmax,
    target_logit) as Python/NumPy scalars following kernels.py:46-82 step by step."""
    z_row = np.asarray(z_row, dtype=np.float32)
    v_total = z_row.shape[0]
    offs = np.arange(bv)
    m_v = np.full(bv, NEG_BIG, np.float32)
    s_v = np.zeros(bv, np.float32)
    t_v = np.zeros(bv, np.float32)
    i_v = np.zeros(bv, np.int32)
    tz_v = np.zeros(bv, np.float32)
    for v0 in range(0, v_total, bv):
        v = v0 + offs
        ok = v < v_total
        z = np.where(ok, z_row[np.minimum(v, v_total - 1)], np.float32(NEG_BIG)).astype(np.float32)
        m_new = np.maximum(m_v, z)
        i_v = np.where(z > m_v, v, i_v).astype(np.int32)       # kernels.py:60 strict '>'
        dm = (m_v - m_new).astype(np.float32)
        sc = np.exp(dm).astype(np.float32)
        d = (z - m_new).astype(np.float32)
        e = np.where(ok, np.exp(d), 0.0).astype(np.float32)
        t_v = (sc * (t_v + s_v * dm) + e * d).astype(np.float32)  # kernels.py:65
        s_v = (sc * s_v + e).astype(np.float32)                   # kernels.py:66
        m_v = m_new
        tz_v = tz_v + np.where(v == tgt, z, 0.0).astype(np.float32)
    big_m = m_v.max()
    dl = (m_v - big_m).astype(np.float32)
    scl = np.exp(dl).astype(np.float32)
    s_tot = np.float32((s_v * scl).sum(dtype=np.float32))
    t_tot = np.float32((scl * (t_v + s_v * dl)).sum(dtype=np.float32))
    best = int(np.where(m_v == big_m, i_v, 2147483647).min())     # kernels.py:75 lowest index
    log_s = np.float32(np.log(s_tot))
    return (np.float32(big_m + log_s), np.float32(log_s - t_tot / s_tot), best,
            np.float32(tz_v.sum(dtype=np.float32)))


def row_softmax_pass2(z_row, lse, tgt, out_dtype=np.float16, g_scale=G_SCALE):
    """kernels.py:84-93: g = (exp(z - lse) - onehot(tgt)) * G_SCALE, rounded to the logits dtype."""
    z = np.asarray(z_row, dtype=np.float32)
    p = np.exp(z - np.float32(lse)).astype(np.float32)
    v = np.arange(z.shape[0])
    g = (np.where(v == tgt, p - 1.0, p) * np.float32(g_scale)).astype(np.float32)
    return g.astype(out_dtype)


# ---------------------------------------------------------------------------------------------
# solution/head/op.py:68-128: _run + _forward, with torch.mm's 16-bit output rounding.
# ---------------------------------------------------------------------------------------------
def chunked_op(x, w16, target, ce_weight, need_grad, chunk_rows=CHUNK_ROWS):
    """CPU restatement of op._forward/_run. Returns (loss, (lse, tlogit, ce, ent, argmax), dx).

    The two cuBLAS calls are restated as fp32 matmuls of the 16-bit inputs with the first
    product rounded to w16.dtype (op.py:90, fp16 out / fp32 accumulate) and the second kept in
    fp32 (op.py:99). Small shapes only: the row kernel restatement is a Python loop."""
    v = w16.shape[0]
    n, h = x.shape
    target = target.to(torch.int64)
    valid = (target >= 0) & (target < v)                                   # op.py:106
    cew = torch.where(valid, ce_weight.to(torch.float32), torch.zeros(()))  # op.py:107
    tgt = torch.where(valid, target, torch.full_like(target, -1))          # op.py:108
    x16 = x.to(w16.dtype)                                                  # op.py:109
    perm = None
    n_live = 0
    if need_grad:                                                          # op.py:112-117
        live = cew != 0
        perm = torch.argsort((~live).to(torch.int8), stable=True)
        n_live = int(live.sum())
        x16, tgt_p, cew_p = x16[perm], tgt[perm], cew[perm]
    else:
        tgt_p, cew_p = tgt, cew
    lse = torch.empty(n)
    ent = torch.empty(n)
    tlogit = torch.empty(n)
    amax = torch.empty(n, dtype=torch.int64)
    dx = torch.zeros(n, h) if need_grad else None                          # op.py:81
    np16 = np.float16 if w16.dtype == torch.float16 else None
    nc = max(1, min(chunk_rows, n))
    w32 = w16.float()
    for r0 in range(0, n, nc):                                             # op.py:87
        nr = min(nc, n - r0)
        z = (x16[r0:r0 + nr].float() @ w32.T).to(w16.dtype)                # op.py:90
        zf = z.float().numpy()
        g = np.zeros((nr, v), np.float32)
        for i in range(nr):                                                # kernels.py, 1 program / row
            t_i = int(tgt_p[r0 + i])
            l, e, a, tz = row_softmax_pass1(zf[i], t_i)
            lse[r0 + i], ent[r0 + i], amax[r0 + i], tlogit[r0 + i] = float(l), float(e), a, float(tz)
            if need_grad and float(cew_p[r0 + i]) != 0.0:
                if np16 is not None:
                    g[i] = row_softmax_pass2(zf[i], l, t_i, np16).astype(np.float32)
                else:  # bf16 logits buffer: round through torch
                    gi = torch.from_numpy(row_softmax_pass2(zf[i], l, t_i, np.float32))
                    g[i] = gi.to(torch.bfloat16).float().numpy()
        nl = min(max(n_live - r0, 0), nr)                                  # op.py:96
        if need_grad and nl:
            dxc = torch.from_numpy(g[:nl]) @ w32                           # op.py:99
            dx[r0:r0 + nl] = dxc * (cew_p[r0:r0 + nl] * (1.0 / G_SCALE))[:, None]  # op.py:100
    if perm is not None:                                                   # op.py:121-124
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(perm.numel())
        lse, tlogit, ent, amax, dx = lse[inv], tlogit[inv], ent[inv], amax[inv], dx[inv]
    tlogit = torch.where(valid, tlogit, torch.zeros(()))                   # op.py:125
    ce = torch.where(valid, lse - tlogit, torch.zeros(()))                 # op.py:126
    loss = (cew * ce).sum()                                                # op.py:127
    return loss, (lse, tlogit, ce, ent, amax), dx


# ---------------------------------------------------------------------------------------------
# Partial records over a vocabulary range and their merge (kernels.py:70-81), vectorised.
# ---------------------------------------------------------------------------------------------
def partial_record(x, w_shard, target, vocab_offset=0, rows_per_step=256):
    """Per-row (m, s, t, tz, idx) of fp32 logits over one vocabulary shard; idx is a GLOBAL id.

    m = max z, s = sum e^(z-m), t = sum e^(z-m)(z-m), tz = z[target] if the shard owns the
    target else 0, idx = lowest index of the max. Returns a float32 array [5, N] whose last row
    carries idx bit-for-bit as int32 (the layout the C ABI exchanges between ranks)."""
    w32 = w_shard.float()
    vl = w_shard.shape[0]
    n = x.shape[0]
    rec = np.zeros((5, n), np.float32)
    idx = np.zeros(n, np.int32)
    for r0 in range(0, n, rows_per_step):
        z = x[r0:r0 + rows_per_step].float() @ w32.T
        mx = z.max(-1)
        m = mx.values
        d = z - m[:, None]
        e = d.exp()
        sl = slice(r0, r0 + z.shape[0])
        rec[0, sl] = m.numpy()
        rec[1, sl] = e.sum(-1).numpy()
        rec[2, sl] = (e * d).sum(-1).numpy()
        t_loc = target[sl].to(torch.int64) - vocab_offset
        own = (t_loc >= 0) & (t_loc < vl)
        safe = torch.where(own, t_loc, torch.zeros_like(t_loc))
        rec[3, sl] = torch.where(own, z.gather(1, safe[:, None])[:, 0], torch.zeros(())).numpy()
        # torch.max returns one of the maximal indices; take the lowest explicitly
        first = (z == m[:, None]).to(torch.int8).argmax(-1)
        idx[sl] = (first + vocab_offset).numpy().astype(np.int32)
    rec[4] = idx.view(np.float32)
    return rec


def merge_records(records):
    """records: array [K, 5, N]. Returns dict lse, entropy, argmax, target_logit (kernels.py:70-81):
    M = max m_k; S = sum s_k e^(m_k-M); T = sum e^(m_k-M)(t_k + s_k(m_k-M)); argmax = lowest idx
    among the partials whose m_k equals M."""
    rec = np.asarray(records, dtype=np.float32)
    m, s, t, tz = rec[:, 0], rec[:, 1], rec[:, 2], rec[:, 3]
    idx = rec[:, 4].copy().view(np.int32)
    big = m.max(0)
    dl = (m - big[None]).astype(np.float32)
    sc = np.exp(dl).astype(np.float32)
    s_tot = (s * sc).sum(0, dtype=np.float32)
    t_tot = (sc * (t + s * dl)).sum(0, dtype=np.float32)
    best = np.where(m == big[None], idx, np.int32(2147483647)).min(0)
    log_s = np.log(s_tot).astype(np.float32)
    return {"lse": big + log_s, "entropy": log_s - t_tot / s_tot, "argmax": best.astype(np.int64),
            "target_logit": tz.sum(0, dtype=np.float32)}


def finalize_records(records, target, ce_weight, v_global):
    """The per-row outputs and scalars the op returns from merged records (op.py:105-108,125-127)."""
    mr = merge_records(records)
    target = np.asarray(target, dtype=np.int64)
    valid = (target >= 0) & (target < v_global)
    cew = np.where(valid, np.asarray(ce_weight, np.float32), np.float32(0))
    tl = np.where(valid, mr["target_logit"], np.float32(0)).astype(np.float32)
    ce = np.where(valid, mr["lse"] - tl, np.float32(0)).astype(np.float32)
    loss = float((cew.astype(np.float64) * ce.astype(np.float64)).sum())
    n_valid = float(valid.sum())
    n_correct = float(((mr["argmax"] == target) & valid).sum())
    ent_sum = float(mr["entropy"][valid].astype(np.float64).sum())
    return {"lse": mr["lse"], "target_logit": tl, "ce": ce, "entropy": mr["entropy"],
            "argmax": mr["argmax"], "cew": cew, "loss": loss,
            "metrics": np.array([loss, n_valid, n_correct, ent_sum], np.float64)}


def shard_dx(x, w_shard, target, cew, lse, vocab_offset=0, rows_per_step=256):
    """Partial dHidden of one vocabulary shard in fp32:
    cew * (e^(z - lse) - onehot restricted to the shard) @ W_shard  (kernels.py:91-92, op.py:99-100)."""
    w32 = w_shard.float()
    vl = w_shard.shape[0]
    n, h = x.shape
    dx = torch.zeros(n, h)
    lse = torch.as_tensor(lse, dtype=torch.float32)
    cew = torch.as_tensor(cew, dtype=torch.float32)
    for r0 in range(0, n, rows_per_step):
        sl = slice(r0, min(r0 + rows_per_step, n))
        z = x[sl].float() @ w32.T
        g = (z - lse[sl, None]).exp()
        t_loc = target[sl].to(torch.int64) - vocab_offset
        own = (t_loc >= 0) & (t_loc < vl)
        rows = torch.nonzero(own)[:, 0]
        g[rows, t_loc[rows]] -= 1.0
        dx[sl] = (g * cew[sl, None]) @ w32
    return dx


# ---------------------------------------------------------------------------------------------
# solution/head/patch.py:562-579 (_step_from_logits): the per-token results from full logits.
# ---------------------------------------------------------------------------------------------
def step_from_logits(hidden, w, labels, want_grad=False):
    """hidden [B,T,H], w [V,H], labels [B,T] -> dict(token_loss [B,T], token_entropy [B,T],
    correct, labelled, loss_mean): logits = hidden @ w^T in fp32, labels padded with -100 on the
    right and shifted by one, CE with ignore_index, entropy of every position, argmax accuracy.
    want_grad adds "dhidden": the gradient of loss_mean with respect to hidden (fp32)."""
    import torch.nn.functional as F

    bsz, seq = labels.shape
    h32 = hidden.float().detach().requires_grad_(want_grad)
    logits = h32 @ w.float().T
    vocab = logits.shape[-1]
    target = F.pad(labels, (0, 1), value=IGNORE_INDEX)[:, 1:]
    valid = target != IGNORE_INDEX
    token_loss = F.cross_entropy(logits.reshape(-1, vocab), target.reshape(-1),
                                 ignore_index=IGNORE_INDEX, reduction="none").view(bsz, seq)
    token_loss = torch.where(valid, token_loss, torch.zeros(()))
    loss_mean = token_loss.sum() / valid.sum()
    out = {}
    if want_grad:
        out["dhidden"] = torch.autograd.grad(loss_mean, h32)[0]
    with torch.no_grad():
        logp = torch.log_softmax(logits, dim=-1)
        token_entropy = -(logp.exp() * logp).sum(-1)
        correct = ((logits.argmax(dim=-1) == target) & valid).sum()
    out.update({"token_loss": token_loss.detach(), "token_entropy": token_entropy,
                "correct": int(correct), "labelled": int(valid.sum()),
                "loss_mean": float(loss_mean.detach())})
    return out


# ---------------------------------------------------------------------------------------------
# solution/body/norm_rope.py:83-109 (_add_rmsnorm_fwd) and :116-162 (_add_rmsnorm_bwd), the final
# norm of solution/body/packed.py:833: the step either side of the head.
# ---------------------------------------------------------------------------------------------
def final_norm_forward(r_in, delta, gamma, eps, out_dtype=torch.float16):
    """r_out = r_in + delta (fp32); y = gamma * (r_out * rsqrt(mean(r_out^2) + eps)) stored as
    out_dtype; rstd per row. delta None: r_out is r_in. All math in fp32 (norm_rope.py:92-106)."""
    r = r_in.to(torch.float32)
    if delta is not None:
        r = r + delta.to(torch.float32)
    ms = (r * r).sum(-1) / r.shape[-1]
    inv = torch.rsqrt(ms + eps)
    xhat = r * inv[:, None]
    y = (gamma.to(torch.float32) * xhat).to(out_dtype)
    return r, y, inv


def final_norm_backward(dy, r_out, rstd, gamma, dr_out=None, delta_dtype=None):
    """Gradient of the residual stream from dy (any dtype, upcast to fp32):
    g = dy * gamma ; proj = sum(g * xhat) / H ; dr = rstd * (g - xhat * proj) (+ dr_out)
    (norm_rope.py:148-157); ddelta = dr rounded to delta's dtype (:158-159)."""
    xhat = r_out.to(torch.float32) * rstd[:, None]
    g = dy.to(torch.float32) * gamma.to(torch.float32)
    proj = (g * xhat).sum(-1, keepdim=True) / r_out.shape[-1]
    dr = rstd[:, None] * (g - xhat * proj)
    if dr_out is not None:
        dr = dr + dr_out.to(torch.float32)
    ddelta = dr.to(delta_dtype) if delta_dtype is not None else None
    return dr, ddelta
