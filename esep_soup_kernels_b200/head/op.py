"""Fused linear + cross-entropy op over the LM head on B200: drop-in for the reference's
``solution/head/op.py`` (same entry signature and outputs), computed by libesep_head.so.

``loss, stats = fused_linear_ce(x, w16, target, ce_weight)``

- x:         [N, H] fp16 / bf16 / fp32 hidden states; fp32 is cast to w16.dtype inside, the
             gradient comes back in x.dtype (reference: op.py:4-5, 109, 145)
- w16:       [V, H] fp16 (as the reference) or bf16 frozen LM-head weight, gets no gradient
- target:    [N] int, -100 (or any id outside [0, V)) = no CE term for the row (op.py:8, 106)
- ce_weight: [N] fp32 weight of each row's CE term (forced to 0 on ignored rows, op.py:107)
- loss:      0-dim fp32, sum_i ce_weight_i * (lse_i - z_i[target_i]); differentiable w.r.t. x
- stats:     dict of detached [N] tensors, every row gets lse / entropy / argmax:
             "lse" fp32, "target_logit" fp32 (0 where ignored), "ce" fp32 (0 where ignored),
             "entropy" fp32, "argmax" int64                                  (op.py:11-13, 148)

As in the reference the input gradient is computed in the forward call when it is needed
(op.py:15-16, 131-145) and the autograd backward only scales it by grad_loss.

One C call (``esep_head_step``) does the whole of op.py:68-128 on the device and is a function of
its arguments only: masks, the stable "rows with a loss first" order, the row counts and the
work split of the kernels are all computed on the GPU, the host never waits for a count (the
reference reads the number of live rows back on every call, op.py:116). Every logit is computed
once. Rows that need a gradient go through two sweeps over the vocabulary by default: a forward
sweep that keeps the statistics and leaves the bf16 softmax weights in the workspace, and a
dHidden sweep that reads them back by TMA (``set_training_path``: "stored_logits" keeps fp16
logits instead, "single_pass" forms statistics and dHidden from the same tiles and writes
nothing per logit). Rows that only need statistics (ignored or zero-weight rows when there are
many of them, every row of a call without gradient) go through the forward sweep alone. The
256-row chunk buffer of op.py:83-84 does not exist, so ``chunk_rows`` is accepted and ignored;
the logits stay fp32 in tensor memory for the statistics instead of being rounded to fp16
(op.py:18, 90), so results sit closer to the fp32 oracle.

The default sweeps and the single pass take their softmax weights (bf16) relative to a per-row
reference maximum from a vocabulary prefix; a row whose true maximum lies more than 115 above
its prefix maximum raises a device flag and the library's guarded two-kernel path (forward
sweep + recomputing backward sweep, queued behind the flag in the same call) replaces the
results - no host synchronisation either way. For an fp16 model the dHidden GEMM of both reads
a cached bf16 copy of the frozen weight (V*H*2 bytes of device memory per model). ``SINGLE_SWEEP = False`` makes calls with gradient use
the two-kernel path directly.
"""

import ctypes
import threading

import torch

from . import _lib

# Kept for callers that import them (reference: op.py:35-44). CHUNK_ROWS is a no-op hint here.
CHUNK_ROWS = 256
G_SCALE = 1024.0
VOCAB = 151936

# Calls with gradient use the library's step (module docstring); False = forward sweep + backward
# sweep over all rows. A switch the caller sets, never something the library infers.
SINGLE_SWEEP = True

_KEYS = ("lse", "target_logit", "ce", "entropy", "argmax")
_DTYPES = {torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16}
_X_DTYPES = {torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16,
             torch.float32: _lib.DTYPE_F32}

# Monitoring only (last_device_status / last_call_fell_back): the workspace of the most recent
# call per device. Results never depend on it.
_state_lock = threading.Lock()
_last_workspace = {}
_last_overflow = {}


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def warmup(device=None, vocab=VOCAB):
    """Launch-free initialisation of the CUDA library for ``device`` (function attributes,
    occupancy, driver entry points). No-op without CUDA. Safe to call from a worker thread.
    Counterpart of the reference's ahead-of-time compile, op.py:47-65 (``vocab`` is unused: the
    kernels are not specialised on it)."""
    if not torch.cuda.is_available():
        return
    device = torch.device("cuda" if device is None else device)
    index = torch.cuda.current_device() if device.index is None else device.index
    _lib.check("esep_head_warmup", _lib.load().esep_head_warmup(index))


def _remember(device, ws, overflow):
    with _state_lock:
        _last_workspace[device.index] = ws
        _last_overflow[device.index] = overflow


class DeviceBackend:
    """The C entry points for one problem size, with the scratch workspace they need. Used by the
    sharded forms (parallel.py) and by the explicit two-kernel path."""

    def __init__(self, x16, w16, need_grad):
        self.lib = _lib.load()
        self.device = x16.device
        self.n, self.h = x16.shape
        self.v_local = w16.shape[0]
        self.dtype = _DTYPES[w16.dtype]
        self.need_grad = bool(need_grad)
        self._ws = None

    @property
    def ws(self):
        """Workspace of the forward / backward sweeps, allocated when one of them first runs."""
        if self._ws is None:
            with torch.cuda.device(self.device):
                nbytes = self.lib.esep_head_workspace_bytes(self.n, self.h, self.v_local,
                                                            self.dtype, int(self.need_grad))
            if nbytes == 0:
                code, _ = _lib.query(self.device.index)
                _lib.check("esep_head_query", code)
                raise _lib.HeadLibraryError("esep_head_workspace_bytes", -1,
                                            "no plan for this size")
            self._ws = torch.empty(nbytes, device=self.device, dtype=torch.uint8)
            self._ws[:256].zero_()   # device status word (a backward-only call never clears it)
            _remember(self.device, self._ws, None)
        return self._ws

    def forward_partial(self, x16, w16, target, vocab_offset=0):
        rec = torch.empty(_lib.RECORD_FIELDS, self.n, device=self.device, dtype=torch.float32)
        with torch.cuda.device(self.device):
            code = self.lib.esep_head_forward_partial(
                _ptr(x16), _ptr(w16), _ptr(target), self.n, self.h, self.v_local, vocab_offset,
                self.dtype, _ptr(rec), _ptr(self.ws), self.ws.numel(), _stream(self.device))
        _lib.check("esep_head_forward_partial", code)
        return rec

    def finalize(self, records, target, ce_weight, v_global):
        n, dev = self.n, self.device
        f = torch.empty(5 * n + 1 + _lib.METRIC_SCALARS, device=dev, dtype=torch.float32)
        out = {"lse": f[0:n], "target_logit": f[n:2 * n], "ce": f[2 * n:3 * n],
               "entropy": f[3 * n:4 * n], "cew": f[4 * n:5 * n], "loss": f[5 * n:5 * n + 1],
               "metrics": f[5 * n + 1:], "argmax": torch.empty(n, device=dev, dtype=torch.int64)}
        k = records.shape[0] if records.dim() == 3 else 1
        with torch.cuda.device(dev):
            code = self.lib.esep_head_finalize(
                _ptr(records), k, _ptr(target), _ptr(ce_weight), n, v_global, _ptr(out["lse"]),
                _ptr(out["target_logit"]), _ptr(out["ce"]), _ptr(out["entropy"]),
                _ptr(out["argmax"]), _ptr(out["cew"]), _ptr(out["loss"]), _ptr(out["metrics"]),
                _ptr(self.ws), self.ws.numel(), _stream(dev))
        _lib.check("esep_head_finalize", code)
        return out

    accepts_out = True   # backward(..., out=) writes dHidden into a caller-owned buffer

    def train(self, x16, w16, w_bf16, target, ce_weight):
        """Single pass over this weight as a vocabulary of its own: statistics and dHidden of
        every row. Returns the finalize() dictionary plus "dx" and "overflow" (device int: 1 if
        the guarded two-kernel path produced the outputs)."""
        out = _run_step(x16, w16, True, target=target, ce_weight=ce_weight, w_bf16=w_bf16,
                        want_top=True)
        out["metrics"] = out["metrics"][:_lib.METRIC_SCALARS]
        return out

    # ---- vocabulary shards on the single pass (formulas: csrc/head_aux.cuh) -----------------
    def vp_prepare(self, target, vocab_offset, v_local, v_global):
        """(local target, unit weight) of every row for this rank's shard."""
        n, dev = self.n, self.device
        local_target = torch.empty(n, device=dev, dtype=torch.int64)
        unit = torch.empty(n, device=dev, dtype=torch.float32)
        with torch.cuda.device(dev):
            code = self.lib.esep_head_vp_prepare(_ptr(target), n, vocab_offset, v_local, v_global,
                                                 _ptr(local_target), _ptr(unit), _stream(dev))
        _lib.check("esep_head_vp_prepare", code)
        return local_target, unit

    def vp_pack(self, out, target, vocab_offset, v_local, v_global):
        """This rank's [5, n] record from the outputs of its local train() call."""
        n, dev = self.n, self.device
        rec = torch.empty(_lib.RECORD_FIELDS, n, device=dev, dtype=torch.float32)
        with torch.cuda.device(dev):
            code = self.lib.esep_head_vp_pack(
                _ptr(out["lse"]), _ptr(out["entropy"]), _ptr(out["top"]), _ptr(out["target_logit"]),
                _ptr(out["argmax"]), _ptr(target), n, vocab_offset, v_local, v_global, _ptr(rec),
                _stream(dev))
        _lib.check("esep_head_vp_pack", code)
        return rec

    def vp_combine(self, records, me, target, ce_weight, w_shard, vocab_offset, v_global, dx):
        """Global statistics from all ranks' records; dx (the local sweep's result) is rewritten
        in place into this rank's share of dHidden."""
        n, dev = self.n, self.device
        f = torch.empty(5 * n + 1 + _lib.METRIC_SCALARS, device=dev, dtype=torch.float32)
        out = {"lse": f[0:n], "target_logit": f[n:2 * n], "ce": f[2 * n:3 * n],
               "entropy": f[3 * n:4 * n], "cew": f[4 * n:5 * n], "loss": f[5 * n:5 * n + 1],
               "metrics": f[5 * n + 1:], "argmax": torch.empty(n, device=dev, dtype=torch.int64)}
        records = records.contiguous()
        with torch.cuda.device(dev):
            code = self.lib.esep_head_vp_combine(
                _ptr(records), records.shape[0], int(me), _ptr(target), _ptr(ce_weight),
                _ptr(w_shard), n, self.h, w_shard.shape[0], vocab_offset, v_global, self.dtype,
                _ptr(dx), _ptr(out["lse"]), _ptr(out["target_logit"]), _ptr(out["ce"]),
                _ptr(out["entropy"]), _ptr(out["argmax"]), _ptr(out["cew"]), _ptr(out["loss"]),
                _ptr(out["metrics"]), _stream(dev))
        _lib.check("esep_head_vp_combine", code)
        return out

    def backward(self, x16, w16, target, cew, lse, vocab_offset=0, out=None):
        if out is None:
            dx = torch.empty(self.n, self.h, device=self.device, dtype=torch.float32)
        else:
            assert out.shape == (self.n, self.h) and out.dtype == torch.float32
            assert out.is_contiguous() and out.device == self.device
            dx = out
        with torch.cuda.device(self.device):
            code = self.lib.esep_head_backward(
                _ptr(x16), _ptr(w16), _ptr(target), _ptr(cew), _ptr(lse), self.n, self.h,
                self.v_local, vocab_offset, self.dtype, _ptr(dx), _ptr(self.ws), self.ws.numel(),
                _stream(self.device))
        _lib.check("esep_head_backward", code)
        return dx


TRAINING_PATHS = {"auto": 0, "single_pass": 1, "stored_logits": 2, "stored_weights": 3}


def set_training_path(path="auto"):
    """Which kernels a call with gradient uses for the rows that need one (process-wide; see
    ``esep_head_set_training_path`` in include/esep_head.h): "stored_weights" keeps the softmax
    weights in the workspace as bf16 between a forward sweep and a dHidden sweep (the fastest path
    on B200), "stored_logits" keeps fp16 logits instead (no bf16 copy of an fp16 W),
    "single_pass" keeps them on the SM (no buffer), "auto" (default) takes "stored_weights"
    wherever the two sweeps apply. Returns the previous setting's name."""
    prev = _lib.load().esep_head_set_training_path(TRAINING_PATHS[path])
    if prev < 0:
        _lib.check("esep_head_set_training_path", prev)
    return {v: k for k, v in TRAINING_PATHS.items()}[prev]


def last_device_status(device=None):
    """Synchronises and returns the device status word of the most recent call on ``device``
    (0 = every kernel ran to completion; see include/esep_head.h). Raises on a non-zero word."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    with _state_lock:
        ws = _last_workspace.get(index)
    if ws is None:
        return 0
    out = ctypes.c_int(0)
    code = _lib.load().esep_head_device_status(_ptr(ws), _stream(ws.device), ctypes.byref(out))
    if code != _lib.ESEP_OK:
        raise _lib.HeadLibraryError("esep_head_device_status", code,
                                    f"{_lib.status_string(code)}; device word {out.value}")
    return out.value


def last_call_used_stored_logits(device=None):
    """True if the most recent call with gradient on the device took a two-sweep path (stored
    weights or stored logits). Synchronises (a test aid)."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    with _state_lock:
        ws = _last_workspace.get(index)
    if ws is None:
        return False
    out = ctypes.c_int(0)
    _lib.check("esep_head_step_path_taken", _lib.load().esep_head_step_path_taken(
        _ptr(ws), _stream(ws.device), ctypes.byref(out)))
    return out.value != 0


def last_call_fell_back(device=None):
    """True if the most recent call on the device raised its overflow flag (single pass or stored
    weights), i.e. its outputs came from the guarded two-kernel path. Synchronises (a test /
    monitoring aid)."""
    device = torch.device("cuda" if device is None else device)
    index = torch.cuda.current_device() if device.index is None else device.index
    with _state_lock:
        flag = _last_overflow.get(index)
    return bool(flag.item()) if flag is not None else False


class _Bf16Copies:
    """bf16 copy of a frozen 16-bit head weight for the single pass's dHidden GEMM, one entry per
    device, keyed like the reference's fp16 weight cache (patch.py:93-101: data pointer, shape,
    dtype, version counter). The entry also HOLDS the source tensor: while it is cached its
    memory cannot be freed and handed to another tensor, so an equal key always means the same
    weight (a key on the address alone would match a new tensor that reuses a freed address).
    Cost: a weight the caller has dropped stays alive until another weight replaces it."""

    def __init__(self):
        self.lock = threading.Lock()
        self.entries = {}

    def get(self, w16):
        if w16.dtype == torch.bfloat16:
            return w16
        key = (w16.data_ptr(), tuple(w16.shape), w16.dtype, w16._version)
        with self.lock:
            hit = self.entries.get(w16.device.index)
            if hit is not None and hit[0] == key:
                return hit[2]
        with torch.no_grad():
            copy = w16.detach().to(torch.bfloat16)
        with self.lock:
            self.entries[w16.device.index] = (key, w16, copy)
        return copy

    def clear(self):
        with self.lock:
            self.entries.clear()


_bf16_copies = _Bf16Copies()


def _bf16_weight(w16):
    return _bf16_copies.get(w16)


def _run_step(x, w16, need_grad, target=None, ce_weight=None, labels=None, attention_mask=None,
              seq_len=0, w_bf16=None, want_top=False):
    """One ``esep_head_step`` call. x: [m, h] contiguous in w16's dtype or fp32. Flat rows
    (target, ce_weight) or a [m / seq_len, seq_len] step (labels, attention_mask). Returns a
    dict of views: the five statistics, "cew", "loss" [1], "metrics" [8], "dx" (or None) and
    "overflow" (device int32 [1]); with want_top also "top", the largest logit of every row."""
    lib = _lib.load()
    dev = x.device
    m, h = x.shape
    v = w16.shape[0]
    dtype = _DTYPES[w16.dtype]
    with torch.cuda.device(dev):
        nbytes = lib.esep_head_step_workspace_bytes(m, h, v, dtype, int(need_grad))
        if nbytes == 0:
            code, _ = _lib.query(dev.index)
            _lib.check("esep_head_query", code)
            raise _lib.HeadLibraryError("esep_head_step_workspace_bytes", -1, "no plan for this size")
        ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
        f = torch.empty(6 * m + 1 + _lib.STEP_SCALARS, device=dev, dtype=torch.float32)
        out = {"lse": f[0:m], "target_logit": f[m:2 * m], "ce": f[2 * m:3 * m],
               "entropy": f[3 * m:4 * m], "cew": f[4 * m:5 * m], "top": f[5 * m:6 * m],
               "loss": f[6 * m:6 * m + 1], "metrics": f[6 * m + 1:],
               "argmax": torch.empty(m, device=dev, dtype=torch.int64),
               "dx": torch.empty(m, h, device=dev, dtype=torch.float32) if need_grad else None}
        overflow = ws[96:100].view(torch.int32)
        # a bf16 copy of W (467 MB for the 1.5B shape) is read by the single pass (0) and, for an
        # fp16 model, by the two sweeps that keep bf16 softmax weights (2)
        if need_grad and w_bf16 is None:
            kind = lib.esep_head_step_uses_stored_logits(m, h, v, dtype, 1)
            if kind == 0 or (kind == 2 and w16.dtype == torch.float16):
                w_bf16 = _bf16_weight(w16)
        code = lib.esep_head_step(
            _ptr(x), _X_DTYPES[x.dtype], _ptr(w16), _ptr(w_bf16), dtype, m, h, v, _ptr(target),
            _ptr(ce_weight), _ptr(labels), _ptr(attention_mask), int(seq_len), int(need_grad),
            _ptr(out["lse"]), _ptr(out["target_logit"]), _ptr(out["ce"]), _ptr(out["entropy"]),
            _ptr(out["argmax"]), _ptr(out["cew"]), _ptr(out["loss"]), _ptr(out["metrics"]),
            _ptr(out["dx"]), _ptr(out["top"]) if want_top else None, None, _ptr(ws), ws.numel(),
            _stream(dev))
    _lib.check("esep_head_step", code)
    out["overflow"] = overflow
    _remember(dev, ws, overflow)
    return out


def _scale_grad(dx, grad_loss, dtype):
    """(dx * grad_loss).to(dtype) in one library kernel (op.py:143-145); grad_loss stays on the
    device."""
    out = torch.empty(dx.shape, device=dx.device, dtype=dtype)
    g = grad_loss.detach().to(device=dx.device, dtype=torch.float32).reshape(1)
    with torch.cuda.device(dx.device):
        code = _lib.load().esep_head_grad_scale(_ptr(dx), _ptr(g), dx.numel(), _X_DTYPES[dtype],
                                                _ptr(out), _stream(dx.device))
    _lib.check("esep_head_grad_scale", code)
    return out


def _prepare(x, w16, target, ce_weight):
    x16 = x.to(w16.dtype).contiguous()                       # op.py:109
    target = target.to(torch.int64).contiguous()
    cew = ce_weight.to(torch.float32).contiguous()
    return x16, target, cew


def _two_kernel(x, w16, target, cew):
    """Forward sweep + recomputing backward sweep over all rows (SINGLE_SWEEP = False)."""
    x16 = x.to(w16.dtype).contiguous()
    be = DeviceBackend(x16, w16, True)
    rec = be.forward_partial(x16, w16, target, 0)
    out = be.finalize(rec, target, cew, w16.shape[0])
    out["dx"] = be.backward(x16, w16, target, out["cew"], out["lse"], 0)
    return out


def _forward(x, w16, target, ce_weight, need_grad, chunk_rows=CHUNK_ROWS):
    """Counterpart of op.py:104-128. Returns (loss, (lse, tlogit, ce, ent, argmax), dx, metrics)."""
    del chunk_rows  # no chunk buffer exists
    x = x.contiguous()
    target = target.to(torch.int64).contiguous()
    cew = ce_weight.to(torch.float32).contiguous()
    if need_grad and not SINGLE_SWEEP:
        out = _two_kernel(x, w16, target, cew)
    else:
        out = _run_step(x, w16, need_grad, target=target, ce_weight=cew)
    stats = tuple(out[k] for k in _KEYS)
    return out["loss"].reshape(()), stats, out["dx"], out["metrics"]


class FusedLinearCE(torch.autograd.Function):
    """Loss is differentiable w.r.t. x; dX is computed in the forward (reference: op.py:131-145)."""

    @staticmethod
    def forward(ctx, x, w16, target, ce_weight, chunk_rows):
        loss, stats, dx, metrics = _forward(x, w16, target, ce_weight, True, chunk_rows)
        ctx.save_for_backward(dx)
        ctx.x_dtype = x.dtype
        ctx.set_materialize_grads(False)   # no zero tensors for the outputs without gradient
        ctx.mark_non_differentiable(*stats, metrics)
        return (loss, *stats, metrics)

    @staticmethod
    def backward(ctx, grad_loss, *unused):
        (dx,) = ctx.saved_tensors
        return _scale_grad(dx, grad_loss, ctx.x_dtype), None, None, None, None


def fused_linear_ce_with_metrics(x, w16, target, ce_weight, need_grad=None,
                                 chunk_rows=CHUNK_ROWS):
    """``fused_linear_ce`` plus the scalars the kernels reduce on the way, as a device tensor
    (no synchronisation): [loss_sum, n_valid, n_correct, entropy_sum over valid rows, ...]
    (include/esep_head.h: ESEP_STEP_SCALARS). They stand for the sums behind the reference's
    metric logging (patch.py:582-615); a data-parallel job all-reduces this one tensor."""
    assert x.dim() == 2 and w16.dim() == 2 and x.shape[1] == w16.shape[1], "shape mismatch"
    assert w16.dtype in _DTYPES, "w16 must be fp16 or bf16"
    assert x.dtype in (w16.dtype, torch.float32), "x must be fp32 or match w16's 16-bit dtype"
    assert target.shape == (x.shape[0],) and ce_weight.shape == (x.shape[0],)
    assert x.is_cuda and w16.is_cuda
    assert x.shape[1] % 8 == 0, "hidden size must be a multiple of 8 (16-byte TMA rows)"
    if need_grad is None:
        need_grad = torch.is_grad_enabled() and x.requires_grad
    w16 = w16.contiguous()
    target = target.to(torch.int64)
    if not x.shape[0]:                                        # op.py:166-169
        z = torch.zeros(0, device=x.device, dtype=torch.float32)
        loss = x.float().sum() * 0.0 if need_grad else z.sum()
        return (loss, dict(zip(_KEYS, (z, z, z, z, z.long()))),
                torch.zeros(_lib.STEP_SCALARS, device=x.device, dtype=torch.float32))
    if need_grad:
        loss, *rest = FusedLinearCE.apply(x, w16, target, ce_weight, chunk_rows)
        stats, metrics = rest[:-1], rest[-1]
    else:
        with torch.no_grad():
            loss, stats, _, metrics = _forward(x, w16, target, ce_weight, False, chunk_rows)
    return loss, dict(zip(_KEYS, stats)), metrics


def fused_linear_ce(x, w16, target, ce_weight, need_grad=None, chunk_rows=CHUNK_ROWS):
    """loss = sum_i ce_weight_i * CE(x_i @ w16^T, target_i), plus per-token stats (module doc).

    need_grad=None means: grad mode is on and x requires grad (op.py:162-163). Without a gradient
    only the forward sweep runs. Same checks as the reference (op.py:157-161), widened to bf16."""
    loss, stats, _ = fused_linear_ce_with_metrics(x, w16, target, ce_weight, need_grad, chunk_rows)
    return loss, stats
