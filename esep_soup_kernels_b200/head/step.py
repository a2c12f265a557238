"""The head part of a causal-LM training step in one library call.

``loss, step = causal_lm_head_step(hidden, labels, w16, attention_mask)`` covers what the
reference does around its op in ``_fused_causal_lm_forward`` (solution/head/patch.py:443-487):
shift the labels by one position, keep the rows that are attended or carry a target, gather
them, run the head, normalise the loss, scatter the per-row CE and entropy back to (B, T) and
count correct / labelled tokens. Here none of that is torch glue: ``esep_head_step`` takes
``hidden [B*T, H]``, ``labels`` and ``attention_mask`` as they are, builds targets and the row
list on the device, and its kernels write per-token loss / entropy straight at their (b, t)
position (zeros elsewhere), dHidden straight into a [B*T, H] buffer (zero rows where there is no
gradient) and the counters into one small tensor. No ``nonzero()``, no host synchronisation.

``step_metrics`` turns the counters into the three numbers the reference's trainer logs
(patch.py:582-615); across data-parallel ranks they travel in ONE all-reduce of eight floats
(the reference gathers five scalars separately).
"""

import torch
import torch.distributed as dist

from . import _lib
from .op import _DTYPES, _run_step, _scale_grad

IGNORE_INDEX = -100

# positions in the scalar vector of a step (include/esep_head.h: ESEP_STEP_SCALARS)
LOSS_SUM, N_VALID, N_CORRECT, ENT_VALID, N_LABELLED, N_ATTENDED, ENT_ATTENDED, N_LIVE = range(8)


class HeadStep:
    """Detached per-token results of one head step (the reference's HeadStep, patch.py:73-82):
    ``token_loss`` / ``token_entropy`` fp32 (B, T), zero where a position has no target / is not
    a selected row; ``correct`` / ``labelled`` 0-dim int64; ``sums`` the eight fp32 scalars the
    kernels reduced (device tensor)."""

    __slots__ = ("token_loss", "token_entropy", "sums")

    def __init__(self, token_loss, token_entropy, sums):
        self.token_loss = token_loss
        self.token_entropy = token_entropy
        self.sums = sums

    @property
    def correct(self):
        return self.sums[N_CORRECT].long()

    @property
    def labelled(self):
        return self.sums[N_LABELLED].long()


class HeadWeight:
    """16-bit copy of a frozen LM-head weight for callers whose parameter is stored wider,
    rebuilt when the parameter's memory, shape, dtype, device or version counter changes (the job
    of the reference's ``_HeadState.weight16``, patch.py:93-101). The entry keeps the source
    tensor alive, so a freed-and-reused address can never pass for the old weight."""

    def __init__(self, dtype=torch.float16):
        assert dtype in _DTYPES
        self.dtype = dtype
        self._src = None
        self._key = None
        self._w16 = None

    def weight16(self, weight):
        key = (weight.data_ptr(), tuple(weight.shape), weight.dtype, weight.device, weight._version)
        if self._w16 is None or key != self._key:
            with torch.no_grad():
                self._w16 = weight.detach().to(self.dtype).contiguous()
            self._key, self._src = key, weight
        return self._w16


class _HeadStepFn(torch.autograd.Function):
    """d loss / d hidden is produced by the forward call; backward scales it (op.py:131-145)."""

    @staticmethod
    def forward(ctx, hidden2d, w16, labels, attention_mask, seq_len):
        out = _run_step(hidden2d, w16, True, labels=labels, attention_mask=attention_mask,
                        seq_len=seq_len)
        ctx.save_for_backward(out["dx"])
        ctx.x_dtype = hidden2d.dtype
        ctx.set_materialize_grads(False)   # no zero tensors for the outputs without gradient
        rest = (out["ce"], out["entropy"], out["metrics"])
        ctx.mark_non_differentiable(*rest)
        return (out["loss"].reshape(()), *rest)

    @staticmethod
    def backward(ctx, grad_loss, *unused):
        (dx,) = ctx.saved_tensors
        return _scale_grad(dx, grad_loss, ctx.x_dtype), None, None, None, None


def causal_lm_head_step(hidden, labels, w16, attention_mask=None, num_items_in_batch=None,
                        need_grad=None):
    """hidden [B, T, H] (output of the final norm; w16's dtype or fp32), labels [B, T]
    -> (loss, HeadStep).

    loss = (sum of CE over valid targets) / num_items_in_batch, or the mean over valid targets
    when num_items_in_batch is None (patch.py:461-468). A 2-D attention_mask selects the rows
    that get statistics (attended or labelled, patch.py:449-452); without one every row does."""
    assert hidden.dim() == 3 and labels.shape == hidden.shape[:2], "hidden [B, T, H], labels [B, T]"
    assert w16.dim() == 2 and w16.dtype in _DTYPES and hidden.shape[2] == w16.shape[1]
    assert hidden.dtype in (w16.dtype, torch.float32), "hidden must be fp32 or w16's dtype"
    assert hidden.is_cuda and w16.is_cuda and hidden.shape[2] % 8 == 0
    bsz, seq, hid = hidden.shape
    dev = hidden.device
    if need_grad is None:
        need_grad = torch.is_grad_enabled() and hidden.requires_grad
    w16 = w16.contiguous()
    labels = labels.to(device=dev, dtype=torch.int64).contiguous()
    mask = None
    if attention_mask is not None and attention_mask.dim() == 2:
        mask = attention_mask.to(device=dev, dtype=torch.int64).contiguous()
    if bsz * seq == 0:
        z = torch.zeros(bsz, seq, device=dev, dtype=torch.float32)
        sums = torch.zeros(_lib.STEP_SCALARS, device=dev, dtype=torch.float32)
        return hidden.float().sum() * 0.0, HeadStep(z, z.clone(), sums)
    hidden2d = hidden.reshape(bsz * seq, hid)
    if not hidden2d.is_contiguous():
        hidden2d = hidden2d.contiguous()
    if need_grad:
        loss_sum, ce, ent, sums = _HeadStepFn.apply(hidden2d, w16, labels, mask, seq)
    else:
        with torch.no_grad():
            out = _run_step(hidden2d, w16, False, labels=labels, attention_mask=mask, seq_len=seq)
        loss_sum, ce, ent, sums = out["loss"].reshape(()), out["ce"], out["entropy"], out["metrics"]
    if num_items_in_batch is None:
        loss = loss_sum / sums[N_LABELLED]
    else:
        if torch.is_tensor(num_items_in_batch):
            num_items_in_batch = num_items_in_batch.to(loss_sum.device)
        loss = loss_sum / num_items_in_batch
    return loss, HeadStep(ce.view(bsz, seq), ent.view(bsz, seq), sums)


def step_sums(step, group=None):
    """The step's eight scalars summed over the ranks of ``group`` (one all-reduce; no host
    synchronisation). Without an initialised process group: the local scalars."""
    sums = step.sums
    if group is not None or (dist.is_available() and dist.is_initialized()
                             and dist.get_world_size() > 1):
        sums = sums.clone()
        dist.all_reduce(sums, group=group)
    return sums


def step_metrics(step, attention_mask=None, group=None):
    """The three numbers TRL logs from a step (patch.py:582-615): mean entropy over attended
    tokens, number of attended tokens, mean token accuracy - from the scalars the kernels
    already reduced, with ONE host read (the reference does five gathers and five reads).
    ``attention_mask`` is accepted for signature compatibility; the mask given to
    ``causal_lm_head_step`` is what the scalars were reduced under."""
    del attention_mask
    s = step_sums(step, group).tolist()
    tok, labelled = s[N_ATTENDED], s[N_LABELLED]
    return {"entropy": s[ENT_ATTENDED] / tok if tok > 0 else 0.0, "num_tokens": int(tok),
            "mean_token_accuracy": s[N_CORRECT] / labelled if labelled > 0 else 0.0}
