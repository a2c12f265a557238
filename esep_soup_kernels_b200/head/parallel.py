"""Multi-GPU forms of the fused LM head on torch.distributed (one process per GPU).

The reference is single-GPU (its harness pins one device, harness/common.py:39-41); these two
sharded forms are additions built from the same C entry points:

token-sharded   rows of x are split across ranks, W is replicated. Every row's loss, stats and
                dHidden depend only on that row and W, so there is NO data-path collective; the
                ranks exchange one 4-float all-reduce {loss, n_valid, n_correct, entropy_sum}
                (it stands for the five metric gathers of solution/head/patch.py:594-612).
vocab-parallel  W is split by vocabulary rows, every rank holds all rows of x. With a gradient
                every rank runs the single pass on its shard as a vocabulary of its own, the
                ranks all-gather one [5, N] record each, a combine kernel turns the local
                results into the rank's share of the global ones and the shares of dHidden
                are summed with an all-reduce: the only torch calls on the way are the two
                collectives. Without the single pass (or without gradient): forward sweep into a
                per-row record (m, s, t, target logit, argmax), all-gather, merge with the rule
                of solution/head/kernels.py:70-81, backward sweep per shard, all-reduce. With
                dx_chunks > 1 that backward sweep runs row group by row group and the all-reduce
                of a finished group runs (asynchronously, on the collective's own stream) while
                the next group is swept.

Both take a `backend_factory` so that the host logic (sharding, exchange, merge order) can be
exercised with CPU ranks on the gloo backend in the tests; the default is the CUDA library.
"""

import torch
import torch.distributed as dist

from . import _lib, op
from .op import _KEYS, DeviceBackend, _prepare


class RankLostError(RuntimeError):
    """A rank of the group is gone: it announced that it left (RankRoster), or a collective of
    the sharded forms failed or ran into the process group's timeout."""


class RankRoster:
    """Host-side roll call through a torch.distributed store (no GPU work, no collective).

    A rank that stops taking part BETWEEN steps calls ``leave()``; the others call ``check()``
    before they launch their next step and get a RankLostError naming the rank instead of
    entering a collective that would never complete. A rank that disappears without announcing
    it is caught by the collective itself (``_collective``), bounded by the group's timeout."""

    def __init__(self, store, rank, world, prefix="esep_head_roster"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def leave(self):
        self.store.set(f"{self.prefix}/left/{self.rank}", b"1")

    def check(self):
        gone = [r for r in range(self.world)
                if r != self.rank and self.store.check([f"{self.prefix}/left/{r}"])]
        if gone:
            raise RankLostError(f"rank(s) {gone} left the group")


def _collective(fn, *args, **kwargs):
    """Runs a torch.distributed collective; a failure (peer gone, timeout) surfaces as
    RankLostError instead of a backend-specific exception."""
    try:
        return fn(*args, **kwargs)
    except RankLostError:
        raise
    except RuntimeError as e:   # DistBackendError, gloo connection errors, timeouts
        raise RankLostError(f"collective {getattr(fn, '__name__', fn)} failed: {e}") from e


def shard_bounds(total, world, rank):
    """[lo, hi) of `rank`'s contiguous shard of `total` items, sizes differing by at most 1."""
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _default_backend(x16, w16, need_grad):
    return DeviceBackend(x16, w16, need_grad)


def token_sharded_linear_ce(x_local, w16, target_local, ce_weight_local, need_grad=True,
                            group=None, backend_factory=_default_backend):
    """This rank's rows through the head, plus the globally reduced metric scalars.

    Returns (loss_local, stats_local, dx_local, metrics) where metrics holds, summed over all
    ranks, {loss, valid rows, correct rows, sum of entropy over valid rows} followed (library
    path) by the four further scalars of a step (include/esep_head.h: ESEP_STEP_SCALARS).
    loss_local / dx_local are this rank's own (dHidden never leaves the row owner)."""
    x16, target, cew = _prepare(x_local, w16, target_local, ce_weight_local)
    be = None if backend_factory is _default_backend else backend_factory(x16, w16, need_grad)
    if be is None and (op.SINGLE_SWEEP or not need_grad):
        # one library call for this rank's rows (the whole W is local); eight scalars
        out = op._run_step(x16, w16, need_grad, target=target, ce_weight=cew)
        dx = out["dx"]
    elif be is not None and need_grad and op.SINGLE_SWEEP and hasattr(be, "train"):
        out = be.train(x16, w16, op._bf16_weight(w16), target, cew)
        dx = out["dx"]
    else:
        be = be if be is not None else backend_factory(x16, w16, need_grad)
        rec = be.forward_partial(x16, w16, target, 0)
        out = be.finalize(rec, target, cew, w16.shape[0])
        dx = be.backward(x16, w16, target, out["cew"], out["lse"], 0) if need_grad else None
    metrics = out["metrics"].clone()
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        _collective(dist.all_reduce, metrics, op=dist.ReduceOp.SUM, group=group)
    stats = {k: out[k] for k in _KEYS}
    return out["loss"].reshape(()), stats, dx, metrics


def row_groups(n, chunks, align=128):
    """Cuts [0, n) into at most `chunks` contiguous groups whose sizes are multiples of `align`
    (row tiles stay whole), the last one taking the remainder."""
    tiles = -(-n // align)
    chunks = max(1, min(int(chunks), tiles))
    out = []
    for k in range(chunks):
        lo, hi = shard_bounds(tiles, chunks, k)
        if hi > lo:
            out.append((lo * align, min(hi * align, n)))
    return out


def _mark(timings, name, device):
    """Records a CUDA event named `name` on the current stream (timings: list or None)."""
    if timings is not None and device.type == "cuda":
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(device))
        timings.append((name, ev))


def _vocab_parallel_sweep(be, x16, w_shard, target, cew, vocab_offset, v_global, world, group,
                          reduce_dx, timings=None):
    """Vocab-parallel training call built on the single pass (formulas: csrc/head_aux.cuh).
    Backend calls: vp_prepare (local targets, unit weights) -> train (local sweep) -> vp_pack
    (this rank's [5, n] record) -> all-gather -> vp_combine (global statistics, this rank's share
    of dHidden, in place) -> all-reduce."""
    dev = x16.device
    v_local = w_shard.shape[0]
    _mark(timings, "start", dev)
    local_target, ones = be.vp_prepare(target, int(vocab_offset), v_local, int(v_global))
    out = be.train(x16, w_shard, op._bf16_weight(w_shard), local_target, ones)
    rec = be.vp_pack(out, target, int(vocab_offset), v_local, int(v_global))
    _mark(timings, "sweep", dev)
    if world > 1:
        allrec = torch.empty((world,) + tuple(rec.shape), device=rec.device, dtype=rec.dtype)
        _collective(dist.all_gather_into_tensor, allrec.view(-1), rec.view(-1), group=group)
        me = dist.get_rank(group)
    else:
        allrec, me = rec.unsqueeze(0), 0
    _mark(timings, "exchange", dev)
    res = be.vp_combine(allrec, me, target, cew, w_shard, int(vocab_offset), int(v_global),
                        out["dx"])
    _mark(timings, "combine", dev)
    dx = out["dx"]
    if world > 1 and reduce_dx:
        _collective(dist.all_reduce, dx, op=dist.ReduceOp.SUM, group=group)
    _mark(timings, "reduce", dev)
    stats = {k: res[k] for k in _KEYS}
    return res["loss"].reshape(()), stats, dx, res["metrics"]


def vocab_parallel_linear_ce(x, w_shard, target, ce_weight, vocab_offset, v_global,
                             need_grad=True, group=None, backend_factory=_default_backend,
                             reduce_dx=True, dx_chunks=1, dx_align=128, single_sweep=None,
                             timings=None):
    """Full-vocabulary loss / stats / dHidden from a vocabulary-sharded weight.

    x, target (GLOBAL ids), ce_weight are replicated on every rank; `w_shard` holds vocabulary rows
    [vocab_offset, vocab_offset + w_shard.shape[0]). Returns (loss, stats, dx): identical on every
    rank (dx is the all-reduced sum of the shard contributions unless reduce_dx=False).
    dx_chunks > 1 overlaps that all-reduce with the backward sweep, row group by row group
    (group sizes are multiples of dx_align rows, the row tile of the backward kernel).
    single_sweep (default: on when the backend has it, a gradient is wanted and dx_chunks == 1):
    each shard runs the single-sweep training kernel and the results are combined after one
    all-gather (_vocab_parallel_sweep); otherwise forward sweep -> record exchange -> backward.
    timings: a list that receives (name, CUDA event) marks at the phase boundaries of the sweep
    form (start, sweep, exchange, combine, reduce)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    x16, target, cew = _prepare(x, w_shard, target, ce_weight)
    be = backend_factory(x16, w_shard, need_grad)
    if single_sweep is None:
        single_sweep = op.SINGLE_SWEEP and need_grad and dx_chunks == 1 and hasattr(be, "train")
    if single_sweep:
        loss, stats, dx, _ = _vocab_parallel_sweep(be, x16, w_shard, target, cew, vocab_offset,
                                                   v_global, world, group, reduce_dx, timings)
        return loss, stats, dx
    rec = be.forward_partial(x16, w_shard, target, int(vocab_offset))
    if world > 1:
        # records are ordered by rank; ties between shards resolve to the lowest global index
        # inside the merge (argmax field carries global ids), so the order does not matter
        parts = [torch.empty_like(rec) for _ in range(world)]
        _collective(dist.all_gather, parts, rec.contiguous(), group=group)
        gathered = torch.stack(parts)
    else:
        gathered = rec.unsqueeze(0)
    out = be.finalize(gathered, target, cew, int(v_global))
    dx = None
    if need_grad and dx_chunks > 1 and world > 1 and reduce_dx:
        n = x16.shape[0]
        dx = torch.empty(n, x16.shape[1], device=x16.device, dtype=torch.float32)
        pending = []
        for lo, hi in row_groups(n, dx_chunks, dx_align):
            sub = be if (lo, hi) == (0, n) else backend_factory(x16[lo:hi], w_shard, True)
            view = dx[lo:hi]
            args = (x16[lo:hi], w_shard, target[lo:hi], out["cew"][lo:hi], out["lse"][lo:hi],
                    int(vocab_offset))
            if getattr(sub, "accepts_out", False):
                sub.backward(*args, out=view)
            else:
                view.copy_(sub.backward(*args))
            # the collective starts when this group is complete and runs beside the next sweep
            pending.append(_collective(dist.all_reduce, view, op=dist.ReduceOp.SUM, group=group,
                                       async_op=True))
        for work in pending:
            _collective(work.wait)
    elif need_grad:
        dx = be.backward(x16, w_shard, target, out["cew"], out["lse"], int(vocab_offset))
        if world > 1 and reduce_dx:
            _collective(dist.all_reduce, dx, op=dist.ReduceOp.SUM, group=group)
    stats = {k: out[k] for k in _KEYS}
    return out["loss"].reshape(()), stats, dx


__all__ = ["shard_bounds", "row_groups", "token_sharded_linear_ce", "vocab_parallel_linear_ce",
           "RankLostError", "RankRoster", "_lib"]
