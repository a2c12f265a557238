"""World-size-2 CPU (gloo) tests of the sharded host logic in head/parallel.py: row / vocabulary
sharding, the record all-gather + merge, the dHidden all-reduce and the metric all-reduce. The
per-rank compute is done by an oracle-backed stand-in defined HERE (tests only); the product's
default backend is the CUDA library."""

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleBackend:
    """CPU stand-in with the DeviceBackend interface, built on oracle/head_oracle.py."""

    def __init__(self, x16, w16, need_grad):
        from oracle import head_oracle as ho

        self.ho = ho

    def forward_partial(self, x16, w16, target, vocab_offset=0):
        return torch.from_numpy(self.ho.partial_record(x16, w16, target, vocab_offset))

    def finalize(self, records, target, ce_weight, v_global):
        rec = records.numpy() if records.dim() == 3 else records.numpy()[None]
        f = self.ho.finalize_records(rec, target.numpy(), ce_weight.numpy(), v_global)
        t = torch.from_numpy
        return {"lse": t(f["lse"]), "target_logit": t(f["target_logit"]), "ce": t(f["ce"]),
                "entropy": t(f["entropy"]), "argmax": t(f["argmax"]), "cew": t(f["cew"]),
                "loss": torch.tensor([f["loss"]], dtype=torch.float32),
                "metrics": torch.tensor(f["metrics"], dtype=torch.float32)}

    def backward(self, x16, w16, target, cew, lse, vocab_offset=0):
        return self.ho.shard_dx(x16, w16, target, cew, lse, vocab_offset)


class OracleSweepBackend(OracleBackend):
    """Adds the single-sweep call (statistics and dHidden of the local vocabulary in one go) and a
    torch restatement of the three small kernels around it (csrc/head_aux.cuh: prepare, pack,
    combine), so that the exchange logic of parallel.py runs on CPU ranks."""

    def train(self, x16, w16, w_bf16, target, ce_weight):
        r = self.ho.full_vocab_reference(x16, w16, target, ce_weight, want_rounded=False)
        valid = (target >= 0) & (target < w16.shape[0])
        zero = torch.zeros_like(r["lse"])
        top = (x16.float() @ w16.float().T).max(-1).values
        return {"lse": r["lse"], "target_logit": torch.where(valid, r["tlogit"], zero),
                "ce": torch.where(valid, r["lse"] - r["tlogit"], zero), "entropy": r["ent"],
                "argmax": r["argmax"], "cew": torch.where(valid, ce_weight.float(), zero),
                "loss": r["loss"].reshape(1), "metrics": torch.zeros(4), "dx": r["dx"].clone(),
                "top": top, "overflow": torch.zeros(1, dtype=torch.int32)}

    def vp_prepare(self, target, vocab_offset, v_local, v_global):
        valid = (target >= 0) & (target < v_global)
        t_loc = target - vocab_offset
        owner = valid & (t_loc >= 0) & (t_loc < v_local)
        local = torch.where(owner, t_loc, torch.where(valid, torch.zeros_like(t_loc),
                                                      torch.full_like(t_loc, -100)))
        return local, valid.to(torch.float32)

    def vp_pack(self, out, target, vocab_offset, v_local, v_global):
        t_loc = target - vocab_offset
        owner = (target >= 0) & (target < v_global) & (t_loc >= 0) & (t_loc < v_local)
        idx = (out["argmax"] + vocab_offset).to(torch.int32).view(torch.float32)
        return torch.stack([out["lse"], out["entropy"], out["top"],
                            torch.where(owner, out["target_logit"], torch.zeros_like(out["top"])),
                            idx])

    def vp_combine(self, records, me, target, ce_weight, w_shard, vocab_offset, v_global, dx):
        lse_k, ent_k, top_k, tz_k = records[:, 0], records[:, 1], records[:, 2], records[:, 3]
        idx_k = records[:, 4].contiguous().view(torch.int32).to(torch.int64)
        lse = torch.logsumexp(lse_k, 0)
        a_k = torch.exp(lse_k - lse)
        entropy = lse - (a_k * (lse_k - ent_k)).sum(0)
        best = top_k.max(0).values
        argmax = torch.where(top_k == best, idx_k, torch.full_like(idx_k, 2 ** 62)).min(0).values
        valid = (target >= 0) & (target < v_global)
        tz = tz_k.sum(0)
        zero = torch.zeros_like(lse)
        ce = torch.where(valid, lse - tz, zero)
        cw = torch.where(valid, ce_weight.float(), zero)
        t_loc = target - vocab_offset
        owner = valid & (t_loc >= 0) & (t_loc < w_shard.shape[0])
        a_me = a_k[me]
        a_rest = a_k.sum(0) - a_me
        coef = torch.where(owner, -a_rest, a_me)
        w_t = w_shard.index_select(0, torch.where(owner, t_loc, torch.zeros_like(t_loc))).float()
        dx.mul_(a_me[:, None]).add_(w_t * coef[:, None]).mul_(cw[:, None])
        loss = (cw * ce).sum().reshape(1)
        metrics = torch.stack([loss[0], valid.sum().float(),
                               ((argmax == target) & valid).sum().float(),
                               torch.where(valid, entropy, zero).sum()])
        return {"lse": lse, "target_logit": torch.where(valid, tz, zero), "ce": ce,
                "entropy": entropy, "argmax": argmax, "cew": cw, "loss": loss, "metrics": metrics}


def _inputs():
    g = torch.Generator().manual_seed(11)
    n, h, v = 61, 64, 1003
    w = (torch.randn(v, h, generator=g) * 0.3).half()
    x = torch.randn(n, h, generator=g).half()
    t = torch.randint(0, v, (n,), generator=g)
    t[::6] = -100
    c = torch.rand(n, generator=g)
    return x, w, t, c


def _worker(rank, world, port, mode, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from esep_soup_kernels_b200.head import parallel as par

    x, w, t, c = _inputs()
    factory = lambda x16, w16, ng: (OracleSweepBackend if mode == "vocab_sweep" else OracleBackend)(
        x16, w16, ng)
    if mode == "token":
        lo, hi = par.shard_bounds(x.shape[0], world, rank)
        loss, stats, dx, metrics = par.token_sharded_linear_ce(
            x[lo:hi], w, t[lo:hi], c[lo:hi], backend_factory=factory)
        np.savez(os.path.join(out_dir, f"r{rank}.npz"), lo=lo, hi=hi, loss=loss.numpy(),
                 dx=dx.numpy(), metrics=metrics.numpy(), lse=stats["lse"].numpy(),
                 argmax=stats["argmax"].numpy())
    else:
        lo, hi = par.shard_bounds(w.shape[0], world, rank)
        loss, stats, dx = par.vocab_parallel_linear_ce(
            x, w[lo:hi], t, c, lo, w.shape[0], backend_factory=factory,
            dx_chunks=3 if mode == "vocab_chunked" else 1, dx_align=16)
        np.savez(os.path.join(out_dir, f"r{rank}.npz"), lo=lo, hi=hi, loss=loss.numpy(),
                 dx=dx.numpy(), lse=stats["lse"].numpy(), ent=stats["entropy"].numpy(),
                 argmax=stats["argmax"].numpy(), ce=stats["ce"].numpy())
    dist.barrier()
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(mode, tmp_path, world=2):
    for attempt in range(2):   # the probed port can be taken before the ranks bind it: retry once
        try:
            mp.spawn(_worker, args=(world, _free_port(), mode, str(tmp_path)), nprocs=world,
                     join=True)
            break
        except Exception:
            if attempt:
                raise
    return [dict(np.load(os.path.join(tmp_path, f"r{r}.npz"))) for r in range(world)]


def test_shard_bounds_partition_everything():
    from esep_soup_kernels_b200.head.parallel import shard_bounds

    for total in (0, 1, 7, 64, 151936):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1


@pytest.mark.timeout(300)
def test_token_sharded_world2_matches_single_process(tmp_path):
    from oracle import head_oracle as ho

    x, w, t, c = _inputs()
    ref = ho.full_vocab_reference(x, w, t, c, want_rounded=False)
    outs = _run("token", tmp_path)
    assert outs[0]["hi"] == outs[1]["lo"] and outs[1]["hi"] == x.shape[0]
    dx = np.concatenate([o["dx"] for o in outs])
    lse = np.concatenate([o["lse"] for o in outs])
    np.testing.assert_allclose(dx, ref["dx"].numpy(), rtol=1e-3, atol=1e-6)
    np.testing.assert_allclose(lse, ref["lse"].numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(sum(float(o["loss"]) for o in outs), float(ref["loss"]), rtol=1e-5)
    valid = (t >= 0)
    for o in outs:                                   # every rank holds the same global scalars
        np.testing.assert_allclose(o["metrics"][0], float(ref["loss"]), rtol=1e-5)
        assert o["metrics"][1] == float(valid.sum())
        assert o["metrics"][2] == float(((ref["argmax"] == t) & valid).sum())
        np.testing.assert_allclose(o["metrics"][3], float(ref["ent"][valid].sum()), rtol=1e-4)


@pytest.mark.timeout(300)
def test_vocab_parallel_world2_matches_single_process(tmp_path):
    from oracle import head_oracle as ho

    x, w, t, c = _inputs()
    ref = ho.full_vocab_reference(x, w, t, c, want_rounded=False)
    outs = _run("vocab", tmp_path)
    assert outs[0]["hi"] == outs[1]["lo"] and outs[1]["hi"] == w.shape[0]
    for o in outs:
        np.testing.assert_allclose(float(o["loss"]), float(ref["loss"]), rtol=1e-5)
        np.testing.assert_allclose(o["lse"], ref["lse"].numpy(), rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(o["ent"], ref["ent"].numpy(), rtol=1e-4, atol=1e-4)
        assert (o["argmax"] == ref["argmax"].numpy()).all()
        np.testing.assert_allclose(o["dx"], ref["dx"].numpy(), rtol=1e-3, atol=1e-6)
    assert np.array_equal(outs[0]["dx"], outs[1]["dx"])


@pytest.mark.timeout(300)
def test_vocab_parallel_chunked_reduction_is_the_same_result(tmp_path):
    """dx_chunks > 1 (row groups reduced while the next group is swept) changes no value."""
    (tmp_path / "plain").mkdir()
    (tmp_path / "chunked").mkdir()
    plain = _run("vocab", tmp_path / "plain")
    chunked = _run("vocab_chunked", tmp_path / "chunked")
    for a, b in zip(plain, chunked):
        assert np.array_equal(a["dx"], b["dx"])
        assert np.array_equal(a["lse"], b["lse"])


def test_row_groups_keep_row_tiles_whole():
    from esep_soup_kernels_b200.head.parallel import row_groups

    assert row_groups(300, 3) == [(0, 128), (128, 256), (256, 300)]
    assert row_groups(300, 8) == [(0, 128), (128, 256), (256, 300)]
    assert row_groups(100, 4) == [(0, 100)]
    assert row_groups(1024, 2) == [(0, 512), (512, 1024)]
    got = row_groups(4340, 5)
    assert got[0][0] == 0 and got[-1][1] == 4340
    assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
    assert all(lo % 128 == 0 for lo, _ in got)


@pytest.mark.timeout(300)
def test_vocab_parallel_single_sweep_composition_matches_single_process(tmp_path):
    """Every rank sweeps its shard as a vocabulary of its own (local softmax, unit weights, a
    stand-in target where the target lives elsewhere); one exchange of per-row numbers must
    recombine them into the full-vocabulary loss, statistics and dHidden."""
    from oracle import head_oracle as ho

    x, w, t, c = _inputs()
    ref = ho.full_vocab_reference(x, w, t, c, want_rounded=False)
    outs = _run("vocab_sweep", tmp_path)
    for o in outs:
        np.testing.assert_allclose(float(o["loss"]), float(ref["loss"]), rtol=1e-5)
        np.testing.assert_allclose(o["lse"], ref["lse"].numpy(), rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(o["ent"], ref["ent"].numpy(), rtol=1e-4, atol=1e-4)
        assert (o["argmax"] == ref["argmax"].numpy()).all()
        valid = (t >= 0).numpy()
        np.testing.assert_allclose(o["ce"][valid], (ref["lse"] - ref["tlogit"]).numpy()[valid],
                                   rtol=1e-4, atol=1e-5)
        assert (o["ce"][~valid] == 0).all()
        np.testing.assert_allclose(o["dx"], ref["dx"].numpy(), rtol=1e-3, atol=1e-6)
        assert np.abs(o["dx"][~valid]).max() == 0.0
    assert np.array_equal(outs[0]["dx"], outs[1]["dx"])


def _leaving_worker(rank, world, port, announce, out_dir):
    """Rank 1 takes part in one step and then stops, between steps, with nothing in flight; rank 0
    goes on and must get a RankLostError within a bounded time instead of waiting forever."""
    import datetime
    import time

    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8))
    from esep_soup_kernels_b200.head import parallel as par
    from torch.distributed.distributed_c10d import _get_default_store

    roster = par.RankRoster(_get_default_store(), rank, world)
    x, w, t, c = _inputs()
    lo, hi = par.shard_bounds(x.shape[0], world, rank)
    factory = lambda x16, w16, ng: OracleBackend(x16, w16, ng)

    def step():
        roster.check()
        return par.token_sharded_linear_ce(x[lo:hi], w, t[lo:hi], c[lo:hi], backend_factory=factory)

    step()                       # a complete step with both ranks
    dist.barrier()
    if rank == 1:
        if announce:
            roster.leave()
        dist.destroy_process_group()
        return
    if announce:                 # give the leaver time to post its note; no collective in between
        deadline = time.time() + 20
        while time.time() < deadline and not _get_default_store().check(["esep_head_roster/left/1"]):
            time.sleep(0.05)
    t0 = time.time()
    try:
        step()
        outcome = "no error"
    except par.RankLostError as e:
        outcome = "RankLostError: " + str(e)[:80]
    with open(os.path.join(out_dir, "outcome.txt"), "w") as f:
        f.write(f"{time.time() - t0:.2f}\n{outcome}\n")


@pytest.mark.timeout(180)
@pytest.mark.parametrize("announce", [True, False])
def test_a_rank_that_leaves_between_steps_ends_the_others_with_an_error(tmp_path, announce):
    """Failure detection on the host, CPU ranks only: with a note in the store the survivor
    learns of it before its next launch; without one the next collective fails or runs into the
    group's (short) timeout. Either way a RankLostError, never a hang."""
    try:
        mp.spawn(_leaving_worker, args=(2, _free_port(), announce, str(tmp_path)), nprocs=2,
                 join=True)
    except Exception:   # the survivor's process group may complain while it is torn down
        pass
    secs, outcome = open(os.path.join(tmp_path, "outcome.txt")).read().splitlines()[:2]
    assert outcome.startswith("RankLostError"), outcome
    assert float(secs) < 30.0
    if announce:
        assert "left the group" in outcome and float(secs) < 2.0
