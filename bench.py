"""Benchmark of the fused LM head (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one forward + backward pass of the head over one batch of synthetic rows: 8 unpadded
sequences of U[128,1024] rows (4 340 rows), fp16, hidden 1536, vocabulary 151 936 - the
Qwen2.5-1.5B training-step head the metric is quoted on. Prints ONE JSON line on rank 0.

With N > 1 (launched by torch.distributed.run, one rank per GPU):
  * `value` is weak scaling of that step: every rank processes its own batch of the same shape,
    the weight is replicated, the ranks exchange one 8-scalar NCCL all-reduce per step;
  * `strong_c3` times the token-sharded form on 16 384 bf16 rows split evenly over the ranks
    (strong scaling, same exchange) next to the same rows on one GPU;
  * `vocab_parallel_c4` times the vocabulary-sharded form on the 7B shape (32 768 rows x 3584 x
    152 064, bf16, W split by vocabulary rows over the ranks): an all-gather of one [5, rows]
    record per rank and an all-reduce of dHidden;
  * both carry a `parity` block: a seeded 64-row subset against the CPU oracle, computed outside
    every timed region.

--impl reference times the reference's CPU path for this computation (the full-vocabulary
cross-entropy of solution/test_head.py:12-51, restated in oracle/head_oracle.py) on the host
cores: every step is one pass over the same batch.
"""

import argparse
import ctypes
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
METRIC = "fused LM-head fwd+bwd tokens/s (Qwen2.5-1.5B shape)"
UNIT = "tokens/s"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d["bf16_tflops_sustained"]),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def _traffic_sum(*kernels):
    parts = [_traffic(k) for k in kernels]
    return None if any(p is None for p in parts) else sum(parts)


def _traffic(kernel):
    """DRAM bytes per launch of `kernel` from the committed ncu summary, if one was recorded."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f).get(kernel)


def _synthetic():
    """The workload generator, loaded by file so that the CPU arm never imports the package
    (whose import maps the CUDA library)."""
    path = os.path.join(ROOT, "esep_soup_kernels_b200", "head", "synthetic.py")
    spec = importlib.util.spec_from_file_location("esep_bench_synthetic", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                pw.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load = those drawing at least 60 % of the highest power seen
        busy = [c for c, w in zip(sm, pw) if w >= 0.6 * max(pw)]
        return {"sm_mhz": statistics.median(busy), "sm_min_mhz": min(busy), "sm_max_mhz": max(mx),
                "power_w_max": max(pw), "samples": len(sm), "samples_under_load": len(busy),
                "reasons": sorted(reasons)}


def _describe(meta, n_gpus):
    return {"workload": f"{meta['name']}: {meta['n']} rows x hidden {meta['h']} x vocab {meta['v']} "
                        f"per GPU, {meta['dtype']}, synthetic (seeded N(0,1) hidden, N(0,0.02) W, "
                        "uniform labels, last token of each of the 8 sequences ignored)",
            "rows_per_gpu": meta["n"], "hidden": meta["h"], "vocab": meta["v"],
            "parallelism": f"dp{n_gpus}",
            "l2": "W (467 MB) is larger than the 126 MB L2 and is re-streamed every step; no flush"}


# ---------------------------------------------------------------------------------------------
# CPU arm
# ---------------------------------------------------------------------------------------------
def cpu_pass(ho, cfg, rows):
    """One pass of the oracle's full-vocabulary cross-entropy (fwd + dX) over the first `rows`
    rows of the batch on all host cores. Returns seconds."""
    x, w, t, c = cfg["x"], cfg["w"], cfg["target"], cfg["ce_weight"]
    x16 = x.to(w.dtype)
    t0 = time.perf_counter()
    ho.full_vocab_reference(x16[:rows], w, t[:rows], c[:rows], want_rounded=False)
    return time.perf_counter() - t0


def cpu_sample_rows(ho, cfg, budget_s):
    """Rows of the batch one CPU step passes over: the whole batch if a pass fits the budget."""
    n = cfg["x"].shape[0]
    cpu_pass(ho, cfg, min(32, n))                      # thread pool, page faults
    probe = min(256, n)
    dt = cpu_pass(ho, cfg, probe)
    rows = int(min(n, max(probe, probe * budget_s / max(dt, 1e-3))))
    return rows


def cpu_baseline_block(cfg, budget_s=15.0):
    """The bounded CPU sample beside a GPU run: passes over the batch for about `budget_s`."""
    from oracle import head_oracle as ho

    torch.set_num_threads(os.cpu_count() or 1)
    rows = cpu_sample_rows(ho, cfg, budget_s / 3)
    total, secs, passes = 0, 0.0, 0
    while secs < budget_s * 0.8 and passes < 8:
        secs += cpu_pass(ho, cfg, rows)
        total += rows
        passes += 1
    return {"value": total / secs, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{passes} pass(es) over the first {rows} of the {cfg['x'].shape[0]} rows, "
                      f"fwd+dX, {secs:.1f} s"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, ROOT)
    from oracle import head_oracle as ho

    torch.set_num_threads(os.cpu_count() or 1)
    cfg = _synthetic().make_config("c2", seed=0)
    meta = cfg["meta"]
    # every step = one pass over the same rows; the whole batch unless that would take the run
    # past a few minutes
    rows = cpu_sample_rows(ho, cfg, budget_s=150.0 / max(1, args.steps + args.warmup))
    for _ in range(args.warmup):
        cpu_pass(ho, cfg, rows)
    secs = [cpu_pass(ho, cfg, rows) for _ in range(args.steps)]
    per_step = sum(secs) / len(secs)
    value = rows / per_step
    cores = torch.get_num_threads()
    sample = (f"each step = one fwd+dX pass over {'all' if rows == meta['n'] else 'the first'} "
              f"{rows} of the {meta['n']} rows; {args.steps} timed steps, {sum(secs):.1f} s")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
            "rows_per_step": rows, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": _describe(meta, args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
            "note": "one host, whatever --gpus says: the CPU path does not scale with the number of "
                    "GPUs, so a ratio against it means something at N = 1 only"}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def _counters():
    from esep_soup_kernels_b200.head import _lib

    buf = (ctypes.c_longlong * 3)()
    _lib.load().esep_head_debug_counters(buf, 3)
    return buf[0], buf[1], buf[2]


def _parity(x, w, t, c, loss_terms, stats, dx, rows):
    """Largest deviations of `rows` from the CPU oracle (fp32 full-vocabulary cross-entropy)."""
    from oracle import head_oracle as ho

    ref = ho.full_vocab_reference(x[rows], w, t[rows], c[rows], want_rounded=False)
    got = {k: v[rows].float().cpu() if k != "argmax" else v[rows].cpu() for k, v in stats.items()}
    z = None
    miss = got["argmax"] != ref["argmax"]
    tie_ok = True
    if bool(miss.any()):   # a different index is fine only where the logits tie
        z = x[rows][miss].float() @ w.float().T
        at = z.gather(1, got["argmax"][miss][:, None]).squeeze(1)
        tie_ok = bool(((z.max(1).values - at).abs() <= 2e-3).all())
    dxr = dx[rows].float().cpu()
    ref_loss = float(ref["loss"])
    return {"rows": int(len(rows)),
            "loss_rel": abs(float(loss_terms[rows].sum()) - ref_loss) / max(abs(ref_loss), 1e-30),
            "lse_max_abs": float((got["lse"] - ref["lse"]).abs().max()),
            "entropy_max_abs": float((got["entropy"] - ref["ent"]).abs().max()),
            "argmax_equal": float((~miss).float().mean()), "argmax_ok_except_ties": tie_ok,
            "dx_rel_fro": float((dxr - ref["dx"]).norm() / ref["dx"].norm()),
            "tolerance": "loss, entropy 1e-3 relative; dHidden 2e-2 relative; argmax exact "
                         "except ties"}


def run_ours(args):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    from esep_soup_kernels_b200.head import (_lib, fused_linear_ce_with_metrics,
                                             last_device_status, warmup)
    from esep_soup_kernels_b200.head import op as head_op
    from esep_soup_kernels_b200.head import parallel as par
    from esep_soup_kernels_b200.head.synthetic import (QWEN_1P5B, QWEN_7B, make_config,
                                                       make_weight)

    path_names = {0: "auto", 1: "single_pass", 2: "stored_logits", 3: "stored_weights"}
    head_op.set_training_path(path_names[args.path])   # 0 unless a profile capture asks otherwise

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # stdout carries one JSON line: NCCL's version banner (printed from the VERSION level up) and
    # anything else it logs go to stderr
    if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "WARN"):
        del os.environ["NCCL_DEBUG"]
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup(dev)

    cfg = make_config("c2", seed=rank)
    meta = cfg["meta"]
    if rank:   # W is replicated: every rank holds the weight of seed 0
        cfg["w"] = make_weight(meta["v"], meta["h"], QWEN_1P5B["w_std"], cfg["w"].dtype, 0)
    n, h, v = meta["n"], meta["h"], meta["v"]
    x_host = cfg["x"].pin_memory()
    t_host = cfg["target"].pin_memory()
    c_host = cfg["ce_weight"].pin_memory()
    w = cfg["w"].to(dev)
    x = x_host.to(dev)
    tgt = t_host.to(dev)
    cew = c_host.to(dev)
    n_live = int((cfg["ce_weight"] != 0).sum())
    # every rank draws its own batch (same sequence lengths, own values): count the rows of all ranks
    rows_all = torch.tensor([float(n)], device=dev)
    if world > 1:
        dist.all_reduce(rows_all)
    total_rows = rows_all.item()
    call_events = []    # (start, end) CUDA events around the library call of a step

    def step_device(record=False, x=x, tgt=tgt, cew=cew):
        xg = x.detach().requires_grad_(True)
        if record:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        loss, stats, m = fused_linear_ce_with_metrics(xg, w, tgt, cew)
        if record:
            b.record()
            call_events.append((a, b))
        loss.backward()
        if world > 1:
            m = m.clone()
            dist.all_reduce(m)      # the one exchange of a data-parallel step: eight scalars
        return loss, xg.grad, m

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, warm):
        for _ in range(warm):
            fn()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps

    # ---- the timed region: K steps, inputs resident; the library call of every step is also
    #      bracketed by its own event pair, so the dominant kernel is timed inside this loop ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = _counters()[2]
    for _ in range(args.warmup):
        step_device()
    launches_warm = _counters()[2]
    ms_step = timed(lambda: step_device(record=True), args.steps, 0)
    launches1 = _counters()[2]
    clocks = sampler.stop() if rank == 0 else None
    call_ms = [a.elapsed_time(b) for a, b in call_events]
    ms_call = statistics.mean(call_ms)
    own_launches = launches1 - launches_warm
    del launches0

    # ---- end to end through the public op with HOST inputs --------------------------------
    # Every step's inputs travel from pinned host memory inside the timed region; like a data
    # loader with one batch of look-ahead, the copy of step i+1 is issued on a copy stream as
    # soon as step i's kernels are queued, into the other of two device buffer sets. The loss
    # is read back (and waited for) every step, as a trainer that logs it does.
    loss_host = torch.zeros(1).pin_memory()
    copy_stream = torch.cuda.Stream(device=dev)
    bufs = [(x, tgt, cew), (torch.empty_like(x), torch.empty_like(tgt), torch.empty_like(cew))]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    state = {"i": 0}

    def enqueue_copy(k):
        with torch.cuda.stream(copy_stream):
            bufs[k][0].copy_(x_host, non_blocking=True)
            bufs[k][1].copy_(t_host, non_blocking=True)
            bufs[k][2].copy_(c_host, non_blocking=True)
            ready[k].record(copy_stream)

    def step_e2e():
        k = state["i"] & 1
        if state["i"] == 0:
            enqueue_copy(0)
        torch.cuda.current_stream().wait_event(ready[k])
        loss, _, _ = step_device(x=bufs[k][0], tgt=bufs[k][1], cew=bufs[k][2])
        # set k^1 was last read by the previous step, which the host has already waited for
        enqueue_copy(k ^ 1)
        loss_host.copy_(loss.detach().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()   # the trainer reads the loss every step
        state["i"] += 1

    ms_e2e = timed(step_e2e, args.steps, max(1, args.warmup // 2))
    copy_stream.synchronize()
    h2d = x_host.numel() * x_host.element_size() + t_host.numel() * 8 + c_host.numel() * 4
    d2h = 4

    peaks = _peaks()
    hv = float(h) * v
    f_alg = 2.0 * hv * n + 2.0 * hv * n_live
    line_extra = {}

    if world == 1 and args.only_timed:
        pass
    elif world == 1:
        # ---- sustained: the same step for at least two seconds, clocks sampled meanwhile ----
        sus_steps = max(50, int(2200.0 / ms_step))
        s2 = ClockSampler(local)
        s2.start()
        time.sleep(0.2)
        ms_sus = timed(step_device, sus_steps, 0)
        sus_clocks = s2.stop()
        sus_tf = f_alg / (ms_sus * 1e-3) / 1e12
        line_extra["sustained"] = {
            "steps": sus_steps, "seconds": sus_steps * ms_sus * 1e-3, "ms_per_step": ms_sus,
            "tokens_s": n / (ms_sus * 1e-3), "achieved_tflops": sus_tf,
            "peak_sustained": peaks["tflops_sustained"],
            "frac_of_sustained": sus_tf / peaks["tflops_sustained"],
            "frac_of_burst": sus_tf / peaks["tflops"], "clocks": sus_clocks}

        # ---- the two-kernel path's sweeps, each timed alone ----------------------------------
        x16, t64, c32 = head_op._prepare(x, w, tgt, cew)
        be = head_op.DeviceBackend(x16, w, True)
        rec = be.forward_partial(x16, w, t64, 0)
        fin = be.finalize(rec, t64, c32, v)

        def timed_kernel(fn, iters):
            evs = []
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            for _ in range(iters):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                evs.append((a, b))
            torch.cuda.synchronize()
            return statistics.mean(a.elapsed_time(b) for a, b in evs)

        ms_fwd = timed_kernel(lambda: be.forward_partial(x16, w, t64, 0), 10)
        ms_bwd = timed_kernel(lambda: be.backward(x16, w, t64, fin["cew"], fin["lse"], 0), 10)
        fwd_tf = 2.0 * hv * n / (ms_fwd * 1e-3) / 1e12
        bwd_tf = 2.0 * hv * n_live / (ms_bwd * 1e-3) / 1e12
        line_extra["roofline_two_kernel_path"] = {
            "head_fwd_kernel": {"achieved": fwd_tf, "frac": fwd_tf / peaks["tflops"], "ms": ms_fwd,
                                "traffic": _traffic("head_fwd_kernel")},
            "head_bwd_kernel": {"achieved": bwd_tf, "frac": bwd_tf / peaks["tflops"], "ms": ms_bwd,
                                "executed_tflops": 4.0 * hv * n / (ms_bwd * 1e-3) / 1e12,
                                "traffic": _traffic("head_bwd_kernel")},
            "note": "the forward sweep also serves rows without a gradient; the pair is the guarded "
                    "second attempt of the single pass and the SINGLE_SWEEP = False path"}

        # ---- the same step on the other training path (logits never leave the SM) ------------
        head_op.set_training_path("single_pass")
        try:
            ms_single = timed(step_device, 10, 3)
        finally:
            head_op.set_training_path(path_names[args.path])
        single_tf = f_alg / (ms_single * 1e-3) / 1e12
        line_extra["single_pass_path"] = {
            "ms_per_step": ms_single, "achieved_tflops": single_tf,
            "frac": single_tf / peaks["tflops"], "traffic": _traffic("head_train_kernel"),
            "note": "esep_head_set_training_path(1): head_train_kernel instead of the two sweeps; "
                    "no logits buffer in the workspace"}
    else:
        line_extra["strong_c3"] = _strong_c3(dist, par, make_config, dev, rank, world, peaks, args)
        line_extra["vocab_parallel_c4"] = _vocab_parallel_c4(dist, par, make_config, make_weight,
                                                             QWEN_7B, dev, rank, world, peaks, args)
    status = last_device_status(dev)

    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    _, caps = _lib.query(local)
    pl = _lib.plan_problem(n, h, v, True, caps.sm_count, caps.max_clusters_bwd)
    tokens_s = total_rows / (ms_step * 1e-3)
    call_tf = f_alg / (ms_call * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": tokens_s, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": meta["dtype"], "data": "synthetic",
        "config": _describe(meta, world),
        "e2e": {"value": total_rows / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e,
                "note": "x, labels and weights copied from pinned host memory every step (the copy of "
                        "the next step's batch overlaps this step's kernels, two device buffer sets); "
                        "the LM-head weight W is a resident model parameter; loss read back and waited "
                        "for every step"},
        "gpu_launches": own_launches,
        "gpu_launches_note": "kernels launched by libesep_head.so inside the timed region, counted "
                             "by the library itself (its counter covers every entry point); torch "
                             "adds the gradient scaling of the autograd backward and, with N > 1, "
                             "NCCL's all-reduce",
        "clocks": clocks,
        "roofline": {"bound": "tensor",
                     "kernel": "head_fwd_kernel<store weights> + head_dx_kernel<direct> (the two "
                               "sweeps of the step: logits GEMM, dHidden GEMM)",
                     "achieved": call_tf,
                     "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": call_tf / peaks["tflops"],
                     "traffic": _traffic_sum("head_fwd_kernel_weights", "head_dx_kernel_weights"),
                     "traffic_note": "DRAM bytes of the two kernels per step (ncu): the softmax "
                                     "weights are written once as bf16 (1.28 GB) and read by the "
                                     "second sweep, W is read by both",
                     "peak_source": peaks["source"] + " burst",
                     "flops": "algorithmic 2*H*V*N + 2*H*V*N_live (logits GEMM + dHidden GEMM, each "
                              "once), which is also what the two sweeps execute",
                     "ms": ms_call, "ms_min": min(call_ms), "ms_max": max(call_ms),
                     "ms_first_last": [call_ms[0], call_ms[-1]],
                     "ms_note": "mean over the timed steps of the CUDA-event time of the whole "
                                "esep_head_step call inside the timed loop (row classes, gather, "
                                "prefix sweep, storing forward sweep, dHidden sweep, row finish, "
                                "scalars); the two sweeps are 90 % of it in the ncu launch list"},
        "step_tensor_frac": f_alg / (ms_step * 1e-3) / 1e12 / peaks["tflops"],
        "device_status": status,
        "plan": {"sm_count": caps.sm_count, "bwd_clusters_resident": caps.max_clusters_bwd,
                 "row_tiles": pl.fwd_row_tiles, "sweep_full_rounds": pl.bwd_full_rounds,
                 "sweep_left_over_tiles": pl.bwd_rem_pairs, "sweep_runs": pl.bwd_rem_splits,
                 "sweep_grid": pl.bwd_grid},
    }
    line.update(line_extra)
    if world == 1 and not args.only_timed:
        line["cpu_baseline"] = cpu_baseline_block(cfg)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def _timed_ranks(dist, dev, fn, steps, warm):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item() / steps


def _strong_c3(dist, par, make_config, dev, rank, world, peaks, args):
    """16 384 bf16 rows split evenly over the ranks (W replicated, one 8-scalar all-reduce)."""
    cfg = make_config("c3", seed=0)                 # the same rows on every rank: each takes its slice
    meta = cfg["meta"]
    n, h, v = meta["n"], meta["h"], meta["v"]
    lo, hi = par.shard_bounds(n, world, rank)
    w = cfg["w"].to(dev)
    xs, ts, cs = cfg["x"][lo:hi].to(dev), cfg["target"][lo:hi].to(dev), cfg["ce_weight"][lo:hi].to(dev)
    steps = max(3, min(args.steps, 10))

    def step():
        return par.token_sharded_linear_ce(xs, w, ts, cs)

    ms = _timed_ranks(dist, dev, step, steps, 3)
    # the same 16 384 rows on ONE GPU (every rank does it; the slowest counts)
    xa, ta, ca = cfg["x"].to(dev), cfg["target"].to(dev), cfg["ce_weight"].to(dev)
    ms1 = _timed_ranks(dist, dev, lambda: _single(xa, w, ta, ca), 3, 2)
    del xa, ta, ca
    loss, stats, dx, metrics = step()
    out = {"rows_total": n, "rows_per_gpu": hi - lo, "dtype": meta["dtype"], "steps": steps,
           "ms_per_step": ms, "tokens_s": n / (ms * 1e-3), "ms_per_step_1gpu_same_rows": ms1,
           "efficiency_vs_1gpu_same_rows": ms1 / (world * ms),
           "step_tensor_frac": 4.0 * h * v * (hi - lo) / (ms * 1e-3) / 1e12 / peaks["tflops"],
           "metrics_all_ranks": [float(m) for m in metrics[:4].tolist()]}
    if rank == 0:
        rows = torch.arange(0, hi - lo, max(1, (hi - lo) // 64))[:64]
        out["parity"] = _parity(cfg["x"][lo:hi], cfg["w"], cfg["target"][lo:hi],
                                cfg["ce_weight"][lo:hi], (stats["ce"] * cs).float().cpu(), stats,
                                dx, rows)
    return out


def _single(x, w, t, c):
    """The token-sharded call without its all-reduce (one GPU's view of the whole batch)."""
    from esep_soup_kernels_b200.head import op as head_op

    return head_op._run_step(x, w, True, target=t, ce_weight=c)


def _vocab_parallel_c4(dist, par, make_config, make_weight, shape, dev, rank, world, peaks, args):
    """32 768 x 3584 bf16 rows against a 152 064-row W split by vocabulary rows over the ranks."""
    n, h, v = 32768, shape["h"], shape["v"]
    g = torch.Generator().manual_seed(4)
    x = torch.randn(n, h, generator=g).to(torch.bfloat16)
    target = torch.randint(0, v, (n,), generator=g)
    target[torch.rand(n, generator=g) < 0.05] = -100
    cew = (target >= 0).float()
    lo, hi = par.shard_bounds(v, world, rank)
    # W = the concatenation of `world` independently seeded shards
    w_shard = make_weight(hi - lo, h, shape["w_std"], torch.bfloat16, seed=100 + rank).to(dev)
    xd, td, cd = x.to(dev), target.to(dev), cew.to(dev)
    steps = max(3, min(args.steps, 6))
    timings = []

    def step(tm=None):
        return par.vocab_parallel_linear_ce(xd, w_shard, td, cd, lo, v, timings=tm)

    ms = _timed_ranks(dist, dev, step, steps, 2)
    loss, stats, dx = step(timings)
    torch.cuda.synchronize()
    marks = dict(timings)
    split = {k: marks[a].elapsed_time(marks[b]) for k, a, b in (
        ("sweep_ms", "start", "sweep"), ("exchange_ms", "sweep", "exchange"),
        ("combine_ms", "exchange", "combine"), ("dx_allreduce_ms", "combine", "reduce"))}
    n_live = int((target >= 0).sum())
    f_alg_gpu = (2.0 * h * (hi - lo) * n + 2.0 * h * (hi - lo) * n_live)
    # every rank must hold the same dHidden bits after the all-reduce
    chk = torch.stack([dx.double().sum(), dx[::97].double().abs().sum()])
    lo_chk, hi_chk = chk.clone(), chk.clone()
    dist.all_reduce(lo_chk, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi_chk, op=dist.ReduceOp.MAX)
    out = {"rows": n, "hidden": h, "vocab": v, "shards": world, "vocab_rows_per_gpu": hi - lo,
           "dtype": "bfloat16", "steps": steps, "ms_per_step": ms, "tokens_s": n / (ms * 1e-3),
           "tensor_frac": f_alg_gpu / (ms * 1e-3) / 1e12 / peaks["tflops"],
           "time_split_rank0": split, "dx_identical_on_all_ranks": bool((lo_chk == hi_chk).all()),
           "note": "hidden 3584 takes the two-sweep path: a forward sweep keeps the softmax weights "
                   "as bf16 in HBM, head_dx_kernel takes them by TMA and turns them into dHidden "
                   "(CTA pairs, 256 rows per W tile)"}
    # parity: the oracle needs the whole W on the host; rank 0 rebuilds the other shards
    sub = torch.arange(0, n, n // 64)[:64]
    if rank == 0:
        shards = [make_weight(par.shard_bounds(v, world, r)[1] - par.shard_bounds(v, world, r)[0], h,
                              shape["w_std"], torch.bfloat16, seed=100 + r) for r in range(world)]
        w_full = torch.cat(shards)
        out["parity"] = _parity(x, w_full, target, cew, (stats["ce"] * cd).float().cpu(), stats, dx,
                                sub)
    return out


def run_norm_bandwidth(rows, hidden, iters=20):
    """The final-norm kernels either side of the head (HBM bound) on inputs larger than L2:
    achieved GB/s on the algorithmic bytes (forward 12 H, backward 14 H per row)."""
    sys.path.insert(0, ROOT)
    from esep_soup_kernels_b200.head import final_norm_backward, final_norm_forward

    dev = torch.device("cuda", torch.cuda.current_device())
    dtype = torch.float16
    r = torch.randn(rows, hidden, device=dev)
    d = torch.randn(rows, hidden, device=dev).to(dtype)
    g = torch.rand(hidden, device=dev) + 0.5
    dy = torch.randn(rows, hidden, device=dev)
    r_out, _, rstd = final_norm_forward(r, d, g, 1e-6, dtype)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    peak = _peaks()["hbm_gbs"]
    out = {"metric": "final-norm kernels GB/s", "rows": rows, "hidden": hidden, "dtype": "float16"}
    for name, per_row, fn in (
            ("forward", 12, lambda: final_norm_forward(r, d, g, 1e-6, dtype)),
            ("backward", 14, lambda: final_norm_backward(dy, r_out, rstd, g, None, dtype))):
        ms = timed(fn)
        nbytes = per_row * hidden * rows
        out[name] = {"us": ms * 1e3, "algorithmic_mb": nbytes / 1e6, "gbs": nbytes / ms / 1e6,
                     "frac_of_measured_hbm": nbytes / ms / 1e6 / peak}
    print(json.dumps(out))


def run_weight_bandwidth(vocab, hidden, lookups, iters=20):
    """The kernels of the shared fp16 head / embedding weight (HBM bound) on a weight larger than
    L2: the cast-and-count pass (4 B read + 2 B written per element), the embedding lookup
    (2 H read + 4 H written per row) and the exact fp32 rebuild (2 B + 4 B per element)."""
    sys.path.insert(0, ROOT)
    from esep_soup_kernels_b200.head.weight import Fp16Fixup

    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator().manual_seed(0)
    w32 = torch.empty(vocab, hidden, device=dev)
    for lo in range(0, vocab, 16384):
        n = min(16384, vocab - lo)
        w32[lo:lo + n] = (torch.randn(n, hidden, generator=g) * 0.02).to(torch.bfloat16).float().to(dev)
    ids = torch.randint(0, vocab, (lookups,), generator=g).to(dev)
    w16, fix = Fp16Fixup.cast(w32)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    peak = _peaks()["hbm_gbs"]
    elems = vocab * hidden
    out = {"metric": "shared fp16 weight kernels GB/s", "vocab": vocab, "hidden": hidden,
           "lookups": lookups, "entries": fix.count, "rows_with_entries": fix.rows,
           "most_in_one_row": fix.width, "table_bytes": fix.nbytes()}
    from esep_soup_kernels_b200.head import _lib
    from esep_soup_kernels_b200.head.op import _ptr, _stream
    lib = _lib.load()
    row_start = torch.empty(vocab + 1, device=dev, dtype=torch.int32)
    stats = torch.empty(3 + (vocab + 1023) // 1024, device=dev, dtype=torch.int64)
    w16b = torch.empty_like(w16)

    def scan():       # the two passes of the set-up on their own (no host read in between)
        _lib.check("esep_weight_fixup_scan", lib.esep_weight_fixup_scan(
            _ptr(w32), _ptr(w16b), 1, vocab, hidden, _ptr(row_start), _ptr(stats), _stream(dev)))

    def fill():
        _lib.check("esep_weight_fixup_fill", lib.esep_weight_fixup_fill(
            _ptr(w32), _ptr(w16), vocab, hidden, _ptr(fix.row_start), _ptr(fix.flat_idx),
            _ptr(fix.flat_val), _stream(dev)))

    for name, nbytes, fn in (
            ("cast_and_count", 6 * elems, scan),
            ("fill", 6 * hidden * fix.rows, fill),
            ("set_up_whole", 6 * elems + 6 * hidden * fix.rows, lambda: Fp16Fixup.cast(w32)),
            ("embed", 6 * hidden * lookups, lambda: fix.embed(w16, ids)),
            ("exact_weight", 6 * elems, lambda: fix.exact_weight(w16))):
        ms = timed(fn)
        out[name] = {"us": ms * 1e3, "algorithmic_mb": nbytes / 1e6, "gbs": nbytes / ms / 1e6,
                     "frac_of_measured_hbm": nbytes / ms / 1e6 / peak}
    print(json.dumps(out))


def run_shape(rows, hidden, vocab, steps, warmup, path=0):
    """fused_linear_ce + backward on a synthetic bf16 problem of the given shape on one GPU (e.g.
    one vocabulary shard of the 7B configuration: 32768 3584 19008): ms per step with a CUDA
    event pair, algorithmic TFLOP/s (4 H V per row) and its share of the measured tensor peak.
    A profiler capture of a kernel at another hidden size uses this with few rows."""
    sys.path.insert(0, ROOT)
    from esep_soup_kernels_b200.head import _lib, fused_linear_ce, last_device_status

    _lib.load().esep_head_set_training_path(int(path))
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator().manual_seed(0)
    x = torch.randn(rows, hidden, generator=g).to(torch.bfloat16).to(dev)
    w = torch.empty(vocab, hidden, dtype=torch.bfloat16, device=dev)
    for lo in range(0, vocab, 16384):      # the weight is built in slices: no fp32 copy of it
        n = min(16384, vocab - lo)
        w[lo:lo + n] = (torch.randn(n, hidden, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    t = torch.randint(0, vocab, (rows,), generator=g).to(dev)
    c = torch.full((rows,), 1.0 / rows, device=dev)

    def step():
        xg = x.detach().requires_grad_(True)
        loss, _ = fused_linear_ce(xg, w, t, c)
        loss.backward()
        return loss

    for _ in range(max(warmup, 1)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    tf = 4.0 * hidden * vocab * rows / (ms * 1e-3) / 1e12
    print(json.dumps({"metric": "head step on a given shape", "rows": rows, "hidden": hidden,
                      "vocab": vocab, "dtype": "bfloat16", "path": path, "steps": steps, "ms_per_step": ms,
                      "rows_s": rows / (ms * 1e-3), "algorithmic_tflops": tf,
                      "frac_of_measured_tensor_peak": tf / _peaks()["tflops"],
                      "loss": float(loss.detach()), "device_status": last_device_status()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only-timed", action="store_true",
                    help="one GPU: stop after the timed region and the end-to-end leg (for short "
                         "profiler captures); the line then lacks sustained / cpu_baseline")
    ap.add_argument("--norm-bandwidth", nargs=2, type=int, metavar=("ROWS", "HIDDEN"),
                    help="instead of the head: time the final-norm kernels on ROWS x HIDDEN")
    ap.add_argument("--weight-bandwidth", nargs=3, type=int, metavar=("VOCAB", "HIDDEN", "LOOKUPS"),
                    help="instead of the head: time the kernels of the shared fp16 weight format")
    ap.add_argument("--path", type=int, default=0, choices=[0, 1, 2, 3],
                    help="training path (esep_head_set_training_path): 0 auto (the default), "
                         "1 single pass, 2 two sweeps over stored fp16 logits, 3 two sweeps over stored bf16 "
                         "softmax weights (what 0 takes wherever the two sweeps apply)")
    ap.add_argument("--shape", nargs=3, type=int, metavar=("ROWS", "HIDDEN", "VOCAB"),
                    help="instead of configuration 2: time the head step (bf16) on this shape")
    args = ap.parse_args()
    if args.norm_bandwidth:
        run_norm_bandwidth(*args.norm_bandwidth)
        return
    if args.shape:
        run_shape(*args.shape, steps=args.steps, warmup=args.warmup, path=args.path)
        return
    if args.weight_bandwidth:
        run_weight_bandwidth(*args.weight_bandwidth)
        return
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        if args.steps > 20:      # a pass over the batch takes seconds on the host
            args.steps = 20
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    sys.path.insert(0, ROOT)
    main()
