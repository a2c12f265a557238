"""GPU parity tests: the CUDA LM head (through the Python op -> C ABI) against the CPU oracle.
Shapes follow the reference's unit tests (solution/test_head.py:118-182) and the benchmark
configurations; inputs are seeded on the CPU so both sides see identical tensors."""

import glob
import os

import numpy as np
import pytest
import torch

from tests.helpers import check_against_oracle, run_op

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["two_sweeps", "stored_logits", "single_pass"])
def training_path(request):
    """Every test runs on the three training paths of the library: the default (two sweeps, bf16
    softmax weights kept between them, wherever that applies), two sweeps over fp16 logits, and
    the single pass that keeps the logits on the SM."""
    from esep_soup_kernels_b200.head.op import set_training_path

    set_training_path("auto" if request.param == "two_sweeps" else request.param)
    yield request.param
    set_training_path("auto")

GOLDEN = sorted(p for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz"))
                if not os.path.basename(p).startswith(("final_norm", "fp16_fixup")))   # head cases only


def _peaked(n, h, v, scale_w, peak, seed, dtype=torch.float16):
    """Inputs of solution/test_head.py:58-75 (_make) from a CPU generator."""
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(v, h, generator=g) * scale_w).to(dtype)
    target = torch.randint(0, v, (n,), generator=g)
    x = torch.randn(n, h, generator=g)
    if peak:
        wt = w[target].float()
        x = x + torch.rand(n, 1, generator=g) * peak * wt / wt.pow(2).sum(-1, keepdim=True)
    x = x.to(dtype)
    cew = torch.rand(n, generator=g) / n
    target[::7] = -100
    cew[::7] = 0.0
    cew[3::11] = 0.0
    return x, w, target, cew


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_golden_cases_match_reference_outputs(path):
    """The committed fixtures hold the reference op's own outputs (fp16-rounded logits)."""
    d = dict(np.load(path))
    x = torch.from_numpy(d["x"].view(np.int16)).view(torch.float16)
    w = torch.from_numpy(d["w"].view(np.int16)).view(torch.float16)
    t, c = torch.from_numpy(d["target"]), torch.from_numpy(d["ce_weight"])
    loss, stats, dx = run_op(x, w, t, c)
    check_against_oracle(x, w, t, c, loss, stats, dx,
                         tie_pairs=[tuple(p) for p in d["tie_pairs"]] if "tie_pairs" in d else None)
    # vs the reference op itself: its logits are rounded to fp16, half an ulp = 2^-11 relative
    # (0.0156 for |z| < 64: the bounds of solution/test_head.py:91-94; the tie case plants
    # logits near 300, hence the relative term)
    np.testing.assert_allclose(float(loss.detach()), float(d["op_loss"]), rtol=1e-3, atol=1e-4)
    np.testing.assert_allclose(stats["lse"].cpu().numpy(), d["op_lse"], rtol=5e-4, atol=1.6e-2)
    np.testing.assert_allclose(stats["entropy"].cpu().numpy(), d["op_ent"], rtol=0, atol=3e-2)
    ref_dx = torch.from_numpy(d["op_dx"])
    err = (dx.float().cpu() - ref_dx).norm() / ref_dx.norm()
    assert err < 1e-2


@pytest.mark.parametrize("n,h,v,scale_w,peak,seed", [
    (77, 64, 1001, 0.3, 20.0, 0),       # solution/test_head.py:118-121
    (300, 128, 5003, 0.2, 25.0, 3),     # solution/test_head.py:166-182
    (1, 64, 257, 0.3, 0.0, 4),          # single row, vocabulary just over one tile
    (129, 256, 4096, 0.1, 10.0, 5),     # one row over a tile boundary
    (513, 1536, 3000, 0.02, 30.0, 6),   # real hidden size, ragged rows and vocabulary
])
def test_small_shapes(n, h, v, scale_w, peak, seed):
    x, w, t, c = _peaked(n, h, v, scale_w, peak, seed)
    if n == 300:
        t[:150] = -100
        c[:150] = 0.0
    loss, stats, dx = run_op(x, w, t, c)
    check_against_oracle(x, w, t, c, loss, stats, dx)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n,h,v", [
    (1, 8, 1),            # smallest legal problem: one row, one 16-byte x row, one vocabulary entry
    (129, 24, 127),       # hidden narrower than one 64-wide k-slice, vocabulary under one tile
    (129, 72, 2049),      # hidden not a multiple of 64 (2-D tensor map for the dHidden GEMM)
    (1, 1000, 129),
    (2, 3584, 700),       # 7B hidden: three passes over the hidden dimension
    (127, 4096, 1030),
    (5, 8192, 300),
])
def test_ragged_hidden_and_vocabulary_sizes(n, h, v, dtype):
    g = torch.Generator().manual_seed(n * 7 + h + v)
    w = (torch.randn(v, h, generator=g) * (1.0 / h ** 0.5)).to(dtype)
    x = torch.randn(n, h, generator=g).to(dtype)
    t = torch.randint(0, v, (n,), generator=g)
    t[::5] = -100
    c = torch.rand(n, generator=g)
    loss, stats, dx = run_op(x, w, t, c)
    check_against_oracle(x, w, t, c, loss, stats, dx)


def test_bf16_and_fp32_input():
    x, w, t, c = _peaked(200, 128, 3001, 0.2, 20.0, 7, dtype=torch.bfloat16)
    loss, stats, dx = run_op(x, w, t, c)
    check_against_oracle(x, w, t, c, loss, stats, dx)
    # fp32 x is cast to the weight dtype inside; dX comes back fp32 (solution/test_head.py:166-182)
    x32 = x.float() + 1e-3
    loss, stats, dx = run_op(x32, w, t, c)
    assert dx.dtype == torch.float32 and loss.dtype == torch.float32 and loss.dim() == 0
    check_against_oracle(x32, w, t, c, loss, stats, dx)


def test_no_grad_path_and_determinism():
    """Without a gradient only the forward sweep runs (solution/test_head.py:132-163); two training
    calls on the same inputs are bit-identical (no atomics, fixed reduction order, and which
    kernel handles which row is decided on the device from the call's own arguments). The call
    without gradient runs a different kernel and agrees to fp32 rounding."""
    from esep_soup_kernels_b200.head import fused_linear_ce

    x, w, t, c = _peaked(77, 64, 1001, 0.3, 20.0, 0)
    xd, wd, td, cd = x.cuda().requires_grad_(True), w.cuda(), t.cuda(), c.cuda()
    with torch.no_grad():
        loss0, st0 = fused_linear_ce(xd, wd, td, cd)
    assert not loss0.requires_grad
    loss1, st1 = fused_linear_ce(xd, wd, td, cd)
    assert loss1.requires_grad
    loss1.backward()
    g1 = xd.grad.clone()
    xd.grad = None
    loss2, st2 = fused_linear_ce(xd, wd, td, cd)
    loss2.backward()
    assert torch.equal(loss1.detach(), loss2.detach())
    torch.testing.assert_close(loss0, loss1.detach(), rtol=1e-5, atol=0.0)
    for k in st1:
        assert torch.equal(st1[k], st2[k])
        if k == "argmax":
            assert torch.equal(st0[k], st1[k])
        else:
            torch.testing.assert_close(st0[k], st1[k], rtol=1e-5, atol=2e-5)
    assert torch.equal(g1, xd.grad)
    # grad_loss scaling in autograd backward (solution/head/op.py:143-145)
    xd.grad = None
    loss3, _ = fused_linear_ce(xd, wd, td, cd)
    (loss3 * 3.0).backward()
    torch.testing.assert_close(xd.grad.float(), g1.float() * 3.0, rtol=2e-3, atol=1e-6)


def test_empty_input():
    from esep_soup_kernels_b200.head import fused_linear_ce

    w = torch.zeros(100, 64, dtype=torch.float16, device="cuda")
    x = torch.zeros(0, 64, dtype=torch.float16, device="cuda", requires_grad=True)
    loss, st = fused_linear_ce(x, w, torch.zeros(0, dtype=torch.long, device="cuda"),
                               torch.zeros(0, device="cuda"))
    assert loss.item() == 0.0 and loss.requires_grad and st["argmax"].dtype == torch.int64
    loss.backward()


def test_bad_arguments_are_rejected_on_the_host():
    from esep_soup_kernels_b200.head import fused_linear_ce

    w = torch.zeros(100, 64, dtype=torch.float16, device="cuda")
    t = torch.zeros(4, dtype=torch.long, device="cuda")
    c = torch.ones(4, device="cuda")
    with pytest.raises(AssertionError):
        fused_linear_ce(torch.zeros(4, 32, dtype=torch.float16, device="cuda"), w, t, c)
    with pytest.raises(AssertionError):
        fused_linear_ce(torch.zeros(4, 64, dtype=torch.float64, device="cuda"), w, t, c)
    with pytest.raises(AssertionError):
        fused_linear_ce(torch.zeros(4, 64, dtype=torch.float16), w, t, c)
    with pytest.raises(AssertionError):
        fused_linear_ce(torch.zeros(4, 64, dtype=torch.float16, device="cuda"), w.float(), t, c)


def test_config1_full_vocab_fp32():
    """Configuration 1 (the CPU reference-path check): 64 rows, fp32 x, 1.5B-shape head, 10 % ignored."""
    from esep_soup_kernels_b200.head.synthetic import make_config

    cfg = make_config("c1")
    loss, stats, dx = run_op(cfg["x"], cfg["w"], cfg["target"], cfg["ce_weight"])
    check_against_oracle(cfg["x"], cfg["w"], cfg["target"], cfg["ce_weight"], loss, stats, dx)


def test_config2_full_size_row_subset():
    """Configuration 2 (8 unpadded sequences, fp16, the metric's workload) at full size; the oracle checks a seeded subset of rows (rows are
    independent) and the loss is checked through sum(ce_weight * ce)."""
    from esep_soup_kernels_b200.head.synthetic import make_config

    cfg = make_config("c2")
    x, w, t, c = cfg["x"], cfg["w"], cfg["target"], cfg["ce_weight"]
    loss, stats, dx = run_op(x, w, t, c)
    np.testing.assert_allclose(float(loss.detach()), float((c.double() * stats["ce"].cpu().double()).sum()),
                               rtol=1e-5)
    ends = torch.cumsum(torch.tensor(cfg["meta"]["seq_lens"]), 0) - 1
    rows = torch.cat([torch.randperm(x.shape[0], generator=torch.Generator().manual_seed(1))[:96],
                      ends])
    check_against_oracle(x, w, t, c, loss, stats, dx, rows=rows)


def test_config3_full_size_rows_are_independent_of_the_batch():
    """Configuration 3 (token-sharded data parallel) on one GPU (16 384 rows, bf16): a seeded row subset against the oracle, the
    loss through sum(ce_weight * ce), and the size-independent property that a row's results do
    not depend on which other rows share the call: the 2 048 rows one GPU gets at 8 GPUs give the
    same statistics and dHidden alone as inside the full batch (the vocabulary is cut into
    different runs in the two calls, so sums may differ in the last bits)."""
    from esep_soup_kernels_b200.head.synthetic import make_config

    cfg = make_config("c3")
    x, w, t, c = cfg["x"], cfg["w"], cfg["target"], cfg["ce_weight"]
    assert x.shape[0] == 16384 and w.dtype == torch.bfloat16
    loss, stats, dx = run_op(x, w, t, c)
    np.testing.assert_allclose(float(loss.detach()), float((c.double() * stats["ce"].cpu().double()).sum()),
                               rtol=1e-5)
    rows = torch.randperm(x.shape[0], generator=torch.Generator().manual_seed(3))[:96]
    check_against_oracle(x, w, t, c, loss, stats, dx, rows=rows)
    lo, hi = 6 * 2048, 7 * 2048
    loss_s, stats_s, dx_s = run_op(x[lo:hi], w, t[lo:hi], c[lo:hi])
    for k in ("lse", "entropy", "ce", "target_logit"):
        np.testing.assert_allclose(stats_s[k].cpu().numpy(), stats[k][lo:hi].cpu().numpy(),
                                   rtol=1e-5, atol=1e-5)
    assert torch.equal(stats_s["argmax"], stats["argmax"][lo:hi])
    a, b = dx_s.float(), dx[lo:hi].float()
    assert float((a - b).norm() / b.norm()) < 1e-3   # both rounded to bf16 by autograd
    assert float(dx[t < 0].abs().max()) == 0.0 if bool((t < 0).any()) else True


def test_config5_edge_cases_row_subset():
    """Configuration 5 (numerics edge cases, 4 099 rows): x scaled x4, 50 % ignored, a zero row, planted argmax ties."""
    from esep_soup_kernels_b200.head.synthetic import make_config

    cfg = make_config("c5")
    x, w, t, c, meta = cfg["x"], cfg["w"], cfg["target"], cfg["ce_weight"], cfg["meta"]
    loss, stats, dx = run_op(x, w, t, c)
    zr = meta["zero_row"]
    v = w.shape[0]
    np.testing.assert_allclose(stats["lse"][zr].item(), np.log(v), rtol=1e-5)
    np.testing.assert_allclose(stats["entropy"][zr].item(), np.log(v), rtol=1e-4)
    assert stats["argmax"][zr].item() == 0
    tie_rows = torch.tensor([p[0] for p in meta["tie_pairs"]])
    rows = torch.cat([torch.randperm(x.shape[0], generator=torch.Generator().manual_seed(2))[:64],
                      tie_rows, torch.tensor([zr, x.shape[0] - 1])]).unique()
    check_against_oracle(x, w, t, c, loss, stats, dx, rows=rows, tie_pairs=meta["tie_pairs"])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_vocab_shards_merge_to_full_vocab_on_one_gpu(dtype):
    """The vocab-parallel entry points (partial records with a vocabulary offset, record merge,
    per-shard dHidden with the global lse) emulated shard after shard on one GPU: three ragged
    shards must reproduce the single-shard result and the oracle."""
    from esep_soup_kernels_b200.head.op import DeviceBackend, _KEYS

    x, w, t, c = _peaked(333, 256, 7001, 0.1, 15.0, 9, dtype=dtype)
    xd, wd, td, cd = x.cuda(), w.cuda(), t.cuda(), c.cuda()
    bounds = [0, 2500, 2501, 7001]
    recs, bes = [], []
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        ws = wd[lo:hi].contiguous()
        be = DeviceBackend(xd, ws, True)
        recs.append(be.forward_partial(xd, ws, td, lo))
        bes.append((be, ws, lo))
    out = bes[0][0].finalize(torch.stack(recs), td, cd, w.shape[0])
    dx = sum(be.backward(xd, ws, td, out["cew"], out["lse"], lo) for be, ws, lo in bes)
    stats = {k: out[k] for k in _KEYS}
    check_against_oracle(x, w, t, c, out["loss"].reshape(()), stats, dx.to(x.dtype))
    loss1, stats1, dx1 = run_op(x, w, t, c)
    torch.testing.assert_close(out["loss"].reshape(()), loss1.detach(), rtol=1e-5, atol=1e-6)
    assert torch.equal(stats["argmax"], stats1["argmax"])
    torch.testing.assert_close(stats["lse"], stats1["lse"], rtol=1e-5, atol=1e-5)


def test_config4_shard_shape_7b_hidden():
    """Configuration 4 (vocab-parallel 7B shape) geometry on one shard: hidden 3584 (three passes of the backward over
    4 x 384 columns), one of eight vocabulary shards of 152064 (19008 rows), bf16, 5 % ignored."""
    from esep_soup_kernels_b200.head.op import DeviceBackend, _KEYS
    from esep_soup_kernels_b200.head.synthetic import make_config

    cfg = make_config("c4", n_override=300, v_override=19008)
    x, w, t, c = cfg["x"], cfg["w"], cfg["target"], cfg["ce_weight"]
    t = torch.where(t >= 0, t % 19008, t)
    loss, stats, dx = run_op(x, w, t, c)
    check_against_oracle(x, w, t, c, loss, stats, dx)


@pytest.mark.parametrize("n,h,v,dtype", [
    (300, 3584, 5003, torch.float16),      # three row tiles, each cut into vocabulary runs
    (2700, 3584, 3000, torch.bfloat16),    # 22 row tiles: full rounds on every cluster + a left-over
    (260, 3200, 2100, torch.bfloat16),     # 25 accumulator blocks: the last CTA's slice is ragged
])
def test_hidden_of_three_passes_runs_as_one_pass_on_eight_cta_clusters(n, h, v, dtype):
    """Hidden sizes whose dHidden accumulator needs three passes of the 4-CTA sweep (3200 - 3584
    columns) run on 8-CTA clusters that hold the whole accumulator: four CTAs compute logits and
    P, all eight accumulate dHidden, every logits tile is computed once. Same results as any
    other size; the library's counter shows that this kernel ran."""
    import ctypes
    from esep_soup_kernels_b200.head import _lib

    def wide_launches():
        buf = (ctypes.c_longlong * 4)()
        assert _lib.load().esep_head_debug_counters(buf, 4) == 0
        return buf[3]

    from esep_soup_kernels_b200.head.op import set_training_path

    g = torch.Generator().manual_seed(n + h + v)
    w = (torch.randn(v, h, generator=g) * (1.0 / h ** 0.5)).to(dtype)
    x = torch.randn(n, h, generator=g).to(dtype)
    t = torch.randint(0, v, (n,), generator=g)
    t[::17] = -100
    c = torch.rand(n, generator=g)
    c[t < 0] = 0.0
    before = wide_launches()
    set_training_path("single_pass")      # at these sizes the default is the two-sweep path
    try:
        loss, stats, dx = run_op(x, w, t, c)
        assert wide_launches() == before + 1
        check_against_oracle(x, w, t, c, loss, stats, dx)
        assert dx[::17].abs().max().item() == 0.0
        loss2, stats2, dx2 = run_op(x, w, t, c)
        assert torch.equal(loss, loss2) and torch.equal(dx, dx2)
    finally:
        set_training_path("auto")


def _dx_launches():
    import ctypes
    from esep_soup_kernels_b200.head import _lib

    buf = (ctypes.c_longlong * 5)()
    assert _lib.load().esep_head_debug_counters(buf, 5) == 0
    return buf[4]


@pytest.mark.parametrize("n,h,v,dtype,peak", [
    (300, 128, 5003, torch.float16, 25.0),     # the reference's unit-test shape, peaked targets
    (513, 1536, 3000, torch.float16, 30.0),    # real hidden size, ragged rows and vocabulary
    (1, 64, 257, torch.bfloat16, 0.0),         # one row, vocabulary just over one tile
    (700, 3584, 6000, torch.bfloat16, 10.0),   # 7B hidden: seven 512-column slices
    (2600, 704, 2100, torch.bfloat16, 5.0),    # eleven row pairs x two slices (the second ragged)
    (129, 192, 40000, torch.float16, 0.0),     # few units, long vocabulary: cut into runs
])
@pytest.mark.parametrize("path", ["stored_logits", "stored_weights"])
def test_two_sweeps_over_stored_logits_match_the_oracle(n, h, v, dtype, peak, path):
    """The training paths that keep the logits: forward sweep storing (logit - reference maximum)
    log2 e as fp16, then dHidden from the stored logits (P = one packed 2^x per two entries), or
    storing bf16 2^((logit - reference maximum) log2 e), which the dHidden kernel takes as it is;
    the target's own term is added in fp32. Same outputs, same tolerances, bit-identical when repeated;
    exact zeros on rows without a loss; the library's counter shows that the kernel ran."""
    from esep_soup_kernels_b200.head.op import set_training_path

    x, w, t, c = _peaked(n, h, v, 1.0 / h ** 0.5, peak, n + h, dtype=dtype)
    set_training_path(path)
    try:
        before = _dx_launches()
        loss, stats, dx = run_op(x, w, t, c)
        assert _dx_launches() == before + 1
        check_against_oracle(x, w, t, c, loss, stats, dx)
        assert dx[::7].abs().max().item() == 0.0
        loss2, stats2, dx2 = run_op(x, w, t, c)
        assert torch.equal(loss, loss2) and torch.equal(dx, dx2)
        for k in stats:
            assert torch.equal(stats[k], stats2[k])
        # many rows without a loss: they take the statistics-only sweep, the others this path
        t[: n // 2] = -100
        c[: n // 2] = 0.0
        loss3, stats3, dx3 = run_op(x, w, t, c)
        check_against_oracle(x, w, t, c, loss3, stats3, dx3)
        assert n < 2 or dx3[: n // 2].abs().max().item() == 0.0
    finally:
        set_training_path("auto")


def test_default_path_is_the_two_sweeps_and_both_paths_agree():
    """Default: two sweeps (bf16 softmax weights kept between them) wherever they apply (hidden a
    multiple of 64), the single pass otherwise or when asked for. Both paths agree to the rounding
    of their 16-bit softmax weights."""
    from esep_soup_kernels_b200.head.op import last_call_used_stored_logits, set_training_path

    set_training_path("auto")
    x, w, t, c = _peaked(400, 1536, 5000, 0.03, 8.0, 21, dtype=torch.bfloat16)
    loss_a, stats_a, dx_a = run_op(x, w, t, c)
    assert last_call_used_stored_logits("cuda:0")
    x1, w1, t1, c1 = _peaked(200, 72, 3000, 0.1, 8.0, 23, dtype=torch.float16)
    run_op(x1, w1, t1, c1)
    assert not last_call_used_stored_logits("cuda:0")        # hidden 72 is not a multiple of 64
    assert set_training_path("single_pass") == "auto"
    try:
        loss_b, stats_b, dx_b = run_op(x, w, t, c)
        assert not last_call_used_stored_logits("cuda:0")
    finally:
        assert set_training_path("auto") == "single_pass"
    torch.testing.assert_close(loss_a, loss_b, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(stats_a["lse"], stats_b["lse"], rtol=1e-5, atol=2e-5)
    assert torch.equal(stats_a["argmax"], stats_b["argmax"])
    rel = ((dx_a.float() - dx_b.float()).norm() / dx_b.float().norm()).item()
    assert rel < 5e-3, rel


def test_rows_without_a_loss_term_take_the_forward_sweep_and_get_zero_gradient():
    """With many ignored rows the library sweeps only the live rows for the gradient and gives
    the others their statistics from a forward sweep (the reference orders the live rows first
    and reads their count on the host, solution/head/op.py:112-117; here the order and the counts
    stay on the device). Every row keeps lse / entropy / argmax, dHidden is exactly zero on dead
    rows, and the result is a function of the call alone: the same call gives the same bits
    whatever ran before it."""
    x, w, t, c = _peaked(900, 256, 6007, 0.1, 15.0, 12)
    t[100:700] = -100                       # two thirds of the rows carry no loss
    c[100:700] = 0.0
    c[710:720] = 0.0                        # valid target, zero weight: ce but no gradient
    loss0, stats0, dx0 = run_op(x, w, t, c)
    check_against_oracle(x, w, t, c, loss0, stats0, dx0)
    assert dx0[100:700].abs().max().item() == 0.0 and dx0[710:720].abs().max().item() == 0.0
    # a different call in between (no dead rows at all) must not change the next result
    x2, w2, t2, c2 = _peaked(300, 256, 6007, 0.1, 15.0, 13)
    run_op(x2, w2, t2, c2)
    loss1, stats1, dx1 = run_op(x, w, t, c)
    assert torch.equal(loss0, loss1) and torch.equal(dx0, dx1)
    for k in stats0:
        assert torch.equal(stats0[k], stats1[k])
    # few dead rows (less than one in eight): they ride along in the sweep
    t3, c3 = t.clone(), c.clone()
    t3[100:700] = torch.randint(0, 6007, (600,), generator=torch.Generator().manual_seed(5))
    c3[100:700] = 1.0
    t3[::11] = -100
    loss3, stats3, dx3 = run_op(x, w, t3, c3)
    check_against_oracle(x, w, t3, c3, loss3, stats3, dx3)
    assert dx3[::11].abs().max().item() == 0.0
    # all rows dead: zero gradient, zero loss, statistics still there
    t[:] = -100
    loss2, stats2, dx2 = run_op(x, w, t, c)
    assert loss2.item() == 0.0 and dx2.abs().max().item() == 0.0
    torch.testing.assert_close(stats2["lse"], stats0["lse"], rtol=1e-5, atol=2e-5)


def test_argmax_is_exact_when_two_logits_are_a_few_ulp_apart():
    """Two logits 8 ulp apart with the LARGER one at the higher vocabulary index: the argmax
    must be that higher index in the single pass and in the forward sweep alike (first index
    of the exact maximum, solution/head/kernels.py:60, 75); bit-equal logits still resolve to
    the lower index."""
    from esep_soup_kernels_b200.head import fused_linear_ce

    g = torch.Generator().manual_seed(3)
    n, h, v = 130, 64, 3001
    lo, hi = 700, 2500
    # logits are x[0] w[j, 0] + x[1] w[j, 1] with x = (1, 2^-10, 0, ...): every other entry is
    # small noise in column 0, entry lo is 1, entry hi is 1 + 2^-20 = 1 + 8 ulp (fp32 at 1.0);
    # all inputs are exactly representable in fp16 and the sums are exact in fp32
    w = torch.zeros(v, h)
    w[:, 0] = torch.randn(v, generator=g) * 0.02
    w[lo, 0] = 1.0
    w[hi, 0] = 1.0
    w[hi, 1] = 2.0 ** -10
    x = torch.zeros(n, h)
    x[:, 0] = 1.0
    x[:, 1] = 2.0 ** -10
    w16 = w.half()
    z = (x.half().float() @ w16.float().t())
    assert z[0, hi] > z[0, lo] and (z[0, hi] - z[0, lo]) <= 2.0 ** -19
    assert int(z[0].argmax()) == hi
    t = torch.randint(0, v, (n,), generator=g)
    c = torch.ones(n)
    xd = x.half().cuda().requires_grad_(True)
    _, st = fused_linear_ce(xd, w16.cuda(), t.cuda(), c.cuda())            # single pass
    assert (st["argmax"].cpu() == hi).all()
    with torch.no_grad():
        _, st0 = fused_linear_ce(xd, w16.cuda(), t.cuda(), c.cuda())       # forward sweep
    assert (st0["argmax"].cpu() == hi).all()
    w16[hi] = w16[lo]                                                       # now bit-equal
    _, st = fused_linear_ce(xd, w16.cuda(), t.cuda(), c.cuda())
    assert (st["argmax"].cpu() == lo).all()


def test_metric_scalars_of_the_op_match_its_per_row_outputs():
    """The eight scalars the kernels reduce (what a data-parallel job all-reduces instead of the
    reference's five metric gathers, solution/head/patch.py:582-615) against the same sums formed
    from the per-row outputs on the host."""
    from esep_soup_kernels_b200.head import fused_linear_ce_with_metrics

    x, w, t, c = _peaked(333, 128, 4001, 0.2, 12.0, 8)
    t[::5] = -100
    t[3] = 4001 + 7                      # out of range but not -100: labelled, no CE term
    c[1::7] = 0.0
    xd = x.cuda().requires_grad_(True)
    loss, st, m = fused_linear_ce_with_metrics(xd, w.cuda(), t.cuda(), c.cuda())
    m = m.cpu()
    valid = (t >= 0) & (t < 4001)
    live = valid & (c != 0)
    ent = st["entropy"].cpu()
    np.testing.assert_allclose(m[0], loss.item(), rtol=1e-6)
    assert m[1] == float(valid.sum())
    assert m[2] == float(((st["argmax"].cpu() == t) & valid).sum())
    np.testing.assert_allclose(m[3], float(ent[valid].double().sum()), rtol=1e-5)
    assert m[4] == float((t != -100).sum())
    assert m[5] == float(t.numel())                       # no mask: every row counts as attended
    np.testing.assert_allclose(m[6], float(ent.double().sum()), rtol=1e-5)
    assert m[7] == float(live.sum())
    with torch.no_grad():
        _, _, m0 = fused_linear_ce_with_metrics(xd, w.cuda(), t.cuda(), c.cuda())
    np.testing.assert_allclose(m0.cpu()[:7], m[:7], rtol=1e-5)


def test_bf16_weight_copy_follows_the_weight_not_its_address():
    """Two training calls with same-shape fp16 weights created as temporaries (the second may
    land on the address the first one freed): each gradient must come from its own weight."""
    from esep_soup_kernels_b200.head import fused_linear_ce
    from oracle import head_oracle as ho

    g = torch.Generator().manual_seed(21)
    n, h, v = 140, 128, 2500
    x = torch.randn(n, h, generator=g).half()
    t = torch.randint(0, v, (n,), generator=g)
    c = torch.ones(n)
    for k in range(3):
        w = (torch.randn(v, h, generator=g) * (0.05 + 0.05 * k)).half()
        xd = x.cuda().requires_grad_(True)
        loss, _ = fused_linear_ce(xd, w.cuda(), t.cuda(), c.cuda())    # w.cuda() is a temporary
        loss.backward()
        ref = ho.full_vocab_reference(x, w, t, c, want_rounded=False)
        err = (xd.grad.float().cpu() - ref["dx"]).norm() / ref["dx"].norm()
        assert err < 1e-2, (k, float(err))


def test_warmup_from_a_worker_thread_and_no_one_time_work_afterwards():
    """The reference's warm-up contract (solution/head/op.py:47-65, solution/test_head.py:185-227):
    no launch, safe from a worker thread while the main thread uses the device, and the first
    real call afterwards finds nothing left to initialise. A repeated call encodes no tensor map
    again (they are cached by address and shape)."""
    import ctypes
    import threading

    from esep_soup_kernels_b200.head import _lib, fused_linear_ce, warmup

    def counters():
        buf = (ctypes.c_longlong * 2)()
        assert _lib.load().esep_head_debug_counters(buf, 2) == 0
        return buf[0], buf[1]

    x, w, t, c = _peaked(200, 128, 3001, 0.1, 10.0, 4)
    xd, wd, td, cd = x.cuda().requires_grad_(True), w.cuda(), t.cuda(), c.cuda()
    errors = []

    def worker():
        try:
            warmup("cuda:0")
            warmup()
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    th = threading.Thread(target=worker)
    th.start()
    busy = torch.randn(512, 512, device="cuda")
    for _ in range(20):
        busy = busy @ busy * 1e-3              # the main thread keeps the device busy meanwhile
    th.join()
    assert not errors
    inits, _ = counters()
    assert inits >= 1
    loss, _ = fused_linear_ce(xd, wd, td, cd)
    loss.backward()
    inits1, maps1 = counters()
    assert inits1 == inits                      # nothing left to initialise after the warm-up
    ws_keep = []
    for _ in range(2):
        xd.grad = None
        loss2, _ = fused_linear_ce(xd, wd, td, cd)
        loss2.backward()
        ws_keep.append(loss2)
    inits2, maps2 = counters()
    assert inits2 == inits
    # the weight's maps are reused; only maps of freshly allocated scratch may be new (per call at
    # most: the compact rows as the forward and as the guarded backward kernel read them, the
    # stored weights as they are written and as they are read)
    assert maps2 - maps1 <= 2 * 4
    assert torch.equal(loss.detach(), loss2.detach())


def test_bounded_wait_gives_up_and_leaves_the_context_usable():
    """Failure detection without faulting the GPU: a wait that can never complete returns after
    its limit, the kernel records a status code and exits normally, the host reads
    ESEP_ERR_DEVICE_TIMEOUT, and the next call on the same context works."""
    import ctypes

    from esep_soup_kernels_b200.head import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    ws = torch.zeros(256, dtype=torch.uint8, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    code = lib.esep_head_selftest_bounded_wait(ctypes.c_void_p(ws.data_ptr()), 256, 2_000_000, stream)
    assert code == 0
    word = ctypes.c_int(0)
    code = lib.esep_head_device_status(ctypes.c_void_p(ws.data_ptr()), stream, ctypes.byref(word))
    assert code == -5 and word.value == 901
    assert "bounded wait" in _lib.status_string(code)
    x, w, t, c = _peaked(77, 64, 1001, 0.3, 20.0, 0)
    loss, stats, dx = run_op(x, w, t, c)          # run_op asserts a clean status word
    check_against_oracle(x, w, t, c, loss, stats, dx)


def test_causal_lm_head_step_matches_the_logits_path():
    """The caller-side step (label shift, row gather, scatter back to [B, T], counts) against the
    oracle's restatement of the reference's logits path (solution/head/patch.py:562-579);
    tolerances of solution/test_head_patch.py:102-117 (loss 1e-3, per-token 2e-3)."""
    from esep_soup_kernels_b200.head.step import HeadWeight, causal_lm_head_step, step_metrics
    from oracle import head_oracle as ho

    g = torch.Generator().manual_seed(31)
    bsz, seq, h, v = 3, 37, 64, 1003
    weight = torch.randn(v, h, generator=g) * 0.3
    hidden = torch.randn(bsz, seq, h, generator=g)
    labels = torch.randint(0, v, (bsz, seq), generator=g)
    mask = torch.ones(bsz, seq, dtype=torch.long)
    mask[0, 30:] = 0
    mask[2, 11:] = 0
    labels[mask == 0] = -100
    labels[:, :5] = -100                                  # prompt tokens carry no loss
    cache = HeadWeight(torch.float16)
    w16 = cache.weight16(weight.cuda())
    hd = hidden.cuda().requires_grad_(True)
    loss, step = causal_lm_head_step(hd, labels.cuda(), w16, attention_mask=mask.cuda())
    loss.backward()
    ref = ho.step_from_logits(hidden.half(), weight.half(), labels, want_grad=True)
    np.testing.assert_allclose(loss.item(), ref["loss_mean"], rtol=1e-3)
    rows = ((mask != 0) | (torch.nn.functional.pad(labels, (0, 1), value=-100)[:, 1:] != -100))
    torch.testing.assert_close(step.token_loss.cpu(), ref["token_loss"], rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(step.token_entropy.cpu()[rows], ref["token_entropy"][rows],
                               rtol=2e-3, atol=2e-3)
    assert (step.token_entropy.cpu()[~rows] == 0).all()
    assert int(step.labelled) == ref["labelled"] and abs(int(step.correct) - ref["correct"]) <= 1
    assert hd.grad.shape == hidden.shape and hd.grad[mask.cuda() == 0].abs().max().item() == 0.0
    m = step_metrics(step, attention_mask=mask.cuda())
    assert m["num_tokens"] == int(mask.sum())
    np.testing.assert_allclose(m["entropy"],
                               float((ref["token_entropy"] * mask).sum() / mask.sum()), rtol=2e-3)
    # num_items_in_batch normalisation (patch.py:461-468)
    loss2, _ = causal_lm_head_step(hd, labels.cuda(), w16, attention_mask=mask.cuda(),
                                   num_items_in_batch=torch.tensor(50))
    np.testing.assert_allclose(loss2.item(), ref["loss_mean"] * ref["labelled"] / 50, rtol=1e-3)
    loss2.backward()
    # dHidden of the two backward calls so far (mean loss, then the sum over 50 items)
    want = ref["dhidden"] * (1.0 + ref["labelled"] / 50)
    assert float((hd.grad.float().cpu() - want).norm() / want.norm()) < 1e-2
    # without gradient (evaluation): same per-token results from the forward sweep alone
    with torch.no_grad():
        loss3, step3 = causal_lm_head_step(hd, labels.cuda(), w16, attention_mask=mask.cuda())
    np.testing.assert_allclose(loss3.item(), loss.item(), rtol=1e-5)
    torch.testing.assert_close(step3.token_loss, step.token_loss, rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(step3.token_entropy, step.token_entropy, rtol=1e-5, atol=2e-5)
    assert int(step3.correct) == int(step.correct)
    # fp32 hidden states and no attention mask: every position is a row
    h32 = hidden.cuda().requires_grad_(True)
    loss4, step4 = causal_lm_head_step(h32, labels.cuda(), w16)
    loss4.backward()
    assert h32.grad.dtype == torch.float32
    np.testing.assert_allclose(loss4.item(), ref["loss_mean"], rtol=1e-3)
    torch.testing.assert_close(step4.token_entropy.cpu(), ref["token_entropy"], rtol=2e-3, atol=2e-3)
    assert step_metrics(step4)["num_tokens"] == bsz * seq


def _planted_outlier_case(scale, h=64):
    """One row whose logit at a vocabulary index past the 2 048-row prefix is about `scale`, far
    above everything the prefix holds."""
    g = torch.Generator().manual_seed(17)
    n, v = 150, 5000
    w = (torch.randn(v, h, generator=g) * 0.3 * (64.0 / h) ** 0.5).half()
    x = torch.randn(n, h, generator=g).half()
    t = torch.randint(0, v, (n,), generator=g)
    c = torch.rand(n, generator=g)
    star = 4321
    x[7] = (scale * w[star].float() / w[star].float().pow(2).sum()).half()
    t[7] = star
    return x, w, t, c


def test_single_sweep_falls_back_when_a_row_maximum_is_far_above_the_prefix():
    """The single sweep takes its softmax weights relative to the row maximum over the first 2 048
    vocabulary rows (plus a margin of 40). A row whose true maximum is more than 115 above the
    prefix maximum must raise the flag, and the guarded two-kernel path queued in the same call
    must deliver the correct outputs; smaller outliers are handled by the sweep itself."""
    from esep_soup_kernels_b200.head.op import last_call_fell_back, set_training_path

    set_training_path("single_pass")
    x, w, t, c = _planted_outlier_case(600.0)
    z7 = x[7].float() @ w.float().T
    assert float(z7.max() - z7[:2048].max()) > 200.0          # the case is what it claims to be
    loss, stats, dx = run_op(x, w, t, c)
    assert last_call_fell_back("cuda:0")
    check_against_oracle(x, w, t, c, loss, stats, dx)
    for scale, lo, hi in ((60.0, 10.0, 55.0), (150.0, 60.0, 110.0)):
        x, w, t, c = _planted_outlier_case(scale)
        z7 = x[7].float() @ w.float().T
        assert lo < float(z7.max() - z7[:2048].max()) < hi
        loss, stats, dx = run_op(x, w, t, c)
        assert not last_call_fell_back("cuda:0")
        check_against_oracle(x, w, t, c, loss, stats, dx)
    # the same guard behind the 8-CTA-cluster sweep (hidden 3584) and behind the two sweeps that
    # keep bf16 weights relative to the same reference; the two sweeps over fp16 logits know the
    # true maximum before they form a weight and need no guard
    x, w, t, c = _planted_outlier_case(600.0, h=3584)
    try:
        for path, falls_back in (("single_pass", True), ("stored_weights", True),
                                 ("stored_logits", False)):
            set_training_path(path)
            loss, stats, dx = run_op(x, w, t, c)
            assert last_call_fell_back("cuda:0") == falls_back
            check_against_oracle(x, w, t, c, loss, stats, dx)
        x, w, t, c = _planted_outlier_case(150.0)
        set_training_path("stored_weights")
        loss, stats, dx = run_op(x, w, t, c)
        assert not last_call_fell_back("cuda:0")
        check_against_oracle(x, w, t, c, loss, stats, dx)
    finally:
        set_training_path("auto")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_single_sweep_and_two_kernel_path_agree(dtype):
    """The same call through both training paths: statistics to fp32 rounding, dHidden within the
    16-bit rounding of the softmax weights, exact zeros on the rows without a loss."""
    from esep_soup_kernels_b200.head import op

    x, w, t, c = _peaked(700, 256, 9001, 0.1, 12.0, 9)
    x, w = x.to(dtype), w.to(dtype)
    t[::6] = -100
    c[5::9] = 0.0
    loss1, stats1, dx1 = run_op(x, w, t, c)
    assert op.SINGLE_SWEEP
    op.SINGLE_SWEEP = False
    try:
        loss2, stats2, dx2 = run_op(x, w, t, c)
    finally:
        op.SINGLE_SWEEP = True
    np.testing.assert_allclose(float(loss1.detach()), float(loss2.detach()), rtol=1e-5)
    for k in ("lse", "entropy", "ce", "target_logit"):
        np.testing.assert_allclose(stats1[k].cpu().numpy(), stats2[k].cpu().numpy(), rtol=1e-5,
                                   atol=2e-5)
    assert torch.equal(stats1["argmax"], stats2["argmax"])
    a, b = dx1.float(), dx2.float()
    assert float((a - b).norm() / b.norm()) < 5e-3
    dead = ((t < 0) | (c == 0)).to(a.device)
    assert float(a[dead].abs().max()) == 0.0 and float(b[dead].abs().max()) == 0.0
    check_against_oracle(x, w, t, c, loss2, stats2, dx2)


def test_train_entry_point_rejects_bad_arguments_and_reports_its_workspace(training_path):
    """esep_head_train through the C ABI: workspace query, argument checks, no launch on error."""
    import ctypes

    from esep_soup_kernels_b200.head import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    n, h, v = 130, 64, 700
    x = torch.zeros(n, h, device=dev, dtype=torch.float16)
    w = torch.zeros(v, h, device=dev, dtype=torch.float16)
    wb = w.bfloat16()
    t = torch.zeros(n, device=dev, dtype=torch.int64)
    c = torch.ones(n, device=dev)
    f = lambda *s: torch.zeros(*s, device=dev)
    lse, tl, ce, ent, cew, loss, met, dx = f(n), f(n), f(n), f(n), f(n), f(1), f(4), f(n, h)
    am = torch.zeros(n, device=dev, dtype=torch.int64)
    flag = torch.zeros(1, device=dev, dtype=torch.int32)
    P = lambda a: ctypes.c_void_p(a.data_ptr())
    with torch.cuda.device(dev):
        need = lib.esep_head_train_workspace_bytes(n, h, v, _lib.DTYPE_F16)
        assert need > lib.esep_head_workspace_bytes(n, h, v, _lib.DTYPE_F16, 1) > 0
        assert lib.esep_head_train_workspace_bytes(n, 60, v, _lib.DTYPE_F16) == 0     # h % 8
        assert lib.esep_head_train_workspace_bytes(n, h, v, 7) == 0                   # dtype
        ws = torch.zeros(need, device=dev, dtype=torch.uint8)
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

        def call(wb_ptr=P(wb), ws_bytes=need, flag_ptr=P(flag)):
            return lib.esep_head_train(P(x), P(w), wb_ptr, P(t), P(c), n, h, v, _lib.DTYPE_F16,
                                       P(lse), P(tl), P(ce), P(ent), P(am), P(cew), P(loss), P(met),
                                       P(dx), flag_ptr, P(ws), ws_bytes, st)

        # the two sweeps over fp16 logits are the one path that reads no bf16 copy of W
        uses_stored = lib.esep_head_step_uses_stored_logits(n, h, v, _lib.DTYPE_F16, 1)
        assert uses_stored == {"two_sweeps": 2, "stored_logits": 1, "single_pass": 0}[training_path]
        assert call(wb_ptr=None) == (0 if uses_stored == 1 else _lib.ERR_BAD_ARG)
        assert call(flag_ptr=None) == _lib.ERR_BAD_ARG
        assert call(ws_bytes=need - 256) == _lib.ERR_WORKSPACE
        assert call() == 0
        torch.cuda.synchronize()
    # all-zero inputs: uniform softmax, every logit 0, argmax 0
    np.testing.assert_allclose(lse.cpu().numpy(), np.log(v), rtol=1e-6)
    np.testing.assert_allclose(ent.cpu().numpy(), np.log(v), rtol=1e-5)
    assert int(am.abs().max()) == 0 and int(flag) == 0
    np.testing.assert_allclose(float(loss), n * np.log(v), rtol=1e-5)


@pytest.mark.parametrize("sweep", [True, False])
def test_vocab_parallel_entry_with_one_shard(sweep):
    """head/parallel.py::vocab_parallel_linear_ce without a process group (one shard = the whole
    vocabulary): the single-sweep composition and the record-exchange form against the oracle."""
    from esep_soup_kernels_b200.head import last_device_status
    from esep_soup_kernels_b200.head.parallel import vocab_parallel_linear_ce

    x, w, t, c = _peaked(333, 256, 5003, 0.1, 12.0, 21)
    t[::4] = -100
    dev = torch.device("cuda", 0)
    loss, stats, dx = vocab_parallel_linear_ce(x.to(dev), w.to(dev), t.to(dev), c.to(dev), 0,
                                               w.shape[0], single_sweep=sweep)
    assert last_device_status(dev) == 0 and dx.dtype == torch.float32
    check_against_oracle(x, w, t, c, loss, stats, dx.to(x.dtype))   # the op hands dx back in x.dtype
