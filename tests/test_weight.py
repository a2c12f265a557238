"""The shared fp16 head / embedding weight (head/weight.py, csrc/head_weight.cuh).

CPU: the numpy oracle against the fixture made by the reference's own ``_Fp16Fixup``
(tests/golden/make_golden_fixup.py). GPU: the CUDA table and lookup kernels against the fixture
and the oracle, bit for bit (32-bit patterns: NaN payloads and signed zeros count), with the
cases of the reference's unit test (solution/test_head_patch.py:299-316)."""

import os

import numpy as np
import pytest
import torch

from oracle import weight_oracle as wo

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "fp16_fixup.npz")
CASES = ("unit", "rows")


def _case(name):
    d = np.load(GOLDEN)
    g = {k[len(name) + 1:]: d[k] for k in d.files if k.startswith(name + "_")}
    g["w32"] = g["w32_bits"].view(np.float32)
    g["w16"] = g["w16_bits"].view(np.float16)
    return g


def _bits(t):
    return t.detach().contiguous().view(torch.int32).cpu().numpy()


@pytest.mark.parametrize("name", CASES)
def test_oracle_table_and_lookups_match_the_reference_class(name):
    g = _case(name)
    flat_idx, flat_val = wo.fixup_table(g["w32"], g["w16"])
    assert np.array_equal(flat_idx, g["flat_idx"])
    assert np.array_equal(flat_val.view(np.int32), g["flat_val_bits"])
    assert wo.table_shape(flat_idx, g["w32"].shape[1]) == (int(g["count"]), int(g["rows"]),
                                                            int(g["width"]))
    out = wo.embedding_rows(g["w16"], g["ids"], flat_idx, flat_val)
    assert np.array_equal(out.view(np.int32), g["apply_rows_bits"])
    assert np.array_equal(wo.exact_weight(g["w16"], flat_idx, flat_val).view(np.int32),
                          g["exact_weight_bits"])
    # what the format promises: the lookup returns the fp32 weight's rows, the rebuild the weight
    assert np.array_equal(g["apply_rows_bits"], g["w32_bits"][g["ids"]])
    assert np.array_equal(g["exact_weight_bits"], g["w32_bits"])


def test_oracle_empty_table():
    w16 = np.linspace(-2, 2, 64 * 16, dtype=np.float32).astype(np.float16).reshape(64, 16)
    flat_idx, flat_val = wo.fixup_table(w16.astype(np.float32), w16)
    assert flat_idx.size == 0 and wo.table_shape(flat_idx, 16) == (0, 0, 1)
    ids = np.array([5, 0, 63])
    assert np.array_equal(wo.embedding_rows(w16, ids, flat_idx, flat_val), w16[ids].astype(np.float32))


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_cuda_table_and_lookups_match_the_reference_class(name):
    from esep_soup_kernels_b200.head.weight import Fp16Fixup, embedding_forward16

    g = _case(name)
    w32 = torch.from_numpy(g["w32_bits"]).view(torch.float32).cuda()
    w16 = torch.from_numpy(g["w16_bits"]).view(torch.float16).cuda()
    ids = torch.from_numpy(g["ids"]).cuda()
    fix = Fp16Fixup(w32, w16)
    # The table is defined by the DEVICE's fp16 -> fp32 conversion (the reference's criterion,
    # solution/test_head_patch.py:312). It differs from the host's only on NaNs: the GPU returns
    # the canonical NaN, so a NaN that survives the round trip on the host needs an entry here
    # (the reference's own test expects that entry on the GPU: "count >= 4", :313).
    dev_idx = (w16.float().view(torch.int32) != w32.view(torch.int32)).reshape(-1).nonzero()[:, 0]
    assert torch.equal(fix.flat_idx, dev_idx) and fix.count == dev_idx.numel()
    assert torch.equal(fix.flat_val.view(torch.int32), w32.reshape(-1)[dev_idx].view(torch.int32))
    host_idx = g["flat_idx"]
    extra = np.setdiff1d(fix.flat_idx.cpu().numpy(), host_idx)
    assert np.isin(host_idx, fix.flat_idx.cpu().numpy()).all()
    assert np.isnan(g["w32"].reshape(-1)[extra]).all()
    if name == "rows":          # no NaN in this case: the reference's table, entry for entry
        assert (fix.count, fix.rows, fix.width) == (int(g["count"]), int(g["rows"]), int(g["width"]))
        assert np.array_equal(fix.flat_idx.cpu().numpy(), host_idx)
        assert np.array_equal(_bits(fix.flat_val), g["flat_val_bits"])
    else:
        assert fix.count >= 4 and fix.rows == 2      # solution/test_head_patch.py:313
    # apply_rows on upcast rows (the reference's two-step form), and the one-kernel lookup
    out = fix.apply_rows(w16[ids].float(), ids)
    assert np.array_equal(_bits(out), g["apply_rows_bits"])
    emb = embedding_forward16(w16, fix, ids.view(1, -1))
    assert emb.shape == (1, ids.numel(), w32.shape[1]) and emb.dtype == torch.float32
    assert np.array_equal(_bits(emb).reshape(ids.numel(), -1), g["apply_rows_bits"])
    assert np.array_equal(_bits(fix.exact_weight(w16)), g["exact_weight_bits"])
    assert not fix.bad_index_seen()


@pytest.mark.gpu
def test_cast_and_count_in_one_pass_at_the_real_hidden_size():
    """``Fp16Fixup.cast`` produces the fp16 tensor torch produces on the device and the same
    table as the two-tensor constructor; the lookup returns the fp32 rows bit for bit. 20 000 x
    1536 with values below fp16's normal range, overflows, NaNs with payloads, infinities and
    negative zeros planted at seeded places (up to 40 in one row)."""
    from esep_soup_kernels_b200.head.weight import Fp16Fixup, share_fp16_weight

    g = torch.Generator().manual_seed(11)
    v, h = 20000, 1536
    w = (torch.randn(v, h, generator=g) * 0.02).to(torch.bfloat16).float()
    rows = torch.randint(0, v, (900,), generator=g)
    cols = torch.randint(0, h, (900,), generator=g)
    w[rows, cols] = ((torch.rand(900, generator=g) * 2 - 1) * 4e-6).to(torch.bfloat16).float()
    w[17, :40] = 1.0e-9
    w[v - 1, h - 1] = -7.0e4
    w[5, 3] = float("inf")
    w[5, 4] = -0.0
    wb = w.view(torch.int32)
    wb[6, 0] = 0x7FC01234          # quiet NaN with a payload
    wb[6, 9] = -8388607            # 0xFF800001: signalling NaN, sign set
    w32 = w.cuda()
    w16_torch = w32.half()
    w16, fix = Fp16Fixup.cast(w32)
    assert torch.equal(w16.view(torch.int16), w16_torch.view(torch.int16))
    dev_idx = (w16_torch.float().view(torch.int32) != w32.view(torch.int32)).reshape(-1).nonzero()[:, 0]
    assert torch.equal(fix.flat_idx, dev_idx) and fix.count > 900
    assert torch.equal(fix.flat_val.view(torch.int32), w32.reshape(-1)[dev_idx].view(torch.int32))
    assert (fix.count, fix.rows, fix.width) == wo.table_shape(dev_idx.cpu().numpy(), h)
    # the host oracle agrees on everything that is not a NaN
    ref_idx, _ = wo.fixup_table(w.numpy(), w16_torch.cpu().numpy())
    finite = ~np.isnan(w.numpy().reshape(-1))
    assert np.array_equal(ref_idx[finite[ref_idx]], dev_idx.cpu().numpy()[finite[dev_idx.cpu().numpy()]])
    two = Fp16Fixup(w32, w16_torch)
    assert torch.equal(two.flat_idx, fix.flat_idx) and torch.equal(two.row_start, fix.row_start)
    ids = torch.cat([rows[:300], torch.tensor([17, v - 1, 5, 6, 0, 17]),
                     torch.randint(0, v, (2000,), generator=g)]).cuda().view(2, -1)
    emb = fix.embed(w16, ids)
    assert np.array_equal(_bits(emb), _bits(w32[ids]))
    assert np.array_equal(_bits(fix.exact_weight(w16)), _bits(w32))
    assert fix.nbytes() == fix.count * 12 + (v + 1) * 4
    # the refusal rule of the reference (more than 64 entries in one row, or more than 1 %)
    assert share_fp16_weight(w32) is not None
    with pytest.warns(UserWarning, match="kept in fp32"):
        assert share_fp16_weight(w32, max_per_row=39) is None


@pytest.mark.gpu
def test_weight_that_is_exactly_fp16_needs_no_table_and_bad_ids_are_reported():
    from esep_soup_kernels_b200.head.weight import Fp16Fixup

    g = torch.Generator().manual_seed(3)
    w16 = torch.randn(777, 64, generator=g).half().cuda()
    fix = Fp16Fixup.exact(w16)
    assert (fix.count, fix.rows, fix.width) == (0, 0, 1) and fix.nbytes() == 0
    ids = torch.tensor([[0, 776, 5], [5, 5, 123]]).cuda()
    assert torch.equal(fix.embed(w16, ids), w16[ids].float())
    assert torch.equal(fix.exact_weight(w16), w16.float())
    built = Fp16Fixup(w16.float(), w16)          # the same through the counting pass
    assert built.count == 0 and torch.equal(built.embed(w16, ids), w16[ids].float())
    out = w16[ids.view(-1)].float()
    assert fix.apply_rows(out, ids) is out
    # an id outside the vocabulary: a zero row and a status word, nothing read out of bounds
    bad = torch.tensor([3, 777, -1, 4]).cuda()
    emb = built.embed(w16, bad)
    assert torch.equal(emb[0], w16[3].float()) and torch.equal(emb[3], w16[4].float())
    assert emb[1].abs().max().item() == 0.0 and emb[2].abs().max().item() == 0.0
    assert built.bad_index_seen() and not built.bad_index_seen()
    assert torch.equal(built.embed(w16, ids), w16[ids].float())      # the context stays usable
