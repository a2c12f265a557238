"""The CPU oracle against the golden vectors produced by the reference's own code
(tests/golden/make_golden.py): row-kernel restatement, chunked op restatement, fp32 reference,
record merge. CPU only."""

import glob
import os

import numpy as np
import pytest
import torch

from oracle import head_oracle as ho

GOLDEN = sorted(p for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz"))
                if not os.path.basename(p).startswith(("final_norm", "fp16_fixup")))   # head cases only


def _load(path):
    d = dict(np.load(path))
    x = torch.from_numpy(d["x"].view(np.int16)).view(torch.float16)
    w = torch.from_numpy(d["w"].view(np.int16)).view(torch.float16)
    return d, x, w, torch.from_numpy(d["target"]), torch.from_numpy(d["ce_weight"])


def test_golden_files_present():
    assert len(GOLDEN) == 3


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_full_vocab_reference_matches_reference_unit_test_oracle(path):
    d, x, w, t, c = _load(path)
    ref = ho.full_vocab_reference(x, w, t, c)
    np.testing.assert_allclose(float(ref["loss"]), float(d["ref_loss"]), rtol=1e-6)
    for k in ("lse", "tlogit", "ent", "maxlogit", "lse16", "tlogit16", "ent16"):
        np.testing.assert_allclose(ref[k].numpy(), d["ref_" + k], rtol=1e-5, atol=1e-5, err_msg=k)
    np.testing.assert_allclose(ref["dx"].numpy(), d["ref_dx"], rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_chunked_op_restatement_matches_reference_op(path):
    """chunked_op (op.py + kernels.py restated) vs the reference op run under the Triton interpreter."""
    d, x, w, t, c = _load(path)
    loss, (lse, tl, ce, ent, amax), dx = ho.chunked_op(x, w, t, c, True, int(d["chunk_rows"]))
    np.testing.assert_allclose(float(loss), float(d["op_loss"]), rtol=2e-6)
    np.testing.assert_allclose(lse.numpy(), d["op_lse"], rtol=1e-6, atol=1e-5)
    np.testing.assert_allclose(tl.numpy(), d["op_tlogit"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(ce.numpy(), d["op_ce"], rtol=1e-6, atol=1e-5)
    np.testing.assert_allclose(ent.numpy(), d["op_ent"], rtol=1e-5, atol=1e-5)
    assert (amax.numpy() == d["op_argmax"]).all()          # same first-index tie rule
    np.testing.assert_allclose(dx.numpy(), d["op_dx"], rtol=1e-4, atol=1e-8)


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_row_kernel_pass2_matches_triton_g_rows(path):
    d, x, w, t, c = _load(path)
    z = (x.float() @ w.float().T).half().float().numpy()
    g_ref = d["g_rows"].view(np.float16).astype(np.float32)
    for k, row in enumerate(d["g_idx"]):
        tg = int(t[row])
        lse, _, _, _ = ho.row_softmax_pass1(z[row], tg)
        g = ho.row_softmax_pass2(z[row], lse, tg).astype(np.float32)
        # one fp16 ulp of slack: exp() of numpy vs the interpreter's
        np.testing.assert_allclose(g, g_ref[k], rtol=2e-3, atol=1e-6)


def test_ties_take_lowest_index_and_zero_row_is_uniform():
    d, x, w, t, c = _load([p for p in GOLDEN if "ties" in p][0])
    v = w.shape[0]
    for r, j1, j2 in d["tie_pairs"]:
        assert d["op_argmax"][r] == min(j1, j2)
    assert d["op_argmax"][1] == 0
    np.testing.assert_allclose(d["op_lse"][1], np.log(v), rtol=1e-6)
    np.testing.assert_allclose(d["op_ent"][1], np.log(v), rtol=1e-5)
    rec = ho.partial_record(x, w, t)
    fin = ho.finalize_records(rec[None], t.numpy(), c.numpy(), v)
    for r, j1, j2 in d["tie_pairs"]:
        assert fin["argmax"][r] == min(j1, j2)
    assert fin["argmax"][1] == 0


@pytest.mark.parametrize("shards", [2, 3, 8])
def test_vocab_shard_records_merge_to_full_vocab(shards):
    """partial_record over vocabulary shards + merge_records == one full-vocabulary record,
    and the shard dX partials sum to the full gradient."""
    d, x, w, t, c = _load([p for p in GOLDEN if "small_odd" in p][0])
    v = w.shape[0]
    bounds = np.linspace(0, v, shards + 1).astype(int)
    recs = np.stack([ho.partial_record(x, w[a:b], t, int(a)) for a, b in zip(bounds[:-1], bounds[1:])])
    fin = ho.finalize_records(recs, t.numpy(), c.numpy(), v)
    np.testing.assert_allclose(fin["lse"], d["ref_lse"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(fin["entropy"], d["ref_ent"], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(fin["target_logit"], d["ref_tlogit"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(fin["loss"], float(d["ref_loss"]), rtol=1e-5)
    ref = ho.full_vocab_reference(x, w, t, c)
    assert (fin["argmax"] == ref["argmax"].numpy()).all()
    dx = sum(ho.shard_dx(x, w[a:b], t, fin["cew"], fin["lse"], int(a))
             for a, b in zip(bounds[:-1], bounds[1:]))
    np.testing.assert_allclose(dx.numpy(), d["ref_dx"], rtol=1e-3, atol=1e-6)
