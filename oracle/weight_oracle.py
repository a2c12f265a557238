"""CPU oracle for the shared fp16 head / embedding weight.  TEST INFRASTRUCTURE ONLY.

Restates, in numpy, what the reference's ``_Fp16Fixup`` computes (paths inside the reference
project): only tests/ may import this file; the product package never does.

  fixup_table      solution/head/patch.py:141-153  elements whose fp16 value does not give back
                                                   the fp32 bits: flat index (ascending) + value
  table_shape      solution/head/patch.py:155-160  rows with entries, most entries in one row
  apply_rows       solution/head/patch.py:201-210  restore the exact values of looked-up rows
  embedding_rows   solution/head/patch.py:217-226  fp16 gather + upcast + apply_rows
  exact_weight     solution/head/patch.py:212-215  the whole fp32 weight, rebuilt

Parity pin: tests/golden/fp16_fixup.npz holds the outputs of the REFERENCE's own class on seeded
CPU tensors (tests/golden/make_golden_fixup.py); tests/test_oracle.py checks every function here
against it, bit for bit. All comparisons are on the 32-bit patterns, so NaN payloads and the sign
of zero count.

NaN: which NaNs need an entry depends on the machine's fp16 -> fp32 conversion (the host keeps the
payload, a GPU returns the canonical NaN), so a table built on a GPU can hold NaN entries this
restatement does not; the looked-up rows and the rebuilt weight are the fp32 weight's bits either
way, and on NaN-free weights the tables are identical. The GPU tests compare accordingly.
"""

import numpy as np


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.int32)


def fixup_table(w32, w16):
    """(flat_idx int64 [K] ascending, flat_val fp32 [K]) for w32 fp32 [V, H], w16 fp16 [V, H]."""
    back = w16.astype(np.float32)
    bad = np.flatnonzero(_bits(back).reshape(-1) != _bits(w32).reshape(-1)).astype(np.int64)
    return bad, np.ascontiguousarray(w32, dtype=np.float32).reshape(-1)[bad].copy()


def table_shape(flat_idx, h):
    """(count, rows with entries, most entries in one row; 1 for an empty table)."""
    if flat_idx.size == 0:
        return 0, 0, 1
    _, counts = np.unique(flat_idx // h, return_counts=True)
    return int(flat_idx.size), int(counts.size), int(counts.max())


def apply_rows(out, ids, flat_idx, flat_val, h):
    """out [N, H] fp32 (upcast fp16 rows of ids [N]) with the exact values written back."""
    out = out.copy()
    rows = flat_idx // h
    cols = flat_idx % h
    for i, r in enumerate(np.asarray(ids).reshape(-1)):
        sel = rows == r
        out[i, cols[sel]] = flat_val[sel]
    return out


def embedding_rows(w16, ids, flat_idx, flat_val):
    ids = np.asarray(ids).reshape(-1)
    return apply_rows(w16[ids].astype(np.float32), ids, flat_idx, flat_val, w16.shape[1])


def exact_weight(w16, flat_idx, flat_val):
    w = w16.astype(np.float32)
    w.reshape(-1)[flat_idx] = flat_val
    return w
