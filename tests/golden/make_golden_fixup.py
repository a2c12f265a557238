"""Writes tests/golden/fp16_fixup.npz from the REFERENCE's own ``_Fp16Fixup``
(solution/head/patch.py:133-215) run on seeded CPU tensors. Needs the reference checkout:

    python tests/golden/make_golden_fixup.py /path/to/reference

Two cases. "unit": the tensor of the reference's own unit test
(solution/test_head_patch.py:299-316: subnormal-range values, an fp16 overflow, a NaN, a negative
zero). "rows": a bf16-representable weight with planted values below fp16's normal range in a few
rows, up to 6 per row (the shape of solution/test_head_patch.py:268-286), 512 x 32.
Everything is stored as bit patterns (int32 / int16) so that NaNs and signed zeros survive.
"""

import os
import sys

import numpy as np
import torch


def _i32(t):
    return t.contiguous().view(torch.int32).numpy().copy()


def _case(fix_cls, w, ids):
    w16 = w.half()
    fix = fix_cls(w, w16)
    out = fix.apply_rows(w16[ids].float(), ids)
    return {"w32_bits": _i32(w), "w16_bits": w16.view(torch.int16).numpy().copy(),
            "ids": ids.numpy().copy(), "flat_idx": fix.flat_idx.numpy().copy(),
            "flat_val_bits": _i32(fix.flat_val), "count": np.int64(fix.count),
            "rows": np.int64(fix.rows), "width": np.int64(fix.width),
            "apply_rows_bits": _i32(out), "exact_weight_bits": _i32(fix.exact_weight(w16))}


def main(ref_root):
    sys.path.insert(0, ref_root)
    from solution.head.patch import _Fp16Fixup

    out = {}
    g = torch.Generator().manual_seed(5)
    w = torch.randn(300, 48, generator=g).to(torch.bfloat16).float()
    w[3, 5] = 1.9e-11
    w[3, 6] = -2.5e-7
    w[17, 0] = 1e5
    w[17, 47] = float("nan")
    w[200, 1] = -0.0
    ids = torch.tensor([3, 17, 0, 3, 200, 299, 17])
    for k, val in _case(_Fp16Fixup, w, ids).items():
        out["unit_" + k] = val

    g = torch.Generator().manual_seed(7)
    v, h = 512, 32
    w = (torch.randn(v, h, generator=g) * 0.02).to(torch.bfloat16).float()
    planted = (0, 3, 7, 100, 300, v - 1)
    for i, row in enumerate(planted):
        cols = torch.randperm(h, generator=g)[: 1 + i % 6]
        vals = (torch.rand(cols.numel(), generator=g) * 2 - 1) * 3e-6
        w[row, cols] = vals.to(torch.bfloat16).float()
    ids = torch.cat([torch.tensor(planted), torch.randint(0, v, (58,), generator=g)])
    for k, val in _case(_Fp16Fixup, w, ids).items():
        out["rows_" + k] = val

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fp16_fixup.npz")
    np.savez_compressed(path, **out)
    print(path, {k: (v.shape if hasattr(v, "shape") else v) for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
