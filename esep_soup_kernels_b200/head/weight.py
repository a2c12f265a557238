"""The head weight's storage format: one fp16 tensor shared by the LM head and the embedding.

Mirror of the reference's ``_Fp16Fixup`` and ``_embedding_forward16``
(solution/head/patch.py:133-215, :217-226; the reasons are at :105-123): the frozen fp32 tied
embed / lm_head weight is replaced by ONE fp16 tensor. The head reads it as it is. The embedding
lookup must keep returning the fp32 values bit for bit, so the few elements that do not survive
fp32 -> fp16 -> fp32 (values below fp16's normal range, overflows, NaN payloads) are kept in a
small table and written back after the upcast.

Here the table is built by two kernels that read the fp32 weight once each (the second one only
the rows that have entries), ``share_fp16_weight`` casts and counts in the same pass, and the
lookup is ONE kernel: gather of fp16 rows, upcast and the rows' entries. The table is stored in
compressed rows (``row_start`` / ``flat_idx`` / ``flat_val``); ``flat_idx`` and ``flat_val`` are
the reference's arrays of the same names (patch.py:151-152).
"""

import warnings

import torch

from . import _lib
from .op import _ptr, _stream

MAX_FIXUP_FRACTION = 0.01   # patch.py:128: refuse when more elements than this need an entry
MAX_FIXUP_PER_ROW = 64      # patch.py:129


def _check_weight(w, dtype, name):
    assert w.dim() == 2 and w.dtype == dtype and w.is_cuda and w.is_contiguous(), \
        f"{name} must be a contiguous 2-D CUDA tensor of {dtype}"
    assert w.shape[1] % 8 == 0, "hidden size must be a multiple of 8"


class Fp16Fixup:
    """The elements of a fp32 weight that fp16 does not hold exactly, and how to restore them
    (``_Fp16Fixup``, patch.py:133-215). ``count`` entries in ``rows`` rows, at most ``width`` in
    one row."""

    def __init__(self, w32, w16):
        _check_weight(w32, torch.float32, "w32")
        _check_weight(w16, torch.float16, "w16")
        assert w32.shape == w16.shape and w32.device == w16.device
        self._build(w32, w16, cast=False)

    def _build(self, w32, w16, cast):
        lib = _lib.load()
        v, h = w32.shape
        dev = w32.device
        with torch.cuda.device(dev):
            self.row_start = torch.empty(v + 1, device=dev, dtype=torch.int32)
            stats = torch.empty(3 + (v + 1023) // 1024, device=dev, dtype=torch.int64)
            _lib.check("esep_weight_fixup_scan", lib.esep_weight_fixup_scan(
                _ptr(w32), _ptr(w16), int(cast), v, h, _ptr(self.row_start), _ptr(stats),
                _stream(dev)))
            # the one host read of the set-up (the reference's .numel(), patch.py:153)
            self.count, self.rows, self.width = (int(s) for s in stats[:3].tolist())
            self.width = max(self.width, 1)
            self.flat_idx = torch.empty(self.count, device=dev, dtype=torch.int64)
            self.flat_val = torch.empty(self.count, device=dev, dtype=torch.float32)
            if self.count:
                _lib.check("esep_weight_fixup_fill", lib.esep_weight_fixup_fill(
                    _ptr(w32), _ptr(w16), v, h, _ptr(self.row_start), _ptr(self.flat_idx),
                    _ptr(self.flat_val), _stream(dev)))
        self.shape = (v, h)
        self.device = dev
        self._status = torch.zeros(1, device=dev, dtype=torch.int32)

    @classmethod
    def exact(cls, w16):
        """The table of a weight whose fp32 values are exactly ``w16.float()``: no entries, no
        fp32 copy of the weight is ever built (patch.py:177-194)."""
        _check_weight(w16, torch.float16, "w16")
        self = cls.__new__(cls)
        dev = w16.device
        self.row_start = None
        self.flat_idx = torch.empty(0, device=dev, dtype=torch.int64)
        self.flat_val = torch.empty(0, device=dev, dtype=torch.float32)
        self.count, self.rows, self.width = 0, 0, 1
        self.shape = tuple(w16.shape)
        self.device = dev
        self._status = torch.zeros(1, device=dev, dtype=torch.int32)
        return self

    @classmethod
    def cast(cls, w32):
        """(w16, table) with ``w16 = w32.to(float16)`` produced by the pass that counts."""
        _check_weight(w32, torch.float32, "w32")
        w16 = torch.empty(w32.shape, device=w32.device, dtype=torch.float16)
        self = cls.__new__(cls)
        self._build(w32, w16, cast=True)
        return w16, self

    def nbytes(self):
        tensors = [self.flat_idx, self.flat_val] + ([self.row_start] if self.row_start is not None
                                                    else [])
        return sum(t.numel() * t.element_size() for t in tensors)

    def _rows(self, w16, ids, out):
        v, h = self.shape
        with torch.cuda.device(self.device):
            _lib.check("esep_embed_rows", _lib.load().esep_embed_rows(
                _ptr(w16), _ptr(ids), ids.numel(), v, h,
                _ptr(self.row_start if self.count else None),
                _ptr(self.flat_idx if self.count else None),
                _ptr(self.flat_val if self.count else None), _ptr(out), _ptr(self._status),
                _stream(self.device)))
        return out

    def apply_rows(self, out, ids):
        """out [N, H] fp32 = upcast fp16 rows of token ids [N]; restores the exact values in
        place (patch.py:201-210)."""
        assert out.dim() == 2 and out.dtype == torch.float32 and out.is_contiguous()
        assert out.shape == (ids.numel(), self.shape[1]) and out.device == self.device
        if not self.rows:
            return out
        ids = ids.reshape(-1).to(device=self.device, dtype=torch.int64).contiguous()
        return self._rows(None, ids, out)

    def embed(self, w16, ids):
        """fp32 [*ids.shape, H]: the rows ``ids`` of the original fp32 weight, bit for bit, from
        the fp16 tensor in one kernel (``_embedding_forward16``, patch.py:217-226)."""
        _check_weight(w16, torch.float16, "w16")
        assert tuple(w16.shape) == self.shape and w16.device == self.device
        flat = ids.reshape(-1).to(device=self.device, dtype=torch.int64).contiguous()
        out = torch.empty(flat.numel(), self.shape[1], device=self.device, dtype=torch.float32)
        self._rows(w16, flat, out)
        return out.view(*ids.shape, self.shape[1])

    def exact_weight(self, w16):
        """The original fp32 weight, rebuilt (patch.py:212-215: the lm_head outside autocast)."""
        _check_weight(w16, torch.float16, "w16")
        assert tuple(w16.shape) == self.shape and w16.device == self.device
        v, h = self.shape
        out = torch.empty(v, h, device=self.device, dtype=torch.float32)
        with torch.cuda.device(self.device):
            _lib.check("esep_weight_exact", _lib.load().esep_weight_exact(
                _ptr(w16), v, h, self.count, _ptr(self.flat_idx if self.count else None),
                _ptr(self.flat_val if self.count else None), _ptr(out), _stream(self.device)))
        return out

    def bad_index_seen(self):
        """True when a lookup since the last call of this method met an id outside the vocabulary
        (such a row comes back as zeros; F.embedding would stop the process). One host read."""
        seen = int(self._status.item()) == _lib.DEV_BAD_INDEX
        if seen:
            self._status.zero_()
        return seen


def embedding_forward16(w16, fixup, input_ids):
    """Drop-in body of the reference's ``_embedding_forward16(module, fixup, input)`` for a
    plain embedding (no max_norm): fp32 output, bit-identical to the fp32-weight lookup."""
    return fixup.embed(w16, input_ids)


def share_fp16_weight(w32, max_fraction=MAX_FIXUP_FRACTION, max_per_row=MAX_FIXUP_PER_ROW):
    """(w16, fixup) for a frozen fp32 weight, or None when too many elements would need an entry
    (the refusal of ``_share_fp16_tied_weight``, patch.py:291-295; swapping the module's Parameter
    is the caller's business)."""
    w16, fixup = Fp16Fixup.cast(w32)
    if fixup.count > max_fraction * w32.numel() or fixup.width > max_per_row:
        warnings.warn(f"fused head: weight kept in fp32, {fixup.count} elements do not round-trip "
                      "through fp16", stacklevel=2)
        return None
    return w16, fixup


__all__ = ["Fp16Fixup", "embedding_forward16", "share_fp16_weight", "MAX_FIXUP_FRACTION",
           "MAX_FIXUP_PER_ROW"]
