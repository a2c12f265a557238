"""ctypes binding of libesep_head.so (declared in include/esep_head.h).

There is no fallback: if the library cannot be loaded the import fails loudly, and if it loads
but the device is not sm_100 every call raises."""

import ctypes
import os

_CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_PATH = os.path.join(_CSRC, "libesep_head.so")

ESEP_OK = 0
ERR_BAD_ARG = -1          # status codes of include/esep_head.h
ERR_UNSUPPORTED_ARCH = -2
ERR_WORKSPACE = -3
ERR_CUDA = -4
ERR_DEVICE_TIMEOUT = -5
ERR_ALIGNMENT = -6
ERR_STATIC_SCRATCH = -7
DTYPE_F16 = 0
DTYPE_BF16 = 1
DTYPE_F32 = 2
RECORD_FIELDS = 5
METRIC_SCALARS = 4
STEP_SCALARS = 8
DEV_BAD_INDEX = 301       # device status: an embedding id outside the vocabulary


class Caps(ctypes.Structure):
    _fields_ = [("cc_major", ctypes.c_int), ("cc_minor", ctypes.c_int), ("sm_count", ctypes.c_int),
                ("max_clusters_bwd", ctypes.c_int), ("supported", ctypes.c_int)]


class Plan(ctypes.Structure):
    _fields_ = [(k, ctypes.c_int) for k in (
        "fwd_row_tiles", "fwd_vocab_tiles", "fwd_tiles_per_unit", "fwd_splits", "fwd_grid",
        "bwd_cluster", "bwd_hslice", "bwd_hblocks", "bwd_passes", "bwd_total_steps",
        "bwd_full_rounds", "bwd_rem_pairs", "bwd_rem_splits", "bwd_steps_per_split", "bwd_grid")] + [(k, ctypes.c_size_t) for k in (
            "ws_status_off", "ws_partial_off", "ws_record_off", "ws_cew_off", "ws_dxpart_off",
            "ws_bytes")]


class HeadLibraryError(RuntimeError):
    """A C entry point returned a non-zero status."""

    def __init__(self, fn, code, text):
        super().__init__(f"{fn} failed: {code} ({text})")
        self.code = code


_P = ctypes.c_void_p
_I64 = ctypes.c_int64
_INT = ctypes.c_int
_SZ = ctypes.c_size_t

# name -> (restype, argtypes); every symbol include/esep_head.h declares.
SIGNATURES = {
    "esep_head_status_string": (ctypes.c_char_p, [_INT]),
    "esep_head_query": (_INT, [_INT, ctypes.POINTER(Caps)]),
    "esep_head_warmup": (_INT, [_INT]),
    "esep_head_plan_problem": (_INT, [_I64, _I64, _I64, _INT, _INT, _INT, ctypes.POINTER(Plan)]),
    "esep_head_workspace_bytes": (_SZ, [_I64, _I64, _I64, _INT, _INT]),
    "esep_head_forward_partial": (_INT, [_P, _P, _P, _I64, _I64, _I64, _I64, _INT, _P, _P, _SZ, _P]),
    "esep_head_finalize": (_INT, [_P, _INT, _P, _P, _I64, _I64, _P, _P, _P, _P, _P, _P, _P, _P,
                                  _P, _SZ, _P]),
    "esep_head_forward": (_INT, [_P, _P, _P, _P, _I64, _I64, _I64, _INT, _P, _P, _P, _P, _P, _P,
                                 _P, _P, _P, _SZ, _P]),
    "esep_head_backward": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _INT, _P, _P, _SZ,
                                  _P]),
    "esep_head_device_status": (_INT, [_P, _P, ctypes.POINTER(_INT)]),
    "esep_head_selftest_bounded_wait": (_INT, [_P, _SZ, _I64, _P]),
    "esep_head_static_scratch_bytes": (_SZ, []),
    "esep_head_forward_static": (_INT, [_P, _P, _P, _P, _I64, _I64, _I64, _INT, _P, _P, _P, _P, _P,
                                        _P, _P, _P, _P]),
    "esep_head_train_workspace_bytes": (_SZ, [_I64, _I64, _I64, _INT]),
    "esep_head_train": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _INT, _P, _P, _P, _P, _P, _P,
                               _P, _P, _P, _P, _P, _SZ, _P]),
    "esep_head_step_workspace_bytes": (_SZ, [_I64, _I64, _I64, _INT, _INT]),
    "esep_head_step": (_INT, [_P, _INT, _P, _P, _INT, _I64, _I64, _I64, _P, _P, _P, _P, _I64, _INT,
                              _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _SZ, _P]),
    "esep_head_vp_prepare": (_INT, [_P, _I64, _I64, _I64, _I64, _P, _P, _P]),
    "esep_head_vp_pack": (_INT, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _P, _P]),
    "esep_head_vp_combine": (_INT, [_P, _INT, _INT, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _INT,
                                    _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "esep_head_grad_scale": (_INT, [_P, _P, _I64, _INT, _P, _P]),
    "esep_head_debug_counters": (_INT, [ctypes.POINTER(ctypes.c_longlong), _INT]),
    "esep_head_set_training_path": (_INT, [_INT]),
    "esep_head_step_path_taken": (_INT, [_P, _P, ctypes.POINTER(_INT)]),
    "esep_head_step_uses_stored_logits": (_INT, [_I64, _I64, _I64, _INT, _INT]),
    "esep_head_norm_forward": (_INT, [_P, _P, _P, _I64, _I64, ctypes.c_float, _INT, _P, _P, _P,
                                      _P]),
    "esep_head_norm_backward": (_INT, [_P, _P, _P, _P, _P, _I64, _I64, _INT, _P, _P, _P]),
    "esep_weight_fixup_scan": (_INT, [_P, _P, _INT, _I64, _I64, _P, _P, _P]),
    "esep_weight_fixup_fill": (_INT, [_P, _P, _I64, _I64, _P, _P, _P, _P]),
    "esep_embed_rows": (_INT, [_P, _P, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P]),
    "esep_weight_exact": (_INT, [_P, _I64, _I64, _I64, _P, _P, _P, _P]),
}

_lib = None


def load():
    """Loads the shared library once. Builds it first when it is missing and nvcc is present."""
    global _lib
    if _lib is not None:
        return _lib
    from ..csrc import build as _build
    if not os.path.exists(LIB_PATH) or (_build.is_stale() and _build.have_nvcc()):
        _build.build()  # raises when nvcc is missing
    try:
        lib = ctypes.CDLL(LIB_PATH)
    except OSError as e:  # pragma: no cover - environment problem
        raise ImportError(f"cannot load the CUDA extension {LIB_PATH}: {e}. "
                          "Build it with `python -m esep_soup_kernels_b200.csrc.build`.") from e
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if a declared symbol is missing
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def status_string(code):
    return load().esep_head_status_string(int(code)).decode()


def check(fn_name, code):
    if code != ESEP_OK:
        raise HeadLibraryError(fn_name, code, status_string(code))


def query(device_index):
    caps = Caps()
    code = load().esep_head_query(int(device_index), ctypes.byref(caps))
    return code, caps


def plan_problem(n, h, v_local, need_grad, sm_count, max_clusters_bwd):
    pl = Plan()
    code = load().esep_head_plan_problem(n, h, v_local, int(bool(need_grad)), sm_count,
                                         max_clusters_bwd, ctypes.byref(pl))
    check("esep_head_plan_problem", code)
    return pl
