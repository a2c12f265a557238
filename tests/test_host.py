"""Host-side checks that need no GPU: the C-ABI library loads, exports every symbol the header
declares, and its planning arithmetic is sane."""

import ctypes
import os
import re
import sys

import pytest

from esep_soup_kernels_b200.head import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "esep_head.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(esep_(?:head|weight|embed)_[a-z_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/esep_head.h but not exported"
    assert sorted(_lib.SIGNATURES) == names      # the Python binding covers the whole header


def test_status_strings():
    assert _lib.status_string(0) == "ok"
    for code in range(-7, 0):
        assert _lib.status_string(code) != "unknown status"
    assert _lib.status_string(-99) == "unknown status"


def test_query_without_a_gpu_reports_an_error_not_a_crash():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    code, caps = _lib.query(0)
    assert code != 0 and caps.supported == 0
    assert _lib.load().esep_head_workspace_bytes(128, 64, 1000, 0, 1) == 0


def test_every_kernel_header_is_a_build_dependency():
    """The library is one translation unit that includes every .cuh of csrc/: a header missing
    from the dependency list would leave a stale library after an edit."""
    import os
    import re

    from esep_soup_kernels_b200.csrc import build

    csrc = os.path.dirname(build.__file__)
    on_disk = {f for f in os.listdir(csrc) if f.endswith(".cuh")}
    assert on_disk <= set(build.HEADERS)
    included = set()
    for name in ["esep_head.cu"] + sorted(on_disk):
        with open(os.path.join(csrc, name)) as fh:
            included |= set(re.findall(r'#include "([\w.]+\.cuh)"', fh.read()))
    assert included <= on_disk and "head_dx.cuh" in included and "head_step.cuh" in included


def test_training_path_setting_is_host_state_with_four_values():
    """0 auto, 1 single pass, 2 stored logits, 3 stored weights; the call returns the previous
    value and refuses anything else. Without a GPU the path query answers 0 (no launch made)."""
    lib = _lib.load()
    first = lib.esep_head_set_training_path(0)
    try:
        prev = 0
        for path in (1, 2, 3, 0):
            assert lib.esep_head_set_training_path(path) == prev
            prev = path
        assert lib.esep_head_set_training_path(4) == _lib.ERR_BAD_ARG
        assert lib.esep_head_set_training_path(-1) == _lib.ERR_BAD_ARG
        assert lib.esep_head_set_training_path(0) == 0      # a refused value changes nothing
        from esep_soup_kernels_b200.head.op import TRAINING_PATHS
        assert sorted(TRAINING_PATHS.values()) == [0, 1, 2, 3]
    finally:
        lib.esep_head_set_training_path(first)


@pytest.mark.parametrize("n,h,v", [(1, 64, 257), (77, 64, 1001), (4340, 1536, 151936),
                                    (16384, 1536, 151936), (32768, 3584, 19008), (4099, 1536, 151936)])
def test_plan_covers_the_problem(n, h, v):
    pl = _lib.plan_problem(n, h, v, True, 148, 33)
    assert pl.fwd_row_tiles * 128 >= n and pl.fwd_vocab_tiles * 256 >= v
    assert pl.fwd_splits * pl.fwd_tiles_per_unit >= pl.fwd_vocab_tiles
    assert (pl.fwd_splits - 1) * pl.fwd_tiles_per_unit < pl.fwd_vocab_tiles
    assert 2 <= pl.fwd_grid <= 148 and pl.fwd_grid % 2 == 0
    assert pl.bwd_cluster == 4 and pl.bwd_grid % 4 == 0 and pl.bwd_grid <= 33 * 4
    assert pl.bwd_hslice == 128 * pl.bwd_hblocks and 1 <= pl.bwd_hblocks <= 3
    assert pl.bwd_passes * 4 * pl.bwd_hslice >= h                   # every H column has an owner
    assert pl.bwd_total_steps * 512 >= v
    ncl = pl.bwd_grid // 4
    pairs = pl.fwd_row_tiles * pl.bwd_passes
    assert pl.bwd_full_rounds * ncl + pl.bwd_rem_pairs == pairs and pl.bwd_rem_pairs < ncl
    if pl.bwd_rem_pairs:
        assert pl.bwd_rem_pairs * pl.bwd_rem_splits <= ncl          # one run per cluster at most
        assert pl.bwd_rem_splits * pl.bwd_steps_per_split >= pl.bwd_total_steps
        assert (pl.bwd_rem_splits - 1) * pl.bwd_steps_per_split < pl.bwd_total_steps
    offs = [pl.ws_status_off, pl.ws_partial_off, pl.ws_record_off, pl.ws_cew_off, pl.ws_dxpart_off]
    assert offs == sorted(offs) and all(o % 256 == 0 for o in offs) and pl.ws_bytes >= offs[-1]
    if pl.bwd_rem_pairs:
        assert (pl.ws_bytes - pl.ws_dxpart_off >=
                pl.bwd_rem_splits * pl.bwd_rem_pairs * 128 * 4 * pl.bwd_hslice * 4)
    # forward-only callers never pay for the dX partial buffers
    assert _lib.plan_problem(n, h, v, False, 148, 33).ws_bytes == pl.ws_dxpart_off


def test_plan_balances_the_backward_clusters():
    pl = _lib.plan_problem(4340, 1536, 151936, True, 148, 33)
    ideal = pl.fwd_row_tiles * pl.bwd_total_steps / 33
    per_cluster = pl.bwd_full_rounds * pl.bwd_total_steps + pl.bwd_steps_per_split
    assert ideal / per_cluster > 0.99


def test_plan_rejects_bad_sizes():
    for n, h, v in [(0, 64, 100), (10, 0, 100), (10, 64, 0), (10, 60, 100), (1 << 31, 64, 100)]:
        with pytest.raises(_lib.HeadLibraryError):
            _lib.plan_problem(n, h, v, True, 148, 33)


def test_bench_cpu_arm_loads_the_workload_without_the_package():
    """`bench.py --impl reference` must not map the CUDA library: it loads the synthetic workload
    by file, so importing the package (whose import loads libesep_head.so) is never needed."""
    import subprocess

    code = ("import sys, bench; m = bench._synthetic(); "
            "cfg = m.make_config('c1', n_override=4, v_override=64, h_override=16); "
            "assert cfg['x'].shape == (4, 16); "
            "assert not any(k.startswith('esep_soup_kernels_b200') for k in sys.modules), "
            "[k for k in sys.modules if k.startswith('esep')]")
    subprocess.run([sys.executable, "-c", code], cwd=ROOT, check=True)
