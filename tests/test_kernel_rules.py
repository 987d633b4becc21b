"""The host-side rules that send a product to one kernel or another, asked of the built library without a GPU
(skipped where the library has not been built)."""
import ctypes

import pytest


@pytest.fixture(scope="module")
def lib():
    from pih_b200.kernels.build import library_path
    try:
        return ctypes.CDLL(library_path(build=False))
    except (RuntimeError, OSError) as e:
        pytest.skip(f"the kernel library is not built here: {e}")


def test_where_the_gate_up_product_runs_on_pairs_of_sms(lib):
    """From 1536 rows, when 256 x 256 tiles fill the rounds of the SM pairs to four fifths (74 pairs where no device
    is asked: 148 SMs)."""
    wanted = lib.pih_pair_swiglu_wanted
    assert wanted(2048, 6144) == 1          # 192 tiles: three rounds, 86 %
    assert wanted(1536, 6144) == 1          # 144 tiles: two rounds, 97 %
    assert wanted(1535, 6144) == 0          # too few rows
    assert wanted(4096, 24576) == 1
    assert wanted(2048, 2 * 136) == 0       # 16 tiles on 74 pairs
    before = lib.pih_set_pair_swiglu_rule(17, 0)
    try:
        assert before == 1536
        assert wanted(17, 2 * 136) == 1 and wanted(16, 2 * 136) == 0
        lib.pih_set_pair_swiglu_rule(0, -1)
        assert wanted(4096, 24576) == 0     # switched off
    finally:
        lib.pih_set_pair_swiglu_rule(before, 80)
    assert wanted(2048, 6144) == 1


def test_top_logprobs_cuts_a_row_into_slices(lib):
    """top_logprobs cuts a row into 8 slices, more for vocabularies whose eighth is more than 40 Ki floats, and
    refuses what 64 slices cannot hold."""
    slices = lib.pih_top_logprobs_slices
    assert slices(151936) == 8 and slices(384) == 8
    assert slices(400001) == 16
    assert slices(64 * 40 * 1024 + 1) == -1
    lib.pih_top_logprobs_scratch_words.restype = ctypes.c_longlong
    assert lib.pih_top_logprobs_scratch_words(3, 151936, 20) == 3 * 8 * 42
