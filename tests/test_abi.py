"""The C-ABI library: it loads, exports every symbol include/moe_b200.h declares, and validates
arguments before touching the GPU. No compute calls, so this runs without a CUDA device."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from oracle import moe_oracle as O


@pytest.fixture(scope="module")
def lib():
    from nanospeaker_b200 import _lib, build
    build.build()
    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "moe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moe_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    from nanospeaker_b200 import _lib
    declared = _declared_symbols()
    assert len(declared) >= 14
    assert declared == sorted(_lib.SIGNATURES), "ctypes table and header differ"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_abi_version_and_error_strings(lib):
    from nanospeaker_b200 import _lib
    assert lib.moe_b200_abi_version() == 2
    assert _lib.error_string(0) == "ok"
    for code in range(-7, 0):
        assert _lib.error_string(code) not in ("ok", "unknown moe_b200 error code")
    assert "unknown" in _lib.error_string(-99)


@pytest.mark.parametrize("m,e", [(0, 8), (1, 8), (3, 8), (100, 8), (12288, 76), (98304, 76),
                                 (786432, 76), (5, 200)])
def test_l_cap_matches_reference_formula(lib, m, e):
    """ceil((M + min(E, M) * 127) / 128) * 128 (src/model/moe_kernel.py:100-108)."""
    from nanospeaker_b200 import kernels
    want = O.l_cap(m, e)
    assert lib.moe_b200_l_cap(m, e) == want == kernels.l_cap(m, e)
    assert want % 128 == 0 and want >= m


def test_scratch_bytes_is_modest(lib):
    assert lib.moe_b200_dispatch_scratch_bytes(0, 76) > 0
    assert lib.moe_b200_dispatch_scratch_bytes(98304, 76) == 96 * 76 * 4   # 1024-pair blocks
    assert lib.moe_b200_dispatch_scratch_bytes(1 << 22, 76) == 128 * 76 * 4  # at most 128 blocks


def test_arguments_are_validated_before_any_launch(lib):
    """Bad shapes / NULL pointers come back as error codes, not faults (no GPU needed)."""
    null = ctypes.c_void_p(0)
    assert lib.moe_b200_router_topk(null, 4, 0, 1, 1, 0, null, null, null, null) == -1   # E < 1
    assert lib.moe_b200_router_topk(null, 4, 300, 1, 1, 0, null, null, null, null) == -1  # E > 256
    assert lib.moe_b200_router_topk(null, 4, 8, 9, 1, 0, null, null, null, null) == -1    # k > E
    assert lib.moe_b200_router_topk(null, 4, 8, 2, 1, 0, null, null, null, null) == -2    # NULL
    assert lib.moe_b200_router_topk(null, 0, 8, 2, 1, 0, null, null, null, null) == 0     # empty
    assert lib.moe_b200_dispatch(null, 10, 8, null, null, null, null, null, null, null, 0, 0, 0, null,
                                 null) == -2
    buf0 = ctypes.create_string_buffer(64)
    q = ctypes.c_void_p(ctypes.addressof(buf0))
    # every pointer the kernels would dereference is checked: topk_idx and inv_ids too
    assert lib.moe_b200_dispatch(null, 10, 8, q, q, q, q, q, q, q, 1 << 20, 0, 0, q, null) == -2
    assert lib.moe_b200_dispatch(q, 10, 8, q, q, q, q, q, null, q, 1 << 20, 0, 0, q, null) == -2
    assert lib.moe_b200_dispatch(q, 10, 8, q, q, q, q, q, q, q, 1 << 20, -1, 0, q, null) == -1  # capacity < 0
    assert lib.moe_b200_dispatch(q, 10, 8, q, q, q, q, q, q, q, 1 << 20, 4, 9, q, null) == -1   # n_capped > E
    assert lib.moe_b200_dispatch_static(null, 10, 8, q, q, q, q, q, q, q, null) == -2
    assert lib.moe_b200_dispatch_static(q, 10, 8, q, q, q, q, q, null, q, null) == -2
    assert lib.moe_b200_permute(null, 4, 100, 2, null, null, 128, null, null) == -1       # D % 8
    assert lib.moe_b200_permute(null, 4, 64, 2, null, null, 128, null, null) == -2
    assert lib.moe_b200_combine(null, null, 4, 2, 64, null, null, null, null) == -2
    assert lib.moe_b200_up_gemm(null, 128, 64, null, 4, null, 0, 64, null, null, 1, null, 0, 0, 0,
                                null, null, null, 0, null, null, null, null) == -2
    buf = ctypes.create_string_buffer(96)
    p = ctypes.c_void_p((ctypes.addressof(buf) + 31) & ~31)
    up = lambda rows, h, fixed, topk, n_extra=0: lib.moe_b200_up_gemm(
        p, rows, 64, p, 4, p, n_extra, h, p, p, fixed, p, topk, 8, 0, p, null, null, 0, null, null,
        p, null)
    assert up(128, 64, 1, 0) == -5      # d_hidden the tiles do not cover
    assert up(100, 128, 0, 0) == -1     # routed rows must be a multiple of 128
    assert up(128, 128, 5, 0) == -1     # more fixed groups than weight matrices
    assert up(128, 128, 1, 2) == -1     # gathered A only on the routed schedule
    assert up(128, 128, 1, 0, 2) == -1  # a second weight stack only on the routed schedule
    # the accumulating GEMMs: the token-major accumulator and the slot -> token map are checked too
    dacc = lambda rows, fixed, sid, topk, acc, n_tok=4, n_pairs=8: lib.moe_b200_down_gemm_acc(
        p, rows, 128, p, 4, null, 0, 64, p, p, fixed, sid, p, n_pairs, topk, acc, n_tok, null, p,
        null)
    assert dacc(128, 0, p, 2, null) == -2        # no accumulator
    assert dacc(128, 0, null, 2, p) == -2        # routed schedule without sorted_ids
    assert dacc(128, 0, p, 0, p) == -1           # top_k < 1
    assert dacc(128, 0, p, 2, p, 4, 9) == -1     # more pairs than n_tokens * top_k
    assert dacc(128, 1, null, 1, p, 100) == -1   # fixed schedule: more rows than tokens
    assert dacc(100, 0, p, 2, p) == -1           # routed rows must be a multiple of 128
    xacc = lambda sid, topk, acc: lib.moe_b200_dx_gemm_acc(
        p, 128, 128, p, 4, null, 0, 64, p, p, 0, sid, 8, topk, acc, 4, null, p, null)
    assert xacc(p, 2, null) == -2
    assert xacc(null, 2, p) == -2
    assert xacc(p, 0, p) == -1
    wg = lambda n_dim, ks, which, po, n_first=4: lib.moe_b200_wgrad(
        p, 0, 64, p, 0, n_dim, 128, po, 4, ks, p, 2, 8, which, p, n_first, null, p, 0, null, 0, 0, p,
        null)
    assert wg(100, 2048, 0, p) == -5    # n_dim % 32
    assert wg(256, 100, 0, p) == -1     # ks_rows % 64
    assert wg(256, 2048, 3, p) == -1    # gather_which out of range
    assert wg(256, 2048, 1, null) == -1 # gather needs the routed schedule
    assert wg(256, 2048, 0, p, 3) == -1 # groups beyond n_first need dw_extra
    assert wg(256, 2048, 0, p) == -4    # scratch too small
    # expert-parallel entry points: shapes first, then NULL / misaligned pointers, nothing launched
    assert lib.moe_b200_ep_plan(p, p, 9, 76, 0, p, p, p, p, p, p, 8, null) == -1     # > 8 ranks
    assert lib.moe_b200_ep_plan(p, p, 8, 76, 8, p, p, p, p, p, p, 8, null) == -1     # rank >= world
    assert lib.moe_b200_ep_plan(null, p, 8, 76, 0, p, p, p, p, p, p, 8, null) == -2
    assert lib.moe_b200_ep_pair_map(p, p, p, p, p, 0, 8, 76, 8, p, p, null) == 0     # no tokens
    assert lib.moe_b200_ep_pair_map(p, p, p, p, p, 4, 8, 76, 9, p, p, null) == -1
    assert lib.moe_b200_ep_pair_map(null, p, p, p, p, 4, 8, 76, 8, p, p, null) == -2
    two = (ctypes.c_void_p * 2)(p.value, p.value + 8)                                # 2nd misaligned
    ok2 = (ctypes.c_void_p * 2)(p.value, p.value)
    assert lib.moe_b200_ep_push_rows(p, 4, 100, 8, p, p, null, 128, p, p, ok2, null, null, 2, null,
                                     null) == -1                                      # D % 8
    assert lib.moe_b200_ep_push_rows(p, 4, 64, 8, p, p, null, 128, p, p, two, null, null, 2, null,
                                     null) == -3                                      # alignment
    assert lib.moe_b200_ep_push_rows(p, 4, 64, 8, p, p, null, 128, p, p, ok2, null, ok2, 2, null,
                                     null) == -2                                      # weights missing
    assert lib.moe_b200_ep_pad_fix(p, p, 0, null, 64, null, 0, null) == 0             # no local experts
    assert lib.moe_b200_ep_pad_fix(p, p, 3, null, 64, null, 0, null) == -2
    assert lib.moe_b200_ep_pull_combine(ok2, 10, p, p, 4, 8, 64, null, p, null) == -1  # > 9 tables
    assert lib.moe_b200_ep_pull_combine(two, 2, p, p, 4, 8, 64, null, p, null) == -3
    assert lib.moe_b200_ep_pull_vec(ok2, 2, p, p, 4, 8, 9, p, null) == -1             # top_k > k_all
    pb = ctypes.c_size_t(0)
    assert lib.moe_b200_wgrad_scratch_bytes(576, 256, 108032, 76, 1, 2048, ctypes.byref(pb)) == 0
    assert pb.value == 4096 + (108032 // 2048 + 76) * 5 * 128 * 256 * 4   # item table + tiles


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from nanospeaker_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no non-CUDA implementation"):
        _lib.load()


def test_block_entry_points_validate_and_size_their_scratch(lib):
    """moe_b200_block_fwd / _bwd: scratch sizes grow with the token count, bad shapes and NULL
    pointers are refused before anything is launched."""
    f = lib.moe_b200_block_fwd_scratch_bytes
    b = lib.moe_b200_block_bwd_scratch_bytes
    assert f(0, 576, 128, 76, 2, 6) == 0 and b(16, 576, 128, 76, 2, 77) == 0      # bad shapes
    small, big = f(256, 576, 128, 76, 2, 6), f(16384, 576, 128, 76, 2, 6)
    assert 0 < small < big
    # hidden rows of every slot + the dispatch's histograms + the column sums
    cap = O.l_cap(16384 * 8, 78)
    assert cap * 128 * 2 <= big <= cap * 128 * 2 + (1 << 20)
    assert b(16384, 576, 128, 76, 2, 6) > cap * (576 + 256 + 128) * 2
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(256)      # never dereferenced: validation comes first
    n_l = ctypes.c_int32(0)
    fwd = lambda x, scratch, nbytes, top_k=6: lib.moe_b200_block_fwd(
        x, 256, 576, one, null, null, one, one, 76, 128, one, one, 2, top_k, 1, 1, 0.01, 0,
        one, one, one, one, one, one, one, one, one, one, one, one, one, one, one, scratch, nbytes,
        ctypes.byref(n_l), one, null)
    assert fwd(null, one, small) == -2           # MOE_B200_ERR_NULL
    assert fwd(one, null, small) == -2
    assert fwd(one, one, small - 1) == -4        # MOE_B200_ERR_SCRATCH
    assert fwd(one, one, small, top_k=0) == -1   # MOE_B200_ERR_SHAPE
