"""CPU checks of the C ABI: the library loads, exports every symbol the header declares, and the
host-side parameter logic matches the reference's (attn_main.cu:35-74, 275-280; run_drivers.cu:9-24)."""
import ctypes
import os
import re

import pytest

from conftest import REFERENCE_CASES, ROOT


def header_symbols():
    text = open(os.path.join(ROOT, "include", "efa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(efa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    names = header_symbols()
    assert len(names) >= 20
    handle = ctypes.CDLL(pkg.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in include/efa_b200.h but not exported"
    assert sorted(pkg.EXPORTED_SYMBOLS) == names, "python binding and header disagree"


def test_abi_version(pkg):
    assert pkg.lib().efa_abi_version() == 1


def test_mode_names_round_trip(pkg):
    names = ["attn", "attn_tiled", "megatron", "sync", "overlap", "stream", "comm"]
    for i, n in enumerate(names):
        assert pkg.mode_name(i) == n
        assert pkg.parse_mode(n) == i
    assert pkg.mode_name(7) == "?" and pkg.mode_name(-1) == "?"
    assert pkg.parse_mode("nope") == -1


@pytest.mark.parametrize("case", REFERENCE_CASES)
@pytest.mark.parametrize("R", [1, 2, 4, 8])
def test_make_params_matches_reference_arithmetic(pkg, case, R):
    S, d, H, tile, nbuf, split, causal = case
    p = pkg.make_params(S, d, H, tile, nbuf, split, causal, R)
    assert (p.S, p.d, p.H, p.R) == (S, d, H, R)
    assert p.H_local == H // R and p.d_h == d // H and p.d_local == (H // R) * (d // H)
    assert p.num_tiles == S // tile
    assert abs(p.flash_tc.scale - (d // H) ** -0.5) < 1e-7
    assert (p.flash_tc.S, p.flash_tc.d_h, p.flash_tc.H_local, p.flash_tc.split, p.flash_tc.causal) == \
        (S, d // H, H // R, split, causal)
    why = pkg.attn_check_params(p)
    if H % R:
        assert why == "H must be divisible by the number of ranks"
    else:
        assert why is None
        assert pkg.blocks_per_tile(p) == (tile // 64) * (H // R) * split


def test_check_params_messages(pkg):
    assert pkg.attn_check_params(pkg.make_params(1024, 516, 8, 256)) == "d must be divisible by H"
    assert pkg.attn_check_params(pkg.make_params(1000, 512, 8, 256)) == "S must be a multiple of tile"
    assert pkg.attn_check_params(pkg.make_params(1024, 512, 8, 256, nbuf=0)) == "nbuf must be >= 1"
    assert pkg.attn_check_params(pkg.make_params(1024, 384, 8, 256)) == "tc: d_h must be 16, 32, 64 or 128"
    assert pkg.attn_check_params(pkg.make_params(1024, 512, 8, 32)) == "tc: tile must be a multiple of 64"
    assert pkg.attn_check_params(pkg.make_params(1024, 512, 8, 256, split=3)) == "tc: S must be a multiple of split * 64"
    fp = pkg.make_params(1024, 512, 8, 256).flash_tc
    assert pkg.flash_attn_tc_check_params(fp, 96) == "tc: tile must be a multiple of 64"
    assert pkg.flash_attn_tc_check_params(fp, 128) is None


def test_single_rank_world_selftest(pkg):
    pkg.world_selftest(pkg.World())


def test_compute_entry_points_fail_loudly_without_a_device(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(pkg.EfaError):
        pkg.make_ctx(pkg.World())
