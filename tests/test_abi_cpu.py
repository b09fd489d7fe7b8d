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
    assert pkg.lib().efa_abi_version() == 3


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


def _plan(pkg, S, d, H, tile, group_tiles=0, R=1, causal=1, order=0):
    p = pkg.make_params(S, d, H, tile, causal=causal, world_size=R)
    p.group_tiles = group_tiles
    p.row_order = order
    return p, *pkg.stream_plan(p)


def test_stream_plan_covers_every_tile_once(pkg):
    # stream mode waits on every tile's counter exactly once, whatever the grouping (run_drivers.cu:227-240)
    for S, tile, gt in [(4096, 128, 0), (4096, 128, 1), (4096, 128, 5), (32768, 128, 0), (65536, 64, 0),
                        (65536, 256, 7), (1024, 256, 0), (256, 256, 0), (8192, 64, 1000)]:
        for causal, order in [(0, 0), (1, 0), (1, 1), (0, 2)]:
            p, groups, band, desc = _plan(pkg, S, 1024, 16, tile, gt, causal=causal, order=order)
            assert desc == (order == 2 or (order == 0 and causal == 1))      # one rank: last rows first when causal
            covered = sorted(t for first, n in groups for t in range(first, first + n))
            assert covered == list(range(p.num_tiles)), (S, tile, gt)
            assert all(n >= 1 for _, n in groups)
            firsts = [first for first, _ in groups]
            assert firsts == sorted(firsts, reverse=desc)          # waited for in the order they complete
            assert band % 256 == 0 and (band == 0 or 512 <= band <= 2048)


def test_stream_plan_per_tile_schedule_is_the_reference_one(pkg):
    p, groups, band, desc = _plan(pkg, 4096, 1024, 16, 128, group_tiles=1, order=1)
    assert groups == [(t, 1) for t in range(32)] and not desc
    assert band == 0                       # strict row order: a tile's rows complete before the next tile's


def test_stream_plan_automatic_grouping_tapers_the_eighth_that_completes_last(pkg):
    # benchmark shape on one rank: S/8 rows per group, then S/16, S/32, S/32; K and V of 32 heads (512 MB) exceed
    # the L2, so the attention kernel works in bands of S/16 rows
    p, groups, band, desc = _plan(pkg, 32768, 4096, 32, 128, R=1, order=1)
    assert [n for _, n in groups] == [32] * 7 + [16, 8, 8] and groups[0] == (0, 32)
    assert band == 2048
    # a band never exceeds the smallest group it has to complete within... except by design the two S/32 groups
    assert band <= 2 * min(n for _, n in groups) * 128
    # the same shape, last rows first (the default under a causal mask): the small groups are the FIRST rows
    p, groups, band, desc = _plan(pkg, 32768, 4096, 32, 128, R=1)
    assert desc and [n for _, n in groups] == [32] * 7 + [16, 8, 8]
    assert groups[0] == (224, 32) and groups[-1] == (0, 8) and groups[-2] == (8, 8)
    # eight ranks: four heads' K and V (64 MB) stay in the L2, strict row order; and first rows first, because a
    # reduction has to keep up with the rows as they complete
    p, groups, band, desc = _plan(pkg, 32768, 4096, 32, 128, R=8)
    assert band == 0 and not desc and groups[0] == (0, 32)
    # explicit grouping: the band is the group
    p, groups, band, desc = _plan(pkg, 32768, 4096, 32, 128, group_tiles=8)
    assert [n for _, n in groups] == [8] * 32 and band == 1024
    # an explicit band, and none
    p.band_rows = 512
    assert pkg.stream_plan(p)[1] == 512
    p.band_rows = -1
    assert pkg.stream_plan(p)[1] == 0
    # small problems: one tile per group when S/8 is below a tile
    p, groups, band, desc = _plan(pkg, 512, 1024, 16, 128)
    assert [n for _, n in groups] == [1, 1, 1, 1] and band == 0


def test_stream_plan_mixed_order(pkg):
    # two 256-row blocks from the end, one from the start; groups of S/16 rows in the order a list schedule completes them
    p = pkg.make_params(32768, 4096, 32, 128, causal=1, world_size=8)
    p.row_order = pkg.ROWS_MIXED
    order = pkg.stream_row_blocks(p)
    assert sorted(order) == list(range(128)) and order[:6] == [127, 126, 0, 125, 124, 1]
    groups, band, desc = pkg.stream_plan(p)
    assert band == 0 and not desc
    assert sorted(groups) == [(16 * g, 16) for g in range(16)]
    assert groups[0] == (0, 16)                         # the lightest rows complete first ...
    assert groups[-1][0] not in (0, 240)                # ... and neither end completes last
    # not causal, or bands in use (K and V of the local heads exceed the L2): plain first-to-last order
    q = pkg.make_params(32768, 4096, 32, 128, causal=0, world_size=8)
    q.row_order = pkg.ROWS_MIXED
    assert pkg.stream_row_blocks(q) == [] and pkg.stream_plan(q)[0][0] == (0, 32)
    q = pkg.make_params(32768, 4096, 32, 128, causal=1, world_size=1)
    q.row_order = pkg.ROWS_MIXED
    assert pkg.stream_row_blocks(q) == [] and pkg.stream_plan(q)[1] == 2048


def test_stream_plan_counts_without_a_buffer_and_rejects_a_short_one(pkg):
    import ctypes as C
    p = pkg.make_params(32768, 4096, 32, 128, causal=1, world_size=1)
    assert pkg.lib().efa_stream_plan(C.byref(p), None, 0, None, None) == 10
    buf = (pkg.StreamGroup * 4)()
    assert pkg.lib().efa_stream_plan(C.byref(p), buf, 4, None, None) == -1
    assert "groups" in pkg.last_error()


def test_python_constants_match_the_header(pkg):
    """Every enumerator of include/efa_b200.h that the ctypes mirror names has the header's value."""
    text = open(os.path.join(ROOT, "include", "efa_b200.h")).read()
    header = {m.group(1): int(m.group(2)) for m in re.finditer(r"\bEFA_([A-Z0-9_]+)\s*=\s*(\d+)", text)}
    checked = 0
    for name, value in vars(pkg).items():
        if name.isupper() and isinstance(value, int) and name.split("_")[0] in ("REDUCE", "WIRE", "ROWS", "MODE"):
            assert header.get(name) == value, (name, value, header.get(name))
            checked += 1
    assert checked >= 18          # 7 modes, 4 reductions, 3 wire types, 4 row orders
    assert header["REDUCE_PULL"] == 3 and pkg.REDUCE_PULL == 3
