"""The attention kernel behind flash_attn_tc_forward against the CPU full-softmax checker, on the
reference's own test shapes (attn_tests.cu:70-85) and on the edge cases of the launch interface."""
import numpy as np
import pytest

from conftest import REFERENCE_CASES, REFERENCE_SEEDS
from helpers import assert_close, ref_inputs_f16, to_dev

pytestmark = pytest.mark.gpu


def run_attention(pkg, torch, p, dev, q_start, q_rows, o_dtype, tile_rows=None, poison=True):
    """One launch over rows [q_start, q_start + q_rows), split partials combined; returns (O, counters)."""
    Qd, Kd, Vd = dev[:3]
    tdtype = torch.float16 if o_dtype == pkg.F16 else torch.float32
    O = torch.full((q_rows, p.d_local), float("nan") if poison else 0.0, dtype=tdtype, device="cuda")
    part = None
    keep = []
    if p.split > 1:
        Op = torch.full((p.split, q_rows, p.d_local), float("nan"), dtype=torch.float32, device="cuda")
        mp = torch.full((p.split, q_rows, p.H_local), float("nan"), dtype=torch.float32, device="cuda")
        lp = torch.full((p.split, q_rows, p.H_local), float("nan"), dtype=torch.float32, device="cuda")
        keep = [Op, mp, lp]
        part = pkg.FlashPartials(Op.data_ptr(), mp.data_ptr(), lp.data_ptr(), q_rows)
    counters = None
    if tile_rows:
        counters = torch.zeros((q_rows + tile_rows - 1) // tile_rows, dtype=torch.int32, device="cuda")
    pkg.kernel_status_reset()
    pkg.flash_attn_tc_forward(Qd, Kd, Vd, O, part, q_start, q_rows, p.flash_tc, None, counters, tile_rows or 0, o_dtype)
    if p.split > 1:
        pkg.flash_attn_tc_combine(part, O, 0, q_rows, p.flash_tc, None, o_dtype)
    torch.cuda.synchronize()
    assert pkg.kernel_status()[0] == 0, f"kernel status {pkg.kernel_status()}"
    return O, counters


@pytest.mark.parametrize("case", REFERENCE_CASES, ids=lambda c: "S%d_d%d_H%d_t%d_n%d_s%d_c%d" % c)
def test_reference_shapes(pkg, oracle, torch_cuda, case):
    torch = torch_cuda
    S, d, H, tile, nbuf, split, causal = case
    p = pkg.make_params(S, d, H, tile, nbuf, split, causal)
    seeds = REFERENCE_SEEDS if S <= 1024 else REFERENCE_SEEDS[:1]
    for seed in seeds:
        bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, seed)
        ref = oracle.attention_rows(vals[0], vals[1], vals[2], causal)
        dev = to_dev(torch, bits)
        for o_dtype in (pkg.F16, pkg.F32):
            O, counters = run_attention(pkg, torch, p, dev, 0, S, o_dtype, tile_rows=tile)
            assert_close(oracle, O.float().cpu().numpy(), ref, f"seed {seed} dtype {o_dtype}")
            assert counters.cpu().tolist() == [pkg.blocks_per_tile(p)] * (S // tile)


@pytest.mark.parametrize("S,d,H,causal,split", [(192, 256, 4, 0, 1), (192, 256, 4, 1, 1), (320, 128, 2, 1, 1),
                                               (192, 64, 4, 1, 3), (448, 512, 4, 0, 1)])
def test_sequence_lengths_that_are_odd_multiples_of_64(pkg, oracle, torch_cuda, S, d, H, causal, split):
    torch = torch_cuda
    p = pkg.make_params(S, d, H, 64, 2, split, causal)
    assert pkg.attn_check_params(p) is None
    bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, 42)
    ref = oracle.attention_rows(vals[0], vals[1], vals[2], causal)
    O, counters = run_attention(pkg, torch, p, to_dev(torch, bits), 0, S, pkg.F32, tile_rows=64)
    assert_close(oracle, O.cpu().numpy(), ref)
    assert counters.cpu().tolist() == [pkg.blocks_per_tile(p)] * (S // 64)


@pytest.mark.parametrize("q_start,q_rows,tile_rows", [(0, 64, 64), (64, 64, 64), (128, 192, 64), (256, 256, 128), (448, 64, 64), (192, 320, 64)])
@pytest.mark.parametrize("causal", [0, 1])
def test_row_windows(pkg, oracle, torch_cuda, q_start, q_rows, tile_rows, causal):
    """Launches over a window of rows: O and the counters are indexed from the launch's first row,
    keys and the causal mask from the absolute row (flash_attn_tc.cuh:39-44)."""
    torch = torch_cuda
    S, d, H = 512, 256, 4
    p = pkg.make_params(S, d, H, tile_rows, 2, 1, causal)
    bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, 123)
    rows = np.arange(q_start, q_start + q_rows, dtype=np.int32)
    ref = oracle.attention_rows(vals[0], vals[1], vals[2], causal, rows)
    O, counters = run_attention(pkg, torch, p, to_dev(torch, bits), q_start, q_rows, pkg.F16, tile_rows=tile_rows)
    assert_close(oracle, O.float().cpu().numpy(), ref)
    total = sum(counters.cpu().tolist())
    assert total == (q_rows // 64) * p.H_local


def test_split_partials_follow_the_reference_layout(pkg, oracle, torch_cuda):
    """m_part is the row max of scale*log2(e)*s, l_part the denominator, O_part unnormalised
    (flash_attn_tc.cuh:25-34): recombining them on the host must give the checker's rows."""
    torch = torch_cuda
    S, d, H, split = 512, 256, 4, 4
    p = pkg.make_params(S, d, H, 128, 2, split, 0)
    bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, 777)
    dev = to_dev(torch, bits)
    Op = torch.zeros((split, S, p.d_local), dtype=torch.float32, device="cuda")
    mp = torch.zeros((split, S, p.H_local), dtype=torch.float32, device="cuda")
    lp = torch.zeros((split, S, p.H_local), dtype=torch.float32, device="cuda")
    part = pkg.FlashPartials(Op.data_ptr(), mp.data_ptr(), lp.data_ptr(), S)
    pkg.flash_attn_tc_forward(dev[0], dev[1], dev[2], None, part, 0, S, p.flash_tc, None, None, 0, pkg.F32)
    torch.cuda.synchronize()
    O_part, m, l = Op.cpu().numpy().astype(np.float64), mp.cpu().numpy().astype(np.float64), lp.cpu().numpy().astype(np.float64)
    M = m.max(axis=0)
    w = np.exp2(m - M)                                   # [split][S][H]
    L = (w * l).sum(axis=0)
    wfull = np.repeat(w, p.d_h, axis=2)
    O = (wfull * O_part).sum(axis=0) / np.repeat(L, p.d_h, axis=1)
    ref = oracle.attention_rows(vals[0], vals[1], vals[2], 0)
    assert_close(oracle, O.astype(np.float32), ref)
    # the per-split maxima are those of the scaled scores of that key range, in the log2 domain
    s = (vals[0][0, 5].astype(np.float64) @ vals[1][0, :128].astype(np.float64).T) * p.flash_tc.scale * 1.4426950408889634
    assert abs(m[0, 5, 0] - s.max()) < 1e-3


def test_illegal_launches_are_rejected(pkg, torch_cuda):
    torch = torch_cuda
    p = pkg.make_params(256, 256, 4, 64)
    x = torch.zeros(4 * 256 * 64, dtype=torch.float16, device="cuda")
    O = torch.zeros(256 * 256, dtype=torch.float16, device="cuda")
    with pytest.raises(pkg.EfaError, match="multiple of 64"):
        pkg.flash_attn_tc_forward(x, x, x, O, None, 0, 96, p.flash_tc)
    with pytest.raises(pkg.EfaError, match="outside"):
        pkg.flash_attn_tc_forward(x, x, x, O, None, 192, 128, p.flash_tc)
    bad = pkg.make_params(256, 192, 4, 64).flash_tc
    with pytest.raises(pkg.EfaError, match="d_h"):
        pkg.flash_attn_tc_forward(x, x, x, O, None, 0, 64, bad)
    p2 = pkg.make_params(256, 256, 4, 64, split=2)
    with pytest.raises(pkg.EfaError, match="workspace"):
        pkg.flash_attn_tc_forward(x, x, x, O, None, 0, 64, p2.flash_tc)


def test_convert_f32_to_f16(pkg, torch_cuda):
    torch = torch_cuda
    x = torch.randn(100003, device="cuda", dtype=torch.float32) * 3
    y = torch.zeros(100003, device="cuda", dtype=torch.float16)
    pkg.convert_f32_to_f16(x, y, x.numel())
    torch.cuda.synchronize()
    assert torch.equal(y, x.to(torch.float16))


@pytest.mark.parametrize("S,H_local,d_h,causal", [(16384, 2, 64, 0), (32768, 2, 64, 1), (65536, 2, 64, 1), (65536, 2, 64, 0), (32768, 4, 128, 1)],
                         ids=lambda v: str(v))
def test_full_size_rank_shards_on_sampled_rows(pkg, oracle, torch_cuda, S, H_local, d_h, causal):
    """One rank's shard of the eight-GPU configurations of the benchmark plan (two heads of d_h = 64 at
    S = 16k/32k/64k; four heads of d_h = 128 at S = 32k), N(0,1) inputs, checked on rows from the first, last
    and interior tiles, plus a size-independent property: with V = 1 every output element is exactly 1."""
    torch = torch_cuda
    R = 8
    p = pkg.make_params(S, R * H_local * d_h, R * H_local, 128, 2, 1, causal, R)
    assert p.H_local == H_local
    bits = [np.zeros((H_local, S, d_h), np.uint16) for _ in range(3)] + [np.zeros((p.d_local, p.d), np.uint16)]
    pkg.fill_host_inputs(p, 3, 42, pkg.RECIPE_NORMAL, *bits)
    vals = [oracle.widen_f16(b) for b in bits[:3]]
    rng = np.random.default_rng(S + d_h)
    rows = np.unique(np.concatenate([np.arange(0, 24), np.arange(S - 24, S), rng.integers(24, S - 24, 48)])).astype(np.int32)
    ref = oracle.attention_rows(vals[0], vals[1], vals[2], causal, rows)
    dev = to_dev(torch, bits[:3])
    O, counters = run_attention(pkg, torch, p, dev, 0, S, pkg.F16, tile_rows=128)
    assert counters.cpu().tolist() == [pkg.blocks_per_tile(p)] * (S // 128)
    assert_close(oracle, O[torch.from_numpy(rows.astype(np.int64)).cuda()].float().cpu().numpy(), ref)
    ones = torch.ones((H_local, S, d_h), dtype=torch.float16, device="cuda")
    O1, _ = run_attention(pkg, torch, p, [dev[0], dev[1], ones], 0, S, pkg.F32)
    assert float((O1 - 1.0).abs().max()) < 2e-3
