"""The allocation-free attention entry point against the ordinary one.

efa_flash_attn_tc_forward_noalloc serves callers that cannot obtain device memory when they call (their
memory pool owns the whole GPU, or they cannot afford an allocation's device-wide synchronisation): it
keeps the split-KV partials in a fixed array inside the library instead of a caller-owned workspace.
This file is collected last on purpose, so that a failure here cannot hide a failure elsewhere.
Two calls in a row, with different shapes and data, check that what the first call left in the
shared array does not leak into the second."""
import numpy as np
import pytest

from conftest import ABS_TOL, REL_TOL
from helpers import assert_close, ref_inputs_f16, to_dev

pytestmark = pytest.mark.gpu


def ordinary(pkg, torch, p, dev, q_start, q_rows, o_dtype):
    """forward into a caller-owned workspace, then combine: the existing entry points."""
    tdtype = torch.float16 if o_dtype == pkg.F16 else torch.float32
    O = torch.zeros((q_rows, p.d_local), dtype=tdtype, device="cuda")
    Op = torch.zeros((p.split, q_rows, p.d_local), dtype=torch.float32, device="cuda")
    mp = torch.zeros((p.split, q_rows, p.H_local), dtype=torch.float32, device="cuda")
    lp = torch.zeros((p.split, q_rows, p.H_local), dtype=torch.float32, device="cuda")
    part = pkg.FlashPartials(Op.data_ptr(), mp.data_ptr(), lp.data_ptr(), q_rows)
    pkg.flash_attn_tc_forward(dev[0], dev[1], dev[2], O, part, q_start, q_rows, p.flash_tc, None, None, 0, o_dtype)
    pkg.flash_attn_tc_combine(part, O, 0, q_rows, p.flash_tc, None, o_dtype)
    torch.cuda.synchronize()
    return O


def test_two_calls_in_a_row_match_the_ordinary_entry_point(pkg, oracle, torch_cuda):
    torch = torch_cuda
    calls = [
        # S, d, H, split, causal, seed, q_start, q_rows, dtype
        (1024, 512, 8, 4, 1, 42, 256, 768, pkg.F16),        # d_h = 64
        (512, 256, 4, 2, 0, 123, 128, 320, pkg.F32),        # d_h = 64, fp32 O
        (512, 256, 4, 1, 1, 7, 64, 448, pkg.F16),           # split = 1: no partials, O written directly
        (1024, 1024, 8, 2, 1, 9, 0, 512, pkg.F16),          # d_h = 128
        (256, 64, 4, 2, 0, 11, 0, 256, pkg.F32),            # d_h = 16
    ]
    pkg.flash_attn_tc_noalloc_status(reset=True)
    for S, d, H, split, causal, seed, q_start, q_rows, o_dtype in calls:
        p = pkg.make_params(S, d, H, 64, 2, split, causal)
        bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, seed)
        dev = to_dev(torch, bits)
        want = ordinary(pkg, torch, p, dev, q_start, q_rows, o_dtype)
        tdtype = torch.float16 if o_dtype == pkg.F16 else torch.float32
        got = torch.full((q_rows, p.d_local), float("nan"), dtype=tdtype, device="cuda")
        pkg.flash_attn_tc_forward_noalloc(dev[0], dev[1], dev[2], got, q_start, q_rows, p.flash_tc, None, o_dtype)
        torch.cuda.synchronize()
        assert pkg.flash_attn_tc_noalloc_status()[0] == 0, pkg.flash_attn_tc_noalloc_status()
        g, w = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert np.isfinite(g).all()
        diff = float(np.abs(g - w).max())
        assert diff <= ABS_TOL and diff <= REL_TOL * float(np.abs(w).max()), diff
        rows = np.arange(q_start, q_start + q_rows, dtype=np.int32)
        assert_close(oracle, g, oracle.attention_rows(vals[0], vals[1], vals[2], causal, rows))


def test_shapes_beyond_the_fixed_array_are_rejected(pkg, torch_cuda):
    torch = torch_cuda
    S, d, H, split = 2048, 1024, 8, 8
    p = pkg.make_params(S, d, H, 64, 2, split, 0)
    need = split * S * (p.d_local + 2 * p.H_local) * 4
    assert need > pkg.STATIC_SCRATCH_BYTES
    x = torch.zeros((H, S, d // H), dtype=torch.float16, device="cuda")
    O = torch.zeros((S, d), dtype=torch.float16, device="cuda")
    with pytest.raises(pkg.EfaError, match="scratch"):
        pkg.flash_attn_tc_forward_noalloc(x, x, x, O, 0, S, p.flash_tc)
