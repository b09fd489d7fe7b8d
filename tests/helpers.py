"""Shared helpers of the GPU parity tests (all calls go through the C ABI via the package)."""
import numpy as np

from conftest import ABS_TOL, REL_TOL


def ref_inputs_f16(oracle, S, d, H, R, rank, seed):
    """Reference-recipe inputs rounded to fp16: (uint16 arrays, the same values widened to fp32)."""
    Q, K, V, W = oracle.ref_inputs(S, d, H, R, rank, seed)
    bits = tuple(oracle.round_f16(x) for x in (Q, K, V, W))
    vals = tuple(oracle.widen_f16(b) for b in bits)
    return bits, vals


def normal_inputs_f16(pkg, oracle, p, rank, seed):
    n = p.H_local * p.S * p.d_h
    bits = [np.zeros((p.H_local, p.S, p.d_h), np.uint16) for _ in range(3)] + [np.zeros((p.d_local, p.d), np.uint16)]
    pkg.fill_host_inputs(p, rank, seed, pkg.RECIPE_NORMAL, *bits)
    assert bits[0].size == n
    return tuple(bits), tuple(oracle.widen_f16(b) for b in bits)


def to_dev(torch, bits):
    return [torch.from_numpy(b.view(np.float16)).cuda() for b in bits]


def assert_close(oracle, got, ref, what=""):
    """max-abs <= 2e-3 and max-abs / max|ref| <= 1e-2 (the reference's own metric, attn_tests.cu:135-137,
    with its 2e-2 tightened to 1e-2)."""
    max_abs, max_ref = oracle.compare(got, ref)
    assert np.isfinite(max_abs), f"{what}: non-finite output"
    assert max_abs <= ABS_TOL, f"{what}: max_abs {max_abs:.3e} > {ABS_TOL}"
    assert max_abs <= REL_TOL * max(max_ref, 1e-20), f"{what}: rel {max_abs / max_ref:.3e} > {REL_TOL}"
    return max_abs, max_ref
