"""The CPU checker against (1) an independent numpy float64 statement of the same mathematics,
(2) the library's own host-side input recipe, (3) golden vectors dumped from the reference's own GPU
checker (tests/golden/README.md says how they were made)."""
import os

import numpy as np
import pytest

from conftest import ROOT

GOLDEN = os.path.join(ROOT, "tests", "golden")


def numpy_attention(Q, K, V, causal):
    H, S, dh = Q.shape
    out = np.zeros((S, H * dh))
    for h in range(H):
        s = (Q[h].astype(np.float64) @ K[h].astype(np.float64).T) / np.sqrt(dh)
        if causal:
            s = np.where(np.tril(np.ones((S, S), bool)), s, -np.inf)
        s -= s.max(axis=1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(axis=1, keepdims=True)
        out[:, h * dh:(h + 1) * dh] = p @ V[h].astype(np.float64)
    return out


@pytest.mark.parametrize("causal", [0, 1])
@pytest.mark.parametrize("shape", [(2, 96, 16), (3, 128, 64), (1, 64, 128)])
def test_oracle_attention_matches_numpy(oracle, shape, causal):
    rng = np.random.default_rng(7)
    Q, K, V = (rng.standard_normal(shape).astype(np.float32) for _ in range(3))
    ref = numpy_attention(Q, K, V, causal)
    got = oracle.attention_rows(Q, K, V, causal)
    assert np.abs(got - ref).max() < 2e-6
    rows = np.array([0, 5, shape[1] - 1], np.int32)
    sub = oracle.attention_rows(Q, K, V, causal, rows)
    assert np.array_equal(sub, got[rows])


def test_oracle_block_is_the_rank_sum(oracle):
    rng = np.random.default_rng(11)
    d, ranks = 64, []
    for _ in range(2):
        Q, K, V = (rng.standard_normal((2, 64, 16)).astype(np.float32) for _ in range(3))
        W = (rng.standard_normal((32, d)) * 0.1).astype(np.float32)
        ranks.append((Q, K, V, W))
    want = sum(numpy_attention(Q, K, V, 1) @ W.astype(np.float64) for Q, K, V, W in ranks)
    got = oracle.block_rows(ranks, d, 1)
    assert np.abs(got - want).max() < 5e-6


def test_f16_rounding_is_ieee_nearest_even(oracle):
    x = np.array([1.0, 1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65504.0, 1e-8, -2.5, 0.1], np.float32)
    assert np.array_equal(oracle.round_f16(x), x.astype(np.float16).view(np.uint16))
    rng = np.random.default_rng(3)
    y = rng.standard_normal(4096).astype(np.float32)
    assert np.array_equal(oracle.round_f16(y), y.astype(np.float16).view(np.uint16))
    assert np.array_equal(oracle.widen_f16(oracle.round_f16(y)), y.astype(np.float16).astype(np.float32))


@pytest.mark.parametrize("S,d,H,R,rank,seed", [(128, 64, 4, 1, 0, 42), (256, 128, 4, 2, 1, 123), (128, 512, 4, 4, 3, 777)])
def test_library_input_recipe_equals_oracle_recipe(pkg, oracle, S, d, H, R, rank, seed):
    """Both restate allocate_and_fill + compute_qkv (attn_main.cu:98-153); the fp16 results must agree
    bit for bit (same glibc rand() stream, same fp32 accumulation order)."""
    p = pkg.make_params(S, d, H, 64, world_size=R)
    n = p.H_local * S * p.d_h
    Qh, Kh, Vh = (np.zeros(n, np.uint16) for _ in range(3))
    Wh = np.zeros(p.d_local * d, np.uint16)
    pkg.fill_host_inputs(p, rank, seed, pkg.RECIPE_REF, Qh, Kh, Vh, Wh)
    Q, K, V, W = oracle.ref_inputs(S, d, H, R, rank, seed)
    assert np.array_equal(Qh, oracle.round_f16(Q).ravel())
    assert np.array_equal(Kh, oracle.round_f16(K).ravel())
    assert np.array_equal(Vh, oracle.round_f16(V).ravel())
    assert np.array_equal(Wh, oracle.round_f16(W).ravel())


def test_normal_recipe_is_rank_count_invariant_and_unit_variance(pkg):
    S, d, H = 256, 256, 4
    full = pkg.make_params(S, d, H, 64, world_size=1)
    n = full.H_local * S * full.d_h
    A = [np.zeros(n, np.uint16) for _ in range(3)] + [np.zeros(full.d_local * d, np.uint16)]
    pkg.fill_host_inputs(full, 0, 42, pkg.RECIPE_NORMAL, *A)
    half = pkg.make_params(S, d, H, 64, world_size=2)
    for rank in range(2):
        m = half.H_local * S * half.d_h
        B = [np.zeros(m, np.uint16) for _ in range(3)] + [np.zeros(half.d_local * d, np.uint16)]
        pkg.fill_host_inputs(half, rank, 42, pkg.RECIPE_NORMAL, *B)
        for t in range(3):
            assert np.array_equal(B[t], A[t][rank * m:(rank + 1) * m])
        assert np.array_equal(B[3], A[3][rank * half.d_local * d:(rank + 1) * half.d_local * d])
    q = A[0].view(np.float16).astype(np.float64)
    assert abs(q.mean()) < 0.02 and abs(q.std() - 1.0) < 0.02
    w = A[3].view(np.float16).astype(np.float64)
    assert abs(w.std() - d ** -0.5) < 0.05 * d ** -0.5


def golden_cases():
    man = os.path.join(GOLDEN, "manifest.txt")
    if not os.path.exists(man):
        return []
    out = []
    for line in open(man):
        if line.startswith("#") or not line.strip():
            continue
        f = line.split()
        name, S, d, H, causal, seed, mx = f[:7]
        ranks = int(f[7]) if len(f) > 7 else 1
        out.append((name, int(S), int(d), int(H), int(causal), int(seed), float(mx), ranks))
    return out


def test_golden_vectors_present():
    assert len(golden_cases()) >= 7, "tests/golden/manifest.txt is missing or incomplete"
    assert sorted(set(c[7] for c in golden_cases())) == [1, 2, 4, 8]


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c[0])
def test_oracle_matches_reference_gpu_checker(oracle, case):
    """The reference's checker works on the fp32 Q/K/V (attn_tests.cu:37); so does this comparison.
    Differences are fp32 GEMM rounding only (cuBLAS SGEMM vs double accumulation). Cases with several ranks are the
    sum of the ranks' partial blocks (rank-specific inputs, head shares), as the checker sums them."""
    name, S, d, H, causal, seed, mx, ranks = case
    gold = np.fromfile(os.path.join(GOLDEN, name + ".f32"), np.float32).reshape(S, d)
    assert abs(np.abs(gold).max() - mx) <= 1e-6 * max(mx, 1.0)
    got = oracle.block_rows([oracle.ref_inputs(S, d, H, ranks, r, seed) for r in range(ranks)], d, causal)
    max_abs, max_ref = oracle.compare(got, gold)
    assert max_abs / max_ref < 2e-5, (max_abs, max_ref)
