"""The waits that guard against a signal that never comes, made to run out on purpose.

The reference has no such guard: a wrong counter target blocks its cuStreamWaitValue32 forever
(run_drivers.cu:228-230) and every error ends in MPI_Abort (attn_defs.cuh:14-63). Here every wait has a limit,
and these tests reach the limit without any fault on the GPU: the HOST asks the consumers of the tile counters
to wait for one count more than the attention kernel will ever deliver (efa_params.debug_target_bias), with the
limits of the context turned down to fractions of a second. The waits give up, report, and the next ordinary
run on the same context is correct. On the CPU, a rank of the shared-memory MPI subset that leaves early makes
the others time out of their barrier instead of spinning."""
import os
import subprocess
import time

import numpy as np
import pytest

from conftest import ROOT
from helpers import assert_close, ref_inputs_f16, to_dev

BIN = os.path.join(ROOT, "eager-flash-attention_b200", "bin")


def _problem(pkg, oracle, torch):
    S, d, H, tile = 1024, 512, 8, 128
    p = pkg.make_params(S, d, H, tile, causal=1)
    bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, 42)
    ref = oracle.block_rows([vals], d, 1)
    dev = to_dev(torch, bits)
    return p, dev, pkg.Weights(*(t.data_ptr() for t in dev)), ref


@pytest.mark.gpu
def test_persistent_kernel_gives_up_waiting_for_counters_and_recovers(pkg, oracle, torch_cuda):
    """Fused projection + reduction kernel on one rank, polling for a count that never comes: after the context's
    device limit (50 ms here) its producer records KS_WAIT_TIMEOUT at the counter wait (site 41), every role leaves
    its loop, the kernel frees its tensor memory and returns; the call itself returns normally."""
    torch = torch_cuda
    p, dev, w, ref = _problem(pkg, oracle, torch)
    ctx = pkg.make_ctx(pkg.World(), ncomm=2)
    try:
        pkg.set_wait_limit_ms(ctx, 50.0, 5000.0)
        p.reduce = pkg.REDUCE_P2P
        out = torch.zeros((p.S, p.d), dtype=torch.float16, device="cuda")
        pkg.kernel_status_reset()
        p.debug_target_bias = 1
        t0 = time.perf_counter()
        pkg.run_mode(ctx, pkg.MODE_STREAM, w, out, p)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 4.0                  # the waits ran out; nothing spun until a watchdog
        code, _block, site, _ = pkg.kernel_status()
        assert code == 1 and site == 41, pkg.kernel_status()   # KS_WAIT_TIMEOUT at the tile-counter wait
        # the same context, an ordinary run
        pkg.kernel_status_reset()
        p.debug_target_bias = 0
        out.fill_(float("nan"))
        pkg.run_mode(ctx, pkg.MODE_STREAM, w, out, p)
        torch.cuda.synchronize()
        assert pkg.kernel_status()[0] == 0
        assert_close(oracle, out.float().cpu().numpy(), ref, "after the timed-out run")
    finally:
        pkg.destroy_ctx(ctx)


@pytest.mark.gpu
def test_pending_stream_waits_are_released_after_the_host_limit(pkg, oracle, torch_cuda):
    """Stream mode with front-end waits (cuStreamWaitValue32) on a target that is one too high: the projection
    stream never gets past its first wait. After the context's host limit (300 ms here) run_mode overwrites the
    counters from another stream, which releases every pending wait, drains the streams and reports the failure."""
    torch = torch_cuda
    p, dev, w, ref = _problem(pkg, oracle, torch)
    ctx = pkg.make_ctx(pkg.World(), ncomm=2)
    try:
        pkg.set_wait_limit_ms(ctx, 50.0, 300.0)
        out = torch.zeros((p.S, p.d), dtype=torch.float16, device="cuda")
        p.debug_target_bias = 1
        t0 = time.perf_counter()
        with pytest.raises(pkg.EfaError, match="released"):
            pkg.run_mode(ctx, pkg.MODE_STREAM, w, out, p)
        assert time.perf_counter() - t0 < 5.0
        torch.cuda.synchronize()                                # nothing is left pending on the device
        p.debug_target_bias = 0
        out.fill_(float("nan"))
        pkg.kernel_status_reset()
        pkg.run_mode(ctx, pkg.MODE_STREAM, w, out, p)
        torch.cuda.synchronize()
        assert pkg.kernel_status()[0] == 0
        assert_close(oracle, out.float().cpu().numpy(), ref, "after the released waits")
    finally:
        pkg.destroy_ctx(ctx)


def _launch(n, *args, timeout_s="1"):
    env = dict(os.environ, EFA_SHIM_TIMEOUT_S=timeout_s)
    return subprocess.run([os.path.join(BIN, "efa_launch"), "-n", str(n), os.path.join(BIN, "shim_selftest"), *args],
                          capture_output=True, text=True, timeout=120, env=env)


def test_mpi_subset_collectives_on_cpu(pkg):
    r = _launch(4, timeout_s="30")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "shim selftest passed on 4 ranks" in r.stdout


def test_a_rank_that_leaves_makes_the_others_time_out_of_the_barrier(pkg):
    """Rank 1 exits before the first barrier. The others wait EFA_SHIM_TIMEOUT_S (one second here), say so and exit
    non-zero; the launcher returns that code."""
    t0 = time.perf_counter()
    r = _launch(3, "--absent", "1")
    assert time.perf_counter() - t0 < 30
    assert r.returncode != 0
    assert "timed out in a barrier" in r.stderr
    assert "passed" not in r.stdout
