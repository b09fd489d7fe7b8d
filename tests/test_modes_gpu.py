"""Every execution mode that writes an output (megatron, sync, overlap, stream) against the CPU checker:
the reference's test matrix (attn_tests.cu:70-87, 124-139) on one rank, plus the single-GPU
configuration of the benchmark plan (S=4096, H=16, d_h=64, tile=128, N(0,1) inputs)."""
import numpy as np
import pytest

from conftest import REFERENCE_CASES, REFERENCE_SEEDS
from helpers import assert_close, normal_inputs_f16, ref_inputs_f16, to_dev

pytestmark = pytest.mark.gpu

CHECKED_MODES = ("megatron", "sync", "overlap", "stream")


@pytest.fixture(scope="module")
def ctx(pkg, torch_cuda):
    c = pkg.make_ctx(pkg.World(), ncomm=3)       # the reference's tests use three communicators
    yield c
    pkg.destroy_ctx(c)


@pytest.mark.parametrize("case", REFERENCE_CASES, ids=lambda c: "S%d_d%d_H%d_t%d_n%d_s%d_c%d" % c)
def test_reference_matrix_single_rank(pkg, oracle, torch_cuda, ctx, case):
    torch = torch_cuda
    S, d, H, tile, nbuf, split, causal = case
    p = pkg.make_params(S, d, H, tile, nbuf, split, causal)
    assert pkg.attn_check_params(p) is None
    seeds = REFERENCE_SEEDS if S <= 512 else REFERENCE_SEEDS[:1]
    for seed in seeds:
        bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, seed)
        ref = oracle.block_rows([vals], d, causal)
        dev = to_dev(torch, bits)
        w = pkg.Weights(*(t.data_ptr() for t in dev))
        for name in CHECKED_MODES:
            out = torch.full((S, d), float("nan"), dtype=torch.float16, device="cuda")
            pkg.kernel_status_reset()
            st = pkg.run_mode(ctx, pkg.parse_mode(name), w, out, p)
            torch.cuda.synchronize()
            assert pkg.kernel_status()[0] == 0
            assert st.wall_ms > 0 and st.kernel_launches > 0
            assert_close(oracle, out.float().cpu().numpy(), ref, f"{name} seed {seed}")


def test_attention_only_modes_leave_output_untouched(pkg, oracle, torch_cuda, ctx):
    torch = torch_cuda
    S, d, H, tile = 512, 256, 4, 128
    p = pkg.make_params(S, d, H, tile)
    bits, _ = ref_inputs_f16(oracle, S, d, H, 1, 0, 42)
    dev = to_dev(torch, bits)
    w = pkg.Weights(*(t.data_ptr() for t in dev))
    out = torch.full((S, d), 7.0, dtype=torch.float16, device="cuda")
    for name in ("attn", "attn_tiled"):
        st = pkg.run_mode(ctx, pkg.parse_mode(name), w, out, p)
        assert st.attn_kernel_ms > 0
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())


def test_diagnostic_flags_skip_stages(pkg, oracle, torch_cuda, ctx):
    """--no_proj / --no_comm (attn_bench.cu:120-121): the run completes and launches fewer kernels."""
    torch = torch_cuda
    S, d, H, tile = 512, 256, 4, 128
    p = pkg.make_params(S, d, H, tile)
    bits, _ = ref_inputs_f16(oracle, S, d, H, 1, 0, 42)
    dev = to_dev(torch, bits)
    w = pkg.Weights(*(t.data_ptr() for t in dev))
    out = torch.zeros((S, d), dtype=torch.float16, device="cuda")
    full = pkg.run_mode(ctx, pkg.MODE_STREAM, w, out, p).kernel_launches
    p.skip_proj = 1
    assert pkg.run_mode(ctx, pkg.MODE_STREAM, w, out, p).kernel_launches == full - p.num_tiles
    p.skip_proj, p.skip_comm = 0, 1
    assert pkg.run_mode(ctx, pkg.MODE_STREAM, w, out, p).kernel_launches == full


@pytest.mark.parametrize("causal", [0, 1])
def test_single_gpu_benchmark_configuration(pkg, oracle, torch_cuda, ctx, causal):
    """S=4096, H=16, d_h=64, D=1024, tile=128, N(0,1) Q/K/V, W_O ~ N(0, 1/1024); modes attn, megatron,
    stream; checked on a fixed sample of rows from the first, last and interior tiles."""
    torch = torch_cuda
    S, d, H, tile = 4096, 1024, 16, 128
    p = pkg.make_params(S, d, H, tile, causal=causal)
    bits, vals = normal_inputs_f16(pkg, oracle, p, 0, 42)
    rng = np.random.default_rng(5)
    rows = np.unique(np.concatenate([np.arange(0, 64), np.arange(S - 64, S), rng.integers(64, S - 64, 128)])).astype(np.int32)
    ref = oracle.block_rows([vals], d, causal, rows)
    dev = to_dev(torch, bits)
    w = pkg.Weights(*(t.data_ptr() for t in dev))
    for name in ("megatron", "stream"):
        out = torch.full((S, d), float("nan"), dtype=torch.float16, device="cuda")
        pkg.run_mode(ctx, pkg.parse_mode(name), w, out, p)
        torch.cuda.synchronize()
        got = out.float().cpu().numpy()
        assert np.isfinite(got).all()
        assert_close(oracle, got[rows], ref, name)


@pytest.mark.parametrize("shape", [(512, 256, 4, 128, 1), (512, 256, 4, 128, 2), (2048, 512, 4, 128, 4), (2048, 1024, 8, 256, 1),
                                   # 64-row tiles: S/8 rows per chunk would be 64 or 192 rows, which the chunking rounds to
                                   # multiples of 128 so that no key stage reaches into rows still being copied in
                                   (512, 256, 4, 64, 1), (1536, 512, 4, 64, 1), (1536, 256, 8, 64, 1)],
                         ids=lambda c: "S%d_d%d_H%d_t%d_s%d" % c)
def test_host_buffer_entry_point(pkg, oracle, torch_cuda, ctx, shape):
    """Stream mode on pinned host buffers: copy-in, compute and copy-out pipelined over row chunks; with
    split-KV every chunk's partials sit at their own rows of one workspace."""
    torch = torch_cuda
    S, d, H, tile, split = shape
    p = pkg.make_params(S, d, H, tile, split=split, causal=1)
    bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, 123)
    ref = oracle.block_rows([vals], d, 1)
    pinned = [torch.from_numpy(b.view(np.float16)).pin_memory() for b in bits]
    out = torch.zeros((S, d), dtype=torch.float16).pin_memory()
    st = pkg.run_mode_host(ctx, pkg.MODE_STREAM, *pinned, out, p)
    assert st.wall_ms > 0
    assert_close(oracle, out.float().numpy(), ref)


@pytest.mark.parametrize("case", [(512, 256, 8, 128, 0), (1024, 512, 8, 256, 1), (1024, 1024, 8, 64, 0), (2048, 1024, 8, 512, 1),
                                  (448, 512, 4, 64, 1), (4096, 1024, 16, 128, 1)],
                         ids=lambda c: "S%d_d%d_H%d_t%d_c%d" % c)
def test_stream_mode_with_the_fused_projection_kernel_single_rank(pkg, oracle, torch_cuda, ctx, case):
    """--reduce p2p on one rank: the persistent kernel polls the tile counters, projects each 128-row
    block as it completes and writes the output directly (nothing to reduce). Run twice: tile counters
    and flags are never reset between runs, the wait targets grow instead."""
    torch = torch_cuda
    S, d, H, tile, causal = case
    p = pkg.make_params(S, d, H, tile, 2, 1, causal)
    p.reduce = pkg.REDUCE_P2P
    bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, 42) if S <= 2048 else normal_inputs_f16(pkg, oracle, p, 0, 42)
    rows = None if S <= 2048 else np.arange(0, S, 13, dtype=np.int32)
    ref = oracle.block_rows([vals], d, causal, rows)
    dev = to_dev(torch, bits)
    w = pkg.Weights(*(t.data_ptr() for t in dev))
    out = torch.full((S, d), float("nan"), dtype=torch.float16, device="cuda")
    for rep in range(3):
        out.fill_(float("nan"))
        pkg.kernel_status_reset()
        st = pkg.run_mode(ctx, pkg.MODE_STREAM, w, out, p)
        torch.cuda.synchronize()
        assert pkg.kernel_status()[0] == 0, pkg.kernel_status()
        assert st.kernel_launches == 2
        got = out.float().cpu().numpy()
        assert_close(oracle, got if rows is None else got[rows], ref, f"rep {rep}")


@pytest.mark.parametrize("order", ["ASCENDING", "DESCENDING", "MIXED"])
@pytest.mark.parametrize("case", [(4096, 1024, 16, 128, 1), (2048, 1024, 8, 64, 2), (1280, 512, 8, 128, 1)],
                         ids=lambda c: "S%d_d%d_H%d_t%d_s%d" % c)
def test_stream_mode_row_orders(pkg, oracle, torch_cuda, ctx, case, order):
    """Causal stream mode with the rows taken first-to-last, last-to-first and mixed (two blocks from the end, one from
    the start): the consumer waits for the groups in the order the attention launch completes them."""
    torch = torch_cuda
    S, d, H, tile, split = case
    p = pkg.make_params(S, d, H, tile, 2, split, 1)
    p.row_order = getattr(pkg, "ROWS_" + order)
    if order == "MIXED":
        assert sorted(pkg.stream_row_blocks(p)) == list(range((S + 255) // 256))
    bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, 42) if S <= 2048 else normal_inputs_f16(pkg, oracle, p, 0, 42)
    rows = None if S <= 2048 else np.arange(0, S, 13, dtype=np.int32)
    ref = oracle.block_rows([vals], d, 1, rows)
    dev = to_dev(torch, bits)
    w = pkg.Weights(*(t.data_ptr() for t in dev))
    for rep in range(2):
        out = torch.full((S, d), float("nan"), dtype=torch.float16, device="cuda")
        pkg.kernel_status_reset()
        pkg.run_mode(ctx, pkg.MODE_STREAM, w, out, p)
        torch.cuda.synchronize()
        assert pkg.kernel_status()[0] == 0, pkg.kernel_status()
        got = out.float().cpu().numpy()
        assert_close(oracle, got if rows is None else got[rows], ref, f"{order} rep {rep}")


@pytest.mark.parametrize("case", [(1024, 512, 8, 128, 1, 1), (2048, 1024, 8, 256, 0, 1), (4096, 1024, 16, 128, 1, 1), (2048, 512, 8, 128, 1, 2)],
                         ids=lambda c: "S%d_d%d_H%d_t%d_c%d_s%d" % c)
def test_stream_mode_with_reserved_sms(pkg, oracle, torch_cuda, ctx, case):
    """The persistent form of the attention kernel: fewer CTAs than SMs, work items taken from a global counter,
    barriers rebuilt per item. 100 reserved SMs leave 48 CTAs, so every CTA processes several items."""
    torch = torch_cuda
    S, d, H, tile, causal, split = case
    p = pkg.make_params(S, d, H, tile, 2, split, causal)
    p.reserve_sms = 100
    bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, 42) if S <= 2048 else normal_inputs_f16(pkg, oracle, p, 0, 42)
    rows = None if S <= 2048 else np.arange(0, S, 13, dtype=np.int32)
    ref = oracle.block_rows([vals], d, causal, rows)
    dev = to_dev(torch, bits)
    w = pkg.Weights(*(t.data_ptr() for t in dev))
    for rep in range(2):
        out = torch.full((S, d), float("nan"), dtype=torch.float16, device="cuda")
        pkg.kernel_status_reset()
        pkg.run_mode(ctx, pkg.MODE_STREAM, w, out, p)
        torch.cuda.synchronize()
        assert pkg.kernel_status()[0] == 0, pkg.kernel_status()
        got = out.float().cpu().numpy()
        assert_close(oracle, got if rows is None else got[rows], ref, f"rep {rep}")


@pytest.mark.parametrize("case", [(512, 256, 4, 128, 2, 1, 0), (1024, 512, 8, 128, 3, 2, 1), (2048, 1024, 8, 256, 2, 1, 1)],
                         ids=lambda c: "S%d_d%d_H%d_t%d_n%d_s%d_c%d" % c)
def test_residual_is_added_to_every_reduced_group(pkg, oracle, torch_cuda, ctx, case):
    """The step after the block (the reference stops at the AllReduce output, run_drivers.cuh:22-24):
    output = residual + block, the residual added group by group as the rows land. Checked bit for bit
    against the same mode without a residual plus one fp16 addition (that run is checked against the CPU checker)."""
    torch = torch_cuda
    S, d, H, tile, nbuf, split, causal = case
    p = pkg.make_params(S, d, H, tile, nbuf, split, causal)
    bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, 42)
    ref = oracle.block_rows([vals], d, causal)
    dev = to_dev(torch, bits)
    w = pkg.Weights(*(t.data_ptr() for t in dev))
    g = torch.Generator(device="cpu").manual_seed(7)
    residual = (torch.rand((S, d), generator=g) - 0.5).to(torch.float16).cuda()
    for name in CHECKED_MODES:
        plain = torch.zeros((S, d), dtype=torch.float16, device="cuda")
        pkg.run_mode(ctx, pkg.parse_mode(name), w, plain, p)
        out = torch.full((S, d), float("nan"), dtype=torch.float16, device="cuda")
        pkg.kernel_status_reset()
        st = pkg.run_mode_residual(ctx, pkg.parse_mode(name), w, residual, out, p)
        torch.cuda.synchronize()
        assert pkg.kernel_status()[0] == 0
        assert st.kernel_launches > 0
        assert torch.equal(out, plain + residual), name
        assert_close(oracle, plain.float().cpu().numpy(), ref, f"{name} without residual")


def test_residual_is_rejected_where_no_block_output_exists(pkg, oracle, torch_cuda, ctx):
    torch = torch_cuda
    S, d, H, tile = 512, 256, 4, 128
    p = pkg.make_params(S, d, H, tile)
    bits, _ = ref_inputs_f16(oracle, S, d, H, 1, 0, 42)
    dev = to_dev(torch, bits)
    w = pkg.Weights(*(t.data_ptr() for t in dev))
    out = torch.zeros((S, d), dtype=torch.float16, device="cuda")
    res = torch.zeros((S, d), dtype=torch.float16, device="cuda")
    for name in ("attn", "attn_tiled", "comm"):
        with pytest.raises(pkg.EfaError, match="no block output"):
            pkg.run_mode_residual(ctx, pkg.parse_mode(name), w, res, out, p)
    p.skip_comm = 1
    with pytest.raises(pkg.EfaError, match="needs the projection and the reduction"):
        pkg.run_mode_residual(ctx, pkg.MODE_STREAM, w, res, out, p)


@pytest.mark.parametrize("case", [(512, 256, 4, 128, 2, 1, 0), (1024, 512, 8, 128, 3, 2, 1), (2048, 1024, 8, 256, 2, 1, 1),
                                  (2048, 4096, 32, 128, 2, 1, 1)],
                         ids=lambda c: "S%d_d%d_H%d_t%d_n%d_s%d_c%d" % c)
def test_fp32_partial_sums_and_output(pkg, oracle, torch_cuda, ctx, case):
    """proj_f32: the projection keeps its fp32 accumulator, the reduction and the output are fp32 (the
    reference's types, attn_main.cu:262-273, run_drivers.cu:26-30). Same gate as the fp16 path, and the
    fp16 path's output must be this one rounded once (single rank: nothing is summed)."""
    torch = torch_cuda
    S, d, H, tile, nbuf, split, causal = case
    p = pkg.make_params(S, d, H, tile, nbuf, split, causal)
    # the wide shape runs the 256-column projection tile; it is checked on a sample of rows
    bits, vals = ref_inputs_f16(oracle, S, d, H, 1, 0, 42) if d < 4096 else normal_inputs_f16(pkg, oracle, p, 0, 42)
    rows = None if d < 4096 else np.arange(0, S, 7, dtype=np.int32)
    ref = oracle.block_rows([vals], d, causal, rows)
    dev = to_dev(torch, bits)
    w = pkg.Weights(*(t.data_ptr() for t in dev))
    for name in CHECKED_MODES:
        half = torch.zeros((S, d), dtype=torch.float16, device="cuda")
        p.proj_f32 = 0
        pkg.run_mode(ctx, pkg.parse_mode(name), w, half, p)
        out = torch.full((S, d), float("nan"), dtype=torch.float32, device="cuda")
        p.proj_f32 = 1
        pkg.kernel_status_reset()
        st = pkg.run_mode(ctx, pkg.parse_mode(name), w, out, p)
        torch.cuda.synchronize()
        assert pkg.kernel_status()[0] == 0
        assert st.kernel_launches > 0
        got = out.cpu().numpy()
        assert_close(oracle, got if rows is None else got[rows], ref, f"{name} fp32")
        assert torch.equal(out.to(torch.float16), half), name
    p.reduce = pkg.REDUCE_P2P
    with pytest.raises(pkg.EfaError, match="NCCL reduction"):
        pkg.run_mode(ctx, pkg.MODE_STREAM, w, out, p)
