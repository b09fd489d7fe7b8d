"""Several ranks on several GPUs (torchrun; gloo for the host control plane, NCCL / peer memory / NVLink multicast
for the data): every output-writing mode and every reduction against the CPU checker's sum over ranks
(attn_tests.cu:27-60, 124-139). Small cases use the reference recipe's rank-specific weights and are checked in
full; the benchmark plan's eight-rank configurations use N(0,1) inputs and are checked on sampled rows of the
first, last and interior tiles. Every path is held to the same gate: max-abs <= 2e-3 and max-abs / max|ref| <= 1e-2.
Skipped on a machine with too few GPUs."""
import json
import os
import subprocess
import sys
import textwrap

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

# reduce: "nccl" | "nvls" | "pull" (fp32 partial sums on the wire, the default) | "nccl_w16" | "nvls_w16" (fp16 partial sums
# on the wire) | "nccl_f32out" (proj_f32: fp32 partial sums AND fp32 output, the reference's types) | "p2p" (fused kernel).
# Paths with fp16 partial sums carry half an fp16 ulp of every partial sum on top of the final rounding; they are held
# to the same gate on two ranks. On eight ranks they do not meet it (measured: 2.23e-3 on S=960, d=1024 with the
# reference's inputs), which is why fp32 partial sums are the default; the option is not part of the eight-rank tests.
WORKER = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
    import numpy as np, torch, torch.distributed as dist
    import __graft_entry__ as entry
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group(backend="cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local))
    pkg = entry.load_package(); oracle = entry.load_oracle()
    cases = json.loads({cases!r})
    ok = True
    ctx = None
    try:
        ctx = pkg.make_ctx(pkg.World.from_torch(None, local_device=local), ncomm=int({ncomm!r}))
        pkg.set_wait_limit_ms(ctx, 20000.0, 60000.0)
        outs = {{}}
        for case in cases:
            S, d, H, tile, nbuf, split, causal = case["shape"]
            if H % world != 0:
                continue
            p = pkg.make_params(S, d, H, tile, nbuf, split, causal, world)
            why = pkg.attn_check_params(p)
            if why:
                print(f"rank {{rank}} skip {{case['shape']}}: {{why}}", flush=True)
                continue

            def inputs(r):
                if case["data"] == "ref":
                    Q, K, V, W = oracle.ref_inputs(S, d, H, world, r, 42)
                    return tuple(oracle.round_f16(x) for x in (Q, K, V, W))
                bits = [np.zeros((p.H_local, S, p.d_h), np.uint16) for _ in range(3)] + [np.zeros((p.d_local, d), np.uint16)]
                pkg.fill_host_inputs(p, r, 42, pkg.RECIPE_NORMAL, *bits)
                return tuple(bits)

            rows = None
            if case.get("rows"):
                rng = np.random.default_rng(7)
                n = int(case["rows"])
                rows = np.unique(np.concatenate([np.arange(0, 8), np.arange(S - 8, S), rng.integers(8, S - 8, n)])).astype(np.int32)
            nref = S if rows is None else len(rows)
            ref = torch.zeros((nref, d), dtype=torch.float32)
            if rank == 0:          # the result is the same on every rank: one rank works out the expected rows
                ref = torch.from_numpy(oracle.block_rows((tuple(oracle.widen_f16(b) for b in inputs(r)) for r in range(world)),
                                                         d, causal, rows))
            dist.broadcast(ref, src=0)
            ref = ref.numpy()
            mine = inputs(rank)
            dev = [torch.from_numpy(b.view(np.float16)).cuda() for b in mine]
            w = pkg.Weights(*(t.data_ptr() for t in dev))
            for reduce in case["reduces"]:
                if reduce == "p2p" and (split != 1 or d % (128 * world) != 0):
                    continue
                p.reduce = dict(nccl=pkg.REDUCE_NCCL, p2p=pkg.REDUCE_P2P, nvls=pkg.REDUCE_NVLS, pull=pkg.REDUCE_PULL)[reduce.split("_")[0]]
                p.proj_f32 = 1 if reduce == "nccl_f32out" else 0
                p.wire = pkg.WIRE_F16 if reduce.endswith("_w16") else pkg.WIRE_AUTO
                odt = torch.float32 if p.proj_f32 else torch.float16
                for name in (case["modes"] if reduce != "p2p" else ["stream"]):
                    for gt in (case.get("group_tiles", [0]) if name == "stream" and reduce != "p2p" else [0]):
                        p.group_tiles = gt
                        out = outs.setdefault((S, d, odt), torch.empty((S, d), dtype=odt, device="cuda"))
                        out.fill_(float("nan"))
                        torch.cuda.synchronize()
                        dist.barrier()
                        pkg.kernel_status_reset()
                        good, msg = False, ""
                        try:
                            for rep in range(2 if reduce in ("p2p", "nvls", "nvls_w16", "pull") else 1):     # counters / flags only grow: run twice
                                pkg.run_mode(ctx, pkg.parse_mode(name), w, out, p)
                            torch.cuda.synchronize()
                            got = out.float().cpu().numpy()
                            ma, mr = oracle.compare(got if rows is None else got[rows], ref)
                            good = bool(np.isfinite(ma)) and ma <= 2e-3 and ma <= 1e-2 * mr and pkg.kernel_status()[0] == 0
                            msg = f"max_abs={{ma:.3e}} max_ref={{mr:.3e}} status={{pkg.kernel_status()}}"
                        except Exception as e:      # reported, never raised: every rank must reach the teardown below
                            msg = f"error: {{e}}"
                        ok &= good
                        print(f"rank {{rank}} S={{S}} d={{d}} H={{H}} tile={{tile}} split={{split}} causal={{causal}} {{reduce}} {{name}} "
                              f"group_tiles={{gt}}: {{msg}} {{'PASS' if good else 'FAIL'}}", flush=True)
            del dev
            outs.clear()
            torch.cuda.empty_cache()
    except Exception as e:
        ok = False
        print(f"rank {{rank}}: {{type(e).__name__}}: {{e}} FAIL", flush=True)
    flag = torch.tensor([1 if ok else 0])
    try:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if ctx is not None:
            pkg.destroy_ctx(ctx)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:
        print(f"rank {{rank}}: teardown: {{e}} FAIL", flush=True)
        flag[0] = 0
    sys.exit(0 if int(flag[0]) == 1 else 1)
""")

ALL_MODES = ["megatron", "sync", "overlap", "stream"]

# S, d, H, tile, nbuf, split, causal — shapes of the reference's matrix (attn_tests.cu:70-84) whose H divides by the ranks
SMALL_2 = [(512, 256, 8, 128, 2, 1, 0), (1024, 512, 8, 256, 2, 1, 1), (1024, 1024, 8, 64, 3, 1, 0),
           (2048, 512, 8, 128, 2, 4, 1), (512, 256, 4, 64, 2, 2, 0), (448, 512, 8, 64, 2, 1, 1)]
SMALL_8 = [(1024, 1024, 8, 128, 2, 1, 1), (960, 1024, 8, 64, 3, 1, 1)]


def small(shapes, reduces, modes=ALL_MODES, group_tiles=(0,)):
    return [dict(shape=list(s), data="ref", reduces=list(reduces), modes=list(modes), group_tiles=list(group_tiles)) for s in shapes]


def run_workers(tmp_path, nproc, cases, ncomm=3, timeout=1500):
    import torch
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT, cases=json.dumps(cases), ncomm=ncomm))
    port = 29600 + (os.getpid() % 1000)
    env = dict(os.environ, OMP_NUM_THREADS="8")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                       capture_output=True, text=True, timeout=timeout, env=env)
    print(r.stdout[-12000:])
    assert r.returncode == 0, r.stdout[-6000:] + r.stderr[-4000:]
    assert "FAIL" not in r.stdout
    assert "PASS" in r.stdout


@pytest.mark.timeout(1700)
def test_two_ranks_nccl_reduction(tmp_path):
    run_workers(tmp_path, 2, small(SMALL_2, ("nccl", "nccl_w16", "nccl_f32out")))


@pytest.mark.timeout(1700)
def test_two_ranks_fused_p2p_reduction(tmp_path):
    """stream mode with the projection + reduction fused in one persistent kernel over peer memory."""
    run_workers(tmp_path, 2, small(SMALL_2, ("p2p",)))


@pytest.mark.timeout(1700)
def test_two_ranks_multicast_reduction(tmp_path):
    """every mode with the reduction done by the NVSwitch (multimem.ld_reduce / multimem.st), and with the sum done on
    the SM over bulk copies of the peers' partial sums, the result multicast (pull)."""
    run_workers(tmp_path, 2, small(SMALL_2, ("nvls", "nvls_w16", "pull"), group_tiles=(0, 1)))


@pytest.mark.timeout(1700)
def test_four_ranks_all_reductions(tmp_path):
    run_workers(tmp_path, 4, small(SMALL_2[:4], ("nccl", "p2p", "nvls", "pull"), modes=["megatron", "stream"]))


@pytest.mark.timeout(1700)
def test_eight_ranks_all_reductions(tmp_path):
    run_workers(tmp_path, 8, small(SMALL_8, ("nccl", "nccl_f32out", "p2p", "nvls", "pull")))


@pytest.mark.timeout(2700)
def test_eight_ranks_benchmark_configurations(tmp_path):
    """The eight-rank configurations of the benchmark plan as whole blocks: S=16384 non-causal and S=32768 causal
    (H=16, d_h=64), S=65536 with 64 / 128 / 256-row tiles, and S=32768, H=32, d_h=128 causal; N(0,1) inputs,
    W_O ~ N(0, 1/d); both schedules (grouped, and one launch per tile where the tile count allows) and all four
    reductions, checked on sampled rows."""
    R = ("nccl", "nvls", "pull", "p2p")
    cases = [
        dict(shape=[16384, 1024, 16, 128, 2, 1, 0], data="normal", rows=40, reduces=R, modes=["megatron", "stream"], group_tiles=[0, 1]),
        dict(shape=[32768, 1024, 16, 128, 2, 1, 1], data="normal", rows=40, reduces=R, modes=["megatron", "stream"], group_tiles=[0]),
        dict(shape=[32768, 4096, 32, 128, 2, 1, 1], data="normal", rows=40, reduces=R, modes=["megatron", "stream"], group_tiles=[0, 1]),
        dict(shape=[65536, 1024, 16, 64, 2, 1, 1], data="normal", rows=32, reduces=("nccl", "nvls", "pull"), modes=["stream"], group_tiles=[0]),
        dict(shape=[65536, 1024, 16, 128, 2, 1, 1], data="normal", rows=32, reduces=R, modes=["stream"], group_tiles=[0]),
        dict(shape=[65536, 1024, 16, 256, 2, 1, 0], data="normal", rows=32, reduces=("nccl", "nvls", "pull"), modes=["stream"], group_tiles=[0]),
    ]
    run_workers(tmp_path, 8, cases, ncomm=4, timeout=2400)


@pytest.mark.timeout(2700)
def test_two_ranks_benchmark_shape(tmp_path):
    """S=32768, H=32, d_h=128 causal on two ranks (16 heads each), all reductions, sampled rows."""
    cases = [dict(shape=[32768, 4096, 32, 128, 2, 1, 1], data="normal", rows=32, reduces=("nccl", "nvls", "pull", "p2p"),
                  modes=["megatron", "stream"], group_tiles=[0])]
    run_workers(tmp_path, 2, cases, ncomm=4, timeout=2400)
