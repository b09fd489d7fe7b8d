#!/usr/bin/env python
"""Benchmark of the tensor-parallel attention block (attention + W_o + AllReduce) on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--mode stream|megatron]

One rank per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE). A step is one pass of the block over
the whole sequence. Workload: S=32768, H=32, d_h=128 (d=4096), causal, tile=128, ncomm=4, heads
sharded over the N ranks (strong scaling: the global problem is fixed). Rank 0 prints one JSON line.

`value` is the block time with the fp16 inputs resident in HBM; `e2e` is the same block through the
host-buffer entry point (pinned host Q/K/V/W_O copied in, fp16 result copied out, every step).
`--impl reference` times the unmodified reference programs built under oracle/_ref (its own CUDA
build; the reference has no CPU implementation), or says why it cannot: at this workload's tile and ncomm,
and at its own best tile (the tiles and split of its sweep script).

Every time in the line is the mean over the timed steps of the same per-step figure (one statistic
throughout): `value`, `modes_ms` and `roofline.attn_kernel_ms` can be compared with one another.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(S=32768, H=32, d_h=128, causal=1, tile=128, ncomm=4, split=1, nbuf=2)
METRIC = "ms per TP attention block (attn+W_o+AllReduce)"
NVLINK_GBS = 900.0      # per direction and GPU, nominal: the link bound the block roofline is taken against

# --reduce auto: the reduction that measured fastest for this workload at each rank count (stream mode, ms per
# block on B200s of one NVSwitch box; the table these figures come from is in the design notes). One rank
# reduces nothing; "nvls" needs NVLink multicast and is only chosen where efa reports it usable.
REDUCE_BY_RANKS = {1: "nccl", 2: "pull", 4: "pull", 8: "pull"}

# DRAM bytes (read + written) of one attention launch of the benchmark shape with all 32 heads on one GPU, by
# (mode, rows taken last-first): ncu captures, one launch each.
ATTN_TRAFFIC_32_HEADS = {("stream", False): 5.105e9, ("stream", True): 5.212e9}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            pk = json.load(f)
        return dict(tflops=float(pk["bf16_tflops"]), tflops_sustained=float(pk.get("bf16_tflops_sustained", pk["bf16_tflops"])),
                    hbm_gbs=float(pk["hbm_gbs"]), source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


def attention_flops(S, d_h, H_local, causal):
    """Algorithmic FLOPs of one rank's attention: 4*S^2*d_h*H_local, or for causal the block-granular
    count of 64-row blocks sweeping keys 0..(i+1)*64."""
    if not causal:
        return 4.0 * S * S * d_h * H_local
    nb = S // 64
    return 4.0 * 64 * 64 * d_h * H_local * nb * (nb + 1) / 2


def bind_near_gpu(device_index):
    """Run this process on the CPUs of the GPU's NUMA node, so that the pinned host buffers it allocates next are
    first touched there: with several ranks on one host, copies from the far socket's memory halve the PCIe rate each
    GPU sees. Returns the node, or None where the topology cannot be read (nothing is changed then)."""
    try:
        import torch
        pr = torch.cuda.get_device_properties(device_index)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read())
        if node < 0:
            return None
        cpus = set()
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if len(allowed) < 4:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


class ClockSampler:
    """SM clock and throttle-reason samples taken DURING the timed region (NVML, every 5 ms, in a thread of
    this process; `nvidia-smi -lms` cannot sample a region of a few tens of milliseconds)."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, device_index):
        self.device_index = device_index
        self.samples, self.masks = [], 0
        self.max_mhz = None
        self.thread = None
        self.stop_flag = False

    def start(self):
        try:
            import threading
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(self.device_index).uuid)
            try:
                h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode() if not uuid.startswith("GPU-") else uuid.encode())
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.device_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self.stop_flag:
                    try:
                        self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        self.masks |= int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                    except Exception:
                        pass
                    time.sleep(0.005)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=[], samples=0)
        if self.thread is None:
            return out
        self.stop_flag = True
        self.thread.join(timeout=2)
        if self.samples:
            out.update(sm_mhz=statistics.median(self.samples), sm_min_mhz=min(self.samples), samples=len(self.samples),
                       reasons=sorted(n for bit, n in self.REASONS.items() if self.masks & bit))
        return out


def cpu_baseline(pkg, oracle, p, bits_rank0, budget_rows):
    """The CPU checker (a port: the reference has no CPU path) timed on a bounded sample of query rows of
    rank 0's shard, scaled to the whole sequence. Rows are spread evenly, so the causal average holds."""
    import numpy as np
    vals = tuple(oracle.widen_f16(b) for b in bits_rank0)
    rows = np.linspace(0, p.S - 1, budget_rows).astype(np.int32)
    t0 = time.perf_counter()
    oracle.block_rows([vals], p.d, p.causal, rows)
    dt = time.perf_counter() - t0
    threads = int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))
    return dict(value=dt * 1e3 * p.S / budget_rows, unit="ms", cores=threads, kind="port",
                sample=f"{budget_rows} evenly spaced query rows of rank 0's {p.H_local} heads, full key sweep, "
                       f"{dt:.1f} s measured, scaled by S/rows (extrapolated)")


def run_reference(args, world_size, rank):
    """The unmodified reference (its own attn_bench, built for sm_100a under oracle/_ref with the
    shared-memory MPI subset), same shape / tile / ncomm, its natural fp32 projection and AllReduce."""
    if rank != 0:
        return None
    W = WORKLOAD
    base = dict(metric=METRIC, unit="ms", n_gpus=world_size, steps=args.steps, warmup=args.warmup,
                higher_is_better=False, scaling="strong", vs_baseline=None, dtype="f16 in / f32 accumulate, projection and reduction in f32",
                data="synthetic", impl="reference",
                config=dict(workload=f"S={W['S']} H={W['H']} d_h={W['d_h']} causal tile={W['tile']} ncomm={W['ncomm']} TP={world_size}",
                            mode=args.mode))
    exe = os.path.join(ROOT, "oracle", "_ref", "attn_bench")
    launch = os.path.join(ROOT, "oracle", "_ref", "efa_launch")
    if not (os.path.exists(exe) and os.path.exists(launch)):
        return dict(impl="reference", unavailable="oracle/_ref/attn_bench is not built (run __graft_entry__.build() where the reference sources are mounted)")
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)

    def run(tile, ncomm, split, modes, warmup, trials):
        cmd = [launch, "-n", str(world_size), exe, "--S", str(W["S"]), "--H", str(W["H"]), "--d_h", str(W["d_h"]),
               "--tile", str(tile), "--ncomm", str(ncomm), "--split", str(split), "--causal", "--modes", modes,
               "--warmup", str(warmup), "--trials", str(trials)]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, env=env)
        except subprocess.TimeoutExpired:
            return None, "the reference attn_bench did not finish within 1500 s"
        if r.returncode != 0:
            return None, "reference attn_bench exited %d: %s" % (r.returncode, r.stderr.strip().splitlines()[-1:] or "")
        rows = {}
        for line in r.stdout.splitlines():
            f = line.split(",")
            if len(f) >= 17 and f[0].isdigit():
                rows[f[11]] = dict(min=float(f[12]), max=float(f[13]), mean=float(f[14]), median=float(f[15]), std=float(f[16]))
        return rows, None

    rows, why = run(W["tile"], W["ncomm"], W["split"], "attn,megatron,stream", args.warmup, args.steps)
    if rows is None:
        return dict(impl="reference", unavailable=why)
    if args.mode not in rows:
        return dict(impl="reference", unavailable="no %s row in the reference's output" % args.mode)
    ms = rows[args.mode]["mean"]
    # The reference at its own best: the tiles and split-KV factor its sweep script uses (S/32 ... S/8, --split 4,
    # eight communicators), fewer trials each. Reported beside the like-for-like figure, not in place of it.
    best = None
    sweep = {}
    for tile in (1024, 2048, 4096):
        r2, _ = run(tile, 8, 4, "stream", 2, max(3, min(args.steps, 5)))
        if r2 and "stream" in r2:
            sweep["tile=%d split=4 ncomm=8" % tile] = r2["stream"]["mean"]
    if sweep:
        k = min(sweep, key=sweep.get)
        best = dict(stream_ms=sweep[k], config=k, all=sweep)
    base.update(value=ms, ms_per_step=ms, tokens_per_s=W["S"] / (ms * 1e-3),
                modes_ms={k: v["mean"] for k, v in rows.items()},
                best_of_its_own_sweep=best,
                best_ms=min([ms, rows.get("megatron", {}).get("mean", ms)] + ([best["stream_ms"]] if best else [])),
                cpu_baseline=dict(value=ms, unit="ms", cores=0, kind="reference",
                                  sample="the reference's own CUDA programs (it has no CPU implementation); whole workload, mean of the timed trials"),
                e2e=dict(value=ms, unit="ms", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=None)
    return base


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="stream", choices=["stream", "megatron"])
    ap.add_argument("--reduce", default="auto", choices=["auto", "nccl", "p2p", "nvls", "pull"],
                    help="how the partial sums are reduced: NCCL AllReduce per group of tiles, the persistent "
                         "projection+reduction kernel over peer memory (stream mode), the NVSwitch through an NVLink "
                         "multicast object, or bulk copies of the peers' fp32 partial sums added on the SM and multicast "
                         "(pull); auto = the one that measured fastest for this rank count")
    ap.add_argument("--reduce-ctas", type=int, default=0,
                    help="thread blocks of the nvls / pull reduction kernel (0 = the library's default)")
    ap.add_argument("--reserve-sms", type=int, default=0,
                    help="stream mode: SMs the attention kernel leaves to the projection and the reduction (0 = none: it "
                         "launches one block per work item and the others take SMs as its blocks retire)")
    ap.add_argument("--wire", default="auto", choices=["auto", "f16", "f32"],
                    help="element type of the partial sums on the links: the fp32 accumulators (auto), or fp16 (half the bytes, "
                         "one more rounding per partial sum)")
    ap.add_argument("--order", default="auto", choices=["auto", "asc", "desc", "mixed"],
                    help="stream mode: order in which the rows are taken and waited for (auto = last rows first under a causal mask)")
    ap.add_argument("--group-tiles", type=int, default=0, help="tiles per projection + AllReduce launch (0 = auto, 1 = per tile)")
    ap.add_argument("--split", type=int, default=0,
                    help="split-KV factor of the attention kernel (the reference's --split); 0 = the value chosen for this rank count")
    ap.add_argument("--cpu-rows", type=int, default=2048,
                    help="query rows of the CPU baseline sample (0 = skip); 2048 rows are about 10 s on 16 host threads")
    ap.add_argument("--S", type=int, default=WORKLOAD["S"], help="override the sequence length (profiling captures only)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.S == WORKLOAD["S"] else args.warmup

    rank = int(os.environ.get("RANK", 0))
    world_size = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.gpus != world_size and rank == 0 and world_size > 1:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world_size}", file=sys.stderr)

    if args.impl == "reference":
        line = run_reference(args, world_size, rank)
        if line is not None:
            emit(line)
        return 0

    import numpy as np
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    pkg = entry.load_package()
    pkg.lib()                                   # fails loudly when the CUDA library is not built
    torch.cuda.set_device(local_rank)
    numa_node = bind_near_gpu(local_rank)
    if world_size > 1:
        dist.init_process_group(backend="cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local_rank))
        world = pkg.World.from_torch(None, local_device=local_rank)
    else:
        world = pkg.World(0, 1, local_rank)

    W = dict(WORKLOAD)
    W["S"] = args.S
    d = W["H"] * W["d_h"]
    if args.split > 0:
        W["split"] = args.split
    p = pkg.make_params(W["S"], d, W["H"], W["tile"], W["nbuf"], W["split"], W["causal"], world_size)
    why = pkg.attn_check_params(p)
    if why:
        raise SystemExit(f"invalid workload for {world_size} ranks: {why}")
    chosen_by_table = args.reduce == "auto"
    reduce_note = None
    if chosen_by_table:
        args.reduce = REDUCE_BY_RANKS.get(world_size, "nccl")
    p.reduce = dict(nccl=pkg.REDUCE_NCCL, p2p=pkg.REDUCE_P2P, nvls=pkg.REDUCE_NVLS, pull=pkg.REDUCE_PULL)[args.reduce]
    p.row_order = dict(auto=pkg.ROWS_AUTO, asc=pkg.ROWS_ASCENDING, desc=pkg.ROWS_DESCENDING, mixed=pkg.ROWS_MIXED)[args.order]
    p.wire = dict(auto=pkg.WIRE_AUTO, f16=pkg.WIRE_F16, f32=pkg.WIRE_F32)[args.wire]
    p.group_tiles = args.group_tiles
    p.reduce_ctas = args.reduce_ctas
    p.reserve_sms = args.reserve_sms
    mode = pkg.parse_mode(args.mode)
    descending = bool(pkg.stream_plan(p)[2])

    # Synthetic inputs in pinned host memory (N(0,1) Q/K/V, W_O ~ N(0, 1/d)), then resident copies.
    qkv_shape = (p.H_local, p.S, p.d_h)
    host = [torch.empty(qkv_shape, dtype=torch.float16).pin_memory() for _ in range(3)]
    host.append(torch.empty((p.d_local, p.d), dtype=torch.float16).pin_memory())
    # The reduced result is identical on every rank: each rank reads back its own share of the rows (S / N of them)
    # over its own PCIe link, so that every row reaches host memory exactly once.
    share = p.S // world_size
    host_out = torch.empty((share, p.d), dtype=torch.float16).pin_memory()
    pkg.fill_host_inputs(p, rank, 42, pkg.RECIPE_NORMAL, *host)
    dev = [h.cuda() for h in host]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")      # > 126 MB L2
    weights = pkg.Weights(*(t.data_ptr() for t in dev))
    ctx = pkg.make_ctx(world, ncomm=W["ncomm"])
    if args.reduce in ("nvls", "pull") and world_size > 1:
        # the multicast reduction writes its result in place into the context's symmetric region
        class _Region:
            def __init__(self, ptr, shape):
                self.__cuda_array_interface__ = dict(shape=shape, typestr="<f2", data=(ptr, False), version=2)
        try:
            out = torch.as_tensor(_Region(pkg.nvls_output(ctx, p), (p.S, p.d)), device="cuda")
        except pkg.EfaError as e:
            # Setting up the multicast region is collective and fails on every rank alike (no NVLink multicast on this
            # machine, no CUDA IPC between the ranks). A reduction named on the command line fails here; the one taken
            # from the table is replaced by NCCL, and the line says so.
            if not chosen_by_table:
                raise
            reduce_note = f"nccl, because {args.reduce} could not be set up: {e}"
            args.reduce = "nccl"
            p.reduce = pkg.REDUCE_NCCL
            out = torch.zeros((p.S, p.d), dtype=torch.float16, device="cuda")
    else:
        out = torch.zeros((p.S, p.d), dtype=torch.float16, device="cuda")

    def barrier():
        torch.cuda.synchronize()
        if world_size > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_step(host_path=False):
        flush.fill_(rank + 1)                   # evict L2 between steps
        barrier()
        if host_path:
            return pkg.run_mode_host(ctx, mode, *host, host_out, p, out_row0=rank * share, out_rows=share)
        return pkg.run_mode(ctx, mode, weights, out, p)

    pkg.kernel_status_reset()
    for _ in range(args.warmup):
        one_step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    stats = [one_step() for _ in range(args.steps)]
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    status = pkg.kernel_status()
    if status[0] != 0:
        raise SystemExit(f"rank {rank}: a kernel reported status {status}")
    wall = [s.wall_ms for s in stats]           # each already the max over ranks
    ms = statistics.mean(wall)
    attn_ms = statistics.mean([s.attn_kernel_ms for s in stats])
    launches = stats[-1].kernel_launches

    def timed(m, output, steps):
        """Mean block time of mode m over `steps` steps after two untimed ones."""
        ts = []
        for i in range(2 + steps):
            flush.fill_(1)
            barrier()
            st = pkg.run_mode(ctx, m, weights, output, p)
            if i >= 2:
                ts.append(st.wall_ms)
        return statistics.mean(ts)

    # other modes, for context (fewer steps)
    few = min(args.steps, 5)
    modes = {args.mode: ms}
    for other in ("attn", "megatron", "stream"):
        if other != args.mode:
            modes[other] = timed(pkg.parse_mode(other), out, few)
    # the same modes with the reference's types (fp32 partial sums, fp32 reduction, fp32 output): the like-for-like
    # precision figure beside the reference arm
    modes_f32 = {}
    out32 = torch.zeros((p.S, p.d), dtype=torch.float32, device="cuda")
    saved_reduce = p.reduce
    p.proj_f32, p.reduce = 1, pkg.REDUCE_NCCL
    for other in ("megatron", "stream"):
        modes_f32[other] = timed(pkg.parse_mode(other), out32, few)
    p.proj_f32, p.reduce = 0, saved_reduce
    del out32
    # exposed communication: (T - T(--no_comm)) / T with the reference's diagnostic flag
    exposed = None
    if world_size > 1:
        p.skip_comm = 1
        t_nc = timed(mode, out, few)
        p.skip_comm = 0
        exposed = max(0.0, (ms - t_nc) / ms)

    # end to end through the host-buffer entry point
    for _ in range(2):
        one_step(host_path=True)
    e2e_ms = statistics.mean([one_step(host_path=True).wall_ms for _ in range(max(3, min(args.steps, 10)))])
    h2d = sum(h.numel() * 2 for h in host) * world_size      # every rank copies its own Q, K, V and W_O slice in
    d2h = p.S * p.d * 2                                       # the result once, S / N rows per rank

    pk = measured_peaks()
    fl = attention_flops(p.S, p.d_h, p.H_local, p.causal)
    achieved = fl / (attn_ms * 1e-3) / 1e12 if attn_ms > 0 else 0.0
    proj_fl = 2.0 * p.S * p.d_local * p.d
    link_bytes = 2.0 * (world_size - 1) / world_size * p.S * p.d * 2
    t_roof = max((fl + proj_fl) / (pk["tflops"] * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3

    line = None
    if rank == 0:
        cpu = None
        if args.cpu_rows > 0 and world_size == 1:      # the CPU baseline is reported at N=1 only
            oracle = entry.load_oracle()
            cpu = cpu_baseline(pkg, oracle, p, [h.numpy().view(np.uint16) for h in host], args.cpu_rows)
        line = dict(
            metric=METRIC, value=ms, unit="ms", n_gpus=world_size, steps=args.steps, warmup=args.warmup,
            ms_per_step=ms, higher_is_better=False, scaling="strong", vs_baseline=None, dtype="f16 (f32 accumulate)",
            data="synthetic",
            config=dict(workload=f"S={p.S} H={p.H} d_h={p.d_h} causal tile={p.tile} ncomm={W['ncomm']} TP={world_size}",
                        mode=args.mode, split=p.split, reduce=(reduce_note or args.reduce), reduce_ctas=(args.reduce_ctas or "default"), reserve_sms=args.reserve_sms, numa_node=numa_node, wire=args.wire, row_order=args.order,
                        group_tiles=args.group_tiles or "auto (S/8 rows per launch)",
                        l2="256 MB buffer written between steps",
                        e2e="pinned host Q/K/V/W_O copied in by every rank, the fp16 [S][d] result (identical on all ranks) copied "
                            "out once, S/N rows by each rank; copy-in, compute and copy-out pipelined over row chunks; bytes "
                            "are totals over the ranks",
                        inputs="Q,K,V ~ N(0,1) fp16 [H_local][S][d_h]; W_O ~ N(0,1/d) fp16; seed 42"),
            tokens_per_s=p.S / (ms * 1e-3),
            modes_ms=modes, modes_ms_proj_f32=modes_f32, exposed_comm_frac=exposed,
            block_roofline=dict(t_ms=t_roof, frac=t_roof / ms,
                                peak=f"{pk['tflops']} TFLOP/s bf16 {pk['source']}; {NVLINK_GBS:.0f} GB/s per direction NVLink nominal"),
            roofline=dict(bound="tensor", kernel="fa_fwd_ws_kernel<128>", achieved=achieved, peak=pk["tflops"], unit="TFLOP/s",
                          frac=achieved / pk["tflops"], peak_source=f"of {pk['source']} (burst bf16)",
                          frac_sustained=achieved / pk["tflops_sustained"], attn_kernel_ms=attn_ms,
                          algorithmic_flops=fl,
                          # dram__bytes_read.sum + dram__bytes_write.sum of this kernel's launch, from one ncu capture of
                          # the benchmark shape on one rank (32 heads); heads are independent, so a rank's traffic is
                          # that figure times H_local / 32. Shapes that were not captured report null.
                          traffic=(ATTN_TRAFFIC_32_HEADS.get((args.mode, descending)) * p.H_local / 32
                                   if (p.S == 32768 and p.d_h == 128 and p.causal and p.split == 1
                                       and (args.mode, descending) in ATTN_TRAFFIC_32_HEADS) else None),
                          algorithmic_bytes=2.0 * p.S * p.d_local * 4),      # Q, K, V read once, O written once (fp16)
            cpu_baseline=cpu,
            e2e=dict(value=e2e_ms, unit="ms", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h),
            gpu_launches=launches * args.steps,
            clocks=clocks,
        )
    pkg.destroy_ctx(ctx)
    if world_size > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        emit(line)
    return 0


_RESULT_FD = 1


def emit(line):
    """The one JSON line, on the process's original standard output."""
    os.write(_RESULT_FD, (json.dumps(line) + "\n").encode())


if __name__ == "__main__":
    # Libraries print to standard output too (NCCL announces its version there): everything but the result line goes to
    # standard error, so that standard output carries exactly one line.
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    sys.exit(main())
