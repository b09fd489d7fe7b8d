"""Which reduction, wire type, row order and grid to use for a rank count: one context, many settings.

attn_bench (like the reference's) measures one setting per process, and on eight ranks most of a process's life is
start-up (CUDA contexts, communicators). This sweep makes one context and times every setting on it, so that the
table behind the defaults costs seconds. Launch with torchrun, one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \\
        eager-flash-attention_b200/sweep/reduce_sweep.py --out reduce_sweep_R8.csv

Rows: mode, reduce, wire, order, reduce_ctas, reserve_sms, mean / min ms of `--trials` steps (each the max over ranks, L2 flushed
between steps), mean attention-kernel ms. Inputs N(0,1), seed 42, as the benchmark plan's configurations.
"""
import argparse
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

DEFAULT_SETTINGS = [
    # mode, reduce, wire, order, reduce_ctas
    ("attn", "nccl", "auto", "auto", 0),
    ("stream", "none", "auto", "asc", 0),
    ("megatron", "nccl", "f32", "auto", 0), ("stream", "nccl", "f32", "asc", 0),
    ("megatron", "nccl", "f16", "auto", 0), ("stream", "nccl", "f16", "asc", 0),
    ("megatron", "nvls", "f32", "auto", 32), ("stream", "nvls", "f32", "asc", 32),
    ("stream", "nvls", "f32", "asc", 48),
    ("stream", "nvls", "f16", "asc", 32),
    ("megatron", "pull", "f32", "auto", 12), ("stream", "pull", "f32", "asc", 12),
    ("megatron", "pull", "f32", "auto", 16), ("stream", "pull", "f32", "asc", 16),
    ("stream", "pull", "f32", "asc", 8), ("stream", "pull", "f32", "asc", 24),
    ("stream", "pull", "f32", "mixed", 16), ("stream", "pull", "f32", "desc", 16),
    ("stream", "p2p", "auto", "asc", 0),
]


MODES = ("attn", "megatron", "sync", "overlap", "stream")
REDUCES = ("none", "nccl", "p2p", "nvls", "pull")
WIRES = ("auto", "f16", "f32")
ORDERS = ("auto", "asc", "desc", "mixed")


def parse_setting(text, traced=False):
    """'mode,reduce,wire,order,reduce_ctas[,reserve_sms]' -> (mode, reduce, wire, order, ctas, reserve, traced)."""
    f = [x.strip() for x in text.split(",")]
    if len(f) not in (5, 6):
        raise ValueError(f"setting {text!r}: five or six comma-separated fields expected")
    if f[0] not in MODES or f[1] not in REDUCES or f[2] not in WIRES or f[3] not in ORDERS:
        raise ValueError(f"setting {text!r}: unknown mode, reduction, wire type or row order")
    return (f[0], f[1], f[2], f[3], int(f[4]), int(f[5]) if len(f) == 6 else 0, traced)


def plan(settings_text="", only="", trace_text=""):
    """The settings to time, in order: the built-in list (optionally only some reductions) or the given ones, then the
    traced one."""
    keep = set(x for x in only.split(",") if x)
    if settings_text:
        out = [parse_setting(t) for t in settings_text.split(";") if t.strip()]
    else:
        out = [s + (0, False) for s in DEFAULT_SETTINGS if not keep or s[1] in keep]
    if trace_text:
        out.append(parse_setting(trace_text, True))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--S", type=int, default=32768)
    ap.add_argument("--H", type=int, default=32)
    ap.add_argument("--d_h", type=int, default=128)
    ap.add_argument("--tile", type=int, default=128)
    ap.add_argument("--causal", type=int, default=1)
    ap.add_argument("--ncomm", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--trials", type=int, default=5)
    ap.add_argument("--only", default="", help="comma-separated reduce kinds to keep (default: all)")
    ap.add_argument("--out", default="")
    ap.add_argument("--settings", default="", help="instead of the built-in list: 'mode,reduce,wire,order,reduce_ctas[,reserve_sms]' "
                                                   "entries separated by ';'")
    ap.add_argument("--trace", default="", help="one more setting, same form, whose last step prints the per-group timeline "
                                                "of every rank (stderr)")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    pkg = entry.load_package()
    pkg.lib()
    rank, world_size, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world_size > 1:
        dist.init_process_group(backend="cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local))
        world = pkg.World.from_torch(None, local_device=local)
    else:
        world = pkg.World(0, 1, local)
    d = args.H * args.d_h
    p = pkg.make_params(args.S, d, args.H, args.tile, 2, 1, args.causal, world_size)
    why = pkg.attn_check_params(p)
    if why:
        raise SystemExit(why)
    host = [torch.empty((p.H_local, p.S, p.d_h), dtype=torch.float16) for _ in range(3)]
    host.append(torch.empty((p.d_local, p.d), dtype=torch.float16))
    pkg.fill_host_inputs(p, rank, 42, pkg.RECIPE_NORMAL, *host)
    dev = [h.cuda() for h in host]
    weights = pkg.Weights(*(t.data_ptr() for t in dev))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    own_out = torch.zeros((p.S, p.d), dtype=torch.float16, device="cuda")
    ctx = pkg.make_ctx(world, ncomm=args.ncomm)
    pkg.set_wait_limit_ms(ctx, 5000.0, 30000.0)

    class _Region:
        def __init__(self, ptr, shape):
            self.__cuda_array_interface__ = dict(shape=shape, typestr="<f2", data=(ptr, False), version=2)

    rows = ["mode,reduce,wire,order,reduce_ctas,reserve_sms,ranks,mean_ms,min_ms,attn_kernel_ms,status"]
    settings = plan(args.settings, args.only, args.trace)
    for mode_s, reduce, wire, order, ctas, reserve, traced in settings:
        if world_size == 1 and reduce not in ("nccl", "none"):
            continue
        p.skip_comm = 1 if reduce == "none" else 0
        p.reduce = dict(none=pkg.REDUCE_NCCL, nccl=pkg.REDUCE_NCCL, p2p=pkg.REDUCE_P2P, nvls=pkg.REDUCE_NVLS, pull=pkg.REDUCE_PULL)[reduce]
        p.wire = dict(auto=pkg.WIRE_AUTO, f16=pkg.WIRE_F16, f32=pkg.WIRE_F32)[wire]
        p.row_order = dict(auto=pkg.ROWS_AUTO, asc=pkg.ROWS_ASCENDING, desc=pkg.ROWS_DESCENDING, mixed=pkg.ROWS_MIXED)[order]
        p.reduce_ctas = ctas
        p.reserve_sms = reserve
        mode = pkg.parse_mode(mode_s)
        status = "ok"
        ts, ks = [], []
        try:
            out = own_out
            if reduce in ("nvls", "pull") and world_size > 1:
                out = torch.as_tensor(_Region(pkg.nvls_output(ctx, p), (p.S, p.d)), device="cuda")
            pkg.kernel_status_reset()
            for i in range(args.warmup + args.trials):
                flush.fill_(1)
                torch.cuda.synchronize()
                if world_size > 1:
                    dist.barrier()
                p.trace = 1 if traced and i == args.warmup + args.trials - 1 else 0
                st = pkg.run_mode(ctx, mode, weights, out, p)
                if i >= args.warmup:
                    ts.append(st.wall_ms)
                    ks.append(st.attn_kernel_ms)
            torch.cuda.synchronize()
            if pkg.kernel_status()[0] != 0:
                status = f"kernel status {pkg.kernel_status()}"
        except Exception as e:                  # reported in the table; the other settings still run
            status = "error: " + str(e).replace(",", ";")[:120]
        bad = torch.tensor([0 if status == "ok" else 1])
        if world_size > 1:
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad[0]) and status == "ok":
            status = "failed on another rank"
        rows.append(f"{mode_s},{reduce},{wire},{order},{ctas},{reserve},{world_size},"
                    f"{statistics.mean(ts) if ts else float('nan'):.4f},{min(ts) if ts else float('nan'):.4f},"
                    f"{statistics.mean(ks) if ks else float('nan'):.4f},{status}")
        if rank == 0:
            print(rows[-1], flush=True)
        if int(bad[0]):
            break                               # a failed collective setting may have left the ranks out of step
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            f.write("\n".join(rows) + "\n")
    pkg.destroy_ctx(ctx)
    if world_size > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
