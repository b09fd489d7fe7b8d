#!/usr/bin/env python
"""Run benchmark suites on this host and append the CSV rows to a file.

    python bench_sweep.py --ranks 8 --suite core,causal --out results/b200_r8.csv [--bench PATH] [--dry-run]

Suites follow bench_sweep.py:73-123 of eager-flash-attention (core, kernel, modes, scaling, model,
causal, comm), with srun replaced by efa_launch and the legacy kernel dropped. Tile sizes include the
small tiles of the B200 plan (64/128/256) next to the reference's S/16 and S/8.

The `overlap` suite is a diagnosis of exposed communication at the scaling shape: stream mode with and
without the collectives, over the knobs that decide how projection and AllReduce launches find SMs while
the attention kernel runs (tiles per launch, split-KV item length, reserved SMs, NCCL's CTA budget), plus
one traced run whose per-group timeline goes to stderr. Its runs differ in flags and environment that
the CSV columns do not show, so each CSV row of that suite is preceded by a `# ...` line naming them.
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
HEADER = ("S,H,d_h,causal,R,kernel,tile,nbuf,split,ncomm,proj,mode,min_ms,max_ms,mean_ms,median_ms,std_ms,"
          "tokens_per_s,attn_kernel_ms,reduce,data,wire")


def suite_commands(name, ranks):
    """Lists of attn_bench argument lists for one suite."""
    cmds = []
    if name == "core":          # headline: megatron vs stream, two tile sizes per S
        for S in (16384, 65536):
            for tile in (128, S // 16, S // 8):
                cmds.append(["--S", S, "--tile", tile, "--ncomm", 4, "--modes", "attn,megatron,stream"])
    elif name == "causal":
        for S in (16384, 32768, 65536):
            for tile in (128, S // 16):
                cmds.append(["--S", S, "--tile", tile, "--ncomm", 4, "--causal", "--modes", "attn,megatron,stream"])
    elif name == "kernel":      # attention only over S
        for S in (1024, 4096, 16384, 65536):
            cmds.append(["--S", S, "--tile", min(S, 256), "--modes", "attn"])
    elif name == "modes":       # every mode at one shape
        cmds.append(["--S", 16384, "--tile", 1024, "--ncomm", 4, "--modes", "attn,attn_tiled,megatron,sync,overlap,stream"])
    elif name == "scaling":     # fixed problem; the rank count is the launcher's
        cmds.append(["--S", 32768, "--H", 32, "--d_h", 128, "--causal", "--tile", 128, "--ncomm", 4,
                     "--modes", "attn,megatron,stream"])
    elif name == "model":       # H=32, d_h=128, d=4096
        for tile in (128, 1024):
            cmds.append(["--S", 16384, "--H", 32, "--d_h", 128, "--tile", tile, "--ncomm", 4, "--modes", "attn,megatron,stream"])
    elif name == "comm":        # AllReduce only, for the alpha/beta fit
        for tile in (128, 256, 512, 1024, 2048, 4096, 8192, 16384):
            cmds.append(["--S", 16384, "--tile", tile, "--group_tiles", 1, "--modes", "comm"])
    elif name == "tiles":       # the small-tile sweep of the B200 plan
        for tile in (64, 128, 256):
            for ncomm in (1, 2, 4, 8):
                for causal in ((), ("--causal",)):
                    cmds.append(["--S", 65536, "--tile", tile, "--ncomm", ncomm, *causal, "--modes", "megatron,stream"])
    elif name == "overlap":
        base = ["--S", 32768, "--H", 32, "--d_h", 128, "--causal", "--tile", 128, "--ncomm", 4]
        cmds.append((base + ["--modes", "attn,megatron,stream"], {}))
        cmds.append((base + ["--modes", "stream", "--no_comm"], {}))
        cmds.append((base + ["--modes", "stream", "--trials", 1, "--warmup", 1, "--trace"], {}))
        for gt in (16, 64, 128):
            cmds.append((base + ["--modes", "stream", "--group_tiles", gt], {}))
        for split in (2, 4):
            cmds.append((base + ["--modes", "stream", "--split", split], {}))
        for ctas in (4, 8, 16):
            cmds.append((base + ["--modes", "stream"], {"NCCL_MAX_CTAS": str(ctas)}))
            cmds.append((base + ["--modes", "stream", "--reserve_sms", 2 * ctas], {"NCCL_MAX_CTAS": str(ctas)}))
        for order in ("asc", "desc"):
            cmds.append((base + ["--modes", "stream", "--order", order], {}))
        for reduce in ("p2p", "nvls"):
            cmds.append((base + ["--modes", "stream", "--reduce", reduce], {}))
    else:
        raise ValueError(f"unknown suite {name!r}")
    out = []
    for c in cmds:
        args, env = c if isinstance(c, tuple) else (c, {})
        out.append(([str(x) for x in args], env))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=1)
    ap.add_argument("--suite", default="core")
    ap.add_argument("--out", default="-")
    ap.add_argument("--bench", default=os.path.join(PKG, "bin", "attn_bench"))
    ap.add_argument("--launcher", default=os.path.join(PKG, "bin", "efa_launch"))
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--trials", type=int, default=5)
    ap.add_argument("--extra", default="", help="extra attn_bench flags, e.g. '--reduce p2p'")
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)

    out = sys.stdout if args.out == "-" else open(args.out, "a")
    if args.out == "-" or os.path.getsize(args.out) == 0:
        print(HEADER, file=out, flush=True)
    rc = 0
    for suite in args.suite.split(","):
        for cmd, env in suite_commands(suite.strip(), args.ranks):
            # flags of the suite come last, so a suite may override --warmup / --trials
            full = [args.launcher, "-n", str(args.ranks), args.bench, "--warmup", str(args.warmup),
                    "--trials", str(args.trials), "--no-header", *args.extra.split(), *cmd]
            label = " ".join(f"{k}={v}" for k, v in env.items())
            if args.dry_run:
                print((label + " " if label else "") + " ".join(full))
                continue
            if env:
                print(f"# {label} {' '.join(cmd)}", file=out, flush=True)
            elif suite.strip() == "overlap":
                print(f"# {' '.join(cmd)}", file=out, flush=True)
            r = subprocess.run(full, capture_output=True, text=True, env=dict(os.environ, **env))
            if "--trace" in cmd:
                sys.stderr.write(r.stderr)
            if r.returncode != 0:
                print(f"# FAILED ({r.returncode}): {' '.join(full)}\n# {r.stderr.strip()[-300:]}", file=sys.stderr)
                rc = 1
                continue
            for line in r.stdout.splitlines():
                if line and line[0].isdigit():
                    print(line, file=out, flush=True)
    return rc


if __name__ == "__main__":
    sys.exit(main())
