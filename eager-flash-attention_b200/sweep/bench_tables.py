#!/usr/bin/env python
"""CSV rows of attn_bench (this build's or the reference's) -> markdown tables.

    python bench_tables.py ours.csv [reference.csv]
    python bench_tables.py --reduce-sweep reduce_sweep.csv

Counterpart of bench_tables.py:33-142 of eager-flash-attention: a headline table (megatron vs stream
per shape, speed-up), and when a second file is given a side-by-side table with the ratio. The second form
turns the rows of reduce_sweep.py (one context, many reduction settings) into a table per rank count with the
exposed communication of every stream setting against the run without a reduction.
"""
import csv
import sys

from cost_model import read_rows


def key(r):
    return (r["S"], r["H"], r["d_h"], r["causal"], r["R"], r["tile"], r["ncomm"])


def pivot(rows):
    out = {}
    for r in rows:
        out.setdefault(key(r), {})[r["mode"] + (":" + r["reduce"] if r.get("reduce") not in (None, "", "nccl") else "")] = r["median_ms"]
    return out


def headline(rows):
    lines = ["| S | H | d_h | causal | R | tile | ncomm | attn | megatron | stream | megatron/stream |",
             "|---|---|---|---|---|---|---|---|---|---|---|"]
    for k, m in sorted(pivot(rows).items()):
        if "megatron" in m and "stream" in m:
            lines.append("| " + " | ".join(str(x) for x in k) +
                         f" | {m.get('attn', float('nan')):.3f} | {m['megatron']:.3f} | {m['stream']:.3f} | {m['megatron'] / m['stream']:.2f}x |")
    return "\n".join(lines)


def side_by_side(ours, ref):
    po, pr = pivot(ours), pivot(ref)
    lines = ["| S | H | d_h | causal | R | tile | ncomm | mode | reference ms | this build ms | speed-up |",
             "|---|---|---|---|---|---|---|---|---|---|---|"]
    for k in sorted(set(po) & set(pr)):
        for mode in ("attn", "megatron", "stream"):
            if mode in po[k] and mode in pr[k]:
                lines.append("| " + " | ".join(str(x) for x in k) +
                             f" | {mode} | {pr[k][mode]:.3f} | {po[k][mode]:.3f} | {pr[k][mode] / po[k][mode]:.2f}x |")
    return "\n".join(lines)


def reduce_sweep_table(path):
    with open(path) as f:
        rows = [r for r in csv.DictReader(f) if r.get("mode") and r.get("status") == "ok"]
    lines = []
    for ranks in sorted({int(r["ranks"]) for r in rows}):
        mine = [r for r in rows if int(r["ranks"]) == ranks]
        bare = [float(r["mean_ms"]) for r in mine if r["mode"] == "stream" and r["reduce"] == "none"]
        attn = [float(r["mean_ms"]) for r in mine if r["mode"] == "attn"]
        lines += [f"N = {ranks}: attention only {attn[0]:.3f} ms, stream without a reduction {bare[0]:.3f} ms"
                  if attn and bare else f"N = {ranks}", "",
                  "| mode | reduce | wire | rows | reduce_ctas | reserved SMs | mean ms | min ms | attention kernel ms | exposed comm |",
                  "|---|---|---|---|---|---|---|---|---|---|"]
        for r in mine:
            if r["mode"] == "attn" or r["reduce"] == "none":
                continue
            t = float(r["mean_ms"])
            exposed = f"{100.0 * (t - bare[0]) / t:.0f} %" if bare and r["mode"] == "stream" else ""
            lines.append(f"| {r['mode']} | {r['reduce']} | {r['wire']} | {r['order']} | {r['reduce_ctas']} | {r.get('reserve_sms', '0') or '0'} | "
                         f"{t:.3f} | {float(r['min_ms']):.3f} | {float(r['attn_kernel_ms']):.3f} | {exposed} |")
        lines.append("")
    return "\n".join(lines)


def main(argv=None):
    argv = argv or sys.argv[1:]
    if len(argv) == 2 and argv[0] == "--reduce-sweep":
        print(reduce_sweep_table(argv[1]))
        return 0
    if not argv:
        print("usage: bench_tables.py ours.csv [reference.csv] | --reduce-sweep reduce_sweep.csv", file=sys.stderr)
        return 2
    ours = read_rows(argv[0])
    print(headline(ours))
    if len(argv) > 1:
        print()
        print(side_by_side(ours, read_rows(argv[1])))
    return 0


if __name__ == "__main__":
    sys.exit(main())
