#!/usr/bin/env python
"""CSV rows of attn_bench (this build's or the reference's) -> markdown tables.

    python bench_tables.py ours.csv [reference.csv]

Counterpart of bench_tables.py:33-142 of eager-flash-attention: a headline table (megatron vs stream
per shape, speed-up), and when a second file is given a side-by-side table with the ratio.
"""
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


def main(argv=None):
    argv = argv or sys.argv[1:]
    if not argv:
        print("usage: bench_tables.py ours.csv [reference.csv]", file=sys.stderr)
        return 2
    ours = read_rows(argv[0])
    print(headline(ours))
    if len(argv) > 1:
        print()
        print(side_by_side(ours, read_rows(argv[1])))
    return 0


if __name__ == "__main__":
    sys.exit(main())
