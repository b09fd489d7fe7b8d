#!/usr/bin/env python
"""Latency/bandwidth model of the per-tile AllReduce and the schedule times it predicts.

Same model as cost_model.py:10-16,62-98 of eager-flash-attention: from the `comm` rows
(num_tiles AllReduces of tile*d elements back to back) fit t_ar(bytes) = alpha + bytes / beta by least
squares; then

    T_megatron = T_attn + T_proj + t_ar(S*d*e)
    T_stream   = max(T_attn, n * t_ar(tile*d*e) / ncomm) + t_proj_tile + t_ar(tile*d*e)

with e the payload element size (2 for this build, 4 for the reference).
"""
import csv
import sys


def read_rows(path):
    with open(path) as f:
        rows = [r for r in csv.DictReader(f) if r.get("mode")]
    for r in rows:
        for k in ("S", "H", "d_h", "R", "tile", "split", "ncomm"):
            r[k] = int(r[k])
        r["causal"] = int(r.get("causal") or 0)
        r["median_ms"] = float(r["median_ms"])
    return rows


def fit_allreduce(rows, elem_bytes=2):
    """(alpha_ms, beta_bytes_per_ms) from comm-mode rows; needs at least two tile sizes."""
    pts = []
    for r in rows:
        if r["mode"] != "comm":
            continue
        n = r["S"] // r["tile"]
        pts.append((r["tile"] * r["H"] * r["d_h"] * elem_bytes, r["median_ms"] / n))
    if len(pts) < 2:
        raise ValueError("need comm rows at two or more tile sizes")
    n = len(pts)
    sx = sum(b for b, _ in pts); sy = sum(t for _, t in pts)
    sxx = sum(b * b for b, _ in pts); sxy = sum(b * t for b, t in pts)
    slope = (n * sxy - sx * sy) / (n * sxx - sx * sx)
    alpha = (sy - slope * sx) / n
    return alpha, (1.0 / slope if slope > 0 else float("inf"))


def t_ar(nbytes, alpha, beta):
    return alpha + nbytes / beta


def predict(S, d, tile, ncomm, t_attn, t_proj, alpha, beta, elem_bytes=2):
    n = S // tile
    ar_tile = t_ar(tile * d * elem_bytes, alpha, beta)
    megatron = t_attn + t_proj + t_ar(S * d * elem_bytes, alpha, beta)
    stream = max(t_attn, n * ar_tile / max(1, ncomm)) + t_proj / n + ar_tile
    return megatron, stream


def main(argv=None):
    argv = argv or sys.argv[1:]
    if not argv:
        print("usage: cost_model.py results.csv [elem_bytes]", file=sys.stderr)
        return 2
    e = int(argv[1]) if len(argv) > 1 else 2
    rows = read_rows(argv[0])
    alpha, beta = fit_allreduce(rows, e)
    print(f"t_ar(bytes) = {alpha * 1e3:.1f} us + bytes / {beta / 1e6:.1f} GB/s")
    by = {}
    for r in rows:
        by.setdefault((r["S"], r["H"], r["d_h"], r["causal"], r["tile"], r["ncomm"]), {})[r["mode"]] = r["median_ms"]
    print("| S | causal | tile | ncomm | megatron meas / pred | stream meas / pred |")
    print("|---|---|---|---|---|---|")
    for (S, H, dh, causal, tile, ncomm), m in sorted(by.items()):
        if not {"attn", "megatron", "stream"} <= set(m):
            continue
        t_proj = 0.0
        meg, st = predict(S, H * dh, tile, ncomm, m["attn"], t_proj, alpha, beta, e)
        print(f"| {S} | {causal} | {tile} | {ncomm} | {m['megatron']:.3f} / {meg:.3f} | {m['stream']:.3f} / {st:.3f} |")
    return 0


if __name__ == "__main__":
    sys.exit(main())
