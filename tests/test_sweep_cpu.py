"""The sweep / table / cost-model tooling on synthetic CSV rows (no GPU)."""
import os
import subprocess
import sys

from conftest import ROOT

SWEEP = os.path.join(ROOT, "eager-flash-attention_b200", "sweep")
HEADER = "S,H,d_h,causal,R,kernel,tile,nbuf,split,ncomm,proj,mode,min_ms,max_ms,mean_ms,median_ms,std_ms,tokens_per_s,attn_kernel_ms,reduce,data"


def write_csv(path, rows, header=HEADER):
    with open(path, "w") as f:
        f.write(header + "\n")
        for r in rows:
            f.write(",".join(str(x) for x in r) + "\n")


def test_cost_model_recovers_alpha_and_beta(tmp_path):
    sys.path.insert(0, SWEEP)
    import cost_model
    alpha, beta = 0.02, 5e8            # 20 us, 500 GB/s expressed in bytes per ms
    rows = []
    for tile in (128, 512, 2048, 8192):
        n = 16384 // tile
        t = n * (alpha + tile * 1024 * 2 / beta)
        rows.append((16384, 16, 64, 0, 8, "tc", tile, 2, 1, 1, "fp16", "comm", t, t, t, t, 0, 0, 0, "nccl", "normal"))
    p = tmp_path / "comm.csv"
    write_csv(p, rows)
    a, b = cost_model.fit_allreduce(cost_model.read_rows(str(p)), 2)
    assert abs(a - alpha) < 1e-9 and abs(b - beta) / beta < 1e-9
    meg, st = cost_model.predict(16384, 1024, 1024, 4, 1.0, 0.1, a, b, 2)
    assert abs(meg - (1.0 + 0.1 + alpha + 16384 * 1024 * 2 / beta)) < 1e-9
    assert st >= 1.0


def test_tables_accept_reference_rows_without_the_new_columns(tmp_path):
    ours = tmp_path / "ours.csv"
    ref = tmp_path / "ref.csv"
    base = (16384, 16, 64, 0, 8, "tc", 128, 2, 1, 4, "fp16")
    write_csv(ours, [base + ("attn", 1, 1, 1, 0.25, 0, 0, 0, "nccl", "normal"),
                     base + ("megatron", 1, 1, 1, 0.45, 0, 0, 0, "nccl", "normal"),
                     base + ("stream", 1, 1, 1, 0.40, 0, 0, 0, "nccl", "normal")])
    ref_header = ",".join(HEADER.split(",")[:17])
    write_csv(ref, [base[:10] + ("fp32", "megatron", 1, 1, 1, 1.05, 0), base[:10] + ("fp32", "stream", 1, 1, 1, 2.4, 0)], ref_header)
    r = subprocess.run([sys.executable, os.path.join(SWEEP, "bench_tables.py"), str(ours), str(ref)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert "1.12x" in r.stdout           # megatron / stream = 0.45 / 0.40
    assert "| stream | 2.400 | 0.400 | 6.00x |" in r.stdout


def test_sweep_dry_run_lists_the_reference_suites():
    r = subprocess.run([sys.executable, os.path.join(SWEEP, "bench_sweep.py"), "--ranks", "8",
                        "--suite", "core,causal,kernel,modes,scaling,model,comm,tiles", "--dry-run"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if "attn_bench" in l]
    assert len(lines) > 40
    assert all("efa_launch -n 8" in l for l in lines)
    assert any("--modes comm" in l for l in lines) and any("--causal" in l for l in lines)


def test_overlap_suite_names_its_environment():
    r = subprocess.run([sys.executable, os.path.join(SWEEP, "bench_sweep.py"), "--ranks", "8", "--suite", "overlap", "--dry-run"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if "attn_bench" in l]
    assert any("--trace" in l for l in lines)
    assert any(l.startswith("NCCL_MAX_CTAS=8 ") and "--reserve_sms 16" in l for l in lines)
    assert any("--no_comm" in l for l in lines) and any("--split 4" in l for l in lines) and any("--reduce p2p" in l for l in lines)
    assert any("--reduce nvls" in l for l in lines) and any("--order desc" in l for l in lines)


def test_reduce_sweep_settings():
    """reduce_sweep.py: the built-in list, a filter by reduction, explicit settings with and without reserved SMs, the
    traced setting last; malformed settings are refused before any GPU work."""
    import pytest
    sys.path.insert(0, SWEEP)
    import reduce_sweep
    builtin = reduce_sweep.plan()
    assert len(builtin) == len(reduce_sweep.DEFAULT_SETTINGS) and all(len(s) == 7 and s[5] == 0 and not s[6] for s in builtin)
    assert {s[1] for s in builtin} == {"none", "nccl", "nvls", "pull", "p2p"}
    assert {s[1] for s in reduce_sweep.plan(only="pull,nccl")} == {"pull", "nccl"}
    got = reduce_sweep.plan("stream,pull,f32,asc,12;stream,pull,f32,asc,12,16;", trace_text="stream,nvls,f16,mixed,32")
    assert got == [("stream", "pull", "f32", "asc", 12, 0, False), ("stream", "pull", "f32", "asc", 12, 16, False),
                   ("stream", "nvls", "f16", "mixed", 32, 0, True)]
    for bad in ("stream,pull,f32,asc", "stream,push,f32,asc,4", "stream,pull,f64,asc,4", "stream,pull,f32,up,4"):
        with pytest.raises(ValueError):
            reduce_sweep.parse_setting(bad)


def test_committed_sweep_results_parse():
    """The CSVs under sweep/results are what the tables in the notes quote: they must stay readable by the tools."""
    sys.path.insert(0, SWEEP)
    import cost_model
    res = os.path.join(SWEEP, "results")
    for name, lo, hi in (("comm_R2_pull.csv", 300e6, 600e6), ("comm_R2_nccl.csv", 250e6, 500e6)):
        alpha, beta = cost_model.fit_allreduce(cost_model.read_rows(os.path.join(res, name)), 4)
        assert 0.005 < alpha < 0.1 and lo < beta < hi, (name, alpha, beta)       # ms, bytes per ms
    for name in ("reduce_sweep_R8_builtin_settings.csv", "reduce_sweep_R8_reserved_sms.csv", "reduce_sweep_R2_builtin_settings.csv"):
        lines = open(os.path.join(res, name)).read().strip().splitlines()
        assert lines[0].startswith("mode,reduce,wire,order,reduce_ctas") and len(lines) > 5
        assert all(l.endswith(",ok") for l in lines[1:])


def test_reduce_sweep_table(tmp_path):
    """bench_tables.py --reduce-sweep: one table per rank count, exposed communication against the run without a
    reduction, attention-only and no-reduction rows in the heading only."""
    sys.path.insert(0, SWEEP)
    import bench_tables
    p = tmp_path / "rs.csv"
    p.write_text("mode,reduce,wire,order,reduce_ctas,reserve_sms,ranks,mean_ms,min_ms,attn_kernel_ms,status\n"
                 "attn,nccl,auto,auto,0,0,8,1.0000,0.9900,0.9800,ok\n"
                 "stream,none,auto,asc,0,0,8,1.5000,1.4900,1.4000,ok\n"
                 "stream,pull,f32,asc,12,0,8,2.0000,1.9000,1.4500,ok\n"
                 "megatron,pull,f32,auto,12,0,8,2.5000,2.4000,1.0000,ok\n"
                 "stream,nvls,f32,asc,32,0,8,9.0000,9.0000,9.0000,error: x\n")
    text = bench_tables.reduce_sweep_table(str(p))
    assert "N = 8: attention only 1.000 ms, stream without a reduction 1.500 ms" in text
    assert "| stream | pull | f32 | asc | 12 | 0 | 2.000 | 1.900 | 1.450 | 25 % |" in text
    assert "| megatron | pull | f32 | auto | 12 | 0 | 2.500 | 2.400 | 1.000 |  |" in text
    assert "nvls" not in text                       # failed settings are left out
    # the committed results render
    res = os.path.join(SWEEP, "results")
    assert "| stream | pull | f32 | asc | 12 |" in bench_tables.reduce_sweep_table(os.path.join(res, "reduce_sweep_R8_reserved_sms.csv"))
