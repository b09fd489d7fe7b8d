"""Sweep, table and cost-model tooling around attn_bench (single host, efa_launch instead of srun).

Counterparts of bench_sweep.py, bench_tables.py and cost_model.py of eager-flash-attention; they
read and write the same 17 leading CSV columns, so tables can mix rows from both programs.
"""
