"""The CUDA path against the vectors that the reference's own GPU checker wrote (tests/golden, single-rank cases):
inputs from the reference's recipe rounded to fp16 (the kernels' input type; the checker worked on the fp32 values,
attn_tests.cu:37), every output-writing mode, the same gate as everywhere (max-abs <= 2e-3, relative <= 1e-2).
The vectors of several ranks pin the CPU checker (tests/test_oracle_cpu.py), which the multi-GPU tests compare with."""
import os

import numpy as np
import pytest

from conftest import ROOT
from helpers import assert_close, ref_inputs_f16, to_dev

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(ROOT, "tests", "golden")


def single_rank_cases():
    out = []
    for line in open(os.path.join(GOLDEN, "manifest.txt")):
        f = line.split()
        if not f or f[0].startswith("#") or (len(f) > 7 and int(f[7]) != 1):
            continue
        out.append((f[0], int(f[1]), int(f[2]), int(f[3]), int(f[4]), int(f[5])))
    return out


@pytest.mark.parametrize("case", single_rank_cases(), ids=lambda c: c[0])
def test_modes_match_the_reference_checkers_vectors(pkg, oracle, torch_cuda, case):
    torch = torch_cuda
    name, S, d, H, causal, seed = case
    gold = np.fromfile(os.path.join(GOLDEN, name + ".f32"), np.float32).reshape(S, d)
    bits, _ = ref_inputs_f16(oracle, S, d, H, 1, 0, seed)
    dev = to_dev(torch, bits)
    w = pkg.Weights(*(t.data_ptr() for t in dev))
    ctx = pkg.make_ctx(pkg.World(), ncomm=2)
    try:
        for tile in (64, 128):
            p = pkg.make_params(S, d, H, tile, causal=causal)
            assert pkg.attn_check_params(p) is None
            for mode in ("megatron", "stream"):
                out = torch.full((S, d), float("nan"), dtype=torch.float16, device="cuda")
                pkg.kernel_status_reset()
                pkg.run_mode(ctx, pkg.parse_mode(mode), w, out, p)
                torch.cuda.synchronize()
                assert pkg.kernel_status()[0] == 0
                assert_close(oracle, out.float().cpu().numpy(), gold, f"{name} tile {tile} {mode}")
    finally:
        pkg.destroy_ctx(ctx)
