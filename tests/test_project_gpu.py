"""The projection kernel behind project() (attn_main.cu:262-273, fp16 data path) against float64 numpy."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,d_local,d", [(64, 16, 64), (128, 64, 64), (128, 128, 1024), (64, 512, 1024),
                                             (256, 1024, 1024), (192, 32, 256), (2048, 512, 512), (4096, 256, 4096),
                                             (128, 4096, 4096), (19072, 128, 1024)])
def test_projection_matches_float64(pkg, torch_cuda, rows, d_local, d):
    torch = torch_cuda
    g = torch.Generator(device="cuda").manual_seed(rows + d_local + d)
    A = torch.randn(rows, d_local, generator=g, device="cuda").to(torch.float16)
    W = (torch.randn(d_local, d, generator=g, device="cuda") / d ** 0.5).to(torch.float16)
    out = torch.full((rows, d), float("nan"), dtype=torch.float16, device="cuda")
    pkg.kernel_status_reset()
    pkg.project(A, W, out, rows, d_local, d)
    torch.cuda.synchronize()
    assert pkg.kernel_status()[0] == 0
    ref = A.double() @ W.double()
    err = (out.double() - ref).abs()
    # one fp16 rounding of the result (2^-11 relative) plus fp32 accumulation noise
    bound = ref.abs() * 2 ** -10 + 1e-4 * ref.abs().max()
    assert torch.isfinite(out).all()
    assert bool((err <= bound).all()), float((err - bound).max())


def test_projection_rejects_bad_shapes(pkg, torch_cuda):
    torch = torch_cuda
    A = torch.zeros(128, 64, dtype=torch.float16, device="cuda")
    W = torch.zeros(64, 64, dtype=torch.float16, device="cuda")
    out = torch.zeros(128, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(pkg.EfaError):
        pkg.project(A, W, out, 100, 64, 64)
    with pytest.raises(pkg.EfaError):
        pkg.project(A, W, out, 128, 24, 64)
    with pytest.raises(pkg.EfaError):
        pkg.project(A, W, out, 128, 64, 96)


@pytest.mark.parametrize("S,d,H_local,d_h", [(512, 512, 4, 128), (1024, 1024, 2, 64), (2048, 256, 4, 64)])
def test_compute_qkv_matches_float64(pkg, torch_cuda, S, d, H_local, d_h):
    """The step before the block (compute_qkv, attn_main.cu:127-153) on fp16 data, head-major output."""
    torch = torch_cuda
    g = torch.Generator(device="cuda").manual_seed(S + d)
    X = (torch.rand(S, d, generator=g, device="cuda") * 2 - 1).to(torch.float16)
    W = [((torch.rand(H_local, d, d_h, generator=g, device="cuda") * 2 - 1) * 0.15).to(torch.float16) for _ in range(3)]
    out = [torch.full((H_local, S, d_h), float("nan"), dtype=torch.float16, device="cuda") for _ in range(3)]
    pkg.compute_qkv(X, W[0], W[1], W[2], out[0], out[1], out[2], S, d, H_local, d_h)
    torch.cuda.synchronize()
    for t in range(3):
        ref = torch.einsum("sk,hkj->hsj", X.double(), W[t].double())
        err = (out[t].double() - ref).abs()
        assert torch.isfinite(out[t]).all()
        assert bool((err <= ref.abs() * 2 ** -10 + 1e-4 * ref.abs().max()).all())
    with pytest.raises(pkg.EfaError, match="d_h"):
        pkg.compute_qkv(X, W[0], W[1], W[2], out[0], out[1], out[2], S, d, H_local, 32)
