"""tcgen05 GEMM against a plain fp32 PyTorch matmul of the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().T if a_mn else a.float()
    B = b.float() if b_mn else b.float().T
    return A @ B


SHAPES = [(128, 256, 64), (256, 512, 256), (384, 768, 320), (200, 264, 72), (4096, 1024, 4096), (1000, 136, 520)]


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("bn", [0, 128, 256])
def test_gemm_matches_fp32(M, N, K, a_mn, b_mn, bn):
    from aws_ofi_nccl_b200.ops.gemm import gemm

    torch.manual_seed(M * 7 + N * 3 + K)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    ref = _ref(a, b, a_mn, b_mn)
    err = (out.float() - ref).abs().max().item()
    tol = 2e-2 * ref.abs().max().item() + 1e-2
    assert err <= tol, f"max err {err} > {tol}"


def test_gemm_fp32_out_and_accumulate():
    from aws_ofi_nccl_b200.ops.gemm import gemm

    a = torch.randn(256, 192, device="cuda").bfloat16()
    b = torch.randn(512, 192, device="cuda").bfloat16()
    ref = a.float() @ b.float().T
    out = gemm(a, b, out_dtype=torch.float32)
    assert torch.allclose(out, ref, rtol=1e-4, atol=1e-3)
    gemm(a, b, out=out, accumulate=True)
    assert torch.allclose(out, 2 * ref, rtol=1e-4, atol=2e-3)
    o16 = gemm(a, b)
    gemm(a, b, out=o16, accumulate=True)
    assert torch.allclose(o16.float(), 2 * ref, rtol=2e-2, atol=0.5)


def test_gemm_strided_rows():
    from aws_ofi_nccl_b200.ops.gemm import gemm

    big = torch.randn(300, 512, device="cuda").bfloat16()
    a = big[:, 64:64 + 256]  # row pitch 512, 256 columns
    b = torch.randn(128, 256, device="cuda").bfloat16()
    out = gemm(a, b)
    ref = a.float() @ b.float().T
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


def test_linear_autograd_matches_torch():
    from aws_ofi_nccl_b200.ops.gemm import linear

    x = torch.randn(384, 256, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(512, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    dy = torch.randn(384, 512, device="cuda").bfloat16()
    y = linear(x, w)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = xr @ wr.T
    yr.backward(dy.float())
    for got, ref in ((y, yr), (x.grad, xr.grad), (w.grad, wr.grad)):
        assert (got.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 128, 128), (512, 1024, 4096), (4096, 4096, 4096), (384, 640, 2064), (8192, 14336, 4096)])
def test_fp8_gemm_matches_the_dequantised_product(M, N, K):
    """Same quantised operands on both sides: the kernel's fp32 accumulation of e4m3 products must
    agree with an fp32 matmul of the dequantised matrices up to the bf16 rounding of the output."""
    from aws_ofi_nccl_b200.ops.gemm import gemm_fp8, quantize_rows_fp8

    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * K ** -0.5).bfloat16()
    xq, xs = quantize_rows_fp8(x)
    wq, ws = quantize_rows_fp8(w)
    # the quantiser itself: one scale per row, at most one e4m3 step of error
    x_dq = xq.float() * xs[:, None]
    assert torch.allclose(xs, x.float().abs().amax(1).clamp_min(1e-12) / 448, rtol=1e-6)
    assert ((x_dq - x.float()).abs() <= x.float().abs() * 0.0625 + xs[:, None] * 2 ** -9 + 1e-6).all()
    out = gemm_fp8(xq, wq, xs, ws)
    ref = (xq.float() @ wq.float().t()) * xs[:, None] * ws[None, :]
    err = (out.float() - ref).norm() / ref.norm()
    assert err < 5e-3, err
    # and against the unquantised product, within fp8 accuracy
    full = x.float() @ w.float().t()
    assert (out.float() - full).norm() / full.norm() < 6e-2
