"""tcgen05 GEMM against fp32 matmul of the same bf16 operands; Newton-Schulz against the fp32 reference iteration."""
import pytest
import torch

from supergrok15_b200.ops import gemm, oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (256, 128, 512), (130, 70, 72), (1000, 520, 264), (64, 40, 8),
                                   (4096, 512, 512), (300, 1000, 2048), (512, 520, 32768), (136, 72, 8200)])
def test_gemm_tn_matches_fp32_matmul(M, N, K):
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    out = gemm.gemm_tn(a, b, out_dtype=torch.float32)
    gemm.check()
    assert torch.allclose(out, ref, rtol=1e-3, atol=1e-2 * (K ** 0.5) * 1e-1), (out - ref).abs().max()
    outb = gemm.gemm_tn(a, b)
    assert torch.allclose(outb.float(), ref, rtol=2e-2, atol=0.5)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 192), (200, 136, 72), (520, 264, 384), (72, 1000, 2056), (264, 520, 16384)])
@pytest.mark.parametrize("a_t", [False, True])
def test_gemm_transposed_operands_read_in_place(M, N, K, a_t):
    """b (and a) stored [K, N] ([K, M]) are consumed through MN-major descriptors: same result as the K-major call."""
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    out = gemm.gemm_tn(a.t().contiguous() if a_t else a, b.t().contiguous(), out_dtype=torch.float32, a_t=a_t, b_t=True)
    gemm.check()
    assert out.shape == ref.shape
    assert torch.allclose(out, ref, rtol=1e-3, atol=1e-3 * (K ** 0.5)), (out - ref).abs().max()


def test_gemm_epilogue_and_transposed_output():
    torch.manual_seed(0)
    M, N, K = 200, 200, 136
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    d = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    out_t = torch.empty(N, M, device="cuda", dtype=torch.float32)
    out = gemm.gemm_tn(a, b, alpha=0.5, beta=-2.0, d=d, bias=bias, diag=3.0, out_dtype=torch.float32, out_t=out_t)
    gemm.check()
    ref = 0.5 * (a.float() @ b.float().t()) - 2.0 * d.float() + bias.float() + 3.0 * torch.eye(M, device="cuda")
    assert torch.allclose(out, ref, rtol=1e-3, atol=2e-2)
    assert torch.equal(out_t, out.t())
    g = gemm.gemm_tn(a, b, act="gelu", out_dtype=torch.float32)
    assert torch.allclose(g, torch.nn.functional.gelu(a.float() @ b.float().t()), rtol=1e-3, atol=2e-2)


def test_linear_autograd_matches_torch():
    torch.manual_seed(1)
    x = torch.randn(96, 4, 264, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(520, 264, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(520, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = gemm.linear(x, w, b)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    g = torch.randn_like(yr)
    (y.float() * g).sum().backward()
    (yr * g).sum().backward()
    gemm.check()
    assert torch.allclose(y.float(), yr, rtol=2e-2, atol=5e-2)
    assert torch.allclose(x.grad.float(), xr.grad, rtol=3e-2, atol=5e-2)
    assert torch.allclose(w.grad.float(), wr.grad, rtol=3e-2, atol=0.3)
    assert torch.allclose(b.grad.float(), br.grad, rtol=3e-2, atol=0.3)


@pytest.mark.parametrize("shape", [(256, 128), (128, 256), (200, 136)])
def test_newton_schulz_split_precision_tracks_the_fp32_iteration(shape):
    """precision="bf16x3": three bf16 products per GEMM on hi / lo splits; an order of magnitude closer to fp32 than plain bf16."""
    torch.manual_seed(3)
    X = torch.randn(shape, device="cuda")
    X = X / (X.norm() + 1e-7)
    ref = oracle.newton_schulz(X.double(), 5).float()
    out3 = gemm.newton_schulz(X, 5, oracle.NS_COEFFS, precision="bf16x3")
    out1 = gemm.newton_schulz(X, 5, oracle.NS_COEFFS, precision="bf16")
    gemm.check()
    e3, e1 = (out3 - ref).norm() / ref.norm(), (out1 - ref).norm() / ref.norm()
    assert e3 < 2e-3 and e3 < 0.2 * e1, (float(e3), float(e1))
    with pytest.raises(ValueError):
        gemm.newton_schulz(X, 5, oracle.NS_COEFFS, precision="fp64")


@pytest.mark.parametrize("shape", [(256, 128), (128, 256), (512, 512), (264, 136), (203, 136), (136, 203)])
def test_newton_schulz_matches_fp32_iteration(shape):
    torch.manual_seed(2)
    X = torch.randn(shape, device="cuda")
    X = X / (X.norm() + 1e-7)
    ref = oracle.newton_schulz(X.double(), 5).float()
    out = gemm.newton_schulz(X, 5, oracle.NS_COEFFS)
    gemm.check()
    # bf16 operands: compare in the metric that matters for Muon (relative Frobenius error and orthogonality)
    rel = (out - ref).norm() / ref.norm()
    assert rel < 0.06, rel
    k = min(shape)
    Q = out @ out.t() if shape[0] <= shape[1] else out.t() @ out
    Qr = ref @ ref.t() if shape[0] <= shape[1] else ref.t() @ ref
    assert (Q - Qr).norm() / k ** 0.5 < 0.1
