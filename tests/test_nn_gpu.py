"""GPU tests of the model-side kernels against plain PyTorch fp32."""
import pytest
import torch
import torch.nn.functional as F

from supergrok15_b200.ops import nn_ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,H,hd", [(4, 8, 64), (4, 4, 32), (8, 2, 64), (8, 4, 32)])
def test_attention_small_forward_backward(S, H, hd, dtype):
    torch.manual_seed(0)
    B, D = 37, H * hd
    qkv = torch.randn(B, S, 3 * D, device="cuda", dtype=dtype, requires_grad=True)
    ref_in = qkv.detach().float().requires_grad_(True)
    out = nn_ops.attention_small(qkv, H)
    ref = nn_ops.attention_small_reference(ref_in, H)
    w = torch.randn_like(ref)
    (out.float() * w).sum().backward()
    (ref * w).sum().backward()
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    assert torch.allclose(out.float(), ref, **tol)
    assert torch.allclose(qkv.grad.float(), ref_in.grad, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,D,res,bias", [(1, 128, True, True), (70, 512, True, True), (257, 256, False, True), (64, 512, True, False)])
def test_layer_norm_residual_forward_backward(rows, D, res, bias, dtype):
    torch.manual_seed(1)
    x = torch.randn(rows, D, device="cuda", dtype=dtype, requires_grad=True)
    r = torch.randn(rows, D, device="cuda", dtype=dtype, requires_grad=True) if res else None
    w = torch.randn(D, device="cuda", dtype=dtype, requires_grad=True)
    b = torch.randn(D, device="cuda", dtype=dtype, requires_grad=True) if bias else None
    y = nn_ops.layer_norm(x, r, w, b)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    rf = r.detach().float().requires_grad_(True) if res else None
    bf = b.detach().float().requires_grad_(True) if bias else None
    z = xf + rf if res else xf
    if dtype == torch.bfloat16 and res:
        z = z + (z.detach().to(dtype).float() - z.detach())          # the kernel rounds the sum to bf16, as x + r in bf16 does
    yr = F.layer_norm(z, (D,), wf, bf)
    g = torch.randn_like(yr)
    (y.float() * g).sum().backward()
    (yr * g).sum().backward()
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=4e-2, atol=4e-2)
    assert torch.allclose(y.float(), yr, **tol)
    assert torch.allclose(x.grad.float(), xf.grad, **tol)
    if res:
        assert torch.allclose(r.grad.float(), rf.grad, **tol)
    wt = dict(rtol=1e-3, atol=1e-3) if dtype == torch.float32 else dict(rtol=5e-2, atol=0.3)
    assert torch.allclose(w.grad.float(), wf.grad, **wt)
    if bias:
        assert torch.allclose(b.grad.float(), bf.grad, **wt)


@pytest.mark.parametrize("rows,C,dtype", [(32768, 1536, torch.bfloat16), (1000, 520, torch.bfloat16), (777, 99, torch.bfloat16),
                                          (4096, 260, torch.float32), (65, 8, torch.float16), (3, 2050, torch.float32)])
def test_col_sum_matches_fp32_sum(rows, C, dtype):
    """Bias gradient of a Linear layer: column sums with fp32 accumulation; strided rows (a padded view) are read in place."""
    from supergrok15_b200 import _build
    torch.manual_seed(rows + C)
    buf = torch.randn(rows, C + 8, device="cuda").to(dtype)
    for x in (buf[:, :C].contiguous(), buf[:, :C]):
        out = _build.require().col_sum(x)
        ref = x.float().sum(0)
        tol = 1e-4 if dtype == torch.float32 else 1e-2
        assert out.dtype == dtype and out.shape == (C,)
        assert torch.allclose(out.float(), ref, rtol=tol, atol=tol * rows ** 0.5), (out.float() - ref).abs().max()
        assert torch.equal(out, _build.require().col_sum(x))                 # fixed summation order: bitwise reproducible


@pytest.mark.parametrize("linear", ["cublas", "tcgen05"])
@pytest.mark.parametrize("side_stream", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_grad_sink_equals_autograd_accumulation(dtype, side_stream, linear, monkeypatch):
    """Inside ``grad_sink`` the Linear and LayerNorm backward kernels add the parameter gradients to ``.grad`` themselves (weight
    gradients on a side stream): after two backward passes every ``.grad`` equals what autograd's own accumulation produces.
    ``tcgen05``: the three GEMMs of every bf16 layer run on the hand-written kernel (wgrad with beta = 1 in its epilogue)."""
    import copy
    from supergrok15_b200.models import Transformer
    if linear == "tcgen05" and dtype != torch.bfloat16:
        pytest.skip("the tcgen05 Linear path takes bf16 layers")
    torch.manual_seed(3)
    a = Transformer(2, 128, 4, 99, 4).cuda().to(dtype)
    b = copy.deepcopy(a)
    x = torch.randint(0, 99, (256, 4), device="cuda")
    y = torch.randint(0, 99, (256,), device="cuda")
    for p in list(a.parameters()) + list(b.parameters()):
        p.grad = torch.zeros_like(p)
    for k in range(2):                                                     # reference: cuBLAS + autograd accumulation
        F.cross_entropy(b(x[k::2]).float(), y[k::2]).backward()
    monkeypatch.setenv("SG_LINEAR", linear)
    stream = torch.cuda.Stream() if side_stream else None
    with nn_ops.grad_sink(True, stream):
        for k in range(2):
            F.cross_entropy(a(x[k::2]).float(), y[k::2]).backward()
    torch.cuda.synchronize()
    if linear == "tcgen05":
        from supergrok15_b200.ops import gemm
        gemm.check()
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        scale = q.grad.float().abs().max().item() + 1e-12
        tol = 1e-5 if dtype == torch.float32 else (1.6e-2 if linear == "cublas" else 3e-2)   # bf16: one rounding fewer than autograd
        assert (p.grad.float() - q.grad.float()).abs().max().item() <= tol * scale, n
        assert p.grad.float().abs().max().item() > 0, n
