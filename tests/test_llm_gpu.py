"""Decoder-model kernels (RMSNorm, rotary embedding, SwiGLU, GELU, embedding, cross-entropy) against PyTorch fp32 references."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from supergrok15_b200 import _build
    _build.require()
    return torch.device("cuda:0")


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("with_res", [False, True])
def test_rms_norm(dtype, with_res):
    from supergrok15_b200.ops import nn_ops
    dev = _dev()
    torch.manual_seed(0)
    x = torch.randn(37, 5, 256, device=dev, dtype=dtype, requires_grad=True)
    r = torch.randn_like(x, requires_grad=True) if with_res else None
    w = (torch.rand(256, device=dev) + 0.5).to(dtype).requires_grad_(True)
    xr, rr, wr = x.detach().float().requires_grad_(True), (r.detach().float().requires_grad_(True) if with_res else None), w.detach().float().requires_grad_(True)
    if with_res:
        y, z = nn_ops.norm_residual(x, r, w, None, 1e-5, rms=True)
        zr = (xr + rr).to(dtype).float() if dtype == torch.bfloat16 else xr + rr
        yr = F.rms_norm(zr, (256,), wr, 1e-5)
        gy, gz = torch.randn_like(yr), torch.randn_like(yr)
        (y.float() * gy + z.float() * gz).sum().backward()
        (yr * gy + zr * gz).sum().backward()
        torch.testing.assert_close(z.float(), zr, **_tol(dtype))
        torch.testing.assert_close(r.grad.float(), rr.grad, **_tol(dtype))
    else:
        y = nn_ops.rms_norm(x, None, w, 1e-5)
        yr = F.rms_norm(xr, (256,), wr, 1e-5)
        gy = torch.randn_like(yr)
        (y.float() * gy).sum().backward()
        (yr * gy).sum().backward()
    torch.testing.assert_close(y.float(), yr, **_tol(dtype))
    torch.testing.assert_close(x.grad.float(), xr.grad, **_tol(dtype))
    wt = dict(rtol=3e-2, atol=0.3) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(w.grad.float(), wr.grad, **wt)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope(dtype):
    from supergrok15_b200.ops import nn_ops
    from supergrok15_b200.models.llama import rope_tables
    dev = _dev()
    torch.manual_seed(1)
    B, S, H, HD = 3, 17, 4, 64
    cos, sin = rope_tables(S, HD, 10000.0, dev)
    x = torch.randn(B, S, H, HD, device=dev, dtype=dtype, requires_grad=True)
    xr = x.detach().float().requires_grad_(True)
    y = nn_ops.rope(x, cos, sin)
    yr = nn_ops.rope_reference(xr, cos, sin)
    g = torch.randn_like(yr)
    (y.float() * g).sum().backward()
    (yr * g).sum().backward()
    torch.testing.assert_close(y.float(), yr, **_tol(dtype))
    torch.testing.assert_close(x.grad.float(), xr.grad, **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_gelu(dtype):
    from supergrok15_b200.ops import nn_ops
    dev = _dev()
    torch.manual_seed(2)
    g = torch.randn(33, 352, device=dev, dtype=dtype, requires_grad=True)
    u = torch.randn(33, 352, device=dev, dtype=dtype, requires_grad=True)
    gr, ur = g.detach().float().requires_grad_(True), u.detach().float().requires_grad_(True)
    y, yr = nn_ops.swiglu(g, u), F.silu(gr) * ur
    w = torch.randn_like(yr)
    (y.float() * w).sum().backward()
    (yr * w).sum().backward()
    torch.testing.assert_close(y.float(), yr, **_tol(dtype))
    torch.testing.assert_close(g.grad.float(), gr.grad, **_tol(dtype))
    torch.testing.assert_close(u.grad.float(), ur.grad, **_tol(dtype))
    x = torch.randn(16, 256, device=dev, dtype=dtype, requires_grad=True)
    xr = x.detach().float().requires_grad_(True)
    y, yr = nn_ops.gelu(x), F.gelu(xr)
    w = torch.randn_like(yr)
    (y.float() * w).sum().backward()
    (yr * w).sum().backward()
    torch.testing.assert_close(y.float(), yr, **_tol(dtype))
    torch.testing.assert_close(x.grad.float(), xr.grad, **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,D", [(300, 128), (115, 520), (5000, 128)])     # small tables: one kernel without a sort; the last one sorts
def test_embedding(dtype, V, D):
    from supergrok15_b200 import _build
    from supergrok15_b200.ops import nn_ops
    dev = _dev()
    torch.manual_seed(3)
    W = torch.randn(V, D, device=dev, dtype=dtype, requires_grad=True)
    ids = torch.randint(0, V, (7, 1000), device=dev)
    ids[0, :200] = 5                                   # a long run of one token
    out = nn_ops.embedding(ids, W)
    assert torch.equal(out, W.detach()[ids])
    g = torch.randn(7, 1000, D, device=dev, dtype=dtype)
    out.backward(g)
    ref = torch.zeros(V, D, device=dev, dtype=torch.float32).index_add_(0, ids.reshape(-1), g.reshape(-1, D).float())
    tol = dict(rtol=2e-2, atol=0.15) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(W.grad.float(), ref, **tol)
    first = W.grad.clone()
    W.grad = None
    nn_ops.embedding(ids, W).backward(g)
    assert torch.equal(first, W.grad), "embedding gradient must be bitwise reproducible"
    base = torch.randn(V, D, device=dev, dtype=dtype)                       # accumulation into an existing gradient buffer
    acc = base.clone()
    assert _build.require().embedding_bwd(ids, g, V, acc).data_ptr() == acc.data_ptr()
    torch.testing.assert_close(acc.float(), ref + base.float(), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cross_entropy(dtype):
    from supergrok15_b200.ops import nn_ops
    dev = _dev()
    torch.manual_seed(4)
    rows, V = 777, 4096 + 8
    x = (torch.randn(rows, V, device=dev) * 3).to(dtype).requires_grad_(True)
    t = torch.randint(0, V, (rows,), device=dev)
    t[::13] = -100
    xr = x.detach().float().requires_grad_(True)
    loss = nn_ops.cross_entropy(x, t)
    ref = F.cross_entropy(xr, t, ignore_index=-100)
    (loss * 1.7).backward()
    (ref * 1.7).backward()
    torch.testing.assert_close(loss, ref, rtol=1e-4, atol=1e-4)
    tol = dict(rtol=2e-2, atol=1e-5) if dtype == torch.bfloat16 else dict(rtol=1e-3, atol=1e-7)
    torch.testing.assert_close(x.grad.float(), xr.grad, **tol)


def test_llama_tiny_matches_reference_ops():
    """The decoder built from the fused kernels equals the same network evaluated with plain PyTorch ops in fp32."""
    from supergrok15_b200.models.llama import Llama, LLAMA_TINY
    dev = _dev()
    torch.manual_seed(5)
    model = Llama(LLAMA_TINY).to(dev)
    ref = Llama(LLAMA_TINY)
    ref.load_state_dict(model.state_dict())
    ids = torch.randint(0, LLAMA_TINY.vocab, (4, 32), device=dev)
    out = model(ids)
    out_ref = ref(ids.cpu())
    torch.testing.assert_close(out.cpu(), out_ref, rtol=2e-3, atol=2e-3)
    out.float().pow(2).mean().backward()
    out_ref.float().pow(2).mean().backward()
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p.grad.cpu(), q.grad, rtol=5e-3, atol=2e-4, msg=lambda m, n=n: f"{n}: {m}")


@pytest.mark.parametrize("shape", [(1, 128, 1, 128, True), (2, 256, 2, 128, True), (1, 512, 2, 64, True), (2, 384, 3, 128, False)])
def test_flash_attention_forward(shape):
    """tcgen05 flash attention (K-major Q/K/P operands, MN-major V operand) against fp32 PyTorch attention."""
    from supergrok15_b200.ops import gemm, nn_ops
    dev = _dev()
    B, S, H, HD, causal = shape
    torch.manual_seed(6)
    qkv = torch.randn(B, S, 3, H, HD, device=dev).to(torch.bfloat16)
    for q, k, v in [tuple(t.contiguous() for t in qkv.unbind(2)), qkv.unbind(2)]:       # contiguous tensors, then strided views
        if not nn_ops.flash_supported(q, k, v):
            continue
        q = q.detach().requires_grad_(True)
        out = nn_ops.attention(q, k, v, causal, impl="tcgen05")
        torch.cuda.synchronize()
        gemm.check(dev)
        ref = nn_ops.attention_reference(q.detach().float(), k.float(), v.float(), causal)
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
        out.float().sum().backward()
        assert torch.isfinite(q.grad).all()


@pytest.mark.parametrize("shape", [(1, 128, 1, 128, True), (1, 256, 2, 128, True), (2, 384, 2, 128, False), (1, 512, 2, 64, True)])
def test_flash_attention_backward(shape):
    """tcgen05 backward kernels (dK/dV per key tile, dQ per query tile) against autograd through fp32 PyTorch attention."""
    from supergrok15_b200.ops import gemm, nn_ops
    dev = _dev()
    B, S, H, HD, causal = shape
    torch.manual_seed(7)
    q, k, v = (torch.randn(B, S, H, HD, device=dev).to(torch.bfloat16).requires_grad_(True) for _ in range(3))
    do = torch.randn(B, S, H, HD, device=dev).to(torch.bfloat16)
    nn_ops.attention(q, k, v, causal, impl="tcgen05").backward(do)
    torch.cuda.synchronize()
    gemm.check(dev)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    nn_ops.attention_reference(qr, kr, vr, causal).backward(do.float())
    for got, ref in zip((q, k, v), (qr, kr, vr)):
        err = float((got.grad.float() - ref.grad).abs().max() / ref.grad.abs().max())
        assert err < 2e-2, err


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gelu_16bit_rational_erf_is_within_one_ulp(dtype):
    """16-bit GELU uses a rational erf approximation (absolute error 1.5e-7): forward and derivative stay within one unit in the
    last place of the 16-bit result of the fp64 erf formula over [-12, 12], tails included."""
    from supergrok15_b200.ops import nn_ops
    dev = _dev()
    x = torch.linspace(-12, 12, 8 * 40001, device=dev).to(dtype).requires_grad_(True)
    xd = x.detach().double()
    cdf = 0.5 * (1 + torch.erf(xd / 2 ** 0.5))
    ref = xd * cdf
    dref = cdf + xd * torch.exp(-0.5 * xd * xd) / (2 * torch.pi) ** 0.5
    y = nn_ops.gelu(x)
    y.backward(torch.ones_like(y))
    ulp = 2.0 ** (-8 if dtype == torch.bfloat16 else -11)
    for got, want in ((y, ref), (x.grad, dref)):
        err = (got.double() - want).abs()
        assert bool((err <= ulp * want.abs() + 2e-6).all()), (err - ulp * want.abs()).max().item()
