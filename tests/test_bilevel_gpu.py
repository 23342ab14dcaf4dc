"""CUDA bilevel gradients (parallel scan adjoint + autograd tail) against full autograd of the PyTorch meta-net."""
import copy

import pytest
import torch

from supergrok15_b200 import optim as O
from supergrok15_b200.ops import sg2 as sg2_ops

pytestmark = pytest.mark.gpu


def _setup(shapes, seed=0):
    torch.manual_seed(seed)
    ps = [torch.nn.Parameter(torch.randn(s, device="cuda") * 0.1) for s in shapes]
    opt = O.SuperGrok2(ps)
    with torch.no_grad():
        mn = opt.meta_net
        for blk in (mn.mamba_fwd, mn.mamba_bwd):
            blk.rope_freq.mul_(20)
        mn.expert_W1.mul_(30); mn.expert_W2.mul_(30)
        for k in list(mn.product_keys_A) + list(mn.product_keys_B):
            k.mul_(10)
    opt._ensure_state()
    for i, p in enumerate(ps):
        opt._flat_sharpness[i].uniform_(0, 1e-2)
        opt._flat_gru_states[i].normal_(0, 0.1)
        opt._flat_mamba_fwd_states[i].normal_(0, 0.1)
        opt._flat_mamba_bwd_states[i].normal_(0, 0.1)
    named = [(f"p{i}", p) for i, p in enumerate(ps)]
    tg = {n: torch.randn_like(p) * 1e-2 for n, p in named}
    vg = {n: torch.randn_like(p) * 1e-2 for n, p in named}
    return opt, named, tg, vg


@pytest.mark.parametrize("shapes,chunk", [([(40,)], 0), ([(17,), (300,), (5, 7)], 0), ([(2500,), (700,)], 512)])
def test_cuda_bilevel_gradients_match_autograd(shapes, chunk):
    opt, named, tg, vg = _setup(shapes)
    mn = opt.meta_net
    if chunk:
        sg2_ops._MIN_CHUNK, old = chunk, sg2_ops._MIN_CHUNK
    try:
        mn.zero_grad()
        n = sg2_ops.bilevel_backward(opt, named, tg, vg)
        assert n == len(shapes)
        got = {k: p.grad.clone() for k, p in mn.named_parameters() if p.grad is not None}
        mn.zero_grad()
        opt.bilevel_force_autograd = True
        sg2_ops.bilevel_backward(opt, named, tg, vg)
        ref = {k: p.grad.clone() for k, p in mn.named_parameters() if p.grad is not None}
    finally:
        if chunk:
            sg2_ops._MIN_CHUNK = old
    assert set(got) == set(ref)
    for k in ref:
        scale = ref[k].abs().max().clamp_min(1e-6)
        err = (got[k] - ref[k]).abs().max() / scale
        assert err < 5e-3, (k, float(err), float(scale))


@pytest.mark.parametrize("interval", [8, 32, 100])
def test_checkpoint_interval_does_not_change_the_gradients(interval):
    """States kept every 16, 32 or 112 timesteps (intervals 8, 32, 100): the recomputation between snapshots is exact, so the
    meta-net gradients are those of interval 1, bit for bit."""
    from supergrok15_b200.ops import sg2_bilevel
    opt, named, tg, vg = _setup([(2500,), (700,), (33,)])
    mn = opt.meta_net
    sg2_ops._MIN_CHUNK, old = 512, sg2_ops._MIN_CHUNK
    try:
        mn.zero_grad()
        sg2_ops.bilevel_backward(opt, named, tg, vg, 1)
        ref = {k: p.grad.clone() for k, p in mn.named_parameters() if p.grad is not None}
        mn.zero_grad()
        sg2_ops.bilevel_backward(opt, named, tg, vg, interval)
        got = {k: p.grad.clone() for k, p in mn.named_parameters() if p.grad is not None}
    finally:
        sg2_ops._MIN_CHUNK = old
    assert opt._bilevel_ws[1].snap_every == sg2_bilevel.snapshot_tiles(interval) == -(-interval // 16)
    assert set(got) == set(ref)
    for k in ref:
        assert torch.equal(got[k], ref[k]), k


def test_bilevel_step_runs_on_cuda_and_keeps_persistent_states():
    opt, named, tg, vg = _setup([(600,), (33, 9)])
    before = [s.clone() for s in opt._flat_mamba_fwd_states]
    mo = torch.optim.Adam(opt.meta_net.parameters(), lr=1e-3)
    w0 = opt.meta_net.mamba_fwd.A_log.detach().clone()
    opt.meta_net.zero_grad()
    sg2_ops.bilevel_backward(opt, named, tg, vg)
    mo.step()
    assert not torch.equal(w0, opt.meta_net.mamba_fwd.A_log)
    assert all(torch.equal(a, b) for a, b in zip(before, opt._flat_mamba_fwd_states))


def _dense_routed(g, ia, ib, wa, wb, W1, b1, W2, b2, pk):
    """PyTorch statement of the routed expert stage (float64): every selected expert evaluated through gathered tables."""
    n, heads, _ = ia.shape
    e = (ia.unsqueeze(3) * pk + ib.unsqueeze(2)).reshape(n, heads * 16).long()                    # [n, heads*16]
    w = (wa.unsqueeze(3) * wb.unsqueeze(2)).reshape(n, heads * 16)
    z = torch.relu(g.view(n, 1, 1) * W1[e] + b1[e])                                               # [n, heads*16, hidden]
    out = (z * W2[e]).sum(-1) + b2[e]
    return (w * out).sum(-1)


@pytest.mark.parametrize("n,heads,E,pk", [(50, 4, 144, 12), (1000, 4, 144, 12), (70001, 4, 144, 12), (333, 2, 64, 8), (257, 8, 100, 10)])
def test_routed_experts_kernel_matches_dense_formulation(n, heads, E, pk):
    from supergrok15_b200.ops import sg2_bilevel
    torch.manual_seed(n + heads)
    dev = "cuda"
    g = torch.randn(n, device=dev)
    ia = torch.rand(n, heads, pk, device=dev).topk(4, dim=-1).indices.int()
    ib = torch.rand(n, heads, pk, device=dev).topk(4, dim=-1).indices.int()
    wa = torch.softmax(torch.randn(n, heads, 4, device=dev), -1).requires_grad_(True)
    wb = torch.softmax(torch.randn(n, heads, 4, device=dev), -1).requires_grad_(True)
    W1, b1, W2 = (torch.randn(E, 16, device=dev).requires_grad_(True) for _ in range(3))
    b2 = torch.randn(E, device=dev).requires_grad_(True)
    dt = torch.randn(n, device=dev)
    leaves = (wa, wb, W1, b1, W2, b2)
    total = sg2_bilevel.routed_experts(g, ia, ib, wa, wb, W1, b1, W2, b2, pk)
    grads = torch.autograd.grad(total, leaves, dt)
    dl = [t.detach().double().requires_grad_(True) for t in leaves]
    ref = _dense_routed(g.double(), ia.long(), ib.long(), *dl, pk)
    rgrads = torch.autograd.grad(ref, dl, dt.double())
    assert torch.allclose(total.double(), ref, rtol=1e-4, atol=1e-4), (total.double() - ref).abs().max()
    for name, a, b in zip(("wa", "wb", "W1", "b1", "W2", "b2"), grads, rgrads):
        scale = b.abs().max().clamp_min(1e-6)
        assert (a.double() - b).abs().max() / scale < 2e-4, (name, float((a.double() - b).abs().max()), float(scale))
    again = torch.autograd.grad(sg2_bilevel.routed_experts(g, ia, ib, wa, wb, W1, b1, W2, b2, pk), leaves, dt)
    for a, b in zip(grads, again):
        assert torch.equal(a, b)                                                                  # fixed summation order


def test_soft_head_expert_kernel_matches_dense_path(monkeypatch):
    opt, named, tg, vg = _setup([(3000,)])
    mn = opt.meta_net
    n = 3000
    torch.manual_seed(5)
    g = torch.randn(n, device="cuda") * 1e-2
    s = torch.rand(n, device="cuda") * 1e-2
    gru = torch.randn(n, mn.gru_hidden, device="cuda") * 0.1
    ctx = torch.randn(n, 16, device="cuda") * 0.1
    vu = torch.randn(n, device="cuda")
    res = {}
    for mode in ("kernel", "dense"):
        monkeypatch.setenv("SG_BILEVEL_EXPERTS", mode)
        mn.zero_grad(set_to_none=True)
        c = ctx.clone().requires_grad_(True)
        smart = mn.soft_head(g, s, gru, c[:, :8], c[:, 8:])
        (smart * vu).sum().backward()
        res[mode] = (smart.detach(), c.grad.clone(), {k: p.grad.clone() for k, p in mn.named_parameters() if p.grad is not None})
    assert torch.allclose(res["kernel"][0], res["dense"][0], rtol=1e-5, atol=1e-7)
    assert torch.allclose(res["kernel"][1], res["dense"][1], rtol=1e-3, atol=1e-6 + 1e-3 * float(res["dense"][1].abs().max()))
    assert set(res["kernel"][2]) == set(res["dense"][2])
    for k, gd in res["dense"][2].items():
        gk = res["kernel"][2][k]
        assert (gk - gd).abs().max() <= 1e-3 * gd.abs().max() + 1e-9, (k, float((gk - gd).abs().max()), float(gd.abs().max()))


@pytest.mark.parametrize("n,IN", [(1, 18), (1000, 18), (70001, 18), (300, 10)])
def test_gru_kernels_match_cpu_loop(n, IN):
    """The CUDA GRU kernels against the C++ CPU loop over the same per-element functions (csrc/sg2_gru_math.h)."""
    from supergrok15_b200.ops import sg2_bilevel
    torch.manual_seed(n)
    cpu = [torch.randn(n, IN), torch.randn(n, 4), torch.randn(3, 4, IN + 4) * 0.5, torch.randn(3, 4) * 0.5]
    gout = torch.randn(n, 4)
    outs = []
    for dev in ("cpu", "cuda"):
        x, h, W, b = (t.to(dev) for t in cpu)
        x.requires_grad_(True), W.requires_grad_(True), b.requires_grad_(True)
        out = sg2_bilevel.gru(x, h, W, b)
        outs.append([t.cpu() for t in (out, *torch.autograd.grad((out * gout.to(dev)).sum(), [x, W, b]))])
    for a, b_ in zip(*outs):
        assert (a - b_).abs().max() <= 1e-3 * a.abs().max() + 1e-6


@pytest.mark.parametrize("n,heads,P,pk", [(1, 4, 22, 12), (1000, 4, 22, 12), (70001, 4, 22, 12), (333, 2, 14, 8)])
def test_routing_kernels_match_cpu_loop(n, heads, P, pk):
    """The CUDA routing kernels against the C++ CPU loop over the same per-element functions (csrc/sg2_routing_math.h)."""
    from supergrok15_b200.ops import sg2_bilevel
    torch.manual_seed(n)
    cpu = [torch.randn(n, P), torch.randn(heads * 8, P) * 0.3, torch.randn(heads, pk, 4), torch.randn(heads, pk, 4)]
    gwa, gwb = torch.randn(n, heads, 4), torch.randn(n, heads, 4)
    outs = []
    for dev in ("cpu", "cuda"):
        leaves = [t.to(dev).requires_grad_(True) for t in cpu]
        ia, ib, wa, wb = sg2_bilevel.routing(*leaves)
        grads = torch.autograd.grad((wa * gwa.to(dev)).sum() + (wb * gwb.to(dev)).sum(), leaves)
        outs.append([t.cpu() for t in (ia, ib, wa, wb, *grads)])
    same = (outs[0][0] == outs[1][0]).all(-1).all(-1) & (outs[0][1] == outs[1][1]).all(-1).all(-1)
    assert same.float().mean() > 0.999                       # a near-tie may be ordered differently by fused multiply-adds
    assert torch.allclose(outs[0][2][same], outs[1][2][same], rtol=1e-4, atol=1e-5)
    for a, b in zip(outs[0][4:], outs[1][4:]):
        assert (a - b).abs().max() <= 2e-3 * a.abs().max() + 1e-6
