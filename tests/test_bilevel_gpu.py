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
