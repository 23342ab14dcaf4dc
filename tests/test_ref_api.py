"""The reference's ``_ops`` entry points (names, argument order, keywords) on this package's kernels: each adapter against the
optimizer class or the PyTorch oracle that implements the same update."""
import copy

import pytest
import torch

import grokking_optimizers as go
from grokking_optimizers import _ops
from supergrok15_b200.ops import oracle

from helpers import make_params


def test_all_reference_entry_points_exist():
    names = ["supergrok15_fused_step", "supergrok15_sam_perturb_all", "supergrok15_sharpness_restore_all", "supergrok11_fused_step",
             "supergrok11_sam_perturb_all", "supergrok11_sharpness_restore_all", "grokadamw_fused_step", "neuralgrok_fused_step",
             "prodigy_fused_step", "grokfast_fused_step", "lion_fused_step", "looksam_perturb_all", "looksam_restore_all",
             "looksam_compute_directions", "looksam_adjust_grads", "muon_fused_step", "supergrok2_mamba_peer_step",
             "supergrok2_mamba_peer_batched_step", "supergrok2_bilevel_fwd_save", "supergrok2_bilevel_backward",
             "supergrok2_bilevel_fwd_save_batched", "supergrok2_bilevel_backward_batched"]
    assert len(names) == 22 and all(callable(getattr(_ops, n)) for n in names)
    import importlib
    assert importlib.import_module("grokking_optimizers._ops") is _ops


def _state(ps):
    return [torch.zeros(p.numel()) for p in ps]


def test_lion_and_grokadamw_adapters_match_the_optimizer_classes():
    shapes = [(33,), (8, 9), (257,)]
    ps = make_params(shapes)
    ref = copy.deepcopy(ps)
    for p, q in zip(ps, ref):
        q.grad = p.grad.clone()
    opt = go.Lion(ref, lr=3e-4, betas=(0.9, 0.99), weight_decay=3.0)
    opt.step()
    m = [torch.zeros_like(p) for p in ps]
    _ops.lion_fused_step(params=ps, grads=[p.grad for p in ps], exp_avgs=m, lr=3e-4, beta1=0.9, beta2=0.99, wd=3.0)
    for p, q in zip(ps, ref):
        assert torch.allclose(p, q, rtol=1e-6, atol=1e-7)
    ps = make_params(shapes, seed=2)
    ref = copy.deepcopy(ps)
    for p, q in zip(ps, ref):
        q.grad = p.grad.clone()
    opt = go.GrokAdamW(ref)
    opt.step()
    g = opt.param_groups[0]
    m, v, e = ([torch.zeros_like(p) for p in ps] for _ in range(3))
    _ops.grokadamw_fused_step(ps, [p.grad for p in ps], m, v, e, [1] * len(ps), g["alpha"], g["lamb"], g["betas"][0], g["betas"][1],
                              g["lr"], g["weight_decay"], g["eps"], g["grad_clip"])
    for p, q in zip(ps, ref):
        assert torch.allclose(p, q, rtol=1e-5, atol=1e-7)


def test_grokfast_looksam_prodigy_muon_adapters_match_the_oracle():
    ps = make_params([(40,), (6, 7)])
    gs = [p.grad.clone() for p in ps]
    e1, e2 = [torch.zeros_like(g) for g in gs], [torch.zeros_like(g) for g in gs]
    g2 = [g.clone() for g in gs]
    _ops.grokfast_fused_step(gs, e1, 0.98, 2.0)
    oracle.grokfast_ema_(g2, e2, 0.98, 2.0)
    assert all(torch.allclose(a, b) for a, b in zip(gs, g2))
    # LookSAM: perturb returns the backups, restore brings the parameters back, directions are unit vectors
    before = [p.detach().clone() for p in ps]
    backups = _ops.looksam_perturb_all(ps, [p.grad for p in ps], 0.05)
    assert not torch.equal(ps[0].detach(), before[0])
    _ops.looksam_restore_all(ps, backups)
    assert all(torch.equal(p.detach(), b) for p, b in zip(ps, before))
    sam = [p.grad + 0.1 * torch.randn_like(p.grad) for p in ps]
    v = [torch.zeros_like(p.grad) for p in ps]
    _ops.looksam_compute_directions(v, sam, [p.grad for p in ps])
    assert all(abs(float(x.norm()) - 1.0) < 1e-5 for x in v)
    gn = [p.grad.clone() for p in ps]
    _ops.looksam_adjust_grads(gn, v, 0.7)
    for a, p, d in zip(gn, ps, v):
        assert torch.allclose(a, p.grad + 0.7 * p.grad.norm() * d, rtol=1e-5, atol=1e-7)
    # Prodigy returns the distance estimate
    m, vv, s = ([torch.zeros_like(p) for p in ps] for _ in range(3))
    p0 = [p.detach().clone() for p in ps]
    d = _ops.prodigy_fused_step(ps, [p.grad for p in ps], m, vv, s, p0, [1, 1], 1e-6, 0.9, 0.999, 1.0, 0.0, 1e-8)
    assert isinstance(d, float) and d >= 1e-6
    # Muon rejects 1-D parameters like the reference and matches the oracle on matrices
    with pytest.raises(RuntimeError, match="matrix"):
        _ops.muon_fused_step([ps[0]], [ps[0].grad], [torch.zeros_like(ps[0])], 0.95, 0.02, 0.0, 5)
    a, b = copy.deepcopy(ps[1]), copy.deepcopy(ps[1])
    ba, bb = torch.zeros_like(a), torch.zeros_like(b)
    _ops.muon_fused_step([a], [ps[1].grad], [ba], 0.95, 0.02, 0.1, 5)
    oracle.muon_([b], [ps[1].grad], [bb], 0.02, 0.95, 0.1, 5)
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)


def test_supergrok15_adapter_matches_the_optimizer_in_reference_compat_mode():
    """The adapter, like the reference's C++, uses step + 1 of the list it is given and never writes the list back."""
    ps = make_params([(50,), (4, 9)], seed=4)
    ref = copy.deepcopy(ps)
    for p, q in zip(ps, ref):
        q.grad = p.grad.clone()
    opt = go.SuperGrok15(ref, warmup_steps=0, warmup_ramp=1)
    with torch.no_grad():
        opt.meta_net.rescale.fill_(0.3)
    opt.step()
    W1, b1, W2, b2, rescale = opt.meta_net.get_weights() if hasattr(opt.meta_net, "get_weights") else (None,) * 5
    if W1 is None:
        pytest.skip("meta-net without get_weights")
    n = len(ps)
    m, v, mu, sh = ([torch.zeros(p.numel()) for p in ps] for _ in range(4))
    steps = [0] * n
    g = opt.param_groups[0]
    _ops.supergrok15_fused_step(ps, [p.grad for p in ps], m, v, mu, sh, steps, list(opt._flat_layer_alphas_eff) if hasattr(opt, "_flat_layer_alphas_eff")
                                else [max(0.0, min(1.0, opt._cached_alpha * a)) for a in opt._flat_layer_alphas], list(opt._flat_layer_beta1s),
                                W1, b1, W2, b2, float(rescale), int(b1.numel()), g["betas"][1], g["lr"], opt._get_effective_wd(g["weight_decay"]),
                                g["eps"], opt.lamb, opt._get_ramp_factor(), opt._get_gate_signal(), opt.gradient_clipping)
    assert steps == [0] * n
    for p, q in zip(ps, ref):
        assert torch.allclose(p, q, rtol=1e-5, atol=1e-7), (p - q).abs().max()


@pytest.mark.gpu
def test_supergrok2_batched_adapter_matches_the_optimizer_step():
    """The reference's 60-argument batched v2 entry point, fed from a SuperGrok2 instance, updates the parameters like SuperGrok2.step()."""
    dev = "cuda"
    ps = make_params([(300,), (17, 9), (2000,)], device=dev, seed=6)
    ref = copy.deepcopy(ps)
    for p, q in zip(ps, ref):
        q.grad = p.grad.clone()
    opt = go.SuperGrok2(ref, warmup_steps=0, warmup_ramp=1, gradient_clipping=1e9)
    opt.step()
    mn = opt.meta_net
    n = len(ps)
    st = lambda *shape: [torch.zeros(p.numel(), *shape, device=dev) for p in ps]  # noqa: E731
    m, v, mu, sh, gru = st(), st(), st(), st(), st(4)
    hf, hb = [torch.zeros(16, 16, device=dev) for _ in ps], [torch.zeros(16, 16, device=dev) for _ in ps]
    W = []
    W += [mn.input_proj.weight, mn.input_proj.bias]
    for blk in (mn.mamba_fwd, mn.mamba_bwd):
        W += [blk.in_proj.weight, blk.dt_proj.weight, blk.dt_proj.bias, blk.B_proj.weight, blk.C_proj.weight, blk.A_log, blk.D, blk.rope_freq,
              blk.out_proj.weight]
    W += [mn.gru.W_z.weight, mn.gru.W_z.bias, mn.gru.W_r.weight, mn.gru.W_r.bias, mn.gru.W_h.weight, mn.gru.W_h.bias]
    W += [torch.stack([q.weight for q in mn.peer_queries]), torch.stack(list(mn.product_keys_A)), torch.stack(list(mn.product_keys_B))]
    W += [mn.expert_W1, mn.expert_b1, mn.expert_W2, mn.expert_b2]
    g = opt.param_groups[0]
    b2 = g["betas"][1]
    lamb_eff = opt.lamb * opt._get_ramp_factor() * opt._get_gate_signal()
    alphas = [max(0.0, min(1.0, opt._cached_alpha * a)) for a in opt._flat_layer_alphas]
    b1s = list(opt._flat_layer_beta1s)
    counts = torch.zeros(144, dtype=torch.int32, device=dev)
    _ops.supergrok2_mamba_peer_batched_step(ps, [p.grad for p in ps], sh, m, v, mu, gru, hf, hb, *W, alphas, [lamb_eff] * n, b1s,
                                            [1 - b ** 1 for b in b1s], [1 - b2] * n, float(mn.rescale), b2, g["lr"],
                                            opt._get_effective_wd(g["weight_decay"]), g["eps"], 8, 16, 16, 4, 4, 12, 16, 144, counts)
    for p, q in zip(ps, ref):
        assert torch.allclose(p, q, rtol=1e-5, atol=1e-7), (p - q).abs().max()
    assert int(counts.sum()) == 4 * sum(p.numel() for p in ps)
