"""CPU tests of the optimizer API and of the PyTorch oracle (no GPU needed)."""
import math
import os

import pytest
import torch
import torch.nn.functional as F

from supergrok15_b200 import optim as O
from supergrok15_b200.models import Transformer
from supergrok15_b200.ops import oracle
from supergrok15_b200.optim.metanet import Mamba3PEERMetaNet, Mamba3ScanBlock, affine_scan_chunked

from helpers import make_params, set_grads


def _model_and_batch(seed=0):
    torch.manual_seed(seed)
    m = Transformer(1, 32, 2)
    x = torch.randint(0, 97, (64, 4))
    y = torch.randint(0, 97, (64,))
    return m, x, y


FACTORIES = {
    "adamw": lambda m: O.AdamW(m.parameters(), lr=1e-3),
    "lion": lambda m: O.Lion(m.parameters()),
    "grokfast": lambda m: O.Grokfast(m.parameters()),
    "grokadamw": lambda m: O.GrokAdamW(m.parameters()),
    "prodigy": lambda m: O.Prodigy(m.parameters(), lr=1e-3),
    "neuralgrok": lambda m: O.NeuralGrok(m.parameters()),
    "looksam": lambda m: O.LookSAM(m.parameters()),
    "muon": lambda m: O.Muon([p for p in m.parameters() if p.dim() == 2], [p for p in m.parameters() if p.dim() != 2]),
    "supergrok15": lambda m: O.SuperGrok15(m.parameters()),
    "supergrok11": lambda m: O.SuperGrok11(m.parameters()),
    "supergrok2": lambda m: O.SuperGrok2(m.parameters()),
}


def test_prodigy_follows_reference_formula():
    """The reference's distance estimate divides by sum(s) with s = EMA of (d*g)^2 (csrc/ops.cpp:470-478), which is
    tiny, so d_lr jumps by many orders of magnitude on the second step.  That behaviour is kept; this test pins it."""
    ps = make_params([(40,), (6, 7)], seed=5)
    opt = O.Prodigy(ps, lr=1e-3)
    p0 = [p.detach().clone() for p in ps]
    g = [p.grad.clone() for p in ps]
    opt.step()
    assert opt.d_lr == 1e-6                         # sum(s) == 0 on the first step: no update of d_lr
    d, b1, b2 = 1e-6, 0.9, 0.999
    for p, q, gg in zip(ps, p0, g):
        m = (1 - b1) * d * gg
        v = (1 - b2) * d * d * gg * gg
        ref = q * (1 - 1e-3 * d * 1.0) - (1e-3 / (1 - b1)) * m / ((v / (1 - b2)).sqrt() + d * 1e-8)
        assert torch.allclose(p, ref, rtol=1e-5, atol=1e-8)
    set_grads(ps, 9)
    opt.step()
    assert opt.d_lr > 1e-6                          # monotone, non-decreasing


@pytest.mark.parametrize("name", [n for n in FACTORIES if n != "prodigy"])
def test_every_optimizer_steps_and_reduces_loss(name):
    m, x, y = _model_and_batch()
    opt = FACTORIES[name](m)
    losses = []
    for _ in range(3 if name == "supergrok2" else 6):
        opt.zero_grad()
        loss = F.cross_entropy(m(x), y)
        loss.backward()
        losses.append(loss.item())
        opt.step()
    assert all(math.isfinite(l) for l in losses)
    assert losses[-1] < losses[0]
    for p in m.parameters():
        assert torch.isfinite(p).all()


def test_adamw_matches_torch():
    a = make_params([(7, 5), (11,)], seed=1)
    b = [torch.nn.Parameter(p.detach().clone()) for p in a]
    oa, ob = O.AdamW(a, lr=1e-2, betas=(0.9, 0.98), weight_decay=0.5), torch.optim.AdamW(b, lr=1e-2, betas=(0.9, 0.98), weight_decay=0.5)
    for s in range(5):
        set_grads(a, s)
        for p, q in zip(a, b):
            q.grad = p.grad.clone()
        oa.step(); ob.step()
    for p, q in zip(a, b):
        assert torch.allclose(p, q, rtol=1e-5, atol=1e-7)


def test_state_dict_layouts_match_reference():
    m, x, y = _model_and_batch()
    expect = {"lion": {"exp_avg"}, "grokfast": {"step", "ema", "exp_avg", "exp_avg_sq"},
              "grokadamw": {"step", "exp_avg", "exp_avg_sq", "ema"}, "prodigy": {"step", "exp_avg", "exp_avg_sq", "s", "param_init"},
              "neuralgrok": {"step", "exp_avg", "exp_avg_sq"}, "looksam": {"step", "exp_avg", "exp_avg_sq", "sam_direction"}}
    for name, keys in expect.items():
        m, x, y = _model_and_batch()
        opt = FACTORIES[name](m)
        F.cross_entropy(m(x), y).backward()
        opt.step()
        sd = opt.state_dict()
        assert set(sd["state"][0].keys()) == keys, name
    opt = FACTORIES["muon"](m)
    opt.zero_grad(); F.cross_entropy(m(x), y).backward(); opt.step()
    sd = opt.state_dict()
    assert sd["param_groups"][0]["group_type"] == "muon" and sd["param_groups"][1]["group_type"] == "adamw"
    assert set(sd["state"][0].keys()) == {"momentum_buffer"}


@pytest.mark.parametrize("name", ["supergrok15", "supergrok11", "supergrok2", "prodigy"])
def test_state_dict_round_trip_resumes_identically(name):
    m, x, y = _model_and_batch()
    opt = FACTORIES[name](m)
    def one(mm, oo):
        oo.zero_grad(); F.cross_entropy(mm(x), y).backward(); oo.step(**({"train_acc": 0.5} if name.startswith("super") else {}))
    one(m, opt); one(m, opt)
    import copy
    m2 = copy.deepcopy(m)
    opt2 = FACTORIES[name](m2)
    opt2.load_state_dict(copy.deepcopy(opt.state_dict()))
    one(m, opt); one(m2, opt2)
    for p, q in zip(m.parameters(), m2.parameters()):
        assert torch.allclose(p, q, rtol=0, atol=0, equal_nan=True)


def test_reference_compat_freezes_bias_correction_and_breaks_sam():
    m, x, y = _model_and_batch()
    opt = O.SuperGrok15(m.parameters(), reference_compat=True)
    crit = torch.nn.CrossEntropyLoss()
    crit(m(x), y).backward()
    with pytest.raises(RuntimeError):
        opt.sam_step(m, x, y, crit)
    assert all(p.grad is None for p in m.parameters())          # the literal reference outcome
    before = [p.detach().clone() for p in m.parameters()]
    opt.step()                                                   # no gradients -> update skipped, step counted
    assert opt.get_global_step() == 1
    assert all(torch.equal(a, b) for a, b in zip(before, m.parameters()))
    # frozen bias correction: two identical gradients give the same first-step-style scaling
    ps = make_params([(50,)], seed=3)
    o1 = O.SuperGrok15(ps, reference_compat=True, gradient_clipping=0.0)
    o1.step(); set_grads(ps, 3); o1.step()
    qs = make_params([(50,)], seed=3)
    o2 = O.SuperGrok15(qs, reference_compat=False, gradient_clipping=0.0)
    o2.step(); set_grads(qs, 3); o2.step()
    assert not torch.allclose(ps[0], qs[0])


def test_sam_step_fills_sharpness_and_restores_grads():
    m, x, y = _model_and_batch()
    opt = O.SuperGrok15(m.parameters())
    crit = torch.nn.CrossEntropyLoss()
    crit(m(x), y).backward()
    g0 = [p.grad.clone() for p in m.parameters()]
    p0 = [p.detach().clone() for p in m.parameters()]
    loss = opt.sam_step(m, x, y, crit)
    assert math.isfinite(loss)
    assert all(torch.equal(a, p.grad) for a, p in zip(g0, m.parameters()))
    assert all(torch.equal(a, p) for a, p in zip(p0, m.parameters()))
    assert sum(float(s.abs().sum()) for s in opt._flat_sharpness) > 0
    # oracle: explicit perturbation
    norm = math.sqrt(sum(float(g.pow(2).sum()) for g in g0)) + 1e-12
    with torch.no_grad():
        for p, g in zip(m.parameters(), g0):
            p.add_(g, alpha=opt.sam_rho / norm)
    m.zero_grad(); crit(m(x), y).backward()
    ref = (list(m.parameters())[3].grad - g0[3]).abs().reshape(-1)
    assert torch.allclose(opt._flat_sharpness[3], ref, rtol=1e-4, atol=1e-7)


def test_bilevel_updates_meta_net_and_restores_grads():
    for cls in (O.SuperGrok15, O.SuperGrok2):
        m, x, y = _model_and_batch()
        opt = cls(m.parameters())
        if cls is O.SuperGrok15:
            with torch.no_grad():
                opt.meta_net.rescale.fill_(0.1)
        crit = torch.nn.CrossEntropyLoss()
        crit(m(x), y).backward()
        g0 = [p.grad.clone() for p in m.parameters()]
        w0 = [p.detach().clone() for p in opt.meta_net.parameters()]
        mo = torch.optim.Adam(opt.meta_net.parameters(), lr=1e-3)
        v = opt.bilevel_step(m, x, y, x, y, crit, mo)
        assert math.isfinite(v)
        assert all(torch.equal(a, p.grad) for a, p in zip(g0, m.parameters()))
        assert any(not torch.equal(a, p) for a, p in zip(w0, opt.meta_net.parameters()))


def test_newton_schulz_gram_form_equals_left_form():
    torch.manual_seed(0)
    for shape in ((24, 8), (8, 24), (16, 16)):
        X = torch.randn(shape, dtype=torch.float64)
        X = X / X.norm()
        assert torch.allclose(oracle.newton_schulz(X, 5), oracle.newton_schulz_gram(X, 5), rtol=1e-8, atol=1e-10)


def test_muon_rejects_1d_in_matrix_group():
    p = torch.nn.Parameter(torch.randn(5)); p.grad = torch.randn(5)
    with pytest.raises(ValueError):
        O.Muon([p]).step()


@pytest.mark.parametrize("N", [1, 2, 15, 16, 17, 63, 64, 65, 200, 1000])
def test_scan_serial_equals_chunked(N):
    torch.manual_seed(N)
    blk = Mamba3ScanBlock().double()
    with torch.no_grad():
        blk.rope_freq.mul_(30)           # make the rotation matter
    x = torch.randn(N, 8, dtype=torch.float64)
    h0 = torch.randn(16, 16, dtype=torch.float64) * 0.1
    a, ha = blk(x, h0, impl="serial")
    b, hb = blk(x, h0, impl="chunked")
    assert torch.allclose(a, b, rtol=1e-9, atol=1e-11) and torch.allclose(ha, hb, rtol=1e-9, atol=1e-11)


def test_scan_gradients_serial_equals_chunked():
    torch.manual_seed(0)
    blk = Mamba3ScanBlock().double()
    x = torch.randn(70, 8, dtype=torch.float64)
    outs = []
    for impl in ("serial", "chunked"):
        blk.zero_grad()
        y, _ = blk(x, None, impl=impl)
        (y * torch.linspace(0, 1, y.numel()).reshape(y.shape)).sum().backward()
        outs.append([p.grad.clone() for p in blk.parameters()])
    for ga, gb in zip(*outs):
        assert torch.allclose(ga, gb, rtol=1e-8, atol=1e-11)


def test_metanet_forward_shapes_and_state_persistence():
    torch.manual_seed(0)
    mn = Mamba3PEERMetaNet()
    g, s = torch.randn(300) * 1e-2, torch.rand(300) * 1e-3
    gru = torch.zeros(300, 4)
    sm, gru2, hf, hb = mn(g, s, gru)
    assert sm.shape == g.shape and gru2.shape == (300, 4) and hf.shape == (16, 16) and hb.shape == (16, 16)
    assert int(mn.expert_counts.sum()) == 300 * 4
    sm2, *_ = mn(g, s, gru2, hf, hb)
    assert not torch.equal(sm, sm2)                 # persistent states change the output
    sb, *_ = mn.forward_for_bilevel(g, s, gru)
    assert sb.shape == g.shape and torch.isfinite(sb).all()


def test_expert_recycling_replaces_dead_experts_reproducibly():
    def run():
        torch.manual_seed(0)
        mn = Mamba3PEERMetaNet()
        mn.expert_counts[:10] = 1000
        gen = torch.Generator().manual_seed(7)
        w_before = mn.expert_W1.detach().clone()
        mn._recycle_dead_experts(generator=gen)
        return mn, w_before
    a, wb = run()
    b, _ = run()
    assert torch.equal(a.expert_W1, b.expert_W1)
    assert int(a.expert_counts.sum()) == 0
    assert torch.equal(a.expert_W1[:10], wb[:10]) and not torch.equal(a.expert_W1[10:], wb[10:])


def test_supergrok_schedules():
    ps = make_params([(10,)])
    o = O.SuperGrok15(ps)
    assert o._get_effective_sam_freq() == 20 and o._get_effective_bilevel_freq() == 30
    o._cached_train_acc = 1.0
    assert o._get_effective_sam_freq() == 4 or o._get_effective_sam_freq() == 3
    assert abs(o.get_effective_wd() - 1.0 * (1 + 4 * o._sigmoid(20, 1.0, 0.9))) < 1e-12
    o._global_step = 150
    assert abs(o._get_ramp_factor() - 0.5) < 1e-12
    o._update_alpha(1.0, 3.0, 0.1)
    assert abs(o.get_cached_alpha() - 0.98 * math.exp(-0.1 * 2.0)) < 1e-12
    o._update_alpha(1e-6, 3.0, 0.1)
    assert abs(o.get_cached_alpha() - 0.98 * math.exp(-1.0)) < 1e-12


def test_cuda_graph_wrapper_is_eager_on_cpu():
    ps = make_params([(10,)])
    w = O.CUDAGraphOptimizer(O.Lion(ps), warmup_steps=1)
    for s in range(3):
        set_grads(ps, s); w.step()
    assert w._graph is None


@pytest.mark.parametrize("name", ["adamw", "lion", "grokfast", "grokadamw", "prodigy", "neuralgrok", "looksam", "muon", "supergrok15", "supergrok11"])
def test_cpp_cpu_kernels_match_pytorch_oracle(name):
    """The C++ CPU kernels (csrc/cpu_kernels.cpp) and the PyTorch oracle give the same parameters over several steps on
    tensors whose sizes straddle the 8,192-element chunk."""
    from supergrok15_b200 import _build
    from supergrok15_b200.ops import elementwise as ew
    from helpers import EDGE_SHAPES
    if not _build.native_available():
        pytest.skip("extension not built")
    shapes = [s for s in EDGE_SHAPES if len(s) == 1][::2] + [(64, 48), (40, 72), (8193,)]

    def build(ps):
        if name == "muon":
            return O.Muon([p for p in ps if p.dim() == 2], [p for p in ps if p.dim() != 2])
        cls = {"adamw": O.AdamW, "lion": O.Lion, "grokfast": O.Grokfast, "grokadamw": O.GrokAdamW, "prodigy": O.Prodigy, "neuralgrok": O.NeuralGrok,
               "looksam": O.LookSAM, "supergrok15": O.SuperGrok15, "supergrok11": O.SuperGrok11}[name]
        torch.manual_seed(0)                                    # same meta-net initialisation in both runs
        return cls(ps, lr=1e-3) if name in ("adamw", "prodigy") else cls(ps)

    results = []
    old = ew.CPU_NATIVE
    try:
        for native in (False, True):
            ew.CPU_NATIVE = native
            ps = make_params(shapes, seed=3)
            opt = build(ps)
            for step in range(3 if name != "prodigy" else 1):
                set_grads(ps, 10 + step)
                opt.step()
            results.append([p.detach().clone() for p in ps])
    finally:
        ew.CPU_NATIVE = old
    for a, b in zip(*results):
        torch.testing.assert_close(a, b, rtol=2e-5, atol=2e-6)
    assert any(not torch.equal(a, p0) for a, p0 in zip(results[1], make_params(shapes, seed=3)))     # something moved


def test_soft_head_batched_routing_matches_per_head_statement():
    """soft_head routes all heads with one query product, one block-diagonal key product, one top-k and one softmax; the plain
    statement below does it head by head with gathered expert tables (as forward_for_bilevel does)."""
    from supergrok15_b200.optim.metanet import Mamba3PEERMetaNet
    torch.manual_seed(3)
    mn = Mamba3PEERMetaNet().double()
    with torch.no_grad():
        mn.expert_W1.mul_(30); mn.expert_W2.mul_(30); mn.expert_b1.normal_(0, 0.1); mn.expert_b2.normal_(0, 0.1)
        for k in list(mn.product_keys_A) + list(mn.product_keys_B):
            k.mul_(10)
    n = 500
    g = torch.randn(n, dtype=torch.float64) * 1e-2
    s = torch.rand(n, dtype=torch.float64) * 1e-2
    gru = (torch.randn(n, mn.gru_hidden) * 0.1).double()                 # soft_head reads the GRU state through fp32
    ctx = (torch.randn(n, 16, dtype=torch.float64) * 0.1).requires_grad_(True)
    vu = torch.randn(n, dtype=torch.float64)

    def per_head(c):
        gs = torch.stack([g, s], -1)
        new_gru = mn.gru(torch.cat([gs, c[:, :8], c[:, 8:]], -1), gru)
        pin = torch.cat([new_gru, c[:, :8], c[:, 8:], gs], -1)
        half, total = mn.d_model // 2, 0.0
        for h in range(mn.num_peer_heads):
            q = mn.peer_queries[h](pin)
            ta, ia = (q[:, :half] @ mn.product_keys_A[h].T).topk(4, dim=-1)
            tb, ib = (q[:, half:] @ mn.product_keys_B[h].T).topk(4, dim=-1)
            wa, wb = torch.softmax(ta * 10.0, -1), torch.softmax(tb * 10.0, -1)
            e = (ia.unsqueeze(2) * mn.pk_dim + ib.unsqueeze(1)).reshape(n, -1)
            w = (wa.unsqueeze(2) * wb.unsqueeze(1)).reshape(n, -1)
            z = torch.relu(g.view(n, 1, 1) * mn.expert_W1.squeeze(-1)[e] + mn.expert_b1[e])
            total = total + (w * ((z * mn.expert_W2.squeeze(1)[e]).sum(-1) + mn.expert_b2.squeeze(-1)[e])).sum(-1)
        return g + mn.rescale * total / mn.num_peer_heads

    names = [k for k, _ in mn.named_parameters()]
    out = {}
    for tag, fn in (("batched", lambda c: mn.soft_head(g, s, gru, c[:, :8], c[:, 8:])), ("per_head", per_head)):
        mn.zero_grad(set_to_none=True)
        ctx.grad = None
        y = fn(ctx)
        (y * vu).sum().backward()
        out[tag] = (y.detach(), ctx.grad.clone(), {k: p.grad.clone() for k, p in mn.named_parameters() if p.grad is not None})
    assert torch.allclose(out["batched"][0], out["per_head"][0], rtol=1e-10, atol=1e-12)
    assert torch.allclose(out["batched"][1], out["per_head"][1], rtol=1e-8, atol=1e-12)
    assert set(out["batched"][2]) == set(out["per_head"][2]) and len(out["batched"][2]) > 10
    for k in out["per_head"][2]:
        assert torch.allclose(out["batched"][2][k], out["per_head"][2][k], rtol=1e-8, atol=1e-12), k


_POISON_SCRIPT = r'''
import torch, torch.nn.functional as F
from supergrok15_b200 import optim as O
from supergrok15_b200.ops import elementwise as ew
torch.manual_seed(0)
x, y = torch.randn(64, 16), torch.randint(0, 10, (64,))
for name in ("GrokAdamW", "Prodigy", "NeuralGrok", "SuperGrok15", "SuperGrok11", "LookSAM", "Lion"):
    torch.manual_seed(1)
    m = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 10))
    opt = getattr(O, name)(m.parameters())
    for _ in range(3):
        opt.zero_grad()
        F.cross_entropy(m(x), y).backward()
        opt.step()
    flat = torch.cat([p.detach().reshape(-1) for p in m.parameters()])
    assert torch.isfinite(flat).all(), name
    print(name, ew.DEBUG_POISON, "%.9e" % float(flat.double().abs().sum()))
'''


def test_grok_debug_poisoned_scratch_changes_nothing():
    """GROK_DEBUG=1 fills every scratch buffer with NaN before it is handed out; a step that read scratch it had not written
    would turn non-finite or differ from the normal run."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    outs = []
    for flag in ("0", "1"):
        r = subprocess.run([sys.executable, "-c", _POISON_SCRIPT], env=dict(os.environ, GROK_DEBUG=flag, PYTHONPATH=root),
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        outs.append([l.split() for l in r.stdout.strip().splitlines()])
    assert all(l[1] == "False" for l in outs[0]) and all(l[1] == "True" for l in outs[1])
    assert [(l[0], l[2]) for l in outs[0]] == [(l[0], l[2]) for l in outs[1]]


@pytest.mark.skipif(os.environ.get("SG_TEST_SANITIZE") != "1",
                    reason="compiles every binding file with -Wall -Werror -fsanitize=address,undefined (minutes): set SG_TEST_SANITIZE=1")
def test_host_code_under_asan_ubsan(tmp_path):
    """The C++ CPU kernels and the binding layer run three steps of every element-wise optimizer under ASan + UBSan."""
    import subprocess
    import sys
    from supergrok15_b200 import _build
    asan = subprocess.run(["gcc", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    if not os.path.isabs(asan) or not os.path.exists(asan):
        pytest.skip("libasan not installed")
    so = _build.build_sanitized(tmp_path)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, SG_EXT_SO=str(so), LD_PRELOAD=asan, PYTHONPATH=root, GROK_DEBUG="1",
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=1", UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    r = subprocess.run([sys.executable, "-c", _POISON_SCRIPT], env=env, capture_output=True, text=True, timeout=1800)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    assert "runtime error" not in r.stderr and "AddressSanitizer" not in r.stderr, r.stderr[-6000:]
    assert len(r.stdout.strip().splitlines()) == 7


@pytest.mark.parametrize("n,heads,P,pk", [(1, 4, 22, 12), (257, 4, 22, 12), (90, 2, 14, 8), (64, 4, 30, 16)])
def test_native_routing_matches_pytorch_statement(n, heads, P, pk):
    """csrc/sg2_routing_math.h (run here through its C++ CPU loop; the CUDA kernels execute the same functions) against the
    PyTorch statement: per head a query product, two score products, top-4 and softmax(10 x), gradients through the weights."""
    from supergrok15_b200 import _build
    if not _build.native_available():
        pytest.skip("native extension not built")
    from supergrok15_b200.ops import sg2_bilevel
    torch.manual_seed(n + heads)
    pin = torch.randn(n, P, requires_grad=True)
    Wq = (torch.randn(heads * 8, P) * 0.3).requires_grad_(True)
    KA = torch.randn(heads, pk, 4, requires_grad=True)
    KB = torch.randn(heads, pk, 4, requires_grad=True)
    gwa, gwb = torch.randn(n, heads, 4), torch.randn(n, heads, 4)
    leaves = (pin, Wq, KA, KB)
    ia, ib, wa, wb = sg2_bilevel.routing(pin, Wq, KA, KB)
    grads = torch.autograd.grad((wa * gwa).sum() + (wb * gwb).sum(), leaves)
    dl = [t.detach().double().requires_grad_(True) for t in leaves]
    q = (dl[0] @ dl[1].T).view(n, heads, 8)
    ta, ra = torch.einsum("nhd,hkd->nhk", q[..., :4], dl[2]).topk(4, dim=-1)
    tb, rb = torch.einsum("nhd,hkd->nhk", q[..., 4:], dl[3]).topk(4, dim=-1)
    wa_r, wb_r = torch.softmax(ta * 10.0, -1), torch.softmax(tb * 10.0, -1)
    rgrads = torch.autograd.grad((wa_r * gwa.double()).sum() + (wb_r * gwb.double()).sum(), dl)
    assert torch.equal(ia.long(), ra) and torch.equal(ib.long(), rb)
    assert torch.allclose(wa.double(), wa_r, rtol=1e-4, atol=1e-5) and torch.allclose(wb.double(), wb_r, rtol=1e-4, atol=1e-5)
    for name, a, b in zip(("pin", "Wq", "KA", "KB"), grads, rgrads):
        assert (a.double() - b).abs().max() <= 2e-4 * b.abs().max() + 1e-7, (name, float((a.double() - b).abs().max()), float(b.abs().max()))


@pytest.mark.parametrize("n,IN", [(1, 18), (300, 18), (513, 10)])
def test_native_gru_matches_minigru(n, IN):
    """csrc/sg2_gru_math.h through its C++ CPU loop against the PyTorch MiniGRU: new state, input gradient, weight gradients."""
    from supergrok15_b200 import _build
    if not _build.native_available():
        pytest.skip("native extension not built")
    from supergrok15_b200.ops import sg2_bilevel
    from supergrok15_b200.optim.metanet import MiniGRU
    torch.manual_seed(n)
    cell = MiniGRU(IN, 4)
    with torch.no_grad():
        for p in cell.parameters():
            p.mul_(3)
    x = torch.randn(n, IN, requires_grad=True)
    h = torch.randn(n, 4)
    gout = torch.randn(n, 4)
    ref = cell(x, h)
    rg = torch.autograd.grad((ref * gout).sum(), [x, *cell.parameters()])
    W = torch.stack([cell.W_z.weight, cell.W_r.weight, cell.W_h.weight]).detach().requires_grad_(True)
    b = torch.stack([cell.W_z.bias, cell.W_r.bias, cell.W_h.bias]).detach().requires_grad_(True)
    out = sg2_bilevel.gru(x, h, W, b)
    gx, gW, gb = torch.autograd.grad((out * gout).sum(), [x, W, b])
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-6)
    assert torch.allclose(gx, rg[0], rtol=1e-4, atol=1e-6)
    for k, (wr, br) in enumerate(((rg[1], rg[2]), (rg[3], rg[4]), (rg[5], rg[6]))):      # parameters() order: W_z, W_r, W_h (weight, bias)
        assert torch.allclose(gW[k], wr, rtol=1e-4, atol=1e-5 * float(wr.abs().max())), k
        assert torch.allclose(gb[k], br, rtol=1e-4, atol=1e-5 * float(br.abs().max())), k


def test_soft_head_with_native_tail_matches_torch_tail(monkeypatch):
    from supergrok15_b200 import _build
    if not _build.native_available():
        pytest.skip("native extension not built")
    torch.manual_seed(4)
    mn = Mamba3PEERMetaNet()
    with torch.no_grad():
        mn.expert_W1.mul_(30); mn.expert_W2.mul_(30)
        for k in list(mn.product_keys_A) + list(mn.product_keys_B):
            k.mul_(10)
    n = 300
    g, s = torch.randn(n) * 1e-2, torch.rand(n) * 1e-2
    gru, vu = torch.randn(n, mn.gru_hidden) * 0.1, torch.randn(n)
    ctx = (torch.randn(n, 16) * 0.1).requires_grad_(True)
    res = {}
    for mode in ("torch", "native"):                             # native: GRU and routing through their C++ / CUDA implementations
        monkeypatch.setenv("SG_BILEVEL_TAIL", mode)
        mn.zero_grad(set_to_none=True)
        ctx.grad = None
        (mn.soft_head(g, s, gru, ctx[:, :8], ctx[:, 8:]) * vu).sum().backward()
        res[mode] = (ctx.grad.clone(), {k: p.grad.clone() for k, p in mn.named_parameters() if p.grad is not None})
    assert torch.allclose(res["native"][0], res["torch"][0], rtol=1e-3, atol=1e-7)
    assert set(res["native"][1]) == set(res["torch"][1])
    for k, gt in res["torch"][1].items():
        assert (res["native"][1][k] - gt).abs().max() <= 1e-3 * gt.abs().max() + 1e-9, k


def test_grad_sink_linear_adds_into_existing_grads():
    """``nn_ops.linear`` inside ``grad_sink``: weight and bias gradients are added to the tensors already in ``.grad`` and autograd
    receives None for them; outside the block (or without a ``.grad``) it is plain ``F.linear``."""
    from supergrok15_b200.ops import nn_ops
    torch.manual_seed(0)
    w = torch.randn(6, 5, requires_grad=True)
    b = torch.randn(6, requires_grad=True)
    x = torch.randn(3, 4, 5, requires_grad=True)
    (F.linear(x, w, b) ** 2).sum().backward()
    gw, gb, gx = w.grad.clone(), b.grad.clone(), x.grad.clone()
    w.grad, b.grad, x.grad = torch.ones_like(w), torch.ones_like(b), None
    held = (w.grad, b.grad)
    with nn_ops.grad_sink(True):
        (nn_ops.linear(x, w, b) ** 2).sum().backward()
    assert w.grad is held[0] and b.grad is held[1]
    assert torch.allclose(w.grad, gw + 1, atol=1e-5) and torch.allclose(b.grad, gb + 1, atol=1e-5) and torch.allclose(x.grad, gx, atol=1e-5)
    w.grad, b.grad, x.grad = None, None, None
    with nn_ops.grad_sink(True):                                    # no .grad to add to: autograd's own path
        (nn_ops.linear(x, w, b) ** 2).sum().backward()
    assert torch.allclose(w.grad, gw, atol=1e-5) and torch.allclose(b.grad, gb, atol=1e-5)


def test_grad_sink_restores_its_state_on_exit_and_on_error():
    """``grad_sink`` blocks nest and always restore the previous state, also when the body raises: a failed step must not leave later
    backward passes writing gradients in place."""
    from supergrok15_b200.ops import nn_ops
    assert not nn_ops._SINK.on
    with nn_ops.grad_sink(True):
        assert nn_ops._SINK.on
        with nn_ops.grad_sink(False):
            assert not nn_ops._SINK.on
        assert nn_ops._SINK.on
        with pytest.raises(RuntimeError):
            with nn_ops.grad_sink(True):
                raise RuntimeError("step failed")
        assert nn_ops._SINK.on
    assert not nn_ops._SINK.on and nn_ops._SINK.stream is None and nn_ops._SINK.keep == []
    w = torch.randn(3, 2, requires_grad=True)
    w.grad = torch.zeros_like(w)
    x = torch.randn(4, 2)
    nn_ops.linear(x, w).sum().backward()                          # outside a block: autograd accumulates as usual
    assert torch.allclose(w.grad, x.sum(0).expand(3, 2))
