"""Device-timed micro-benchmarks of the decoder kernels against their PyTorch counterparts (1 GPU).

    python -m supergrok15_b200.ops.bench_nn --what flash            # tcgen05 flash attention fwd / bwd vs F.scaled_dot_product_attention
    python -m supergrok15_b200.ops.bench_nn --what ce               # fused cross-entropy fwd / bwd vs F.cross_entropy
    python -m supergrok15_b200.ops.bench_nn --what norm             # RMSNorm with fused residual vs F.rms_norm(x + r)
    python -m supergrok15_b200.ops.bench_nn --what linear           # tcgen05 Linear (forward, dgrad, wgrad) vs cuBLAS on the flagship's layer shapes
    python -m supergrok15_b200.ops.bench_nn --what small_ops        # GELU, bias-gradient column sums, small-table embedding gradient, LayerNorm backward
    ... --what linear --kernels                                      # plus the device time of every kernel of one autograd call
    ... --small                                                      # one modest shape, few iterations (profiler captures)

Timing: CUDA events on the launching stream after warm-up; every shape's working set exceeds the 126 MB L2 except with --small.
Prints one JSON line per measurement.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.nn.functional as F


def timed(fn, it, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(it):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / it


def bench_flash(small: bool, it: int):
    from .. import _build
    from . import gemm, nn_ops
    C = _build.require()
    dev = torch.device("cuda:0")
    shapes = [(4, 1024, 8, 128)] if small else [(8, 2048, 16, 128), (4, 4096, 16, 128), (8, 2048, 32, 64)]
    for B, S, H, HD in shapes:
        q, k, v = (torch.randn(B, S, H, HD, device=dev).to(torch.bfloat16).requires_grad_(True) for _ in range(3))
        do = torch.randn(B, S, H, HD, device=dev).to(torch.bfloat16)
        err = gemm._err_flag(dev)
        out, lse = C.flash_fwd(q, k, v, True, err)
        t_f = timed(lambda: C.flash_fwd(q, k, v, True, err), it)
        t_b = timed(lambda: C.flash_bwd(q, k, v, out, lse, do, True, err), it)
        o2 = nn_ops.attention_reference(q, k, v, True)
        t_rf = timed(lambda: nn_ops.attention_reference(q, k, v, True), it)
        t_rb = timed(lambda: torch.autograd.grad(o2, (q, k, v), do, retain_graph=True), it)
        gemm.check(dev)
        fl = 4.0 * B * H * S * S * HD / 2                      # causal forward FLOPs; backward = 2.5x
        print(json.dumps({"kernel": "flash_attention_causal", "B": B, "S": S, "H": H, "hd": HD, "fwd_ms": t_f, "fwd_tflops": fl / t_f / 1e9,
                          "bwd_ms": t_b, "bwd_tflops": 2.5 * fl / t_b / 1e9, "sdpa_fwd_ms": t_rf, "sdpa_bwd_ms": t_rb}), flush=True)


def bench_ce(small: bool, it: int):
    from . import nn_ops
    dev = torch.device("cuda:0")
    rows, V = (4096, 32000) if small else (16384, 32000)
    x = (torch.randn(rows, V, device=dev) * 2).to(torch.bfloat16).requires_grad_(True)
    t = torch.randint(0, V, (rows,), device=dev)

    def own():
        x.grad = None
        nn_ops.cross_entropy(x, t).backward()

    def ref():
        x.grad = None
        F.cross_entropy(x.float(), t).backward()
    t_o, t_r = timed(own, it), timed(ref, it)
    by = rows * V * 2 * 3                                       # logits read twice, gradient written once
    print(json.dumps({"kernel": "cross_entropy_fwd_bwd", "rows": rows, "V": V, "ms": t_o, "GBps": by / t_o / 1e6, "torch_ms": t_r}), flush=True)


def bench_norm(small: bool, it: int):
    from . import nn_ops
    dev = torch.device("cuda:0")
    rows, D = (16384, 2048) if small else (65536, 2048)
    x = torch.randn(rows, D, device=dev).to(torch.bfloat16).requires_grad_(True)
    r = torch.randn(rows, D, device=dev).to(torch.bfloat16).requires_grad_(True)
    w = torch.ones(D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(rows, D, device=dev).to(torch.bfloat16)

    def own():
        y, z = nn_ops.norm_residual(x, r, w, None, 1e-5, rms=True)
        torch.autograd.grad((y, z), (x, r, w), (g, g))

    def ref():
        z = x + r
        y = F.rms_norm(z, (D,), w, 1e-5)
        torch.autograd.grad((y, z), (x, r, w), (g, g))
    t_o, t_r = timed(own, it), timed(ref, it)
    by = rows * D * 2 * (4 + 4)                                 # fwd: x, r in, y, z out; bwd: z, dy, dz_in in, dz out
    print(json.dumps({"kernel": "rmsnorm_residual_fwd_bwd", "rows": rows, "D": D, "ms": t_o, "GBps": by / t_o / 1e6, "torch_ms": t_r}), flush=True)


def bench_linear(small: bool, it: int):
    """Forward, dgrad and wgrad GEMMs of a Linear layer on the tcgen05 kernel (dgrad / wgrad read W, dy and x in place through
    MN-major descriptors) against torch.matmul (cuBLAS), then the whole autograd function against F.linear.  Four sets of
    operands are used in rotation so that consecutive calls do not find their inputs in L2."""
    from . import gemm
    dev = torch.device("cuda:0")
    T = 8192 if small else 32768
    for din, dout in ([(512, 1536)] if small else [(512, 1536), (512, 512), (512, 2048), (2048, 512)]):
        sets = [(torch.randn(T, din, device=dev).to(torch.bfloat16), (torch.randn(dout, din, device=dev) * 0.05).to(torch.bfloat16),
                 torch.randn(T, dout, device=dev).to(torch.bfloat16)) for _ in range(4)]
        k = [0]

        def nxt():
            k[0] = (k[0] + 1) % len(sets)
            return sets[k[0]]

        def run(fn):
            return timed(lambda: fn(*nxt()), it)
        r = {"kernel": "linear_gemms", "tokens": T, "in": din, "out": dout}
        r["fwd_us"] = 1e3 * run(lambda x, w, dy: gemm.gemm_tn(x, w))
        r["dgrad_us"] = 1e3 * run(lambda x, w, dy: gemm.gemm_tn(dy, w, b_t=True))
        r["wgrad_us"] = 1e3 * run(lambda x, w, dy: gemm.gemm_tn(dy, x, a_t=True, b_t=True))
        r["cublas_fwd_us"] = 1e3 * run(lambda x, w, dy: x @ w.t())
        r["cublas_dgrad_us"] = 1e3 * run(lambda x, w, dy: dy @ w)
        r["cublas_wgrad_us"] = 1e3 * run(lambda x, w, dy: dy.t() @ x)
        bias = torch.zeros(dout, device=dev, dtype=torch.bfloat16, requires_grad=True)

        def auto(lin):
            def f(x, w, dy):
                x.requires_grad_(True), w.requires_grad_(True)
                torch.autograd.grad(lin(x, w, bias), (x, w, bias), dy)
            return f
        r["autograd_us"] = 1e3 * run(auto(gemm.linear))
        r["cublas_autograd_us"] = 1e3 * run(auto(F.linear))
        if KERNELS:                                                  # device time of every kernel of one forward + backward of the layer
            from torch.profiler import ProfilerActivity, profile
            fn = auto(gemm.linear)
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for _ in range(3):
                    fn(*nxt())
                torch.cuda.synchronize()
            rows = sorted((e for e in prof.key_averages() if e.device_time_total > 0), key=lambda e: -e.device_time_total)
            r["autograd_kernels_us"] = [[e.key[:60], round(e.device_time_total / 3, 1), e.count // 3] for e in rows[:10]]
        gemm.check(dev)
        fl = 2.0 * T * din * dout
        r["fwd_tflops"], r["dgrad_tflops"], r["wgrad_tflops"] = (fl / r[k_] / 1e6 for k_ in ("fwd_us", "dgrad_us", "wgrad_us"))
        print(json.dumps({k_: (round(v, 1) if isinstance(v, float) else v) for k_, v in r.items()}), flush=True)


KERNELS = False


def bench_small_ops(small: bool, it: int):
    """The memory-bound kernels around the flagship decoder's GEMMs (32,768 tokens, d512, mlp 2048, 115 tokens in the table)."""
    from . import nn_ops
    from .. import _build
    C = _build.require()
    dev = torch.device("cuda:0")
    rows, D, F4, V = (4096 if small else 32768), 512, 2048, 115
    h = torch.randn(rows, F4, device=dev).to(torch.bfloat16).requires_grad_(True)
    g = torch.randn(rows, F4, device=dev).to(torch.bfloat16)
    for name, fn in (("gelu_own", nn_ops.gelu), ("gelu_torch", F.gelu)):
        t_f = timed(lambda: fn(h), it)
        y = fn(h)
        t_b = timed(lambda: torch.autograd.grad(y, h, g, retain_graph=True), it)
        print(json.dumps({"kernel": name, "rows": rows, "C": F4, "fwd_ms": t_f, "bwd_ms": t_b, "fwd_GBps": rows * F4 * 4 / t_f / 1e6,
                          "bwd_GBps": rows * F4 * 6 / t_b / 1e6}), flush=True)
    out = torch.empty_like(g)
    t_c = timed(lambda: out.copy_(g), it)
    t_a = timed(lambda: torch.add(g, 1.0, out=out), it)
    print(json.dumps({"kernel": "torch_copy_and_add_same_shape", "rows": rows, "C": F4, "copy_ms": t_c, "copy_GBps": rows * F4 * 4 / t_c / 1e6,
                      "add_ms": t_a, "add_GBps": rows * F4 * 4 / t_a / 1e6}), flush=True)
    for Cw in (D, 3 * D, F4):
        dy = torch.randn(rows, Cw, device=dev).to(torch.bfloat16)
        t_o, t_r = timed(lambda: C.col_sum(dy), it), timed(lambda: dy.sum(0), it)
        print(json.dumps({"kernel": "col_sum", "rows": rows, "C": Cw, "ms": t_o, "GBps": rows * Cw * 2 / t_o / 1e6, "torch_ms": t_r}), flush=True)
    ids = torch.randint(0, V, (rows // 4, 4), device=dev)
    W = torch.randn(V, D, device=dev).to(torch.bfloat16).requires_grad_(True)
    dout = torch.randn(rows // 4, 4, D, device=dev).to(torch.bfloat16)
    t_o = timed(lambda: C.embedding_bwd(ids, dout, V), it)
    e = F.embedding(ids, W)
    t_r = timed(lambda: torch.autograd.grad(e, W, dout, retain_graph=True), it)
    print(json.dumps({"kernel": "embedding_bwd_small_table", "tokens": rows, "V": V, "D": D, "ms": t_o, "torch_ms": t_r}), flush=True)
    x = torch.randn(rows, D, device=dev).to(torch.bfloat16).requires_grad_(True)
    r = torch.randn(rows, D, device=dev).to(torch.bfloat16).requires_grad_(True)
    w = torch.ones(D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    b = torch.zeros(D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(rows, D, device=dev).to(torch.bfloat16)
    y = nn_ops.layer_norm(x, r, w, b)
    t_o = timed(lambda: torch.autograd.grad(y, (x, r, w, b), gy, retain_graph=True), it)
    y2 = F.layer_norm(x + r, (D,), w, b)
    t_r = timed(lambda: torch.autograd.grad(y2, (x, r, w, b), gy, retain_graph=True), it)
    print(json.dumps({"kernel": "layernorm_residual_bwd", "rows": rows, "D": D, "ms": t_o, "torch_ms": t_r}), flush=True)


def main():
    global KERNELS
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernels", action="store_true", help="linear: also list the device time of every kernel of one autograd call (torch.profiler)")
    ap.add_argument("--what", default="flash", choices=["flash", "ce", "norm", "linear", "small_ops", "all"])
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=None)
    a = ap.parse_args()
    KERNELS = a.kernels
    it = a.iters or (2 if a.small else 20)
    for name, fn in (("flash", bench_flash), ("ce", bench_ce), ("norm", bench_norm), ("linear", bench_linear), ("small_ops", bench_small_ops)):
        if a.what in (name, "all"):
            fn(a.small, it)


if __name__ == "__main__":
    main()
