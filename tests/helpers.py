"""Shared fixtures: tiny parameter sets with seeded gradients, CPU/CUDA twins."""
import copy

import torch


def make_params(shapes, dtype=torch.float32, device="cpu", seed=0, grad_scale=1e-2):
    g = torch.Generator().manual_seed(seed)
    ps = []
    for s in shapes:
        p = torch.nn.Parameter((torch.randn(s, generator=g) * 0.1).to(dtype).to(device))
        p.grad = (torch.randn(s, generator=g) * grad_scale).to(dtype).to(device)
        ps.append(p)
    return ps


def set_grads(ps, seed, grad_scale=1e-2):
    g = torch.Generator().manual_seed(seed)
    for p in ps:
        p.grad = (torch.randn(p.shape, generator=g) * grad_scale).to(p.dtype).to(p.device)


EDGE_SHAPES = [(1,), (2,), (15,), (16, 1), (17,), (255,), (256,), (257,), (511,), (32, 16), (513,), (1023,), (1024,),
               (4097,), (8192,), (8193,), (3, 5, 7)]


def tol(dtype):
    return {torch.float32: (2e-5, 1e-6), torch.bfloat16: (2e-2, 2e-3), torch.float16: (4e-3, 4e-4)}[dtype]
