"""Data generators of the race (reference grokking_race_v2.py:231-307) plus modular addition on token sequences."""
from __future__ import annotations

import random
from typing import Tuple

import torch

Split = Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]


def _split(rows, labels, frac_train, rng) -> Split:
    c = list(zip(rows, labels))
    rng.shuffle(c)
    rows, labels = zip(*c)
    n = int(len(rows) * frac_train)
    x = torch.tensor(rows, dtype=torch.long)
    y = torch.tensor(labels, dtype=torch.long)
    return x[:n], y[:n], x[n:], y[n:]


def make_data(p: int = 97, frac_train: float = 0.5, seed: int = 42) -> Split:
    """(a / b) mod p for all a and all b != 0, as sequences [a, p, b, p+1]."""
    rng = random.Random(seed)
    rows, labels = [], []
    for a in range(p):
        for b in range(1, p):
            rows.append([a, p, b, p + 1])
            labels.append((a * pow(b, p - 2, p)) % p)
    return _split(rows, labels, frac_train, rng)


def make_addition_data(p: int = 97, frac_train: float = 0.5, seed: int = 0) -> Split:
    """(a + b) mod p for all p*p pairs, as sequences [a, p, b, p+1] (vocabulary p + 2)."""
    rng = random.Random(seed)
    rows, labels = [], []
    for a in range(p):
        for b in range(p):
            rows.append([a, p, b, p + 1])
            labels.append((a + b) % p)
    return _split(rows, labels, frac_train, rng)


def make_sequential_division_data(p: int = 97, chain_length: int = 3, frac_train: float = 0.5, seed: int = 42) -> Split:
    """a / b1 / b2 / ... mod p on p*(p-1) distinct random chains: [a, p, b1, p, b2, ..., p+1]."""
    rng = random.Random(seed)
    target = p * (p - 1)
    seen, rows, labels = set(), [], []
    while len(rows) < target:
        a = rng.randint(0, p - 1)
        bs = tuple(rng.randint(1, p - 1) for _ in range(chain_length))
        if (a, *bs) in seen:
            continue
        seen.add((a, *bs))
        res = a
        for b in bs:
            res = (res * pow(b, p - 2, p)) % p
        seq = [a]
        for b in bs:
            seq.extend([p, b])
        seq.append(p + 1)
        rows.append(seq)
        labels.append(res)
    return _split(rows, labels, frac_train, rng)


def _digit_glyphs(rng: random.Random):
    """14x14 digit images.  MNIST through torchvision when it is installed and already on disk; otherwise seeded
    synthetic glyphs (a fixed random 14x14 prototype per digit plus noise), so the ViT task runs offline."""
    try:
        import torchvision
        from torchvision import transforms
        tf = transforms.Compose([transforms.Resize((14, 14)), transforms.ToTensor()])
        mnist = torchvision.datasets.MNIST(root="./data", train=True, download=False, transform=tf)
        by_digit = {d: [] for d in range(10)}
        for img, label in mnist:
            if len(by_digit[label]) < 64:
                by_digit[label].append(img.squeeze(0))
        return by_digit
    except Exception:  # noqa: BLE001
        g = torch.Generator().manual_seed(rng.randint(0, 2 ** 31 - 1))
        protos = (torch.rand(10, 14, 14, generator=g) > 0.6).float()
        return {d: [(protos[d] + 0.1 * torch.randn(14, 14, generator=g)).clamp(0, 1) for _ in range(8)] for d in range(10)}


def make_mnist_addition_data(p: int = 97, frac_train: float = 0.5, seed: int = 42) -> Split:
    """(a + b) mod p where a and b are shown as two-digit images; 16 patches of 7x7 pixels per sample."""
    rng = random.Random(seed)
    glyphs = _digit_glyphs(rng)
    number_images = {}
    for n in range(p):
        t, o = divmod(n, 10)
        number_images[n] = torch.cat([rng.choice(glyphs[t]), rng.choice(glyphs[o])], dim=1)      # [14, 28]
    pairs, labels = [], []
    for a in range(p):
        for b in range(p):
            pairs.append((a, b))
            labels.append((a + b) % p)
    c = list(zip(pairs, labels))
    rng.shuffle(c)
    pairs, labels = zip(*c)
    n_split = int(len(pairs) * frac_train)
    imgs = []
    for a, b in pairs:
        full = torch.cat([number_images[a], number_images[b]], dim=0)                           # [28, 28]
        imgs.append(full.unfold(0, 7, 7).unfold(1, 7, 7).contiguous().reshape(16, 49))
    x = torch.stack(imgs)
    y = torch.tensor(labels, dtype=torch.long)
    return x[:n_split], y[:n_split], x[n_split:], y[n_split:]


def make_data_for_task(c: dict, seed: int) -> Split:
    mt, ft, p = c.get("model_type", "decoder"), c.get("frac_train", 0.5), c.get("p", 97)
    if mt in ("decoder", "decoder_preln"):
        if c.get("task", "division") == "addition":
            return make_addition_data(p, ft, seed)
        return make_data(p, ft, seed)
    if mt == "vit":
        return make_mnist_addition_data(p, ft, seed)
    if mt == "mamba":
        return make_sequential_division_data(p, c.get("chain_length", 3), ft, seed)
    raise ValueError(f"Unknown model_type: {mt}")
