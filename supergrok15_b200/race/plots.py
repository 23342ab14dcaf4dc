"""Plots of a race (curves with mean +- std over seeds, race bars, split / architecture heat maps; reference
grokking_race_v2.py:965-1039, 1359-1478).  matplotlib with the CPU ``Agg`` backend when it is installed; otherwise the
functions return False and the JSON results remain the record."""
from __future__ import annotations

import os
from typing import Dict, List

import numpy as np

from .config import DISPLAY_NAMES

COLORS = {"adamw": "#1f77b4", "grokadamw": "#ff7f0e", "neuralgrok": "#2ca02c", "supergrok11": "#d62728", "supergrok15": "#9467bd",
          "supergrok2": "#8c564b", "grokfast": "#7f7f7f", "muon": "#17a2b8", "lion": "#e377c2", "looksam": "#bcbd22", "prodigy": "#17becf"}


def _plt():
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        return plt
    except Exception:  # noqa: BLE001
        return None


def ema(xs: List[float], a: float = 0.92) -> List[float]:
    out, m = [], None
    for x in xs:
        m = x if m is None else a * m + (1 - a) * x
        out.append(m)
    return out


def plot_comparison(rbo: Dict[str, list], save_dir: str = "results", tag: str = "") -> bool:
    plt = _plt()
    if plt is None:
        return False
    os.makedirs(save_dir, exist_ok=True)
    fig, axes = plt.subplots(1, 3, figsize=(18, 5))
    for name, runs in rbo.items():
        col = COLORS.get(name)
        n = min(len(r.steps) for r in runs) if runs else 0
        if n == 0:
            continue
        steps = runs[0].steps[:n]
        for ax, key in ((axes[0], "val_accs"), (axes[1], "train_accs")):
            arr = np.array([ema(getattr(r, key)[:n]) for r in runs])
            mu, sd = arr.mean(0), arr.std(0)
            ax.plot(steps, mu, label=DISPLAY_NAMES.get(name, name), color=col)
            ax.fill_between(steps, mu - sd, mu + sd, color=col, alpha=0.15)
    axes[0].set_title("validation accuracy"); axes[1].set_title("train accuracy")
    for ax in axes[:2]:
        ax.set_xscale("log"); ax.set_xlabel("step"); ax.legend(fontsize=7)
    names = list(rbo)
    walls = [np.mean([r.grokking_wall or r.wall_time for r in rbo[k]]) for k in names]
    axes[2].barh([DISPLAY_NAMES.get(k, k) for k in names], walls, color=[COLORS.get(k) for k in names])
    axes[2].set_title("wall-clock to grok (s)")
    fig.tight_layout()
    fig.savefig(os.path.join(save_dir, f"race{tag}.png"), dpi=120)
    plt.close(fig)
    return True


def plot_heatmap(table: Dict[str, Dict[str, float]], title: str, path: str) -> bool:
    """table[row][col] -> value (e.g. optimizer x train split -> steps to grok)."""
    plt = _plt()
    if plt is None:
        return False
    rows = list(table)
    cols = list(next(iter(table.values()))) if rows else []
    arr = np.array([[table[r].get(c, np.nan) for c in cols] for r in rows], dtype=float)
    fig, ax = plt.subplots(figsize=(1.5 * len(cols) + 3, 0.5 * len(rows) + 2))
    im = ax.imshow(arr, aspect="auto", cmap="viridis_r")
    ax.set_xticks(range(len(cols))); ax.set_xticklabels(cols)
    ax.set_yticks(range(len(rows))); ax.set_yticklabels([DISPLAY_NAMES.get(r, r) for r in rows])
    ax.set_title(title)
    fig.colorbar(im)
    fig.tight_layout()
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    fig.savefig(path, dpi=120)
    plt.close(fig)
    return True


def plot_grouped_bars(table: Dict[str, Dict[str, float]], title: str, path: str) -> bool:
    """One group of bars per row of ``table`` (train split or architecture), one bar per optimizer
    (reference grokking_race_v2.py:1359-1478)."""
    plt = _plt()
    if plt is None or not table:
        return False
    groups = list(table)
    names = sorted({n for row in table.values() for n in row})
    fig, ax = plt.subplots(figsize=(max(6, 1.2 * len(groups) * max(len(names), 1) / 3), 4))
    w = 0.8 / max(len(names), 1)
    for k, n in enumerate(names):
        ax.bar([g + k * w for g in range(len(groups))], [table[g].get(n, 0.0) for g in groups], width=w, label=n)
    ax.set_xticks([g + 0.4 - w / 2 for g in range(len(groups))])
    ax.set_xticklabels(groups)
    ax.set_ylabel("steps")
    ax.set_title(title)
    ax.legend(fontsize=7, ncol=2)
    fig.tight_layout()
    fig.savefig(path, dpi=120)
    plt.close(fig)
    return True
