"""Race driver: data generators, every registry entry end to end on a tiny model, JSON schema, status server."""
import json
import urllib.request

import pytest
import torch

from supergrok15_b200 import race
from supergrok15_b200.race import status
from supergrok15_b200.race.config import ALL_OPTIMIZERS, RaceConfig

TINY = dict(dim_model=32, num_heads=2, num_layers=1, max_steps=4, log_every=2, p=11, num_tokens=13, early_stop_patience=2)


def test_data_generators():
    tx, ty, vx, vy = race.make_data(97, 0.5, 42)
    assert tx.shape == (4656, 4) and vx.shape == (4656, 4) and int(tx[:, 1].unique()) == 97 and int(tx[:, 3].unique()) == 98
    a, b = int(tx[0, 0]), int(tx[0, 2])
    assert (int(ty[0]) * b) % 97 == a                       # label = a / b mod p
    ax, ay, _, _ = race.make_addition_data(97, 0.5, 0)
    assert ax.shape == (4704, 4) and int(ay[5]) == (int(ax[5, 0]) + int(ax[5, 2])) % 97
    sx, sy, _, _ = race.make_sequential_division_data(11, 3, 0.5, 1)
    assert sx.shape[1] == 8 and sx.shape[0] == 55
    mx, my, _, _ = race.make_mnist_addition_data(7, 0.5, 1)
    assert mx.shape[1:] == (16, 49)
    assert torch.equal(race.make_data(97, 0.5, 42)[0], tx)  # deterministic in the seed


@pytest.mark.parametrize("name", ALL_OPTIMIZERS)
def test_every_registry_entry_trains(name, tmp_path):
    rbo = race.run_pipeline(dict(TINY), optimizers=[name], seeds=[1], device="cpu", save_dir=str(tmp_path), plot=False, verbose=False)
    r = rbo[name][0]
    assert r.total_steps == 4 and len(r.steps) >= 1 and all(isinstance(v, float) for v in r.val_accs)
    d = json.load(open(tmp_path / "results_decoder_ft50.json"))
    assert set(d["_meta"]) >= {"total_wall", "model_type", "frac_train"}
    assert set(d[name][0]) >= {"seed", "steps", "train_losses", "train_accs", "val_losses", "val_accs", "wall_time", "total_steps",
                               "grokking_step", "grokking_wall", "final_val_acc", "final_train_acc", "model_type", "frac_train"}


def test_architectures_and_compat_flag(tmp_path):
    for mt in ("decoder_preln", "mamba", "vit"):
        cfg = dict(TINY, model_type=mt, p=7, num_tokens=9)
        rbo = race.run_pipeline(cfg, optimizers=["adamw"], seeds=[1], device="cpu", save_dir=None, verbose=False)
        assert rbo["adamw"][0].total_steps == 4
    cfg = dict(TINY, reference_compat=True, max_steps=25, supergrok15_sam_freq_max=3, supergrok15_sam_freq_min=3)
    rbo = race.run_pipeline(cfg, optimizers=["supergrok15"], seeds=[1], device="cpu", save_dir=None, verbose=False)
    assert any("sam_step failed" in e for e in rbo["supergrok15"][0].events)     # recorded, not silenced


def test_status_server_and_config():
    status.reset(3)
    status.update("adamw", 1, 10, 0.5, 0.1, 1.0, 2.0)
    status.job_done("adamw", 1, {"grok": None})
    srv = status.start_status_server(0)
    port = srv.server_address[1]
    s = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/status", timeout=5).read())
    srv.shutdown()
    assert s["total_jobs"] == 3 and s["done_jobs"] == 1 and "eta_s" in s
    c = RaceConfig(model_scale="medium", dtype="bf16").flat()
    assert c["dim_model"] == 256 and c["use_amp"] and c["max_steps"] == 20000
    assert not status.ntfy(None, "x")


def test_reference_import_surface():
    import grokking_optimizers as go
    from grokking_optimizers.supergrok2 import SuperGrok2
    from grokking_optimizers.mamba3_peer_metanet import Mamba3PEERMetaNet  # noqa: F401
    assert go.__version__ == "2.0.0" and go.SuperGrok2 is SuperGrok2
    for n in ("SuperGrok15", "SuperGrok11", "GrokAdamW", "NeuralGrok", "Prodigy", "Grokfast", "Lion", "LookSAM", "Muon",
              "CUDAGraphOptimizer", "SharpnessMetaNet"):
        assert hasattr(go, n)


def test_resume_skips_finished_jobs(tmp_path):
    """An interrupted race picks up where it stopped: finished (optimizer, seed) jobs come from the progress file."""
    from supergrok15_b200.race import runner
    base = dict(dim_model=32, num_heads=2, num_layers=1, max_steps=30, p=23, log_every=10)
    kw = dict(save_dir=str(tmp_path), plot=False, verbose=False, device="cpu")
    first = runner.run_pipeline(base, optimizers=["adamw"], seeds=[1, 2], **kw)
    assert len(first["adamw"]) == 2
    calls = []
    orig = runner._run_one

    def spy(name, seed, *a, **k):
        calls.append((name, seed))
        return orig(name, seed, *a, **k)
    runner._run_one = spy
    try:
        again = runner.run_pipeline(base, optimizers=["adamw", "lion"], seeds=[1, 2], resume=True, **kw)
    finally:
        runner._run_one = orig
    assert calls == [("lion", 1), ("lion", 2)]                       # the two AdamW jobs were not run again
    assert len(again["adamw"]) == 2 and len(again["lion"]) == 2
    assert again["adamw"][0].train_losses == first["adamw"][0].train_losses
    assert runner.main(["--no-status-server", "--optimizers", "adamw", "--seeds", "1", "--max-steps", "5", "--save-dir", str(tmp_path / "cli"),
                        "--resume"]) == 0


def test_ntfy_status_query_is_answered_with_the_progress_report():
    from supergrok15_b200.race import status
    status.reset(4)
    status.job_done("adamw", 1, {"grok": 120})
    status.job_done("lion", 1, {"grok": None})
    sent = []
    line = b'{"event": "message", "message": " Status "}'
    assert status.handle_ntfy_line("topic", line, send=lambda t, m, title: sent.append((t, m, title)))
    assert sent and "2/4 runs complete" in sent[0][1] and "1 grokked | 1 DNF" in sent[0][1]
    assert not status.handle_ntfy_line("topic", b'{"event": "message", "message": "hello"}', send=lambda *a: sent.append(a))
    assert not status.handle_ntfy_line("topic", b'{"event": "open"}') and status.start_ntfy_listener(None) is None


def test_grouped_bar_chart(tmp_path):
    from supergrok15_b200.race.plots import plot_grouped_bars
    ok = plot_grouped_bars({"25% train": {"adamw": 900.0, "lion": 700.0}, "50% train": {"adamw": 400.0, "lion": 350.0}}, "steps to grok",
                           str(tmp_path / "bars.png"))
    assert ok is False or (tmp_path / "bars.png").stat().st_size > 0       # False only when matplotlib is not installed
