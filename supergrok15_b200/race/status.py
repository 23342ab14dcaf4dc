"""Progress bookkeeping and the optional observers of a race: HTTP ``GET /status`` (JSON with ETA) and ntfy push
(reference grokking_race_v2.py:87-203).  Both are off unless asked for; nothing here is needed for a benchmark."""
from __future__ import annotations

import json
import threading
import time
from http.server import BaseHTTPRequestHandler, HTTPServer
from typing import Optional

_LOCK = threading.Lock()
PROGRESS = {"started": None, "phase": "idle", "total_jobs": 0, "done_jobs": 0, "current": {}, "errors": [], "results": {}}


def reset(total_jobs: int, phase: str = "running") -> None:
    with _LOCK:
        PROGRESS.update(started=time.time(), phase=phase, total_jobs=total_jobs, done_jobs=0, current={}, errors=[], results={})


def update(name: str, seed: int, step: int, train_acc: float, val_acc: float, train_loss: float, val_loss: float) -> None:
    with _LOCK:
        PROGRESS["current"][f"{name}/{seed}"] = {"step": step, "train_acc": train_acc, "val_acc": val_acc, "train_loss": train_loss,
                                                 "val_loss": val_loss, "t": time.time()}


def job_done(name: str, seed: int, summary: Optional[dict] = None, error: Optional[str] = None) -> None:
    with _LOCK:
        PROGRESS["done_jobs"] += 1
        PROGRESS["current"].pop(f"{name}/{seed}", None)
        if error:
            PROGRESS["errors"].append({"job": f"{name}/{seed}", "error": error})
        if summary:
            PROGRESS["results"][f"{name}/{seed}"] = summary


def snapshot() -> dict:
    with _LOCK:
        s = json.loads(json.dumps(PROGRESS))
    if s["started"] and s["done_jobs"]:
        el = time.time() - s["started"]
        s["elapsed_s"] = el
        s["eta_s"] = el / s["done_jobs"] * max(s["total_jobs"] - s["done_jobs"], 0)
    return s


class _Handler(BaseHTTPRequestHandler):
    def do_GET(self):  # noqa: N802
        if self.path.rstrip("/") in ("/status", ""):
            body = json.dumps(snapshot()).encode()
            self.send_response(200)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)
        else:
            self.send_response(404)
            self.end_headers()

    def log_message(self, *a):  # silence
        pass


def start_status_server(port: int = 8765, host: str = "127.0.0.1") -> HTTPServer:
    srv = HTTPServer((host, port), _Handler)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv


def ntfy(topic: Optional[str], message: str, title: str = "grokking race") -> bool:
    """Push a notification to ntfy.sh/<topic>; a no-op without a topic, without `requests` or without network."""
    if not topic:
        return False
    try:
        import requests
        requests.post(f"https://ntfy.sh/{topic}", data=message.encode(), headers={"Title": title}, timeout=5)
        return True
    except Exception:  # noqa: BLE001
        return False


def status_text(snap: Optional[dict] = None) -> str:
    """Progress report as the reply to a "status" query (reference grokking_race_v2.py:176-193)."""
    s = snap or snapshot()
    res = s.get("results", {})
    grokked = sum(1 for r in res.values() if r and r.get("grok") is not None)
    lines = [f"{s['done_jobs']}/{s['total_jobs']} runs complete", f"{grokked} grokked | {len(res) - grokked} DNF | {len(s['errors'])} errors"]
    if "elapsed_s" in s:
        lines.append(f"elapsed {int(s['elapsed_s'])} s, ETA {int(s['eta_s'])} s")
    if s.get("current"):
        lines.append("current: " + ", ".join(f"{k} step {v['step']} val {v['val_acc']:.3f}" for k, v in list(s["current"].items())[:4]))
    return "\n".join(lines)


QUERIES = ("status", "progress", "update", "?", "eta")


def handle_ntfy_line(topic: str, line: bytes, send=None) -> bool:
    """One line of the topic's JSON stream: a message whose text is one of QUERIES is answered with the progress report."""
    try:
        msg = json.loads(line)
    except Exception:  # noqa: BLE001
        return False
    if msg.get("event") != "message" or msg.get("message", "").strip().lower() not in QUERIES:
        return False
    (send or ntfy)(topic, status_text(), "Progress Report")
    return True


def start_ntfy_listener(topic: Optional[str]) -> Optional[threading.Thread]:
    """Listen on ntfy.sh/<topic>/json and answer "status" / "progress" / "eta" / "?" with the progress report
    (reference grokking_race_v2.py:161-203).  Without a topic, without `requests` or without network it does nothing."""
    if not topic:
        return None

    def listen():
        try:
            import requests
        except Exception:  # noqa: BLE001
            return
        while True:
            try:
                r = requests.get(f"https://ntfy.sh/{topic}/json", stream=True, timeout=600)
                for line in r.iter_lines():
                    if line:
                        handle_ntfy_line(topic, line)
            except Exception:  # noqa: BLE001
                time.sleep(10)                        # reconnect
    t = threading.Thread(target=listen, daemon=True)
    t.start()
    return t
