"""Terminal dashboard: ``legion top`` (poll a server's ``/v1/stats``) and ``serve --tui`` (same view in the
server's own terminal). Plain ANSI, no curses dependency (``src/dashboard/*`` is a ratatui TUI in the reference)."""
from __future__ import annotations

import json
import sys
import threading
import time
import urllib.request
from typing import Optional


def bar(frac: float, width: int = 30) -> str:
    frac = max(0.0, min(1.0, frac))
    n = int(round(frac * width))
    return "[" + "#" * n + "." * (width - n) + f"] {frac * 100:5.1f}%"


def render(snap: dict) -> str:
    e = snap.get("engine", {})
    kv_t = max(1, e.get("kv_blocks_total", 1))
    spec = e.get("spec", {})
    lines = [
        f"legion-b200   uptime {snap.get('uptime_s', 0):.0f}s   in flight {snap.get('in_flight', 0)}   replicas {snap.get('replicas', 1)}"
        + ("   WARMING" if e.get("warming") else ""),
        f"running {e.get('running', 0):4d}   waiting {e.get('waiting', 0):4d}   steps {e.get('steps', 0)}   step {e.get('step_ms', 0):.2f} ms",
        f"KV blocks  {bar(e.get('kv_blocks_used', 0) / kv_t)}  {e.get('kv_blocks_used', 0)}/{kv_t}   preemptions {e.get('kv_preemptions', 0)}",
        f"tokens     prompt {e.get('prompt_tokens', 0)}   generated {e.get('completion_tokens', 0)}   prefix-cache hits {e.get('prefix_cache_hit_tokens', 0)}",
        f"spec       drafted {spec.get('draft_tokens', 0)}   accepted {spec.get('accepted_tokens', 0)}   rate {spec.get('acceptance_rate', 0):.2f}"
        f"   tokens/verify {spec.get('mean_accepted_length', 0):.2f}",
    ]
    return "\n".join(lines)


def run_top(url: str, api_key: Optional[str], interval: float, once: bool) -> int:
    headers = {"authorization": f"Bearer {api_key}"} if api_key else {}
    while True:
        try:
            req = urllib.request.Request(url.rstrip("/") + "/v1/stats", headers=headers)
            snap = json.loads(urllib.request.urlopen(req, timeout=5).read())
            out = render(snap)
        except Exception as e:  # noqa: BLE001
            out = f"cannot reach {url}: {e}"
            if once:
                print(out)
                return 1
        if once:
            print(out)
            return 0
        sys.stdout.write("\x1b[2J\x1b[H" + out + "\n")
        sys.stdout.flush()
        time.sleep(interval)


def start_tui(engine, interval: float = 1.0):
    def loop():
        t0 = time.time()
        while True:
            st = engine.stats()
            snap = {"uptime_s": time.time() - t0, "in_flight": st.running, "replicas": len(engine.replica_stats()),
                    "engine": {"running": st.running, "waiting": st.waiting, "steps": st.steps, "step_ms": st.step_ms_ewma,
                               "kv_blocks_used": st.kv_blocks_used, "kv_blocks_total": st.kv_blocks_total,
                               "kv_preemptions": st.kv_preemptions, "prompt_tokens": st.prompt_tokens,
                               "completion_tokens": st.completion_tokens, "warming": st.warming,
                               "prefix_cache_hit_tokens": st.prefix_cache_hit_tokens,
                               "spec": {"draft_tokens": st.spec_draft_tokens, "accepted_tokens": st.spec_accepted_tokens,
                                        "acceptance_rate": st.spec_acceptance_rate,
                                        "mean_accepted_length": st.spec_mean_accepted_length}}}
            sys.stderr.write("\x1b[s\x1b[H" + render(snap) + "\x1b[u")
            sys.stderr.flush()
            time.sleep(interval)
    threading.Thread(target=loop, daemon=True).start()
