"""``legion bench``: load generator against an OpenAI- or Anthropic-compatible server (ours or another).

Workloads (``docs/bench.md:1-67`` of the reference): ``bench`` = concurrency sweep (total tok/s, per-user decode
rate, TTFT, inter-token latency); ``chats`` = multi-turn conversations that share a growing prefix; ``prefill`` =
one prompt per size with ``max_tokens`` 1 (tok/s to first token); ``mixed`` = chat latency under background long
prompts; ``bandwidth`` = scrape ``/metrics`` before and after. Always temperature 0 and ``ignore_eos``.
"""
from __future__ import annotations

import json
import os
import random
import statistics
import threading
import time
import urllib.request
from typing import List, Optional


def _words(n: int, seed: int) -> str:
    rng = random.Random(seed)
    vocab = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta", "iota", "kappa", "lambda", "mu"]
    return " ".join(rng.choice(vocab) for _ in range(n))


class Result:
    def __init__(self):
        self.ttft = None
        self.gaps: List[float] = []
        self.tokens = 0
        self.t_end = 0.0
        self.t_first = 0.0
        self.error: Optional[str] = None
        self.cached = 0


def stream_chat(url: str, api: str, key: Optional[str], messages: list, max_tokens: int) -> Result:
    res = Result()
    headers = {"content-type": "application/json"}
    if key:
        headers["authorization"] = f"Bearer {key}"
        headers["x-api-key"] = key
    if api == "anthropic":
        body = {"model": "default", "max_tokens": max_tokens, "stream": True, "temperature": 0, "messages": messages}
        path = "/v1/messages"
    else:
        body = {"model": "default", "max_tokens": max_tokens, "stream": True, "temperature": 0, "ignore_eos": True,
                "stream_options": {"include_usage": True}, "messages": messages}
        path = "/v1/chat/completions"
    t0 = time.perf_counter()
    last = None
    try:
        req = urllib.request.Request(url.rstrip("/") + path, data=json.dumps(body).encode(), headers=headers)
        with urllib.request.urlopen(req, timeout=3600) as r:
            for raw in r:
                line = raw.decode("utf-8", "replace").strip()
                if not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                d = json.loads(line[6:])
                got = False
                if api == "anthropic":
                    got = d.get("type") == "content_block_delta"
                    if d.get("type") == "message_delta":
                        res.tokens = d.get("usage", {}).get("output_tokens", res.tokens)
                else:
                    ch = d.get("choices") or []
                    got = bool(ch and (ch[0].get("delta", {}).get("content") or ch[0].get("delta", {}).get("reasoning_content")))
                    if d.get("usage"):
                        res.tokens = d["usage"].get("completion_tokens", res.tokens)
                        res.cached = d["usage"].get("prompt_tokens_details", {}).get("cached_tokens", 0)
                if got:
                    now = time.perf_counter()
                    if last is None:
                        res.ttft = now - t0
                        res.t_first = now
                    else:
                        res.gaps.append(now - last)
                    last = now
    except Exception as e:  # noqa: BLE001
        res.error = repr(e)
    res.t_end = time.perf_counter()
    if not res.tokens:
        res.tokens = len(res.gaps) + (1 if res.ttft is not None else 0)
    return res


def _level(url, api, key, conc: int, prompt_tokens: int, max_tokens: int, seed: int) -> dict:
    results: List[Result] = [None] * conc
    def work(i):
        results[i] = stream_chat(url, api, key, [{"role": "user", "content": _words(prompt_tokens, seed * 1000 + i)}], max_tokens)
    t0 = time.perf_counter()
    ths = [threading.Thread(target=work, args=(i,)) for i in range(conc)]
    [t.start() for t in ths]
    [t.join() for t in ths]
    wall = time.perf_counter() - t0
    ok = [r for r in results if r and not r.error]
    per_user = [(r.tokens - 1) / max(r.t_end - r.t_first, 1e-9) for r in ok if r.tokens > 1 and r.t_first]
    gaps = [g for r in ok for g in r.gaps]
    return {"concurrency": conc, "requests_ok": len(ok), "errors": [r.error for r in results if r and r.error][:3],
            "total_tok_s": sum(r.tokens for r in ok) / wall if wall > 0 else 0.0,
            "decode_tok_s_per_user": [min(per_user), max(per_user)] if per_user else None,
            "ttft_s_median": statistics.median([r.ttft for r in ok if r.ttft is not None]) if ok else None,
            "itl_ms_median": statistics.median(gaps) * 1e3 if gaps else None,
            "itl_ms_p99": (sorted(gaps)[int(0.99 * (len(gaps) - 1))] * 1e3) if gaps else None, "wall_s": wall}


def _scrape(url: str) -> dict:
    out = {}
    try:
        with urllib.request.urlopen(url.rstrip("/") + "/metrics", timeout=10) as r:
            for line in r.read().decode().splitlines():
                if line and not line.startswith("#"):
                    k, _, v = line.rpartition(" ")
                    try:
                        out[k] = float(v)
                    except ValueError:
                        pass
    except Exception:
        pass
    return out


def run_bench(a) -> int:
    report = {"workload": a.workload, "url": a.url, "api": a.api, "time": time.time(), "rows": []}
    if a.workload == "bench":
        for c in [int(x) for x in str(a.concurrency).split(",")]:
            rounds = [_level(a.url, a.api, a.api_key, c, a.prompt_tokens, a.max_tokens, r) for r in range(a.rounds)]
            rounds.sort(key=lambda r: r["total_tok_s"])
            report["rows"].append(rounds[len(rounds) // 2])
    elif a.workload == "prefill":
        for n in [int(x) for x in str(a.prefill_sizes).split(",")]:
            r = stream_chat(a.url, a.api, a.api_key, [{"role": "user", "content": _words(n, n)}], 1)
            report["rows"].append({"prompt_words": n, "ttft_s": r.ttft, "words_per_s": n / r.ttft if r.ttft else None,
                                   "error": r.error})
    elif a.workload == "chats":
        history = []
        for turn in range(6):
            history.append({"role": "user", "content": _words(a.prompt_tokens // 4, turn)})
            r = stream_chat(a.url, a.api, a.api_key, history, a.max_tokens)
            history.append({"role": "assistant", "content": "ok " * max(1, r.tokens // 2)})
            report["rows"].append({"turn": turn, "ttft_s": r.ttft, "tokens": r.tokens, "cached_tokens": r.cached, "error": r.error})
    elif a.workload == "mixed":
        stop = threading.Event()
        def background():
            i = 0
            while not stop.is_set():
                stream_chat(a.url, a.api, a.api_key, [{"role": "user", "content": _words(4 * a.prompt_tokens, 77 + i)}], 8)
                i += 1
        bg = threading.Thread(target=background, daemon=True)
        bg.start()
        time.sleep(0.2)
        report["rows"].append(dict(_level(a.url, a.api, a.api_key, 1, 32, a.max_tokens, 5), note="chat under background long prompts"))
        stop.set()
    elif a.workload == "bandwidth":
        before = _scrape(a.url)
        row = _level(a.url, a.api, a.api_key, 4, a.prompt_tokens, a.max_tokens, 9)
        after = _scrape(a.url)
        row["metrics_delta"] = {k: after[k] - before.get(k, 0.0) for k in after if k.startswith("legion_") and
                                after[k] != before.get(k, 0.0)}
        report["rows"].append(row)
    print(json.dumps(report, indent=1))
    if a.save:
        os.makedirs(a.save, exist_ok=True)
        json.dump(report, open(os.path.join(a.save, "result.json"), "w"), indent=1)
        json.dump({"argv": vars(a) if hasattr(a, "__dict__") else {}, "time": report["time"]},
                  open(os.path.join(a.save, "meta.json"), "w"), indent=1, default=str)
        with open(os.path.join(a.save, "README.md"), "w") as f:
            f.write(f"# legion bench {a.workload}\n\n`result.json` holds one row per level; `meta.json` the arguments.\n")
    return 0 if all(not r.get("errors") and not r.get("error") for r in report["rows"]) else 1
