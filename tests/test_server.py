"""HTTP surface over the mock engine: every route, SSE framing, error shapes, auth, overload, metrics; and one
end-to-end pass over a real (tiny, CPU) engine."""
import json

import pytest
from fastapi.testclient import TestClient

from legion_b200.engine.mock import MockEngine
from legion_b200.server.app import ServerConfig, create_app


def client(**kw):
    eng = kw.pop("engine", None) or MockEngine("mock")
    return TestClient(create_app(eng, ServerConfig(**kw)))


def sse(text):
    out = []
    ev = None
    for line in text.splitlines():
        if line.startswith("event: "):
            ev = line[7:]
        elif line.startswith("data: "):
            d = line[6:]
            out.append((ev, d if d == "[DONE]" else json.loads(d)))
            ev = None
    return out


def test_health_models_stats_metrics_webui():
    c = client()
    assert c.get("/health").json()["status"] == "ok"
    assert c.get("/v1/models").json()["data"][0]["id"] == "mock"
    assert c.get("/models").json()["object"] == "list"
    assert c.get("/v1/models/mock").json()["id"] == "mock"
    r = c.get("/v1/models/nope")
    assert r.status_code == 404 and r.json()["error"]["type"] == "not_found_error"
    assert c.get("/v1/stats").json()["schema"] == 1
    c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "a b c"}]})
    m = c.get("/metrics").text
    assert "legion_http_requests_total" in m and "legion_completion_tokens_total 3.0" in m
    assert "legion_engine_kv_blocks_total" in m and "legion_time_to_first_token_bucket" in m
    assert "<title>legion-b200</title>" in c.get("/").text
    assert "x-request-id" in c.get("/health").headers


def test_chat_completion_and_stream():
    c = client()
    r = c.post("/v1/chat/completions", json={"model": "whatever", "messages": [{"role": "user", "content": "one two three"}],
                                             "unknown_field": 1, "logprobs": True, "top_logprobs": 1})
    j = r.json()
    assert r.status_code == 200 and j["object"] == "chat.completion" and j["model"] == "mock"
    assert j["choices"][0]["message"]["content"] == "one two three" and j["choices"][0]["finish_reason"] == "stop"
    assert j["usage"]["completion_tokens"] == 3 and "timings" in j and len(j["choices"][0]["logprobs"]["content"]) == 3
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "a b"}], "stream": True,
                                             "stream_options": {"include_usage": True}})
    ev = sse(r.text)
    assert ev[-1][1] == "[DONE]"
    chunks = [d for _, d in ev[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    assert "".join(ch["choices"][0]["delta"].get("content", "") for ch in chunks if ch["choices"]) == "a b"
    assert chunks[-2]["choices"][0]["finish_reason"] == "stop" and chunks[-1]["usage"]["completion_tokens"] == 2
    # length, stop sequences, tools
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "a b c d"}], "max_tokens": 2})
    assert r.json()["choices"][0]["finish_reason"] == "length"
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "a b STOP d"}], "stop": "STOP"})
    assert r.json()["choices"][0]["message"]["content"] == "a b "
    tools = [{"type": "function", "function": {"name": "get", "parameters": {"type": "object"}}}]
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": '/tool get {"x": 1}'}], "tools": tools})
    msg = r.json()["choices"][0]
    assert msg["finish_reason"] == "tool_calls" and msg["message"]["tool_calls"][0]["function"]["name"] == "get"
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "response_format": {"type": "json_object"}})
    assert json.loads(r.json()["choices"][0]["message"]["content"]) == {"echo": "x"}


def test_completions_anthropic_responses():
    c = client()
    r = c.post("/v1/completions", json={"prompt": "say this", "max_tokens": 8, "echo": True})
    assert r.json()["choices"][0]["text"] == "say thissay this" and r.json()["object"] == "text_completion"
    r = c.post("/v1/completions", json={"prompt": "a b", "stream": True})
    assert sse(r.text)[-1][1] == "[DONE]"
    r = c.post("/v1/messages", json={"model": "m", "max_tokens": 16, "system": "s",
                                     "messages": [{"role": "user", "content": [{"type": "text", "text": "hey there"}]}]})
    j = r.json()
    assert j["type"] == "message" and j["content"][0]["text"] == "hey there" and j["stop_reason"] == "end_turn"
    r = c.post("/v1/messages", json={"max_tokens": 16, "stream": True, "messages": [{"role": "user", "content": "a b"}]})
    names = [e for e, _ in sse(r.text)]
    assert names[:3] == ["message_start", "ping", "content_block_start"]
    assert names[-3:] == ["content_block_stop", "message_delta", "message_stop"] and "content_block_delta" in names
    assert c.post("/v1/messages/count_tokens", json={"messages": [{"role": "user", "content": "a b c"}]}).json()["input_tokens"] > 0
    r = c.post("/v1/responses", json={"input": "hello you", "instructions": "be nice"})
    j = r.json()
    assert j["object"] == "response" and j["status"] == "completed" and j["output_text"] == "hello you"
    r = c.post("/v1/responses", json={"input": "x y", "stream": True})
    names = [e for e, _ in sse(r.text)]
    assert names[0] == "response.created" and names[-1] == "response.completed"
    assert c.post("/v1/responses", json={"input": "x", "previous_response_id": "r1"}).status_code == 400
    assert c.post("/v1/responses", json={"input": "x", "store": True}).status_code == 400


def test_validation_errors_in_the_callers_shape():
    c = client()
    for body in ({"messages": []}, {"messages": [{"role": "user", "content": "x"}], "temperature": 3},
                 {"messages": [{"role": "user", "content": "x"}], "top_p": 0},
                 {"messages": [{"role": "user", "content": "x"}], "top_logprobs": 21},
                 {"messages": [{"role": "user", "content": "x"}], "min_tokens": 9, "max_tokens": 2},
                 {"messages": [{"role": "wizard", "content": "x"}]},
                 {"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "http://x/y.png"}}]}]},
                 {"messages": [{"role": "user", "content": "x"}], "chat_template_kwargs": {"enable_thinking": "yes"}}):
        r = c.post("/v1/chat/completions", json=body)
        assert r.status_code == 400 and r.json()["error"]["type"] == "invalid_request_error", body
    r = c.post("/v1/chat/completions", content=b"{not json", headers={"content-type": "application/json"})
    assert r.status_code == 400 and "invalid JSON" in r.json()["error"]["message"]
    r = c.post("/v1/messages", json={"max_tokens": 5, "temperature": 1.5, "messages": [{"role": "user", "content": "x"}]})
    assert r.status_code == 400 and r.json()["type"] == "error" and r.json()["error"]["type"] == "invalid_request_error"


def test_auth_body_limit_overload():
    c = client(api_keys=["sekret"])
    assert c.get("/health").status_code == 200
    assert c.get("/v1/models").status_code == 401
    assert c.get("/v1/models", headers={"authorization": "Bearer sekret"}).status_code == 200
    assert c.get("/v1/models", headers={"x-api-key": "sekret"}).status_code == 200
    r = c.post("/v1/messages", json={}, headers={"x-api-key": "bad"})
    assert r.status_code == 401 and r.json()["error"]["type"] == "authentication_error"
    c = client(max_request_mb=0)
    assert c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x" * 100}]}).status_code == 413
    busy = MockEngine("mock", max_in_flight=0)
    c = client(engine=busy)
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]})
    assert r.status_code == 429
    r = c.post("/v1/messages", json={"max_tokens": 4, "messages": [{"role": "user", "content": "x"}]})
    assert r.status_code == 529 and r.json()["error"]["type"] == "overloaded_error"


def test_real_engine_behind_the_server():
    from legion_b200.config import tiny_hybrid_moe
    from legion_b200.engine.lm import EngineConfig, build_engine
    eng = build_engine(tiny_hybrid_moe(), engine_cfg=EngineConfig(ctx_size=256, max_seqs=2, block_size=16))
    c = client(engine=eng)
    body = {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0, "ignore_eos": True}
    a = c.post("/v1/chat/completions", json=body).json()
    b = c.post("/v1/chat/completions", json=body).json()
    assert a["usage"]["completion_tokens"] == 6 and a["choices"][0]["finish_reason"] == "length"
    assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]
    assert b["usage"]["prompt_tokens_details"]["cached_tokens"] > 0
    r = c.post("/v1/chat/completions", json=dict(body, max_tokens=100000))
    assert r.status_code == 200     # max_tokens is clamped to the context
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x" * 400}], "max_tokens": 4})
    assert r.status_code == 400 and "context" in r.json()["error"]["message"]
    assert c.get("/v1/stats").json()["engine"]["prefix_cache_hit_tokens"] > 0
    eng.shutdown()


def test_tls_listener_serves_https(tmp_path):
    """`--tls-cert / --tls-key`: the listener speaks TLS; a client that trusts the certificate gets the API, a plain
    HTTP client does not."""
    import datetime
    import socket
    import threading
    import time

    import requests
    import uvicorn
    from cryptography import x509
    from cryptography.hazmat.primitives import hashes, serialization
    from cryptography.hazmat.primitives.asymmetric import rsa
    from cryptography.x509.oid import NameOID
    import ipaddress

    key = rsa.generate_private_key(public_exponent=65537, key_size=2048)
    name = x509.Name([x509.NameAttribute(NameOID.COMMON_NAME, "127.0.0.1")])
    now = datetime.datetime.now(datetime.timezone.utc)
    cert = (x509.CertificateBuilder().subject_name(name).issuer_name(name).public_key(key.public_key())
            .serial_number(x509.random_serial_number()).not_valid_before(now - datetime.timedelta(minutes=1))
            .not_valid_after(now + datetime.timedelta(hours=1))
            .add_extension(x509.SubjectAlternativeName([x509.IPAddress(ipaddress.ip_address("127.0.0.1"))]), False)
            .sign(key, hashes.SHA256()))
    cert_path, key_path = tmp_path / "cert.pem", tmp_path / "key.pem"
    cert_path.write_bytes(cert.public_bytes(serialization.Encoding.PEM))
    key_path.write_bytes(key.private_bytes(serialization.Encoding.PEM, serialization.PrivateFormat.TraditionalOpenSSL,
                                           serialization.NoEncryption()))
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    app = create_app(MockEngine("mock"), ServerConfig())
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error",
                                           ssl_certfile=str(cert_path), ssl_keyfile=str(key_path)))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    try:
        for _ in range(100):
            if server.started:
                break
            time.sleep(0.05)
        assert server.started
        r = requests.get(f"https://127.0.0.1:{port}/v1/models", verify=str(cert_path), timeout=10)
        assert r.status_code == 200 and r.json()["data"][0]["id"] == "mock"
        r = requests.post(f"https://127.0.0.1:{port}/v1/chat/completions", verify=str(cert_path), timeout=10,
                          json={"model": "mock", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4})
        assert r.status_code == 200 and r.json()["choices"][0]["message"]["content"]
        with pytest.raises(requests.exceptions.RequestException):
            requests.get(f"http://127.0.0.1:{port}/v1/models", timeout=5)
    finally:
        server.should_exit = True
        th.join(timeout=10)


def test_metric_families_roofline_stages_parallel_and_gpu_counters_from_a_fake_nvml():
    """Roofline, per-phase host time, KV / prefix tiers, tensor-parallel traffic and the GPU counter family; the GPU
    counters are read from a fake NVML (reads only: nothing in the sampler sets anything)."""
    from types import SimpleNamespace as NS

    from legion_b200.engine.types import EngineStats
    from legion_b200.server.metrics import Metrics
    m = Metrics()
    st = EngineStats(running=2, model_bytes_step=13_100_000_000, step_ms_ewma=4.0, kv_swap_out=3, prefix_host_spilled=5)
    st.host_ms.update(plan=1.5, forward=7.0)
    m.update_engine(st)
    m.update_roofline(st, peaks={"hbm_gbs": 6550.0, "bf16_tflops": 1654.0, "nvlink_gbs": 770.0})
    m.update_parallel({"all_reduce": 96, "bytes": 96 * 65536})

    calls = []

    class FakeNvml:
        NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX, NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX = 138, 139
        NVML_PCIE_UTIL_RX_BYTES, NVML_PCIE_UTIL_TX_BYTES, NVML_CLOCK_SM = 1, 0, 1

        def __getattr__(self, name):                       # any call that is not a read below fails the test
            raise AssertionError(f"unexpected NVML call {name}")

        def nvmlDeviceGetCount(self):
            return 2

        def nvmlDeviceGetHandleByIndex(self, i):
            return i

        def nvmlDeviceGetFieldValues(self, h, fields):
            calls.append(("field", h, fields[0]))
            return [NS(value=NS(ullVal=1000 * (h + 1) + (fields[0] - 138)))]

        def nvmlDeviceGetPcieThroughput(self, h, which):
            return 10 + which

        def nvmlDeviceGetClockInfo(self, h, which):
            return 1965

        def nvmlDeviceGetPowerUsage(self, h):
            return 650_000

        def nvmlDeviceGetMemoryInfo(self, h):
            return NS(used=50 << 30)

        def nvmlDeviceGetUtilizationRates(self, h):
            return NS(gpu=50, memory=25)

    fake = FakeNvml()
    assert m.sample_gpus(fake, now=100.0) == 2
    assert m.sample_gpus(fake, now=104.0) == 2             # 4 s at 50 % / 25 % busy
    text = m.render()
    for want in ('legion_engine_host_ms{phase="forward"} 7.0', "legion_engine_kv_swap_out 3.0",
                 "legion_engine_prefix_host_spilled 5.0", "legion_roofline_hbm_gbs 6550.0",
                 "legion_roofline_step_floor_ms 2.0", "legion_roofline_step_bandwidth_fraction 0.5",
                 "legion_tp_all_reduce_calls 96.0", 'legion_gpu_nvlink_rx_bytes{gpu="1"} 2.048e+06',
                 'legion_gpu_nvlink_tx_bytes{gpu="0"} 1.025024e+06', 'legion_gpu_sm_busy_seconds{gpu="0"} 2.0',
                 'legion_gpu_memory_busy_seconds{gpu="1"} 1.0', 'legion_gpu_power_watts{gpu="0"} 650.0',
                 'legion_gpu_sm_clock_mhz{gpu="1"} 1965.0'):
        assert want in text, want


def test_numa_binding_from_a_fake_sysfs(tmp_path):
    """The GPU's PCI device names its NUMA node, the node names its CPUs, the process is restricted to them."""
    import os

    from legion_b200.hw import numa
    assert numa.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    sysfs = tmp_path / "sys"
    (sysfs / "bus/pci/devices/0000:1b:00.0").mkdir(parents=True)
    (sysfs / "bus/pci/devices/0000:1b:00.0/numa_node").write_text("1\n")
    (sysfs / "devices/system/node/node1").mkdir(parents=True)
    allowed = sorted(os.sched_getaffinity(0))
    (sysfs / "devices/system/node/node1/cpulist").write_text(",".join(str(c) for c in allowed[:2]) + ",9999\n")
    done = {}
    r = numa.bind_to_gpu(3, sysfs=str(sysfs), bus_id="0000:1b:00.0", apply=lambda pid, cpus: done.update(pid=pid, cpus=cpus))
    assert r["node"] == 1 and r["bound"] and done["cpus"] == set(allowed[:2])       # CPUs outside the cpuset dropped
    (sysfs / "bus/pci/devices/0000:1b:00.0/numa_node").write_text("-1\n")
    r = numa.bind_to_gpu(3, sysfs=str(sysfs), bus_id="0000:1b:00.0", apply=lambda *a: done.update(again=True))
    assert r["node"] is None and not r["bound"] and "again" not in done


def test_only_one_choice_per_request():
    c = client()
    msg = {"messages": [{"role": "user", "content": "a"}]}
    assert c.post("/v1/chat/completions", json=dict(msg, n=1)).status_code == 200
    for bad in (2, 0):
        r = c.post("/v1/chat/completions", json=dict(msg, n=bad))
        assert r.status_code == 400 and r.json()["error"]["param"] == "n"
