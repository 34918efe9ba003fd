"""End to end through the command line: ``serving_server.py`` is started as a separate process with the tiny CPU
configuration, answers over real HTTP (JSON and NUL-separated streaming), and two identical greedy requests return
identical text; SIGTERM ends it cleanly."""
import json
import os
import signal
import socket
import subprocess
import sys
import time

import requests

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_server_process_generate_and_shutdown():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, KSANA_SKIP_WARMUP="1", PYTHONPATH=ROOT)
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "serving_server.py"), "--config_file",
                             os.path.join(ROOT, "examples", "tiny_cpu.yaml"), "--synthetic-model", "tiny-llama",
                             "--device", "cpu", "--host", "127.0.0.1", "--port", str(port)],
                            env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    base = f"http://127.0.0.1:{port}"
    try:
        for _ in range(240):
            try:
                if requests.get(base + "/health", timeout=1).status_code == 200:
                    break
            except requests.RequestException:
                pass
            assert proc.poll() is None, "server exited during start-up"
            time.sleep(0.25)
        else:
            raise AssertionError("server did not come up")
        body = {"prompt": "The capital of France is", "stream": False,
                "sampling_config": {"max_new_tokens": 12, "topk": 1, "ignore_eos": True}}
        a = requests.post(base + "/generate", data=json.dumps(body), timeout=60).json()
        b = requests.post(base + "/generate", data=json.dumps(body), timeout=60).json()
        assert a["texts"] == b["texts"] and len(a["output_token_ids"][0]) == 12
        with requests.post(base + "/generate", data=json.dumps(dict(body, stream=True)), stream=True, timeout=60) as r:
            chunks = [json.loads(c) for c in r.content.split(b"\0") if c]
        assert chunks[-1]["output_token_ids"] == a["output_token_ids"]
        chat = requests.post(base + "/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}],
                                                                  "max_tokens": 5, "temperature": 0}, timeout=60)
        assert chat.status_code == 200 and chat.json()["usage"]["completion_tokens"] <= 5
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            assert proc.wait(timeout=30) == 0
        finally:
            if proc.poll() is None:
                proc.kill()
