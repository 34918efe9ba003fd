"""The C++ /forward client (examples/cpp/forward_client.cpp) is compiled with g++ and run against a server process:
its msgpack request is understood, and the tensors it prints equal the ones the Python client decodes."""
import base64
import os
import shutil
import signal
import socket
import subprocess
import sys
import time

import msgpack
import numpy as np
import pytest
import requests

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_cpp_forward_client_against_a_live_server(tmp_path):
    exe = str(tmp_path / "forward_client")
    subprocess.run(["g++", "-O1", "-std=c++17", "-Wall", "-Werror", "-o", exe,
                    os.path.join(ROOT, "examples", "cpp", "forward_client.cpp")], check=True)
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
        tokens = [5, 9, 77, 120, 33, 4]
        out = subprocess.run([exe, "127.0.0.1", str(port)] + [str(t) for t in tokens], capture_output=True, text=True,
                             timeout=60)
        assert out.returncode == 0, out.stderr
        lines = out.stdout.strip().splitlines()
        assert len(lines) == 2 and lines[0].startswith("layernorm shape=[1, ") and lines[1].startswith("logits shape=[5]")
        req = {"requests": [{"input_tokens": tokens, "request_target": [
            {"target_name": "layernorm", "slice_pos": [[-1, -1]], "token_reduce_mode": "GATHER_ALL"},
            {"target_name": "logits", "slice_pos": [[0, -2]], "token_reduce_mode": "GATHER_TOKEN_ID"}]}]}
        r = requests.post(base + "/forward", data=msgpack.packb(req), headers={"Content-Type": "application/x-msgpack"},
                          timeout=60)
        want = msgpack.unpackb(r.content, raw=False)["responses"][0]["response"]
        for line, t in zip(lines, want):
            a = np.frombuffer(base64.b64decode(t["tensor"]["data"]), dtype=np.float32).reshape(-1)[:8]
            got = np.array([float(x) for x in line.split("values=")[1].split()], dtype=np.float32)
            assert np.allclose(got, a[:len(got)], rtol=1e-4, atol=1e-6)
        bad = subprocess.run([exe, "127.0.0.1", "1"], capture_output=True, text=True, timeout=30)
        assert bad.returncode == 1 and "cannot connect" in bad.stderr
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.wait(timeout=30)
        finally:
            if proc.poll() is None:
                proc.kill()
