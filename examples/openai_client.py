"""OpenAI-compatible routes with plain HTTP (no SDK needed).

    python examples/openai_client.py --port 8080 --stream"""
import argparse
import json

import requests


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--stream", action="store_true")
    ns = ap.parse_args()
    base = f"http://{ns.host}:{ns.port}/v1"
    model = requests.get(base + "/models", timeout=60).json()["data"][0]["id"]
    body = {"model": model, "messages": [{"role": "user", "content": "Say hello in three languages."}],
            "max_tokens": 64, "temperature": 0.7, "stream": ns.stream}
    if not ns.stream:
        print(requests.post(base + "/chat/completions", json=body, timeout=600).json()["choices"][0]["message"]["content"])
        return
    with requests.post(base + "/chat/completions", json=body, stream=True, timeout=600) as r:
        for line in r.iter_lines():
            if not line.startswith(b"data: ") or line == b"data: [DONE]":
                continue
            delta = json.loads(line[6:])["choices"][0]["delta"].get("content")
            if delta:
                print(delta, end="", flush=True)
    print()


if __name__ == "__main__":
    main()
