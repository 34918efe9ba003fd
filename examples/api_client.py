"""Minimal /generate client (non-streaming and streaming).

    python examples/api_client.py --port 8080 --prompt "Hello" --max-new-tokens 32 [--stream]

Request / response format: {"prompt" | "input_tokens", "sampling_config": {...}, "stream": bool} ->
{"texts": [...], "output_token_ids": [[...]], "input_token_ids": [...]}; streaming replies are JSON objects
separated by NUL bytes, each carrying the whole output so far."""
import argparse
import json

import requests


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--prompt", default="Hello, my name is")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--topk", type=int, default=1)
    ap.add_argument("--topp", type=float, default=1.0)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--stream", action="store_true")
    ns = ap.parse_args()
    body = {"prompt": ns.prompt, "stream": ns.stream,
            "sampling_config": {"max_new_tokens": ns.max_new_tokens, "topk": ns.topk, "topp": ns.topp,
                                "temperature": ns.temperature}}
    url = f"http://{ns.host}:{ns.port}/generate"
    if not ns.stream:
        r = requests.post(url, data=json.dumps(body), timeout=600)
        r.raise_for_status()
        print(r.json()["texts"][0])
        return
    shown = 0
    with requests.post(url, data=json.dumps(body), stream=True, timeout=600) as r:
        r.raise_for_status()
        buf = b""
        for chunk in r.iter_content(chunk_size=None):
            buf += chunk
            while b"\0" in buf:
                part, buf = buf.split(b"\0", 1)
                if not part:
                    continue
                text = json.loads(part)["texts"][0]
                print(text[shown:], end="", flush=True)
                shown = len(text)
    print()


if __name__ == "__main__":
    main()
