"""/forward client: intermediate tensors of one prefill pass, msgpack in and out.

    python examples/forward_client.py --port 8080 --tokens 1 2 3 4 5

Targets: "transformer" (residual stream before the final norm), "layernorm" (after it), "logits" (GATHER_ALL: all
vocabulary logits of the chosen rows; GATHER_TOKEN_ID: probability of the next input token) and, for layer-wise
rerankers, "lm_head" with "cutoff_layer". Rows: "slice_pos" = [[first, last], ...] (negative = from the end) or
"token_id" = [positions]."""
import argparse
import base64

import msgpack
import numpy as np
import requests


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--tokens", type=int, nargs="+", default=[1, 2, 3, 4, 5])
    ns = ap.parse_args()
    req = {"requests": [{"input_tokens": ns.tokens, "request_target": [
        {"target_name": "layernorm", "slice_pos": [[-1, -1]], "token_reduce_mode": "GATHER_ALL"},
        {"target_name": "logits", "slice_pos": [[0, -2]], "token_reduce_mode": "GATHER_TOKEN_ID"}]}]}
    r = requests.post(f"http://{ns.host}:{ns.port}/forward", data=msgpack.packb(req),
                      headers={"Content-Type": "application/x-msgpack"}, timeout=600)
    r.raise_for_status()
    for resp in msgpack.unpackb(r.content, raw=False)["responses"]:
        for t in resp["response"]:
            a = np.frombuffer(base64.b64decode(t["tensor"]["data"]), dtype=np.float32).reshape(t["tensor"]["shape"])
            print(t["target_name"], a.shape, a.reshape(-1)[:8])


if __name__ == "__main__":
    main()
