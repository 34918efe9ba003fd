#!/usr/bin/env python
"""Entry point: ``python serving_server.py --config_file examples/ksana_llm.yaml --port 8080``.

Multi-GPU: start one process per GPU, e.g.
``python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 serving_server.py --config_file ...``
(rank 0 opens the HTTP port, the other ranks execute their tensor-parallel shard).
"""
from ksanallm_b200.serving.server import main

if __name__ == "__main__":
    main()
