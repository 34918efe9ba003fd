"""Every shipped example configuration parses, validates and names only known sections."""
import glob
import os

import pytest

from ksanallm_b200.config.schema import load_serving_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(ROOT, "examples", "*.yaml"))))
def test_example_config_loads(path):
    cfg = load_serving_config(path)
    g = cfg.setting.global_
    assert g.tensor_para_size >= 1 and g.pipeline_para_size >= 1
    assert cfg.setting.batch_scheduler.max_token_len > 0
    assert not cfg.setting.extra, f"unknown top-level setting keys: {list(cfg.setting.extra)}"
    assert not cfg.setting.batch_scheduler.extra, f"unknown batch_scheduler keys: {list(cfg.setting.batch_scheduler.extra)}"
    if "disaggregating" in path:
        assert cfg.setting.connector.group_role in ("prefill", "decode") and cfg.setting.connector.router_addr
