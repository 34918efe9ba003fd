"""Import names of the reference's Python package, for code written against it:

    from ksana_llm import KsanaLLMEngine, EngineArgs, PluginConfig, TokenizerProcessorOpBase

Everything lives in ``ksanallm_b200``; this package only re-exports (reference: src/ksana_llm/python/ksana_llm/__init__.py).
"""
from dataclasses import dataclass

from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine, KsanaPythonOutput, Status  # noqa: F401
from ksanallm_b200.serving.tokenizer import TokenizerProcessor


@dataclass
class PluginConfig:
    model_dir: str = ""
    config_file: str = ""
    plugin_name: str = ""
    enable_trt: bool = False  # (no TensorRT engines here: vision towers run in PyTorch)
    thread_pool_size: int = 1
    vit_model_type: str = ""


class TokenizerProcessorOpBase(TokenizerProcessor):
    """The reference's constructor order: (model_dir, tokenizer_path, tokenization settings)."""

    def __init__(self, model_dir, tokenizer_path=None, tokenization=None):
        add = getattr(tokenization, "add_special_tokens", True) if tokenization is not None else True
        skip = getattr(tokenization, "skip_special_tokens", True) if tokenization is not None else True
        super().__init__(tokenizer_path or model_dir, add_special_tokens=add, skip_special_tokens=skip)
