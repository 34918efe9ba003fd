"""ksanallm_b200: a Blackwell-native (sm_100a) LLM inference and serving engine."""
__version__ = "0.1.0"
