"""Plugins shipped with the package; a model directory selects one with a one-line ``ksana_plugin.py``
(``from ksanallm_b200.serving.plugins.qwen2_vl import KsanaPlugin``) or ``model_spec.plugin_model.plugin_path``."""
