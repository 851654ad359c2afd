"""Model definitions: configs, functional fp32/bf16 oracles, HF-format weights."""

from .config import ModelConfig, PRESETS, get_preset
from .functional import causal_lm_forward, decoder_layer_forward
from .weights import LazyRandomWeights, init_random_weights, load_safetensors_dir, save_safetensors_dir

__all__ = [
    "ModelConfig", "PRESETS", "get_preset", "causal_lm_forward", "decoder_layer_forward",
    "LazyRandomWeights", "init_random_weights", "load_safetensors_dir", "save_safetensors_dir",
]
