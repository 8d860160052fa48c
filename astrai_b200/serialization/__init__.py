from astrai_b200.serialization.checkpoint import (
    Checkpoint, is_complete, latest_complete, load_json, load_model_config, load_model_weights, load_safetensors,
    load_state_dict, load_torch, save_json, save_model, save_safetensors, save_torch,
)
from astrai_b200.serialization.hf import (
    HF_MODEL_TYPES, adapt_config, convert_hf_config, convert_hf_weights, looks_like_hf_state_dict,
)
from astrai_b200.serialization.shards import load_bin, load_bin_offsets, save_bin

__all__ = [
    "Checkpoint", "HF_MODEL_TYPES", "adapt_config", "convert_hf_config", "convert_hf_weights", "is_complete",
    "latest_complete", "load_bin", "load_bin_offsets", "load_json", "load_model_config", "load_model_weights",
    "load_safetensors", "load_state_dict", "load_torch", "looks_like_hf_state_dict", "save_bin", "save_json",
    "save_model", "save_safetensors", "save_torch",
]
