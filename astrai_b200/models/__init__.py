from astrai_b200.config.train_config import LoRAConfig
from astrai_b200.models.attention import GQA, MLA, AttnFactory
from astrai_b200.models.automodel import AutoModel, ModelFactory
from astrai_b200.models.decoder import DecoderBlock
from astrai_b200.models.encoder import EmbeddingEncoder
from astrai_b200.models.ffn import MLP, DeepSeekMoE, FFNFactory
from astrai_b200.models.layers import Embedding, Linear, RMSNorm, RotaryEmbedding, apply_rotary_emb, get_rotary_emb
from astrai_b200.models.lm import AutoRegressiveLM
from astrai_b200.models.lora import LoRALinear, inject_lora, load_lora, merge_lora, save_lora

__all__ = [
    "AttnFactory", "AutoModel", "AutoRegressiveLM", "DecoderBlock", "DeepSeekMoE", "Embedding", "EmbeddingEncoder",
    "FFNFactory", "GQA", "Linear", "LoRAConfig", "LoRALinear", "MLA", "MLP", "ModelFactory", "RMSNorm",
    "RotaryEmbedding", "apply_rotary_emb", "get_rotary_emb", "inject_lora", "load_lora", "merge_lora", "save_lora",
]
