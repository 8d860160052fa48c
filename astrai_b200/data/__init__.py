from astrai_b200.data.dataset import (
    BaseDataset, DatasetFactory, DPODataset, GRPODataset, SEQDataset, SFTDataset, SyntheticTokenDataset,
    dpo_collate_fn, dpo_processor, dpo_tokenize, grpo_collate_fn,
)
from astrai_b200.data.sampler import RDSampler
from astrai_b200.data.storage import JsonlSource, JsonlStore, MmapStore, Recordable, Store, StoreFactory, Streamable, detect_format
from astrai_b200.serialization import load_bin, save_bin

__all__ = [
    "BaseDataset", "DPODataset", "DatasetFactory", "GRPODataset", "JsonlSource", "JsonlStore", "MmapStore", "RDSampler", "Recordable", "Streamable",
    "SEQDataset", "SFTDataset", "Store", "StoreFactory", "SyntheticTokenDataset", "detect_format", "dpo_collate_fn",
    "dpo_processor", "dpo_tokenize", "grpo_collate_fn", "load_bin", "save_bin",
]
