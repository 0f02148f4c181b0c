from .packing import IGNORE_INDEX, PackedCollator, SyntheticPackedDataset, pack_documents
from .synthetic_vlm import SyntheticVLMDataset

__all__ = ["IGNORE_INDEX", "PackedCollator", "SyntheticPackedDataset", "SyntheticVLMDataset", "pack_documents"]
