from .packing import IGNORE_INDEX, PackedCollator, SyntheticPackedDataset, pack_documents

__all__ = ["IGNORE_INDEX", "PackedCollator", "SyntheticPackedDataset", "pack_documents"]
