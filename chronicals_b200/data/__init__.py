from .sequence_packer import (BinPackingAlgorithm, DataPrefetcher, DoubleBufferPrefetcher, FixedShapeSequencePacker,
                              PackedBatch, PackedDataLoader, PackedDataset, SequencePacker, create_cu_seqlens,
                              create_cu_seqlens_from_position_ids)
from .data_loader import (DataCollator, DataCollatorWithFlattening, InstructionDataset, PackingDataCollator,
                          SyntheticTokenDataset, create_dataloader, create_packed_dataloader)

__all__ = ["BinPackingAlgorithm", "DataPrefetcher", "DoubleBufferPrefetcher", "FixedShapeSequencePacker", "PackedBatch",
           "PackedDataLoader", "PackedDataset", "SequencePacker", "create_cu_seqlens",
           "create_cu_seqlens_from_position_ids", "DataCollator", "DataCollatorWithFlattening", "InstructionDataset",
           "PackingDataCollator", "SyntheticTokenDataset", "create_dataloader", "create_packed_dataloader"]
