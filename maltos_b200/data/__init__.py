"""Resumable data loaders: token shards (pretraining), packed SFT shards, in-memory tensors, background prefetch."""
from .prefetch import PrefetchDataLoader
from .pretrain import PretrainingDataLoader, PretrainingDataState, TokenShardDataset
from .protocols import StatefulDataLoaderProtocol
from .sft import PackedSFTDataset, SFTDataLoader, SFTDataState
from .simple import SimpleDataLoaderState, SimpleTensorDataLoader

__all__ = ["PackedSFTDataset", "PrefetchDataLoader", "PretrainingDataLoader", "PretrainingDataState", "SFTDataLoader",
           "SFTDataState", "SimpleDataLoaderState", "SimpleTensorDataLoader", "StatefulDataLoaderProtocol", "TokenShardDataset"]
