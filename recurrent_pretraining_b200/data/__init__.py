"""Data path: token sources, collate/shift, mixture scheduling, goldfish masking, tokenizer, stateful loader."""
from .collate import generic_collate_fn  # noqa: F401
from .datasets import (BufferShuffledParquet, HuggingfaceDataset, ParquetStream, RandomTokens, TextRows,  # noqa: F401
                       WeightedMixture)
from .goldfish import apply_tld  # noqa: F401
from .loader import StatefulLoader  # noqa: F401
from .scheduler import DataScheduler, DataSchedulerTracker  # noqa: F401
from .tokenizer import Tokenizer  # noqa: F401
