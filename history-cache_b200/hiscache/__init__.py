"""hiscache: the Python API of HisCache on libhiscache_b200.

Export list of the reference package (hiscache/__init__.py:1-6) plus HistoryCache, which its
README documents (README.md:62-68) but its __init__ does not export.
"""
from hiscache_backend import count_history_reconstruct, get_graph_structure_score, record_history

from .comm import all2all, all2all_prealloc, all2allnaive, all2allnaive_prealloc, post_transfer, prepare_transfer
from .feature_store import HostFeatureStore
from .history_cache import HistoryCache
from .history_model import get_model
from .history_table import HistoryTable
from .history_trainer import HistoryTableTrainer, HistoryTrainer
from .multi_gpu_history_trainer import MultiGpuHistoryTrainer
from .sampler import get_loader
from .sharded import PeerHistoryTable, ShardedHistoryTable
from .util import Config, make_config

__all__ = [
    "HistoryTable", "HistoryTrainer", "HistoryCache", "count_history_reconstruct",
    "get_graph_structure_score", "record_history", "get_model", "MultiGpuHistoryTrainer",
    "all2all", "all2allnaive", "all2all_prealloc", "all2allnaive_prealloc", "prepare_transfer",
    "post_transfer", "HostFeatureStore", "HistoryTableTrainer", "get_loader", "Config", "make_config",
    "PeerHistoryTable", "ShardedHistoryTable",
]
