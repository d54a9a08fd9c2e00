from .generate import ensure_recall_datasets, recall_dataset_paths
from .recall import gold_ranks, run_recall

__all__ = ["ensure_recall_datasets", "recall_dataset_paths", "gold_ranks", "run_recall"]
