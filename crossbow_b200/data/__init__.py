"""Data sets: in-memory / synthetic batches in pinned host memory, binary partition files, record files."""
from .dataset import Dataset, SyntheticDataset, ArrayDataset  # noqa: F401
