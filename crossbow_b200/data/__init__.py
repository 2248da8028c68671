"""Data sets: in-memory / synthetic batches in pinned host memory, binary partition files, record files."""
from .dataset import Dataset, SyntheticDataset, ArrayDataset  # noqa: F401


def __getattr__(name):
    """The file-backed data sets load the native runtime, so they are imported on first use.  `LightWeightDataset` is the
    reference's name of the slot-ring data set; its `Dataset` (mapped partition files) is `BasicDataset` here."""
    if name in ("BasicDataset", "LightDataset", "DatasetWriter"):
        from . import native
        return getattr(native, name)
    if name == "LightWeightDataset":
        from .native import LightDataset
        return LightDataset
    if name in ("RecordDataset", "RecordWriter"):
        from . import records
        return getattr(records, name)
    if name in ("convert_imagenet", "read_tfrecord", "parse_example"):
        from . import tfrecords
        return getattr(tfrecords, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
