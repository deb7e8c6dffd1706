from .base import Dataset, DatasetMeta, IterableDataset, LazyDataset
from .packing import IterablePackingDataset, PackingDataset, pack_to_constant_volume

dataset_mapping = {c.__name__: c for c in (Dataset, LazyDataset, IterableDataset, PackingDataset, IterablePackingDataset)}
