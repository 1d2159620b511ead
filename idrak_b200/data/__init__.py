"""Datasets, the batch loader (sharding for data parallel ranks, bucketing, prefetch) and record readers."""
from .loader import DataLoader, Dataset, MappedDataset, Subset, TensorDataset, TokenWindows, collate
from .sources import (MinMaxScaler, StandardScaler, csv_dataset, dedupe, filter_rows, load_scaler, map_rows, mix, read_code,
                      read_delimited, read_json, read_jsonl, read_parquet, read_records, read_text, shuffle_rows, split_rows,
                      write_jsonl)
