"""On-disk formats of the reference project, read and written with numpy: the files its preprocessor emits and its trainer
loads, so that a dataset directory or a checkpoint made by one side is usable by the other.

  edges/{train,validation,test}_edges.bin      raw row-major [n, 2|3] int32 or int64 (src[, rel], dst)
                                               (python/tools/preprocess/converters/writers/torch_writer.py:47-57 of the reference)
  edges/{train,...}_partition_offsets.txt      P * P lines: number of edges of bucket src_part * P + dst_part, the edges file
                                               being sorted by that bucket id (partitioners/torch_partitioner.py:12-31, writer :59-68)
  dataset.yaml                                 flat `key: value` statistics (DatasetConfig, tools/configuration/gege_config.py:417-428)
  <model_dir>/embeddings.bin, embeddings_state.bin   raw row-major fp32 [num_nodes, D] (cpp/src/storage/io.cpp:139-140,
                                               cpp/include/configuration/constants.h:11-44)
  <model_dir>/metadata.csv                     seven lines (cpp/src/storage/checkpointer.cpp:111-122)

No torch, no device code: these are host-side files."""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Optional, Sequence, Tuple

import numpy as np

EDGES_DIR = "edges"
SPLITS = {"train": "train_", "valid": "validation_", "test": "test_"}
EDGES_FILE = "edges.bin"
OFFSETS_FILE = "partition_offsets.txt"
DATASET_YAML = "dataset.yaml"
EMBEDDINGS_FILE = "embeddings.bin"
EMBEDDINGS_STATE_FILE = "embeddings_state.bin"
METADATA_FILE = "metadata.csv"

_STAT_KEYS = ("dataset_dir", "num_edges", "num_nodes", "num_relations", "num_train", "num_valid", "num_test", "node_feature_dim",
              "rel_feature_dim", "num_classes", "initialized")


def partition_edges(edges: np.ndarray, num_nodes: int, num_partitions: int) -> Tuple[np.ndarray, np.ndarray]:
    """Edges sorted by bucket id src_part * P + dst_part with partition_size = ceil(num_nodes / P), and the P * P bucket
    sizes (torch_partitioner.py:12-31).  The order inside a bucket is the input order (a stable sort; the reference's sort
    leaves it unspecified)."""
    psize = -(-num_nodes // num_partitions)
    bucket = (edges[:, 0] // psize) * num_partitions + edges[:, -1] // psize
    order = np.argsort(bucket, kind="stable")
    sizes = np.bincount(bucket, minlength=num_partitions * num_partitions).astype(np.int64)
    return np.ascontiguousarray(edges[order]), sizes


def write_dataset(directory, train: np.ndarray, valid: Optional[np.ndarray], test: Optional[np.ndarray], num_nodes: int,
                  num_relations: int = 1, num_partitions: int = 1, dtype=np.int32,
                  offsets: Optional[Dict[str, Sequence[int]]] = None) -> Dict[str, object]:
    """Writes the dataset directory the reference's trainer reads.  With num_partitions > 1 the train edges must already be
    bucket-sorted (partition_edges) and offsets["train"] given (valid / test offsets only for partitioned evaluation)."""
    d = Path(directory)
    (d / EDGES_DIR).mkdir(parents=True, exist_ok=True)
    cols = train.shape[1]
    if cols not in (2, 3):
        raise ValueError("edge lists have 2 or 3 columns")
    if np.dtype(dtype) == np.int32 and max(num_nodes, num_relations) > np.iinfo(np.int32).max:
        raise ValueError("ids do not fit int32")
    stats = dict(dataset_dir=str(d.resolve()) + "/", num_edges=int(train.shape[0]), num_nodes=int(num_nodes), num_relations=int(num_relations),
                 num_train=int(train.shape[0]), num_valid=int(valid.shape[0]) if valid is not None else -1,
                 num_test=int(test.shape[0]) if test is not None else -1, node_feature_dim=-1, rel_feature_dim=-1, num_classes=-1,
                 initialized=False)
    with open(d / DATASET_YAML, "w") as f:
        for k in _STAT_KEYS:
            v = stats[k]
            f.write(f"{k}: {str(v).lower() if isinstance(v, bool) else v}\n")
    for split, arr in (("train", train), ("valid", valid), ("test", test)):
        if arr is None:
            continue
        if arr.shape[1] != cols:
            raise ValueError("all splits must have the same number of columns")
        np.ascontiguousarray(arr, dtype=dtype).tofile(d / EDGES_DIR / (SPLITS[split] + EDGES_FILE))
    if num_partitions > 1:
        if offsets is None or "train" not in offsets:
            raise ValueError("partitioned datasets need the train bucket sizes")
        for split, off in offsets.items():
            if len(off) != num_partitions * num_partitions:
                raise ValueError("P * P bucket sizes expected")
            with open(d / EDGES_DIR / (SPLITS[split] + OFFSETS_FILE), "w") as f:
                f.writelines(f"{int(o)}\n" for o in off)
    return stats


def read_dataset(directory, mmap: bool = True) -> Dict[str, object]:
    """{"stats": dict, "train" / "valid" / "test": [n, cols] arrays (memory-mapped), "offsets": {split: int64[P*P]}}.
    The edge dtype (int32 / int64) and the column count follow from the file size, the edge count in dataset.yaml and
    num_relations (3 columns when there is more than one relation type, cpp/src/storage/io.cpp:35-38)."""
    d = Path(directory)
    stats: Dict[str, object] = {}
    for line in open(d / DATASET_YAML):
        line = line.split("#")[0].strip()
        if not line or ":" not in line:
            continue
        k, v = (x.strip() for x in line.split(":", 1))
        if k == "dataset_dir":
            stats[k] = v
        elif v.lower() in ("true", "false"):
            stats[k] = v.lower() == "true"
        else:
            try:
                stats[k] = int(v)
            except ValueError:
                stats[k] = v
    cols = 3 if int(stats.get("num_relations", 1)) > 1 else 2
    out: Dict[str, object] = {"stats": stats, "offsets": {}}
    for split, key in (("train", "num_train"), ("valid", "num_valid"), ("test", "num_test")):
        path = d / EDGES_DIR / (SPLITS[split] + EDGES_FILE)
        n = int(stats.get(key, -1))
        if n < 0 or not path.exists():
            continue
        size = path.stat().st_size
        if n == 0:
            out[split] = np.zeros((0, cols), np.int64)
            continue
        item = size // (n * cols)
        if item not in (4, 8) or item * n * cols != size:
            raise ValueError(f"{path}: {size} bytes do not hold {n} x {cols} int32 or int64 ids")
        dt = np.int32 if item == 4 else np.int64
        out[split] = (np.memmap(path, dtype=dt, mode="r", shape=(n, cols)) if mmap else np.fromfile(path, dtype=dt).reshape(n, cols))
        off = d / EDGES_DIR / (SPLITS[split] + OFFSETS_FILE)
        if off.exists():
            o = np.array([int(x) for x in open(off).read().split()], np.int64)
            if int(o.sum()) != n:
                raise ValueError(f"{off}: bucket sizes add up to {int(o.sum())}, the split has {n} edges")
            out["offsets"][split] = o
    return out


def write_embeddings(model_dir, table: np.ndarray, state: Optional[np.ndarray] = None):
    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    np.ascontiguousarray(table, dtype=np.float32).tofile(d / EMBEDDINGS_FILE)
    if state is not None:
        if state.shape != table.shape:
            raise ValueError("the optimizer state has the table's shape")
        np.ascontiguousarray(state, dtype=np.float32).tofile(d / EMBEDDINGS_STATE_FILE)


def read_embeddings(model_dir, num_nodes: int, dim: int, mmap: bool = True):
    """(table, state or None), fp32 [num_nodes, dim]"""
    d = Path(model_dir)

    def load(path):
        if not path.exists():
            return None
        if path.stat().st_size != num_nodes * dim * 4:
            raise ValueError(f"{path}: expected {num_nodes} x {dim} float32")
        return np.memmap(path, dtype=np.float32, mode="r", shape=(num_nodes, dim)) if mmap else np.fromfile(path, np.float32).reshape(num_nodes, dim)

    table = load(d / EMBEDDINGS_FILE)
    if table is None:
        raise FileNotFoundError(d / EMBEDDINGS_FILE)
    return table, load(d / EMBEDDINGS_STATE_FILE)


def write_metadata(model_dir, name: str, num_epochs: int, checkpoint_id: int, link_prediction: bool = True, has_state: bool = True,
                   has_encoded: bool = False, has_model: bool = True):
    with open(Path(model_dir) / METADATA_FILE, "w") as f:
        for v in (name, num_epochs, checkpoint_id, int(link_prediction), int(has_state), int(has_encoded), int(has_model)):
            f.write(f"{v}\n")


def read_metadata(model_dir) -> Dict[str, object]:
    lines = open(Path(model_dir) / METADATA_FILE).read().splitlines()
    keys = ("name", "num_epochs", "checkpoint_id", "link_prediction", "has_state", "has_encoded", "has_model")
    out: Dict[str, object] = {"name": lines[0]}
    for k, v in zip(keys[1:3], lines[1:3]):
        out[k] = int(v)
    for k, v in zip(keys[3:], lines[3:7]):
        out[k] = bool(int(v))
    return out
