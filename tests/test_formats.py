"""The reference project's on-disk formats (edge files, bucket offsets, dataset.yaml, embedding files, checkpoint metadata):
what formats.py writes is laid out as the reference's writer lays it out, and reads back bit for bit."""
from importlib import import_module

import numpy as np
import pytest

import ge2_oracle as O


@pytest.fixture(scope="module")
def formats():
    return import_module("ge-2_b200.formats")


@pytest.mark.parametrize("cols,dtype", [(3, np.int32), (2, np.int64)])
def test_dataset_round_trip(formats, tmp_path, cols, dtype):
    rng = np.random.default_rng(1)
    nodes, R, P = 1000, 7 if cols == 3 else 1, 4
    mk = lambda n: np.stack([rng.integers(0, nodes, n)] + ([rng.integers(0, R, n)] if cols == 3 else []) + [rng.integers(0, nodes, n)], 1).astype(np.int64)
    train, valid, test = mk(5000), mk(300), mk(200)
    train_sorted, sizes = formats.partition_edges(train, nodes, P)
    # same buckets as the oracle's restatement of the preprocessor
    exp_sorted, exp_sizes = O.bucket_sort_edges(train, P, -(-nodes // P))
    assert np.array_equal(sizes, exp_sizes) and np.array_equal(train_sorted, exp_sorted)
    stats = formats.write_dataset(tmp_path, train_sorted, valid, test, nodes, R, P, dtype=dtype, offsets={"train": sizes})
    assert stats["num_train"] == 5000 and stats["num_valid"] == 300
    # byte layout: raw row-major ids, nothing else in the file
    raw = np.fromfile(tmp_path / "edges" / "train_edges.bin", dtype=dtype)
    assert raw.size == 5000 * cols and np.array_equal(raw.reshape(5000, cols), train_sorted.astype(dtype))
    assert (tmp_path / "edges" / "train_partition_offsets.txt").read_text().split() == [str(int(s)) for s in sizes]
    assert "num_nodes: 1000" in (tmp_path / "dataset.yaml").read_text()
    back = formats.read_dataset(tmp_path)
    assert back["stats"]["num_nodes"] == nodes and back["stats"]["num_relations"] == R and back["stats"]["initialized"] is False
    assert back["train"].dtype == dtype
    assert np.array_equal(back["train"], train_sorted) and np.array_equal(back["valid"], valid) and np.array_equal(back["test"], test)
    assert np.array_equal(back["offsets"]["train"], sizes)
    # the buckets really are where the offsets say
    psize = -(-nodes // P)
    begin = np.concatenate([[0], np.cumsum(sizes)])
    for b in (0, 5, P * P - 1):
        rows = np.asarray(back["train"][begin[b]:begin[b + 1]])
        assert np.all(rows[:, 0] // psize == b // P) and np.all(rows[:, -1] // psize == b % P)


def test_bad_files_are_refused(formats, tmp_path):
    rng = np.random.default_rng(2)
    train = rng.integers(0, 50, (100, 2)).astype(np.int64)
    with pytest.raises(ValueError):
        formats.write_dataset(tmp_path, train, None, None, 50, 1, 4)           # partitioned without offsets
    formats.write_dataset(tmp_path, train, None, None, 50, 1, 1)
    with open(tmp_path / "edges" / "train_edges.bin", "ab") as f:
        f.write(b"\0\0\0")
    with pytest.raises(ValueError):
        formats.read_dataset(tmp_path)


def test_embeddings_and_metadata_round_trip(formats, tmp_path):
    rng = np.random.default_rng(3)
    table = rng.standard_normal((123, 50)).astype(np.float32)
    state = rng.random((123, 50)).astype(np.float32)
    formats.write_embeddings(tmp_path, table, state)
    assert (tmp_path / "embeddings.bin").stat().st_size == 123 * 50 * 4
    t, s = formats.read_embeddings(tmp_path, 123, 50)
    assert np.array_equal(t, table) and np.array_equal(s, state)
    with pytest.raises(ValueError):
        formats.read_embeddings(tmp_path, 124, 50)
    formats.write_metadata(tmp_path, "run", 3, 7)
    assert (tmp_path / "metadata.csv").read_text().splitlines() == ["run", "3", "7", "1", "1", "0", "1"]
    m = formats.read_metadata(tmp_path)
    assert m == dict(name="run", num_epochs=3, checkpoint_id=7, link_prediction=True, has_state=True, has_encoded=False, has_model=True)
