"""Host-side data path (IDX readers, batch sampler, CSV log); no GPU needed.  Cases follow the
reference's own tests of the loader (hyperscalees-envs/src/snn_mnist.rs:262-312: round trip of a
hand-built IDX buffer, gzip detection, bad magic, truncated payload)."""
import gzip
import os
import struct

import numpy as np
import pytest

from hyperscalees_b200 import data


def idx_images(px: np.ndarray) -> bytes:
    n, rows, cols = px.shape
    return struct.pack(">IIII", 0x803, n, rows, cols) + px.astype(np.uint8).tobytes()


def idx_labels(lb: np.ndarray) -> bytes:
    return struct.pack(">II", 0x801, len(lb)) + lb.astype(np.uint8).tobytes()


def test_idx_round_trip_plain_and_gzip():
    px = np.arange(2 * 3 * 4, dtype=np.uint8).reshape(2, 3, 4) * 10
    for blob in (idx_images(px), gzip.compress(idx_images(px))):
        flat, n, per = data.read_idx_images(blob)
        assert (n, per) == (2, 12) and flat.dtype == np.float32
        assert np.array_equal(flat, px.reshape(-1).astype(np.float32) / np.float32(255.0))
    lb = np.array([3, 1, 4, 1, 5, 9], dtype=np.uint8)
    for blob in (idx_labels(lb), gzip.compress(idx_labels(lb))):
        assert np.array_equal(data.read_idx_labels(blob), lb)


def test_idx_errors():
    px = np.zeros((2, 2, 2), dtype=np.uint8)
    with pytest.raises(ValueError):
        data.read_idx_images(b"\x00" * 8)                                   # header too short
    with pytest.raises(ValueError):
        data.read_idx_images(struct.pack(">IIII", 0x801, 2, 2, 2) + b"\x00" * 8)   # labels magic
    with pytest.raises(ValueError):
        data.read_idx_images(idx_images(px)[:-1])                            # payload underflow
    with pytest.raises(ValueError):
        data.read_idx_labels(struct.pack(">II", 0x803, 1) + b"\x00")         # images magic
    with pytest.raises(ValueError):
        data.read_idx_labels(struct.pack(">II", 0x801, 5) + b"\x00" * 4)     # payload underflow
    with pytest.raises(ValueError):
        data.read_idx_images(struct.pack(">IIII", 0x803, 1 << 20, 1 << 10, 2))   # larger than the cap


def test_load_mnist_from_dir(tmp_path):
    rng = np.random.default_rng(0)
    shapes = {"train": 5, "test": 3}
    want = {}
    for (split, img_name), (_, lbl_name) in zip(data.IDX_IMAGES, data.IDX_LABELS):
        px = rng.integers(0, 256, (shapes[split], 28, 28), dtype=np.uint8)
        lb = rng.integers(0, 10, shapes[split], dtype=np.uint8)
        want[split] = (px, lb)
        (tmp_path / img_name).write_bytes(gzip.compress(idx_images(px)))
        # one file stored unpacked, without the suffix
        name = lbl_name[:-3] if split == "test" else lbl_name
        (tmp_path / name).write_bytes(idx_labels(lb) if split == "test" else gzip.compress(idx_labels(lb)))
    (tr_x, tr_y), (te_x, te_y) = data.load_mnist_from_dir(str(tmp_path))
    assert tr_x.shape == (5 * 784,) and te_x.shape == (3 * 784,)
    assert np.array_equal(tr_y, want["train"][1]) and np.array_equal(te_y, want["test"][1])
    assert np.allclose(te_x * 255.0, want["test"][0].reshape(-1))


def test_shuffled_indices_is_the_reference_stream():
    """accumulate_train.rs:157-174, restated independently with numpy uint64 wrap-around."""
    def ref(n, count, seed):
        state = np.uint64((seed ^ 0x9E3779B97F4A7C15) | 1)
        idx = list(range(n))
        with np.errstate(over="ignore"):
            for i in range(count):
                state ^= state << np.uint64(13)
                state ^= state >> np.uint64(7)
                state ^= state << np.uint64(17)
                r = int(state * np.uint64(0x2545F4914F6CDD1D))
                j = i + r % (n - i)
                idx[i], idx[j] = idx[j], idx[i]
        return idx[:count]
    for n, count, seed in ((10, 10, 0), (60000, 64, 42), (7, 3, 2**63 + 5)):
        got = data.shuffled_indices(n, count, seed)
        assert got == ref(n, count, seed)
        assert len(set(got)) == count and all(0 <= g < n for g in got)
    assert data.shuffled_indices(100, 10, 1) == data.shuffled_indices(100, 10, 1)
    assert data.shuffled_indices(100, 10, 1) != data.shuffled_indices(100, 10, 2)
    with pytest.raises(ValueError):
        data.shuffled_indices(3, 4, 0)


def test_csv_log_schema(tmp_path):
    path = tmp_path / "out" / "log.csv"
    log = data.CsvLog(str(path))
    log.row(0, 0.25, 0.5, 1.2345)
    log.row(1, 0.75, None, 0.5)
    log.row(2, 0.5, 0.4, 0.25)
    log.close()
    lines = path.read_text().splitlines()
    assert lines[0] == "epoch,train_acc,val_acc,best_val,best_train,epoch_time,cum_time"
    assert lines[1] == "0,0.250000,0.500000,0.500000,0.250000,1.234,1.2"
    assert lines[2] == "1,0.750000,,0.500000,0.750000,0.500,1.7"
    assert lines[3] == "2,0.500000,0.400000,0.500000,0.750000,0.250,2.0"
