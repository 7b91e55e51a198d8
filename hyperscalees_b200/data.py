"""Data side of the SNN-MNIST trainer: IDX readers, the deterministic batch sampler and the
CSV log of the training loop.  Host-only code (numpy); nothing here touches the GPU.

Mirrors hyperscalees-envs/src/snn_mnist.rs:14-130 (IDX parsing, gzip detection, limits and
error cases) and hyperscalees/src/bin/accumulate_train.rs:157-174, 698-708 (sampler, CSV
schema)."""
from __future__ import annotations

import gzip
import os
from typing import List, Optional, Tuple

import numpy as np

GZIP_MAGIC = b"\x1f\x8b"
IDX_MAGIC_IMAGES = 0x803
IDX_MAGIC_LABELS = 0x801
MAX_ELEMS = 1 << 30
IDX_IMAGES = (("train", "train-images-idx3-ubyte.gz"), ("test", "t10k-images-idx3-ubyte.gz"))
IDX_LABELS = (("train", "train-labels-idx1-ubyte.gz"), ("test", "t10k-labels-idx1-ubyte.gz"))
CSV_HEADER = "epoch,train_acc,val_acc,best_val,best_train,epoch_time,cum_time"
_U64 = (1 << 64) - 1


def _gunzip_if_needed(data: bytes) -> bytes:
    return gzip.decompress(data) if data[:2] == GZIP_MAGIC else data


def _be_u32(raw: bytes, offset: int) -> int:
    return int.from_bytes(raw[offset:offset + 4], "big")


def read_idx_images(data: bytes) -> Tuple[np.ndarray, int, int]:
    """snn_mnist.rs:57-88: (pixels / 255 as float32, flat; n; rows*cols).  Plain or gzipped."""
    raw = _gunzip_if_needed(data)
    if len(raw) < 16:
        raise ValueError("images IDX buffer too short for header")
    magic = _be_u32(raw, 0)
    if magic != IDX_MAGIC_IMAGES:
        raise ValueError(f"expected images magic 0x{IDX_MAGIC_IMAGES:x}, got 0x{magic:x}")
    n, rows, cols = _be_u32(raw, 4), _be_u32(raw, 8), _be_u32(raw, 12)
    per = rows * cols
    total = n * per
    if total > MAX_ELEMS:
        raise ValueError("images payload size out of range")
    if 16 + total > len(raw):
        raise ValueError("images payload underflow")
    px = np.frombuffer(raw, dtype=np.uint8, count=total, offset=16)
    return px.astype(np.float32) / np.float32(255.0), n, per


def read_idx_labels(data: bytes) -> np.ndarray:
    """snn_mnist.rs:91-108: raw uint8 labels."""
    raw = _gunzip_if_needed(data)
    if len(raw) < 8:
        raise ValueError("labels IDX buffer too short for header")
    magic = _be_u32(raw, 0)
    if magic != IDX_MAGIC_LABELS:
        raise ValueError(f"expected labels magic 0x{IDX_MAGIC_LABELS:x}, got 0x{magic:x}")
    n = _be_u32(raw, 4)
    if n > MAX_ELEMS or 8 + n > len(raw):
        raise ValueError("labels payload underflow")
    return np.frombuffer(raw, dtype=np.uint8, count=n, offset=8).copy()


def load_mnist_from_dir(path: str):
    """snn_mnist.rs:115-130: ((train_images, train_labels), (test_images, test_labels)); images are
    flat float32 in [0, 1], labels raw uint8.  The files carry the `.gz` names of the reference;
    an unpacked copy without the suffix is accepted as well."""
    def read(name: str) -> bytes:
        p = os.path.join(path, name)
        if not os.path.exists(p) and name.endswith(".gz") and os.path.exists(p[:-3]):
            p = p[:-3]
        with open(p, "rb") as fh:
            return fh.read()
    train = (read_idx_images(read(IDX_IMAGES[0][1]))[0], read_idx_labels(read(IDX_LABELS[0][1])))
    test = (read_idx_images(read(IDX_IMAGES[1][1]))[0], read_idx_labels(read(IDX_LABELS[1][1])))
    return train, test


def shuffled_indices(n: int, count: int, seed: int) -> List[int]:
    """accumulate_train.rs:157-174: the first `count` entries of a partial Fisher-Yates shuffle of
    0..n-1 driven by xorshift64 (13, 7, 17) times 0x2545F4914F6CDD1D, state = (seed ^ phi) | 1."""
    if count > n:
        raise ValueError(f"count({count}) must not exceed n({n})")
    state = ((seed & _U64) ^ 0x9E3779B97F4A7C15) | 1
    idx = list(range(n))
    for i in range(count):
        state ^= (state << 13) & _U64
        state ^= state >> 7
        state ^= (state << 17) & _U64
        r = (state * 0x2545F4914F6CDD1D) & _U64
        j = i + r % (n - i)
        idx[i], idx[j] = idx[j], idx[i]
    return idx[:count]


class CsvLog:
    """The trainer's per-epoch log (accumulate_train.rs:698-708): creates the directory, writes
    the header once, then one row per epoch; best values and cumulative time are tracked here."""

    def __init__(self, path: Optional[str]):
        self.path = path
        self.best_val = 0.0
        self.best_train = 0.0
        self.cum_time = 0.0
        self._fh = None
        if path:
            parent = os.path.dirname(path)
            if parent:
                os.makedirs(parent, exist_ok=True)
            self._fh = open(path, "w")
            self._fh.write(CSV_HEADER + "\n")

    def row(self, epoch: int, train_acc: float, val_acc: Optional[float], epoch_time: float) -> str:
        """One line in the reference's format (accumulate_train.rs:975-988): accuracies with six
        decimals (an epoch without validation leaves the field empty), epoch time with three,
        cumulative time with one."""
        if val_acc is not None:
            self.best_val = max(self.best_val, val_acc)
        self.best_train = max(self.best_train, train_acc)
        self.cum_time += epoch_time
        val = "" if val_acc is None else f"{val_acc:.6f}"
        line = (f"{epoch},{train_acc:.6f},{val},{self.best_val:.6f},{self.best_train:.6f},"
                f"{epoch_time:.3f},{self.cum_time:.1f}")
        if self._fh:
            self._fh.write(line + "\n")
            self._fh.flush()
        return line

    def close(self) -> None:
        if self._fh:
            self._fh.close()
            self._fh = None
