"""Datasets and loaders: MNIST IDX files, one-hot labels, accuracy, augmentations, batch
iteration with shuffling, and a prefetching loader that stages batches in pinned memory and
copies them to the device on a side stream.

Reference counterparts: cg_mnist_load / cg_mnist_get_batch / cg_labels_to_onehot /
augmentations / cg_data_iter_* (include/cg_datasets.h:17-78, src/datasets/mnist.c), and
cg_dataloader_* / cg_tensor_onehot / cg_tensor_argmax / cg_compute_accuracy
(src/utils/dataloader.c).
"""
from __future__ import annotations

import struct

import numpy as np
import torch


def load_mnist(images_path: str, labels_path: str):
    """Returns (images fp32 [N, rows*cols] in [0, 1], labels int64 [N])."""
    with open(images_path, "rb") as f:
        magic, n, rows, cols = struct.unpack(">IIII", f.read(16))
        if magic != 2051:
            raise ValueError(f"{images_path}: not an IDX image file (magic {magic})")
        img = np.frombuffer(f.read(n * rows * cols), dtype=np.uint8)
    with open(labels_path, "rb") as f:
        magic, n2 = struct.unpack(">II", f.read(8))
        if magic != 2049 or n2 != n:
            raise ValueError(f"{labels_path}: not the matching IDX label file")
        lab = np.frombuffer(f.read(n), dtype=np.uint8)
    if img.size != n * rows * cols or lab.size != n:
        raise ValueError("truncated IDX file")
    return torch.from_numpy(img.astype(np.float32) / 255.0).view(n, rows * cols), torch.from_numpy(lab.astype(np.int64))


def onehot(labels: torch.Tensor, num_classes: int) -> torch.Tensor:
    return torch.nn.functional.one_hot(labels.long(), num_classes).float()


def accuracy(logits: torch.Tensor, labels: torch.Tensor) -> float:
    want = labels if labels.dim() == 1 else labels.argmax(-1)
    return float((logits.argmax(-1) == want.to(logits.device)).float().mean())


def gaussian_noise_(x: torch.Tensor, std: float, generator=None) -> torch.Tensor:
    return x.add_(torch.randn(x.shape, generator=generator).to(x.device) * std)


def horizontal_flip_(x: torch.Tensor, prob: float, width: int | None = None, generator=None) -> torch.Tensor:
    """x: [N, rows*cols] (square unless `width` is given) or [N, ..., W]; flips whole samples."""
    N = x.shape[0]
    pick = torch.rand(N, generator=generator) < prob
    if x.dim() == 2:
        W = width or int(round(x.shape[1] ** 0.5))
        v = x.view(N, -1, W)
        v[pick] = v[pick].flip(-1)
    else:
        x[pick] = x[pick].flip(-1)
    return x


class BatchIterator:
    """Shuffling batch iterator over in-memory tensors (last batch may be short)."""

    def __init__(self, data: torch.Tensor, labels: torch.Tensor | None, batch_size: int, shuffle: bool = True, seed: int = 0,
                 drop_last: bool = False):
        if labels is not None and labels.shape[0] != data.shape[0]:
            raise ValueError("data and labels disagree on the number of samples")
        self.data, self.labels, self.bs, self.shuffle, self.seed, self.drop_last = data, labels, batch_size, shuffle, seed, drop_last
        self.epoch = 0

    def __len__(self):
        n = self.data.shape[0]
        return n // self.bs if self.drop_last else (n + self.bs - 1) // self.bs

    def __iter__(self):
        n = self.data.shape[0]
        if self.shuffle:
            order = torch.randperm(n, generator=torch.Generator().manual_seed(self.seed + self.epoch))
        else:
            order = torch.arange(n)
        self.epoch += 1
        for i in range(len(self)):
            idx = order[i * self.bs:(i + 1) * self.bs]
            yield self.data[idx], (None if self.labels is None else self.labels[idx])


class PrefetchLoader:
    """Wraps an iterable of (x, y) host batches: each batch is copied into one of two pinned
    staging buffers and sent to the device on a side stream while the previous one is in use."""

    def __init__(self, batches, device):
        self.batches, self.device = batches, torch.device(device)
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._pinned = [None, None]

    def __len__(self):
        return len(self.batches)

    def _stage(self, slot, x, y):
        if self.stream is None:
            return x, y
        bufs = self._pinned[slot]
        if bufs is None or bufs[0].shape != x.shape or (y is not None and bufs[1].shape != y.shape):
            bufs = (torch.empty(x.shape, dtype=x.dtype).pin_memory(), None if y is None else torch.empty(y.shape, dtype=y.dtype).pin_memory())
            self._pinned[slot] = bufs
        bufs[0].copy_(x)
        if y is not None:
            bufs[1].copy_(y)
        with torch.cuda.stream(self.stream):
            dx = bufs[0].to(self.device, non_blocking=True)
            dy = None if y is None else bufs[1].to(self.device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(self.stream)
        return dx, dy, ev

    def __iter__(self):
        nxt, slot = None, 0
        for x, y in self.batches:
            cur, nxt = nxt, self._stage(slot, x, y)
            slot ^= 1
            if cur is not None:
                yield self._ready(cur)
        if nxt is not None:
            yield self._ready(nxt)

    def _ready(self, staged):
        if self.stream is None:
            return staged[0], staged[1]
        dx, dy, ev = staged
        torch.cuda.current_stream(self.device).wait_event(ev)
        dx.record_stream(torch.cuda.current_stream(self.device))
        if dy is not None:
            dy.record_stream(torch.cuda.current_stream(self.device))
        return dx, dy


class SyntheticTokens:
    """Uniform random token ids with next-token targets, one fresh batch per step (what the
    benchmark configurations specify)."""

    def __init__(self, vocab_size: int, batch: int, seq_len: int, steps: int, seed: int = 0, pin: bool = False):
        self.V, self.B, self.T, self.steps, self.seed, self.pin = vocab_size, batch, seq_len, steps, seed, pin

    def __len__(self):
        return self.steps

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed)
        for _ in range(self.steps):
            ids = torch.randint(0, self.V, (self.B, self.T + 1), generator=g)
            x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
            yield (x.pin_memory(), y.pin_memory()) if self.pin else (x, y)
