"""Token datasets and batch sampling.

``get_batch`` keeps the reference's contract (implementation/train_utils.py:46-141):
mock batches draw ``(B, ctx+1)`` ids from the caller's numpy generator and split
them into inputs and next-token targets; dataset batches copy windows at random
or serial starts; tensors are int64, staged in pinned memory and copied
asynchronously when the device is CUDA.  ``BatchStager`` adds a reusable pinned
staging area so the per-step host-to-device copy allocates nothing.
"""
from __future__ import annotations

import numpy as np
import torch

__all__ = ["load_dataset", "get_batch", "BatchStager"]


def load_dataset(path, vocab_size: int | None = None, validate: bool = False):
    """Memory-map a 1-D integer ``.npy`` token file (reference train_utils.py:12-31)."""
    tokens = np.load(path, mmap_mode="r")
    if tokens.ndim != 1:
        raise ValueError(f"Expected a 1D token dataset, got shape {tokens.shape}")
    if not np.issubdtype(tokens.dtype, np.integer):
        raise TypeError(f"Expected an integer token dataset, got dtype {tokens.dtype}")
    if validate:
        if vocab_size is None:
            raise ValueError("vocab_size must be provided when validate=True")
        low, high = int(tokens.min()), int(tokens.max())
        if low < 0 or high >= vocab_size:
            raise ValueError(
                f"Dataset token range [{low}, {high}] is incompatible with vocab_size={vocab_size}")
    return tokens


def _check_range(name: str, array: np.ndarray, vocab_size: int) -> None:
    low, high = int(array.min()), int(array.max())
    if low < 0 or high >= vocab_size:
        raise ValueError(f"Invalid {name} token range [{low}, {high}] for vocab_size={vocab_size}")


def _sample_numpy(tokens, batch_size, context_length, serial_sampling, start_idx, rng,
                  vocab_size, validate, mock_data):
    if rng is None:
        rng = np.random.default_rng()
    if batch_size <= 0:
        raise ValueError(f"batch_size must be positive, got {batch_size}")
    if context_length <= 0:
        raise ValueError(f"context_length must be positive, got {context_length}")
    if mock_data:
        if vocab_size is None or vocab_size <= 0:
            raise ValueError("vocab_size must be positive when mock_data=True")
        ids = rng.integers(low=0, high=vocab_size, size=(batch_size, context_length + 1), dtype=np.int64)
        inputs, targets = ids[:, :-1].copy(), ids[:, 1:].copy()
    else:
        if tokens.ndim != 1:
            raise ValueError(f"Expected a 1D token dataset, got shape {tokens.shape}")
        if not np.issubdtype(tokens.dtype, np.integer):
            raise TypeError(f"Expected an integer token dataset, got dtype {tokens.dtype}")
        if tokens.size <= context_length:
            raise ValueError(
                f"Dataset length {tokens.size} must be greater than context_length {context_length}")
        limit = tokens.size - context_length
        if serial_sampling:
            starts = np.arange(start_idx, min(start_idx + context_length * batch_size, limit),
                               context_length, dtype=np.int64)
        else:
            starts = rng.integers(low=start_idx, high=limit, size=batch_size, dtype=np.int64)
        window = np.arange(context_length + 1, dtype=np.int64)
        ids = np.asarray(tokens)[starts[:, None] + window[None, :]].astype(np.int64, copy=False)
        inputs, targets = np.ascontiguousarray(ids[:, :-1]), np.ascontiguousarray(ids[:, 1:])
    if validate:
        if vocab_size is None:
            raise ValueError("vocab_size must be provided when validate=True")
        _check_range("input", inputs, vocab_size)
        _check_range("target", targets, vocab_size)
    return inputs, targets


def get_batch(tokens, batch_size, context_length, device, serial_sampling: bool = False,
              start_idx: int = 0, rng: np.random.Generator | None = None,
              vocab_size: int | None = None, validate: bool = False, mock_data: bool = False):
    """Input and next-token target tensors of shape ``(batch, context)``, int64."""
    inputs, targets = _sample_numpy(tokens, batch_size, context_length, serial_sampling, start_idx,
                                    rng, vocab_size, validate, mock_data)
    x, y = torch.from_numpy(inputs), torch.from_numpy(targets)
    device = torch.device(device)
    if device.type == "cuda":
        x, y = x.pin_memory(), y.pin_memory()
    return x.to(device, non_blocking=True), y.to(device, non_blocking=True)


class BatchStager:
    """Pinned host staging plus device buffers reused every step.

    ``next(...)`` samples on the host with the same generator semantics as
    ``get_batch``, writes into the pinned pair and issues two async copies on
    the current stream; the returned device tensors are valid for the step that
    follows on that stream.  ``h2d_bytes`` is the byte count of one call.
    """

    def __init__(self, batch_size: int, context_length: int, device):
        self.device = torch.device(device)
        self.shape = (batch_size, context_length)
        pin = self.device.type == "cuda"
        self.host = [torch.empty(self.shape, dtype=torch.int64, pin_memory=pin) for _ in range(2)]
        self.dev = [torch.empty(self.shape, dtype=torch.int64, device=self.device) for _ in range(2)]
        self.h2d_bytes = 2 * self.host[0].numel() * 8

    def next(self, tokens, rng, vocab_size, validate=False, mock_data=False, **kwargs):
        inputs, targets = _sample_numpy(tokens, self.shape[0], self.shape[1],
                                        kwargs.get("serial_sampling", False), kwargs.get("start_idx", 0),
                                        rng, vocab_size, validate, mock_data)
        self.host[0].numpy()[...] = inputs
        self.host[1].numpy()[...] = targets
        for host, dev in zip(self.host, self.dev):
            dev.copy_(host, non_blocking=True)
        return self.dev[0], self.dev[1]
