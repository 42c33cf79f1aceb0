"""Batch sampling: the contract of ``get_batch`` (coverage modelled on the
reference's tests/test_train_utils.py)."""
import numpy as np
import pytest
import torch

from b200moe.utils.data import BatchStager, get_batch, load_dataset
from implementation.train_utils import get_batch as shim_get_batch


def test_shim_is_same_function():
    assert shim_get_batch is get_batch


@pytest.mark.parametrize("vocab", [1, 17, 32000])
def test_mock_batch_shape_range_and_shift(vocab):
    x, y = get_batch(None, 4, 8, "cpu", vocab_size=vocab, mock_data=True, rng=np.random.default_rng(7),
                     validate=True)
    for t in (x, y):
        assert t.shape == (4, 8) and t.dtype == torch.long and t.is_contiguous()
        assert int(t.min()) >= 0 and int(t.max()) < vocab
    assert torch.equal(x[:, 1:], y[:, :-1])


def test_mock_batch_follows_generator_state():
    rng = np.random.default_rng(3)
    saved = rng.bit_generator.state
    a = get_batch(None, 2, 16, "cpu", rng=rng, vocab_size=50, mock_data=True)
    b = get_batch(None, 2, 16, "cpu", rng=rng, vocab_size=50, mock_data=True)
    assert not torch.equal(a[0], b[0])
    rng.bit_generator.state = saved
    c = get_batch(None, 2, 16, "cpu", rng=rng, vocab_size=50, mock_data=True)
    assert torch.equal(a[0], c[0]) and torch.equal(a[1], c[1])


@pytest.mark.parametrize("vocab", [None, 0, -5])
def test_mock_needs_positive_vocab(vocab):
    with pytest.raises(ValueError, match="vocab_size must be positive"):
        get_batch(None, 2, 4, "cpu", vocab_size=vocab, mock_data=True)


@pytest.mark.parametrize("batch,ctx", [(0, 4), (-2, 4), (2, 0), (2, -1)])
def test_dimensions_must_be_positive(batch, ctx):
    with pytest.raises(ValueError, match="must be positive"):
        get_batch(None, batch, ctx, "cpu", vocab_size=9, mock_data=True)


@pytest.mark.parametrize("serial", [False, True])
def test_dataset_windows(serial):
    tokens = np.arange(100, dtype=np.int64)
    x, y = get_batch(tokens, 4, 8, "cpu", serial_sampling=serial, start_idx=2, rng=np.random.default_rng(42),
                     vocab_size=100, validate=True)
    starts = np.arange(2, 34, 8) if serial else np.random.default_rng(42).integers(2, 92, size=4)
    want = np.stack([tokens[s:s + 8] for s in starts])
    assert torch.equal(x, torch.from_numpy(want))
    assert torch.equal(y, x + 1)


def test_dataset_validation_and_loading(tmp_path):
    path = tmp_path / "tokens.npy"
    np.save(path, np.arange(64, dtype=np.int32))
    tokens = load_dataset(path, vocab_size=64, validate=True)
    assert tokens.shape == (64,)
    with pytest.raises(ValueError, match="incompatible"):
        load_dataset(path, vocab_size=10, validate=True)
    np.save(path, np.zeros((4, 4), dtype=np.int32))
    with pytest.raises(ValueError, match="1D"):
        load_dataset(path)
    np.save(path, np.zeros(8, dtype=np.float32))
    with pytest.raises(TypeError, match="integer"):
        load_dataset(path)
    with pytest.raises(ValueError, match="Invalid input token range"):
        get_batch(np.arange(100), 2, 8, "cpu", vocab_size=10, validate=True, rng=np.random.default_rng(0))


def test_stager_matches_get_batch():
    stager = BatchStager(3, 8, "cpu")
    a = stager.next(None, np.random.default_rng(5), 100, mock_data=True)
    b = get_batch(None, 3, 8, "cpu", rng=np.random.default_rng(5), vocab_size=100, mock_data=True)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    assert stager.h2d_bytes == 2 * 3 * 8 * 8
