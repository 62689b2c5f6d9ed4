"""The C++ host helpers against the Python packer (their oracle)."""
import random

import pytest
import torch

from chronicals_b200.data.sequence_packer import BinPackingAlgorithm, SequencePacker
from chronicals_b200.utils import native


@pytest.fixture(scope="module", autouse=True)
def _built():
    native.build()


@pytest.mark.parametrize("strategy", sorted(BinPackingAlgorithm.STRATEGIES))
def test_native_bins_equal_python_bins(strategy):
    rng = random.Random(7)
    for n, cap in [(0, 64), (1, 64), (17, 128), (300, 512), (2000, 2048)]:
        lens = [rng.randint(0, int(cap * 1.3)) for _ in range(n)]
        assert native.native_pack(lens, cap, strategy) == BinPackingAlgorithm.pack(lens, cap, strategy)


def test_native_pack_rejects_unknown_strategy():
    assert native.native_pack([1, 2, 3], 8, "no-such-strategy") is None


def test_fill_rows_matches_manual_layout():
    items = [[1, 2, 3], [4, 5], [6, 7, 8, 9]]
    out = native.native_fill_rows(items, [[2, 0], [1]], capacity=8, pad_id=0, ignore_index=-100)
    assert out["input_ids"].tolist() == [[6, 7, 8, 9, 1, 2, 3, 0], [4, 5, 0, 0, 0, 0, 0, 0]]
    assert out["labels"].tolist() == [[-100, 7, 8, 9, -100, 2, 3, -100], [-100, 5] + [-100] * 6]
    assert out["position_ids"].tolist() == [[0, 1, 2, 3, 0, 1, 2, 0], [0, 1, 0, 0, 0, 0, 0, 0]]
    assert out["sequence_ids"].tolist() == [[0, 0, 0, 0, 1, 1, 1, -1], [0, 0, -1, -1, -1, -1, -1, -1]]
    assert out["cu_seqlens"].tolist() == [[0, 4, 7], [0, 2, 2]]
    assert out["n_docs"].tolist() == [2, 1]


def test_fill_rows_truncates_to_capacity_and_uses_given_labels():
    items = [list(range(10)), [50, 51]]
    labels = [[-100] * 5 + list(range(5, 10)), None]
    out = native.native_fill_rows(items, [[0, 1]], capacity=8, labels=labels, mask_first_label=False)
    assert out["input_ids"].tolist() == [[0, 1, 2, 3, 4, 5, 6, 7]]
    assert out["labels"].tolist() == [[-100] * 5 + [5, 6, 7]]
    assert out["n_docs"].tolist() == [1]


def test_sequence_packer_uses_native_bins():
    rng = random.Random(3)
    seqs = [[rng.randint(1, 99) for _ in range(rng.randint(3, 40))] for _ in range(60)]
    p = SequencePacker(max_seq_length=64, strategy="bfd")
    batches = p.pack_all_sequences(seqs)
    total = sum(min(len(s), 64) for s in seqs)
    assert sum(int((b.input_ids != p.pad_token_id).sum()) for b in batches) <= total
    assert 0.5 < p.efficiency <= 1.0
    assert all(isinstance(b.input_ids, torch.Tensor) for b in batches)
