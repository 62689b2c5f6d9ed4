"""Packers, cu_seqlens helpers, collators, datasets."""
import random

import pytest
import torch

from chronicals_b200.data import data_loader as dl
from chronicals_b200.data.sequence_packer import (BinPackingAlgorithm, FixedShapeSequencePacker, PackedBatch,
                                                  PackedDataset, PackedDataLoader, SequencePacker,
                                                  analyze_dataset_for_packing, create_cu_seqlens,
                                                  create_cu_seqlens_from_position_ids)


@pytest.mark.parametrize("strategy", ["ffd", "bfd", "bfd_heap", "spfhp", "greedy"])
def test_bin_packing_every_item_once_and_within_capacity(strategy):
    rng = random.Random(0)
    lengths = [rng.randint(1, 400) for _ in range(300)]
    bins = BinPackingAlgorithm.pack(lengths, 512, strategy)
    flat = sorted(i for b in bins for i in b)
    assert flat == list(range(300))
    assert all(sum(lengths[i] for i in b) <= 512 for b in bins)
    lower = -(-sum(lengths) // 512)
    assert len(bins) <= (2.0 if strategy == "greedy" else 1.35) * lower + 1


def test_bfd_variants_agree_on_bin_count():
    rng = random.Random(1)
    lengths = [rng.randint(10, 1000) for _ in range(500)]
    a = BinPackingAlgorithm.best_fit_decreasing(lengths, 1024)
    b = BinPackingAlgorithm.best_fit_decreasing_heap(lengths, 1024)
    assert len(a) == len(b)


def test_packer_output_contract():
    pk = FixedShapeSequencePacker(max_seq_length=32, pad_token_id=9, strategy="bfd")
    seqs = [{"input_ids": list(range(100, 110))}, {"input_ids": list(range(200, 215))}, {"input_ids": [1, 2, 3]},
            {"input_ids": list(range(300, 330))}]
    batches = pk.pack_all_sequences(seqs)
    assert all(isinstance(b, PackedBatch) and b.input_ids.shape == (1, 32) for b in batches)
    tokens = sorted(t for b in batches for t in b.input_ids[0, : b.total_tokens].tolist())
    assert tokens == sorted(t for s in seqs for t in s["input_ids"])
    for b in batches:
        cu = b.cu_seqlens.tolist()
        assert cu[0] == 0 and all(x < y for x, y in zip(cu, cu[1:])) and cu[-1] == b.total_tokens
        assert b.cu_seqlens.dtype == torch.int32 and b.max_seqlen == max(b.sequence_lengths)
        for di, (a, e) in enumerate(b.sequence_boundaries):
            assert b.position_ids[0, a:e].tolist() == list(range(e - a))
            if di > 0:
                assert b.labels[0, a].item() == -100          # first token of a later document is masked
        pad = b.total_tokens
        assert (b.labels[0, pad:] == -100).all() and (b.input_ids[0, pad:] == 9).all()
        assert (b.position_ids[0, pad:] == 0).all()
        assert torch.equal(b.loss_mask[0], (b.labels[0] != -100).float())
        assert abs(b.packing_efficiency - b.total_tokens / 32) < 1e-9
    assert pk.pack_sequences([]).cu_seqlens.tolist() == [0]
    assert SequencePacker is FixedShapeSequencePacker
    assert FixedShapeSequencePacker(max_seq_len=64).max_seq_length == 64      # the reference trainer's keyword


def test_block_causal_mask_when_varlen_is_off():
    pk = FixedShapeSequencePacker(max_seq_length=8, use_flash_varlen=False)
    b = pk.pack_all_sequences([[1, 2, 3], [4, 5]])[0]
    m = b.attention_mask[0, 0]
    assert m[2, 0] == 0 and m[0, 2] == float("-inf") and m[3, 2] == float("-inf") and m[4, 3] == 0


def test_cu_seqlens_helpers():
    cu, mx = create_cu_seqlens([3, 5, 2])
    assert cu.tolist() == [0, 3, 8, 10] and mx == 5
    pos = torch.tensor([0, 1, 2, 0, 1, 0, 1, 2, 3, 0, 0, 0])       # trailing padding
    cu2, mx2 = create_cu_seqlens_from_position_ids(pos)
    assert cu2.tolist() == [0, 3, 5, 9, 12] and mx2 == 4
    cu3, _ = create_cu_seqlens_from_position_ids(torch.arange(6))
    assert cu3.tolist() == [0, 6]


def test_synthetic_dataset_is_seeded_and_clipped():
    a = dl.SyntheticTokenDataset(50, 1000, "lognormal", seed=3, max_len=256)
    b = dl.SyntheticTokenDataset(50, 1000, "lognormal", seed=3, max_len=256)
    assert a.lengths == b.lengths and all(32 <= l <= 256 for l in a.lengths)
    assert torch.equal(a[7]["input_ids"], b[7]["input_ids"])


def test_packed_dataloader_and_micro_batches():
    ds = dl.SyntheticTokenDataset(64, 500, "lognormal", seed=0, max_len=128)
    loader = dl.create_packed_dataloader(ds, batch_size=2, max_length=256, pin_memory=False)
    n = 0
    for batch in loader:
        assert batch["input_ids"].shape == (1, 512)
        cu = batch["cu_seqlens"].tolist()
        assert cu[-1] == 512 and batch["max_seqlen"] == max(batch["seqlens_host"])
        n += 1
    assert n == len(loader) and n > 0
    # two ranks see disjoint rows
    r0 = list(dl.create_packed_dataloader(ds, 1, 256, rank=0, world_size=2, pin_memory=False))
    r1 = list(dl.create_packed_dataloader(ds, 1, 256, rank=1, world_size=2, pin_memory=False))
    assert len(r0) == len(r1) and not torch.equal(r0[0]["input_ids"], r1[0]["input_ids"])


def test_packed_dataset_statistics():
    ds = dl.SyntheticTokenDataset(40, 100, "lognormal", seed=1, max_len=64)
    pd = PackedDataset(ds, FixedShapeSequencePacker(128), batch_size=16)
    st = pd.get_statistics()
    assert st["total_tokens"] == sum(ds.lengths) and 0.5 < st["packing_efficiency"] <= 1.0
    assert len(list(PackedDataLoader(pd))) == len(pd)
    an = analyze_dataset_for_packing(ds.lengths, 128)
    assert an["speedup"] >= 1.0


class _Tok:
    pad_token_id = 0

    def encode(self, text, add_special_tokens=False):
        return [ord(c) % 251 + 1 for c in text]


def test_instruction_dataset_masks_prompt():
    data = [{"instruction": "add", "input": "1 2", "output": "3"}, {"instruction": "hi", "output": "there"}]
    for template in ("alpaca", "chatml", "llama", "dolly"):
        ds = dl.InstructionDataset(data, _Tok(), 512, template)
        s = ds[0]
        assert s["input_ids"].shape == s["labels"].shape
        n_masked = int((s["labels"] == -100).sum())
        assert 0 < n_masked < len(s["labels"])
        assert (s["labels"][n_masked:] == s["input_ids"][n_masked:]).all()


def test_collators_and_samplers():
    samples = [{"input_ids": [1, 2, 3]}, {"input_ids": [4, 5]}]
    b = dl.DataCollator(pad_token_id=0)(samples)
    assert b["input_ids"].shape == (2, 3) and b["labels"][1, 2] == -100 and b["attention_mask"].sum() == 5
    f = dl.DataCollatorWithFlattening()(samples)
    assert f["cu_seqlens"].tolist() == [0, 3, 5] and f["position_ids"].tolist() == [[0, 1, 2, 0, 1]]
    assert f["labels"][0, 3] == -100
    lengths = [5, 50, 7, 60, 6, 55]
    order = list(dl.LengthAwareSampler(lengths, 2, shuffle=False))
    assert sorted(order) == list(range(6)) and {order[0], order[1]} == {3, 5}
    cs = dl.CurriculumSampler(lengths, start_ratio=0.5, curriculum_epochs=2)
    assert set(cs) <= {0, 2, 4}
    cs.set_epoch(2)
    assert len(list(cs)) == 6
