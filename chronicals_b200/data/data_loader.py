"""Datasets, collators, samplers and dataloader factories.

Mirrors the reference module (chronicals/data/data_loader.py:65-243 collators,
:250-496 instruction datasets with prompt masking, :503-666 samplers, :673-761
dataset loaders, :768-984 ``create_dataloader`` / ``create_packed_dataloader``,
:991-1305 helpers) and adds seeded synthetic token datasets, which is what the
benchmarks use (no network on the training machines).
"""
from __future__ import annotations

import math
import random
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence

import torch
from torch.utils.data import DataLoader, Dataset, IterableDataset, Sampler

from .sequence_packer import (IGNORE_INDEX, DataPrefetcher, FixedShapeSequencePacker, PackedBatch, PackedDataLoader,
                              PackedDataset)

# ------------------------------------------------------------------------------------------- prompt templates
PROMPT_TEMPLATES: Dict[str, Dict[str, str]] = {
    "alpaca": {
        "with_input": "### Instruction:\n{instruction}\n\n### Input:\n{input}\n\n### Response:\n{output}",
        "no_input": "### Instruction:\n{instruction}\n\n### Response:\n{output}",
        "response_marker": "### Response:",
    },
    "dolly": {
        "with_input": "### Instruction:\n{instruction}\n\n### Context:\n{input}\n\n### Response:\n{output}",
        "no_input": "### Instruction:\n{instruction}\n\n### Response:\n{output}",
        "response_marker": "### Response:",
    },
    "chatml": {
        "with_input": "<|im_start|>user\n{instruction}\n{input}<|im_end|>\n<|im_start|>assistant\n{output}<|im_end|>",
        "no_input": "<|im_start|>user\n{instruction}<|im_end|>\n<|im_start|>assistant\n{output}<|im_end|>",
        "response_marker": "<|im_start|>assistant",
    },
    "llama": {
        "with_input": "[INST] {instruction}\n{input} [/INST] {output}",
        "no_input": "[INST] {instruction} [/INST] {output}",
        "response_marker": "[/INST]",
    },
}


def format_example(example: Dict[str, Any], template: str = "alpaca") -> str:
    t = PROMPT_TEMPLATES[template]
    instruction = example.get("instruction") or example.get("question") or example.get("prompt") or ""
    inp = example.get("input") or example.get("context") or ""
    out = example.get("output") or example.get("response") or example.get("answer") or ""
    key = "with_input" if str(inp).strip() else "no_input"
    return t[key].format(instruction=instruction, input=inp, output=out)


def _find_subsequence(haystack: Sequence[int], needle: Sequence[int]) -> int:
    n = len(needle)
    if n == 0:
        return -1
    for i in range(len(haystack) - n + 1):
        if list(haystack[i:i + n]) == list(needle):
            return i
    return -1


# ------------------------------------------------------------------------------------------- collators
class DataCollator:
    """Pads ``input_ids`` / ``labels`` to the longest sample of the batch."""

    def __init__(self, pad_token_id: int = 0, ignore_index: int = IGNORE_INDEX, max_length: Optional[int] = None,
                 pad_to_multiple_of: Optional[int] = None):
        self.pad_token_id, self.ignore_index = pad_token_id, ignore_index
        self.max_length, self.pad_to_multiple_of = max_length, pad_to_multiple_of

    def __call__(self, samples: List[Dict[str, Any]]) -> Dict[str, torch.Tensor]:
        L = max(len(s["input_ids"]) for s in samples)
        if self.max_length:
            L = min(L, self.max_length)
        if self.pad_to_multiple_of:
            L = (L + self.pad_to_multiple_of - 1) // self.pad_to_multiple_of * self.pad_to_multiple_of
        ids = torch.full((len(samples), L), self.pad_token_id, dtype=torch.long)
        lab = torch.full((len(samples), L), self.ignore_index, dtype=torch.long)
        mask = torch.zeros(len(samples), L, dtype=torch.long)
        for i, s in enumerate(samples):
            x = torch.as_tensor(s["input_ids"], dtype=torch.long)[:L]
            y = torch.as_tensor(s.get("labels", s["input_ids"]), dtype=torch.long)[:L]
            ids[i, :len(x)], lab[i, :len(y)], mask[i, :len(x)] = x, y, 1
        return {"input_ids": ids, "labels": lab, "attention_mask": mask}


class DataCollatorWithFlattening:
    """Concatenates the samples into one padding-free row with ``cu_seqlens`` / ``position_ids``."""

    def __init__(self, ignore_index: int = IGNORE_INDEX, mask_first_token: bool = True):
        self.ignore_index, self.mask_first_token = ignore_index, mask_first_token

    def __call__(self, samples: List[Dict[str, Any]]) -> Dict[str, Any]:
        ids, lab, pos, lens = [], [], [], []
        for i, s in enumerate(samples):
            x = torch.as_tensor(s["input_ids"], dtype=torch.long)
            y = torch.as_tensor(s.get("labels", s["input_ids"]), dtype=torch.long).clone()
            if self.mask_first_token and i > 0 and len(y):
                y[0] = self.ignore_index
            ids.append(x)
            lab.append(y)
            pos.append(torch.arange(len(x)))
            lens.append(len(x))
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
        cu[1:] = torch.cumsum(torch.tensor(lens, dtype=torch.int32), 0)
        return {"input_ids": torch.cat(ids)[None], "labels": torch.cat(lab)[None], "position_ids": torch.cat(pos)[None],
                "cu_seqlens": cu, "max_seqlen": max(lens) if lens else 0, "seqlens_host": lens}


class PackingDataCollator:
    """Packs the samples of a batch into fixed-length rows and returns the ``PackedBatch`` list."""

    def __init__(self, packer: FixedShapeSequencePacker):
        self.packer = packer

    def __call__(self, samples: List[Dict[str, Any]]) -> List[PackedBatch]:
        return self.packer.pack_all_sequences(samples)


def stack_packed_rows(rows: Sequence[PackedBatch]) -> Dict[str, Any]:
    """Several one-row ``PackedBatch`` objects → one flat micro-batch ``[1, rows * L]`` whose
    ``cu_seqlens`` spans all rows (the padding tail of each row becomes its own masked segment)."""
    L = rows[0].seq_length
    ids = torch.cat([r.input_ids.reshape(-1) for r in rows])[None]
    lab = torch.cat([r.labels.reshape(-1) for r in rows])[None]
    pos = torch.cat([r.position_ids.reshape(-1) for r in rows])[None]
    lens: List[int] = []
    for r in rows:
        lens.extend(r.sequence_lengths)
        if r.total_padding_tokens:
            lens.append(r.total_padding_tokens)         # padding segment: labels are all ignore_index there
    if rows and rows[0].total_padding_tokens:           # positions inside padding segments count up, harmless
        pass
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens, dtype=torch.int32), 0)
    return {"input_ids": ids, "labels": lab, "position_ids": pos, "cu_seqlens": cu,
            "max_seqlen": max(lens) if lens else L, "seqlens_host": lens}


# ------------------------------------------------------------------------------------------- datasets
class InstructionDataset(Dataset):
    """Tokenises instruction data with a prompt template; labels before the response are masked."""

    def __init__(self, data: Sequence[Dict[str, Any]], tokenizer, max_length: int = 4096, template: str = "alpaca",
                 mask_prompt: bool = True, ignore_index: int = IGNORE_INDEX):
        if template not in PROMPT_TEMPLATES:
            raise ValueError(f"unknown template {template!r}")
        self.data, self.tok, self.max_length = data, tokenizer, max_length
        self.template, self.mask_prompt, self.ignore_index = template, mask_prompt, ignore_index
        marker = PROMPT_TEMPLATES[template]["response_marker"]
        self._marker_ids = self._encode(marker)

    def _encode(self, text: str) -> List[int]:
        try:
            return list(self.tok.encode(text, add_special_tokens=False))
        except TypeError:
            return list(self.tok.encode(text))

    def __len__(self) -> int:
        return len(self.data)

    def __getitem__(self, i: int) -> Dict[str, torch.Tensor]:
        text = format_example(self.data[i], self.template)
        ids = self._encode(text)[: self.max_length]
        labels = list(ids)
        if self.mask_prompt:
            at = _find_subsequence(ids, self._marker_ids)
            if at >= 0:
                end = at + len(self._marker_ids)
                labels[:end] = [self.ignore_index] * end
        return {"input_ids": torch.tensor(ids, dtype=torch.long), "labels": torch.tensor(labels, dtype=torch.long)}


class StreamingInstructionDataset(IterableDataset):
    """Same as ``InstructionDataset`` over an iterable source (nothing held in memory)."""

    def __init__(self, source: Iterable[Dict[str, Any]], tokenizer, max_length: int = 4096, template: str = "alpaca",
                 mask_prompt: bool = True):
        self.source = source
        self._proto = InstructionDataset([], tokenizer, max_length, template, mask_prompt)

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        for ex in self.source:
            self._proto.data = [ex]
            yield self._proto[0]


class SyntheticTokenDataset(Dataset):
    """Seeded uniform token ids in ``[0, vocab)``.

    ``lengths``: fixed int, or ``"lognormal"`` with ``mu/sigma`` clipped to ``[min_len, max_len]``
    (the variable-length document distribution of the LoRA benchmark configuration)."""

    def __init__(self, num_samples: int, vocab_size: int, lengths: Any = 1024, seed: int = 0, mu: float = 5.5,
                 sigma: float = 1.0, min_len: int = 32, max_len: int = 2048):
        g = torch.Generator().manual_seed(seed)
        if isinstance(lengths, int):
            self.lengths = [lengths] * num_samples
        elif lengths == "lognormal":
            raw = torch.empty(num_samples).log_normal_(mu, sigma, generator=g)
            self.lengths = raw.clamp(min_len, max_len).round().long().tolist()
        else:
            self.lengths = [int(x) for x in lengths]
        self.vocab_size, self.seed = vocab_size, seed

    def __len__(self) -> int:
        return len(self.lengths)

    def __getitem__(self, i: int) -> Dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        ids = torch.randint(0, self.vocab_size, (self.lengths[i],), generator=g)
        return {"input_ids": ids, "labels": ids.clone()}


# ------------------------------------------------------------------------------------------- samplers
class LengthAwareSampler(Sampler):
    """Batches samples of similar length (sorted inside shuffled mega-batches) to cut padding."""

    def __init__(self, lengths: Sequence[int], batch_size: int, shuffle: bool = True, seed: int = 42,
                 mega_batch_mult: int = 50):
        self.lengths, self.batch_size, self.shuffle, self.seed = list(lengths), batch_size, shuffle, seed
        self.mega = batch_size * mega_batch_mult
        self.epoch = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __iter__(self) -> Iterator[int]:
        idx = list(range(len(self.lengths)))
        rng = random.Random(self.seed + self.epoch)
        if self.shuffle:
            rng.shuffle(idx)
        out: List[int] = []
        for s in range(0, len(idx), self.mega):
            chunk = sorted(idx[s:s + self.mega], key=lambda i: self.lengths[i], reverse=True)
            batches = [chunk[b:b + self.batch_size] for b in range(0, len(chunk), self.batch_size)]
            if self.shuffle:
                rng.shuffle(batches)
            for b in batches:
                out.extend(b)
        return iter(out)

    def __len__(self) -> int:
        return len(self.lengths)


class CurriculumSampler(Sampler):
    """Short-to-long curriculum: epoch ``e`` draws from the shortest ``start_ratio → 1`` fraction."""

    def __init__(self, lengths: Sequence[int], start_ratio: float = 0.25, curriculum_epochs: int = 1, seed: int = 42):
        self.order = sorted(range(len(lengths)), key=lambda i: lengths[i])
        self.start_ratio, self.curriculum_epochs, self.seed = start_ratio, max(1, curriculum_epochs), seed
        self.epoch = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __iter__(self) -> Iterator[int]:
        frac = min(1.0, self.start_ratio + (1 - self.start_ratio) * self.epoch / self.curriculum_epochs)
        pool = self.order[: max(1, int(len(self.order) * frac))]
        random.Random(self.seed + self.epoch).shuffle(pool)
        return iter(pool)

    def __len__(self) -> int:
        frac = min(1.0, self.start_ratio + (1 - self.start_ratio) * self.epoch / self.curriculum_epochs)
        return max(1, int(len(self.order) * frac))


# ------------------------------------------------------------------------------------------- dataset loading
def load_dataset_hf(name: str, split: str = "train", max_samples: Optional[int] = None, **kw) -> List[Dict[str, Any]]:
    """HuggingFace ``datasets`` download; raises a clear error when offline."""
    try:
        from datasets import load_dataset
        ds = load_dataset(name, split=split, **kw)
    except Exception as e:
        raise RuntimeError(f"could not load dataset {name!r} (no network or not cached): {e}") from e
    if max_samples:
        ds = ds.select(range(min(max_samples, len(ds))))
    return [dict(x) for x in ds]


def load_alpaca(max_samples: Optional[int] = None):
    return load_dataset_hf("tatsu-lab/alpaca", max_samples=max_samples)


def load_dolly(max_samples: Optional[int] = None):
    return load_dataset_hf("databricks/databricks-dolly-15k", max_samples=max_samples)


def load_slimorca(max_samples: Optional[int] = None):
    return load_dataset_hf("Open-Orca/SlimOrca", max_samples=max_samples)


_LOADERS = {"alpaca": load_alpaca, "dolly": load_dolly, "slimorca": load_slimorca}


# ------------------------------------------------------------------------------------------- factories
class _MicroBatchLoader:
    """Groups pre-packed rows into micro-batches of ``batch_size`` rows (flat varlen layout),
    sharded round-robin across data-parallel ranks."""

    def __init__(self, rows: Sequence[PackedBatch], batch_size: int, rank: int = 0, world_size: int = 1,
                 shuffle: bool = False, seed: int = 42, pin_memory: bool = False, drop_last: bool = True):
        self.rows, self.batch_size, self.rank, self.world = list(rows), max(1, batch_size), rank, max(1, world_size)
        self.shuffle, self.seed, self.pin, self.drop_last = shuffle, seed, pin_memory, drop_last
        self.epoch = 0

    def __len__(self) -> int:
        per_rank = len(self.rows) // self.world
        return per_rank // self.batch_size if self.drop_last else math.ceil(per_rank / self.batch_size)

    def __iter__(self):
        idx = list(range(len(self.rows)))
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(idx)
        self.epoch += 1
        mine = idx[self.rank::self.world][: (len(idx) // self.world)]
        for s in range(0, len(mine), self.batch_size):
            chunk = [self.rows[i] for i in mine[s:s + self.batch_size]]
            if len(chunk) < self.batch_size and self.drop_last:
                break
            b = stack_packed_rows(chunk)
            if self.pin and torch.cuda.is_available():
                b = {k: (v.pin_memory() if isinstance(v, torch.Tensor) else v) for k, v in b.items()}
            yield b


def create_packed_dataloader(dataset: Sequence[Dict[str, Any]], batch_size: int = 1, max_length: int = 4096,
                             strategy: str = "bfd", use_packing: bool = True, pad_token_id: int = 0, seed: int = 42,
                             shuffle: bool = False, rank: int = 0, world_size: int = 1, pin_memory: bool = True,
                             mask_first_token: bool = True):
    """Tokenised samples → packed fixed-length rows → micro-batches of ``batch_size`` rows."""
    if not use_packing:
        coll = DataCollator(pad_token_id, max_length=max_length)
        # every rank gets the same number of samples (a rank with one batch more would start a step alone)
        idx = list(range(len(dataset)))[rank::world_size][: len(dataset) // max(1, world_size)]
        sub = [dataset[i] for i in idx]
        return DataLoader(sub, batch_size=batch_size, shuffle=shuffle, collate_fn=coll, drop_last=True)
    packer = FixedShapeSequencePacker(max_seq_length=max_length, pad_token_id=pad_token_id, strategy=strategy,
                                      mask_first_token_of_packed=mask_first_token)
    rows = packer.pack_all_sequences(dataset[i] for i in range(len(dataset)))
    return _MicroBatchLoader(rows, batch_size, rank, world_size, shuffle, seed, pin_memory)


def create_dataloader(dataset_name: str = "alpaca", tokenizer=None, batch_size: int = 1, max_length: int = 4096,
                      max_samples: Optional[int] = None, shuffle: bool = True, prompt_template: str = "alpaca",
                      use_packing: bool = True, packing_strategy: str = "bfd", use_prefetching: bool = True,
                      num_workers: int = 4, pin_memory: bool = True, device=None, curriculum_learning: bool = False,
                      curriculum_epochs: int = 1, vocab_size: int = 32000, seed: int = 42, data=None):
    """One call from a dataset name to a ready loader.  ``dataset_name="synthetic"`` (or ``data=`` a
    list of examples) works offline; named HF datasets need network access."""
    if data is None and dataset_name == "synthetic":
        ds: Any = SyntheticTokenDataset(max_samples or 1024, vocab_size, "lognormal", seed, max_len=max_length)
    else:
        raw = data if data is not None else (_LOADERS[dataset_name](max_samples) if dataset_name in _LOADERS
                                             else load_dataset_hf(dataset_name, max_samples=max_samples))
        if tokenizer is None:
            raise ValueError("a tokenizer is required for text datasets")
        ds = InstructionDataset(raw, tokenizer, max_length, prompt_template)
    if use_packing:
        packer = FixedShapeSequencePacker(max_seq_length=max_length, strategy=packing_strategy,
                                          pad_token_id=getattr(tokenizer, "pad_token_id", 0) or 0)
        pds = PackedDataset(ds, packer, batch_size=max(1, batch_size) * 4, shuffle=shuffle, seed=seed,
                            curriculum=curriculum_learning)
        return PackedDataLoader(pds, shuffle=shuffle, device=device, use_prefetcher=use_prefetching,
                                pin_memory=pin_memory, seed=seed)
    coll = DataCollator(getattr(tokenizer, "pad_token_id", 0) or 0, max_length=max_length)
    sampler = None
    if curriculum_learning:
        sampler = CurriculumSampler([len(ds[i]["input_ids"]) for i in range(len(ds))], curriculum_epochs=curriculum_epochs)
    dl = DataLoader(ds, batch_size=batch_size, shuffle=shuffle and sampler is None, sampler=sampler, collate_fn=coll,
                    num_workers=num_workers, pin_memory=pin_memory and torch.cuda.is_available(),
                    persistent_workers=num_workers > 0, prefetch_factor=2 if num_workers > 0 else None, drop_last=True)
    if use_prefetching and device is not None and torch.device(device).type == "cuda":
        return DataPrefetcher(dl, device)
    return dl


def get_tokenizer(model_name: str, **kw):
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(model_name, **kw)
    if tok.pad_token is None:
        tok.pad_token = tok.eos_token
    return tok


def analyze_dataset(dataset: Sequence[Dict[str, Any]], max_length: int = 4096) -> Dict[str, float]:
    lens = [min(len(dataset[i]["input_ids"]), max_length) for i in range(len(dataset))]
    if not lens:
        return {"num_samples": 0}
    s = sorted(lens)
    return {"num_samples": len(lens), "mean_length": sum(lens) / len(lens), "median_length": s[len(s) // 2],
            "p95_length": s[int(0.95 * (len(s) - 1))], "max_length": s[-1], "min_length": s[0],
            "total_tokens": sum(lens), "padding_waste_if_padded": 1 - sum(lens) / (len(lens) * max(lens))}


def estimate_training_throughput(num_params: float, peak_tflops: float = 2250.0, mfu: float = 0.4) -> float:
    """Tokens/s from the 6·N FLOPs-per-token rule."""
    return mfu * peak_tflops * 1e12 / (6.0 * num_params)


class ChronicalsDataPipeline:
    """dataset → (tokenise) → pack → micro-batches → device prefetch, with statistics."""

    def __init__(self, dataset: Sequence[Dict[str, Any]], batch_size: int = 1, max_length: int = 4096,
                 strategy: str = "bfd", device=None, seed: int = 42, rank: int = 0, world_size: int = 1):
        self.loader = create_packed_dataloader(dataset, batch_size, max_length, strategy, seed=seed, rank=rank,
                                               world_size=world_size)
        self.device = device
        self.stats = analyze_dataset(dataset, max_length)

    def __iter__(self):
        if self.device is not None and torch.device(self.device).type == "cuda":
            return iter(DataPrefetcher(self.loader, self.device))
        return iter(self.loader)

    def __len__(self) -> int:
        return len(self.loader)


def create_optimized_dataloader(dataset, batch_size: int = 1, max_length: int = 4096, device=None, **kw):
    return ChronicalsDataPipeline(dataset, batch_size, max_length, device=device, **kw)
