"""Sequence packing: many short documents per fixed-length row, with the
metadata varlen attention needs (``cu_seqlens``, per-document ``position_ids``).

Public surface follows the reference (chronicals/data/sequence_packer.py:81-195
``PackedBatch``, :198-578 bin packing, :585-977 ``FixedShapeSequencePacker``,
:984-1068 cu_seqlens helpers, :1132-1342 prefetchers, :1349-1653 packed dataset
and loader, :1660-1906 helpers).  Differences on purpose: every bin is kept
(the reference's ``pack_sequences`` drops all bins after the first), the
heap-based best fit keeps exact remaining capacities, and ``cu_seqlens`` is
always produced (the reference only builds it when flash-attn imports).
"""
from __future__ import annotations

import bisect
import heapq
import random
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple, Union

import torch

IGNORE_INDEX = -100


# ----------------------------------------------------------------------------------------------- PackedBatch
@dataclass
class PackedBatch:
    input_ids: torch.Tensor                    # [rows, max_seq_length]
    position_ids: torch.Tensor                 # restarts at 0 for every document, 0 in padding
    labels: torch.Tensor                       # IGNORE_INDEX at padding (and first token of later documents)
    attention_mask: Optional[torch.Tensor] = None
    sequence_lengths: List[int] = field(default_factory=list)
    num_sequences: int = 0
    cu_seqlens: Optional[torch.Tensor] = None  # int32 [num_sequences + 1], padding excluded
    max_seqlen: int = 0
    sequence_boundaries: List[Tuple[int, int]] = field(default_factory=list)
    loss_mask: Optional[torch.Tensor] = None
    total_padding_tokens: int = 0
    packing_efficiency_cached: Optional[float] = None

    @property
    def use_varlen(self) -> bool:
        return self.cu_seqlens is not None

    @property
    def total_tokens(self) -> int:
        return int(sum(self.sequence_lengths))

    @property
    def batch_size(self) -> int:
        return int(self.input_ids.shape[0])

    @property
    def seq_length(self) -> int:
        return int(self.input_ids.shape[-1])

    @property
    def packing_efficiency(self) -> float:
        if self.packing_efficiency_cached is not None:
            return self.packing_efficiency_cached
        cap = self.input_ids.numel()
        return self.total_tokens / cap if cap else 0.0

    def _map(self, fn) -> "PackedBatch":
        kw = dict(self.__dict__)
        for k in ("input_ids", "position_ids", "labels", "attention_mask", "cu_seqlens", "loss_mask"):
            if kw[k] is not None:
                kw[k] = fn(kw[k])
        return PackedBatch(**kw)

    def to(self, device, non_blocking: bool = False) -> "PackedBatch":
        return self._map(lambda t: t.to(device, non_blocking=non_blocking))

    def pin_memory(self) -> "PackedBatch":
        return self._map(lambda t: t.pin_memory() if not t.is_cuda else t)

    def to_dict(self) -> Dict[str, Any]:
        d = {"input_ids": self.input_ids, "position_ids": self.position_ids, "labels": self.labels}
        if self.attention_mask is not None:
            d["attention_mask"] = self.attention_mask
        if self.cu_seqlens is not None:
            d["cu_seqlens"] = self.cu_seqlens
            d["max_seqlen"] = self.max_seqlen
        if self.loss_mask is not None:
            d["loss_mask"] = self.loss_mask
        d["seqlens_host"] = list(self.sequence_lengths)
        return d


# ----------------------------------------------------------------------------------------------- bin packing
@dataclass
class Bin:
    capacity: int
    items: List[int] = field(default_factory=list)     # indices into the length list
    used: int = 0

    @property
    def remaining(self) -> int:
        return self.capacity - self.used

    def fits(self, length: int) -> bool:
        return length <= self.remaining

    def add(self, index: int, length: int) -> None:
        self.items.append(index)
        self.used += length


class BinPackingAlgorithm:
    """Offline bin packing of sequence lengths into bins of ``capacity`` tokens.
    Every method returns a list of bins, each a list of indices into ``lengths``.
    Items longer than the capacity get a bin of their own (the packer truncates them)."""

    @staticmethod
    def _order(lengths: Sequence[int], descending: bool = True) -> List[int]:
        return sorted(range(len(lengths)), key=lambda i: lengths[i], reverse=descending)

    @staticmethod
    def first_fit_decreasing(lengths: Sequence[int], capacity: int) -> List[List[int]]:
        bins: List[Bin] = []
        for i in BinPackingAlgorithm._order(lengths):
            L = min(lengths[i], capacity)
            for b in bins:
                if b.fits(L):
                    b.add(i, L)
                    break
            else:
                nb = Bin(capacity)
                nb.add(i, L)
                bins.append(nb)
        return [b.items for b in bins]

    @staticmethod
    def best_fit_decreasing(lengths: Sequence[int], capacity: int) -> List[List[int]]:
        """Tightest bin that still fits; remaining capacities kept sorted for O(log n) lookup."""
        bins: List[Bin] = []
        rem: List[Tuple[int, int]] = []                 # sorted (remaining, bin index)
        for i in BinPackingAlgorithm._order(lengths):
            L = min(lengths[i], capacity)
            j = bisect.bisect_left(rem, (L, -1))
            if j < len(rem):
                r, bi = rem.pop(j)
                bins[bi].add(i, L)
                bisect.insort(rem, (r - L, bi))
            else:
                nb = Bin(capacity)
                nb.add(i, L)
                bins.append(nb)
                bisect.insort(rem, (capacity - L, len(bins) - 1))
        return [b.items for b in bins]

    @staticmethod
    def best_fit_decreasing_heap(lengths: Sequence[int], capacity: int) -> List[List[int]]:
        """Best fit via buckets of bins keyed by exact remaining capacity."""
        bins: List[Bin] = []
        buckets: Dict[int, List[int]] = {}
        keys: List[int] = []                             # sorted distinct remaining capacities in use
        for i in BinPackingAlgorithm._order(lengths):
            L = min(lengths[i], capacity)
            j = bisect.bisect_left(keys, L)
            if j < len(keys):
                r = keys[j]
                bi = buckets[r].pop()
                if not buckets[r]:
                    del buckets[r]
                    keys.pop(j)
            else:
                bins.append(Bin(capacity))
                bi, r = len(bins) - 1, capacity
            bins[bi].add(i, L)
            nr = r - L
            if nr not in buckets:
                buckets[nr] = []
                bisect.insort(keys, nr)
            buckets[nr].append(bi)
        return [b.items for b in bins]

    @staticmethod
    def shortest_pack_first_histogram(lengths: Sequence[int], capacity: int) -> List[List[int]]:
        """Histogram packing: longest first, each placed in the currently emptiest-fitting
        "open pack" chosen by a min-heap on fill level (balances bins)."""
        heap: List[Tuple[int, int]] = []                 # (used, bin index)
        bins: List[Bin] = []
        for i in BinPackingAlgorithm._order(lengths):
            L = min(lengths[i], capacity)
            placed = False
            if heap and heap[0][0] + L <= capacity:
                used, bi = heapq.heappop(heap)
                bins[bi].add(i, L)
                heapq.heappush(heap, (used + L, bi))
                placed = True
            if not placed:
                bins.append(Bin(capacity))
                bins[-1].add(i, L)
                heapq.heappush(heap, (L, len(bins) - 1))
        return [b.items for b in bins]

    @staticmethod
    def greedy_length_ordered(lengths: Sequence[int], capacity: int, sort: bool = True) -> List[List[int]]:
        """Fill the current bin until the next item does not fit, then open a new one."""
        order = BinPackingAlgorithm._order(lengths, descending=False) if sort else list(range(len(lengths)))
        out: List[List[int]] = []
        cur: List[int] = []
        used = 0
        for i in order:
            L = min(lengths[i], capacity)
            if used + L > capacity and cur:
                out.append(cur)
                cur, used = [], 0
            cur.append(i)
            used += L
        if cur:
            out.append(cur)
        return out

    STRATEGIES = {"ffd": "first_fit_decreasing", "bfd": "best_fit_decreasing", "bfd_heap": "best_fit_decreasing_heap",
                  "spfhp": "shortest_pack_first_histogram", "greedy": "greedy_length_ordered"}

    @classmethod
    def pack(cls, lengths: Sequence[int], capacity: int, strategy: str = "bfd") -> List[List[int]]:
        if strategy not in cls.STRATEGIES:
            raise ValueError(f"unknown packing strategy {strategy!r}; choose from {sorted(cls.STRATEGIES)}")
        return getattr(cls, cls.STRATEGIES[strategy])(lengths, capacity)


def _native_pack(lengths: Sequence[int], capacity: int, strategy: str) -> Optional[List[List[int]]]:
    """Use the C++ packer when it has been built (see csrc/host); otherwise None."""
    try:
        from ..utils.native import native_pack
    except Exception:
        return None
    return native_pack(lengths, capacity, strategy)


# ----------------------------------------------------------------------------------------------- packer
Seq = Union[Dict[str, Any], Sequence[int], torch.Tensor]


def _as_ids_labels(seq: Seq) -> Tuple[List[int], Optional[List[int]]]:
    if isinstance(seq, dict):
        ids = seq["input_ids"]
        labels = seq.get("labels")
    else:
        ids, labels = seq, None
    if isinstance(ids, torch.Tensor):
        ids = ids.reshape(-1).tolist()
    if isinstance(labels, torch.Tensor):
        labels = labels.reshape(-1).tolist()
    return list(ids), (list(labels) if labels is not None else None)


class FixedShapeSequencePacker:
    """Packs documents into rows of exactly ``max_seq_length`` tokens
    (static shapes: one CUDA graph serves every batch)."""

    def __init__(self, max_seq_length: int = 4096, pad_token_id: int = 0, strategy: str = "bfd",
                 use_flash_varlen: bool = True, generate_loss_mask: bool = True, generate_attention_mask: bool = True,
                 ignore_index: int = IGNORE_INDEX, mask_first_token_of_packed: bool = True,
                 dtype: torch.dtype = torch.long, padding_token_id: Optional[int] = None,
                 max_seq_len: Optional[int] = None):
        if max_seq_len is not None:          # keyword the reference's own trainer passes
            max_seq_length = max_seq_len
        self.max_seq_length = int(max_seq_length)
        self.pad_token_id = pad_token_id if padding_token_id is None else padding_token_id
        self.strategy = strategy
        self.use_flash_varlen = use_flash_varlen
        self.generate_loss_mask = generate_loss_mask
        self.generate_attention_mask = generate_attention_mask
        self.ignore_index = ignore_index
        self.mask_first_token_of_packed = mask_first_token_of_packed
        self.dtype = dtype
        # README-style counters
        self.original_tokens = 0
        self.packed_tokens = 0

    # -- API -------------------------------------------------------------------------------------------
    def pack_all_sequences(self, sequences: Iterable[Seq]) -> List[PackedBatch]:
        seqs = [_as_ids_labels(s) for s in sequences]
        if not seqs:
            return [self._empty_batch()]
        lengths = [min(len(s[0]), self.max_seq_length) for s in seqs]
        bins = _native_pack(lengths, self.max_seq_length, self.strategy) or \
            BinPackingAlgorithm.pack(lengths, self.max_seq_length, self.strategy)
        out = [self._create_batch_from_bin([seqs[i] for i in b]) for b in bins]
        self.original_tokens += sum(lengths)
        self.packed_tokens += len(out) * self.max_seq_length
        return out

    def pack_sequences(self, sequences: Iterable[Seq]) -> Union[PackedBatch, List[PackedBatch]]:
        """One ``PackedBatch`` when everything fits one row, otherwise the list of all rows."""
        batches = self.pack_all_sequences(sequences)
        return batches[0] if len(batches) == 1 else batches

    def pack(self, dataset: Iterable[Seq]) -> List[PackedBatch]:
        return self.pack_all_sequences(dataset)

    @property
    def efficiency(self) -> float:
        return self.original_tokens / self.packed_tokens if self.packed_tokens else 0.0

    # -- internals -------------------------------------------------------------------------------------
    def _empty_batch(self) -> PackedBatch:
        L = self.max_seq_length
        return PackedBatch(
            input_ids=torch.full((1, L), self.pad_token_id, dtype=self.dtype),
            position_ids=torch.zeros(1, L, dtype=self.dtype),
            labels=torch.full((1, L), self.ignore_index, dtype=self.dtype),
            attention_mask=None, sequence_lengths=[], num_sequences=0,
            cu_seqlens=torch.zeros(1, dtype=torch.int32), max_seqlen=0, sequence_boundaries=[],
            loss_mask=torch.zeros(1, L) if self.generate_loss_mask else None,
            total_padding_tokens=L, packing_efficiency_cached=0.0)

    def _create_batch_from_bin(self, seqs: List[Tuple[List[int], Optional[List[int]]]]) -> PackedBatch:
        L = self.max_seq_length
        ids = torch.full((L,), self.pad_token_id, dtype=self.dtype)
        pos = torch.zeros(L, dtype=self.dtype)
        lab = torch.full((L,), self.ignore_index, dtype=self.dtype)
        lens: List[int] = []
        bounds: List[Tuple[int, int]] = []
        o = 0
        for di, (tok, labels) in enumerate(seqs):
            n = min(len(tok), L - o)
            if n <= 0:
                break
            ids[o:o + n] = torch.as_tensor(tok[:n], dtype=self.dtype)
            pos[o:o + n] = torch.arange(n, dtype=self.dtype)
            lab[o:o + n] = torch.as_tensor((labels if labels is not None else tok)[:n], dtype=self.dtype)
            if self.mask_first_token_of_packed and di > 0:
                lab[o] = self.ignore_index
            lens.append(n)
            bounds.append((o, o + n))
            o += n
        cu = torch.tensor([0] + [b for _, b in bounds], dtype=torch.int32)
        mask = None
        if self.generate_attention_mask and not self.use_flash_varlen:
            mask = self._create_block_causal_mask(bounds, L)
        return PackedBatch(
            input_ids=ids[None], position_ids=pos[None], labels=lab[None], attention_mask=mask,
            sequence_lengths=lens, num_sequences=len(lens), cu_seqlens=cu, max_seqlen=max(lens) if lens else 0,
            sequence_boundaries=bounds, loss_mask=(lab != self.ignore_index).float()[None] if self.generate_loss_mask else None,
            total_padding_tokens=L - o, packing_efficiency_cached=o / L)

    @staticmethod
    def _create_block_causal_mask(bounds: List[Tuple[int, int]], L: int) -> torch.Tensor:
        """Additive ``[1, 1, L, L]`` mask: 0 inside each document's causal triangle, -inf elsewhere."""
        m = torch.full((L, L), float("-inf"))
        for a, b in bounds:
            n = b - a
            m[a:b, a:b] = torch.triu(torch.full((n, n), float("-inf")), diagonal=1)
        if bounds and bounds[-1][1] < L:                      # padding attends to itself only (keeps softmax finite)
            p = bounds[-1][1]
            idx = torch.arange(p, L)
            m[idx, idx] = 0.0
        return m[None, None]

    def create_attention_mask(self, sequence_ids: torch.Tensor, causal: bool = True) -> torch.Tensor:
        """Boolean ``[L, L]`` mask from per-token document ids (README-documented helper)."""
        same = sequence_ids[:, None] == sequence_ids[None, :]
        if causal:
            same = same & torch.ones_like(same).tril()
        return same

    def compute_packing_statistics(self, batches: Sequence[PackedBatch]) -> Dict[str, float]:
        tok = sum(b.total_tokens for b in batches)
        cap = sum(b.input_ids.numel() for b in batches)
        docs = sum(b.num_sequences for b in batches)
        return {"num_batches": len(batches), "num_sequences": docs, "total_tokens": tok, "capacity": cap,
                "padding_tokens": cap - tok, "packing_efficiency": tok / cap if cap else 0.0,
                "avg_sequences_per_batch": docs / len(batches) if batches else 0.0}


SequencePacker = FixedShapeSequencePacker


# ----------------------------------------------------------------------------------------------- cu_seqlens helpers
def create_cu_seqlens(sequence_lengths: Sequence[int], device=None) -> Tuple[torch.Tensor, int]:
    lens = torch.as_tensor(list(sequence_lengths), dtype=torch.int32)
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    return (cu.to(device) if device is not None else cu), int(lens.max()) if len(lens) else 0


def create_cu_seqlens_from_position_ids(position_ids: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """Document starts are where ``position_ids == 0``.  A run of consecutive zeros at the
    tail (padding) is folded into one segment so it does not become many length-1 documents.
    Reads the positions on the host (one synchronisation); the hot path passes ``cu_seqlens``."""
    flat = position_ids.reshape(-1)
    T = flat.numel()
    starts = (flat == 0).nonzero(as_tuple=True)[0].tolist()
    if not starts or starts[0] != 0:
        starts = [0] + starts
    end = T
    while len(starts) >= 2 and starts[-1] == end - 1 and starts[-2] == starts[-1] - 1:
        end = starts.pop()
    bounds = starts + [T]
    cu = torch.tensor(bounds, dtype=torch.int32, device=flat.device)
    max_len = max(b - a for a, b in zip(bounds[:-1], bounds[1:])) if T else 0
    return cu, int(max_len)


def apply_flash_attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                                 max_seqlen: int, causal: bool = True, softmax_scale: Optional[float] = None) -> torch.Tensor:
    from ..ops import attention_varlen
    return attention_varlen(q, k, v, cu_seqlens, max_seqlen, causal, softmax_scale)


# ----------------------------------------------------------------------------------------------- prefetchers
def _to_device(batch, device, non_blocking=True):
    if isinstance(batch, PackedBatch):
        return batch.to(device, non_blocking=non_blocking)
    if isinstance(batch, dict):
        return {k: (v.to(device, non_blocking=non_blocking) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
    if isinstance(batch, torch.Tensor):
        return batch.to(device, non_blocking=non_blocking)
    if isinstance(batch, (list, tuple)):
        return type(batch)(_to_device(b, device, non_blocking) for b in batch)
    return batch


def _record_stream(batch, stream):
    if isinstance(batch, PackedBatch):
        batch = batch.to_dict()
    if isinstance(batch, dict):
        batch = list(batch.values())
    if isinstance(batch, torch.Tensor):
        batch = [batch]
    for t in batch if isinstance(batch, (list, tuple)) else []:
        if isinstance(t, torch.Tensor) and t.is_cuda:
            t.record_stream(stream)


class DataPrefetcher:
    """Copies the next batch host→device on a side stream while the current one computes."""

    def __init__(self, loader: Iterable, device=None):
        self.loader = loader
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda" if torch.cuda.is_available() else "cpu")
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._it: Optional[Iterator] = None
        self._next = None

    def _preload(self) -> None:
        try:
            batch = next(self._it)
        except StopIteration:
            self._next = None
            return
        if self.stream is None:
            self._next = _to_device(batch, self.device, False)
            return
        with torch.cuda.stream(self.stream):
            self._next = _to_device(batch, self.device, True)

    def __iter__(self):
        self._it = iter(self.loader)
        self._preload()
        return self

    def __next__(self):
        if self._next is None:
            raise StopIteration
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
            _record_stream(self._next, torch.cuda.current_stream(self.device))
        batch = self._next
        self._preload()
        return batch

    def __len__(self):
        return len(self.loader)  # type: ignore[arg-type]


class DoubleBufferPrefetcher(DataPrefetcher):
    """Keeps two batches in flight (one more copy of look-ahead than ``DataPrefetcher``)."""

    def __iter__(self):
        self._it = iter(self.loader)
        self._queue: List[Any] = []
        for _ in range(2):
            self._preload()
            if self._next is not None:
                self._queue.append(self._next)
        return self

    def __next__(self):
        if not self._queue:
            raise StopIteration
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
            _record_stream(self._queue[0], torch.cuda.current_stream(self.device))
        batch = self._queue.pop(0)
        self._preload()
        if self._next is not None:
            self._queue.append(self._next)
        return batch


# ----------------------------------------------------------------------------------------------- dataset / loader
class PackedDataset(torch.utils.data.Dataset):
    """Pre-packs a dataset of tokenised samples (dicts with ``input_ids``/``labels``)."""

    def __init__(self, dataset: Sequence[Seq], packer: FixedShapeSequencePacker, batch_size: int = 64,
                 shuffle: bool = True, seed: int = 42, curriculum: bool = False, lazy: bool = False):
        self.dataset, self.packer, self.batch_size = dataset, packer, max(1, int(batch_size))
        self.shuffle, self.seed, self.curriculum, self.lazy = shuffle, seed, curriculum, lazy
        self.batches: List[PackedBatch] = []
        self._order: List[int] = []
        self._prepack_dataset()

    def _prepack_dataset(self) -> None:
        n = len(self.dataset)
        order = list(range(n))
        if self.curriculum:
            order.sort(key=lambda i: len(_as_ids_labels(self.dataset[i])[0]))
        elif self.shuffle:
            random.Random(self.seed).shuffle(order)
        self._order = order
        if self.lazy:
            return
        self.batches = []
        for s in range(0, n, self.batch_size):
            chunk = [self.dataset[i] for i in order[s:s + self.batch_size]]
            self.batches.extend(self.packer.pack_all_sequences(chunk))

    def __len__(self) -> int:
        if self.lazy:
            return (len(self.dataset) + self.batch_size - 1) // self.batch_size
        return len(self.batches)

    def __getitem__(self, i: int):
        if self.lazy:
            chunk = [self.dataset[j] for j in self._order[i * self.batch_size:(i + 1) * self.batch_size]]
            return self.packer.pack_all_sequences(chunk)[0]
        return self.batches[i]

    def get_statistics(self) -> Dict[str, float]:
        return self.packer.compute_packing_statistics(self.batches)


class PackedDataLoader:
    """Iterates ``PackedBatch`` objects, optionally through a device prefetcher."""

    def __init__(self, dataset: PackedDataset, shuffle: bool = False, device=None, use_prefetcher: bool = True,
                 double_buffer: bool = False, pin_memory: bool = True, seed: int = 42):
        self.dataset, self.shuffle, self.device, self.seed = dataset, shuffle, device, seed
        self.use_prefetcher = use_prefetcher and device is not None and torch.device(device).type == "cuda"
        self.double_buffer, self.pin_memory = double_buffer, pin_memory
        self._epoch = 0

    def _host_iter(self):
        idx = list(range(len(self.dataset)))
        if self.shuffle:
            random.Random(self.seed + self._epoch).shuffle(idx)
        self._epoch += 1
        for i in idx:
            b = self.dataset[i]
            yield b.pin_memory() if (self.pin_memory and torch.cuda.is_available()) else b

    def __iter__(self):
        if self.use_prefetcher:
            cls = DoubleBufferPrefetcher if self.double_buffer else DataPrefetcher
            return iter(cls(_Reiterable(self._host_iter), self.device))
        return self._host_iter()

    def __len__(self) -> int:
        return len(self.dataset)


SequencePackerDataLoader = PackedDataLoader


class _Reiterable:
    def __init__(self, fn):
        self.fn = fn

    def __iter__(self):
        return self.fn()


# ----------------------------------------------------------------------------------------------- helpers
def compute_padding_free_loss(per_token_loss: torch.Tensor, loss_mask: torch.Tensor) -> torch.Tensor:
    m = loss_mask.to(per_token_loss.dtype)
    return (per_token_loss * m).sum() / m.sum().clamp_min(1)


def compute_tokens_per_second(num_tokens: int, elapsed_s: float) -> float:
    return num_tokens / elapsed_s if elapsed_s > 0 else 0.0


class DynamicBatchSizeAdjuster:
    """Grows / shrinks the micro-batch from observed peak-memory fractions."""

    def __init__(self, initial: int = 2, minimum: int = 1, maximum: int = 64, target_utilization: float = 0.85):
        self.batch_size, self.minimum, self.maximum, self.target = initial, minimum, maximum, target_utilization

    def update(self, memory_fraction: float, oom: bool = False) -> int:
        if oom or memory_fraction > 0.97:
            self.batch_size = max(self.minimum, self.batch_size // 2)
        elif memory_fraction < self.target * 0.7:
            self.batch_size = min(self.maximum, self.batch_size * 2)
        elif memory_fraction < self.target:
            self.batch_size = min(self.maximum, self.batch_size + 1)
        return self.batch_size


def analyze_dataset_for_packing(lengths: Sequence[int], max_seq_length: int, strategy: str = "bfd") -> Dict[str, float]:
    lens = [min(int(l), max_seq_length) for l in lengths]
    if not lens:
        return {"num_sequences": 0, "packing_efficiency": 0.0, "padding_efficiency": 0.0, "speedup": 1.0, "num_bins": 0}
    bins = BinPackingAlgorithm.pack(lens, max_seq_length, strategy)
    tok = sum(lens)
    return {"num_sequences": len(lens), "mean_length": tok / len(lens), "max_length": max(lens),
            "num_bins": len(bins), "packing_efficiency": tok / (len(bins) * max_seq_length),
            "padding_efficiency": tok / (len(lens) * max_seq_length),
            "speedup": len(lens) / len(bins)}
