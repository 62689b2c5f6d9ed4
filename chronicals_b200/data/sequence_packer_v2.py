"""Second-generation packer: flat, padding-free ``[total_tokens]`` batches for varlen attention.

Reference: chronicals/data/sequence_packer_v2.py:106-265 ``PackedBatchV2``, :272-410 cu_seqlens
helpers, :424-546 ``flash_attention_varlen``, :553-983 ``SequencePackerV2``, :990-1051 mask
builders, :1058-1183 loss and statistics helpers.  The flat layout is exactly what this
framework's decoder consumes (``[T, hidden]`` activations + ``cu_seqlens``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .sequence_packer import (IGNORE_INDEX, BinPackingAlgorithm, _as_ids_labels,
                              create_cu_seqlens_from_position_ids as compute_cu_seqlens_from_position_ids)


@dataclass
class PackedBatchV2:
    input_ids: torch.Tensor                 # [T]
    labels: torch.Tensor                    # [T]
    position_ids: torch.Tensor              # [T]
    cu_seqlens_q: torch.Tensor              # int32 [n + 1]
    cu_seqlens_k: torch.Tensor
    max_seqlen_q: int
    max_seqlen_k: int
    sequence_ids: Optional[torch.Tensor] = None     # [T] document index of every token (-1 for padding)
    loss_mask: Optional[torch.Tensor] = None
    num_sequences: int = 0
    sequence_lengths: List[int] = field(default_factory=list)
    num_padding_tokens: int = 0

    @property
    def total_tokens(self) -> int:
        return int(self.input_ids.numel())

    @property
    def num_real_tokens(self) -> int:
        return self.total_tokens - self.num_padding_tokens

    @property
    def packing_efficiency(self) -> float:
        return self.num_real_tokens / max(1, self.total_tokens)

    def to(self, device, non_blocking: bool = False) -> "PackedBatchV2":
        kw = dict(self.__dict__)
        for k, v in kw.items():
            if isinstance(v, torch.Tensor):
                kw[k] = v.to(device, non_blocking=non_blocking)
        return PackedBatchV2(**kw)

    def pin_memory(self) -> "PackedBatchV2":
        kw = dict(self.__dict__)
        for k, v in kw.items():
            if isinstance(v, torch.Tensor) and not v.is_cuda:
                kw[k] = v.pin_memory()
        return PackedBatchV2(**kw)

    def to_flash_attn_kwargs(self) -> Dict[str, Any]:
        return {"cu_seqlens_q": self.cu_seqlens_q, "cu_seqlens_k": self.cu_seqlens_k,
                "max_seqlen_q": self.max_seqlen_q, "max_seqlen_k": self.max_seqlen_k}

    def to_model_inputs(self) -> Dict[str, Any]:
        """Keyword arguments for ``CausalLM.forward`` / a trainer batch."""
        return {"input_ids": self.input_ids[None], "labels": self.labels[None], "position_ids": self.position_ids[None],
                "cu_seqlens": self.cu_seqlens_q, "max_seqlen": self.max_seqlen_q,
                "seqlens_host": list(self.sequence_lengths) + ([self.num_padding_tokens] if self.num_padding_tokens else [])}

    to_dict = to_model_inputs


def compute_cu_seqlens(sequence_lengths: Sequence[int], device=None) -> torch.Tensor:
    cu = torch.zeros(len(sequence_lengths) + 1, dtype=torch.int32)
    if len(sequence_lengths):
        cu[1:] = torch.cumsum(torch.as_tensor(list(sequence_lengths), dtype=torch.int32), 0)
    return cu.to(device) if device is not None else cu


def cu_seqlens_to_sequence_lengths(cu_seqlens: torch.Tensor) -> List[int]:
    return (cu_seqlens[1:] - cu_seqlens[:-1]).tolist()


def is_packed_sequence(position_ids: Optional[torch.Tensor]) -> bool:
    if position_ids is None or position_ids.numel() < 2:
        return False
    return bool((position_ids.reshape(-1)[1:] == 0).any().item())


def flash_attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                           cu_seqlens_k: Optional[torch.Tensor] = None, max_seqlen_q: Optional[int] = None,
                           max_seqlen_k: Optional[int] = None, causal: bool = True,
                           softmax_scale: Optional[float] = None) -> torch.Tensor:
    from ..ops import attention_varlen
    return attention_varlen(q, k, v, cu_seqlens_q, max_seqlen_q, causal, softmax_scale)


class SequencePackerV2:
    """Packs documents into flat batches of at most ``max_seq_length`` tokens.

    ``strategy``: ``greedy`` (in order, no sorting — keeps data order), ``ffd``, ``bfd``, ``spfhp``.
    ``fixed_output_shape`` pads every batch to exactly ``max_seq_length`` tokens (one padding
    segment at the end, labels ignored) so one CUDA graph serves all batches."""

    def __init__(self, max_seq_length: int = 4096, pad_token_id: int = 0, strategy: str = "greedy",
                 ignore_index: int = IGNORE_INDEX, mask_first_token: bool = True, generate_loss_mask: bool = True,
                 generate_sequence_ids: bool = True, fixed_output_shape: bool = False, dtype: torch.dtype = torch.long):
        self.max_seq_length, self.pad_token_id, self.strategy = int(max_seq_length), pad_token_id, strategy
        self.ignore_index, self.mask_first_token = ignore_index, mask_first_token
        self.generate_loss_mask, self.generate_sequence_ids = generate_loss_mask, generate_sequence_ids
        self.fixed_output_shape, self.dtype = fixed_output_shape, dtype

    def _bins(self, lengths: List[int]) -> List[List[int]]:
        if self.strategy == "greedy":
            return BinPackingAlgorithm.greedy_length_ordered(lengths, self.max_seq_length, sort=False)
        return BinPackingAlgorithm.pack(lengths, self.max_seq_length, self.strategy)

    def pack(self, sequences: Iterable[Any]) -> List[PackedBatchV2]:
        seqs = [_as_ids_labels(s) for s in sequences]
        lengths = [min(len(s[0]), self.max_seq_length) for s in seqs]
        return [self._build([seqs[i] for i in b]) for b in self._bins(lengths)] if seqs else []

    pack_all_sequences = pack

    def _build(self, seqs) -> PackedBatchV2:
        ids, labs, pos, sid, lens = [], [], [], [], []
        room = self.max_seq_length
        for di, (tok, labels) in enumerate(seqs):
            n = min(len(tok), room)
            if n <= 0:
                break
            x = torch.as_tensor(tok[:n], dtype=self.dtype)
            y = torch.as_tensor((labels if labels is not None else tok)[:n], dtype=self.dtype).clone()
            if self.mask_first_token and di > 0:
                y[0] = self.ignore_index
            ids.append(x)
            labs.append(y)
            pos.append(torch.arange(n, dtype=self.dtype))
            sid.append(torch.full((n,), di, dtype=self.dtype))
            lens.append(n)
            room -= n
        pad = room if self.fixed_output_shape else 0
        if pad:
            ids.append(torch.full((pad,), self.pad_token_id, dtype=self.dtype))
            labs.append(torch.full((pad,), self.ignore_index, dtype=self.dtype))
            pos.append(torch.arange(pad, dtype=self.dtype))
            sid.append(torch.full((pad,), -1, dtype=self.dtype))
        seg = lens + ([pad] if pad else [])
        cu = compute_cu_seqlens(seg)
        labels = torch.cat(labs)
        return PackedBatchV2(input_ids=torch.cat(ids), labels=labels, position_ids=torch.cat(pos), cu_seqlens_q=cu,
                             cu_seqlens_k=cu, max_seqlen_q=max(seg) if seg else 0, max_seqlen_k=max(seg) if seg else 0,
                             sequence_ids=torch.cat(sid) if self.generate_sequence_ids else None,
                             loss_mask=(labels != self.ignore_index).float() if self.generate_loss_mask else None,
                             num_sequences=len(lens), sequence_lengths=lens, num_padding_tokens=pad)


def create_block_causal_mask(cu_seqlens: torch.Tensor, total_tokens: Optional[int] = None) -> torch.Tensor:
    """Boolean ``[T, T]`` mask: token i may attend token j iff same document and j <= i."""
    T = int(total_tokens if total_tokens is not None else cu_seqlens[-1].item())
    idx = torch.arange(T, device=cu_seqlens.device)
    doc = torch.searchsorted(cu_seqlens[1:].long().contiguous(), idx, right=True)
    return (doc[:, None] == doc[None, :]) & (idx[None, :] <= idx[:, None])


def create_4d_attention_mask(cu_seqlens: torch.Tensor, total_tokens: Optional[int] = None,
                             dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Additive ``[1, 1, T, T]`` mask (0 / -inf) for attention implementations without varlen support."""
    m = create_block_causal_mask(cu_seqlens, total_tokens)
    out = torch.zeros(m.shape, dtype=dtype, device=m.device).masked_fill(~m, float("-inf"))
    return out[None, None]


def compute_packed_loss(per_token_loss: torch.Tensor, batch: PackedBatchV2, per_sequence: bool = False):
    """Mean over labelled tokens; with ``per_sequence`` also the mean loss of every document."""
    mask = batch.loss_mask if batch.loss_mask is not None else (batch.labels != IGNORE_INDEX).float()
    mask = mask.to(per_token_loss.device, per_token_loss.dtype)
    total = (per_token_loss * mask).sum() / mask.sum().clamp_min(1)
    if not per_sequence:
        return total
    b = batch.cu_seqlens_q.tolist()
    per = [((per_token_loss[s:e] * mask[s:e]).sum() / mask[s:e].sum().clamp_min(1)) for s, e in zip(b[:-1], b[1:])]
    return total, torch.stack(per[: batch.num_sequences]) if per else torch.zeros(0)


def compute_packing_statistics(batches: Sequence[PackedBatchV2], max_seq_length: Optional[int] = None) -> Dict[str, float]:
    real = sum(b.num_real_tokens for b in batches)
    cap = sum(max_seq_length or b.total_tokens for b in batches)
    docs = sum(b.num_sequences for b in batches)
    return {"num_batches": len(batches), "num_sequences": docs, "real_tokens": real, "capacity": cap,
            "packing_efficiency": real / cap if cap else 0.0,
            "avg_sequences_per_batch": docs / len(batches) if batches else 0.0}
