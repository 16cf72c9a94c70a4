"""Constant-size GLA state slots: the surface of vllm_hymeta/model_for_7B/gla_cache.py
(GLACacheParams, GLACacheManager) and of my_fused_recurrent_gla
(vllm_hymeta/model_for_7B/my_fused_recurrent.py:138-153), over the libsbk kernel.

Differences from the reference, all deliberate:
  * the state is float32 (the reference allocates bfloat16, modeling_gla_swa.py:361-364);
  * the state tensor is zero-initialised and a slot is zeroed when it is handed to a new
    sequence (the reference allocates with torch.empty and clears in
    GLAswaModel._clear_prefill_cache, modeling_gla_swa.py:391-414);
  * `_copy_cache` copies along the SLOT axis (the reference indexes the head axis,
    gla_cache.py:29-33).
"""
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from . import ops


@dataclass
class GLACacheParams:
    gla_cache: torch.Tensor = field(default_factory=torch.Tensor)
    state_indices_tensor: torch.Tensor = field(default_factory=torch.Tensor)

    def at_layer_idx(self, layer_idx: int) -> "GLACacheParams":
        return GLACacheParams(self.gla_cache[layer_idx, ...], self.state_indices_tensor)


class GLACacheManager:
    """State tensor [n_gla_layers, max_num_seqs, heads, D, D] plus the request -> slot map
    (the ConstantSizeCache behaviour the reference inherits): finished requests give their
    slot back, unseen sequences get a free slot, forked sequences copy their parent's."""

    def __init__(self, dtype: torch.dtype, cache_shape: Tuple[int, ...], device="cuda"):
        if dtype != torch.float32:
            raise ValueError("the GLA state of this implementation is float32")
        if len(cache_shape) != 5:
            raise ValueError("cache_shape must be (layers, max_num_seqs, heads, D, D)")
        self._gla_cache = torch.zeros(size=cache_shape, dtype=dtype, device=device)
        self.max_batch_size = cache_shape[1]
        self.cache_indices_mapping: Dict[str, Dict[int, int]] = {}
        self.free_cache_indices: List[int] = list(range(self.max_batch_size))

    @property
    def cache(self) -> torch.Tensor:
        return self._gla_cache

    def _copy_cache(self, from_index: int, to_index: int) -> None:
        self._gla_cache[:, to_index].copy_(self._gla_cache[:, from_index], non_blocking=True)

    def clear_slots(self, slots: Iterable[int]) -> None:
        slots = list(slots)
        if slots:
            idx = torch.tensor(slots, device=self._gla_cache.device, dtype=torch.long)
            self._gla_cache[:, idx] = 0

    def _release_finished(self, finished_requests_ids: Iterable[str]) -> None:
        for rid in finished_requests_ids:
            for slot in self.cache_indices_mapping.pop(rid, {}).values():
                self.free_cache_indices.append(slot)

    def _assign(self, rid: str, seq_id: int, to_clear: List[int]) -> int:
        seqs = self.cache_indices_mapping.setdefault(rid, {})
        if seq_id in seqs:
            return seqs[seq_id]
        if not self.free_cache_indices:
            raise RuntimeError("no free GLA state slot (max_num_seqs exceeded)")
        slot = self.free_cache_indices.pop()
        if seqs:  # a fork of a running request starts from its sibling's state
            self._copy_cache(next(iter(seqs.values())), slot)
        else:
            to_clear.append(slot)
        seqs[seq_id] = slot
        return slot

    def current_run_tensors(self, request_ids_to_seq_ids: Dict[str, List[int]],
                            finished_requests_ids: Optional[List[str]] = None,
                            pad_to: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """(state tensor, state_indices_tensor[int64]) for this step's sequences, in the order
        of ``request_ids_to_seq_ids``; ``pad_to`` appends -1 entries (captured-graph batches)."""
        self._release_finished(finished_requests_ids or [])
        to_clear: List[int] = []
        slots = [self._assign(rid, sid, to_clear) for rid, sids in request_ids_to_seq_ids.items() for sid in sids]
        self.clear_slots(to_clear)   # slots handed to new sequences start from a zero state, in one launch
        if pad_to is not None:
            slots += [-1] * (pad_to - len(slots))
        if len(set(s for s in slots if s >= 0)) != sum(1 for s in slots if s >= 0):
            raise RuntimeError("two sequences of one step share a GLA slot")
        idx = torch.tensor(slots, dtype=torch.int64, device=self._gla_cache.device)
        return self._gla_cache, idx


def my_fused_recurrent_gla(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor = None,
                           kv_caches: torch.Tensor = None, slot_idx: torch.Tensor = None,
                           scale: Optional[float] = None, initial_state: torch.Tensor = None,
                           output_final_state: bool = False, reverse: bool = False,
                           status: Optional[torch.Tensor] = None,
                           out: Optional[torch.Tensor] = None, **fused) -> torch.Tensor:
    """Single-token GLA decode, in place on ``kv_caches`` [slots, H, D, D] (float32).
    q [B, H, 1, D]; k, v, g [B, H, 1, D] or, un-repeated, [B, Hkv, 1, D]; returns o [B, H, D]
    in q's dtype (written into ``out`` [B, H, D] when given, e.g. a static buffer of a captured
    graph). Rows whose slot is -1 are left alone and their output row is unspecified.
    ``fused``: the keyword arguments of ops.gla_step that fold the layer's neighbours in
    (relu_qk, gate_logit_normalizer, norm_weight, norm_eps); see gla_decode_layer."""
    if q.dim() != 4 or q.shape[2] != 1:
        raise ValueError("q must be [B, H, 1, D] (one token per sequence)")
    if initial_state is not None or output_final_state or reverse:
        raise NotImplementedError("the decode step updates kv_caches in place; no other mode exists")
    B, H, _, D = q.shape
    if k.shape[0] != B or k.shape[2:] != (1, D) or v.shape != k.shape or g.shape != k.shape:
        raise ValueError("k, v, g must be [B, H or Hkv, 1, D]")
    sq = lambda t: t.reshape(B, t.shape[1], D).contiguous()
    if slot_idx is not None and slot_idx.dtype != torch.int64:
        slot_idx = slot_idx.to(torch.int64)
    return ops.gla_step(sq(q), sq(k), sq(v), sq(g), kv_caches, slot_idx, scale=scale, out=out,
                        status=status, **fused)


def gla_decode_layer(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gk: torch.Tensor,
                     kv_caches: torch.Tensor, slot_idx: torch.Tensor, g_norm_weight: torch.Tensor, *,
                     gate_logit_normalizer: float = 16.0, norm_eps: float = 1e-5,
                     scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
                     status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode branch of GatedLinearAttention.forward between the projections and the output gate
    (vllm_hymeta/model_for_7B/gla_attention.py:250-267 and _decode_infer :213-235) in ONE launch:
    q [B, H, D] and k, v, gk [B, Hkv, D] are the projection outputs as they come (no feature map,
    gate logits, kv heads not repeated); the kernel applies relu to q and k, turns gk into
    logsigmoid(gk) / gate_logit_normalizer, steps the slots' states, and applies g_norm
    (``g_norm_weight`` [D]) to the read-out. Returns o [B, H, D] in q's dtype."""
    if slot_idx is not None and slot_idx.dtype != torch.int64:
        slot_idx = slot_idx.to(torch.int64)
    return ops.gla_step(q.contiguous(), k.contiguous(), v.contiguous(), gk.contiguous(), kv_caches,
                        slot_idx, scale=scale, out=out, status=status, relu_qk=True,
                        gate_logit_normalizer=gate_logit_normalizer, norm_weight=g_norm_weight,
                        norm_eps=norm_eps)


def gla_prefill_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
                     kv_caches: torch.Tensor, slot_idx: torch.Tensor, query_start_loc: torch.Tensor,
                     context_lens: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                     status: Optional[torch.Tensor] = None, max_query_len: int = 0,
                     workspace: Optional[torch.Tensor] = None, **fused) -> torch.Tensor:
    """The prefill half of GatedLinearAttention._prefill_and_mix_infer
    (vllm_hymeta/model_for_7B/gla_attention.py:179-211) in one launch for all prompt sequences:
    q [T, H, D], k/v/g [T, H or Hkv, D] are the prompt tokens of `len(slot_idx)` sequences laid
    end to end (`query_start_loc`); each sequence's state slot is advanced over its tokens and the
    outputs [T, H, D] returned. A sequence whose `context_lens` entry is 0 is a new prompt and
    starts from a zero state whatever its slot holds (the reference zeroes such slots beforehand,
    modeling_gla_swa.py:391-414, and treats NaN-filled slots as empty, gla_attention.py:196-198).
    ``fused``: relu_qk, gate_logit_normalizer, norm_weight, norm_eps of ops.gla_scan.
    ``max_query_len`` (the metadata's host-side longest prompt run): when given, a call with few
    long runs spreads each run over several CTAs, the counterpart of the reference's chunk-parallel
    chunk_gla / fused_chunk_gla; ``workspace`` (ops.gla_scan_workspace) is allocated here if
    omitted."""
    reset = None
    if context_lens is not None:
        reset = (context_lens == 0).to(torch.uint8)
    if slot_idx.dtype != torch.int64:
        slot_idx = slot_idx.to(torch.int64)
    if max_query_len > 0 and workspace is None:
        workspace = ops.gla_scan_workspace(slot_idx.numel(), max_query_len, q.shape[1], q.shape[2], q.device)
    return ops.gla_scan(q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous(), kv_caches,
                        query_start_loc.to(torch.int32), slot_idx, reset, scale=scale, status=status,
                        max_query_len=max_query_len, workspace=workspace, **fused)
