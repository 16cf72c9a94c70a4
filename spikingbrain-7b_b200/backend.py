"""The attention-backend surface of vllm_hymeta/attention/meta_attention.py over libsbk.

Mirrors, name for name and argument for argument, `MetaAttentionBackend` (:53-126),
`MetaAttentionMetadata` (:128-409), `MetaAttentionMetadataBuilder` (:411-608) and
`MetaAttentionImpl` (:611-982) of the reference, without importing vLLM: the few vLLM V0
helper types the reference leans on (`AttentionType`, `PAD_SLOT_ID`, the slot-mapping
helpers) are restated here from their documented behaviour.

What runs where
  cache write         -> sbk_kv_append / sbk_rope_kv_append (reference: reshape_and_cache_flash, :790-799)
  one-token decode    -> sbk_swa_decode  (reference: flash-attn fwd_kvcache, :955-981)
  prefill with tables -> sbk_swa_prefill (reference: flash-attn varlen forward with block
                         tables, :900-919): 16 query tokens x one kv group per CTA, tcgen05
  prompt run without block tables (the un-chunked first prompt, the memory-profiling run)
                      -> sbk_swa_prefill_dense over key/value as passed (reference :843-884)
  multi-token decode  -> sbk_swa_prefill, the queries being the tail of each sequence (:924-953)
  meta tokens         -> key2/value2 are streamed as extra always-visible leading tiles of the same
                         softmax (reference: second flash-attn pass + LSE merge,
                         fa_kernel_metatoken.py:124-194); the meta tokens' own queries (query2) run
                         non-causally over key2/value2 through sbk_swa_prefill_dense (:262-280)
  fp8 KV, ALiBi, soft-cap, encoder and cross attention, head sizes the kernels are not built for
                      -> NotImplementedError, never a fallback.
"""
from collections import defaultdict
from dataclasses import dataclass
from itertools import accumulate
from typing import Any, Dict, List, Optional, Tuple, Type

import torch

from . import ops

PAD_SLOT_ID = -1


class AttentionType:
    DECODER = "decoder"
    ENCODER = "encoder"
    ENCODER_ONLY = "encoder_only"
    ENCODER_DECODER = "encoder_decoder"


# ------------------------------------------------------------------ slot-mapping helpers
def is_block_tables_empty(block_tables) -> bool:
    """True for the memory-profiling run: no table at all, or only empty ones."""
    if block_tables is None:
        return True
    return isinstance(block_tables, dict) and all(v is None for v in block_tables.values())


def compute_slot_mapping_start_idx(is_prompt: bool, query_len: int, context_len: int,
                                   sliding_window: Optional[int]) -> int:
    """First position of a prompt that is still worth writing: tokens a sliding window will
    never look at again are masked out of the slot mapping."""
    if is_prompt and sliding_window is not None:
        return max(0, query_len - sliding_window)
    return 0


def compute_slot_mapping(is_profile_run: bool, slot_mapping: List[int], seq_id: int, seq_len: int,
                         context_len: int, start_idx: int, block_size: int,
                         block_tables: Dict[int, List[int]]) -> None:
    """Append the flat slots of positions context_len..seq_len-1 of one sequence."""
    if is_profile_run:
        slot_mapping.extend([PAD_SLOT_ID] * (seq_len - context_len))
        return
    masked = max(0, start_idx - context_len)
    slot_mapping.extend([PAD_SLOT_ID] * masked)
    table = block_tables[seq_id]
    for pos in range(max(start_idx, context_len), seq_len):
        slot_mapping.append(table[pos // block_size] * block_size + pos % block_size)


def _to_device(data, dtype, device, pin_memory=False) -> torch.Tensor:
    t = torch.tensor(data, dtype=dtype, pin_memory=pin_memory and torch.cuda.is_available(), device="cpu")
    return t.to(device=device, non_blocking=True)


def _pad_tables(tables: List[List[int]], pad: int, device) -> torch.Tensor:
    width = max((len(t) for t in tables), default=0)
    out = torch.full((len(tables), width), pad, dtype=torch.int32)
    for i, t in enumerate(tables):
        if t:
            out[i, :len(t)] = torch.as_tensor(t, dtype=torch.int32)
    return out.to(device=device, non_blocking=True)


# ----------------------------------------------------------------------------- backend
class MetaAttentionBackend:

    accept_output_buffer: bool = True

    @staticmethod
    def get_supported_head_sizes() -> List[int]:
        """The reference lists 32 ... 256 in steps of 32 (meta_attention.py:57-59, what flash-attn
        takes); the kernels here are built for the head size of the 7B model only, and the list says
        so instead of advertising sizes whose construction would then fail."""
        return [128]

    @staticmethod
    def get_name() -> str:
        return "META_FLASH_ATTN"

    @staticmethod
    def get_impl_cls() -> Type["MetaAttentionImpl"]:
        return MetaAttentionImpl

    @staticmethod
    def get_metadata_cls() -> Type["MetaAttentionMetadata"]:
        return MetaAttentionMetadata

    @staticmethod
    def get_builder_cls() -> Type["MetaAttentionMetadataBuilder"]:
        return MetaAttentionMetadataBuilder

    @staticmethod
    def get_state_cls():
        raise NotImplementedError("CommonAttentionState belongs to the serving engine, not to this path")

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int,
                           head_size: int) -> Tuple[int, ...]:
        if block_size % 16 != 0 or block_size < 16:
            raise ValueError(
                f"Invalid block size {block_size}. Must be a multiple of 16 and at least 16.")
        return (2, num_blocks, block_size, num_kv_heads, head_size)

    @staticmethod
    def swap_blocks(src_kv_cache: torch.Tensor, dst_kv_cache: torch.Tensor,
                    scr_to_dst: torch.Tensor) -> None:
        """Copy whole blocks between two caches (preemption); `scr_to_dst` is [n, 2] int64."""
        pairs = scr_to_dst.to("cpu").tolist()
        for src, dst in pairs:
            dst_kv_cache[:, dst].copy_(src_kv_cache[:, src], non_blocking=True)

    @staticmethod
    def copy_blocks(kv_caches: List[torch.Tensor], src_to_dists: torch.Tensor) -> None:
        """Copy blocks inside every layer's cache (beam fork); `src_to_dists` is [n, 2] int64."""
        src = src_to_dists[:, 0].long()
        dst = src_to_dists[:, 1].long()
        for kv in kv_caches:
            kv[:, dst.to(kv.device)] = kv[:, src.to(kv.device)]


@dataclass
class MetaAttentionMetadata:
    # fields of the engine's base metadata class
    num_prefills: int
    num_prefill_tokens: int
    num_decode_tokens: int
    slot_mapping: Optional[torch.Tensor]
    # fields of the reference subclass (meta_attention.py:131-204)
    seq_lens: Optional[List[int]]
    seq_lens_tensor: Optional[torch.Tensor]
    max_prefill_seq_len: int
    max_decode_seq_len: int
    context_lens_tensor: Optional[torch.Tensor]
    block_tables: Optional[torch.Tensor]
    use_cuda_graph: bool
    multi_modal_placeholder_index_maps: Optional[Dict[str, Any]] = None
    enable_kv_scales_calculation: bool = True
    max_query_len: Optional[int] = None
    max_decode_query_len: Optional[int] = None
    query_start_loc: Optional[torch.Tensor] = None
    seq_start_loc: Optional[torch.Tensor] = None
    _cached_prefill_metadata: Optional["MetaAttentionMetadata"] = None
    _cached_decode_metadata: Optional["MetaAttentionMetadata"] = None
    encoder_seq_lens: Optional[List[int]] = None
    encoder_seq_lens_tensor: Optional[torch.Tensor] = None
    encoder_seq_start_loc: Optional[torch.Tensor] = None
    max_encoder_seq_len: Optional[int] = None
    num_encoder_tokens: Optional[int] = None
    cross_slot_mapping: Optional[torch.Tensor] = None
    cross_block_tables: Optional[torch.Tensor] = None

    @property
    def is_all_encoder_attn_metadata_set(self) -> bool:
        return (self.encoder_seq_lens is not None and self.encoder_seq_lens_tensor is not None
                and self.max_encoder_seq_len is not None)

    @property
    def is_all_cross_attn_metadata_set(self) -> bool:
        return (self.is_all_encoder_attn_metadata_set and self.cross_slot_mapping is not None
                and self.cross_block_tables is not None)

    @property
    def prefill_metadata(self) -> Optional["MetaAttentionMetadata"]:
        """The prefill sequences (they come first in every per-sequence field) as a view."""
        if self.num_prefills == 0:
            return None
        if self._cached_prefill_metadata is not None:
            return self._cached_prefill_metadata
        assert (self.seq_lens is not None) or (self.encoder_seq_lens is not None)
        assert (self.seq_lens_tensor is not None) or (self.encoder_seq_lens_tensor is not None)
        n = self.num_prefills
        cut = lambda t, m: None if t is None else t[:m]
        self._cached_prefill_metadata = MetaAttentionMetadata(
            num_prefills=n, num_prefill_tokens=self.num_prefill_tokens, num_decode_tokens=0,
            slot_mapping=cut(self.slot_mapping, self.num_prefill_tokens),
            multi_modal_placeholder_index_maps=self.multi_modal_placeholder_index_maps,
            enable_kv_scales_calculation=self.enable_kv_scales_calculation,
            seq_lens=cut(self.seq_lens, n), seq_lens_tensor=cut(self.seq_lens_tensor, n),
            max_query_len=self.max_query_len, max_prefill_seq_len=self.max_prefill_seq_len,
            max_decode_query_len=0, max_decode_seq_len=0,
            query_start_loc=cut(self.query_start_loc, n + 1),
            seq_start_loc=cut(self.seq_start_loc, n + 1),
            context_lens_tensor=cut(self.context_lens_tensor, n),
            block_tables=cut(self.block_tables, n), use_cuda_graph=False,
            encoder_seq_lens=self.encoder_seq_lens,
            encoder_seq_lens_tensor=self.encoder_seq_lens_tensor,
            encoder_seq_start_loc=self.encoder_seq_start_loc,
            max_encoder_seq_len=self.max_encoder_seq_len,
            cross_slot_mapping=self.cross_slot_mapping, cross_block_tables=self.cross_block_tables)
        return self._cached_prefill_metadata

    @property
    def decode_metadata(self) -> Optional["MetaAttentionMetadata"]:
        """The decode sequences (after the prefills) as a view; query offsets rebased to 0."""
        if self.num_decode_tokens == 0:
            return None
        if self._cached_decode_metadata is not None:
            return self._cached_decode_metadata
        assert (self.seq_lens_tensor is not None) or (self.encoder_seq_lens_tensor is not None)
        n = self.num_prefills
        rest = lambda t, m: None if t is None else t[m:]
        self._cached_decode_metadata = MetaAttentionMetadata(
            num_prefills=0, num_prefill_tokens=0, num_decode_tokens=self.num_decode_tokens,
            slot_mapping=rest(self.slot_mapping, self.num_prefill_tokens),
            multi_modal_placeholder_index_maps=None, enable_kv_scales_calculation=True,
            seq_lens=None, seq_lens_tensor=rest(self.seq_lens_tensor, n),
            max_decode_query_len=self.max_decode_query_len, max_query_len=self.max_query_len,
            max_prefill_seq_len=0, max_decode_seq_len=self.max_decode_seq_len,
            query_start_loc=(self.query_start_loc[n:] - self.query_start_loc[n])
            if self.query_start_loc is not None else None,
            seq_start_loc=rest(self.seq_start_loc, n), context_lens_tensor=None,
            block_tables=rest(self.block_tables, n), use_cuda_graph=self.use_cuda_graph,
            encoder_seq_lens=self.encoder_seq_lens,
            encoder_seq_lens_tensor=self.encoder_seq_lens_tensor,
            encoder_seq_start_loc=self.encoder_seq_start_loc,
            max_encoder_seq_len=self.max_encoder_seq_len,
            cross_slot_mapping=self.cross_slot_mapping, cross_block_tables=self.cross_block_tables)
        return self._cached_decode_metadata

    def advance_step(self, model_input, sampled_token_ids: Optional[torch.Tensor], block_size: int,
                     num_seqs: int, num_queries: int, turn_prefills_into_decodes: bool = False):
        """Advance a decode-only batch by one token in place, on the device: lengths grow by one
        and every query's slot becomes the next position of its sequence (the work of
        ops.advance_step_flashattn in the reference, :401-409)."""
        if num_seqs != num_queries:
            assert num_seqs > num_queries
            assert self.use_cuda_graph
        if turn_prefills_into_decodes:
            assert self.num_decode_tokens + self.num_prefills == num_seqs
            self.num_decode_tokens += self.num_prefills
            self.num_prefills = 0
            self.num_prefill_tokens = 0
            self.max_prefill_seq_len = 0
            self.max_query_len = 1
            self.slot_mapping = self.slot_mapping[:num_seqs]
        else:
            assert self.seq_lens is not None
            assert self.max_decode_seq_len == max(self.seq_lens)
        assert self.num_prefills == 0 and self.num_prefill_tokens == 0
        assert self.num_decode_tokens == num_seqs
        assert self.slot_mapping.shape == (num_seqs, )
        assert self.seq_lens is not None and len(self.seq_lens) == num_seqs
        assert self.seq_lens_tensor is not None and self.seq_lens_tensor.shape == (num_seqs, )
        assert self.max_query_len == 1 and self.max_prefill_seq_len == 0
        assert self.query_start_loc is not None and self.query_start_loc.shape == (num_queries + 1, )
        assert self.seq_start_loc is not None and self.seq_start_loc.shape == (num_seqs + 1, )
        assert self.context_lens_tensor is not None and self.context_lens_tensor.shape == (num_queries, )
        assert self.block_tables is not None and self.block_tables.shape[0] == num_seqs
        for i in range(num_queries):
            self.seq_lens[i] += 1
        self.max_decode_seq_len = max(self.seq_lens)
        q = num_queries
        if model_input is not None and sampled_token_ids is not None:
            model_input.input_tokens[:q] = sampled_token_ids[:q].reshape(-1)
        pos = self.seq_lens_tensor[:q].long()          # position of the token that comes next
        if model_input is not None:
            model_input.input_positions[:q] = pos
        self.seq_lens_tensor[:q] += 1
        blk = torch.gather(self.block_tables[:q].long(), 1, (pos // block_size).unsqueeze(1)).squeeze(1)
        self.slot_mapping[:q] = blk * block_size + pos % block_size


class MetaAttentionMetadataBuilder:
    """Collects per-sequence data of one scheduler step and uploads it as MetaAttentionMetadata.
    `input_builder` is the engine's model-input builder; the attributes read from it and from
    its `inter_data_list` entries are those the reference reads (:415-494, :532-583)."""

    def __init__(self, input_builder):
        self.input_builder = input_builder
        self.runner = input_builder.runner
        self.sliding_window = input_builder.sliding_window
        self.block_size = input_builder.block_size

    def prepare(self):
        self.slot_mapping: List[int] = []
        self.prefill_seq_lens: List[int] = []
        self.context_lens: List[int] = []
        self.block_tables: List[List[int]] = []
        self.curr_seq_lens: List[int] = []
        self.multimodal_placeholder_maps: Dict[str, Any] = defaultdict(list)
        self.num_prefills = 0
        self.num_prefill_tokens = 0
        self.num_decode_tokens = 0
        self.has_prefix_cache_hit = False

    def _add_seq_group(self, inter_data, chunked_prefill_enabled: bool, prefix_cache_hit: bool):
        is_prompt = inter_data.is_prompt
        block_tables = inter_data.block_tables
        for (seq_id, token_len, seq_len, curr_seq_len, query_len, context_len,
             curr_sliding_window_block) in zip(
                 inter_data.seq_ids, [len(t) for t in inter_data.input_tokens],
                 inter_data.orig_seq_lens, inter_data.seq_lens, inter_data.query_lens,
                 inter_data.context_lens, inter_data.curr_sliding_window_blocks):
            self.context_lens.append(context_len)
            if is_prompt:
                self.num_prefills += 1
                self.num_prefill_tokens += token_len
                self.prefill_seq_lens.append(seq_len)
            else:
                self.num_decode_tokens += query_len
                self.curr_seq_lens.append(curr_seq_len)
            # A decode (or chunked-prefill) sequence under a sliding window hands over only the
            # trailing blocks that can still hold visible tokens (:479-485).
            block_table: List[int] = []
            if prefix_cache_hit:
                block_table = block_tables[seq_id]
            elif (chunked_prefill_enabled or not is_prompt) and block_tables is not None:
                if curr_sliding_window_block == 0:
                    block_table = block_tables[seq_id]
                else:
                    block_table = block_tables[seq_id][-curr_sliding_window_block:]
            self.block_tables.append(block_table)
            is_profile_run = is_block_tables_empty(block_tables)
            start_idx = compute_slot_mapping_start_idx(is_prompt, query_len, context_len,
                                                       self.sliding_window)
            compute_slot_mapping(is_profile_run, self.slot_mapping, seq_id, seq_len, context_len,
                                 start_idx, self.block_size, inter_data.block_tables)

    def _get_graph_runner_block_tables(self, num_seqs: int, block_tables: List[List[int]]) -> torch.Tensor:
        max_batch_size, max_blocks = self.runner.graph_block_tables.shape
        assert max_batch_size >= num_seqs
        graph_block_tables = self.runner.graph_block_tables[:num_seqs]
        for i, block_table in enumerate(block_tables):
            if block_table:
                n = min(len(block_table), max_blocks)
                graph_block_tables[i, :n] = block_table[:n]
        return torch.from_numpy(graph_block_tables).to(device=self.runner.device, non_blocking=True)

    def build(self, seq_lens: List[int], query_lens: List[int], cuda_graph_pad_size: int,
              batch_size: int) -> MetaAttentionMetadata:
        prefix_cache_hit = any(d.prefix_cache_hit for d in self.input_builder.inter_data_list)
        for inter_data in self.input_builder.inter_data_list:
            self._add_seq_group(inter_data, self.input_builder.chunked_prefill_enabled, prefix_cache_hit)
        device = self.runner.device
        use_captured_graph = cuda_graph_pad_size != -1
        max_query_len = max(query_lens)
        decode_query_lens = query_lens[self.num_prefills:]
        max_decode_query_len = max(decode_query_lens) if len(decode_query_lens) > 0 else 1
        max_prefill_seq_len = max(self.prefill_seq_lens, default=0)
        max_decode_seq_len = max(self.curr_seq_lens, default=0)
        num_decode_tokens = self.num_decode_tokens
        query_start_loc = list(accumulate(query_lens, initial=0))
        seq_start_loc = list(accumulate(seq_lens, initial=0))
        num_seqs = len(seq_lens)
        if use_captured_graph:
            self.slot_mapping.extend([PAD_SLOT_ID] * cuda_graph_pad_size)
            self.block_tables.extend([[] for _ in range(cuda_graph_pad_size)])
            num_decode_tokens = batch_size - self.num_prefill_tokens
            block_tables = self._get_graph_runner_block_tables(num_seqs, self.block_tables)
        else:
            block_tables = _pad_tables(self.block_tables, 0, device)
        assert max_query_len > 0, "query_lens: {}".format(query_lens)
        pin = getattr(self.runner, "pin_memory", False)
        return MetaAttentionMetadata(
            num_prefills=self.num_prefills,
            slot_mapping=_to_device(self.slot_mapping, torch.long, device, pin),
            num_prefill_tokens=self.num_prefill_tokens, num_decode_tokens=num_decode_tokens,
            seq_lens=seq_lens, multi_modal_placeholder_index_maps={},
            enable_kv_scales_calculation=True,
            seq_lens_tensor=_to_device(seq_lens, torch.int, device, pin),
            max_query_len=max_query_len, max_decode_query_len=max_decode_query_len,
            max_prefill_seq_len=max_prefill_seq_len, max_decode_seq_len=max_decode_seq_len,
            query_start_loc=_to_device(query_start_loc, torch.int32, device, pin),
            seq_start_loc=_to_device(seq_start_loc, torch.int32, device, pin),
            context_lens_tensor=_to_device(self.context_lens, torch.int, device, pin),
            block_tables=block_tables, use_cuda_graph=use_captured_graph)


class MetaAttentionImpl:
    """Token layout of one call: |prefill_0 ... prefill_N-1 | decode_0 ... decode_M-1 | padding|,
    prompts of any length first, then one token per decoding sequence (:611-639)."""

    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int,
                 alibi_slopes: Optional[List[float]], sliding_window: Optional[int],
                 kv_cache_dtype: str, blocksparse_params: Optional[Dict[str, Any]] = None,
                 logits_soft_cap: Optional[float] = None, attn_type: str = AttentionType.DECODER,
                 kv_sharing_target_layer_name: Optional[str] = None, use_irope: bool = False,
                 num_meta_tokens: int = 128):
        if kv_sharing_target_layer_name is not None:
            raise NotImplementedError("KV sharing is not supported in V0 MetaAttention.")
        if blocksparse_params is not None:
            raise ValueError("MetaAttention does not support blocksparse attention.")
        if alibi_slopes is not None:
            raise NotImplementedError("ALiBi is not part of the sliding-window decode kernel")
        if logits_soft_cap:
            raise NotImplementedError("logits soft-capping is not part of the sliding-window decode kernel")
        if kv_cache_dtype != "auto":
            raise NotImplementedError(
                f"MetaAttention does not support {kv_cache_dtype} kv-cache on this device "
                "(the paged cache holds bf16)")
        if attn_type != AttentionType.DECODER:
            raise NotImplementedError("only decoder self-attention is implemented")
        self.num_heads = num_heads
        self.head_size = head_size
        self.scale = float(scale)
        self.num_kv_heads = num_kv_heads
        self.alibi_slopes = None
        # a window of `sliding_window` tokens = the query plus sliding_window-1 keys to its left
        self.sliding_window = ((sliding_window - 1, 0) if sliding_window is not None else (-1, -1))
        self.kv_cache_dtype = kv_cache_dtype
        self.num_meta_tokens = num_meta_tokens
        self.logits_soft_cap = 0
        self.num_queries_per_kv = self.num_heads // self.num_kv_heads
        support_head_sizes = MetaAttentionBackend.get_supported_head_sizes()
        if self.head_size not in support_head_sizes:
            raise ValueError(f"Head size {head_size} is not supported by MetaAttention. "
                             f"Supported head sizes are {support_head_sizes}.")
        self.attn_type = attn_type
        self._status: Optional[torch.Tensor] = None
        self._workspace: Dict[Any, Optional[torch.Tensor]] = {}

    def _scratch(self, B: int, max_pieces: int, device) -> Optional[torch.Tensor]:
        # one zero-initialised buffer per batch geometry: the counters at its head are laid out
        # by batch size and are handed back zeroed by every call
        key = (B, max_pieces, str(device))
        ws = self._workspace.get(key)
        if ws is None:
            ws = self._workspace[key] = ops.swa_workspace(B, self.num_heads, self.head_size, max_pieces, device)
        return ws

    def status(self) -> int:
        """Device-side status bits accumulated by this layer's kernels (synchronises). After
        SBK_ST_WAIT_TIMEOUT the decode workspaces are stale (the kernel marks them and every later
        call would report the timeout again): they are dropped here, the next call gets fresh ones."""
        bits = 0 if self._status is None else int(self._status.item())
        if bits & 4:
            self._workspace.clear()
        return bits

    def forward(self, layer, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                query2: Optional[torch.Tensor], key2: Optional[torch.Tensor],
                value2: Optional[torch.Tensor], kv_cache: torch.Tensor,
                attn_metadata: MetaAttentionMetadata, output: Optional[torch.Tensor] = None,
                output_scale: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None,
                cos_sin_cache: Optional[torch.Tensor] = None) -> torch.Tensor:
        """query [T, H, D]; key, value [T, KVH, D]; kv_cache [2, NB, BS, KVH, D] (numel 0 on the
        memory-profiling run); writes into `output` ([T, H, D] or [T, H*D]) and returns it.

        With ``positions`` [T] int64 and ``cos_sin_cache`` (ops.build_cos_sin_cache) the rotary
        embedding the reference applies just before this call
        (vllm_hymeta/model_for_7B/modeling_gla_swa.py:215) is folded into the cache write: pass
        the UN-rotated query and key; both are rotated in place by the same launch that appends."""
        assert output is not None, "Output tensor must be provided."
        if output_scale is not None:
            raise NotImplementedError("fused output quantization is not supported in MetaAttention.")
        if layer is not None:
            assert (getattr(layer, "_k_scale_float", 1.0) == 1.0
                    and getattr(layer, "_v_scale_float", 1.0) == 1.0), (
                "key/v_scale is only supported with an fp8 cache, which this path does not have")
        if (key2 is None) != (value2 is None):
            raise ValueError("key2 and value2 come together")
        if key2 is not None:
            assert self.num_meta_tokens == key2.shape[0], "num_meta_tokens differs from key2"
            key2 = key2.view(-1, self.num_kv_heads, self.head_size).contiguous()
            value2 = value2.view(-1, self.num_kv_heads, self.head_size).contiguous()
        H, D = self.num_heads, self.head_size
        query = query.view(-1, H, D)
        out3 = output.view(-1, H, D)
        if self._status is None or self._status.device != query.device:
            self._status = torch.zeros(1, dtype=torch.int32, device=query.device)
        if query2 is not None:
            # The step that first computes the meta (sink) tokens: their own queries attend over all of
            # key2/value2, not causally (fa_kernel_metatoken.py:262-276), and their outputs come first
            # in `output` (:279-280); everything else follows behind them.
            if key2 is None:
                raise ValueError("query2 needs key2/value2")
            if attn_metadata.num_decode_tokens:
                raise NotImplementedError("the meta tokens' own queries go with a prompt run, not with decode tokens "
                                          "(the reference asserts the same)")
            M = self.num_meta_tokens
            q2 = query2.view(-1, H, D)
            assert q2.shape[0] == M, "num_meta_tokens differs from query2"
            if out3.shape[0] != query.shape[0] + M:
                raise ValueError("with query2 the output holds num_meta_tokens rows ahead of the query tokens")
            loc = torch.tensor([0, M], dtype=torch.int32, device=q2.device)
            m_out = out3[:M]
            m_tmp = m_out if m_out.stride()[1:] == (D, 1) else torch.empty_like(m_out, memory_format=torch.contiguous_format)
            ops.swa_prefill_dense(q2 if q2.stride()[1:] == (D, 1) else q2.contiguous(), key2, value2, loc, loc, M,
                                  window_left=-1, causal=False, scale=self.scale, out=m_tmp, status=self._status)
            if m_tmp is not m_out:
                m_out.copy_(m_tmp)
            out3 = out3[M:]
        if (positions is None) != (cos_sin_cache is None):
            raise ValueError("positions and cos_sin_cache come together")
        if kv_cache.numel() > 0 and key is not None and value is not None:
            if positions is not None:
                ops.rope_kv_append(query, key.view(-1, self.num_kv_heads, D),
                                   value.view(-1, self.num_kv_heads, D), kv_cache[0], kv_cache[1],
                                   attn_metadata.slot_mapping.flatten(), positions.flatten(),
                                   cos_sin_cache, key_in_place=True, status=self._status)
            else:
                ops.kv_append(key.view(-1, self.num_kv_heads, D), value.view(-1, self.num_kv_heads, D),
                              kv_cache[0], kv_cache[1], attn_metadata.slot_mapping.flatten(),
                              status=self._status)
        elif positions is not None:
            raise NotImplementedError("the fused rotary embedding rides on the cache write; without a "
                                      "cache (profile run) rotate query and key beforehand")

        num_prefill_tokens = attn_metadata.num_prefill_tokens
        num_decode_tokens = attn_metadata.num_decode_tokens
        decode_query = query[num_prefill_tokens:]
        prefill_query = query[:num_prefill_tokens]
        assert decode_query.shape[0] == num_decode_tokens, (
            f"decode_query.shape: {decode_query.shape}, num_decode_tokens: {num_decode_tokens}")
        window_left = self.sliding_window[0]

        if prefill_meta := attn_metadata.prefill_metadata:
            pq = prefill_query if prefill_query.stride()[1:] == (D, 1) else prefill_query.contiguous()
            po = out3[:num_prefill_tokens]
            tmp = po if po.stride()[1:] == (D, 1) else torch.empty_like(po, memory_format=torch.contiguous_format)
            if (kv_cache.numel() == 0 or prefill_meta.block_tables is None
                    or prefill_meta.block_tables.numel() == 0):
                # prompt run without block tables (the un-chunked first prompt, the memory-profiling
                # run): q and k are the prompt itself and have the same lengths (reference :843-884)
                if key is None or value is None:
                    raise ValueError("the prompt run without block tables attends over key/value; they are required")
                n_kv = num_prefill_tokens
                qsl = prefill_meta.query_start_loc.to(torch.int32).contiguous()
                ksl = qsl if prefill_meta.seq_start_loc is None else prefill_meta.seq_start_loc.to(torch.int32).contiguous()
                ops.swa_prefill_dense(pq, key.view(-1, self.num_kv_heads, D)[:n_kv],
                                      value.view(-1, self.num_kv_heads, D)[:n_kv], qsl, ksl,
                                      prefill_meta.max_query_len, window_left=window_left, scale=self.scale,
                                      out=tmp, key2=key2, value2=value2, status=self._status)
                if tmp is not po:
                    po.copy_(tmp)
                prefill_meta = None
        if prefill_meta:
            # windowed attention of the prompt tokens over the paged cache (their own K/V included:
            # the append above has run), 16 queries and one kv group per CTA
            ops.swa_prefill(pq, kv_cache[0], kv_cache[1], prefill_meta.block_tables.contiguous(),
                            prefill_meta.query_start_loc.to(torch.int32).contiguous(),
                            prefill_meta.context_lens_tensor.to(torch.int32).contiguous(),
                            prefill_meta.max_query_len, window_left=window_left, scale=self.scale, out=tmp,
                            key2=key2, value2=value2, status=self._status)
            if tmp is not po:
                po.copy_(tmp)

        if decode_meta := attn_metadata.decode_metadata:
            if decode_meta.max_decode_query_len is not None and decode_meta.max_decode_query_len > 1:
                # several query tokens per sequence (reference :924-953, varlen attention over the
                # cache through the block tables): the prefill kernel, each sequence's queries being
                # the tail of its seq_len tokens
                if decode_meta.query_start_loc is None:
                    raise ValueError("multi-token decode needs decode_metadata.query_start_loc")
                dq = decode_query if decode_query.stride()[1:] == (D, 1) else decode_query.contiguous()
                do = out3[num_prefill_tokens:]
                dtmp = do if do.stride()[1:] == (D, 1) else torch.empty_like(do, memory_format=torch.contiguous_format)
                dqsl = decode_meta.query_start_loc.to(torch.int32).contiguous()
                ctx = (decode_meta.seq_lens_tensor.to(torch.int32) - (dqsl[1:] - dqsl[:-1])).contiguous()
                ops.swa_prefill(dq, kv_cache[0], kv_cache[1], decode_meta.block_tables.contiguous(), dqsl, ctx,
                                decode_meta.max_decode_query_len, window_left=window_left, scale=self.scale,
                                out=dtmp, key2=key2, value2=value2, status=self._status)
                if dtmp is not do:
                    do.copy_(dtmp)
                return output
            self._decode(decode_query, kv_cache, decode_meta.block_tables, decode_meta.seq_lens_tensor,
                         window_left, out3[num_prefill_tokens:], key2, value2)
        return output

    def _decode(self, q, kv_cache, block_tables, seq_lens, window_left, out, key2=None, value2=None) -> None:
        B = q.shape[0]
        if B == 0:
            return
        bs = kv_cache.shape[2]
        width = block_tables.shape[1] * bs
        vis = width if window_left < 0 else min(width, window_left + 1)
        split = ops.swa_auto_split(B, vis, q.device)
        max_pieces = ops.swa_max_pieces(vis, split, B, q.device)
        D = self.head_size
        if q.stride()[1:] != (D, 1):
            q = q.contiguous()
        tmp = out if out.stride()[1:] == (D, 1) else torch.empty_like(out, memory_format=torch.contiguous_format)
        ops.swa_decode(q, kv_cache[0], kv_cache[1], block_tables.contiguous(), seq_lens.contiguous(),
                       window_left=window_left, scale=self.scale, out=tmp,
                       workspace=self._scratch(B, max_pieces, q.device), max_pieces=max_pieces,
                       split_chunks=split, key2=key2, value2=value2, status=self._status)
        if tmp is not out:
            out.copy_(tmp)
