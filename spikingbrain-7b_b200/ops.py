"""Tensor-level wrappers of the libsbk kernels.

Each wrapper checks device, dtype and layout on the host, passes raw device
pointers and the current CUDA stream through the C ABI, and raises on a
non-zero return code. Nothing here computes on the CPU and nothing falls back
to PyTorch ops: without a CUDA device and libsbk.so these functions raise.
"""
from typing import Optional, Sequence, Tuple

import ctypes

import torch

from . import _abi
from ._abi import SBK_BF16, SBK_F32

_DTYPE_CODE = {torch.bfloat16: SBK_BF16, torch.float32: SBK_F32}
DEFAULT_SPLIT_CHUNKS = 32  # 16-token chunks per split of a sequence (512 tokens)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("libsbk ops take CUDA tensors only (there is no CPU path)")


def _cache_geometry(k_cache: torch.Tensor, v_cache: torch.Tensor) -> Tuple[int, int, int, int, int]:
    """k_cache / v_cache: [num_blocks, block_size, kvh, D], rows of a block contiguous."""
    if k_cache.dim() != 4 or k_cache.shape != v_cache.shape or k_cache.dtype != v_cache.dtype:
        raise ValueError("k_cache and v_cache must be equal-shaped [num_blocks, block, kvh, D] tensors")
    nb, bs, kvh, d = k_cache.shape
    for c in (k_cache, v_cache):
        if nb and c.stride()[1:] != (kvh * d, d, 1):
            raise ValueError("the rows of a cache block must be contiguous")
    if k_cache.stride(0) != v_cache.stride(0):
        raise ValueError("k_cache and v_cache must share one block stride")
    return nb, bs, kvh, d, k_cache.stride(0) * k_cache.element_size()


def _append_args(key, value, k_cache, v_cache, slot_mapping, block_tables, seq_lens, query_start_loc,
                 retired_out):
    """Shared validation of the two append entry points -> (nb, bs, kvh, d, bstride, T, B,
    max_blocks, max_ret, es, tok_stride)."""
    _need_cuda(key, value, k_cache, v_cache, slot_mapping, block_tables, seq_lens, query_start_loc, retired_out)
    nb, bs, kvh, d, bstride = _cache_geometry(k_cache, v_cache)
    T = key.shape[0]
    if key.shape != (T, kvh, d) or value.shape != key.shape:
        raise ValueError(f"key/value must be [T, {kvh}, {d}], got {tuple(key.shape)} / {tuple(value.shape)}")
    if key.dtype != k_cache.dtype or value.dtype != k_cache.dtype:
        raise ValueError("key/value dtype differs from the cache dtype")
    for t in (key, value):  # strides of size-1 dimensions carry no meaning
        if T and ((d > 1 and t.stride(2) != 1) or (kvh > 1 and t.stride(1) != d)):
            raise ValueError("key/value rows must be contiguous")
    if T > 1 and value.stride(0) != key.stride(0):
        raise ValueError("key and value must share one token stride")
    if slot_mapping.dtype != torch.int64 or slot_mapping.numel() != T or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a contiguous int64 tensor with one entry per token")
    B = max_blocks = max_ret = 0
    if block_tables is not None:
        if seq_lens is None:
            raise ValueError("retirement needs seq_lens")
        B, max_blocks = block_tables.shape
        for t, n in ((block_tables, None), (seq_lens, B), (query_start_loc, B + 1)):
            if t is None:
                continue
            if t.dtype != torch.int32 or not t.is_contiguous() or (n is not None and t.numel() != n):
                raise ValueError("block_tables / seq_lens / query_start_loc must be contiguous int32 of matching size")
        if retired_out is not None:
            if retired_out.dtype != torch.int32 or not retired_out.is_contiguous() or retired_out.shape[0] != B:
                raise ValueError("retired_out must be contiguous int32 [B, max_retired]")
            max_ret = retired_out.shape[1]
    es = k_cache.element_size()
    tok_stride = (key.stride(0) if T else kvh * d) * es
    return nb, bs, kvh, d, bstride, T, B, max_blocks, max_ret, es, tok_stride


def kv_append(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              slot_mapping: torch.Tensor, *, block_tables: Optional[torch.Tensor] = None,
              seq_lens: Optional[torch.Tensor] = None,
              query_start_loc: Optional[torch.Tensor] = None, window_left: int = -1,
              retired_out: Optional[torch.Tensor] = None,
              status: Optional[torch.Tensor] = None) -> None:
    """Write key/value [T, kvh, D] into the paged cache at ``slot_mapping`` and, when
    ``block_tables`` is given, replace table entries of blocks that left the window by -1
    (their ids are listed in ``retired_out`` [B, max_retired])."""
    _need_cuda(status)
    nb, bs, kvh, d, bstride, T, B, max_blocks, max_ret, es, tok_stride = _append_args(
        key, value, k_cache, v_cache, slot_mapping, block_tables, seq_lens, query_start_loc, retired_out)
    rc = _abi.lib.sbk_kv_append(
        _ptr(key), _ptr(value), _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping), T, kvh, d, es,
        tok_stride, nb, bs, bstride, _ptr(block_tables), max_blocks, _ptr(seq_lens),
        _ptr(query_start_loc), B, window_left, _ptr(retired_out), max_ret, _ptr(status), _stream())
    _abi.check("sbk_kv_append", rc)


def build_cos_sin_cache(rot_dim: int, max_position: int, base: float = 10000.0,
                        dtype: torch.dtype = torch.bfloat16, device="cuda") -> torch.Tensor:
    """The [max_position, rot_dim] cos|sin table sbk_rope_kv_append reads, computed as
    GLAswaRotaryEmbedding._compute_cos_sin_cache does (vllm_hymeta/model_for_7B/
    modeling_gla_swa.py:66-79): fp32 angles position x base^(-2i/rot_dim), cos and sin taken in
    fp32, then one cast to ``dtype``. The HF RotaryEmbedding (hf_7B_model/window_attention.py:
    23-47) produces the same cos/sin values per call. The table is always computed by the host's
    libm and then moved to ``device``: device cos/sin differ from it in the last fp32 bit often
    enough to flip roundings to bf16, and the fixtures recorded from the reference are host values."""
    inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float) / rot_dim))
    t = torch.arange(max_position, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).to(dtype).contiguous().to(device)


def rope_kv_append(query: Optional[torch.Tensor], key: torch.Tensor, value: torch.Tensor,
                   k_cache: torch.Tensor, v_cache: torch.Tensor, slot_mapping: torch.Tensor,
                   positions: torch.Tensor, cos_sin_cache: torch.Tensor, *, key_in_place: bool = False,
                   block_tables: Optional[torch.Tensor] = None, seq_lens: Optional[torch.Tensor] = None,
                   query_start_loc: Optional[torch.Tensor] = None, window_left: int = -1,
                   retired_out: Optional[torch.Tensor] = None,
                   status: Optional[torch.Tensor] = None) -> None:
    """kv_append with the NeoX rotary embedding folded in: ``query`` [T, H, D] (optional) is rotated
    in place, ``key`` [T, kvh, D] is rotated on its way into the cache (and in place too with
    ``key_in_place``), ``value`` is copied. ``positions`` [T] int64 index ``cos_sin_cache``
    [max_position, rot_dim] (build_cos_sin_cache)."""
    _need_cuda(query, positions, cos_sin_cache, status)
    nb, bs, kvh, d, bstride, T, B, max_blocks, max_ret, es, tok_stride = _append_args(
        key, value, k_cache, v_cache, slot_mapping, block_tables, seq_lens, query_start_loc, retired_out)
    if k_cache.dtype not in _DTYPE_CODE:
        raise ValueError("the fused rotary append takes bf16 or fp32 tensors")
    if cos_sin_cache.dim() != 2 or cos_sin_cache.dtype != k_cache.dtype or not cos_sin_cache.is_contiguous():
        raise ValueError("cos_sin_cache must be contiguous [max_position, rot_dim] in the cache dtype")
    max_pos, rot_dim = cos_sin_cache.shape
    if positions.dtype != torch.int64 or positions.numel() != T or not positions.is_contiguous():
        raise ValueError("positions must be a contiguous int64 tensor with one entry per token")
    H = q_stride = 0
    if query is not None:
        if query.dim() != 3 or query.shape[0] != T or query.shape[2] != d or query.dtype != k_cache.dtype:
            raise ValueError(f"query must be [T, H, {d}] in the cache dtype")
        H = query.shape[1]
        if T and ((d > 1 and query.stride(2) != 1) or (H > 1 and query.stride(1) != d)):
            raise ValueError("query rows must be contiguous")
        q_stride = (query.stride(0) if T else H * d) * es
    rc = _abi.lib.sbk_rope_kv_append(
        _ptr(query), H, q_stride, _ptr(key), _ptr(value), int(key_in_place), _ptr(k_cache), _ptr(v_cache),
        _ptr(slot_mapping), _ptr(positions), _ptr(cos_sin_cache), rot_dim, max_pos, T, kvh, d,
        _DTYPE_CODE[k_cache.dtype], tok_stride, nb, bs, bstride, _ptr(block_tables), max_blocks,
        _ptr(seq_lens), _ptr(query_start_loc), B, window_left, _ptr(retired_out), max_ret, _ptr(status),
        _stream())
    _abi.check("sbk_rope_kv_append", rc)


def kv_gather(k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
              seq_lens: torch.Tensor, n_out: int, *, window_left: int = -1,
              status: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense head-first copies [B, kvh, n_out, D] of every sequence's visible window."""
    _need_cuda(k_cache, v_cache, block_tables, seq_lens, status)
    nb, bs, kvh, d, bstride = _cache_geometry(k_cache, v_cache)
    B, max_blocks = block_tables.shape
    if block_tables.dtype != torch.int32 or seq_lens.dtype != torch.int32 or seq_lens.numel() != B:
        raise ValueError("block_tables / seq_lens must be int32 with one row / entry per sequence")
    if not (block_tables.is_contiguous() and seq_lens.is_contiguous()):
        raise ValueError("block_tables / seq_lens must be contiguous")
    k_out = torch.empty((B, kvh, n_out, d), dtype=k_cache.dtype, device=k_cache.device)
    v_out = torch.empty_like(k_out)
    rc = _abi.lib.sbk_kv_gather(
        _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), max_blocks, _ptr(seq_lens), B, kvh, d,
        k_cache.element_size(), nb, bs, bstride, window_left, _ptr(k_out), _ptr(v_out), n_out,
        _ptr(status), _stream())
    _abi.check("sbk_kv_gather", rc)
    return k_out, v_out


_SM_COUNT = {}


def _check_meta(key2, value2, kvh: int, d: int) -> int:
    """Sink-token tensors [n_meta, kvh, D] bf16, contiguous, n_meta a multiple of 16; returns n_meta."""
    if key2 is None and value2 is None:
        return 0
    if key2 is None or value2 is None:
        raise ValueError("key2 and value2 come together")
    _need_cuda(key2, value2)
    for t in (key2, value2):
        if t.dtype != torch.bfloat16 or t.dim() != 3 or t.shape[1:] != (kvh, d) or not t.is_contiguous():
            raise ValueError(f"key2 / value2 must be contiguous bf16 [n_meta, {kvh}, {d}]")
    if key2.shape != value2.shape or key2.shape[0] % 16:
        raise ValueError("key2 / value2 must share a token count that is a multiple of 16")
    return key2.shape[0]


def swa_auto_split(B: int, max_visible_tokens: int, device) -> int:
    """The default ``split_chunks`` of swa_decode: negative = balanced mode, in which the kernel
    cuts the batch's chunks (of 16 tokens) into one equal run per CTA (two CTAs per SM) whatever
    the spread of lengths; the magnitude is the shortest run it may cut (8 chunks = 128 tokens =
    256 KiB of K and V at 4 kv heads, below which the per-item cost outweighs the balance)."""
    return -8


def _n_ctas(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return 2 * _SM_COUNT[idx]


def swa_max_pieces(max_visible_tokens: int, split_chunks: int = DEFAULT_SPLIT_CHUNKS, B: int = 0,
                   device=None) -> int:
    """Upper bound on the splits of one sequence whose window holds ``max_visible_tokens``; sizes
    the workspace. Fixed pieces (split_chunks > 0): ceil(chunks / split_chunks). Balanced mode
    (split_chunks < 0): the kernel keeps every sequence within the bound it is given, so the bound
    only has to allow the balance: about CTAs / B runs per sequence, plus the two it may share
    with its neighbours, and never more than the shortest run permits."""
    chunks = (max(int(max_visible_tokens), 1) + 15) // 16 + 1  # +1: a window rarely starts on a chunk edge
    if split_chunks > 0:
        return max(1, -(-chunks // split_chunks))
    n_ctas = _n_ctas(device) if device is not None else 296
    by_balance = -(-n_ctas // max(B, 1)) + 2
    by_run = -(-chunks // max(-split_chunks, 1)) + 1
    return max(2, min(by_balance, by_run, 33))


def swa_workspace(B: int, H: int, D: int, max_pieces: int, device) -> Optional[torch.Tensor]:
    """Scratch for swa_decode with exactly these B and max_pieces. It starts with the ticket
    and per-sequence completion counters, which must be zero before the first call and which
    every call leaves at zero; hence zero-filled, and not to be shared between batch sizes."""
    n = _abi.lib.sbk_swa_workspace_bytes(B, H, D, max_pieces)
    return torch.zeros(n, dtype=torch.uint8, device=device) if n else None


class PeerTargets:
    """Where sbk_swa_decode_gather stores besides its own `out`: per peer the address of this
    rank's head slice in the peer's gathered buffer and of this rank's slot in the peer's flag
    array, and the value the flags take when the step's rows are complete."""

    def __init__(self, out_addrs: Sequence[int], flag_addrs: Sequence[int], flag_value: int,
                 flag_base: Optional[torch.Tensor] = None):
        if len(out_addrs) != len(flag_addrs):
            raise ValueError("one buffer address and one flag address per peer")
        self.n = len(out_addrs)
        self.out_table = (ctypes.c_void_p * max(self.n, 1))(*out_addrs)
        self.flag_table = (ctypes.c_void_p * max(self.n, 1))(*flag_addrs)
        self.flag_value = int(flag_value)
        if flag_base is not None and (flag_base.dtype != torch.int32 or not flag_base.is_cuda):
            raise ValueError("flag_base is an int32 word on the device")
        self.flag_base = flag_base      # the flags take flag_value + flag_base[0], read on the device


def swa_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
               block_tables: torch.Tensor, seq_lens: torch.Tensor, *, window_left: int,
               scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
               out_dtype: Optional[torch.dtype] = None, lse: Optional[torch.Tensor] = None,
               workspace: Optional[torch.Tensor] = None, max_pieces: Optional[int] = None,
               split_chunks: Optional[int] = None, item_cost: int = -1,
               key2: Optional[torch.Tensor] = None, value2: Optional[torch.Tensor] = None,
               status: Optional[torch.Tensor] = None, peers: Optional["PeerTargets"] = None) -> torch.Tensor:
    """Single-query sliding-window attention over the paged cache; q [B, H, D] bf16.
    ``split_chunks`` > 0: fixed pieces of that many 16-token chunks, drawn by the CTAs from a ticket
    counter; < 0: balanced mode (equal runs of chunks per CTA, runs no shorter than -split_chunks);
    default swa_auto_split. ``item_cost``: balanced mode's charge per sequence in chunks (-1: the
    library's tuned value).
    ``key2`` / ``value2`` [n_meta, kvh, D]: sink tokens every query sees besides its window.
    ``peers``: head-sharded use -- ``out`` is this rank's head slice of its gathered buffer, and the
    kernel also stores every finished row to the peers and raises their flags (PeerTargets)."""
    _need_cuda(q, k_cache, v_cache, block_tables, seq_lens, out, lse, workspace, status)
    nb, bs, kvh, d, bstride = _cache_geometry(k_cache, v_cache)
    if q.dim() != 3 or q.shape[2] != d or q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise ValueError("q must be bf16 [B, H, D] and the cache bf16")
    B, H, _ = q.shape
    if B and q.stride()[1:] != (d, 1):
        raise ValueError("the heads of q must be contiguous")
    if block_tables.shape[0] != B or seq_lens.numel() != B:
        raise ValueError("block_tables / seq_lens need one row / entry per query")
    if block_tables.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise ValueError("block_tables / seq_lens must be int32")
    if not (block_tables.is_contiguous() and seq_lens.is_contiguous()):
        raise ValueError("block_tables / seq_lens must be contiguous")
    if out is None:
        out = torch.empty((B, H, d), dtype=out_dtype or torch.bfloat16, device=q.device)
    elif out.shape != (B, H, d) or (B and out.stride()[1:] != (d, 1)):
        raise ValueError("out must be [B, H, D] with contiguous heads")
    if out.dtype not in _DTYPE_CODE:
        raise ValueError("out must be bf16 or fp32")
    if lse is not None and (lse.dtype != torch.float32 or lse.shape != (B, H) or not lse.is_contiguous()):
        raise ValueError("lse must be contiguous fp32 [B, H]")
    max_blocks = block_tables.shape[1]
    vis = max_blocks * bs if window_left < 0 else min(max_blocks * bs, window_left + 1)
    if split_chunks is None:
        split_chunks = swa_auto_split(B, vis, q.device) if B else DEFAULT_SPLIT_CHUNKS
    if max_pieces is None:
        max_pieces = swa_max_pieces(vis, split_chunks, B, q.device)
    if workspace is None:
        workspace = swa_workspace(B, H, d, max_pieces, q.device)
    if scale is None:
        scale = d ** -0.5
    n_meta = _check_meta(key2, value2, kvh, d)
    if peers is not None:
        if out.dtype != torch.bfloat16 or lse is not None:
            raise ValueError("the gathered head outputs are bf16, without lse")
        rc = _abi.lib.sbk_swa_decode_gather(
            _ptr(q), q.stride(0) if B else H * d, _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
            max_blocks, _ptr(seq_lens), B, H, kvh, d, nb, bs, bstride, window_left, float(scale),
            _ptr(out), out.stride(0) if B else H * d, _ptr(workspace),
            workspace.numel() if workspace is not None else 0, split_chunks, max_pieces, int(item_cost),
            _ptr(key2), _ptr(value2), n_meta, peers.out_table, peers.flag_table, peers.n, peers.flag_value,
            _ptr(peers.flag_base), _ptr(status), _stream())
        _abi.check("sbk_swa_decode_gather", rc)
    else:
        rc = _abi.lib.sbk_swa_decode(
            _ptr(q), q.stride(0) if B else H * d, _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
            max_blocks, _ptr(seq_lens), B, H, kvh, d, nb, bs, bstride, window_left, float(scale),
            _ptr(out), _DTYPE_CODE[out.dtype], out.stride(0) if B else H * d, _ptr(lse),
            _ptr(workspace), workspace.numel() if workspace is not None else 0, split_chunks,
            max_pieces, int(item_cost), _ptr(key2), _ptr(value2), n_meta, _ptr(status), _stream())
        _abi.check("sbk_swa_decode", rc)
    return out


GLA_RELU_QK = 1
GLA_GATE_LOGITS = 2


def _gla_fusion_args(q, D, relu_qk, gate_logit_normalizer, norm_weight):
    flags = GLA_RELU_QK if relu_qk else 0
    gnorm = 0.0
    if gate_logit_normalizer is not None:
        if not gate_logit_normalizer > 0:
            raise ValueError("gate_logit_normalizer must be positive")
        flags |= GLA_GATE_LOGITS
        gnorm = float(gate_logit_normalizer)
    if norm_weight is not None and (norm_weight.shape != (D,) or norm_weight.dtype != q.dtype
                                    or not norm_weight.is_contiguous()):
        raise ValueError("norm_weight must be contiguous [D] in the dtype of q")
    return flags, gnorm


def gla_step(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
             state: torch.Tensor, slot_idx: Optional[torch.Tensor] = None, *,
             scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
             out_dtype: Optional[torch.dtype] = None, relu_qk: bool = False,
             gate_logit_normalizer: Optional[float] = None,
             norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 1e-5,
             status: Optional[torch.Tensor] = None, peers: Optional["PeerTargets"] = None,
             peer_counter: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In-place GLA state step on ``state`` [slots, H, D, D] fp32; q [B, H, D], k/v/g [B, Hkv, D].

    Fused neighbours of the reference layer (all off by default): ``relu_qk`` applies the feature
    map to q and k; ``gate_logit_normalizer`` makes ``g`` gate logits, turned into
    ``logsigmoid(g) / normalizer`` in the kernel; ``norm_weight`` [D] applies the per-head RMS norm
    (g_norm) to the read-out.
    ``peers`` (head-sharded use, bf16): ``out`` is this rank's head slice of its gathered buffer
    (rows may be strided); the kernel stores the rows to the peers too and raises their flags;
    ``peer_counter`` is one zeroed int32 kept for these calls."""
    _need_cuda(q, k, v, g, state, slot_idx, out, status, norm_weight, peer_counter)
    flags, gnorm = _gla_fusion_args(q, D=q.shape[-1], relu_qk=relu_qk,
                                    gate_logit_normalizer=gate_logit_normalizer, norm_weight=norm_weight)
    if q.dim() != 3 or k.dim() != 3:
        raise ValueError("q must be [B, H, D] and k, v, g [B, Hkv, D]")
    B, H, D = q.shape
    Hkv = k.shape[1]
    if k.shape != (B, Hkv, D) or v.shape != k.shape or g.shape != k.shape:
        raise ValueError("k, v, g must share the shape [B, Hkv, D]")
    if q.dtype not in _DTYPE_CODE or any(t.dtype != q.dtype for t in (k, v, g)):
        raise ValueError("q, k, v, g must share one dtype (bf16 or fp32)")
    if not all(t.is_contiguous() for t in (q, k, v, g)):
        raise ValueError("q, k, v, g must be contiguous")
    if state.dtype != torch.float32 or state.dim() != 4 or state.shape[1:] != (H, D, D) or not state.is_contiguous():
        raise ValueError(f"state must be contiguous fp32 [slots, {H}, {D}, {D}]")
    if slot_idx is not None and (slot_idx.dtype != torch.int64 or slot_idx.numel() != B or not slot_idx.is_contiguous()):
        raise ValueError("slot_idx must be contiguous int64 [B]")
    if slot_idx is None and state.shape[0] < B:
        raise ValueError("state has fewer slots than sequences")
    if scale is None:
        scale = D ** -0.5
    if peers is not None:
        if q.dtype != torch.bfloat16 or out is None or out.dtype != torch.bfloat16:
            raise ValueError("the gathered GLA step takes bf16 inputs and a bf16 out slice")
        if out.shape != (B, H, D) or (B and out.stride()[1:] != (D, 1)):
            raise ValueError("out must be [B, H, D] with contiguous heads")
        if peer_counter is None or peer_counter.dtype != torch.int32:
            raise ValueError("peer_counter: one zeroed int32 on the device")
        rc = _abi.lib.sbk_gla_step_gather(
            _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(state), state.shape[0], _ptr(slot_idx), B, H, Hkv, D,
            float(scale), _ptr(out), out.stride(0) if B else H * D, flags, gnorm, _ptr(norm_weight),
            float(norm_eps), _ptr(peer_counter), peers.out_table, peers.flag_table, peers.n, peers.flag_value,
            _ptr(peers.flag_base), _ptr(status), _stream())
        _abi.check("sbk_gla_step_gather", rc)
        return out
    if out is None:
        out = torch.empty((B, H, D), dtype=out_dtype or q.dtype, device=q.device)
    elif out.shape != (B, H, D) or not out.is_contiguous() or out.dtype not in _DTYPE_CODE:
        raise ValueError("out must be contiguous [B, H, D] bf16 or fp32")
    rc = _abi.lib.sbk_gla_step(
        _ptr(q), _ptr(k), _ptr(v), _ptr(g), _DTYPE_CODE[q.dtype], _ptr(state), state.shape[0],
        _ptr(slot_idx), B, H, Hkv, D, float(scale), _ptr(out), _DTYPE_CODE[out.dtype],
        flags, gnorm, _ptr(norm_weight), float(norm_eps), _ptr(status), _stream())
    _abi.check("sbk_gla_step", rc)
    return out


def gla_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, state: torch.Tensor,
             query_start_loc: torch.Tensor, slot_idx: Optional[torch.Tensor] = None,
             reset: Optional[torch.Tensor] = None, *, scale: Optional[float] = None,
             out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
             relu_qk: bool = False, gate_logit_normalizer: Optional[float] = None,
             norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 1e-5,
             max_query_len: int = 0, workspace: Optional[torch.Tensor] = None,
             status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """GLA over runs of tokens with state carry. q [T, H, D], k/v/g [T, Hkv, D] token-major;
    sequence s owns rows query_start_loc[s]:query_start_loc[s+1]; ``state`` [slots, H, D, D] fp32 is
    advanced in place; ``reset`` [n_seqs] uint8/bool marks sequences that start from zero. The
    fused neighbours (``relu_qk``, ``gate_logit_normalizer``, ``norm_weight``) are those of gla_step.
    ``max_query_len`` (the longest run, a host value) with ``workspace`` (gla_scan_workspace) lets a
    call with few long runs spread every run over several CTAs (chunk-parallel form; results agree
    with the one-chain scan to fp32 rounding instead of bit for bit)."""
    _need_cuda(q, k, v, g, state, query_start_loc, slot_idx, reset, out, status, norm_weight, workspace)
    flags, gnorm = _gla_fusion_args(q, D=q.shape[-1], relu_qk=relu_qk,
                                    gate_logit_normalizer=gate_logit_normalizer, norm_weight=norm_weight)
    if q.dim() != 3 or k.dim() != 3:
        raise ValueError("q must be [T, H, D] and k, v, g [T, Hkv, D]")
    T, H, D = q.shape
    Hkv = k.shape[1]
    if k.shape != (T, Hkv, D) or v.shape != k.shape or g.shape != k.shape:
        raise ValueError("k, v, g must share the shape [T, Hkv, D]")
    if q.dtype not in _DTYPE_CODE or any(t.dtype != q.dtype for t in (k, v, g)):
        raise ValueError("q, k, v, g must share one dtype (bf16 or fp32)")
    if not all(t.is_contiguous() for t in (q, k, v, g)):
        raise ValueError("q, k, v, g must be contiguous")
    if state.dtype != torch.float32 or state.dim() != 4 or state.shape[1:] != (H, D, D) or not state.is_contiguous():
        raise ValueError(f"state must be contiguous fp32 [slots, {H}, {D}, {D}]")
    if query_start_loc.dtype != torch.int32 or query_start_loc.dim() != 1 or not query_start_loc.is_contiguous():
        raise ValueError("query_start_loc must be contiguous int32 [n_seqs + 1]")
    n_seqs = query_start_loc.numel() - 1
    if slot_idx is not None and (slot_idx.dtype != torch.int64 or slot_idx.numel() != n_seqs or not slot_idx.is_contiguous()):
        raise ValueError("slot_idx must be contiguous int64 [n_seqs]")
    if slot_idx is None and state.shape[0] < n_seqs:
        raise ValueError("state has fewer slots than sequences")
    if reset is not None:
        if reset.dtype == torch.bool:
            reset = reset.to(torch.uint8)
        if reset.dtype != torch.uint8 or reset.numel() != n_seqs or not reset.is_contiguous():
            raise ValueError("reset must be contiguous uint8/bool [n_seqs]")
    if out is None:
        out = torch.empty((T, H, D), dtype=out_dtype or q.dtype, device=q.device)
    elif out.shape != (T, H, D) or not out.is_contiguous() or out.dtype not in _DTYPE_CODE:
        raise ValueError("out must be contiguous [T, H, D] bf16 or fp32")
    if scale is None:
        scale = D ** -0.5
    rc = _abi.lib.sbk_gla_scan(
        _ptr(q), _ptr(k), _ptr(v), _ptr(g), _DTYPE_CODE[q.dtype], _ptr(query_start_loc), n_seqs,
        _ptr(state), state.shape[0], _ptr(slot_idx), _ptr(reset), H, Hkv, D, float(scale), _ptr(out),
        _DTYPE_CODE[out.dtype], flags, gnorm, _ptr(norm_weight), float(norm_eps),
        int(max_query_len) if workspace is not None else 0, _ptr(workspace),
        workspace.numel() * workspace.element_size() if workspace is not None else 0, _ptr(status), _stream())
    _abi.check("sbk_gla_scan", rc)
    return out


def gla_scan_workspace(n_seqs: int, max_query_len: int, H: int, D: int, device) -> Optional[torch.Tensor]:
    """Scratch for the chunk-parallel form of gla_scan, or None when a call of this shape runs as
    one chain per (sequence, head) anyway. Contents need no initialisation."""
    n = _abi.lib.sbk_gla_scan_workspace_bytes(n_seqs, max_query_len, H, D)
    return torch.empty(n, dtype=torch.uint8, device=device) if n else None


PREFILL_KERNELS = {"auto": _abi.PREFILL_AUTO, "tcgen05": _abi.PREFILL_TCGEN05, "mma_sync": _abi.PREFILL_MMA_SYNC,
                   "tcgen05_pair": _abi.PREFILL_TCGEN05_PAIR}


def swa_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                query_start_loc: torch.Tensor, context_lens: torch.Tensor, max_query_len: int, *,
                window_left: int, scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
                key2: Optional[torch.Tensor] = None, value2: Optional[torch.Tensor] = None,
                kernel: str = "auto", status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sliding-window attention of runs of query tokens (q [T, H, D] bf16, token-major) over the
    paged cache, the runs' own K/V already appended. Sequence s owns rows
    query_start_loc[s]:query_start_loc[s+1] and had context_lens[s] tokens cached before.
    ``kernel``: "auto" (tcgen05 where q / out allow 16-byte vectors, else mma.sync), "tcgen05",
    "mma_sync"."""
    _need_cuda(q, k_cache, v_cache, block_tables, query_start_loc, context_lens, out, status)
    nb, bs, kvh, d, bstride = _cache_geometry(k_cache, v_cache)
    if q.dim() != 3 or q.shape[2] != d or q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise ValueError("q must be bf16 [T, H, D] and the cache bf16")
    T, H, _ = q.shape
    if T and q.stride()[1:] != (d, 1):
        raise ValueError("the heads of q must be contiguous")
    n_seqs = block_tables.shape[0]
    for t, n in ((block_tables, None), (query_start_loc, n_seqs + 1), (context_lens, n_seqs)):
        if t.dtype != torch.int32 or not t.is_contiguous() or (n is not None and t.numel() != n):
            raise ValueError("block_tables / query_start_loc / context_lens must be contiguous int32 of matching size")
    if out is None:
        out = torch.empty((T, H, d), dtype=torch.bfloat16, device=q.device)
    elif out.shape != (T, H, d) or out.dtype != torch.bfloat16 or (T and out.stride()[1:] != (d, 1)):
        raise ValueError("out must be bf16 [T, H, D] with contiguous heads")
    if scale is None:
        scale = d ** -0.5
    rc = _abi.lib.sbk_swa_prefill(
        _ptr(q), q.stride(0) if T else H * d, _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
        block_tables.shape[1], _ptr(query_start_loc), _ptr(context_lens), n_seqs, int(max_query_len), H,
        kvh, d, nb, bs, bstride, window_left, float(scale), _ptr(out), out.stride(0) if T else H * d,
        _ptr(key2), _ptr(value2), _check_meta(key2, value2, kvh, d), PREFILL_KERNELS[kernel], _ptr(status),
        _stream())
    _abi.check("sbk_swa_prefill", rc)
    return out


# ----------------------------------------------------------------- device-resident planning
def _i32(t, name, n=None):
    if t is None:
        return
    if t.dtype != torch.int32 or not t.is_contiguous() or (n is not None and t.numel() != n):
        raise ValueError(f"{name} must be contiguous int32" + (f" with {n} entries" if n is not None else ""))


def pool_init(ring: torch.Tensor, ctrl: torch.Tensor, seq_lens: Optional[torch.Tensor] = None,
              block_tables: Optional[torch.Tensor] = None) -> None:
    """ring [num_blocks] int32 <- 0..num_blocks-1, ctrl [4] int64 counters reset; lengths and
    tables cleared when given."""
    _need_cuda(ring, ctrl, seq_lens, block_tables)
    _i32(ring, "ring")
    if ctrl.dtype != torch.int64 or ctrl.numel() != 4 or not ctrl.is_contiguous():
        raise ValueError("ctrl must be contiguous int64 [4]")
    B = max_blocks = 0
    if block_tables is not None:
        _i32(block_tables, "block_tables")
        B, max_blocks = block_tables.shape
    if seq_lens is not None:
        _i32(seq_lens, "seq_lens", B if block_tables is not None else None)
        B = seq_lens.numel()
    rc = _abi.lib.sbk_pool_init(_ptr(ring), _ptr(ctrl), ring.numel(), _ptr(seq_lens), _ptr(block_tables),
                                max_blocks, B, _stream())
    _abi.check("sbk_pool_init", rc)


def plan_step(seq_lens: torch.Tensor, block_tables: torch.Tensor, slot_mapping: torch.Tensor, *,
              block_size: int, num_blocks: int, window_left: int = -1, retire: bool = True, trim: bool = False,
              n_new: Optional[torch.Tensor] = None, ring: Optional[torch.Tensor] = None,
              ctrl: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None,
              context_lens: Optional[torch.Tensor] = None, query_start_loc: Optional[torch.Tensor] = None,
              status: Optional[torch.Tensor] = None) -> None:
    """One launch that retires out-of-window blocks, allocates the blocks of the new tokens from
    the ring, writes slot_mapping / positions / context_lens / query_start_loc and advances
    seq_lens, all on device-resident state (see sbk_plan_step in include/sbk.h). ``trim``: rows
    without new tokens also give back the blocks their next token will not see."""
    _need_cuda(seq_lens, block_tables, slot_mapping, n_new, ring, ctrl, positions, context_lens,
               query_start_loc, status)
    B, max_blocks = block_tables.shape
    _i32(block_tables, "block_tables")
    _i32(seq_lens, "seq_lens", B)
    _i32(n_new, "n_new", B)
    _i32(ring, "ring", num_blocks if ring is not None else None)
    _i32(context_lens, "context_lens", B)
    _i32(query_start_loc, "query_start_loc", B + 1)
    T = slot_mapping.numel()
    for t, nm in ((slot_mapping, "slot_mapping"), (positions, "positions")):
        if t is not None and (t.dtype != torch.int64 or not t.is_contiguous() or t.numel() != T):
            raise ValueError(f"{nm} must be contiguous int64 [T]")
    if (ring is None) != (ctrl is None):
        raise ValueError("ring and ctrl come together")
    if ctrl is not None and (ctrl.dtype != torch.int64 or ctrl.numel() != 4 or not ctrl.is_contiguous()):
        raise ValueError("ctrl must be contiguous int64 [4]")
    if n_new is not None and query_start_loc is None:
        raise ValueError("n_new needs a query_start_loc buffer")
    rc = _abi.lib.sbk_plan_step(_ptr(n_new), _ptr(seq_lens), _ptr(block_tables), max_blocks, B, block_size,
                                window_left, 2 if (trim and retire) else int(retire), _ptr(ring), _ptr(ctrl), num_blocks,
                                _ptr(slot_mapping), _ptr(positions), _ptr(context_lens),
                                _ptr(query_start_loc), T, _ptr(status), _stream())
    _abi.check("sbk_plan_step", rc)


def release_rows(rows: torch.Tensor, seq_lens: torch.Tensor, block_tables: torch.Tensor, *,
                 block_size: int, num_blocks: int, ring: Optional[torch.Tensor] = None,
                 ctrl: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> None:
    """Give the blocks of the finished sequences ``rows`` [n] int32 back to the ring."""
    _need_cuda(rows, seq_lens, block_tables, ring, ctrl, status)
    B, max_blocks = block_tables.shape
    _i32(rows, "rows")
    _i32(block_tables, "block_tables")
    _i32(seq_lens, "seq_lens", B)
    _i32(ring, "ring", num_blocks if ring is not None else None)
    rc = _abi.lib.sbk_release_rows(_ptr(rows), rows.numel(), _ptr(seq_lens), _ptr(block_tables), max_blocks,
                                   B, block_size, _ptr(ring), _ptr(ctrl), num_blocks, _ptr(status), _stream())
    _abi.check("sbk_release_rows", rc)


def swa_prefill_dense(q: torch.Tensor, key: torch.Tensor, value: torch.Tensor, query_start_loc: torch.Tensor,
                      k_start_loc: torch.Tensor, max_query_len: int, *, window_left: int, causal: bool = True,
                      scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
                      key2: Optional[torch.Tensor] = None, value2: Optional[torch.Tensor] = None,
                      status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sliding-window causal attention of runs of query tokens over K/V given as tensors
    (key/value [Tk, kvh, D] bf16, possibly strided views of a wider projection output) instead of
    a paged cache: the prompt run without block tables. Sequence s owns query rows
    query_start_loc[s]:query_start_loc[s+1] and key rows k_start_loc[s]:k_start_loc[s+1]; its last
    query sees its last key. ``causal=False``: every query sees every key of its sequence."""
    _need_cuda(q, key, value, query_start_loc, k_start_loc, out, status)
    if q.dim() != 3 or key.dim() != 3 or key.shape != value.shape or q.shape[2] != key.shape[2]:
        raise ValueError("q must be [T, H, D] and key/value equal-shaped [Tk, kvh, D]")
    T, H, d = q.shape
    Tk, kvh, _ = key.shape
    if any(t.dtype != torch.bfloat16 for t in (q, key, value)):
        raise ValueError("q, key, value must be bf16")
    for t in (key, value):
        if Tk and ((d > 1 and t.stride(2) != 1) or (kvh > 1 and t.stride(1) != d)):
            raise ValueError("the heads of key/value must be contiguous")
    if Tk > 1 and key.stride(0) != value.stride(0):
        raise ValueError("key and value must share one token stride")
    if T and q.stride()[1:] != (d, 1):
        raise ValueError("the heads of q must be contiguous")
    n_seqs = query_start_loc.numel() - 1
    _i32(query_start_loc, "query_start_loc")
    _i32(k_start_loc, "k_start_loc", n_seqs + 1)
    if out is None:
        out = torch.empty((T, H, d), dtype=torch.bfloat16, device=q.device)
    elif out.shape != (T, H, d) or out.dtype != torch.bfloat16 or (T and out.stride()[1:] != (d, 1)):
        raise ValueError("out must be bf16 [T, H, D] with contiguous heads")
    if scale is None:
        scale = d ** -0.5
    n_meta = _check_meta(key2, value2, kvh, d)
    rc = _abi.lib.sbk_swa_prefill_dense(
        _ptr(q), q.stride(0) if T else H * d, _ptr(key), _ptr(value), key.stride(0) if Tk > 1 else kvh * d, Tk,
        _ptr(query_start_loc), _ptr(k_start_loc), n_seqs, int(max_query_len), H, kvh, d, window_left,
        int(causal), float(scale), _ptr(out), out.stride(0) if T else H * d, _ptr(key2), _ptr(value2), n_meta, _ptr(status),
        _stream())
    _abi.check("sbk_swa_prefill_dense", rc)
    return out
