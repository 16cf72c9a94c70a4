"""The HF ``Cache`` surface of hf_7B_model/cache.py over paged device memory.

Same constructor, ``update`` / ``get_seq_length`` / ``get_max_length`` /
``to_legacy_cache`` / ``from_legacy_cache`` and container protocol as the reference
class, same values in everything it returns -- but the sliding-window K/V of a layer
live in a paged pool that is appended to in place (2 KiB per token and layer at 7B
shapes) instead of being rolled or re-concatenated on every step
(hf_7B_model/cache.py:94-107 moves the whole window per token).

What a caller gets back from ``update(...)['attn_state']`` is gathered on demand through
the block table, so a caller that only wants attention over the window should use the
fast paths instead and never materialise it:
    cache.swa_decode(q, layer_idx)           sliding-window attention on the paged K/V
    cache.gla_step(q, k, v, g, layer_idx)    in-place GLA state step + read-out

Behaviour at the edges of the reference class (hf_7B_model/cache.py:96-107):
  * an append of n tokens onto a FULL window with n > window raises RuntimeError (the
    reference fails with a shape mismatch there);
  * an append that takes a not-yet-full window past the window size raises
    NotImplementedError: the reference silently stops trimming from then on and grows
    without bound, which no caller wants from a paged pool.
Tensors must live on a CUDA device: there is no CPU path.
"""
from typing import Any, Dict, List, Optional, Tuple

import torch
import transformers

from . import ops
from .block_pool import DeviceStepPlanner


class _PagedWindow:
    """Paged K/V of one sliding-window layer for a fixed batch of equally long sequences. Lengths,
    block table, free ring and slot mapping live on the device (DeviceStepPlanner): an append is
    one planner launch and one append launch, with nothing copied from the host."""

    def __init__(self, B: int, kvh: int, D: int, dtype: torch.dtype, device, window: Optional[int],
                 block_size: int, capacity_tokens: int):
        self.B, self.kvh, self.D, self.dtype, self.device = B, kvh, D, dtype, device
        self.window = window
        self.bs = block_size
        self.n_cached = 0  # tokens the reference class would hold now
        self.L = 0         # length the planner holds for every row (relative to the table's column 0)
        self._scratch: Dict[int, Tuple[torch.Tensor, int, int]] = {}   # query heads -> decode workspace
        self._alloc(capacity_tokens)

    def _alloc(self, capacity_tokens: int) -> None:
        self.max_blocks = -(-capacity_tokens // self.bs) + 2
        if self.window is None:
            per_row = self.max_blocks
        else:  # the window, the partial blocks at both ends, and a chunk of up to `window` new tokens
            per_row = min(self.max_blocks, 2 * (-(-self.window // self.bs)) + 3)
        nb = self.B * per_row
        self.plan = DeviceStepPlanner(nb, self.bs, -1 if self.window is None else self.window - 1,
                                      self.B, self.max_blocks, self.device, max_tokens=self.B)
        self.kv = torch.zeros(2, nb, self.bs, self.kvh, self.D, dtype=self.dtype, device=self.device)
        self.table_d, self.lens_d, self.status = self.plan.block_tables, self.plan.seq_lens, self.plan.status
        self._n_new = torch.zeros(self.B, dtype=torch.int32, device=self.device)
        self.L = 0
        self._first_live = 0   # table columns the planner has retired so far (the same for every row)
        self._scratch.clear()  # sized by the table width

    # The logical block index of a sequence only ever grows; before it would run off the table
    # the live blocks are moved back to column 0 (positions are relative, nothing else changes).
    def _make_room(self, n: int) -> None:
        if (self.L + n + self.bs - 1) // self.bs <= self.max_blocks:
            return
        if self.window is None:  # unbounded layer: double the pool and carry the contents over
            k_all, v_all = self.gather()
            self._alloc(2 * (self.L + n))
            self.n_cached = 0
            self.append(k_all, v_all)
            return
        # every row has the same length, so the same leading blocks have been retired
        shift = self._first_live
        if shift == 0:
            raise RuntimeError("window layer out of table columns with nothing retired")
        t = self.table_d
        moved = t[:, shift:].clone()
        t.fill_(-1)
        t[:, :self.max_blocks - shift] = moved
        self.lens_d.sub_(shift * self.bs)
        self.L -= shift * self.bs
        self._first_live = 0
        if (self.L + n + self.bs - 1) // self.bs > self.max_blocks:
            raise RuntimeError(f"{n} new tokens do not fit the table of a window-{self.window} layer")

    def append(self, k: torch.Tensor, v: torch.Tensor, rope=None) -> Optional[torch.Tensor]:
        """k, v: [B, kvh, n, D] -- the reference layout of `attn_state`. ``rope`` = (q [B, H, n, D]
        or None, position_ids [B, n], cos_sin_cache): k arrives un-rotated and is rotated on its way
        into the cache by the same launch, which also rotates q; the rotated q is returned."""
        n = n_in = k.shape[-2]
        W = self.window
        if self.n_cached == 0:
            if W is not None and n > W:  # first insert keeps the last `window` tokens (cache.py:81-83)
                n = W
                if rope is None:
                    k, v = k[..., -W:, :], v[..., -W:, :]
            n_cached = n
        elif W is not None and self.n_cached == W:
            if n > W:
                raise RuntimeError(f"cannot roll {n} new tokens into a full window of {W}")
            n_cached = W
        else:
            if W is not None and self.n_cached + n > W:
                raise NotImplementedError(
                    f"appending {n} tokens to {self.n_cached} cached ones crosses the window of {W}; "
                    "the reference class stops trimming in this case and grows without bound")
            n_cached = self.n_cached + n
        self._make_room(n)
        self.n_cached = n_cached
        if W is not None:   # what this step's planner launch retires (rule of sbk_plan_step)
            self._first_live = max(self._first_live, max(0, self.L - (W - 1)) // self.bs)
        self.L += n
        plan = self.plan
        if plan.slot_mapping.numel() < self.B * n:
            plan.slot_mapping = torch.full((self.B * n,), -1, dtype=torch.int64, device=self.device)
            plan.positions = torch.zeros(self.B * n, dtype=torch.int64, device=self.device)
        if n == 1:
            plan.plan()
        else:
            self._n_new.fill_(n)
            plan.plan(self._n_new)
        slots = plan.slot_mapping[:self.B * n]
        # token-major rows [T, kvh, D]; a view for one new token, a copy for a prompt chunk
        tm = lambda t: t.transpose(1, 2).reshape(self.B * t.shape[-2], t.shape[1], self.D).contiguous()
        kt, vt = tm(k), tm(v)
        if rope is None:
            ops.kv_append(kt, vt, self.kv[0], self.kv[1], slots, status=self.status)
            return None
        q, position_ids, table = rope
        if n_in != n:  # prompt longer than the window: every token is rotated, the last W are cached
            full = torch.full((self.B, n_in), -1, dtype=torch.int64, device=self.device)
            full[:, n_in - n:] = slots.view(self.B, n)
            slots = full.view(-1)
        qt = tm(q) if q is not None else None
        ops.rope_kv_append(qt, kt, vt, self.kv[0], self.kv[1], slots,
                           position_ids.to(torch.int64).expand(self.B, n_in).reshape(-1).contiguous(), table,
                           status=self.status)
        return None if qt is None else qt.view(self.B, n_in, q.shape[1], self.D).transpose(1, 2)

    def gather(self) -> Tuple[torch.Tensor, torch.Tensor]:
        return ops.kv_gather(self.kv[0], self.kv[1], self.table_d, self.lens_d, self.n_cached,
                             window_left=self.n_cached - 1, status=self.status)

    def decode(self, q: torch.Tensor, scale: Optional[float], out=None) -> torch.Tensor:
        # one zero-initialised workspace per head count, sized for the fixed batch and the widest
        # window the table can hold: no allocation and no memset per step
        H = q.shape[1]
        if H not in self._scratch:
            vis = self.max_blocks * self.bs if self.window is None else min(self.max_blocks * self.bs, self.window)
            split = ops.swa_auto_split(self.B, vis, self.device)
            pieces = ops.swa_max_pieces(vis, split, self.B, self.device)
            self._scratch[H] = (ops.swa_workspace(self.B, H, self.D, pieces, self.device), split, pieces)
        ws, split, pieces = self._scratch[H]
        return ops.swa_decode(q, self.kv[0], self.kv[1], self.table_d, self.lens_d,
                              window_left=self.n_cached - 1, scale=scale, out=out, workspace=ws,
                              split_chunks=split, max_pieces=pieces, status=self.status)


class _LayerState(dict):
    """The per-layer dict of the reference class; 'attn_state' of a paged layer is gathered
    through the block table when it is read."""

    def __init__(self, recurrent_state=None, attn_state=None, conv_state=None,
                 paged: Optional[_PagedWindow] = None):
        super().__init__(recurrent_state=recurrent_state, attn_state=attn_state, conv_state=conv_state)
        self.paged = paged

    def __getitem__(self, key):
        if key == "attn_state" and self.paged is not None:
            return self.paged.gather()
        return super().__getitem__(key)

    def get(self, key, default=None):
        return self[key] if key in self else default

    def materialise(self) -> Dict[str, Any]:
        return {k: self[k] for k in ("recurrent_state", "attn_state", "conv_state")}


class Cache(transformers.cache_utils.Cache):
    """Drop-in for hf_7B_model/cache.py:11 `Cache` (same public surface and values)."""

    def __init__(self, seen_tokens: int = 0, *, block_size: int = 16, unbounded_capacity: int = 4096):
        # like the reference, the transformers base initialiser is not chained
        self.states: List[_LayerState] = []
        self._seen_tokens = seen_tokens
        self._block_size = block_size
        self._unbounded_capacity = unbounded_capacity

    def __getitem__(self, layer_idx: int) -> Dict[str, Any]:
        if layer_idx < len(self):
            return self.states[layer_idx]
        raise KeyError(f"Cache only has {len(self)} layers, attempted to access layer with index {layer_idx}")

    def __iter__(self):
        for state in self.states:
            yield state

    def __len__(self):
        return len(self.states)

    def _new_paged(self, attn_state, window) -> _PagedWindow:
        k = attn_state[0]
        if not k.is_cuda:
            raise RuntimeError("this Cache keeps K/V in paged CUDA memory; CPU tensors are not supported")
        B, kvh, n, D = k.shape
        cap = 3 * window + 2 * self._block_size if window is not None else max(self._unbounded_capacity, 2 * n)
        return _PagedWindow(B, kvh, D, k.dtype, k.device, window, self._block_size, cap)

    def update(self, recurrent_state: torch.Tensor = None,
               attn_state: Tuple[torch.Tensor, torch.Tensor] = None,
               conv_state: Tuple[torch.Tensor] = None, layer_idx: int = 0,
               offset: Optional[int] = 1, cache_kwargs: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        if layer_idx == 0:
            self._seen_tokens += offset
        window = rope = None
        if attn_state is not None:
            window = (cache_kwargs or {}).get("window_size", None)
            rope = (cache_kwargs or {}).get("rotary", None)
            if not isinstance(attn_state, tuple) or len(attn_state) != 2:
                raise ValueError("`attn_state` must be a tuple of two tensors for key/value states")
        if len(self.states) <= layer_idx:
            paged = None
            if attn_state is not None:
                paged = self._new_paged(attn_state, window)
                self._rotated_q = paged.append(*attn_state, rope=rope)
            state = _LayerState(recurrent_state=recurrent_state, conv_state=conv_state, paged=paged)
            self.states.append(state)
            return state
        state = self.states[layer_idx]
        if recurrent_state is not None:
            dict.__setitem__(state, "recurrent_state", recurrent_state)
        if attn_state is not None:
            if state.paged is None:  # a layer restored from a legacy tuple: page it now
                dense = dict.__getitem__(state, "attn_state")
                state.paged = self._new_paged(dense if dense is not None else attn_state, window)
                if dense is not None:
                    # restored tensors are what the reference would hold: already trimmed
                    state.paged.append(*dense)
                    dict.__setitem__(state, "attn_state", None)
            if state.paged.window != window:
                raise ValueError("window_size changed between updates of one layer")
            self._rotated_q = state.paged.append(*attn_state, rope=rope)
        if conv_state is not None:
            dict.__setitem__(state, "conv_state", conv_state)
        return state

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        if len(self.states) <= layer_idx:
            return 0
        return self._seen_tokens

    def get_max_length(self) -> Optional[int]:
        return None

    def to_legacy_cache(self) -> Tuple[Dict[str, Any], ...]:
        return tuple(s.materialise() for s in self.states)

    @classmethod
    def from_legacy_cache(cls, past_key_values: Optional[Tuple[Dict[str, Any], ...]] = None,
                          seen_tokens: int = 0) -> "Cache":
        cache = cls(seen_tokens)
        if past_key_values is not None:
            for d in past_key_values:
                cache.states.append(_LayerState(recurrent_state=d.get("recurrent_state"),
                                                attn_state=d.get("attn_state"),
                                                conv_state=d.get("conv_state")))
        return cache

    def status(self) -> int:
        """The device-side status bits (SBK_ST_*) raised so far by the planner and the kernels of every
        paged layer, OR-ed together; 0 = nothing to report. One device synchronisation. A non-zero
        word means some step did not do what was asked: e.g. SBK_ST_OUT_OF_BLOCKS / SBK_ST_TABLE_FULL
        from the planner, after which that step's tokens were NOT appended. After SBK_ST_WAIT_TIMEOUT
        the decode workspaces are stale; they are dropped here so that the next step gets fresh ones."""
        words = [s.paged.status for s in self.states if s.paged is not None]
        if not words:
            return 0
        acc = words[0].clone()
        for w in words[1:]:
            acc |= w
        bits = int(acc.item())
        if bits & 4:   # SBK_ST_WAIT_TIMEOUT
            for s in self.states:
                if s.paged is not None:
                    s.paged._scratch.clear()
        return bits

    # ------------------------------------------------------------------ fast paths
    def update_rotary(self, q: Optional[torch.Tensor], k: torch.Tensor, v: torch.Tensor,
                      position_ids: torch.Tensor, cos_sin_cache: torch.Tensor, layer_idx: int,
                      window_size: Optional[int] = None) -> Optional[torch.Tensor]:
        """`apply_rotary_pos_emb(q, k, cos, sin)` followed by `update(attn_state=(k, v), layer_idx,
        offset=n, cache_kwargs={"window_size": W})` (hf_7B_model/window_attention.py:161-175) as one
        launch: q [B, H, n, D], k and v [B, kvh, n, D] come un-rotated, `position_ids` [B, n] (or
        [1, n]) index ``cos_sin_cache`` (ops.build_cos_sin_cache). Returns the rotated q
        [B, H, n, D] (for n == 1 contiguous input it is q itself, rotated in place)."""
        self._rotated_q = None
        self.update(attn_state=(k, v), layer_idx=layer_idx, offset=k.shape[-2],
                    cache_kwargs={"window_size": window_size, "rotary": (q, position_ids, cos_sin_cache)})
        q_rot, self._rotated_q = self._rotated_q, None
        return q_rot

    def swa_decode(self, q: torch.Tensor, layer_idx: int, scale: Optional[float] = None,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Attention of one query token per sequence over the layer's cached window, the
        query's own K/V having been appended by `update` first. q: [B, H, D] or [B, H, 1, D]
        (bf16); returns [B, H, D]. Equals softmax(q K^T * scale) V over exactly the tokens
        `update(...)['attn_state']` would return."""
        state = self[layer_idx]
        if state.paged is None:
            raise ValueError(f"layer {layer_idx} holds no paged attention state")
        if q.dim() == 4:
            q = q.squeeze(2)
        return state.paged.decode(q.contiguous(), scale, out)

    def gla_step(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
                 layer_idx: int, scale: Optional[float] = None, **fused) -> torch.Tensor:
        """One-token GLA step of layer `layer_idx`, in place on its recurrent state:
        what `fused_recurrent_gla(q, k, v, g, initial_state=S, output_final_state=True)`
        followed by `update(recurrent_state=S', layer_idx, offset=1)` does in
        hf_7B_model/gla_attention.py:153-168, without allocating a new state.
        q [B, H, 1, D] or [B, H, D]; k, v, g likewise with H or Hkv heads. Returns o [B, H, D].
        ``fused`` (relu_qk, gate_logit_normalizer, norm_weight, norm_eps of ops.gla_step) folds in
        the layer's feature map, gate and g_norm (:134-145, :170)."""
        sq = lambda t: (t.squeeze(2) if t.dim() == 4 else t).contiguous()
        q, k, v, g = sq(q), sq(k), sq(v), sq(g)
        B, H, D = q.shape
        S = self[layer_idx]["recurrent_state"] if layer_idx < len(self) else None
        if S is None:
            S = torch.zeros(B, H, D, D, dtype=torch.float32, device=q.device)
        o = ops.gla_step(q, k, v, g, S, scale=scale, **fused)
        self.update(recurrent_state=S, layer_idx=layer_idx, offset=1)
        return o

    def gla_chunk(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
                  layer_idx: int, scale: Optional[float] = None, **fused) -> torch.Tensor:
        """A run of T tokens through the GLA layer `layer_idx` with state carry: what
        `chunk_gla(q, k, v, g, initial_state=S, output_final_state=True)` followed by
        `update(recurrent_state=S', layer_idx, offset=T)` does in hf_7B_model/gla_attention.py:155-168.
        q [B, H, T, D] (the reference's head-first layout), k/v/g [B, H or Hkv, T, D];
        returns o [B, H, T, D]. The state tensor of the layer is advanced in place. ``fused`` as
        in gla_step."""
        B, H, T, D = q.shape
        tm = lambda t: t.transpose(1, 2).reshape(B * T, t.shape[1], D).contiguous()   # token-major rows
        S = self[layer_idx]["recurrent_state"] if layer_idx < len(self) else None
        if S is None:
            S = torch.zeros(B, H, D, D, dtype=torch.float32, device=q.device)
        qsl = torch.arange(B + 1, dtype=torch.int32, device=q.device) * T
        # few long runs are spread over the GPU (chunk-parallel form), as the reference's chunk_gla is
        ws = ops.gla_scan_workspace(B, T, H, D, q.device)
        o = ops.gla_scan(tm(q), tm(k), tm(v), tm(g), S, qsl, scale=scale, max_query_len=T, workspace=ws, **fused)
        self.update(recurrent_state=S, layer_idx=layer_idx, offset=T)
        return o.view(B, T, H, D).transpose(1, 2)
