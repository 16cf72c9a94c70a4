"""Plain-PyTorch CPU restatements of the reference algorithms (test infrastructure only).

Each function names the reference file:line it follows (paths inside
BICLab/SpikingBrain-7B).
"""
from typing import Dict, List, Optional, Tuple

import torch


# --------------------------------------------------------------------------- HF cache
class RefWindowCache:
    """Restates Cache.update / get_seq_length of hf_7B_model/cache.py:40-118.

    states[i] is a dict(recurrent_state, attn_state, conv_state). The seen-token
    counter moves only for layer 0 (:70-71). First insert of a layer trims to the
    last `window_size` tokens (:81-83); afterwards a layer whose cached length
    EQUALS the window rolls left and overwrites its tail (:94-104), any other
    length concatenates (:105-107).
    """

    def __init__(self, seen_tokens: int = 0):
        self.states: List[Dict] = []
        self._seen_tokens = seen_tokens

    def __len__(self):
        return len(self.states)

    def __getitem__(self, i):
        if i < len(self.states):
            return self.states[i]
        raise KeyError(f"Cache only has {len(self)} layers, attempted to access layer with index {i}")

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return 0 if len(self.states) <= layer_idx else self._seen_tokens

    def update(self, recurrent_state=None, attn_state=None, conv_state=None, layer_idx: int = 0,
               offset: int = 1, cache_kwargs: Optional[dict] = None) -> Dict:
        if layer_idx == 0:
            self._seen_tokens += offset
        window = None
        n_new = 0
        if attn_state is not None:
            n_new = attn_state[0].shape[-2]
            window = cache_kwargs.get("window_size", None)
            if not isinstance(attn_state, tuple) or len(attn_state) != 2:
                raise ValueError("`attn_state` must be a tuple of two tensors for key/value states")
        if len(self.states) <= layer_idx:
            if attn_state is not None and window is not None and n_new > window:
                attn_state = tuple(t[..., -window:, :].contiguous() for t in attn_state)
            state = dict(recurrent_state=recurrent_state, attn_state=attn_state, conv_state=conv_state)
            self.states.append(state)
            return state
        state = self.states[layer_idx]
        if recurrent_state is not None:
            state["recurrent_state"] = recurrent_state
        if attn_state is not None:
            k_old, v_old = state["attn_state"]
            if window is not None and k_old.shape[-2] == window:
                k_new = k_old.roll(-n_new, -2)
                v_new = v_old.roll(-n_new, -2)
                k_new[..., -n_new:, :] = attn_state[0]
                v_new[..., -n_new:, :] = attn_state[1]
            else:
                k_new = torch.cat([k_old, attn_state[0]], -2)
                v_new = torch.cat([v_old, attn_state[1]], -2)
            state["attn_state"] = (k_new, v_new)
        if conv_state is not None:
            state["conv_state"] = conv_state
        return state


# ------------------------------------------------------------------------ paged cache
def paged_append(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor,
                 v_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """reshape_and_cache_flash as called at vllm_hymeta/attention/meta_attention.py:790-799
    with kv_cache_dtype "auto": token i goes to cache[slot // block, slot % block];
    negative slots (PAD_SLOT_ID, :558) are skipped. In place."""
    bs = k_cache.shape[1]
    for i, s in enumerate(slot_mapping.tolist()):
        if s < 0:
            continue
        k_cache[s // bs, s % bs] = key[i]
        v_cache[s // bs, s % bs] = value[i]


def first_visible(seq_len: int, n_new: int, window_left: int) -> int:
    """First token the oldest query of this step still sees: the flash-attn rule the
    reference relies on (keys in [i - window_left, i]) for the step's first query
    at position seq_len - n_new."""
    if window_left < 0:
        return 0
    return max(0, seq_len - n_new - window_left)


def retire_blocks(block_tables: torch.Tensor, seq_lens: List[int], n_new: List[int],
                  window_left: int, block_size: int) -> List[List[int]]:
    """Sliding-window block retirement: logical blocks that end before the first visible
    token are dropped from the table (entry -> -1) and their ids returned per sequence in
    logical order. This is the policy behind the window-truncated block table of
    meta_attention.py:479-485 (the reference delegates it to vLLM's block manager)."""
    out = []
    for b, (L, n) in enumerate(zip(seq_lens, n_new)):
        first_live = min(first_visible(L, max(n, 1), window_left) // block_size, block_tables.shape[1])
        ids = []
        for j in range(first_live):
            if block_tables[b, j] >= 0:
                ids.append(int(block_tables[b, j]))
                block_tables[b, j] = -1
        out.append(ids)
    return out


def window_gather(k_cache: torch.Tensor, v_cache: torch.Tensor, table: torch.Tensor, seq_len: int,
                  window_left: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Tokens [t0, seq_len) of one sequence through its block table, head-first
    [kvh, n_vis, D] -- the layout of attn_state in hf_7B_model/cache.py:94-108."""
    bs = k_cache.shape[1]
    t0 = first_visible(seq_len, 1, window_left)
    toks = torch.arange(t0, seq_len)
    blk = table[toks // bs].long()
    k = k_cache[blk, toks % bs]  # [n, kvh, D]
    v = v_cache[blk, toks % bs]
    return k.transpose(0, 1).contiguous(), v.transpose(0, 1).contiguous()


# -------------------------------------------------------------------------- attention
def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[.., kvh, L, D] -> [.., kvh*n_rep, L, D], repeat_interleave order
    (hf_7B_model/window_attention_sdpa.py repeat_kv; same in gla_attention.py:24-34)."""
    if n_rep == 1:
        return x
    *lead, kvh, L, D = x.shape
    return x.unsqueeze(-3).expand(*lead, kvh, n_rep, L, D).reshape(*lead, kvh * n_rep, L, D)


def swa_decode_ref(q: torch.Tensor, k_win: torch.Tensor, v_win: torch.Tensor, scale: float,
                   window: Optional[int] = None, return_lse: bool = False):
    """One query per sequence against its cached window, in fp32, following
    hf_7B_model/window_attention_sdpa.py:140-214: keys repeated per query group, mask
    `k_pos <= q_abs and k_pos > q_abs - window` (:144-148) with the query at the last
    key position, softmax(q k^T * scale) v.
      q [H, D]; k_win, v_win [kvh, n, D] (the n most recent tokens, query token last)."""
    H, D = q.shape
    kvh, n, _ = k_win.shape
    k = repeat_kv(k_win.float(), H // kvh)
    v = repeat_kv(v_win.float(), H // kvh)
    s = torch.einsum("hd,hnd->hn", q.float(), k) * scale
    if window is not None:
        k_pos = torch.arange(n)
        q_abs = n - 1
        allowed = (k_pos <= q_abs) & (k_pos > q_abs - window)
        s = s.masked_fill(~allowed[None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("hn,hnd->hd", p, v)
    if return_lse:
        return o, torch.logsumexp(s, dim=-1)
    return o


def swa_paged_decode_ref(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         block_tables: torch.Tensor, seq_lens: List[int], window_left: int,
                         scale: float, return_lse: bool = False, key2: Optional[torch.Tensor] = None,
                         value2: Optional[torch.Tensor] = None):
    """The decode call of meta_attention.py:955-981 (flash_attn fwd_kvcache with causal=True,
    window (window_left, -1), fa_kernel_metatoken.py:84-105): per sequence gather the visible
    tokens through the block table, then swa_decode_ref. q [B, H, D] -> [B, H, D] fp32.
    key2 / value2 [n_meta, kvh, D]: meta tokens of the 76B-style backend use (None for the 7B path)."""
    outs, lses = [], []
    for b, L in enumerate(seq_lens):
        if L <= 0:
            outs.append(torch.zeros(q.shape[1:], dtype=torch.float32))
            lses.append(torch.full((q.shape[1],), float("-inf")))
            continue
        k, v = window_gather(k_cache, v_cache, block_tables[b], L, window_left)
        if key2 is not None:
            # meta (sink) tokens: always visible, in front of the window -- the mask of
            # vllm_hymeta/attention/fa_kernel_metatoken.py:390-391 and the key order of :397-398;
            # the reference reaches the same softmax by a second pass over k2/v2 and a
            # log-sum-exp merge (:157-192)
            k = torch.cat([key2.transpose(0, 1), k], 1)
            v = torch.cat([value2.transpose(0, 1), v], 1)
        o, lse = swa_decode_ref(q[b], k, v, scale, return_lse=True)
        outs.append(o)
        lses.append(lse)
    o = torch.stack(outs)
    return (o, torch.stack(lses)) if return_lse else o


# -------------------------------------------------------------------------------- GLA
def gla_step_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
                 state: torch.Tensor, slot_idx: Optional[torch.Tensor] = None,
                 scale: Optional[float] = None) -> torch.Tensor:
    """Single-token GLA step in fp32, in place on `state` [slots, H, D, D], in the order of
    vllm_hymeta/model_for_7B/my_fused_recurrent.py:60-80: decay the old state by exp(g)
    along the key index, add the outer product k v^T, read the output out of the NEW
    state with q * scale. q [B, H, D]; k, v, g [B, Hkv, D] (Hkv divides H; head h uses
    kv head h // (H // Hkv), the repeat_kv order of gla_attention.py:265-267).
    slot -1 leaves the state row untouched and the output row zero (:34-36)."""
    B, H, D = q.shape
    Hkv = k.shape[1]
    rep = H // Hkv
    if scale is None:
        scale = D ** -0.5
    out = torch.zeros(B, H, D, dtype=torch.float32)
    kf = k.float().repeat_interleave(rep, dim=1)
    vf = v.float().repeat_interleave(rep, dim=1)
    gf = g.float().repeat_interleave(rep, dim=1)
    qf = q.float() * scale
    for b in range(B):
        s = b if slot_idx is None else int(slot_idx[b])
        if s < 0:
            continue
        new = torch.exp(gf[b])[:, :, None] * state[s] + kf[b][:, :, None] * vf[b][:, None, :]
        state[s] = new
        out[b] = torch.einsum("hk,hkv->hv", qf[b], new)
    return out


def gla_scan_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, state: torch.Tensor,
                 query_start_loc: List[int], slot_idx: Optional[List[int]] = None,
                 reset: Optional[List[bool]] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Runs of tokens through the recurrence with state carry: the per-sequence prefill loop of
    vllm_hymeta/model_for_7B/gla_attention.py:179-211 (fused_chunk_gla with initial_state from the
    slot, final state copied back), restated as gla_step_ref applied token after token.
    q [T, H, D], k/v/g [T, Hkv, D] token-major -> [T, H, D] fp32; `state` advanced in place."""
    out = torch.zeros(q.shape, dtype=torch.float32)
    for s in range(len(query_start_loc) - 1):
        slot = s if slot_idx is None else int(slot_idx[s])
        if slot < 0:
            continue
        if reset is not None and reset[s]:
            state[slot] = 0
        for t in range(query_start_loc[s], query_start_loc[s + 1]):
            out[t] = gla_step_ref(q[t:t + 1], k[t:t + 1], v[t:t + 1], g[t:t + 1], state,
                                  torch.tensor([slot]), scale=scale)[0]
    return out


def gla_prepare_inputs(q_proj: torch.Tensor, k_proj: torch.Tensor, gk_proj: torch.Tensor,
                       normalizer: float = 16.0):
    """Input preparation of hf_7B_model/gla_attention.py:134-145: ReLU feature map on q and k,
    log-decay g = logsigmoid(gk) / gate_logit_normalizer."""
    return torch.relu(q_proj), torch.relu(k_proj), torch.nn.functional.logsigmoid(gk_proj) / normalizer


def gla_norm_ref(o: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """The GLA layer's g_norm on the read-out [.., H, D]: RMS norm over each head's D values
    (hf_7B_model/gla_attention.py:89,170; vllm_hymeta/model_for_7B/gla_attention.py:177,233), in the
    arithmetic of the reference's rms_norm_ref (hf_7B_model/layernorm.py:39-52), kept in fp32."""
    of = o.float()
    rstd = 1.0 / torch.sqrt(of.square().mean(dim=-1, keepdim=True) + eps)
    return of * rstd * weight.float()


def gla_layer_step_ref(q_proj: torch.Tensor, k_proj: torch.Tensor, v: torch.Tensor, gk_logits: torch.Tensor,
                       state: torch.Tensor, slot_idx: Optional[torch.Tensor] = None,
                       normalizer: float = 16.0, norm_weight: Optional[torch.Tensor] = None,
                       eps: float = 1e-5, scale: Optional[float] = None) -> torch.Tensor:
    """Decode branch of the GLA layer between its projections and its output gate
    (vllm_hymeta/model_for_7B/gla_attention.py:250-267 then :225-233): feature map, gate,
    the recurrent step, g_norm. Rows with slot -1 stay zero. Returns fp32 [B, H, D]."""
    q, k, g = gla_prepare_inputs(q_proj, k_proj, gk_logits, normalizer)
    o = gla_step_ref(q, k, v, g, state, slot_idx, scale=scale)
    if norm_weight is None:
        return o
    normed = gla_norm_ref(o, norm_weight, eps)
    if slot_idx is not None:
        normed[torch.as_tensor(slot_idx) < 0] = 0
    return normed


def rope_cos_sin_ref(positions: torch.Tensor, rot_dim: int, base: float, dtype: torch.dtype):
    """cos, sin [T, rot_dim] of RotaryEmbedding.forward (hf_7B_model/window_attention.py:23-47):
    fp32 angles position * base^(-2i/rot_dim), the half-table repeated twice, cast to `dtype`."""
    inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.int64).float() / rot_dim))
    freqs = positions.float()[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rope_ref(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """apply_rotary_pos_emb (hf_7B_model/window_attention.py:49-80) on token-major x [T, heads, D]
    with cos, sin [T, D]: (x * cos) + (rotate_half(x) * sin), every tensor op in x's dtype."""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return (x * cos[:, None, :]) + (rot * sin[:, None, :])


class StepPlannerRef:
    """CPU model of the device-resident step planner (libsbk's sbk_pool_init / sbk_plan_step /
    sbk_release_rows): per-row lengths and block tables, a FIFO ring of free block ids. It carries
    out, with the same visibility rule as retire_blocks / first_visible above, the per-sequence
    work of MetaAttentionMetadataBuilder._add_seq_group (vllm_hymeta/attention/meta_attention.py:
    435-494) and of MetaAttentionMetadata.advance_step (:338-409), plus the block hand-out the
    reference leaves to the engine's block manager. Policy: rows in index order; within a step
    every row's out-of-window blocks are pushed (oldest first) before any block is popped; a step
    that cannot be served changes nothing and returns None."""

    def __init__(self, num_blocks: int, block_size: int, B: int, max_blocks: int,
                 window_left: int = -1, allocate: bool = True):
        self.bs, self.B, self.max_blocks, self.wl = block_size, B, max_blocks, window_left
        self.num_blocks = num_blocks
        self.ring = list(range(num_blocks)) if allocate else None
        self.lens = [0] * B
        self.table = [[-1] * max_blocks for _ in range(B)]
        self.min_free = num_blocks

    def plan(self, n_new: Optional[List[int]] = None, T: Optional[int] = None, retire: bool = True,
             trim: bool = False):
        """``trim``: rows without new tokens give back what their next token will not see."""
        n_new = [1] * self.B if n_new is None else [max(0, int(n)) for n in n_new]
        total = sum(n_new)
        T = total if T is None else T
        pushes, need = [], 0
        for b, n in enumerate(n_new):
            if n == 0 and not (trim and retire):
                continue
            L = self.lens[b]
            if n > 0:
                lb0, lb1 = L // self.bs, (L + n - 1) // self.bs
                if lb1 >= self.max_blocks or total > T:
                    return None
                need += sum(1 for lb in range(lb0, lb1 + 1) if self.table[b][lb] < 0)
            if retire:
                first_live = min(first_visible(L + n, n, self.wl) // self.bs, self.max_blocks)
                j = first_live - 1
                while j >= 0 and self.table[b][j] >= 0:
                    j -= 1
                pushes.append((b, j + 1, first_live))
        n_push = sum(hi - lo for _, lo, hi in pushes)
        if need > ((len(self.ring) + n_push) if self.ring is not None else 0):
            return None
        for b, lo, hi in pushes:
            for j in range(lo, hi):
                if self.ring is not None:
                    self.ring.append(self.table[b][j])
                self.table[b][j] = -1
        slots, positions, ctx, qsl = [], [], [], [0]
        for b, n in enumerate(n_new):
            L = self.lens[b]
            ctx.append(L)
            qsl.append(qsl[-1] + n)
            for lb in range(L // self.bs, (L + n - 1) // self.bs + 1 if n else 0):
                if self.table[b][lb] < 0:
                    self.table[b][lb] = self.ring.pop(0)
            for t in range(L, L + n):
                slots.append(self.table[b][t // self.bs] * self.bs + t % self.bs)
                positions.append(t)
            self.lens[b] = L + n
        if self.ring is not None:
            self.min_free = min(self.min_free, len(self.ring))
        slots += [-1] * (T - total)
        positions += [0] * (T - total)
        return dict(slot_mapping=slots, positions=positions, context_lens=ctx, query_start_loc=qsl)

    def release(self, rows: List[int]) -> None:
        for b in rows:
            L = self.lens[b]
            last = min((L - 1) // self.bs if L > 0 else -1, self.max_blocks - 1)
            j = last
            while j >= 0 and self.table[b][j] >= 0:
                j -= 1
            for i in range(j + 1, last + 1):
                if self.ring is not None:
                    self.ring.append(self.table[b][i])
                self.table[b][i] = -1
            self.lens[b] = 0


def swa_prefill_dense_ref(q: torch.Tensor, key: torch.Tensor, value: torch.Tensor, query_start_loc: List[int],
                          k_start_loc: List[int], window_left: int, scale: float,
                          key2: Optional[torch.Tensor] = None, value2: Optional[torch.Tensor] = None,
                          causal: bool = True) -> torch.Tensor:
    """The prompt run without block tables (vllm_hymeta/attention/meta_attention.py:843-884:
    varlen attention of q over the prompt's own key/value, causal, window (window_left, 0)), in
    fp32: query i of a sequence with n_q queries and n_k keys sits at key position n_k - n_q + i
    (flash-attn aligns the causal mask to the end of the keys) and sees keys
    [position - window_left, position] plus the sink keys key2/value2 if given. causal=False: every
    query sees every key of its sequence (the pass of the sink tokens' own queries over key2/value2,
    fa_kernel_metatoken.py:262-276).
    q [T, H, D]; key, value [Tk, kvh, D] -> [T, H, D] fp32."""
    T, H, D = q.shape
    kvh = key.shape[1]
    out = torch.zeros(T, H, D)
    for s in range(len(query_start_loc) - 1):
        q0, q1 = query_start_loc[s], query_start_loc[s + 1]
        k0, k1 = k_start_loc[s], k_start_loc[s + 1]
        n_q, n_k = q1 - q0, k1 - k0
        ks = repeat_kv(key[k0:k1].float().transpose(0, 1), H // kvh)       # [H, n_k, D]
        vs = repeat_kv(value[k0:k1].float().transpose(0, 1), H // kvh)
        sc = torch.einsum("ihd,hnd->hin", q[q0:q1].float(), ks) * scale       # [H, n_q, n_k]
        pos = (n_k - n_q) + torch.arange(n_q)[:, None]
        kp = torch.arange(n_k)[None, :]
        ok = kp <= pos if causal else torch.ones(n_q, n_k, dtype=torch.bool)
        if causal and window_left >= 0:
            ok = ok & (kp >= pos - window_left)
        sc = sc.masked_fill(~ok[None], float("-inf"))
        if key2 is not None:
            k2 = repeat_kv(key2.float().transpose(0, 1), H // kvh)
            v2 = repeat_kv(value2.float().transpose(0, 1), H // kvh)
            s2 = torch.einsum("ihd,hnd->hin", q[q0:q1].float(), k2) * scale
            p = torch.softmax(torch.cat([s2, sc], dim=-1), dim=-1)
            o = torch.einsum("hin,hnd->ihd", p[..., :k2.shape[1]], v2) + torch.einsum("hin,hnd->ihd", p[..., k2.shape[1]:], vs)
        else:
            o = torch.einsum("hin,hnd->ihd", torch.softmax(sc, dim=-1), vs)
        out[q0:q1] = o
    return out
