"""GPU: the reference-facing surfaces (HF Cache, attention backend, GLA slot op) against the
golden fixtures recorded from the reference's own code and against the oracle."""
import hashlib
import math
import os

import numpy as np
import pytest
import torch

from oracle import ref_ops
from tests.helpers import mean_rel, rel_err
from tests.test_oracle_golden import CACHE_CASES, GOLD, golden_state, stream_kv

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def digest(t):
    return hashlib.sha256(t.contiguous().cpu().numpy().tobytes()).hexdigest()


@pytest.fixture(scope="module")
def pkg(sb):
    assert torch.cuda.is_available()
    return sb


# ---------------------------------------------------------------------------- HF Cache
@pytest.mark.parametrize("name", CACHE_CASES)
def test_hf_cache_stream_bit_exact_vs_reference(pkg, name):
    """The same K/V streams the reference class was run on: what update() returns (gathered
    through the block table from the paged pool) has the reference's bytes at every step."""
    from spikingbrain_7b_b200.hf_cache import Cache
    gold = np.load(os.path.join(GOLD, "cache_streams.npz"))
    meta = gold[name + "/meta"].tolist()
    B, kvh, D, W, prefill = meta[:5]
    cache = Cache()
    t = 0
    for step, n in enumerate([prefill] + meta[5:]):
        rs = torch.full((B, 2, 4, 4), float(step), device=DEV)
        cache.update(recurrent_state=rs, layer_idx=0, offset=n)
        assert cache[0]["recurrent_state"] is rs
        k, v = stream_kv(B, kvh, n, D, t, salt=len(name))
        st = cache.update(attn_state=(k.to(DEV), v.to(DEV)), layer_idx=1, offset=n, cache_kwargs={"window_size": W})
        kc, vc = st["attn_state"]
        assert digest(kc) + digest(vc) == str(gold[name + "/digests"][step]), f"step {step}"
        assert [cache.get_seq_length(0), cache.get_seq_length(1), kc.shape[-2]] == gold[name + "/seen"][step].tolist()
        t += n
    assert torch.equal(kc.cpu(), torch.from_numpy(gold[name + "/final_k"]))
    assert cache[1].paged.status.item() == 0
    legacy = cache.to_legacy_cache()
    assert torch.equal(legacy[1]["attn_state"][1].cpu(), torch.from_numpy(gold[name + "/final_v"]))
    # round trip through the legacy tuple, then keep appending
    c2 = Cache.from_legacy_cache(legacy, seen_tokens=cache.get_seq_length())
    ref = ref_ops.RefWindowCache()
    ref.update(attn_state=(kc.cpu(), vc.cpu()), layer_idx=0, offset=0, cache_kwargs={"window_size": W})
    k, v = stream_kv(B, kvh, 1, D, t, salt=3)
    c2.update(recurrent_state=None, layer_idx=0, offset=1)
    got = c2.update(attn_state=(k.to(DEV), v.to(DEV)), layer_idx=1, offset=1, cache_kwargs={"window_size": W})["attn_state"]
    exp = ref.update(attn_state=(k, v), layer_idx=0, offset=1, cache_kwargs={"window_size": W})["attn_state"]
    assert torch.equal(got[0].cpu(), exp[0]) and torch.equal(got[1].cpu(), exp[1])


def test_hf_cache_long_decode_rebases_table_and_unbounded_layer_grows(pkg):
    """Many more decode steps than the block table has columns (the live blocks are moved back),
    and a layer without a window that outgrows its pool: contents stay those of the reference."""
    from spikingbrain_7b_b200.hf_cache import Cache
    B, kvh, D, W = 2, 2, 64, 32
    cache, ref = Cache(unbounded_capacity=64), ref_ops.RefWindowCache()
    t = 0
    for step in range(400):
        n = 40 if step == 0 else 1
        k, v = stream_kv(B, kvh, n, D, t, salt=5)
        for layer, win in ((0, W), (1, None)):
            got = cache.update(attn_state=(k.to(DEV), v.to(DEV)), layer_idx=layer, offset=n,
                               cache_kwargs={"window_size": win})
            exp = ref.update(attn_state=(k, v), layer_idx=layer, offset=n, cache_kwargs={"window_size": win})
            if step % 37 == 0 or step == 399:
                g, e = got["attn_state"], exp["attn_state"]
                assert torch.equal(g[0].cpu(), e[0]) and torch.equal(g[1].cpu(), e[1]), f"step {step} layer {layer}"
        t += n
    assert cache.get_seq_length() == ref.get_seq_length() == 439


def test_hf_cache_edges_raise(pkg):
    from spikingbrain_7b_b200.hf_cache import Cache
    mk = lambda n: tuple(torch.zeros(1, 1, n, 64, device=DEV) for _ in range(2))
    c = Cache()
    c.update(attn_state=mk(60), layer_idx=0, offset=60, cache_kwargs={"window_size": 64})
    with pytest.raises(NotImplementedError):      # the reference would stop trimming here and grow for ever
        c.update(attn_state=mk(8), layer_idx=0, offset=8, cache_kwargs={"window_size": 64})
    c = Cache()
    c.update(attn_state=mk(64), layer_idx=0, offset=64, cache_kwargs={"window_size": 64})
    with pytest.raises(RuntimeError):             # the reference fails with a shape mismatch
        c.update(attn_state=mk(128), layer_idx=0, offset=128, cache_kwargs={"window_size": 64})


def test_hf_cache_fast_paths_match_reference_attention_layer(pkg):
    """cache.swa_decode on the paged window == the reference's SDPA attention layer run on the
    same injected q/k/v (fixture swa_sdpa.npz), within the bf16 attention bar."""
    from spikingbrain_7b_b200.hf_cache import Cache
    gold = np.load(os.path.join(GOLD, "swa_sdpa.npz"))
    for name in ("g7", "short"):
        B, H, kvh, D, W, prefill, steps = gold[name + "/meta"].tolist()
        x = torch.from_numpy(gold[name + "/x_bf16"]).view(torch.bfloat16).to(DEV)
        q = x[..., :H * D].view(B, -1, H, D)
        k = x[..., H * D:(H + kvh) * D].view(B, -1, kvh, D).transpose(1, 2)   # [B, kvh, T, D]
        v = x[..., (H + kvh) * D:].view(B, -1, kvh, D).transpose(1, 2)
        ref_out = torch.from_numpy(gold[name + "/decode_out"]).view(B, steps, H, D)
        cache = Cache()
        cache.update(attn_state=(k[:, :, :prefill], v[:, :, :prefill]), layer_idx=0, offset=prefill,
                     cache_kwargs={"window_size": W})
        for s in range(steps):
            pos = prefill + s
            cache.update(attn_state=(k[:, :, pos:pos + 1], v[:, :, pos:pos + 1]), layer_idx=0, offset=1,
                         cache_kwargs={"window_size": W})
            o = cache.swa_decode(q[:, pos].contiguous(), 0).float().cpu()
            tgt = ref_out[:, s].bfloat16().float()
            assert float((o - tgt).abs().max()) <= 2e-2 and mean_rel(o, tgt) <= 1e-3, f"{name} step {s}"


def test_hf_cache_gla_step_carries_state_like_the_reference_kernel(pkg):
    """cache.gla_step twice == the reference Triton kernel's two chained steps (fixture)."""
    from spikingbrain_7b_b200.hf_cache import Cache
    gold = np.load(os.path.join(GOLD, "gla_triton.npz"))
    name = "f32_d64"
    B, H, D, slots, _ = gold[name + "/meta"].tolist()
    q, k, v, g = (torch.from_numpy(gold[f"{name}/{n}"]).to(DEV) for n in "qkvg")
    slot = gold[name + "/slot"].tolist()
    state = golden_state(slots, H, D)[slot].contiguous().to(DEV)       # the cache holds one state per sequence
    cache = Cache()
    cache.update(recurrent_state=state, layer_idx=0, offset=5)
    o1 = cache.gla_step(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), g.unsqueeze(2), 0)
    o2 = cache.gla_step(q, k, v, g, 0)
    assert cache.get_seq_length() == 7 and cache[0]["recurrent_state"] is state
    assert rel_err(o1.cpu(), torch.from_numpy(gold[name + "/out1"])) <= 1e-4
    assert rel_err(o2.cpu(), torch.from_numpy(gold[name + "/out2"])) <= 1e-4
    assert rel_err(state.cpu(), torch.from_numpy(gold[name + "/state2"])[slot]) <= 1e-4


# --------------------------------------------------------------------------- GLA slot op
@pytest.mark.parametrize("name", ["f32_d128", "f32_d64", "f32_d128_g7"])
def test_my_fused_recurrent_gla_matches_reference_kernel(pkg, name):
    """The drop-in of my_fused_recurrent_gla on the reference kernel's own inputs and outputs."""
    from spikingbrain_7b_b200.gla_slots import my_fused_recurrent_gla
    gold = np.load(os.path.join(GOLD, "gla_triton.npz"))
    B, H, D, slots, _ = gold[name + "/meta"].tolist()
    q, k, v, g = (torch.from_numpy(gold[f"{name}/{n}"]).unsqueeze(2).to(DEV) for n in "qkvg")
    slot = torch.from_numpy(gold[name + "/slot"]).to(DEV)
    state0 = golden_state(slots, H, D)
    state = state0.to(DEV)
    o1 = my_fused_recurrent_gla(q, k, v, g, kv_caches=state, slot_idx=slot).cpu()
    o2 = my_fused_recurrent_gla(q, k, v, g, kv_caches=state, slot_idx=slot).cpu()
    live = (slot >= 0).cpu()
    assert o1.shape == (B, H, D)
    assert rel_err(o1[live], torch.from_numpy(gold[name + "/out1"])[live]) <= 1e-4
    assert rel_err(o2[live], torch.from_numpy(gold[name + "/out2"])[live]) <= 1e-4
    assert rel_err(state.cpu(), torch.from_numpy(gold[name + "/state2"])) <= 1e-4
    untouched = [s for s in range(slots) if s not in slot.tolist()]
    assert torch.equal(state[untouched].cpu(), state0[untouched])


def test_gla_prefill_scan_matches_reference_kernel_chain(pkg):
    """The reference kernel applied twice to the same token == one scan over that token laid down
    twice; a sequence with context_len 0 starts from zero whatever its slot holds."""
    from spikingbrain_7b_b200.gla_slots import gla_prefill_scan
    gold = np.load(os.path.join(GOLD, "gla_triton.npz"))
    name = "f32_d128"
    B, H, D, slots, _ = gold[name + "/meta"].tolist()
    q, k, v, g = (torch.from_numpy(gold[f"{name}/{n}"]) for n in "qkvg")          # [B, H, D]
    slot = torch.from_numpy(gold[name + "/slot"])
    live = [b for b in range(B) if slot[b] >= 0]
    twice = lambda t: torch.stack([t[live], t[live]], 1).reshape(2 * len(live), H, D).to(DEV)   # sequence-major
    state = golden_state(slots, H, D).to(DEV)
    qsl = torch.arange(len(live) + 1, dtype=torch.int32, device=DEV) * 2
    o = gla_prefill_scan(twice(q), twice(k), twice(v), twice(g), state, slot[live].to(DEV), qsl,
                         context_lens=torch.ones(len(live), dtype=torch.int32, device=DEV)).view(len(live), 2, H, D).cpu()
    assert rel_err(o[:, 0], torch.from_numpy(gold[name + "/out1"])[live]) <= 1e-4
    assert rel_err(o[:, 1], torch.from_numpy(gold[name + "/out2"])[live]) <= 1e-4
    assert rel_err(state.cpu(), torch.from_numpy(gold[name + "/state2"])) <= 1e-4
    # a new prompt (context_len 0) on a dirty slot
    state2 = torch.full((1, H, D, D), float("nan"), device=DEV)
    o2 = gla_prefill_scan(twice(q)[:2], twice(k)[:2], twice(v)[:2], twice(g)[:2], state2,
                          torch.zeros(1, dtype=torch.int64, device=DEV), qsl[:2],
                          context_lens=torch.zeros(1, dtype=torch.int32, device=DEV))
    ref_state = torch.zeros(1, H, D, D)
    ref = ref_ops.gla_scan_ref(twice(q)[:2].cpu(), twice(k)[:2].cpu(), twice(v)[:2].cpu(), twice(g)[:2].cpu(),
                               ref_state, [0, 2])
    assert torch.isfinite(state2).all() and rel_err(o2.cpu(), ref) <= 1e-4 and rel_err(state2.cpu(), ref_state) <= 1e-4


# ------------------------------------------------------------------------------- backend
def _decode_meta(Meta, slots, lens, table):
    return Meta(num_prefills=0, num_prefill_tokens=0, num_decode_tokens=len(lens), slot_mapping=slots,
                seq_lens=None, seq_lens_tensor=lens, max_prefill_seq_len=0, max_decode_seq_len=int(lens.max()),
                context_lens_tensor=None, block_tables=table, use_cuda_graph=False, max_query_len=1,
                max_decode_query_len=1)


def test_backend_forward_decode_steps_vs_oracle(pkg):
    """Impl.forward over several decode steps with the V0-style window-truncated tables the
    builder hands over: cache contents bit-exact, outputs within the attention bar."""
    from spikingbrain_7b_b200.backend import MetaAttentionBackend, MetaAttentionImpl, MetaAttentionMetadata
    H, kvh, D, bs, sw = 28, 4, 128, 16, 65            # sliding_window 65 -> window_left 64
    lens = [10, 64, 65, 66, 200]
    B, steps = len(lens), 20
    nb = B * ((max(lens) + steps) // bs + 2)
    g = torch.Generator().manual_seed(5)
    kv = torch.zeros(MetaAttentionBackend.get_kv_cache_shape(nb, bs, kvh, D), dtype=torch.bfloat16)
    tables = [torch.randperm(nb, generator=g)[b * (nb // B):(b + 1) * (nb // B)].tolist() for b in range(B)]
    for b, L in enumerate(lens):
        for t in range(L):
            kv[:, tables[b][t // bs], t % bs] = (torch.randn(2, kvh, D, generator=g) / math.sqrt(D)).bfloat16()
    kv_d = kv.to(DEV)
    impl = MetaAttentionImpl(H, D, D ** -0.5, kvh, None, sw, "auto")
    wl = impl.sliding_window[0]
    for step in range(steps):
        q = (torch.randn(B, H * D, generator=g) / math.sqrt(D)).bfloat16()
        k = (torch.randn(B, kvh * D, generator=g) / math.sqrt(D)).bfloat16()
        v = (torch.randn(B, kvh * D, generator=g) / math.sqrt(D)).bfloat16()
        slots = torch.tensor([tables[b][L // bs] * bs + L % bs for b, L in enumerate(lens)])
        lens = [L + 1 for L in lens]
        ref_ops.paged_append(k.view(B, kvh, D), v.view(B, kvh, D), kv[0], kv[1], slots)
        # what the V0 model runner passes under a sliding window: trailing blocks, clipped length
        sw_blocks = (sw + bs - 1) // bs
        trunc_tables, trunc_lens = [], []
        for b, L in enumerate(lens):
            n_blocks = (L + bs - 1) // bs
            suff = L % bs
            cur = sw_blocks + (1 if suff else 0)
            trunc_lens.append(min(L, sw_blocks * bs + suff) if suff else min(L, sw_blocks * bs))
            trunc_tables.append(tables[b][:n_blocks][-cur:])
        width = max(len(t) for t in trunc_tables)
        tt = torch.tensor([t + [0] * (width - len(t)) for t in trunc_tables], dtype=torch.int32)
        full_t = torch.tensor([t[:(max(lens) + bs - 1) // bs] for t in tables], dtype=torch.int32)
        ref = ref_ops.swa_paged_decode_ref(q.view(B, H, D), kv[0], kv[1], full_t, lens, wl, D ** -0.5)
        md = _decode_meta(MetaAttentionMetadata, slots.to(DEV), torch.tensor(trunc_lens, dtype=torch.int32, device=DEV),
                          tt.to(DEV))
        out = torch.empty(B, H * D, dtype=torch.bfloat16, device=DEV)
        ret = impl.forward(None, q.to(DEV), k.to(DEV), v.to(DEV), None, None, None, kv_d, md, output=out)
        assert ret is out
        o = out.view(B, H, D).float().cpu()
        tgt = ref.bfloat16().float()
        assert float((o - tgt).abs().max()) <= 2e-2 and mean_rel(o, tgt) <= 1e-3, f"step {step}"
    assert torch.equal(kv_d.cpu(), kv) and impl.status() == 0


def test_backend_forward_chunked_prefill_plus_decode(pkg):
    """A mixed batch: two prompt chunks (one continuing a cached context) followed by two decodes.
    Every prompt token attends causally inside the window through its sequence's block table."""
    from spikingbrain_7b_b200.backend import MetaAttentionImpl, MetaAttentionMetadata
    H, kvh, D, bs, sw = 14, 2, 128, 16, 33
    g = torch.Generator().manual_seed(6)
    ctx = [0, 40, 90, 7]            # cached tokens before this step
    new = [50, 30, 1, 1]            # tokens of this step (2 prefill chunks, 2 decodes)
    B = 4
    nb = 40
    perm = torch.randperm(nb, generator=g).tolist()
    tables = [perm[b * 10:(b + 1) * 10] for b in range(B)]
    kv = torch.zeros(2, nb, bs, kvh, D, dtype=torch.bfloat16)
    for b in range(B):
        for t in range(ctx[b]):
            kv[:, tables[b][t // bs], t % bs] = (torch.randn(2, kvh, D, generator=g) / math.sqrt(D)).bfloat16()
    T = sum(new)
    q = (torch.randn(T, H, D, generator=g) / math.sqrt(D)).bfloat16()
    k = (torch.randn(T, kvh, D, generator=g) / math.sqrt(D)).bfloat16()
    v = (torch.randn(T, kvh, D, generator=g) / math.sqrt(D)).bfloat16()
    slots, owner = [], []
    for b in range(B):
        for p in range(ctx[b], ctx[b] + new[b]):
            slots.append(tables[b][p // bs] * bs + p % bs)
            owner.append((b, p))
    slots = torch.tensor(slots)
    kv_d = kv.to(DEV)
    ref_ops.paged_append(k, v, kv[0], kv[1], slots)
    impl = MetaAttentionImpl(H, D, D ** -0.5, kvh, None, sw, "auto")
    wl = impl.sliding_window[0]
    tab = torch.tensor(tables, dtype=torch.int32)
    ref = torch.stack([ref_ops.swa_paged_decode_ref(q[i:i + 1], kv[0], kv[1], tab[b:b + 1], [p + 1], wl, D ** -0.5)[0]
                       for i, (b, p) in enumerate(owner)])
    seq_lens = [c + n for c, n in zip(ctx, new)]
    qsl = [0, 50, 80, 81, 82]
    md = MetaAttentionMetadata(
        num_prefills=2, num_prefill_tokens=80, num_decode_tokens=2, slot_mapping=slots.to(DEV), seq_lens=seq_lens,
        seq_lens_tensor=torch.tensor(seq_lens, dtype=torch.int32, device=DEV), max_prefill_seq_len=70,
        max_decode_seq_len=91, context_lens_tensor=torch.tensor(ctx, dtype=torch.int32, device=DEV),
        block_tables=tab.to(DEV), use_cuda_graph=False, max_query_len=50, max_decode_query_len=1,
        query_start_loc=torch.tensor(qsl, dtype=torch.int32, device=DEV),
        seq_start_loc=torch.tensor([0, 50, 120, 211, 219], dtype=torch.int32, device=DEV))
    out = torch.empty(T, H, D, dtype=torch.bfloat16, device=DEV)
    impl.forward(None, q.to(DEV), k.to(DEV), v.to(DEV), None, None, None, kv_d, md, output=out)
    assert torch.equal(kv_d.cpu(), kv) and impl.status() == 0
    o, tgt = out.float().cpu(), ref.bfloat16().float()
    assert float((o - tgt).abs().max()) <= 2e-2 and mean_rel(o, tgt) <= 1e-3


def test_backend_forward_with_meta_tokens(pkg):
    """The 76B-style use of the backend: key2/value2 (128 sink tokens) with query2=None, a decode
    batch. Equals one softmax over sink keys + window keys."""
    from spikingbrain_7b_b200.backend import MetaAttentionImpl, MetaAttentionMetadata
    from tests.helpers import make_paged_kv
    H, kvh, D, bs, sw = 28, 4, 128, 16, 129
    lens = [300, 5, 128]
    kv, table, nb = make_paged_kv(lens, -1, kvh, D, bs, seed=80)
    g = torch.Generator().manual_seed(81)
    q = (torch.randn(3, H, D, generator=g) / math.sqrt(D)).bfloat16()
    k2 = (torch.randn(128, kvh, D, generator=g) / math.sqrt(D)).bfloat16()
    v2 = (torch.randn(128, kvh, D, generator=g) / math.sqrt(D)).bfloat16()
    impl = MetaAttentionImpl(H, D, D ** -0.5, kvh, None, sw, "auto", num_meta_tokens=128)
    md = _decode_meta(MetaAttentionMetadata, torch.full((3,), -1, dtype=torch.int64, device=DEV),
                      torch.tensor(lens, dtype=torch.int32, device=DEV), table.to(DEV))
    out = torch.empty(3, H, D, dtype=torch.bfloat16, device=DEV)
    knew = torch.zeros(3, kvh, D, dtype=torch.bfloat16, device=DEV)      # slots are -1: nothing is appended
    impl.forward(None, q.to(DEV), knew, knew, None, k2.to(DEV), v2.to(DEV), kv.to(DEV), md, output=out)
    ref = ref_ops.swa_paged_decode_ref(q, kv[0], kv[1], table, lens, sw - 1, D ** -0.5, key2=k2, value2=v2)
    o, tgt = out.float().cpu(), ref.bfloat16().float()
    assert impl.status() == 0
    assert float((o - tgt).abs().max()) <= 2e-2 and mean_rel(o, tgt) <= 1e-3


def test_backend_forward_unsupported_paths_raise(pkg):
    from spikingbrain_7b_b200.backend import MetaAttentionImpl, MetaAttentionMetadata
    impl = MetaAttentionImpl(28, 128, 1.0, 4, None, 65, "auto")
    q = torch.zeros(2, 28, 128, dtype=torch.bfloat16, device=DEV)
    kx = torch.zeros(2, 4, 128, dtype=torch.bfloat16, device=DEV)
    kv = torch.zeros(2, 4, 16, 4, 128, dtype=torch.bfloat16, device=DEV)
    md = _decode_meta(MetaAttentionMetadata, torch.tensor([0, 16], device=DEV),
                      torch.tensor([1, 1], dtype=torch.int32, device=DEV),
                      torch.tensor([[0], [1]], dtype=torch.int32, device=DEV))
    with pytest.raises(AssertionError):
        impl.forward(None, q, kx, kx, None, None, None, kv, md, output=None)
    impl2 = MetaAttentionImpl(28, 128, 1.0, 4, None, 65, "auto", num_meta_tokens=2)
    with pytest.raises(NotImplementedError):       # the meta tokens' own queries do not go with decode tokens
        impl2.forward(None, q, kx, kx, q, kx, kx, kv, md, output=torch.empty(4, 28, 128, dtype=torch.bfloat16, device=DEV))
    pm = MetaAttentionMetadata(num_prefills=1, num_prefill_tokens=2, num_decode_tokens=0,
                               slot_mapping=torch.tensor([-1, -1], device=DEV), seq_lens=[2],
                               seq_lens_tensor=torch.tensor([2], dtype=torch.int32, device=DEV),
                               max_prefill_seq_len=2, max_decode_seq_len=0,
                               context_lens_tensor=torch.tensor([0], dtype=torch.int32, device=DEV),
                               block_tables=torch.zeros(1, 0, dtype=torch.int32, device=DEV), use_cuda_graph=False,
                               max_query_len=2, query_start_loc=torch.tensor([0, 2], dtype=torch.int32, device=DEV),
                               seq_start_loc=torch.tensor([0, 2], dtype=torch.int32, device=DEV))
    # a prompt whose K/V cannot be reached through tables attends over the key/value tensors themselves
    out = torch.empty_like(q)
    impl.forward(None, q, kx, kx, None, None, None, kv, pm, output=out)
    want = ref_ops.swa_prefill_dense_ref(q.view(2, 28, 128).cpu(), kx.view(2, 4, 128).cpu(), kx.view(2, 4, 128).cpu(),
                                         [0, 2], [0, 2], impl.sliding_window[0], impl.scale)
    assert float((out.view(2, 28, 128).float().cpu() - want).abs().max()) <= 2e-2


def test_backend_multi_token_decode_through_block_tables(pkg):
    """max_decode_query_len > 1 (several new tokens per sequence, e.g. speculative decoding): every
    query attends causally inside the window over the cache, its own K/V appended by the same call."""
    from spikingbrain_7b_b200.backend import MetaAttentionBackend, MetaAttentionImpl, MetaAttentionMetadata
    H, kvh, D, bs, sw = 28, 4, 128, 16, 65
    ctx, new = [100, 7, 64], [3, 1, 5]
    B, T = len(ctx), sum(new)
    g = torch.Generator().manual_seed(81)
    nb = 40
    perm = torch.randperm(nb, generator=g).tolist()
    tables = [perm[b * 10:(b + 1) * 10] for b in range(B)]
    kv = torch.zeros(MetaAttentionBackend.get_kv_cache_shape(nb, bs, kvh, D), dtype=torch.bfloat16)
    for b in range(B):
        for t in range(ctx[b]):
            kv[:, tables[b][t // bs], t % bs] = (torch.randn(2, kvh, D, generator=g) / math.sqrt(D)).bfloat16()
    q = (torch.randn(T, H * D, generator=g) / math.sqrt(D)).bfloat16()
    k = (torch.randn(T, kvh * D, generator=g) / math.sqrt(D)).bfloat16()
    v = (torch.randn(T, kvh * D, generator=g) / math.sqrt(D)).bfloat16()
    qsl, slots = [0], []
    for b in range(B):
        qsl.append(qsl[-1] + new[b])
        slots += [tables[b][t // bs] * bs + t % bs for t in range(ctx[b], ctx[b] + new[b])]
    lens = [c + n for c, n in zip(ctx, new)]
    impl = MetaAttentionImpl(H, D, D ** -0.5, kvh, None, sw, "auto")
    wl = impl.sliding_window[0]
    md = MetaAttentionMetadata(num_prefills=0, num_prefill_tokens=0, num_decode_tokens=T,
                               slot_mapping=torch.tensor(slots, device=DEV), seq_lens=lens,
                               seq_lens_tensor=torch.tensor(lens, dtype=torch.int32, device=DEV),
                               max_prefill_seq_len=0, max_decode_seq_len=max(lens), context_lens_tensor=None,
                               block_tables=torch.tensor(tables, dtype=torch.int32, device=DEV), use_cuda_graph=False,
                               max_query_len=max(new), max_decode_query_len=max(new),
                               query_start_loc=torch.tensor(qsl, dtype=torch.int32, device=DEV),
                               seq_start_loc=None)
    kv_d = kv.to(DEV)
    out = torch.empty(T, H * D, dtype=torch.bfloat16, device=DEV)
    impl.forward(None, q.to(DEV), k.to(DEV), v.to(DEV), None, None, None, kv_d, md, output=out)
    assert impl.status() == 0
    ref_ops.paged_append(k.view(T, kvh, D), v.view(T, kvh, D), kv[0], kv[1], torch.tensor(slots))
    assert torch.equal(kv_d.cpu(), kv)
    table_t = torch.tensor(tables, dtype=torch.int32)
    for b in range(B):
        for i in range(new[b]):
            pos = ctx[b] + i
            ref = ref_ops.swa_paged_decode_ref(q[qsl[b] + i].view(1, H, D), kv[0], kv[1], table_t[b:b + 1], [pos + 1], wl,
                                               D ** -0.5)[0].bfloat16().float()
            got = out[qsl[b] + i].view(H, D).float().cpu()
            assert float((got - ref).abs().max()) <= 2e-2, (b, i)


def test_backend_prompt_run_with_the_meta_tokens_own_queries(pkg):
    """query2: the step that first computes the sink tokens. Their queries see all of key2/value2 (not
    causally) and their outputs come first; the prompt's tokens see the sinks plus their causal window."""
    from spikingbrain_7b_b200.backend import MetaAttentionImpl, MetaAttentionMetadata
    H, kvh, D, sw, M = 14, 2, 128, 33, 32
    lens = [50, 9]
    T = sum(lens)
    g = torch.Generator().manual_seed(82)
    rn = lambda *s: (torch.randn(*s, generator=g) / math.sqrt(D)).bfloat16()
    q, k, v = rn(T, H * D), rn(T, kvh * D), rn(T, kvh * D)
    q2, k2, v2 = rn(M, H * D), rn(M, kvh * D), rn(M, kvh * D)
    qsl = [0, 50, 59]
    impl = MetaAttentionImpl(H, D, D ** -0.5, kvh, None, sw, "auto", num_meta_tokens=M)
    wl = impl.sliding_window[0]
    md = MetaAttentionMetadata(num_prefills=2, num_prefill_tokens=T, num_decode_tokens=0,
                               slot_mapping=torch.full((T,), -1, device=DEV), seq_lens=lens,
                               seq_lens_tensor=torch.tensor(lens, dtype=torch.int32, device=DEV),
                               max_prefill_seq_len=max(lens), max_decode_seq_len=0,
                               context_lens_tensor=torch.zeros(2, dtype=torch.int32, device=DEV),
                               block_tables=torch.zeros(2, 0, dtype=torch.int32, device=DEV), use_cuda_graph=False,
                               max_query_len=max(lens), query_start_loc=torch.tensor(qsl, dtype=torch.int32, device=DEV),
                               seq_start_loc=torch.tensor(qsl, dtype=torch.int32, device=DEV))
    out = torch.empty(M + T, H * D, dtype=torch.bfloat16, device=DEV)
    impl.forward(None, q.to(DEV), k.to(DEV), v.to(DEV), q2.to(DEV), k2.to(DEV), v2.to(DEV),
                 torch.empty(0, dtype=torch.bfloat16, device=DEV), md, output=out)
    assert impl.status() == 0
    k2r, v2r = k2.view(M, kvh, D), v2.view(M, kvh, D)
    want_meta = ref_ops.swa_prefill_dense_ref(q2.view(M, H, D), k2r, v2r, [0, M], [0, M], -1, D ** -0.5, causal=False)
    want_rest = ref_ops.swa_prefill_dense_ref(q.view(T, H, D), k.view(T, kvh, D), v.view(T, kvh, D), qsl, qsl, wl,
                                              D ** -0.5, k2r, v2r)
    got = out.view(M + T, H, D).float().cpu()
    assert float((got[:M] - want_meta.bfloat16().float()).abs().max()) <= 2e-2
    assert float((got[M:] - want_rest.bfloat16().float()).abs().max()) <= 2e-2
    assert mean_rel(got[M:], want_rest.bfloat16().float()) <= 1e-3


def test_backend_prompt_run_without_block_tables(pkg):
    """The un-chunked first prompt (and the profiling run, kv_cache.numel() == 0): q, k, v are column
    slices of one projection output; attention over the prompt's own K/V, K/V also appended."""
    from spikingbrain_7b_b200.backend import MetaAttentionBackend, MetaAttentionImpl, MetaAttentionMetadata
    H, kvh, D, bs, sw = 28, 4, 128, 16, 129
    lens = [200, 1, 77, 350]
    T = sum(lens)
    g = torch.Generator().manual_seed(80)
    qkv = (torch.randn(T, (H + 2 * kvh) * D, generator=g) / math.sqrt(D)).bfloat16().to(DEV)
    q, k, v = qkv[:, :H * D], qkv[:, H * D:(H + kvh) * D], qkv[:, (H + kvh) * D:]
    qsl = [0]
    for n in lens:
        qsl.append(qsl[-1] + n)
    nb = sum((n + bs - 1) // bs for n in lens) + 2
    perm = torch.randperm(nb, generator=g).tolist()
    slots, used = [], 0
    for n in lens:
        blocks = perm[used:used + (n + bs - 1) // bs]; used += len(blocks)
        slots += [blocks[t // bs] * bs + t % bs for t in range(n)]
    impl = MetaAttentionImpl(H, D, D ** -0.5, kvh, None, sw, "auto")
    wl = impl.sliding_window[0]
    want = ref_ops.swa_prefill_dense_ref(q.view(T, H, D).cpu(), k.reshape(T, kvh, D).cpu(), v.reshape(T, kvh, D).cpu(),
                                         qsl, qsl, wl, D ** -0.5).bfloat16().float()
    for kv in (torch.zeros(MetaAttentionBackend.get_kv_cache_shape(nb, bs, kvh, D), dtype=torch.bfloat16, device=DEV),
               torch.empty(0, dtype=torch.bfloat16, device=DEV)):
        md = MetaAttentionMetadata(num_prefills=len(lens), num_prefill_tokens=T, num_decode_tokens=0,
                                   slot_mapping=torch.tensor(slots, device=DEV), seq_lens=lens,
                                   seq_lens_tensor=torch.tensor(lens, dtype=torch.int32, device=DEV),
                                   max_prefill_seq_len=max(lens), max_decode_seq_len=0,
                                   context_lens_tensor=torch.zeros(len(lens), dtype=torch.int32, device=DEV),
                                   block_tables=torch.zeros(len(lens), 0, dtype=torch.int32, device=DEV),
                                   use_cuda_graph=False, max_query_len=max(lens),
                                   query_start_loc=torch.tensor(qsl, dtype=torch.int32, device=DEV),
                                   seq_start_loc=torch.tensor(qsl, dtype=torch.int32, device=DEV))
        out = torch.empty(T, H * D, dtype=torch.bfloat16, device=DEV)
        impl.forward(None, q, k, v, None, None, None, kv, md, output=out)
        assert impl.status() == 0
        o = out.view(T, H, D).float().cpu()
        assert float((o - want).abs().max()) <= 2e-2 and mean_rel(o, want) <= 1e-3
        if kv.numel():   # the prompt's K/V went into the cache as well
            flat = kv.view(2, nb * bs, kvh, D)
            assert torch.equal(flat[0, torch.tensor(slots, device=DEV)], k.reshape(T, kvh, D))
            assert torch.equal(flat[1, torch.tensor(slots, device=DEV)], v.reshape(T, kvh, D))


# ------------------------------------------------------- fused neighbours through the surfaces
def test_hf_cache_update_rotary_equals_rotate_then_update(pkg):
    """update_rotary (one launch) == the oracle's apply_rotary_pos_emb on q, k followed by update():
    a prompt longer than the window (every token rotated, the last W cached), then decode steps."""
    from spikingbrain_7b_b200 import ops
    from spikingbrain_7b_b200.hf_cache import Cache
    B, H, kvh, D, W, prompt = 2, 4, 2, 128, 32, 45
    table = ops.build_cos_sin_cache(D, 512, 10000.0, torch.bfloat16, device=DEV)
    g = torch.Generator().manual_seed(70)
    fused, plain = Cache(), Cache()
    t = 0
    for n in [prompt] + [1] * 6:
        q = torch.randn(B, H, n, D, generator=g).bfloat16()
        k = torch.randn(B, kvh, n, D, generator=g).bfloat16()
        v = torch.randn(B, kvh, n, D, generator=g).bfloat16()
        pos = torch.arange(t, t + n)[None, :]
        cos, sin = ref_ops.rope_cos_sin_ref(pos[0], D, 10000.0, torch.bfloat16)
        rot = lambda x: ref_ops.rope_ref(x.transpose(1, 2).reshape(B * n, -1, D), cos.repeat(B, 1),
                                         sin.repeat(B, 1)).view(B, n, -1, D).transpose(1, 2)
        q_rot = fused.update_rotary(q.to(DEV), k.to(DEV), v.to(DEV), pos.to(DEV), table, layer_idx=0,
                                    window_size=W)
        want = plain.update(attn_state=(rot(k).to(DEV), v.to(DEV)), layer_idx=0, offset=n,
                            cache_kwargs={"window_size": W})["attn_state"]
        got = fused[0]["attn_state"]
        assert torch.equal(q_rot.cpu(), rot(q))
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
        assert fused.get_seq_length() == plain.get_seq_length() == t + n
        t += n
    assert fused[0].paged.status.item() == 0


def test_backend_forward_with_fused_rotary_equals_rotate_then_forward(pkg):
    """MetaAttentionImpl.forward(positions=, cos_sin_cache=) on un-rotated q, k == forward on
    q, k rotated beforehand by the oracle: same cache bytes, same attention output."""
    from spikingbrain_7b_b200 import ops
    from spikingbrain_7b_b200.backend import MetaAttentionImpl, MetaAttentionMetadata
    B, H, kvh, D, bs, W = 3, 28, 4, 128, 16, 64
    g = torch.Generator().manual_seed(71)
    seq_lens = torch.tensor([90, 17, 64], dtype=torch.int32)
    max_blocks = 8
    nb = B * max_blocks
    tables = torch.arange(nb, dtype=torch.int32).view(B, max_blocks)
    cache0 = torch.randn(2, nb, bs, kvh, D, generator=g).bfloat16()
    slots = torch.tensor([int(tables[b, (int(seq_lens[b]) - 1) // bs]) * bs + (int(seq_lens[b]) - 1) % bs
                          for b in range(B)], dtype=torch.int64)
    q = torch.randn(B, H, D, generator=g).bfloat16()
    k = torch.randn(B, kvh, D, generator=g).bfloat16()
    v = torch.randn(B, kvh, D, generator=g).bfloat16()
    positions = (seq_lens - 1).to(torch.int64)
    table = ops.build_cos_sin_cache(D, 128, 1000000.0, torch.bfloat16, device=DEV)
    cos, sin = ref_ops.rope_cos_sin_ref(positions, D, 1000000.0, torch.bfloat16)

    def run(qi, ki, **kw):
        impl = MetaAttentionImpl(H, D, D ** -0.5, kvh, None, W + 1, "auto")
        meta = _decode_meta(MetaAttentionMetadata, slots.to(DEV), seq_lens.to(DEV), tables.to(DEV))
        kv = cache0.clone().to(DEV)
        out = torch.empty(B, H * D, dtype=torch.bfloat16, device=DEV)
        impl.forward(None, qi.to(DEV), ki.to(DEV), v.to(DEV), None, None, None, kv, meta, output=out, **kw)
        assert impl.status() == 0
        return out, kv

    o_fused, kv_fused = run(q.clone(), k.clone(), positions=positions.to(DEV), cos_sin_cache=table)
    o_plain, kv_plain = run(ref_ops.rope_ref(q, cos, sin), ref_ops.rope_ref(k, cos, sin))
    assert torch.equal(kv_fused, kv_plain) and torch.equal(o_fused, o_plain)


def test_gla_decode_layer_surface_matches_layer_oracle(pkg):
    """gla_decode_layer (projection outputs in, normed read-out out, one launch) == the oracle of
    the layer's decode branch; bf16 in and out."""
    from spikingbrain_7b_b200.gla_slots import gla_decode_layer
    B, H, Hkv, D, slots = 6, 28, 4, 128, 9
    g = torch.Generator().manual_seed(72)
    qp = torch.randn(B, H, D, generator=g).bfloat16()
    kp = torch.randn(B, Hkv, D, generator=g).bfloat16()
    v = torch.randn(B, Hkv, D, generator=g).bfloat16()
    gl = (3 * torch.randn(B, Hkv, D, generator=g)).bfloat16()
    w = (1 + 0.3 * torch.randn(D, generator=g)).bfloat16()
    state = torch.randn(slots, H, D, D, generator=g)
    slot = torch.randperm(slots, generator=g)[:B].to(torch.int64)
    ref_state = state.clone()
    want = ref_ops.gla_layer_step_ref(qp, kp, v, gl, ref_state, slot, 16.0, w, 1e-5)
    state_d = state.to(DEV)
    got = gla_decode_layer(qp.to(DEV), kp.to(DEV), v.to(DEV), gl.to(DEV), state_d, slot.to(DEV), w.to(DEV))
    assert got.dtype == torch.bfloat16
    assert rel_err(state_d.cpu(), ref_state) <= 1e-4
    diff = (got.float().cpu() - want).abs()
    assert float((diff / want.abs().clamp_min(1e-2)).max()) <= 2 ** -7   # one bf16 rounding of the output
