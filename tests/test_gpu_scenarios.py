"""GPU: the two serving scenarios of the scope table at reduced scale, through the surfaces.

  * long-context eviction: a long prompt prefilled in chunks, then decode; only the window's blocks
    stay resident, retired blocks are handed out again, outputs follow the dense-history oracle;
  * continuous-batching churn: sequences of Zipf-distributed length finish and are replaced every
    step over a fragmenting pool, with the heads also split four ways (one kv head per shard) and
    the shard outputs gathered.
"""
import math

import numpy as np
import pytest
import torch

from oracle import ref_ops
from tests.helpers import mean_rel

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
H, KVH, D, BS = 28, 4, 128, 16


def _dense_ref(q, k_hist, v_hist, pos, wl):
    """Oracle on the dense history of one sequence: query at `pos` sees [pos - wl, pos]."""
    lo = max(0, pos - wl)
    return ref_ops.swa_decode_ref(q, k_hist[lo:pos + 1].transpose(0, 1), v_hist[lo:pos + 1].transpose(0, 1), D ** -0.5)


def test_long_context_chunked_prefill_then_decode_with_eviction(sb):
    from spikingbrain_7b_b200.backend import MetaAttentionBackend, MetaAttentionImpl, MetaAttentionMetadata
    from spikingbrain_7b_b200.block_pool import SlidingWindowBlockManager
    B, prompt, chunk, steps, sw = 2, 2048, 512, 40, 257
    impl = MetaAttentionImpl(H, D, D ** -0.5, KVH, None, sw, "auto")
    wl = impl.sliding_window[0]
    max_blocks = (prompt + steps) // BS + 2
    live_bound = (wl + chunk) // BS + 3
    nb = B * live_bound + 8          # far fewer blocks than the 2 x 131 the whole history would need
    mgr = SlidingWindowBlockManager(nb, BS, wl, B, max_blocks)
    for r in range(B):
        mgr.admit(r)
    kv_d = torch.zeros(MetaAttentionBackend.get_kv_cache_shape(nb, BS, KVH, D), dtype=torch.bfloat16, device=DEV)
    g = torch.Generator().manual_seed(40)
    T = prompt + steps
    k_hist = (torch.randn(B, T, KVH, D, generator=g) / math.sqrt(D)).bfloat16()
    v_hist = (torch.randn(B, T, KVH, D, generator=g) / math.sqrt(D)).bfloat16()
    q_hist = (torch.randn(B, T, H, D, generator=g) / math.sqrt(D)).bfloat16()
    ever_retired, reused = set(), 0

    def check(out, rows, positions):
        for o, b, p in zip(out, rows, positions):
            tgt = _dense_ref(q_hist[b, p], k_hist[b], v_hist[b], p, wl).bfloat16().float()
            assert float((o - tgt).abs().max()) <= 2e-2 and mean_rel(o, tgt) <= 1e-3, f"seq {b} pos {p}"

    pos = 0
    while pos < prompt:                                   # ---- chunked prefill
        plan = mgr.advance(np.full(B, chunk), pad_inactive=False)
        reused += sum(1 for e in plan.new_entries.tolist() if e[2] in ever_retired)
        for ids in plan.retired:
            ever_retired.update(ids)
        assert max(mgr.resident_blocks(r) for r in range(B)) <= live_bound
        sl = slice(pos, pos + chunk)
        q = q_hist[:, sl].reshape(B * chunk, H, D).to(DEV)
        k = k_hist[:, sl].reshape(B * chunk, KVH, D).to(DEV)
        v = v_hist[:, sl].reshape(B * chunk, KVH, D).to(DEV)
        md = MetaAttentionMetadata(
            num_prefills=B, num_prefill_tokens=B * chunk, num_decode_tokens=0,
            slot_mapping=torch.from_numpy(plan.slot_mapping).to(DEV), seq_lens=[pos + chunk] * B,
            seq_lens_tensor=torch.full((B,), pos + chunk, dtype=torch.int32, device=DEV),
            max_prefill_seq_len=pos + chunk, max_decode_seq_len=0,
            context_lens_tensor=torch.full((B,), pos, dtype=torch.int32, device=DEV),
            block_tables=torch.from_numpy(mgr.table).to(DEV), use_cuda_graph=False, max_query_len=chunk,
            query_start_loc=torch.from_numpy(plan.query_start_loc).to(DEV),
            seq_start_loc=torch.arange(B + 1, dtype=torch.int32, device=DEV) * (pos + chunk))
        out = torch.empty(B * chunk, H, D, dtype=torch.bfloat16, device=DEV)
        impl.forward(None, q, k, v, None, None, None, kv_d, md, output=out)
        sample = [0, 1, 15, 16, 255, 256, 257, chunk - 1]
        idx = [b * chunk + s for b in range(B) for s in sample]
        check(out[idx].float().cpu(), [b for b in range(B) for _ in sample], [pos + s for _ in range(B) for s in sample])
        pos += chunk
    assert ever_retired, "the prompt is several windows long: blocks must have been retired"

    for step in range(steps):                             # ---- decode
        plan = mgr.advance(np.ones(B, dtype=np.int64))
        reused += sum(1 for e in plan.new_entries.tolist() if e[2] in ever_retired)
        for ids in plan.retired:
            ever_retired.update(ids)
        assert max(mgr.resident_blocks(r) for r in range(B)) <= wl // BS + 2
        md = MetaAttentionMetadata(
            num_prefills=0, num_prefill_tokens=0, num_decode_tokens=B,
            slot_mapping=torch.from_numpy(plan.slot_mapping).to(DEV), seq_lens=None,
            seq_lens_tensor=torch.from_numpy(plan.seq_lens).to(DEV), max_prefill_seq_len=0,
            max_decode_seq_len=pos + 1, context_lens_tensor=None, block_tables=torch.from_numpy(mgr.table).to(DEV),
            use_cuda_graph=False, max_query_len=1, max_decode_query_len=1)
        out = torch.empty(B, H, D, dtype=torch.bfloat16, device=DEV)
        impl.forward(None, q_hist[:, pos].to(DEV), k_hist[:, pos].to(DEV), v_hist[:, pos].to(DEV), None, None, None,
                     kv_d, md, output=out)
        check(out.float().cpu(), list(range(B)), [pos] * B)
        pos += 1
    assert reused > 0, "retired blocks must come back through the free list"
    assert impl.status() == 0
    assert mgr.pool.num_free + int((mgr.table >= 0).sum()) == nb


def test_long_context_at_full_scale_on_the_device_planner(sb):
    """The long-context configuration at its stated lengths, scaled in layers (one sliding-window and
    one GLA layer), on the planner that lives on the GPU: a 131072-token prompt in 16 chunks of 8192
    through MetaAttentionImpl.forward (append + windowed attention over the block tables) and the
    chunk-parallel GLA scan, then 512 one-token steps. Checked: the resident blocks return to the
    window after every chunk (trim) and every step, the peak is the window plus the chunk in flight,
    retired block ids come back, sampled query rows follow the dense-history oracle, and the GLA
    state after the whole prompt equals a single token-by-token scan on two sampled heads."""
    from spikingbrain_7b_b200 import ops
    from spikingbrain_7b_b200.backend import MetaAttentionImpl, MetaAttentionMetadata
    from spikingbrain_7b_b200.block_pool import DeviceStepPlanner
    from spikingbrain_7b_b200.gla_slots import GLACacheManager, gla_prefill_scan, my_fused_recurrent_gla
    from tests.helpers import rel_err
    prompt, chunk, steps, wl = 131072, 8192, 512, 4096
    impl = MetaAttentionImpl(H, D, D ** -0.5, KVH, None, wl + 1, "auto")
    assert impl.sliding_window[0] == wl
    max_blocks = (prompt + steps) // BS + 2
    n_blocks = (wl + chunk) // BS + 4 + 16          # the whole history would need 8224 blocks
    plan = DeviceStepPlanner(n_blocks, BS, wl, 1, max_blocks, DEV, max_tokens=chunk)
    kv_d = torch.zeros(2, n_blocks, BS, KVH, D, dtype=torch.bfloat16, device=DEV)
    gla = GLACacheManager(torch.float32, (1, 1, H, D, D), device=DEV)
    _, slot_idx = gla.current_run_tensors({"r0": [0]})
    scan_ws = ops.gla_scan_workspace(1, chunk, H, D, DEV)
    assert scan_ws is not None
    Ttot = prompt + steps
    k_hist = torch.empty(Ttot, KVH, D, dtype=torch.bfloat16)
    v_hist = torch.empty(Ttot, KVH, D, dtype=torch.bfloat16)
    heads = (2, 25)                                   # GLA heads followed on the CPU (kv heads 0 and 3)
    g_hist = {h: [torch.empty(prompt, 1, D, dtype=torch.bfloat16) for _ in range(4)] for h in heads}
    n_new = torch.full((1,), chunk, dtype=torch.int32, device=DEV)
    gla_status = torch.zeros(1, dtype=torch.int32, device=DEV)
    seen_blocks, reused, peak = set(), 0, 0
    mk = lambda n, h, seed: (torch.randn(n, h, D, device=DEV, generator=torch.Generator(DEV).manual_seed(seed)) / math.sqrt(D)).bfloat16()

    def check_rows(out, q_rows, positions):
        for o, qr, p in zip(out, q_rows, positions):
            tgt = _dense_ref(qr, k_hist, v_hist, p, wl).bfloat16().float()
            assert float((o - tgt).abs().max()) <= 2e-2 and mean_rel(o, tgt) <= 1e-3, f"position {p}"

    def account():
        nonlocal reused, peak
        row = plan.block_tables[0].tolist()
        live = {e for e in row if e >= 0}
        return live

    for c in range(prompt // chunk):                                     # ---- chunked prefill
        pos = c * chunk
        q, k, v = mk(chunk, H, 100 + c), mk(chunk, KVH, 200 + c), mk(chunk, KVH, 300 + c)
        gq, gk, gv = torch.relu(mk(chunk, H, 400 + c)), torch.relu(mk(chunk, KVH, 500 + c)), mk(chunk, KVH, 600 + c)
        gg = (torch.nn.functional.logsigmoid(math.sqrt(D) * mk(chunk, KVH, 700 + c).float()) / 16).bfloat16()
        k_hist[pos:pos + chunk], v_hist[pos:pos + chunk] = k.cpu(), v.cpu()
        for h in heads:
            for dst, src, hh in zip(g_hist[h], (gq, gk, gv, gg), (h, h // 7, h // 7, h // 7)):
                dst[pos:pos + chunk] = src[:, hh:hh + 1].cpu()
        before = account()
        plan.plan(n_new)
        live = account()
        reused += len((live - before) & seen_blocks)
        seen_blocks |= live
        peak = max(peak, len(live))
        md = MetaAttentionMetadata(
            num_prefills=1, num_prefill_tokens=chunk, num_decode_tokens=0, slot_mapping=plan.slot_mapping,
            seq_lens=[pos + chunk], seq_lens_tensor=plan.seq_lens, max_prefill_seq_len=pos + chunk, max_decode_seq_len=0,
            context_lens_tensor=plan.context_lens, block_tables=plan.block_tables, use_cuda_graph=False,
            max_query_len=chunk, query_start_loc=plan.query_start_loc)
        out = torch.empty(chunk, H, D, dtype=torch.bfloat16, device=DEV)
        impl.forward(None, q, k, v, None, None, None, kv_d, md, output=out)
        gla_prefill_scan(gq, gk, gv, gg, gla.cache[0], slot_idx, plan.query_start_loc, plan.context_lens,
                         status=gla_status, max_query_len=chunk, workspace=scan_ws)
        sample = [0, 1, 15, 16, 4095, 4096, 4097, chunk - 1]
        check_rows(out[sample].float().cpu(), q[sample].cpu(), [pos + i for i in sample])
        plan.trim()
        assert len(account()) <= wl // BS + 2, f"chunk {c}: {len(account())} blocks resident after the chunk"
    assert peak <= (wl + chunk) // BS + 3
    assert plan.seq_lens.tolist() == [prompt]
    # the GLA state after 131072 tokens in 16 x 10 sub-chunks against one token-by-token scan
    state = gla.cache[0][int(slot_idx[0])].cpu()
    for h in heads:
        ref_state = torch.zeros(1, 1, D, D)
        ref_ops.gla_scan_ref(*g_hist[h], ref_state, [0, prompt])
        assert rel_err(state[h], ref_state[0, 0]) <= 1e-4, f"GLA head {h}"

    gq1 = [t.view(1, t.shape[1], 1, D) for t in (torch.relu(mk(1, H, 800)), torch.relu(mk(1, KVH, 801)), mk(1, KVH, 802))]
    gg1 = (torch.nn.functional.logsigmoid(torch.randn(1, KVH, 1, D, device=DEV)) / 16).bfloat16()
    for step in range(steps):                                            # ---- decode
        pos = prompt + step
        q, k, v = mk(1, H, 1000 + step), mk(1, KVH, 2000 + step), mk(1, KVH, 3000 + step)
        k_hist[pos], v_hist[pos] = k[0].cpu(), v[0].cpu()
        before = account()
        plan.plan()
        live = account()
        reused += len((live - before) & seen_blocks)
        seen_blocks |= live
        assert len(live) <= wl // BS + 2
        md = MetaAttentionMetadata(
            num_prefills=0, num_prefill_tokens=0, num_decode_tokens=1, slot_mapping=plan.slot_mapping[:1], seq_lens=None,
            seq_lens_tensor=plan.seq_lens, max_prefill_seq_len=0, max_decode_seq_len=pos + 1, context_lens_tensor=None,
            block_tables=plan.block_tables, use_cuda_graph=False, max_query_len=1, max_decode_query_len=1)
        out = torch.empty(1, H, D, dtype=torch.bfloat16, device=DEV)
        impl.forward(None, q, k, v, None, None, None, kv_d, md, output=out)
        my_fused_recurrent_gla(*gq1, gg1, kv_caches=gla.cache[0], slot_idx=slot_idx, status=gla_status)
        if step % 37 == 0 or step == steps - 1:
            check_rows(out.float().cpu(), q.cpu(), [pos])
    assert reused > 0, "retired blocks must come back through the ring"
    assert impl.status() == 0 and plan.status.item() == 0 and gla_status.item() == 0
    snap = plan.snapshot()
    assert len(snap["free"]) + sum(1 for e in snap["table"][0] if e >= 0) == n_blocks      # nothing leaked


def test_gla_state_carried_across_chunks_equals_single_scan(sb):
    """A prompt pushed through the GLA slot cache in chunks (token steps on the device, new
    slots handed out by the manager) leaves the state a single sequential scan leaves."""
    from spikingbrain_7b_b200.gla_slots import GLACacheManager, my_fused_recurrent_gla
    B, T, chunk = 3, 96, 32
    mgr = GLACacheManager(torch.float32, (1, 5, H, D, D), device=DEV)
    g = torch.Generator().manual_seed(41)
    q = torch.relu(torch.randn(B, T, H, D, generator=g) / math.sqrt(D)).bfloat16()
    k = torch.relu(torch.randn(B, T, KVH, D, generator=g) / math.sqrt(D)).bfloat16()
    v = (torch.randn(B, T, KVH, D, generator=g) / math.sqrt(D)).bfloat16()
    gk = (torch.nn.functional.logsigmoid(torch.randn(B, T, KVH, D, generator=g)) / 16).bfloat16()
    ref_state = torch.zeros(B, H, D, D)
    ref_out = [ref_ops.gla_step_ref(q[:, t], k[:, t], v[:, t], gk[:, t], ref_state) for t in range(T)]
    from spikingbrain_7b_b200.gla_slots import gla_prefill_scan
    outs = []
    for c0 in range(0, T, chunk):
        cache, idx = mgr.current_run_tensors({f"req{b}": [0] for b in range(B)})   # same slots every chunk
        if c0 == 0:        # first chunk token by token (the decode op), later chunks as scans
            for t in range(c0, c0 + chunk):
                dv = lambda x: x[:, t].unsqueeze(2).to(DEV)
                outs.append(my_fused_recurrent_gla(dv(q), dv(k), dv(v), dv(gk), kv_caches=cache[0], slot_idx=idx).float().cpu())
        else:
            fl = lambda x: x[:, c0:c0 + chunk].reshape(B * chunk, x.shape[2], D).contiguous().to(DEV)
            qsl = torch.arange(B + 1, dtype=torch.int32, device=DEV) * chunk
            o = gla_prefill_scan(fl(q), fl(k), fl(v), fl(gk), cache[0], idx, qsl,
                                 context_lens=torch.full((B,), c0, dtype=torch.int32, device=DEV))
            outs.extend(o.view(B, chunk, H, D).float().cpu().unbind(1))
    state = mgr.cache[0][idx.cpu()].cpu()
    assert float((state - ref_state).abs().max() / ref_state.abs().max()) <= 1e-4
    for t in (0, 31, 32, 95):
        assert float((outs[t] - ref_out[t].bfloat16().float()).abs().max() / ref_out[t].abs().max()) <= 2 ** -7


def test_churn_over_fragmented_pool_with_head_shards(sb):
    """Zipf-length sequences come and go over a small pool; every step appends one token per live
    sequence and decodes. Checked against the oracle on a CPU shadow of each sequence's history,
    both with all four kv heads on one device and split four ways (one kv head and seven query heads
    per shard, outputs concatenated the way an all-gather of head slices would)."""
    from spikingbrain_7b_b200 import ops
    from spikingbrain_7b_b200.block_pool import SlidingWindowBlockManager
    rng = np.random.default_rng(0)
    R, wl, steps, max_len = 48, 255, 24, 1024
    max_blocks = (max_len + steps) // BS + 2
    nb = R * ((wl // BS) + 3)
    mgr = SlidingWindowBlockManager(nb, BS, wl, R, max_blocks)
    mgr.pool._free = [int(x) for x in rng.permutation(nb)]
    kv = torch.zeros(2, nb, BS, KVH, D, dtype=torch.bfloat16, device=DEV)
    table_d = torch.full((R, max_blocks), -1, dtype=torch.int32, device=DEV)
    g = torch.Generator().manual_seed(42)
    hist = {}

    def new_len():
        return int(np.clip(rng.zipf(1.2) * 16, 16, max_len))

    def admit(row):
        L = new_len()
        mgr.admit(row)
        plan = mgr.advance(np.where(np.arange(R) == row, L, 0), pad_inactive=False)
        kh = (torch.randn(L, KVH, D, generator=g) / math.sqrt(D)).bfloat16()
        vh = (torch.randn(L, KVH, D, generator=g) / math.sqrt(D)).bfloat16()
        hist[row] = [kh, vh]
        ops.kv_append(kh.to(DEV), vh.to(DEV), kv[0], kv[1], torch.from_numpy(plan.slot_mapping).to(DEV))

    for row in range(R - 4):          # four rows stay empty at first
        admit(row)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for step in range(steps):
        active = mgr.active.copy()
        plan = mgr.advance(active.astype(np.int64))
        q = (torch.randn(R, H, D, generator=g) / math.sqrt(D)).bfloat16()
        kn = (torch.randn(R, KVH, D, generator=g) / math.sqrt(D)).bfloat16()
        vn = (torch.randn(R, KVH, D, generator=g) / math.sqrt(D)).bfloat16()
        for row in np.nonzero(active)[0]:
            hist[row][0] = torch.cat([hist[row][0], kn[row:row + 1]])
            hist[row][1] = torch.cat([hist[row][1], vn[row:row + 1]])
        table_d.copy_(torch.from_numpy(mgr.table))
        lens_d = torch.from_numpy(plan.seq_lens).to(DEV)
        ops.kv_append(kn.to(DEV), vn.to(DEV), kv[0], kv[1], torch.from_numpy(plan.slot_mapping).to(DEV), status=status)
        out = ops.swa_decode(q.to(DEV), kv[0], kv[1], table_d, lens_d, window_left=wl, status=status).float().cpu()
        shards = []
        for r in range(KVH):          # head shard r: kv head r, query heads 7r..7r+6, its own slice of the pool
            kv_r = kv[:, :, :, r:r + 1].contiguous()
            shards.append(ops.swa_decode(q[:, 7 * r:7 * r + 7].contiguous().to(DEV), kv_r[0], kv_r[1], table_d, lens_d,
                                         window_left=wl, status=status))
        gathered = torch.cat(shards, dim=1).float().cpu()
        assert not out[~active].any() and not gathered[~active].any()       # empty rows give zero rows
        for row in np.nonzero(active)[0][:: 3 if step % 4 else 1]:
            kh, vh = hist[row]
            tgt = _dense_ref(q[row], kh, vh, kh.shape[0] - 1, wl).bfloat16().float()
            for o in (out[row], gathered[row]):
                assert float((o - tgt).abs().max()) <= 2e-2 and mean_rel(o, tgt) <= 1e-3, f"step {step} row {row}"
        # 5 % of the live sequences finish and fresh ones take free rows
        for row in rng.choice(np.nonzero(mgr.active)[0], size=max(1, int(0.05 * mgr.active.sum())), replace=False):
            mgr.finish(int(row))
            hist.pop(int(row))
        for row in np.nonzero(~mgr.active)[0][:3]:
            admit(int(row))
    assert status.item() == 0
    assert mgr.pool.num_free + int((mgr.table >= 0).sum()) == nb
