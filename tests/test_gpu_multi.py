"""GPU, several ranks (one process per GPU): the head-sharded decode step. Each rank holds its share
of the kv heads (its slice of the paged K/V pool) and of the query heads (its slice of the GLA state),
runs the same kernels on its slice, and the head outputs are gathered on every rank -- by NCCL, or by
the kernels themselves through peer stores. Two ranks split 28/4 heads as 14/2, four ranks as 7/1
(the split the churn configuration names); eight GPUs run as 4 head shards x 2 sequence groups.
Every test is skipped on a box with fewer GPUs than it needs."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, math, json
    sys.path.insert(0, {root!r})
    import torch
    import torch.distributed as dist
    from oracle import ref_ops
    from tests.helpers import make_paged_kv, mean_rel, rel_err
    from spikingbrain_7b_b200 import ops
    from spikingbrain_7b_b200.head_shard import all_gather_heads, shard_heads

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    H, KVH, D, bs, wl = 28, 4, 128, 16, 1023
    lens = [1500, 17, 1024, 1025, 300, 64]
    B = len(lens)
    # the same global problem on every rank (seeded), of which a rank keeps its head slice
    kv, table, nb = make_paged_kv(lens, wl, KVH, D, bs, seed=50)
    g = torch.Generator().manual_seed(51)
    q = (torch.randn(B, H, D, generator=g) / math.sqrt(D)).bfloat16()
    gq = torch.relu(torch.randn(B, H, D, generator=g) / math.sqrt(D)).bfloat16()
    gk = torch.relu(torch.randn(B, KVH, D, generator=g) / math.sqrt(D)).bfloat16()
    gv = (torch.randn(B, KVH, D, generator=g) / math.sqrt(D)).bfloat16()
    gg = (torch.nn.functional.logsigmoid(torch.randn(B, KVH, D, generator=g)) / 16).bfloat16()
    state = torch.randn(B, H, D, D, generator=g)
    qh, kh = shard_heads(H, KVH, world, rank)
    kv_l = kv[:, :, :, kh.start:kh.stop].contiguous().to(dev)        # [2, NB, bs, kvh/tp, D]
    lens_d = torch.tensor(lens, dtype=torch.int32, device=dev)
    o_l = ops.swa_decode(q[:, qh.start:qh.stop].contiguous().to(dev), kv_l[0], kv_l[1], table.to(dev), lens_d,
                         window_left=wl)
    o = all_gather_heads(o_l)
    state_l = state[:, qh.start:qh.stop].contiguous().to(dev)
    go_l = ops.gla_step(gq[:, qh.start:qh.stop].contiguous().to(dev), gk[:, kh.start:kh.stop].contiguous().to(dev),
                        gv[:, kh.start:kh.stop].contiguous().to(dev), gg[:, kh.start:kh.stop].contiguous().to(dev),
                        state_l, out_dtype=torch.float32)
    go = all_gather_heads(go_l)
    torch.cuda.synchronize()
    ref = ref_ops.swa_paged_decode_ref(q, kv[0], kv[1], table, lens, wl, D ** -0.5).bfloat16().float()
    ref_state = state.clone()
    gref = ref_ops.gla_step_ref(gq, gk, gv, gg, ref_state)
    a = o.float().cpu()
    assert a.shape == (B, H, D)
    assert float((a - ref).abs().max()) <= 2e-2 and mean_rel(a, ref) <= 1e-3      # every rank holds all heads
    assert rel_err(go.cpu(), gref) <= 1e-4
    assert rel_err(state_l.cpu(), ref_state[:, qh.start:qh.stop]) <= 1e-4
    dist.barrier()
    if rank == 0:
        print(json.dumps({{"ok": True}}))
    dist.destroy_process_group()
""")


def _run_ranks(n_ranks, script_text, tmp_path, name, extra_env=None):
    """One child process per rank on GPUs 0 .. n_ranks-1; every one must exit 0."""
    if torch.cuda.device_count() < n_ranks:
        pytest.skip(f"needs {n_ranks} GPUs")
    script = tmp_path / name
    script.write_text(script_text)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for rank in range(n_ranks):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(n_ranks),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=600) for p in procs]
    for p, (out, err) in zip(procs, outs):
        assert p.returncode == 0, err[-3000:]
    return outs


@pytest.mark.parametrize("n_ranks", [2, 4])
def test_head_sharded_decode_nccl(sb, tmp_path, n_ranks):
    outs = _run_ranks(n_ranks, WORKER.format(root=ROOT), tmp_path, "worker.py")
    assert '"ok": true' in outs[0][0]


FUSED_WORKER = textwrap.dedent("""
    import os, sys, math, json
    sys.path.insert(0, {root!r})
    import torch
    import datetime
    import torch.distributed as dist
    from oracle import ref_ops
    from tests.helpers import make_paged_kv, mean_rel
    from spikingbrain_7b_b200 import ops
    from spikingbrain_7b_b200.head_shard import FusedHeadGather, all_gather_heads, shard_heads

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # a rank that fails an assertion must not keep the other one waiting in a collective for long
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    H, KVH, D, bs, wl = 28, 4, 128, 16, 1023
    lens = [1500, 17, 1024, 1025, 300, 64, 0, 5000]
    B = len(lens)
    kv, table, nb = make_paged_kv(lens, wl, KVH, D, bs, seed=52)
    qh, kh = shard_heads(H, KVH, world, rank)
    kv_l = kv[:, :, :, kh.start:kh.stop].contiguous().to(dev)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=dev)
    table_d = table.to(dev)
    fg = FusedHeadGather(16, H, D, device=dev, timeout_ms=5000)
    g = torch.Generator().manual_seed(53)
    for step in range(4):                                   # both buffers, twice
        q = (torch.randn(B, H, D, generator=g) / math.sqrt(D)).bfloat16()
        q_l = q[:, qh.start:qh.stop].contiguous().to(dev)
        o = fg.decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl)
        got = o.clone()
        o_nccl = all_gather_heads(ops.swa_decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl))
        torch.cuda.synchronize()
        assert fg.status.item() == 0, fg.status.item()
        assert torch.equal(got, o_nccl)                     # the same rows, delivered by stores
        ref = ref_ops.swa_paged_decode_ref(q, kv[0], kv[1], table, lens, wl, D ** -0.5).bfloat16().float()
        a = got.float().cpu()
        assert float((a - ref).abs().max()) <= 2e-2 and mean_rel(a, ref) <= 1e-3
    # the GLA layer's head outputs the same way (odd number of calls so far or not: the buffers alternate)
    gq = torch.randn(B, H, D, generator=g).bfloat16()
    gk, gv = torch.randn(B, KVH, D, generator=g).bfloat16(), torch.randn(B, KVH, D, generator=g).bfloat16()
    gg = (3 * torch.randn(B, KVH, D, generator=g)).bfloat16()
    gw = (1 + 0.3 * torch.randn(D, generator=g)).bfloat16().to(dev)
    gstate = torch.randn(B, H, D, D, generator=g)
    fused_kw = dict(relu_qk=True, gate_logit_normalizer=16.0, norm_weight=gw, norm_eps=1e-5)
    loc = [t[:, hs.start:hs.stop].contiguous().to(dev) for t, hs in ((gq, qh), (gk, kh), (gv, kh), (gg, kh))]
    s_a = gstate[:, qh.start:qh.stop].contiguous().to(dev)
    s_b = s_a.clone()
    for step in range(3):
        og = fg.gla_step(*loc, s_a, **fused_kw).clone()
        o_nccl_g = all_gather_heads(ops.gla_step(*loc, s_b, out_dtype=torch.bfloat16, **fused_kw))
        torch.cuda.synchronize()
        assert fg.status.item() == 0
        assert torch.equal(og, o_nccl_g) and torch.equal(s_a, s_b)
    if fg.calls & 1:
        fg.decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl)
    # device time of the two ways to get [B, H, D] on every rank (CUDA events, a few repeats)
    def timed(fn, n=20):
        for _ in range(3):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    t_fused = timed(lambda: fg.decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl))
    t_nccl = timed(lambda: all_gather_heads(ops.swa_decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl)))
    assert fg.status.item() == 0
    # the same pair of calls replayed from a CUDA graph: nothing in them depends on a host-side step number
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ws = ops.swa_workspace(B, len(qh), D, ops.swa_max_pieces(wl + 1, ops.swa_auto_split(B, wl + 1, dev), B, dev), dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            o0 = fg.decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl, workspace=ws)
            keep0 = o0.clone()
            o1 = fg.decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl, workspace=ws)
            keep1 = o1.clone()
    torch.cuda.current_stream().wait_stream(side)
    dist.barrier(); torch.cuda.synchronize()
    for _ in range(5):
        keep0.zero_(); keep1.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert fg.status.item() == 0
        assert torch.equal(keep0, o_nccl) and torch.equal(keep1, o_nccl)
    t_graph = timed(graph.replay) / 2
    fg.close()
    dist.barrier()
    if rank == 0:
        print(json.dumps({{"ok": True, "fused_ms": t_fused, "nccl_ms": t_nccl, "fused_graph_ms": t_graph}}))
    dist.destroy_process_group()
""")


@pytest.mark.parametrize("n_ranks", [2, 4])
def test_fused_head_gather(sb, tmp_path, n_ranks):
    """One process per GPU: the decode kernel (and the GLA step) stores each rank's head slice into
    every other rank's buffer through NVLink and raises its flag there; the result equals the
    collective's bit for bit and the oracle within the attention / GLA bars. Four ranks: 7 query
    heads and 1 kv head per rank, three peers per rank."""
    outs = _run_ranks(n_ranks, FUSED_WORKER.format(root=ROOT), tmp_path, "fused_worker.py")
    assert '"ok": true' in outs[0][0]
    print(outs[0][0].strip().splitlines()[-1])


HYBRID_WORKER = textwrap.dedent("""
    import os, sys, math, json, datetime
    sys.path.insert(0, {root!r})
    import torch
    import torch.distributed as dist
    from oracle import ref_ops
    from tests.helpers import make_paged_kv, mean_rel, rel_err
    from spikingbrain_7b_b200 import ops
    from spikingbrain_7b_b200.head_shard import FusedHeadGather, all_gather_heads, make_hybrid_layout, shard_heads

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    tp = {tp}
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    lay = make_hybrid_layout(tp)
    assert lay.n_seq_groups == world // tp and lay.tp_rank == rank % tp and lay.seq_group == rank // tp
    H, KVH, D, bs, wl = 28, 4, 128, 16, 1023
    all_lens = [1500, 17, 1024, 1025, 300, 64, 0, 5000, 33, 2048, 700]
    kv, table, nb = make_paged_kv(all_lens, wl, KVH, D, bs, seed=56)          # the same global problem everywhere
    mine = lay.my_sequences(len(all_lens))                                   # this group's sequences ...
    qh, kh = shard_heads(H, KVH, tp, lay.tp_rank)                            # ... and this rank's heads
    lens = all_lens[mine.start:mine.stop]
    B = len(lens)
    kv_l = kv[:, :, :, kh.start:kh.stop].contiguous().to(dev)
    table_d = table[mine.start:mine.stop].contiguous().to(dev)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=dev)
    fg = FusedHeadGather(16, H, D, group=lay.tp_group, device=dev, timeout_ms=5000)
    g = torch.Generator().manual_seed(57)
    for step in range(4):
        q = (torch.randn(len(all_lens), H, D, generator=g) / math.sqrt(D)).bfloat16()
        q_l = q[mine.start:mine.stop, qh.start:qh.stop].contiguous().to(dev)
        got = fg.decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl).clone()
        want = all_gather_heads(ops.swa_decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl),
                                group=lay.tp_group)
        torch.cuda.synchronize()
        assert fg.status.item() == 0, fg.status.item()
        assert got.shape == (B, H, D) and torch.equal(got, want)             # gathered inside the group only
        ref = ref_ops.swa_paged_decode_ref(q[mine.start:mine.stop], kv[0], kv[1], table[mine.start:mine.stop], lens,
                                           wl, D ** -0.5).bfloat16().float()
        a = got.float().cpu()
        assert float((a - ref).abs().max()) <= 2e-2 and mean_rel(a, ref) <= 1e-3
    gq = torch.relu(torch.randn(len(all_lens), H, D, generator=g) / math.sqrt(D)).bfloat16()
    gk = torch.relu(torch.randn(len(all_lens), KVH, D, generator=g) / math.sqrt(D)).bfloat16()
    gv = (torch.randn(len(all_lens), KVH, D, generator=g) / math.sqrt(D)).bfloat16()
    gg = (torch.nn.functional.logsigmoid(torch.randn(len(all_lens), KVH, D, generator=g)) / 16).bfloat16()
    gstate = torch.randn(len(all_lens), H, D, D, generator=g)
    sl = lambda t, hs: t[mine.start:mine.stop, hs.start:hs.stop].contiguous().to(dev)
    s_l = sl(gstate, qh)
    og = fg.gla_step(sl(gq, qh), sl(gk, kh), sl(gv, kh), sl(gg, kh), s_l).clone()
    torch.cuda.synchronize()
    assert fg.status.item() == 0
    ref_state = gstate[mine.start:mine.stop].clone()
    gref = ref_ops.gla_step_ref(gq[mine.start:mine.stop], gk[mine.start:mine.stop], gv[mine.start:mine.stop],
                                gg[mine.start:mine.stop], ref_state)
    assert float((og.float().cpu() - gref.bfloat16().float()).abs().max()) <= 2e-2 * float(gref.abs().max())
    assert rel_err(s_l.cpu(), ref_state[:, qh.start:qh.stop]) <= 1e-4
    if fg.calls & 1:
        fg.gla_step(sl(gq, qh), sl(gk, kh), sl(gv, kh), sl(gg, kh), s_l)
    fg.close()
    dist.barrier()
    if rank == 0:
        print(json.dumps({{"ok": True, "groups": lay.n_seq_groups, "tp": tp}}))
    dist.destroy_process_group()
""")


@pytest.mark.parametrize("n_ranks,tp", [(4, 2), (8, 4)])
def test_hybrid_layout_head_shards_times_sequence_groups(sb, tmp_path, n_ranks, tp):
    """n_ranks GPUs as n_ranks/tp sequence groups of tp head shards (eight GPUs: 4 x 2, because 28
    heads do not split eight ways): every group decodes its own sequences, the fused gather and the
    collective run inside a group only, and each rank ends up with all 28 heads of its group's
    sequences -- bit-equal between the two gathers and within the bars of the oracle."""
    outs = _run_ranks(n_ranks, HYBRID_WORKER.format(root=ROOT, tp=tp), tmp_path, "hybrid_worker.py")
    assert '"ok": true' in outs[0][0]


MISSED_STEP_WORKER = textwrap.dedent("""
    import os, sys, math, json, datetime, time
    sys.path.insert(0, {root!r})
    import torch
    import torch.distributed as dist
    from tests.helpers import make_paged_kv
    from spikingbrain_7b_b200 import _abi, ops
    from spikingbrain_7b_b200.head_shard import FusedHeadGather, all_gather_heads, shard_heads

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    H, KVH, D, bs, wl = 28, 4, 128, 16, 255
    lens = [300, 17, 64]
    B = len(lens)
    kv, table, nb = make_paged_kv(lens, wl, KVH, D, bs, seed=54)
    qh, kh = shard_heads(H, KVH, world, rank)
    kv_l = kv[:, :, :, kh.start:kh.stop].contiguous().to(dev)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=dev)
    table_d = table.to(dev)
    g = torch.Generator().manual_seed(55)
    q = (torch.randn(B, H, D, generator=g) / math.sqrt(D)).bfloat16()
    q_l = q[:, qh.start:qh.stop].contiguous().to(dev)
    want = all_gather_heads(ops.swa_decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl)).clone()
    fg = FusedHeadGather(8, H, D, device=dev, timeout_ms=300)
    def step():
        o = fg.decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl).clone()
        torch.cuda.synchronize()
        return o
    assert torch.equal(step(), want) and fg.status.item() == 0
    dist.barrier()
    # the last rank sits the next step out (between steps, nothing of its own in flight): the others'
    # wait runs out after 300 ms, says so in the status word and returns; the context stays usable
    if rank != world - 1:
        t0 = time.time()
        step()
        assert fg.status.item() == _abi.ST_WAIT_TIMEOUT
        assert 0.25 <= time.time() - t0 <= 10.0
        assert int((lens_d + 1).sum().item()) == sum(lens) + B
    fg.resync()                                  # both ranks: counters, flags and buffer turn back to the start
    assert fg.status.item() == 0
    for _ in range(3):
        assert torch.equal(step(), want) and fg.status.item() == 0
    fg.close()
    dist.barrier()
    if rank == 0:
        print(json.dumps({{"ok": True}}))
    dist.destroy_process_group()
""")


@pytest.mark.parametrize("n_ranks", [2, 4])
def test_fused_head_gather_missed_step_is_reported_and_recovered(sb, tmp_path, n_ranks):
    """A peer that does not take a step (the last rank sits it out): the bounded flag wait of every
    other rank reports it (no hang, no fault), and after a host-side resync the gather works again."""
    # in-switch reduction off in the collective library for a test in which a rank falls out of step
    outs = _run_ranks(n_ranks, MISSED_STEP_WORKER.format(root=ROOT), tmp_path, "missed_step_worker.py",
                      extra_env={"NCCL_NVLS_ENABLE": "0"})
    assert '"ok": true' in outs[0][0]
