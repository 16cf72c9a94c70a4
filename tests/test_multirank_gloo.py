"""CPU, two ranks over gloo: the multi-rank plumbing of bench.py (join, slowest-rank timing,
whole-job throughput) and the independence of the per-rank block managers. Sequences are
sharded across ranks without any data-path collective, so this is all the N>1 logic there is."""
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, {root!r})
    import numpy as np
    import torch
    import torch.distributed as dist
    import bench
    from spikingbrain_7b_b200.block_pool import SlidingWindowBlockManager

    rank, world = bench.dist_setup("gloo")
    assert (rank, world) == (int(os.environ["RANK"]), 2) and dist.get_backend() == "gloo"
    # every rank owns its own sequences, pool and tables: same shapes, different contents
    B, bs, wl = 6, 16, 63
    mgr = SlidingWindowBlockManager(B * 12, bs, wl, B, 40)
    rng = np.random.default_rng(100 + rank)
    mgr.pool._free = [int(x) for x in rng.permutation(B * 12)]
    for r in range(B):
        mgr.admit(r)
    mgr.advance(rng.integers(1, 150, B))
    slots = [mgr.advance(np.ones(B, dtype=np.int64)).slot_mapping for _ in range(40)]
    digest = torch.tensor([int(np.concatenate(slots).sum()), int(mgr.lens.sum()), mgr.pool.num_free])
    gathered = [torch.zeros_like(digest) for _ in range(world)]
    dist.all_gather(gathered, digest)           # test-side only: the data path itself never communicates
    assert gathered[0][0] != gathered[1][0], "ranks must not mirror each other's block assignment"
    for r in range(B):
        assert mgr.resident_blocks(r) <= (wl + 1 + bs - 1) // bs + 1
    # the job's step time is the slowest rank's; throughput adds up over ranks
    ms = bench.max_over_ranks(5.0 + 2.0 * rank, "cpu")
    assert ms == 7.0
    assert bench.job_tokens_per_s(256, world, ms) == 2 * 256 / 7.0e-3
    # head-sharded gather: rank r contributes heads [r*Hl, (r+1)*Hl) of every token
    from spikingbrain_7b_b200.head_shard import all_gather_heads, shard_heads
    full = torch.arange(5 * 8 * 4, dtype=torch.float32).view(5, 8, 4)
    qh, kvh = shard_heads(8, 2, world, rank)
    assert (list(qh), list(kvh)) == ([4 * rank + i for i in range(4)], [rank])
    got = all_gather_heads(full[:, qh.start:qh.stop].contiguous())
    assert torch.equal(got, full)
    dist.barrier()
    if rank == 0:
        print(json.dumps({{"ok": True, "ms": ms}}))
    dist.destroy_process_group()
""")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gloo_ranks_time_and_shard_independently(sb, tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=240) for p in procs]
    for p, (out, err) in zip(procs, outs):
        assert p.returncode == 0, err[-2000:]
    assert '"ok": true' in outs[0][0] and outs[1][0].strip() == ""


def test_reference_arm_runs_on_rank_zero_only(monkeypatch, capsys):
    """Under a multi-rank launch the CPU reference arm is rank 0's job; the others leave quietly."""
    sys.path.insert(0, ROOT)
    import bench
    monkeypatch.setenv("RANK", "1")
    monkeypatch.setenv("WORLD_SIZE", "2")
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--gpus", "2", "--steps", "1"])
    assert bench.run_reference(bench.parse_args()) is None
    assert capsys.readouterr().out == ""


def test_cache_byte_model_matches_the_shapes():
    sys.path.insert(0, ROOT)
    import bench
    total, swa, gla = bench.cache_bytes_per_step([8193] * 256, 14, 14)
    assert swa == 256 * (4097 * 2048 + 2048)            # window of K/V read + one token appended
    assert gla == 256 * 2 * 28 * 128 * 128 * 4          # state read + written
    assert total == 14 * (swa + gla) == 43232788480
    assert bench.cache_bytes_per_step([100, 100], 1, 0)[0] == 2 * (100 * 2048 + 2048)
    assert bench.cache_bytes_per_step([100, 9000], 1, 0)[1] == (100 + 4097) * 2048 + 2 * 2048      # ragged batch


def test_head_shard_rules_follow_the_reference():
    import pytest
    from spikingbrain_7b_b200.head_shard import shard_heads
    assert [list(shard_heads(28, 4, 4, r)[0])[0] for r in range(4)] == [0, 7, 14, 21]
    assert [list(shard_heads(28, 4, 4, r)[1]) for r in range(4)] == [[0], [1], [2], [3]]
    assert list(shard_heads(28, 4, 2, 1)[1]) == [2, 3] and len(shard_heads(28, 4, 2, 1)[0]) == 14
    assert [list(shard_heads(28, 4, 28, r)[1]) for r in (0, 6, 7, 27)] == [[0], [0], [1], [3]]   # kv heads replicated
    with pytest.raises(ValueError):
        shard_heads(28, 4, 8, 0)          # 28 query heads do not split eight ways: the reference rejects it too
    with pytest.raises(ValueError):
        shard_heads(24, 4, 6, 0)


def test_fused_gather_layout_and_peer_addresses():
    """Host side of the fused all-gather: where a writer's head slice and flag land in each peer's
    allocation. A model of the stores (every rank writes its slice to every allocation) must fill
    each gathered row exactly once, in rank order, and touch nothing else."""
    import numpy as np
    import pytest
    from spikingbrain_7b_b200.head_shard import gather_layout, peer_addresses
    T, H, D, tp = 5, 28, 128, 4
    lay = gather_layout(T, H, D, tp)
    assert lay["row_bytes"] == H * D * 2 and lay["slice_bytes"] == 7 * D * 2
    assert lay["buffer_offsets"][1] % 256 == 0 and lay["flag_offset"] == 2 * lay["buffer_bytes"]
    assert lay["total_bytes"] >= lay["flag_offset"] + 4 * tp
    mem = [np.zeros(lay["total_bytes"], dtype=np.uint8) for _ in range(tp)]    # rank p's allocation
    bases = [1 << 20, 3 << 20, 7 << 20, 9 << 20]                                # as mapped by the writer
    for parity in (0, 1):
        for m in mem:
            m[:] = 0
        for r in range(tp):
            outs, flags = peer_addresses(lay, bases, r, parity)
            assert len(outs) == len(flags) == tp - 1
            others = [p for p in range(tp) if p != r]
            # own slice in the own allocation, as the kernel's `out` would address it
            own = lay["buffer_offsets"][parity] + r * lay["slice_bytes"]
            targets = [(r, own)] + [(p, a - bases[p]) for p, a in zip(others, outs)]
            for p, off in targets:
                for t in range(T):
                    o = off + t * lay["row_bytes"]
                    assert not mem[p][o:o + lay["slice_bytes"]].any()             # nobody wrote here before
                    mem[p][o:o + lay["slice_bytes"]] = r + 1
            for p, a in zip(others, flags):
                assert a - bases[p] == lay["flag_offset"] + 4 * r
        for m in mem:
            buf = m[lay["buffer_offsets"][parity]:][:T * lay["row_bytes"]].reshape(T, tp, lay["slice_bytes"])
            assert all((buf[:, r] == r + 1).all() for r in range(tp))
            other = m[lay["buffer_offsets"][1 - parity]:][:T * lay["row_bytes"]]
            assert not other.any()
    with pytest.raises(ValueError):
        gather_layout(T, 28, 128, 8)
    with pytest.raises(ValueError):
        gather_layout(T, 32, 128, 16)


HYBRID_WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, {root!r})
    import torch
    import torch.distributed as dist
    from spikingbrain_7b_b200.head_shard import all_gather_heads, make_hybrid_layout, shard_heads

    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    lay = make_hybrid_layout(2)                     # 4 ranks = 2 sequence groups x 2 head shards
    assert (lay.n_seq_groups, lay.seq_group, lay.tp_rank) == (2, rank // 2, rank % 2)
    seqs = lay.my_sequences(7)
    assert list(seqs) == ([0, 1, 2, 3] if lay.seq_group == 0 else [4, 5, 6])
    # the group's sequences, all 8 heads; a rank computes its 4 heads and gathers inside its group only
    full = torch.arange(7 * 8 * 4, dtype=torch.float32).view(7, 8, 4)[seqs.start:seqs.stop]
    qh, kvh = shard_heads(8, 2, lay.tp_size, lay.tp_rank)
    got = all_gather_heads(full[:, qh.start:qh.stop].contiguous(), group=lay.tp_group)
    assert torch.equal(got, full)
    dist.barrier()
    if rank == 0:
        print(json.dumps({{"ok": True}}))
    dist.destroy_process_group()
""")


def test_hybrid_layout_four_gloo_ranks(sb, tmp_path):
    """Head shards inside a group, sequences across groups: the gather stays inside the group."""
    script = tmp_path / "hybrid_worker.py"
    script.write_text(HYBRID_WORKER.format(root=ROOT))
    port = _free_port()
    procs = []
    for rank in range(4):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="4", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=240) for p in procs]
    for p, (out, err) in zip(procs, outs):
        assert p.returncode == 0, err[-2000:]
    assert '"ok": true' in outs[0][0]


def test_split_sequences_covers_without_overlap():
    from spikingbrain_7b_b200.head_shard import split_sequences
    for n, g in ((1024, 2), (7, 3), (2, 4), (0, 2)):
        parts = [split_sequences(n, g, i) for i in range(g)]
        assert [x for p in parts for x in p] == list(range(n))
        assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
