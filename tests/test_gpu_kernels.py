"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle."""
import math

import pytest
import torch

from oracle import ref_ops
from tests.helpers import make_paged_kv, mean_rel, rel_err

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
# bf16 attention: max-abs 2e-2 and mean-rel 1e-3 against the fp32 oracle rounded to the
# output dtype; fp32 GLA state and output: rel 1e-4 of the largest magnitude.
ATTN_MAX_ABS, ATTN_MEAN_REL = 2e-2, 1e-3
GLA_REL = 1e-4


@pytest.fixture(scope="module")
def ops(sb):
    from spikingbrain_7b_b200 import ops as _ops
    assert torch.cuda.is_available()
    return _ops


def _status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ append / retire / gather
@pytest.mark.parametrize("dtype,kvh,D,bs", [(torch.bfloat16, 4, 128, 16), (torch.float32, 2, 64, 16),
                                           (torch.bfloat16, 1, 128, 64)])
def test_kv_append_bit_exact(ops, dtype, kvh, D, bs):
    g = torch.Generator().manual_seed(1)
    nb, T = 37, 53
    kc = torch.randn(nb, bs, kvh, D, generator=g).to(dtype)
    vc = torch.randn(nb, bs, kvh, D, generator=g).to(dtype)
    key = torch.randn(T, kvh, D, generator=g).to(dtype)
    val = torch.randn(T, kvh, D, generator=g).to(dtype)
    slots = torch.randperm(nb * bs, generator=g)[:T].to(torch.int64)
    slots[::7] = -1  # padding tokens are skipped
    kc_ref, vc_ref = kc.clone(), vc.clone()
    ref_ops.paged_append(key, val, kc_ref, vc_ref, slots)
    kc_d, vc_d = kc.to(DEV), vc.to(DEV)
    st = _status()
    ops.kv_append(key.to(DEV), val.to(DEV), kc_d, vc_d, slots.to(DEV), status=st)
    assert st.item() == 0
    assert torch.equal(kc_d.cpu().view(torch.uint8), kc_ref.view(torch.uint8))
    assert torch.equal(vc_d.cpu().view(torch.uint8), vc_ref.view(torch.uint8))


def test_kv_append_strided_views_and_bad_slot(ops):
    """key/value as column slices of a fused qkv row (the layout the attention layer hands
    over), caches as the two halves of one [2, NB, bs, kvh, D] tensor; an out-of-pool slot
    raises the status bit and writes nothing."""
    g = torch.Generator().manual_seed(2)
    kvh, D, bs, nb, T, H = 4, 128, 16, 9, 5, 28
    qkv = torch.randn(T, (H + 2 * kvh) * D, generator=g).bfloat16().to(DEV)
    key = qkv[:, H * D:(H + kvh) * D].view(T, kvh, D)
    val = qkv[:, (H + kvh) * D:].view(T, kvh, D)
    kv = torch.zeros(2, nb, bs, kvh, D, dtype=torch.bfloat16, device=DEV)
    slots = torch.tensor([3, 17, nb * bs, 40, 41], dtype=torch.int64)
    st = _status()
    ops.kv_append(key, val, kv[0], kv[1], slots.to(DEV), status=st)
    assert st.item() == 1  # SBK_ST_BAD_SLOT
    kc_ref = torch.zeros(nb, bs, kvh, D, dtype=torch.bfloat16)
    vc_ref = torch.zeros_like(kc_ref)
    good = slots.clone(); good[2] = -1
    ref_ops.paged_append(key.cpu(), val.cpu(), kc_ref, vc_ref, good)
    assert torch.equal(kv[0].cpu(), kc_ref) and torch.equal(kv[1].cpu(), vc_ref)


@pytest.mark.parametrize("bs", [16, 32])
def test_retire_matches_oracle_over_steps(ops, bs):
    """Decode steps that move the window across block edges: the device table edits and the
    retired ids equal the oracle's, step by step."""
    B, wl, steps = 5, 40, 70
    lens = [1, 15, 41, 64, 100]
    max_blocks = (max(lens) + steps + bs - 1) // bs
    table = torch.arange(B * max_blocks, dtype=torch.int32).view(B, max_blocks).contiguous()
    table_d = table.to(DEV)
    kvh, D = 1, 128
    kv = torch.zeros(2, B * max_blocks, bs, kvh, D, dtype=torch.bfloat16, device=DEV)
    st = _status()
    for step in range(steps):
        lens = [L + 1 for L in lens]
        slots = torch.tensor([int(table[b, (L - 1) // bs]) * bs + (L - 1) % bs if table[b, (L - 1) // bs] >= 0 else -1
                              for b, L in enumerate(lens)], dtype=torch.int64)
        exp = ref_ops.retire_blocks(table, lens, [1] * B, wl, bs)
        retired = torch.full((B, 4), -7, dtype=torch.int32, device=DEV)
        kx = torch.zeros(B, kvh, D, dtype=torch.bfloat16, device=DEV)
        ops.kv_append(kx, kx, kv[0], kv[1], slots.to(DEV), block_tables=table_d,
                      seq_lens=torch.tensor(lens, dtype=torch.int32, device=DEV), window_left=wl,
                      retired_out=retired, status=st)
        assert torch.equal(table_d.cpu(), table), f"step {step}"
        got = [[x for x in row if x >= 0] for row in retired.cpu().tolist()]
        assert got == exp, f"step {step}"
    assert st.item() == 0


def test_retire_multi_token_and_overflow(ops):
    """A chunk of new tokens per sequence (query_start_loc given): the window edge is taken
    from the chunk's first query; too few retired_out columns raise the overflow bit but
    the table is still edited."""
    bs, wl = 16, 32
    lens = [200, 90]
    n_new = [64, 8]
    max_blocks = 16
    table = torch.arange(2 * max_blocks, dtype=torch.int32).view(2, max_blocks).contiguous()
    exp_table = table.clone()
    exp = ref_ops.retire_blocks(exp_table, lens, n_new, wl, bs)
    assert len(exp[0]) > 2
    table_d = table.to(DEV)
    retired = torch.full((2, 2), -7, dtype=torch.int32, device=DEV)
    st = _status()
    kv = torch.zeros(2, 2, bs, 1, 128, dtype=torch.bfloat16, device=DEV)
    empty = torch.zeros(0, 1, 128, dtype=torch.bfloat16, device=DEV)
    ops.kv_append(empty, empty, kv[0], kv[1], torch.zeros(0, dtype=torch.int64, device=DEV),
                  block_tables=table_d, seq_lens=torch.tensor(lens, dtype=torch.int32, device=DEV),
                  query_start_loc=torch.tensor([0, 64, 72], dtype=torch.int32, device=DEV),
                  window_left=wl, retired_out=retired, status=st)
    assert torch.equal(table_d.cpu(), exp_table)
    assert st.item() == 8  # SBK_ST_RETIRE_OVERFLOW
    assert retired.cpu().tolist()[0] == exp[0][:2]


@pytest.mark.parametrize("dtype,kvh,D", [(torch.bfloat16, 4, 128), (torch.float32, 2, 64)])
def test_kv_gather_bit_exact(ops, dtype, kvh, D):
    bs, wl = 16, 63
    lens = [1, 16, 17, 64, 65, 200, 333]
    kv, table, nb = make_paged_kv(lens, wl, kvh, D, bs, dtype=dtype, seed=3)
    n_out = max(min(L, wl + 1) for L in lens)
    st = _status()
    k_out, v_out = ops.kv_gather(kv[0].to(DEV), kv[1].to(DEV), table.to(DEV),
                                 torch.tensor(lens, dtype=torch.int32, device=DEV), n_out,
                                 window_left=wl, status=st)
    assert st.item() == 0
    for b, L in enumerate(lens):
        k_ref, v_ref = ref_ops.window_gather(kv[0], kv[1], table[b], L, wl)
        n = k_ref.shape[1]
        assert torch.equal(k_out[b, :, :n].cpu(), k_ref) and torch.equal(v_out[b, :, :n].cpu(), v_ref)
        assert not k_out[b, :, n:].any() and not v_out[b, :, n:].any()


# ------------------------------------------------------------------------------ attention
def _run_attn(ops, lens, wl, H, kvh, bs, seed, out_dtype=torch.bfloat16, split_chunks=32, max_pieces=None,
              full_retention=False):
    D = 128
    kv, table, nb = make_paged_kv(lens, wl, kvh, D, bs, seed=seed, full_retention=full_retention)
    g = torch.Generator().manual_seed(seed + 100)
    q = (torch.randn(len(lens), H, D, generator=g) / math.sqrt(D)).bfloat16()
    scale = D ** -0.5
    ref, lse_ref = ref_ops.swa_paged_decode_ref(q, kv[0], kv[1], table, lens, wl, scale, return_lse=True)
    st = _status()
    lse = torch.empty(len(lens), H, dtype=torch.float32, device=DEV)
    kv_d = kv.to(DEV)
    out = ops.swa_decode(q.to(DEV), kv_d[0], kv_d[1], table.to(DEV),
                         torch.tensor(lens, dtype=torch.int32, device=DEV), window_left=wl,
                         scale=scale, out_dtype=out_dtype, lse=lse, split_chunks=split_chunks,
                         max_pieces=max_pieces, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    return out.cpu(), ref, lse.cpu(), lse_ref


def _check_attn(out, ref, lse, lse_ref):
    assert torch.isfinite(out.float()).all()
    tgt = ref.to(out.dtype).float()
    assert float((out.float() - tgt).abs().max()) <= ATTN_MAX_ABS
    assert mean_rel(out.float(), tgt) <= ATTN_MEAN_REL
    fin = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(lse), fin)
    assert float((lse[fin] - lse_ref[fin]).abs().max()) <= 1e-3


@pytest.mark.parametrize("lens", [[1], [16], [17], [15, 31, 33], [64, 65, 66, 127, 128, 129]])
def test_swa_decode_small_edges(ops, lens):
    out, ref, lse, lse_ref = _run_attn(ops, lens, wl=63, H=28, kvh=4, bs=16, seed=5)
    _check_attn(out, ref, lse, lse_ref)


@pytest.mark.parametrize("wl", [0, 1, 15, 16, 17, 4095, 4096, -1])
def test_swa_decode_window_edges(ops, wl):
    lens = [5000, 4097, 4096, 4095, 33, 1]
    out, ref, lse, lse_ref = _run_attn(ops, lens, wl=wl, H=28, kvh=4, bs=16, seed=6)
    _check_attn(out, ref, lse, lse_ref)


@pytest.mark.parametrize("H,kvh", [(7, 1), (14, 2), (28, 4), (32, 4), (4, 4), (16, 2), (1, 1)])
def test_swa_decode_head_layouts(ops, H, kvh):
    lens = [700, 129, 4100]
    out, ref, lse, lse_ref = _run_attn(ops, lens, wl=2047, H=H, kvh=kvh, bs=16, seed=7)
    _check_attn(out, ref, lse, lse_ref)


@pytest.mark.parametrize("bs", [16, 32, 64, 128])
def test_swa_decode_block_sizes_full_retention(ops, bs):
    lens = [3000, 777, 64, 2049]
    out, ref, lse, lse_ref = _run_attn(ops, lens, wl=1024, H=28, kvh=4, bs=bs, seed=8, full_retention=True)
    _check_attn(out, ref, lse, lse_ref)


@pytest.mark.parametrize("split_chunks,max_pieces", [(1, 300), (3, 7), (32, 1), (1000, 4)])
def test_swa_decode_split_settings(ops, split_chunks, max_pieces):
    lens = [4100, 513, 40, 2000]
    out, ref, lse, lse_ref = _run_attn(ops, lens, wl=4096, H=28, kvh=4, bs=16, seed=9,
                                      split_chunks=split_chunks, max_pieces=max_pieces)
    _check_attn(out, ref, lse, lse_ref)


@pytest.mark.parametrize("split_chunks,max_pieces", [(-1, 2), (-1, 300), (-4, 3), (-8, None), (-1000, 2), (-3, 1)])
def test_swa_decode_balanced_runs(ops, split_chunks, max_pieces):
    """Balanced mode: equal runs of chunks per CTA that cross sequence boundaries; the bound on
    pieces per sequence is honoured whatever it is (max_pieces 1 falls back to whole sequences)."""
    lens = [4100, 513, 40, 2000, 0, 1, 16, 8193, 333]
    out, ref, lse, lse_ref = _run_attn(ops, lens, wl=4096, H=28, kvh=4, bs=16, seed=13,
                                      split_chunks=split_chunks, max_pieces=max_pieces)
    _check_attn(out, ref, lse, lse_ref)


@pytest.mark.parametrize("lens,H,kvh", [([8193], 28, 4), ([8193, 5000, 4097], 28, 4), ([8193], 7, 1), ([6000, 8193], 14, 2)])
def test_swa_decode_few_long_sequences_share_their_fold(ops, lens, H, kvh):
    """Few sequences per launch are cut into many pieces (33 at one sequence); their fold goes head by
    head and is shared out over the CTAs that hold the pieces, which wait for one another (cooperative
    launch). Against the oracle, launch after launch on one workspace (the piece counters must come
    back to zero), with the log-sum-exp, and against the ticket mode's result."""
    D, bs, wl = 128, 16, 4096
    kv, table, nb = make_paged_kv(lens, wl, kvh, D, bs, seed=91)
    g = torch.Generator().manual_seed(92)
    q = (torch.randn(len(lens), H, D, generator=g) / math.sqrt(D)).bfloat16()
    ref, lse_ref = ref_ops.swa_paged_decode_ref(q, kv[0], kv[1], table, lens, wl, D ** -0.5, return_lse=True)
    kv_d, q_d, table_d = kv.to(DEV), q.to(DEV), table.to(DEV)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=DEV)
    v = min(table.shape[1] * bs, wl + 1)
    split = ops.swa_auto_split(len(lens), v, torch.device(DEV))
    mp = ops.swa_max_pieces(v, split)
    assert split < 0 and 2 * (mp - 1) >= H          # balanced, and enough pieces for the head-by-head form
    ws = ops.swa_workspace(len(lens), H, D, mp, DEV)
    st = _status()
    outs = []
    for _ in range(4):
        lse = torch.empty(len(lens), H, dtype=torch.float32, device=DEV)
        outs.append(ops.swa_decode(q_d, kv_d[0], kv_d[1], table_d, lens_d, window_left=wl, lse=lse, workspace=ws,
                                   max_pieces=mp, split_chunks=split, status=st))
        torch.cuda.synchronize()
        assert st.item() == 0
        _check_attn(outs[-1].cpu(), ref, lse.cpu(), lse_ref)
        assert torch.equal(outs[-1], outs[0])
    head = ws[:32 + 4 * ((len(lens) + 3) // 4 * 4)].view(torch.int32)
    assert not head.any()                            # tickets, counters and the stale mark are back at zero
    ticket = ops.swa_decode(q_d, kv_d[0], kv_d[1], table_d, lens_d, window_left=wl, split_chunks=8, max_pieces=mp, status=st)
    assert st.item() == 0
    assert float((ticket.float() - outs[0].float()).abs().max()) <= 2.0 ** -7 * float(outs[0].float().abs().max())


@pytest.mark.parametrize("H,kvh", [(7, 1), (14, 2), (28, 4)])
def test_swa_decode_balanced_head_layouts_and_many_sequences(ops, H, kvh):
    """More sequences than CTAs, lengths from 0 to a few windows, every kv-head layout (stages of
    1, 2 and 4 sub-chunks): runs start and end in the middle of stages."""
    g = torch.Generator().manual_seed(14)
    lens = torch.randint(0, 700, (400,), generator=g).tolist()
    out, ref, lse, lse_ref = _run_attn(ops, lens, wl=255, H=H, kvh=kvh, bs=16, seed=15, split_chunks=-2)
    _check_attn(out, ref, lse, lse_ref)


def test_swa_decode_balanced_uniform_batch_takes_whole_sequences(ops):
    """Near-equal lengths filling half the CTAs or more: the kernel streams whole sequences
    (no partials); same numbers either way."""
    lens = [600 + (i % 5) for i in range(300)]
    out, ref, lse, lse_ref = _run_attn(ops, lens, wl=511, H=28, kvh=4, bs=16, seed=16, split_chunks=-8)
    _check_attn(out, ref, lse, lse_ref)


def test_swa_decode_fp32_out_tight(ops):
    """With fp32 output the only bf16 rounding left is that of the probabilities."""
    lens = [4100, 900, 77]
    out, ref, lse, lse_ref = _run_attn(ops, lens, wl=4096, H=28, kvh=4, bs=16, seed=10, out_dtype=torch.float32)
    assert rel_err(out, ref) <= 2e-3
    assert mean_rel(out, ref) <= ATTN_MEAN_REL


def test_swa_decode_empty_and_bad_block(ops):
    """seq_len 0 yields a zero row; a table entry outside the pool inside the window raises
    the status bit, and every output stays finite."""
    D, H, kvh, bs, wl = 128, 28, 4, 16, 63
    lens = [0, 100, 50]
    kv, table, nb = make_paged_kv([1, 100, 50], wl, kvh, D, bs, seed=11)
    table[2, 50 // bs] = nb + 5
    q = torch.randn(3, H, D).bfloat16()
    st = _status()
    kv_d = kv.to(DEV)
    out = ops.swa_decode(q.to(DEV), kv_d[0], kv_d[1], table.to(DEV),
                         torch.tensor(lens, dtype=torch.int32, device=DEV), window_left=wl, status=st)
    torch.cuda.synchronize()
    assert st.item() == 2  # SBK_ST_BAD_BLOCK
    assert not out[0].any() and torch.isfinite(out.float()).all()
    ref = ref_ops.swa_paged_decode_ref(q[1:2], kv[0], kv[1], table[1:2], [100], wl, D ** -0.5)
    assert float((out[1].float().cpu() - ref[0]).abs().max()) <= ATTN_MAX_ABS


def test_swa_decode_config2_shapes(ops):
    """The single-step op test: 28/4 heads, D 128, window 4096, batch 64, context lengths
    uniform in [1k, 32k], block 16, permuted block table, q/k/v ~ N(0,1)/sqrt(128)."""
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(1024, 32769, (64,), generator=g).tolist()
    out, ref, lse, lse_ref = _run_attn(ops, lens, wl=4096, H=28, kvh=4, bs=16, seed=12)
    _check_attn(out, ref, lse, lse_ref)


def _big_paged_case(lens, wl, H, kvh, bs, seed):
    """A large paged pool built on the device (every visible block of every sequence, random block
    order, -1 for blocks before the window) -> (q, kv, table, lens tensor) on the GPU."""
    D = 128
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    first = [max(0, L - 1 - wl) // bs if wl >= 0 else 0 for L in lens]
    last = [(L - 1) // bs for L in lens]
    n_live = [l - f + 1 for f, l in zip(first, last)]
    nb = sum(n_live) + 5
    perm = torch.randperm(nb, generator=g).to(torch.int32)
    table = torch.full((B, max(last) + 1), -1, dtype=torch.int32)
    o = 0
    for b in range(B):
        table[b, first[b]:last[b] + 1] = perm[o:o + n_live[b]]
        o += n_live[b]
    torch.manual_seed(seed)
    kv = (torch.randn(2, nb, bs, kvh, D, device=DEV, dtype=torch.bfloat16) / math.sqrt(D))
    q = (torch.randn(B, H, D, device=DEV) / math.sqrt(D)).bfloat16()
    return q, kv, table.to(DEV), torch.tensor(lens, dtype=torch.int32, device=DEV)


def test_swa_decode_benchmarked_geometry_b256_ctx8192(ops):
    """The shape the decode benchmark times: 256 sequences at 8192 tokens, window_left 4096 (4097 visible
    keys), block 16, 28/4 heads, default split -- the whole-sequence partition with one CTA per
    sequence. Every output row against the oracle."""
    H, kvh, bs, wl, D = 28, 4, 16, 4096, 128
    lens = [8192] * 256
    q, kv, table, lens_d = _big_paged_case(lens, wl, H, kvh, bs, seed=40)
    st = _status()
    lse = torch.empty(len(lens), H, dtype=torch.float32, device=DEV)
    out = ops.swa_decode(q, kv[0], kv[1], table, lens_d, window_left=wl, lse=lse, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    kv_c = kv.cpu()
    ref, lse_ref = ref_ops.swa_paged_decode_ref(q.cpu(), kv_c[0], kv_c[1], table.cpu(), lens, wl, D ** -0.5,
                                                return_lse=True)
    _check_attn(out.cpu(), ref, lse.cpu(), lse_ref)


def test_swa_decode_churn_lengths_b1024_default_split(ops):
    """The churn workload's batch: 1024 sequences (the most one launch takes), lengths
    clip(zipf(1.2), 128, 65536) drawn with numpy's default_rng(0), window_left 4096, default split
    (the balanced partition: equal runs of chunks per CTA across sequence boundaries)."""
    import numpy as np
    H, kvh, bs, wl, D = 28, 4, 16, 4096, 128
    lens = np.clip(np.random.default_rng(0).zipf(1.2, size=1024), 128, 65536).astype(int).tolist()
    q, kv, table, lens_d = _big_paged_case(lens, wl, H, kvh, bs, seed=41)
    st = _status()
    lse = torch.empty(len(lens), H, dtype=torch.float32, device=DEV)
    out = ops.swa_decode(q, kv[0], kv[1], table, lens_d, window_left=wl, lse=lse, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    kv_c = kv.cpu()
    ref, lse_ref = ref_ops.swa_paged_decode_ref(q.cpu(), kv_c[0], kv_c[1], table.cpu(), lens, wl, D ** -0.5,
                                                return_lse=True)
    _check_attn(out.cpu(), ref, lse.cpu(), lse_ref)


def test_swa_decode_more_sequences_than_one_launch_default_split(ops):
    """1500 short sequences: two launches (1024 + 476) sharing one workspace, balanced partition."""
    g = torch.Generator().manual_seed(42)
    lens = torch.randint(1, 400, (1500,), generator=g).tolist()
    out, ref, lse, lse_ref = _run_attn(ops, lens, wl=255, H=28, kvh=4, bs=16, seed=43, split_chunks=None)
    _check_attn(out, ref, lse, lse_ref)


@pytest.mark.parametrize("split", [-8, 4])
def test_swa_decode_marked_workspace_reports_instead_of_computing(ops, split):
    """A call in which a wait ran out leaves its counters where they stood and marks the workspace
    (word 4 of its head). A later call given that workspace must not fold stale partials into
    rows it reports as good: it raises SBK_ST_WAIT_TIMEOUT again and writes nothing. Once the head
    is zeroed the workspace serves again. The mark is planted by hand here (no wait is made to
    run out), together with stale counters."""
    from spikingbrain_7b_b200 import _abi
    H, kvh, bs, wl, D = 28, 4, 16, 1023, 128
    lens = [1500, 17, 1024, 1025, 300, 64]
    kv, table, nb = make_paged_kv(lens, wl, kvh, D, bs, seed=44)
    q = (torch.randn(len(lens), H, D, generator=torch.Generator().manual_seed(45)) / math.sqrt(D)).bfloat16()
    ref = ref_ops.swa_paged_decode_ref(q, kv[0], kv[1], table, lens, wl, D ** -0.5)
    pieces = 9
    ws = ops.swa_workspace(len(lens), H, D, pieces, DEV)
    head = ws[:32 + 4 * 8].view(torch.int32)
    head[0] = 3          # a ticket counter that was never rewound
    head[4] = 1          # the mark
    head[8:14] = 2       # completion counters of sequences that were half done
    kv_d = kv.to(DEV)
    args = (q.to(DEV), kv_d[0], kv_d[1], table.to(DEV), torch.tensor(lens, dtype=torch.int32, device=DEV))
    st = _status()
    out = torch.full((len(lens), H, D), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.swa_decode(*args, window_left=wl, out=out, workspace=ws, max_pieces=pieces, split_chunks=split, status=st)
    torch.cuda.synchronize()
    assert st.item() == _abi.ST_WAIT_TIMEOUT
    assert bool((out == 7.0).all()), "a marked workspace must not produce rows"
    ws[:head.numel() * 4].zero_()
    st.zero_()
    ops.swa_decode(*args, window_left=wl, out=out, workspace=ws, max_pieces=pieces, split_chunks=split, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    tgt = ref.bfloat16().float()
    assert float((out.float().cpu() - tgt).abs().max()) <= ATTN_MAX_ABS and mean_rel(out.float().cpu(), tgt) <= ATTN_MEAN_REL
    assert not head.any(), "a clean call leaves the head of the workspace at zero"


@pytest.mark.parametrize("H,kvh,n_meta", [(28, 4, 128), (7, 1, 16), (14, 2, 48)])
def test_swa_decode_with_sink_tokens(ops, H, kvh, n_meta):
    """Meta (sink) tokens every query sees besides its window: one softmax over both."""
    D, bs, wl = 128, 16, 511
    lens = [1, 40, 512, 513, 2000, 0]
    kv, table, nb = make_paged_kv([max(L, 1) for L in lens], wl, kvh, D, bs, seed=70)
    g = torch.Generator().manual_seed(71)
    q = (torch.randn(len(lens), H, D, generator=g) / math.sqrt(D)).bfloat16()
    k2 = (torch.randn(n_meta, kvh, D, generator=g) / math.sqrt(D)).bfloat16()
    v2 = (torch.randn(n_meta, kvh, D, generator=g) / math.sqrt(D)).bfloat16()
    ref, lse_ref = ref_ops.swa_paged_decode_ref(q, kv[0], kv[1], table, lens, wl, D ** -0.5, return_lse=True,
                                                key2=k2, value2=v2)
    st = _status()
    kv_d = kv.to(DEV)
    lse = torch.empty(len(lens), H, dtype=torch.float32, device=DEV)
    for split in (None, 4, -1):
        out = ops.swa_decode(q.to(DEV), kv_d[0], kv_d[1], table.to(DEV), torch.tensor(lens, dtype=torch.int32, device=DEV),
                             window_left=wl, lse=lse, split_chunks=split, key2=k2.to(DEV), value2=v2.to(DEV), status=st)
        torch.cuda.synchronize()
        assert st.item() == 0
        _check_attn(out.cpu(), ref, lse.cpu(), lse_ref)


def test_swa_prefill_with_sink_tokens(ops, prefill_kernel):
    D, H, kvh, bs, wl, n_meta = 128, 28, 4, 16, 63, 128
    ctx, new = [0, 90], [50, 33]
    total = [c + n for c, n in zip(ctx, new)]
    kv, table, nb = make_paged_kv(total, -1, kvh, D, bs, seed=72)
    g = torch.Generator().manual_seed(73)
    q = (torch.randn(sum(new), H, D, generator=g) / math.sqrt(D)).bfloat16()
    k2 = (torch.randn(n_meta, kvh, D, generator=g) / math.sqrt(D)).bfloat16()
    v2 = (torch.randn(n_meta, kvh, D, generator=g) / math.sqrt(D)).bfloat16()
    kv_d = kv.to(DEV)
    st = _status()
    out = ops.swa_prefill(q.to(DEV), kv_d[0], kv_d[1], table.to(DEV), torch.tensor([0, 50, 83], dtype=torch.int32, device=DEV),
                          torch.tensor(ctx, dtype=torch.int32, device=DEV), 50, window_left=wl, key2=k2.to(DEV),
                          value2=v2.to(DEV), kernel=prefill_kernel, status=st).float().cpu()
    assert st.item() == 0
    row = 0
    for s in range(2):
        for i in range(new[s]):
            ref = ref_ops.swa_paged_decode_ref(q[row][None], kv[0], kv[1], table[s:s + 1], [ctx[s] + i + 1], wl, D ** -0.5,
                                               key2=k2, value2=v2)[0].bfloat16().float()
            assert float((out[row] - ref).abs().max()) <= ATTN_MAX_ABS and mean_rel(out[row], ref) <= 2 * ATTN_MEAN_REL
            row += 1


# --------------------------------------------------------------------- prefill attention
def _prefill_case(ops, ctx, new, wl, H, kvh, bs, seed, kernel="auto"):
    """Sequences with `ctx[s]` cached tokens get `new[s]` more: append, then windowed attention of
    the new tokens; the oracle treats every new token as a one-token decode at its position."""
    D = 128
    B = len(ctx)
    total = [c + n for c, n in zip(ctx, new)]
    kv, table, nb = make_paged_kv(total, -1, kvh, D, bs, seed=seed)       # every token resident
    g = torch.Generator().manual_seed(seed + 1)
    T = sum(new)
    q = (torch.randn(T, H, D, generator=g) / math.sqrt(D)).bfloat16()
    qsl = [0]
    for n in new:
        qsl.append(qsl[-1] + n)
    st = _status()
    kv_d = kv.to(DEV)
    out = ops.swa_prefill(q.to(DEV), kv_d[0], kv_d[1], table.to(DEV), torch.tensor(qsl, dtype=torch.int32, device=DEV),
                          torch.tensor(ctx, dtype=torch.int32, device=DEV), max(new), window_left=wl, kernel=kernel, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    o = out.float().cpu()
    assert torch.isfinite(o).all()
    worst, num, den = 0.0, 0.0, 0.0
    rng = torch.Generator().manual_seed(seed + 2)
    for s in range(B):
        picks = sorted(set([0, 1, 15, 16, 17, new[s] - 1] + torch.randint(0, new[s], (12,), generator=rng).tolist()))
        for i in [p for p in picks if 0 <= p < new[s]]:
            pos = ctx[s] + i
            ref = ref_ops.swa_paged_decode_ref(q[qsl[s] + i][None], kv[0], kv[1], table[s:s + 1], [pos + 1], wl,
                                               D ** -0.5)[0].bfloat16().float()
            d = (o[qsl[s] + i] - ref).abs()
            worst = max(worst, float(d.max())); num += float(d.sum()); den += float(ref.abs().sum())
    assert worst <= ATTN_MAX_ABS and num / den <= ATTN_MEAN_REL, (worst, num / den)


@pytest.fixture(params=["tcgen05", "tcgen05_pair", "mma_sync"])
def prefill_kernel(request):
    """The prefill entry point has three kernels, chosen by its `kernel` argument: tcgen05 with one
    query tile per CTA, tcgen05 with two tiles taking turns (between them what "auto" takes for aligned
    q / out) and mma.sync."""
    return request.param


@pytest.mark.parametrize("ctx,new", [([0], [1]), ([0], [16]), ([0], [17]), ([5], [40]), ([0, 100, 33], [70, 3, 129])])
def test_swa_prefill_small_edges(ops, prefill_kernel, ctx, new):
    _prefill_case(ops, ctx, new, wl=63, H=28, kvh=4, bs=16, seed=60, kernel=prefill_kernel)


@pytest.mark.parametrize("wl", [0, 15, 16, 255, 4096, -1])
def test_swa_prefill_window_edges(ops, prefill_kernel, wl):
    _prefill_case(ops, [300, 0, 1000], [200, 513, 64], wl=wl, H=28, kvh=4, bs=16, seed=61, kernel=prefill_kernel)


@pytest.mark.parametrize("H,kvh,bs", [(7, 1, 16), (14, 2, 32), (32, 4, 64), (4, 4, 16), (16, 2, 128)])
def test_swa_prefill_head_layouts_and_block_sizes(ops, prefill_kernel, H, kvh, bs):
    _prefill_case(ops, [700, 0], [300, 260], wl=511, H=H, kvh=kvh, bs=bs, seed=62, kernel=prefill_kernel)


def test_swa_prefill_long_chunk_at_model_shapes(ops, prefill_kernel):
    """One 2048-token chunk on top of 6000 cached tokens, window 4096, 28/4 heads."""
    _prefill_case(ops, [6000], [2048], wl=4096, H=28, kvh=4, bs=16, seed=63, kernel=prefill_kernel)


def _set_token(kv, table, s, i, bs, k=None, v=None):
    pb = int(table[s, i // bs])
    if k is not None:
        kv[0, pb, i % bs] = k
    if v is not None:
        kv[1, pb, i % bs] = v


def test_swa_prefill_scores_that_keep_growing_move_the_offset(ops, prefill_kernel):
    """Keys whose scores rise by about 13 (log2 units) per 128-key tile: the softmax offset, which the
    tcgen05 kernels move only when a row's maximum outgrows it by 2^8, moves on every tile, and the
    output accumulated so far is rescaled in tensor memory each time. (Random keys never do this after
    a row's first tile.)"""
    D, H, kvh, bs, wl = 128, 28, 4, 16, 1023
    ctx, new = [900], [400]
    kv, table, nb = make_paged_kv([1300], -1, kvh, D, bs, seed=81)
    g = torch.Generator().manual_seed(82)
    u = torch.randn(D, generator=g)
    u = u / u.norm()
    for i in range(1300):
        k = (0.07 * i * math.sqrt(D) / 8) * u + 0.05 * torch.randn(kvh, D, generator=g)
        _set_token(kv, table, 0, i, bs, k=k.bfloat16())
    q = (8 * u + 0.3 * torch.randn(400, H, D, generator=g)).bfloat16()
    st = _status()
    kv_d = kv.to(DEV)
    out = ops.swa_prefill(q.to(DEV), kv_d[0], kv_d[1], table.to(DEV), torch.tensor([0, 400], dtype=torch.int32, device=DEV),
                          torch.tensor(ctx, dtype=torch.int32, device=DEV), 400, window_left=wl, kernel=prefill_kernel,
                          status=st).float().cpu()
    assert st.item() == 0 and torch.isfinite(out).all()
    num = den = worst = 0.0
    for i in (0, 1, 17, 18, 35, 36, 127, 200, 399):
        ref = ref_ops.swa_paged_decode_ref(q[i][None], kv[0], kv[1], table[0:1], [900 + i + 1], wl, D ** -0.5)[0]
        d = (out[i] - ref.bfloat16().float()).abs()
        worst = max(worst, float(d.max())); num += float(d.sum()); den += float(ref.abs().sum())
    assert worst <= ATTN_MAX_ABS and num / den <= ATTN_MEAN_REL, (worst, num / den)


def test_swa_prefill_bad_block_is_reported_and_contained(ops, prefill_kernel):
    """A block-table entry outside the pool inside one sequence's window: the kernels raise
    SBK_ST_BAD_BLOCK, skip the keys of that tile (nothing is read through the bad id), keep every output
    finite, and the other sequence's rows are untouched by it."""
    from spikingbrain_7b_b200 import _abi
    D, H, kvh, bs, wl = 128, 28, 4, 16, 511
    ctx, new = [600, 300], [200, 150]
    kv, table, nb = make_paged_kv([800, 450], -1, kvh, D, bs, seed=85)
    g = torch.Generator().manual_seed(86)
    q = (torch.randn(350, H, D, generator=g) / math.sqrt(D)).bfloat16()
    bad = table.clone()
    bad[0, 500 // bs] = nb + 3                       # inside the window of every new token of sequence 0
    st = _status()
    kv_d = kv.to(DEV)
    out = ops.swa_prefill(q.to(DEV), kv_d[0], kv_d[1], bad.to(DEV), torch.tensor([0, 200, 350], dtype=torch.int32, device=DEV),
                          torch.tensor(ctx, dtype=torch.int32, device=DEV), 200, window_left=wl, kernel=prefill_kernel,
                          status=st).float().cpu()
    assert st.item() == _abi.ST_BAD_BLOCK
    assert torch.isfinite(out).all()
    for i in (0, 17, 18, 36, 149):
        ref = ref_ops.swa_paged_decode_ref(q[200 + i][None], kv[0], kv[1], table[1:2], [300 + i + 1], wl, D ** -0.5)[0]
        ref = ref.bfloat16().float()
        assert float((out[200 + i] - ref).abs().max()) <= ATTN_MAX_ABS and mean_rel(out[200 + i], ref) <= ATTN_MEAN_REL


def test_swa_prefill_value_range_of_the_two_tile_kernel(ops):
    """The two-tile tcgen05 kernel multiplies P and V in fp16. Values up to fp16's largest magnitude
    go through it unharmed; one beyond raises SBK_ST_VALUE_RANGE there, and the one-tile kernel (bf16
    throughout) serves the same cache with status 0."""
    from spikingbrain_7b_b200 import _abi
    D, H, kvh, bs, wl = 128, 28, 4, 16, 255
    kv, table, nb = make_paged_kv([500], -1, kvh, D, bs, seed=83)
    g = torch.Generator().manual_seed(84)
    q = (torch.randn(200, H, D, generator=g) / math.sqrt(D)).bfloat16()
    big = (torch.randn(kvh, D, generator=g) * 2.0e4).clamp(-6.0e4, 6.0e4).bfloat16()     # inside fp16 range
    _set_token(kv, table, 0, 350, bs, v=big)
    args = lambda kvt: (q.to(DEV), kvt[0], kvt[1], table.to(DEV), torch.tensor([0, 200], dtype=torch.int32, device=DEV),
                        torch.tensor([300], dtype=torch.int32, device=DEV), 200)

    def check(out):
        for i in (0, 49, 50, 51, 120, 199):
            ref = ref_ops.swa_paged_decode_ref(q[i][None], kv[0], kv[1], table[0:1], [300 + i + 1], wl, D ** -0.5)[0]
            ref = ref.bfloat16().float()
            assert mean_rel(out[i], ref) <= ATTN_MEAN_REL and float((out[i] - ref).abs().max()) <= 2.0 ** -7 * float(ref.abs().max())

    st = _status()
    out = ops.swa_prefill(*args(kv.to(DEV)), window_left=wl, kernel="tcgen05_pair", status=st).float().cpu()
    assert st.item() == 0
    check(out)
    over = torch.zeros(kvh, D)
    over[1, 5] = 1.0e5
    _set_token(kv, table, 0, 360, bs, v=over.bfloat16())
    st = _status()
    ops.swa_prefill(*args(kv.to(DEV)), window_left=wl, kernel="tcgen05_pair", status=st)
    assert st.item() == _abi.ST_VALUE_RANGE
    st = _status()
    out = ops.swa_prefill(*args(kv.to(DEV)), window_left=wl, kernel="tcgen05", status=st).float().cpu()
    assert st.item() == 0
    check(out)


@pytest.mark.parametrize("wl,n_meta", [(63, 0), (-1, 0), (300, 48), (0, 0)])
def test_swa_prefill_dense_matches_oracle(ops, wl, n_meta):
    """K/V as tensors instead of a paged cache: ragged sequences, more keys than queries in some
    (the queries are the tail), keys and values as strided column slices, optional sink keys."""
    H, kvh, D = 28, 4, 128
    n_k = [300, 16, 1, 129, 77]
    n_q = [300, 5, 1, 129, 20]
    ksl, qsl = [0], [0]
    for a, b in zip(n_k, n_q):
        ksl.append(ksl[-1] + a); qsl.append(qsl[-1] + b)
    g = torch.Generator().manual_seed(66)
    q = (torch.randn(qsl[-1], H, D, generator=g) / math.sqrt(D)).bfloat16()
    kvbuf = (torch.randn(ksl[-1], 2 * kvh * D + 64, generator=g) / math.sqrt(D)).bfloat16()
    key = kvbuf[:, :kvh * D].view(-1, kvh, D)
    value = kvbuf[:, kvh * D:2 * kvh * D].view(-1, kvh, D)
    k2 = (torch.randn(n_meta, kvh, D, generator=g) / math.sqrt(D)).bfloat16() if n_meta else None
    v2 = (torch.randn(n_meta, kvh, D, generator=g) / math.sqrt(D)).bfloat16() if n_meta else None
    want = ref_ops.swa_prefill_dense_ref(q, key, value, qsl, ksl, wl, D ** -0.5, k2, v2).bfloat16().float()
    kvd = kvbuf.to(DEV)
    st = _status()
    out = ops.swa_prefill_dense(q.to(DEV), kvd[:, :kvh * D].view(-1, kvh, D), kvd[:, kvh * D:2 * kvh * D].view(-1, kvh, D),
                                torch.tensor(qsl, dtype=torch.int32, device=DEV),
                                torch.tensor(ksl, dtype=torch.int32, device=DEV), max(n_q), window_left=wl,
                                key2=None if k2 is None else k2.to(DEV), value2=None if v2 is None else v2.to(DEV),
                                status=st)
    assert st.item() == 0
    o = out.float().cpu()
    assert torch.isfinite(o).all()
    assert float((o - want).abs().max()) <= ATTN_MAX_ABS and mean_rel(o, want) <= ATTN_MEAN_REL


def test_swa_prefill_unaligned_views_take_the_vector_free_kernel(ops):
    """q and out as views whose rows start 4 bytes off a 16-byte boundary: the tcgen05 kernel moves
    them as 16-byte vectors, so the entry point must fall back to the mma.sync kernel by itself."""
    D, H, kvh, bs, wl = 128, 28, 4, 16, 63
    ctx, new = [40], [50]
    kv, table, nb = make_paged_kv([90], -1, kvh, D, bs, seed=64)
    g = torch.Generator().manual_seed(65)
    q = (torch.randn(50, H, D, generator=g) / math.sqrt(D)).bfloat16()
    qbuf = torch.zeros(50 * H * D + 2, dtype=torch.bfloat16, device=DEV)
    obuf = torch.zeros_like(qbuf)
    qv, ov = qbuf[2:].view(50, H, D), obuf[2:].view(50, H, D)
    qv.copy_(q)
    assert qv.data_ptr() % 16 == 4
    kv_d = kv.to(DEV)
    st = _status()
    ops.swa_prefill(qv, kv_d[0], kv_d[1], table.to(DEV), torch.tensor([0, 50], dtype=torch.int32, device=DEV),
                    torch.tensor(ctx, dtype=torch.int32, device=DEV), 50, window_left=wl, out=ov, status=st)
    assert st.item() == 0
    for i in (0, 17, 49):
        ref = ref_ops.swa_paged_decode_ref(q[i][None], kv[0], kv[1], table, [41 + i], wl, D ** -0.5)[0].bfloat16().float()
        assert float((ov[i].float().cpu() - ref).abs().max()) <= ATTN_MAX_ABS


# ------------------------------------------------------------------------------------ GLA
def _gla_inputs(B, H, Hkv, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.relu(torch.randn(B, H, D, generator=g) / math.sqrt(D)).to(dtype)
    k = torch.relu(torch.randn(B, Hkv, D, generator=g) / math.sqrt(D)).to(dtype)
    v = (torch.randn(B, Hkv, D, generator=g) / math.sqrt(D)).to(dtype)
    gk = (torch.nn.functional.logsigmoid(torch.randn(B, Hkv, D, generator=g)) / 16).to(dtype)
    return q, k, v, gk, g


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,H,Hkv,D", [(3, 28, 4, 128), (2, 28, 28, 128), (2, 8, 2, 64), (5, 7, 1, 128)])
def test_gla_step_matches_oracle(ops, dtype, B, H, Hkv, D):
    q, k, v, gk, g = _gla_inputs(B, H, Hkv, D, dtype, seed=20)
    slots = B + 3
    state = torch.randn(slots, H, D, D, generator=g)
    slot_idx = torch.randperm(slots, generator=g)[:B].to(torch.int64)
    slot_idx[0] = -1
    ref_state = state.clone()
    ref_out = ref_ops.gla_step_ref(q, k, v, gk, ref_state, slot_idx)
    state_d = state.to(DEV)
    out = torch.full((B, H, D), 123.0, dtype=torch.float32, device=DEV)
    st = _status()
    ops.gla_step(q.to(DEV), k.to(DEV), v.to(DEV), gk.to(DEV), state_d, slot_idx.to(DEV), out=out, status=st)
    assert st.item() == 0
    assert rel_err(state_d.cpu(), ref_state) <= GLA_REL
    assert rel_err(out[1:].cpu(), ref_out[1:]) <= GLA_REL
    assert (out[0] == 123.0).all()  # slot -1: output row not written
    untouched = [s for s in range(slots) if s not in slot_idx.tolist()]
    assert torch.equal(state_d[untouched].cpu(), state[untouched])  # bit-exact: never touched


def test_gla_step_carry_and_bf16_out(ops):
    """32 chained steps carry the state; bf16 output equals the oracle output to one bf16 ulp."""
    B, H, Hkv, D = 4, 28, 4, 128
    g = torch.Generator().manual_seed(21)
    state = torch.zeros(B, H, D, D)
    state_d = state.to(DEV)
    for step in range(32):
        q, k, v, gk, _ = _gla_inputs(B, H, Hkv, D, torch.bfloat16, seed=100 + step)
        ref_out = ref_ops.gla_step_ref(q, k, v, gk, state)
        out = ops.gla_step(q.to(DEV), k.to(DEV), v.to(DEV), gk.to(DEV), state_d)
        assert out.dtype == torch.bfloat16
        diff = (out.float().cpu() - ref_out.bfloat16().float()).abs()
        assert float((diff / ref_out.abs().clamp_min(1e-6)).max()) <= 2 ** -7
    assert rel_err(state_d.cpu(), state) <= GLA_REL


def test_gla_step_config2_shapes(ops):
    """Batch 64, 28 heads, fp32 state [64, 28, 128, 128] ~ N(0,1), g = logsigmoid(N(0,1))/16."""
    B, H, Hkv, D = 64, 28, 4, 128
    q, k, v, gk, g = _gla_inputs(B, H, Hkv, D, torch.bfloat16, seed=0)
    state = torch.randn(B, H, D, D, generator=g)
    ref_state = state.clone()
    ref_out = ref_ops.gla_step_ref(q, k, v, gk, ref_state)
    state_d = state.to(DEV)
    out = ops.gla_step(q.to(DEV), k.to(DEV), v.to(DEV), gk.to(DEV), state_d, out_dtype=torch.float32)
    assert rel_err(state_d.cpu(), ref_state) <= GLA_REL
    assert rel_err(out.cpu(), ref_out) <= GLA_REL


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("H,Hkv,D", [(28, 4, 128), (8, 2, 64), (7, 7, 128)])
def test_gla_scan_matches_oracle_on_ragged_runs(ops, dtype, H, Hkv, D):
    """Several sequences of different lengths (one empty, one with slot -1, one restarted from
    zero) scanned in one launch: outputs and final states equal the token-by-token oracle."""
    runs = [5, 0, 37, 1, 64, 9]
    qsl = [0]
    for n in runs:
        qsl.append(qsl[-1] + n)
    T, n_seqs = qsl[-1], len(runs)
    g = torch.Generator().manual_seed(30)
    q = torch.relu(torch.randn(T, H, D, generator=g) / math.sqrt(D)).to(dtype)
    k = torch.relu(torch.randn(T, Hkv, D, generator=g) / math.sqrt(D)).to(dtype)
    v = (torch.randn(T, Hkv, D, generator=g) / math.sqrt(D)).to(dtype)
    gk = (torch.nn.functional.logsigmoid(torch.randn(T, Hkv, D, generator=g)) / 16).to(dtype)
    slots = n_seqs + 2
    state = torch.randn(slots, H, D, D, generator=g)
    slot_idx = torch.randperm(slots, generator=g)[:n_seqs].to(torch.int64)
    slot_idx[3] = -1
    reset = [False, False, True, False, False, True]
    ref_state = state.clone()
    ref = ref_ops.gla_scan_ref(q, k, v, gk, ref_state, qsl, slot_idx.tolist(), reset)
    state_d = state.to(DEV)
    st = _status()
    out = ops.gla_scan(q.to(DEV), k.to(DEV), v.to(DEV), gk.to(DEV), state_d,
                       torch.tensor(qsl, dtype=torch.int32, device=DEV), slot_idx.to(DEV),
                       torch.tensor(reset, device=DEV), out_dtype=torch.float32, status=st)
    assert st.item() == 0
    live = torch.ones(T, dtype=torch.bool)
    live[qsl[3]:qsl[4]] = False
    assert rel_err(out.cpu()[live], ref[live]) <= GLA_REL
    assert rel_err(state_d.cpu(), ref_state) <= GLA_REL
    untouched = [s for s in range(slots) if s not in slot_idx.tolist()] + [int(slot_idx[1])]
    assert torch.equal(state_d[untouched].cpu(), state[untouched])


def test_gla_scan_long_runs_at_model_shapes(ops):
    """Eight sequences of 512 tokens at the model's shapes (28/4 heads, head dim 128, bf16 inputs) with a
    carried-in state: 64 rounds of eight tokens per (sequence, head) against the token-by-token oracle."""
    H, Hkv, D, n_seqs, n = 28, 4, 128, 8, 512
    T = n_seqs * n
    qsl = [i * n for i in range(n_seqs + 1)]
    g = torch.Generator().manual_seed(33)
    q = torch.relu(torch.randn(T, H, D, generator=g) / math.sqrt(D)).bfloat16()
    k = torch.relu(torch.randn(T, Hkv, D, generator=g) / math.sqrt(D)).bfloat16()
    v = (torch.randn(T, Hkv, D, generator=g) / math.sqrt(D)).bfloat16()
    gk = (torch.nn.functional.logsigmoid(torch.randn(T, Hkv, D, generator=g)) / 16).bfloat16()
    state = torch.randn(n_seqs, H, D, D, generator=g) * 0.1
    ref_state = state.clone()
    ref = ref_ops.gla_scan_ref(q, k, v, gk, ref_state, qsl)
    state_d = state.to(DEV)
    st = _status()
    out = ops.gla_scan(q.to(DEV), k.to(DEV), v.to(DEV), gk.to(DEV), state_d,
                       torch.tensor(qsl, dtype=torch.int32, device=DEV), out_dtype=torch.float32, status=st)
    assert st.item() == 0
    assert rel_err(out.cpu(), ref) <= GLA_REL
    assert rel_err(state_d.cpu(), ref_state) <= GLA_REL


def test_gla_scan_equals_chained_steps_and_chunking_is_invisible(ops):
    """One scan over 48 tokens == three scans over 16 == 48 single-token steps of sbk_gla_step."""
    B, T, H, Hkv, D = 2, 48, 28, 4, 128
    g = torch.Generator().manual_seed(31)
    mk = lambda h, relu=False: ((torch.relu if relu else (lambda x: x))(torch.randn(B, T, h, D, generator=g) / math.sqrt(D))).bfloat16().to(DEV)
    q, k, v = mk(H, True), mk(Hkv, True), mk(Hkv)
    gk = (torch.nn.functional.logsigmoid(torch.randn(B, T, Hkv, D, generator=g)) / 16).bfloat16().to(DEV)
    flat = lambda t: t.reshape(B * T, t.shape[2], D)
    s_all = torch.zeros(B, H, D, D, device=DEV)
    o_all = ops.gla_scan(flat(q), flat(k), flat(v), flat(gk), s_all,
                         torch.tensor([0, T, 2 * T], dtype=torch.int32, device=DEV), out_dtype=torch.float32)
    s_chunks = torch.zeros_like(s_all)
    s_steps = torch.zeros_like(s_all)
    o_chunks, o_steps = [], []
    for c in range(0, T, 16):
        sl = lambda t: t[:, c:c + 16].reshape(B * 16, t.shape[2], D).contiguous()
        o_chunks.append(ops.gla_scan(sl(q), sl(k), sl(v), sl(gk), s_chunks,
                                     torch.tensor([0, 16, 32], dtype=torch.int32, device=DEV),
                                     out_dtype=torch.float32).view(B, 16, H, D))
    for t in range(T):
        o_steps.append(ops.gla_step(q[:, t].contiguous(), k[:, t].contiguous(), v[:, t].contiguous(),
                                    gk[:, t].contiguous(), s_steps, out_dtype=torch.float32))
    o_all = o_all.view(B, T, H, D)
    assert torch.equal(torch.cat(o_chunks, 1), o_all) and torch.equal(s_chunks, s_all)      # same arithmetic, same bits
    assert rel_err(torch.stack(o_steps, 1), o_all) <= 1e-6 and rel_err(s_steps, s_all) <= 1e-6


def _scan_inputs(T, H, Hkv, D, seed, dtype=torch.bfloat16, strong_decay=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.relu(torch.randn(T, H, D, generator=g) / math.sqrt(D)).to(dtype)
    k = torch.relu(torch.randn(T, Hkv, D, generator=g) / math.sqrt(D)).to(dtype)
    v = (torch.randn(T, Hkv, D, generator=g) / math.sqrt(D)).to(dtype)
    gk = torch.nn.functional.logsigmoid(torch.randn(T, Hkv, D, generator=g)) / (0.05 if strong_decay else 16)
    return q, k, v, gk.to(dtype)


@pytest.mark.parametrize("runs,H,Hkv,D,carry_in,dtype", [
    ([8192], 28, 4, 128, True, torch.bfloat16), ([8192], 28, 4, 128, False, torch.bfloat16),
    ([3000, 700, 2049], 28, 4, 128, True, torch.bfloat16), ([1537, 1024], 7, 1, 128, True, torch.bfloat16),
    ([130, 4000, 1, 257], 14, 2, 128, True, torch.bfloat16),
    ([8192], 28, 4, 128, True, torch.float32), ([4096], 8, 2, 64, True, torch.bfloat16),
    ([2049, 3000], 7, 7, 128, False, torch.float32)])
def test_gla_scan_long_runs_chunked_forms_match_one_chain_and_oracle(ops, runs, H, Hkv, D, carry_in, dtype):
    """Long runs: given the longest run and a workspace the scan leaves the one-chain, token-by-token
    form. bf16 tokens at head dim 128 go through the chunked form on the tensor cores (128-token
    chunks, split-bf16 operands); other inputs, when the runs are few, are cut into sub-chunks owned by
    different CTAs (local scans, carry, scan proper). Either way the recurrence is linear in the state
    and the result is the one-chain scan's in another association: outputs and final states within 1e-5
    of it (tolerance, not bit equality), and within the 1e-4 bar of the token-by-token oracle on two
    sampled heads."""
    n_seqs = len(runs)
    qsl = [0]
    for n in runs:
        qsl.append(qsl[-1] + n)
    T = qsl[-1]
    q, k, v, gk = _scan_inputs(T, H, Hkv, D, seed=35, dtype=dtype)
    g = torch.Generator().manual_seed(36)
    state = torch.randn(n_seqs + 1, H, D, D, generator=g) * 0.1
    slot_idx = torch.arange(n_seqs, 0, -1, dtype=torch.int64)             # slots n_seqs .. 1; slot 0 stays untouched
    reset = [not carry_in] + [False] * (n_seqs - 1)
    ws = ops.gla_scan_workspace(n_seqs, max(runs), H, D, DEV)
    assert ws is not None, "this shape is meant to leave the one-chain form"
    dev = lambda t: t.to(DEV)
    qsl_d = torch.tensor(qsl, dtype=torch.int32, device=DEV)
    reset_d = torch.tensor(reset, device=DEV)
    s_one, s_par = dev(state), dev(state)
    st = _status()
    o_one = ops.gla_scan(dev(q), dev(k), dev(v), dev(gk), s_one, qsl_d, dev(slot_idx), reset_d,
                         out_dtype=torch.float32, status=st)
    ws.fill_(0xFF)                                                        # the scratch needs no initialisation (NaNs)
    o_par = ops.gla_scan(dev(q), dev(k), dev(v), dev(gk), s_par, qsl_d, dev(slot_idx), reset_d,
                         out_dtype=torch.float32, max_query_len=max(runs), workspace=ws, status=st)
    torch.cuda.synchronize()
    assert st.item() == 0
    assert torch.isfinite(o_par).all() and torch.isfinite(s_par).all()
    assert rel_err(o_par, o_one) <= 1e-5 and rel_err(s_par, s_one) <= 1e-5
    assert torch.equal(s_par[0].cpu(), state[0])
    G = H // Hkv
    for h in sorted({1 % H, H - 2}):
        hk = h // G
        ref_state = state[:, h:h + 1].clone()
        ref = ref_ops.gla_scan_ref(q[:, h:h + 1], k[:, hk:hk + 1], v[:, hk:hk + 1], gk[:, hk:hk + 1], ref_state, qsl,
                                   slot_idx.tolist(), reset)
        assert rel_err(o_par[:, h:h + 1].cpu(), ref) <= GLA_REL
        assert rel_err(s_par[:, h:h + 1].cpu(), ref_state) <= GLA_REL


@pytest.mark.parametrize("n_seqs", [3, 1])
def test_gla_scan_hand_over_in_the_middle_of_a_run(ops, n_seqs):
    """Gates that turn strong half way through a run: the tensor-core form takes the chunks whose
    summed log-decay stays inside its range and stops at the first one that does not; the
    token-by-token kernel picks the run up at that token with the state the first one left in the
    slot. The seam must not show. With a single sequence the runs are cut into pieces owned by
    different CTAs, a piece in the middle meets the strong gates, and the whole run is handed over."""
    H, Hkv, D, T1 = 28, 4, 128, 3000
    T = n_seqs * T1
    q, k, v, gk = _scan_inputs(T, H, Hkv, D, seed=46)
    _, _, _, strong = _scan_inputs(T, H, Hkv, D, seed=47, strong_decay=True)
    for s in range(n_seqs):
        gk[s * T1 + 1300:s * T1 + 2000] = strong[s * T1 + 1300:s * T1 + 2000]     # chunks 10..15 are out of range
    qsl = [s * T1 for s in range(n_seqs + 1)]
    qsl_d = torch.tensor(qsl, dtype=torch.int32, device=DEV)
    ws = ops.gla_scan_workspace(n_seqs, T1, H, D, DEV)
    dev = lambda t: t.to(DEV)
    state = torch.randn(n_seqs, H, D, D, generator=torch.Generator().manual_seed(48)) * 0.1
    s_one, s_tc = dev(state), dev(state)
    st = _status()
    o_one = ops.gla_scan(dev(q), dev(k), dev(v), dev(gk), s_one, qsl_d, out_dtype=torch.float32, status=st)
    o_tc = ops.gla_scan(dev(q), dev(k), dev(v), dev(gk), s_tc, qsl_d, out_dtype=torch.float32, max_query_len=T1,
                        workspace=ws, status=st)
    assert st.item() == 0
    stops = ws[:4 * H * n_seqs].view(torch.int32).view(n_seqs, H).tolist()
    if n_seqs == 1:
        assert stops == [[0] * H]                                  # cut into pieces: the run is handed over whole
    else:
        assert stops == [[s * T1 + 1280] * H for s in range(n_seqs)]   # every head stopped ahead of its 11th chunk
    assert torch.isfinite(o_tc).all()
    assert rel_err(o_tc, o_one) <= 1e-5 and rel_err(s_tc, s_one) <= 1e-5
    # bf16 outputs: the same values rounded once
    s_b = dev(state)
    o_b = ops.gla_scan(dev(q), dev(k), dev(v), dev(gk), s_b, qsl_d, out_dtype=torch.bfloat16, max_query_len=T1, workspace=ws)
    assert float((o_b.float() - o_one).abs().max()) <= 2.0 ** -8 * float(o_one.abs().max())
    assert torch.equal(s_b, s_tc)


def test_gla_scan_chunk_parallel_strong_decay_and_fused_neighbours(ops):
    """The chunked forms with gates strong enough that a sub-chunk's decay product underflows to zero
    (the carried state then contributes nothing, as in the one-chain scan; the tensor-core form hands
    such runs over whole), and with the fused neighbours (ReLU on q/k, gate logits, per-head RMS norm)
    switched on."""
    H, Hkv, D, T = 28, 4, 128, 4096
    q, k, v, gk = _scan_inputs(T, H, Hkv, D, seed=37, strong_decay=True)
    qsl_d = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    ws = ops.gla_scan_workspace(1, T, H, D, DEV)
    dev = lambda t: t.to(DEV)
    g = torch.Generator().manual_seed(38)
    state = torch.randn(1, H, D, D, generator=g)
    s_one, s_par = dev(state), dev(state)
    o_one = ops.gla_scan(dev(q), dev(k), dev(v), dev(gk), s_one, qsl_d, out_dtype=torch.float32)
    o_par = ops.gla_scan(dev(q), dev(k), dev(v), dev(gk), s_par, qsl_d, out_dtype=torch.float32, max_query_len=T,
                         workspace=ws)
    assert torch.isfinite(o_par).all()
    assert rel_err(o_par, o_one) <= 1e-5 and rel_err(s_par, s_one) <= 1e-5
    # fused: un-prepared projections in, normalised read-out out
    qp = (torch.randn(T, H, D, generator=g)).bfloat16()
    kp = (torch.randn(T, Hkv, D, generator=g)).bfloat16()
    logits = (3 * torch.randn(T, Hkv, D, generator=g)).bfloat16()
    w = (1 + 0.3 * torch.randn(D, generator=g)).bfloat16().to(DEV)
    kw = dict(relu_qk=True, gate_logit_normalizer=16.0, norm_weight=w, norm_eps=1e-5, out_dtype=torch.float32)
    s_one, s_par = dev(state), dev(state)
    o_one = ops.gla_scan(dev(qp), dev(kp), dev(v), dev(logits), s_one, qsl_d, **kw)
    o_par = ops.gla_scan(dev(qp), dev(kp), dev(v), dev(logits), s_par, qsl_d, max_query_len=T, workspace=ws, **kw)
    assert rel_err(o_par, o_one) <= 1e-5 and rel_err(s_par, s_one) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gla_scan_run_longer_than_the_caller_said(ops, dtype):
    """`max_query_len` only plans the cut: a run longer than stated (here 4096 tokens against a stated
    1024 and 2048) still comes out right, its last piece taking the rest, and nothing is written past the
    workspace sized for the stated length."""
    H, Hkv, D, T = 28, 4, 128, 4096
    q, k, v, gk = _scan_inputs(T, H, Hkv, D, seed=52, dtype=dtype)
    qsl_d = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    dev = lambda t: t.to(DEV)
    state = torch.randn(1, H, D, D, generator=torch.Generator().manual_seed(53)) * 0.1
    s_one = dev(state)
    o_one = ops.gla_scan(dev(q), dev(k), dev(v), dev(gk), s_one, qsl_d, out_dtype=torch.float32)
    for stated in (1024, 2048):
        ws = ops.gla_scan_workspace(1, stated, H, D, DEV)
        guard = torch.full((ws.numel() + 4096,), 0x5A, dtype=torch.uint8, device=DEV)
        inner = guard[:ws.numel()]
        s_par, st = dev(state), _status()
        o_par = ops.gla_scan(dev(q), dev(k), dev(v), dev(gk), s_par, qsl_d, out_dtype=torch.float32,
                             max_query_len=stated, workspace=inner, status=st)
        assert st.item() == 0
        assert rel_err(o_par, o_one) <= 1e-5 and rel_err(s_par, s_one) <= 1e-5
        assert bool((guard[ws.numel():] == 0x5A).all())


def test_gla_scan_workspace_too_small_is_refused(ops):
    from spikingbrain_7b_b200 import _abi
    H, Hkv, D, T = 28, 4, 128, 2048
    q, k, v, gk = (t.to(DEV) for t in _scan_inputs(T, H, Hkv, D, seed=39))
    state = torch.zeros(1, H, D, D, device=DEV)
    small = torch.empty(1024, dtype=torch.uint8, device=DEV)
    with pytest.raises(_abi.SbkError) as e:
        ops.gla_scan(q, k, v, gk, state, torch.tensor([0, T], dtype=torch.int32, device=DEV), max_query_len=T,
                     workspace=small)
    assert e.value.code == _abi.SBK_E_WORKSPACE


# ------------------------------------------------------------- rotary embedding in the append
@pytest.mark.parametrize("name", ["bf16_d128_theta1e6", "bf16_d128_theta1e4", "f32_d64_theta1e4"])
def test_rope_append_is_bit_exact_with_reference_fixture(ops, name):
    """Query rotated in place, key rotated into the cache (and in place), value copied: all equal,
    bit for bit, to the reference's RotaryEmbedding + apply_rotary_pos_emb outputs (rope.npz)."""
    import os
    import numpy as np
    from tests.test_oracle_golden import GOLD, ROPE_POSITIONS, rope_case
    gold = np.load(os.path.join(GOLD, "rope.npz"))
    (H, kvh, D, base, dtype), q, k, want = rope_case(gold, name)
    T, bs, nb = len(ROPE_POSITIONS), 16, 4
    table = ops.build_cos_sin_cache(D, 131072, base, dtype, device=DEV)
    g = torch.Generator().manual_seed(50)
    v = torch.randn(T, kvh, D, generator=g).to(dtype)
    kc = torch.zeros(nb, bs, kvh, D, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(nb * bs, generator=g)[:T].to(torch.int64)
    slots[3] = -1                                     # padding token: rotated, not cached
    qd, kd = q.to(DEV), k.to(DEV)
    st = _status()
    ops.rope_kv_append(qd, kd, v.to(DEV), kc, vc, slots.to(DEV),
                       torch.tensor(ROPE_POSITIONS, dtype=torch.int64, device=DEV), table,
                       key_in_place=True, status=st)
    assert st.item() == 0
    assert torch.equal(qd.cpu(), want["q"]) and torch.equal(kd.cpu(), want["k"])
    flat_k, flat_v = kc.view(nb * bs, kvh, D).cpu(), vc.view(nb * bs, kvh, D).cpu()
    live = slots >= 0
    assert torch.equal(flat_k[slots[live]], want["k"][live]) and torch.equal(flat_v[slots[live]], v[live])
    untouched = torch.ones(nb * bs, dtype=torch.bool)
    untouched[slots[live]] = False
    assert not flat_k[untouched].any() and not flat_v[untouched].any()


@pytest.mark.parametrize("rot_dim", [128, 64, 32])
def test_rope_append_matches_oracle_with_retirement_and_partial_rotation(ops, rot_dim):
    """Model shapes (28/4 heads, D 128), strided q/k/v views of one projection output, key left
    as it was, partial rotary widths, and the block retirement of the plain append."""
    T = B = 6
    H, kvh, D, bs, wl = 28, 4, 128, 16, 31
    g = torch.Generator().manual_seed(51)
    qkv = torch.randn(T, (H + 2 * kvh) * D, generator=g).bfloat16().to(DEV)
    q = qkv[:, :H * D].view(T, H, D)
    k = qkv[:, H * D:(H + kvh) * D].view(T, kvh, D)
    v = qkv[:, (H + kvh) * D:].view(T, kvh, D)
    q0, k0 = q.clone().cpu(), k.clone().cpu()
    seq_lens = torch.tensor([70, 33, 48, 80, 1, 97], dtype=torch.int32)
    positions = (seq_lens - 1).to(torch.int64)
    max_blocks = 16
    tables = torch.arange(B * max_blocks, dtype=torch.int32).view(B, max_blocks)
    ref_tables = tables.clone()
    slots = torch.tensor([int(tables[b, (int(seq_lens[b]) - 1) // bs]) * bs + (int(seq_lens[b]) - 1) % bs
                          for b in range(B)], dtype=torch.int64)
    nb = B * max_blocks
    kc = torch.zeros(nb, bs, kvh, D, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    table = ops.build_cos_sin_cache(rot_dim, 256, 10000.0, torch.bfloat16, device=DEV)
    tables_d = tables.to(DEV)
    retired = torch.full((B, 4), -7, dtype=torch.int32, device=DEV)
    st = _status()
    ops.rope_kv_append(q, k, v, kc, vc, slots.to(DEV), positions.to(DEV), table, block_tables=tables_d,
                       seq_lens=seq_lens.to(DEV), window_left=wl, retired_out=retired, status=st)
    assert st.item() == 0
    cos, sin = ref_ops.rope_cos_sin_ref(positions, rot_dim, 10000.0, torch.bfloat16)
    rot = lambda x: torch.cat((ref_ops.rope_ref(x[..., :rot_dim], cos, sin), x[..., rot_dim:]), dim=-1)
    assert torch.equal(q.cpu(), rot(q0))
    assert torch.equal(k.cpu(), k0)                                   # key_in_place off
    assert torch.equal(kc.view(nb * bs, kvh, D)[slots.to(DEV)].cpu(), rot(k0))
    assert torch.equal(vc.view(nb * bs, kvh, D)[slots.to(DEV)].cpu(), v.cpu())
    want_ret = ref_ops.retire_blocks(ref_tables, seq_lens.tolist(), [1] * B, wl, bs)
    assert torch.equal(tables_d.cpu(), ref_tables)
    for b in range(B):
        assert retired[b].tolist()[:len(want_ret[b])] == want_ret[b]


def test_rope_append_flags_positions_outside_the_table(ops):
    kc = torch.zeros(2, 16, 1, 64, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    k = torch.ones(2, 1, 64, dtype=torch.bfloat16, device=DEV)
    table = ops.build_cos_sin_cache(64, 8, 10000.0, torch.bfloat16, device=DEV)
    st = _status()
    ops.rope_kv_append(None, k, k.clone(), kc, vc, torch.tensor([0, 1], device=DEV),
                       torch.tensor([3, 8], device=DEV), table, status=st)
    assert st.item() == 16                       # SBK_ST_BAD_POSITION; token 1 skipped
    assert kc[0, 0].any() and not kc[0, 1].any()


# ------------------------------------------------------------- GLA with fused neighbours
@pytest.mark.parametrize("name", ["d128_h2_kv1", "d64_h8_kv8"])
def test_gla_fused_step_matches_reference_layer_fixture(ops, name):
    """relu / gate / step / g_norm in one launch == the reference layer's pieces chained around
    its Triton kernel (tests/golden/gla_fused.npz), fp32, two steps, a slot of -1."""
    import numpy as np
    from tests.test_oracle_golden import GOLD, fused_case, golden_state
    import os
    gold = np.load(os.path.join(GOLD, "gla_fused.npz"))
    (B, H, Hkv, D, slots), (qp, kp, v, gl, w), slot = fused_case(gold, name)
    state_d = golden_state(slots, H, D).to(DEV)
    live = slot >= 0
    for step in (1, 2):
        o = ops.gla_step(qp.to(DEV), kp.to(DEV), v.to(DEV), gl.to(DEV), state_d, slot.to(DEV),
                         relu_qk=True, gate_logit_normalizer=16.0, norm_weight=w.to(DEV), norm_eps=1e-5)
        assert rel_err(o.cpu()[live], torch.from_numpy(gold[f"{name}/out{step}"])[live]) <= GLA_REL
    assert rel_err(state_d.cpu(), torch.from_numpy(gold[name + "/state2"])) <= GLA_REL


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,H,Hkv,D", [(5, 28, 4, 128), (3, 8, 2, 64)])
def test_gla_fused_step_equals_separate_ops(ops, dtype, B, H, Hkv, D):
    """The fused call == torch relu / logsigmoid-gate in the input dtype, the plain kernel, and
    the oracle's g_norm on its fp32 read-out. The state must agree bit for bit: the prologue
    reproduces the roundings of the reference's tensor expressions."""
    g = torch.Generator().manual_seed(40)
    qp = torch.randn(B, H, D, generator=g).to(dtype).to(DEV)
    kp = torch.randn(B, Hkv, D, generator=g).to(dtype).to(DEV)
    v = torch.randn(B, Hkv, D, generator=g).to(dtype).to(DEV)
    gl = (3 * torch.randn(B, Hkv, D, generator=g)).to(dtype).to(DEV)
    w = (1 + 0.3 * torch.randn(D, generator=g)).to(dtype).to(DEV)
    state = torch.randn(B, H, D, D, generator=g).to(DEV)
    s_fused, s_plain = state.clone(), state.clone()
    o_fused = ops.gla_step(qp, kp, v, gl, s_fused, relu_qk=True, gate_logit_normalizer=16.0,
                           norm_weight=w, norm_eps=1e-5, out_dtype=torch.float32)
    gk = torch.nn.functional.logsigmoid(gl) / 16
    assert gk.dtype == dtype
    o_plain = ops.gla_step(torch.relu(qp), torch.relu(kp), v, gk, s_plain, out_dtype=torch.float32)
    if dtype == torch.bfloat16:
        assert torch.equal(s_fused, s_plain)
    else:
        assert rel_err(s_fused, s_plain) <= 1e-6
    want = ref_ops.gla_norm_ref(o_plain.cpu(), w.cpu(), 1e-5)
    assert rel_err(o_fused.cpu(), want) <= GLA_REL


@pytest.mark.parametrize("D,H,Hkv", [(128, 28, 4), (64, 8, 8)])
def test_gla_fused_scan_equals_fused_steps(ops, D, H, Hkv):
    """Ragged runs through the fused scan == the fused single-token kernel token after token."""
    runs = [3, 9, 1, 6]
    qsl = [0]
    for n in runs:
        qsl.append(qsl[-1] + n)
    T = qsl[-1]
    g = torch.Generator().manual_seed(41)
    mk = lambda h, s=1.0: (s * torch.randn(T, h, D, generator=g)).bfloat16().to(DEV)
    qp, kp, v, gl = mk(H), mk(Hkv), mk(Hkv), mk(Hkv, 3.0)
    w = (1 + 0.3 * torch.randn(D, generator=g)).bfloat16().to(DEV)
    fused = dict(relu_qk=True, gate_logit_normalizer=16.0, norm_weight=w, norm_eps=1e-5)
    s_scan = torch.randn(len(runs), H, D, D, generator=g).to(DEV)
    s_step = s_scan.clone()
    o_scan = ops.gla_scan(qp, kp, v, gl, s_scan, torch.tensor(qsl, dtype=torch.int32, device=DEV),
                          out_dtype=torch.float32, **fused)
    o_step = torch.zeros_like(o_scan)
    for s, n in enumerate(runs):
        slot = torch.tensor([s], dtype=torch.int64, device=DEV)
        for t in range(qsl[s], qsl[s + 1]):
            o_step[t] = ops.gla_step(qp[t:t + 1], kp[t:t + 1], v[t:t + 1], gl[t:t + 1], s_step, slot,
                                     out_dtype=torch.float32, **fused)[0]
    assert rel_err(o_scan, o_step) <= 1e-5 and rel_err(s_scan, s_step) <= 1e-6


def test_gla_fusion_argument_errors(ops):
    from spikingbrain_7b_b200._abi import SbkError, lib
    q = torch.zeros(1, 4, 128, dtype=torch.bfloat16, device=DEV)
    S = torch.zeros(1, 4, 128, 128, device=DEV)
    with pytest.raises(ValueError):
        ops.gla_step(q, q, q, q, S, gate_logit_normalizer=0.0)
    with pytest.raises(ValueError):
        ops.gla_step(q, q, q, q, S, norm_weight=torch.ones(64, dtype=torch.bfloat16, device=DEV))
    rc = lib.sbk_gla_step(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), 0, S.data_ptr(), 1, None,
                          1, 4, 4, 128, 1.0, q.data_ptr(), 0, 64, 0.0, None, 0.0, None, None)
    assert rc == -1 and b"fuse_flags" in lib.sbk_last_error()


# ---------------------------------------------------------------------- argument errors
def test_argument_errors_are_reported(ops):
    from spikingbrain_7b_b200._abi import SbkError
    kv = torch.zeros(2, 4, 16, 4, 128, dtype=torch.bfloat16, device=DEV)
    q = torch.zeros(1, 28, 128, dtype=torch.bfloat16, device=DEV)
    table = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    lens = torch.ones(1, dtype=torch.int32, device=DEV)
    with pytest.raises(SbkError) as e:
        ops.swa_decode(q, kv[0], kv[1], table, lens, window_left=63, max_pieces=3,
                       workspace=torch.empty(16, dtype=torch.uint8, device=DEV))
    assert e.value.code == -3
    with pytest.raises(SbkError):
        ops.swa_decode(torch.zeros(1, 36, 128, dtype=torch.bfloat16, device=DEV), kv[0], kv[1], table, lens,
                       window_left=63)  # 9 query heads per kv head
    with pytest.raises(RuntimeError):
        ops.gla_step(q.cpu(), q.cpu(), q.cpu(), q.cpu(), torch.zeros(1, 28, 128, 128))


# ---------------------------------------------------------------- device-resident planner
def _planner_pair(num_blocks, bs, B, max_blocks, wl, T=None):
    from spikingbrain_7b_b200.block_pool import DeviceStepPlanner
    dev = DeviceStepPlanner(num_blocks, bs, wl, B, max_blocks, DEV, max_tokens=T)
    ref = ref_ops.StepPlannerRef(num_blocks, bs, B, max_blocks, wl)
    return dev, ref


def _same_state(dev, ref):
    snap = dev.snapshot()
    assert snap["lens"] == ref.lens and snap["table"] == ref.table
    assert snap["free"] == ref.ring and snap["min_free"] == ref.min_free
    return snap


def test_plan_step_decode_stream_is_bit_exact_with_cpu_model(ops):
    """Prompts of ragged lengths, then 100 one-token steps: every slot, position, table entry and
    the order of the free ring equal the CPU model; resident blocks stay within the window."""
    B, bs, wl, max_blocks = 7, 16, 40, 64
    dev, ref = _planner_pair(B * 5 + 3, bs, B, max_blocks, wl, T=256)
    n0 = [33, 1, 64, 17, 0, 48, 90]
    want = ref.plan(n0, T=256)
    dev.plan(torch.tensor(n0, dtype=torch.int32, device=DEV))
    assert dev.slot_mapping.tolist() == want["slot_mapping"]
    assert dev.positions.tolist()[:sum(n0)] == want["positions"][:sum(n0)]
    assert dev.query_start_loc.tolist() == want["query_start_loc"]
    assert dev.context_lens.tolist() == want["context_lens"]
    _same_state(dev, ref)
    for step in range(100):
        want = ref.plan(None, T=256)
        dev.plan()
        assert dev.slot_mapping.tolist() == want["slot_mapping"], f"step {step}"
        assert dev.positions.tolist()[:B] == want["positions"][:B]
    snap = _same_state(dev, ref)
    assert snap["status"] == 0
    for row in snap["table"]:
        assert sum(1 for x in row if x >= 0) <= (wl + 1 + bs - 1) // bs + 1
    live = [x for row in snap["table"] for x in row if x >= 0]
    assert len(set(live)) == len(live) and not set(live) & set(snap["free"])
    assert len(live) + len(snap["free"]) == dev.num_blocks            # no block lost, none owned twice


def test_plan_step_churn_with_releases_and_chunked_prompts(ops):
    """Rows finish and are re-admitted with new prompts (some in chunks) while others decode."""
    import random
    rng = random.Random(5)
    B, bs, wl, max_blocks = 24, 16, 63, 40
    dev, ref = _planner_pair(B * 6, bs, B, max_blocks, wl, T=B * 96)
    T = B * 96
    active = [False] * B
    for step in range(60):
        done = [b for b in range(B) if active[b] and (rng.random() < 0.08 or ref.lens[b] > 500)]
        if done:
            ref.release(done)
            dev.release(torch.tensor(done, dtype=torch.int32, device=DEV))
            for b in done:
                active[b] = False
        n_new = []
        for b in range(B):
            if active[b]:
                n_new.append(1)
            elif rng.random() < 0.5:
                n_new.append(rng.choice([1, 15, 16, 17, 50, 96]))
                active[b] = True
            else:
                n_new.append(0)
        want = ref.plan(n_new, T=T)
        assert want is not None
        dev.plan(torch.tensor(n_new, dtype=torch.int32, device=DEV))
        assert dev.slot_mapping.tolist() == want["slot_mapping"], f"step {step}"
        assert dev.query_start_loc.tolist() == want["query_start_loc"]
        assert dev.context_lens.tolist() == want["context_lens"]
    snap = _same_state(dev, ref)
    assert snap["status"] == 0 and snap["steps"] == 60


def test_plan_step_trim_gives_back_a_chunks_look_back_window(ops):
    """After a prompt chunk a row still holds the blocks the chunk's first token looked back on; a
    trim launch (no new tokens) returns every row to what its next token will see. Device state,
    ring order included, equals the CPU model after every launch."""
    B, bs, wl, max_blocks = 3, 16, 63, 64
    dev, ref = _planner_pair(B * 20, bs, B, max_blocks, wl, T=B * 128)
    T = B * 128
    for n_new in ([128, 40, 0], [128, 128, 7], [1, 0, 100]):
        want = ref.plan(n_new, T=T)
        assert want is not None
        dev.plan(torch.tensor(n_new, dtype=torch.int32, device=DEV))
        assert dev.slot_mapping.tolist() == want["slot_mapping"]
        _same_state(dev, ref)
        held = [sum(1 for e in row if e >= 0) for row in ref.table]
        assert ref.plan([0] * B, T=T, trim=True) is not None
        dev.trim()
        snap = _same_state(dev, ref)
        after = [sum(1 for e in row if e >= 0) for row in snap["table"]]
        assert all(a <= wl // bs + 2 for a in after), after
        assert sum(after) <= sum(held)
    assert snap["status"] == 0


def test_release_rows_names_a_row_twice_releases_it_once(ops):
    """A repeated entry in the list of finished rows must not count the row's blocks twice (the ring's
    tail would run ahead of what was pushed and a block would later be handed to two sequences): the
    device state equals the CPU model's, in which the second mention finds an empty row."""
    B, bs, wl, max_blocks = 6, 16, -1, 12
    dev, ref = _planner_pair(B * 12, bs, B, max_blocks, wl, T=B * 64)
    n_new = [40, 17, 64, 1, 33, 50]
    assert ref.plan(n_new, T=B * 64) is not None
    dev.plan(torch.tensor(n_new, dtype=torch.int32, device=DEV))
    rows = [2, 4, 2, 0, 4, 2]
    ref.release(rows)
    dev.release(torch.tensor(rows, dtype=torch.int32, device=DEV))
    snap = _same_state(dev, ref)
    assert snap["status"] == 0
    assert len(snap["free"]) == len(set(snap["free"])), "a block id sits in the ring twice"
    # the pool still serves: re-admit the released rows and compare every slot
    n_new = [16, 0, 70, 0, 5, 0]
    want = ref.plan(n_new, T=B * 64)
    dev.plan(torch.tensor(n_new, dtype=torch.int32, device=DEV))
    assert dev.slot_mapping.tolist() == want["slot_mapping"]
    _same_state(dev, ref)


def test_plan_step_refuses_cleanly_when_the_ring_is_empty_or_a_row_is_full(ops):
    dev, ref = _planner_pair(4, 16, 2, 8, -1, T=2)      # no window: nothing is ever retired
    for _ in range(32):                                  # 2 rows x 2 blocks = the whole pool
        dev.plan(); ref.plan(None, T=2)
    before = _same_state(dev, ref)
    dev.plan()                                           # both rows need a third block
    assert ref.plan(None, T=2) is None
    after = dev.snapshot()
    assert after["status"] == 32 and dev.slot_mapping.tolist() == [-1, -1]
    assert {k: after[k] for k in ("lens", "table", "free")} == {k: before[k] for k in ("lens", "table", "free")}
    dev2, _ = _planner_pair(64, 16, 1, 2, -1, T=1)       # a table row of two columns
    for _ in range(32):
        dev2.plan()
    assert dev2.snapshot()["status"] == 0
    dev2.plan()
    assert dev2.snapshot()["status"] == 64 and dev2.seq_lens.item() == 32


def test_plan_step_without_ring_is_advance_step(ops):
    """Tables filled by the engine: lengths and slots advance, a missing block is reported."""
    B, bs = 3, 16
    tables = torch.tensor([[5, 9, -1], [2, -1, -1], [7, 1, 3]], dtype=torch.int32, device=DEV)
    lens = torch.tensor([20, 15, 40], dtype=torch.int32, device=DEV)
    slots = torch.empty(4, dtype=torch.int64, device=DEV)
    pos = torch.empty(4, dtype=torch.int64, device=DEV)
    st = _status()
    ops.plan_step(lens, tables, slots, block_size=bs, num_blocks=10, retire=False, positions=pos, status=st)
    assert slots.tolist() == [9 * 16 + 4, 2 * 16 + 15, 3 * 16 + 8, -1] and pos.tolist()[:3] == [20, 15, 40]
    assert lens.tolist() == [21, 16, 41] and st.item() == 0
    ops.plan_step(lens, tables, slots, block_size=bs, num_blocks=10, retire=False, status=st)   # row 1 needs a block
    assert st.item() == 32 and lens.tolist() == [21, 16, 41] and slots.tolist() == [-1] * 4


# ------------------------------------------------------------------ fused all-gather of the head outputs
def _emulated_gather(ops, lens, wl, H, kvh, tp, seed, split_chunks, step=1, base=None):
    """Ranks of a head-sharded group run one after the other on this GPU, each with buffers of its
    own: rank r computes its head slice and stores it to every other rank's buffer. No kernel
    waits for another (the waits are enqueued after every writer has finished)."""
    from spikingbrain_7b_b200.head_shard import shard_heads
    D, bs = 128, 16
    B = len(lens)
    kv, table, nb = make_paged_kv(lens, wl, kvh, D, bs, seed=seed)
    g = torch.Generator().manual_seed(seed + 100)
    q = (torch.randn(B, H, D, generator=g) / math.sqrt(D)).bfloat16()
    ref = ref_ops.swa_paged_decode_ref(q, kv[0], kv[1], table, lens, wl, D ** -0.5)
    bufs = [torch.full((B, H, D), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(tp)]
    flags = [torch.zeros(tp, dtype=torch.int32, device=DEV) for _ in range(tp)]
    st = _status()
    lens_d = torch.tensor(lens, dtype=torch.int32, device=DEV)
    table_d = table.to(DEV)
    plain = []
    for r in range(tp):
        qh, kh = shard_heads(H, kvh, tp, r)
        kv_l = kv[:, :, :, kh.start:kh.stop].contiguous().to(DEV)
        q_l = q[:, qh.start:qh.stop].contiguous().to(DEV)
        others = [p for p in range(tp) if p != r]
        slice_bytes = len(qh) * D * 2
        peers = ops.PeerTargets([bufs[p].data_ptr() + r * slice_bytes for p in others],
                                [flags[p].data_ptr() + 4 * r for p in others], step, base)
        ops.swa_decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl, out=bufs[r][:, qh.start:qh.stop],
                       peers=peers, split_chunks=split_chunks, status=st)
        plain.append(ops.swa_decode(q_l, kv_l[0], kv_l[1], table_d, lens_d, window_left=wl,
                                    split_chunks=split_chunks, status=st))
    torch.cuda.synchronize()
    return bufs, flags, torch.cat(plain, dim=1), ref, st


@pytest.mark.parametrize("tp,H,kvh,split_chunks", [(2, 28, 4, -8), (4, 28, 4, -2), (2, 28, 4, 32), (1, 14, 2, -8),
                                                   (4, 32, 8, -4), (7, 28, 28, -8)])
def test_swa_decode_gather_fills_every_ranks_buffer(ops, tp, H, kvh, split_chunks):
    """sbk_swa_decode_gather: every rank's buffer ends up with all heads, bit-identical to the plain
    kernel's output (the rows are copied, not recomputed), flags raised to the step value; whole and
    split sequences, empty ones, kv-head layouts of 1, 2 and 4 per rank."""
    lens = [4100, 513, 40, 2000, 0, 1, 16, 8193, 333]
    bufs, flags, plain, ref, st = _emulated_gather(ops, lens, 4096, H, kvh, tp, seed=60 + tp, split_chunks=split_chunks,
                                                  step=5)
    assert st.item() == 0
    for r in range(tp):
        assert torch.equal(bufs[r], plain)                      # NaN prefill: every element was written
        want = [5] * tp
        want[r] = 0                                             # nobody raises a rank's own slot
        assert flags[r].tolist() == want
    a = plain.float().cpu()
    tgt = ref.bfloat16().float()
    assert float((a - tgt).abs().max()) <= ATTN_MAX_ABS and mean_rel(a, tgt) <= ATTN_MEAN_REL


def test_swa_decode_gather_many_sequences_two_launches(ops):
    """More sequences than one launch takes: the peers' rows of the later launch land at the right
    offset and only the last launch raises the flags."""
    g = torch.Generator().manual_seed(70)
    lens = torch.randint(0, 90, (1100,), generator=g).tolist()
    bufs, flags, plain, ref, st = _emulated_gather(ops, lens, 63, 14, 2, 2, seed=71, split_chunks=-8, step=3)
    assert st.item() == 0
    assert torch.equal(bufs[0], plain) and torch.equal(bufs[1], plain)
    assert flags[0].tolist() == [0, 3] and flags[1].tolist() == [3, 0]


def test_swa_decode_gather_flag_value_relative_to_device_counter(ops):
    """The flag value is flag_value + a word read on the device at the end of the kernel."""
    base = torch.tensor([40], dtype=torch.int32, device=DEV)
    bufs, flags, plain, ref, st = _emulated_gather(ops, [700, 3, 64], 255, 14, 2, 2, seed=72, split_chunks=-8, step=2,
                                                  base=base)
    assert st.item() == 0 and torch.equal(bufs[0], plain) and torch.equal(bufs[1], plain)
    assert flags[0].tolist() == [0, 42] and flags[1].tolist() == [42, 0] and base.item() == 40


def test_peer_wait_passes_and_times_out_cleanly(ops):
    """sbk_peer_wait returns at once when every peer's flag has reached the value, and after its
    time limit otherwise: status bit raised, kernel returned, context still usable."""
    from spikingbrain_7b_b200 import _abi
    flags = torch.tensor([7, 0, 9, 7], dtype=torch.int32, device=DEV)      # rank 1 is the reader
    st = _status()
    stream = torch.cuda.current_stream().cuda_stream
    _abi.check("sbk_peer_wait", _abi.lib.sbk_peer_wait(flags.data_ptr(), 4, 1, 7, None, 0, 50, st.data_ptr(), stream))
    torch.cuda.synchronize()
    assert st.item() == 0
    base = torch.tensor([4], dtype=torch.int32, device=DEV)                # value relative to a device word
    _abi.check("sbk_peer_wait", _abi.lib.sbk_peer_wait(flags.data_ptr(), 4, 1, 3, base.data_ptr(), 2, 50,
                                                       st.data_ptr(), stream))
    torch.cuda.synchronize()
    assert st.item() == 0 and base.item() == 6
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    _abi.check("sbk_peer_wait", _abi.lib.sbk_peer_wait(flags.data_ptr(), 4, 1, 2, base.data_ptr(), 1, 50,
                                                       st.data_ptr(), stream))
    ev1.record()
    torch.cuda.synchronize()
    assert st.item() == _abi.ST_WAIT_TIMEOUT and base.item() == 7          # the counter moves on regardless
    assert 40.0 <= ev0.elapsed_time(ev1) <= 1000.0
    assert int((flags + 1).sum().item()) == 27                              # the context still works
    with pytest.raises(_abi.SbkError):
        _abi.check("sbk_peer_wait", _abi.lib.sbk_peer_wait(flags.data_ptr(), 4, 1, 8, None, 0, 0, st.data_ptr(), stream))


def test_peer_memory_alloc_export_and_signal(ops):
    """Peer-visible memory: zeroed on allocation, exportable as a handle of the advertised size;
    sbk_peer_signal raises flags inside it."""
    import ctypes
    from spikingbrain_7b_b200 import _abi
    from spikingbrain_7b_b200.head_shard import _DeviceBytes
    lib = _abi.lib
    base = ctypes.c_void_p()
    _abi.check("sbk_peer_alloc", lib.sbk_peer_alloc(4096, ctypes.byref(base)))
    try:
        hb = lib.sbk_peer_handle_bytes()
        assert hb == 64
        handle = ctypes.create_string_buffer(hb)
        _abi.check("sbk_peer_export", lib.sbk_peer_export(base.value, handle, hb))
        assert any(handle.raw)
        with pytest.raises(_abi.SbkError):
            _abi.check("sbk_peer_export", lib.sbk_peer_export(base.value, handle, hb - 1))
        t = torch.as_tensor(_DeviceBytes(base.value, 4096), device=DEV)
        assert t.data_ptr() == base.value and not t.any()
        flags = t[:16].view(torch.int32)
        table = (ctypes.c_void_p * 2)(base.value + 4, base.value + 12)
        _abi.check("sbk_peer_signal", lib.sbk_peer_signal(table, 2, 11, None, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert flags.tolist() == [0, 11, 0, 11]
        del t, flags
    finally:
        _abi.check("sbk_peer_free", lib.sbk_peer_free(base.value))


@pytest.mark.parametrize("tp,fused", [(2, False), (4, True), (1, True)])
def test_gla_step_gather_fills_every_ranks_buffer(ops, tp, fused):
    """sbk_gla_step_gather with the ranks emulated one after the other on this GPU: each rank's
    state slice and head outputs equal the plain kernel's bit for bit, every buffer holds all heads,
    padded sequences (slot -1) leave their rows alone, flags carry the step value."""
    from spikingbrain_7b_b200.head_shard import shard_heads
    B, H, Hkv, D, step = 6, 28, 4, 128, 9
    g = torch.Generator().manual_seed(80 + tp)
    q = torch.randn(B, H, D, generator=g).bfloat16()
    k = torch.randn(B, Hkv, D, generator=g).bfloat16()
    v = torch.randn(B, Hkv, D, generator=g).bfloat16()
    gl = (3 * torch.randn(B, Hkv, D, generator=g)).bfloat16()
    w = (1 + 0.3 * torch.randn(D, generator=g)).bfloat16().to(DEV)
    state = torch.randn(B + 2, H, D, D, generator=g)
    slot = torch.tensor([3, 0, -1, 7, 5, 1], dtype=torch.int64, device=DEV)
    kw = dict(relu_qk=True, gate_logit_normalizer=16.0, norm_weight=w, norm_eps=1e-5) if fused else {}
    if not fused:
        gl = (torch.nn.functional.logsigmoid(gl.float()) / 16).bfloat16()
    bufs = [torch.full((B, H, D), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(tp)]
    flags = [torch.zeros(tp, dtype=torch.int32, device=DEV) for _ in range(tp)]
    counter = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = _status()
    plain = torch.full((B, H, D), 7.0, dtype=torch.bfloat16, device=DEV)
    for r in range(tp):
        qh, kh = shard_heads(H, Hkv, tp, r)
        args = [t[:, hs.start:hs.stop].contiguous().to(DEV) for t, hs in ((q, qh), (k, kh), (v, kh), (gl, kh))]
        s_gather = state[:, qh.start:qh.stop].contiguous().to(DEV)
        s_plain = s_gather.clone()
        others = [p for p in range(tp) if p != r]
        peers = ops.PeerTargets([bufs[p].data_ptr() + r * len(qh) * D * 2 for p in others],
                                [flags[p].data_ptr() + 4 * r for p in others], step)
        ops.gla_step(*args, s_gather, slot, out=bufs[r][:, qh.start:qh.stop], peers=peers, peer_counter=counter,
                     status=st, **kw)
        o = ops.gla_step(*args, s_plain, slot, out_dtype=torch.bfloat16, status=st, **kw)
        live = slot >= 0
        plain[:, qh.start:qh.stop][live] = o[live]
        torch.cuda.synchronize()
        assert torch.equal(s_gather, s_plain) and counter.item() == 0
    assert st.item() == 0
    for r in range(tp):
        assert torch.equal(bufs[r], plain)
        want = [step] * tp
        want[r] = 0
        assert flags[r].tolist() == want


@pytest.mark.parametrize("H,kvh", [(7, 1), (14, 2)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_swa_decode_output_rows_need_no_alignment(ops, H, kvh, out_dtype):
    """Head layouts whose warps share a kv head write four outputs at a time where the address
    allows it; an output tensor that starts one element into its storage takes the scalar stores."""
    D, bs, wl = 128, 16, 255
    lens = [300, 17, 64, 0, 1000]
    B = len(lens)
    kv, table, nb = make_paged_kv(lens, wl, kvh, D, bs, seed=90)
    g = torch.Generator().manual_seed(91)
    q = (torch.randn(B, H, D, generator=g) / math.sqrt(D)).bfloat16()
    ref = ref_ops.swa_paged_decode_ref(q, kv[0], kv[1], table, lens, wl, D ** -0.5)
    kv_d = kv.to(DEV)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=DEV)
    outs = []
    for off in (0, 1):
        store = torch.full((B * H * D + 8,), float("nan"), dtype=out_dtype, device=DEV)
        out = store[off:off + B * H * D].view(B, H, D)
        st = _status()
        ops.swa_decode(q.to(DEV), kv_d[0], kv_d[1], table.to(DEV), lens_d, window_left=wl, out=out, status=st)
        torch.cuda.synchronize()
        assert st.item() == 0 and torch.isfinite(out.float()).all()
        assert torch.isnan(store[:off].float()).all() and torch.isnan(store[off + B * H * D:].float()).all()
        outs.append(out.clone())
    assert torch.equal(outs[0], outs[1])
    a = outs[0].float().cpu()
    tgt = ref.to(out_dtype).float()
    assert float((a - tgt).abs().max()) <= ATTN_MAX_ABS and mean_rel(a, tgt) <= ATTN_MEAN_REL
