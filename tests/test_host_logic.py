"""CPU: host-side logic -- the C ABI exports, the block manager, the backend metadata classes,
the GLA slot manager and the argument checking of the surfaces. No kernel is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from oracle import ref_ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ------------------------------------------------------------------------------- C ABI
def test_library_exports_every_declared_symbol(sb):
    header = open(os.path.join(ROOT, "include", "sbk.h")).read()
    declared = set(re.findall(r"\b(sbk_[a-z_0-9]+)\s*\(", header))
    assert {"sbk_kv_append", "sbk_kv_gather", "sbk_swa_decode", "sbk_swa_workspace_bytes",
            "sbk_gla_step", "sbk_gla_scan", "sbk_swa_prefill", "sbk_last_error", "sbk_abi_version", "sbk_swa_copy_mode"} <= declared
    lib = ctypes.CDLL(os.path.join(ROOT, "spikingbrain-7b_b200", "libsbk.so"))
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/sbk.h but not exported"
    from spikingbrain_7b_b200 import _abi
    assert set(_abi.SIGNATURES) == declared
    assert _abi.lib.sbk_abi_version() == _abi.ABI_VERSION == 5
    assert int(re.search(r"#define SBK_ABI_VERSION (\d+)", header).group(1)) == _abi.ABI_VERSION


def _header_prototypes():
    """name -> (return class, [argument class]) of every function include/sbk.h declares; a class is
    'ptr', 'float', 'i32', 'i64' or 'size'."""
    text = open(os.path.join(ROOT, "include", "sbk.h")).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = "\n".join(l for l in text.splitlines() if not l.lstrip().startswith("#"))

    def cls(decl):
        decl = decl.strip()
        if "*" in decl:
            return "ptr"
        base = re.sub(r"\b(const|unsigned)\b", "", decl).split()
        ty = base[0] if base else decl
        return {"float": "float", "int": "i32", "int32_t": "i32", "int64_t": "i64", "size_t": "size",
                "void": "void"}[ty]

    protos = {}
    for ret, name, args in re.findall(r"([A-Za-z_0-9\s\*]+?)\b(sbk_[a-z_0-9]+)\s*\(([^)]*)\)\s*;", text):
        args = args.strip()
        arg_list = [] if args in ("", "void") else [cls(a) for a in args.split(",")]
        protos[name] = (cls(ret), arg_list)
    return protos


def test_binding_signatures_match_the_header(sb):
    """Every prototype of include/sbk.h against _abi.SIGNATURES: same argument count, and pointer /
    float / 32-bit / 64-bit / size class of every argument and of the return value, so the header,
    the ctypes binding and the stub in INTEGRATION.md (generated from the binding) cannot drift."""
    from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
    from spikingbrain_7b_b200 import _abi
    to_cls = {c_void_p: "ptr", c_char_p: "ptr", c_float: "float", c_int: "i32", c_int32: "i32", c_int64: "i64",
              c_size_t: "size"}
    protos = _header_prototypes()
    assert set(protos) == set(_abi.SIGNATURES)
    for name, (restype, argtypes) in _abi.SIGNATURES.items():
        h_ret, h_args = protos[name]
        assert to_cls[restype] == h_ret, f"{name}: return type"
        assert len(argtypes) == len(h_args), f"{name}: {len(argtypes)} bound arguments, {len(h_args)} declared"
        for i, (a, b) in enumerate(zip(argtypes, h_args)):
            assert to_cls[a] == b, f"{name}: argument {i} bound as {to_cls[a]}, declared {b}"


def test_integration_doc_stub_is_the_current_binding(sb):
    """The sample ctypes stub in INTEGRATION.md lists sbk_gla_step's arguments: they must be the
    header's, in number and order."""
    text = open(os.path.join(ROOT, "include", "sbk.h")).read()
    m = re.search(r"int sbk_gla_step\(([^;]*)\);", text)
    names = [a.strip().split()[-1].lstrip("*") for a in m.group(1).replace("\n", " ").split(",")]
    doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    stub = re.search(r"sbk_gla_step\.argtypes = \[(.*?)\]", doc, flags=re.S)
    assert stub is not None, "INTEGRATION.md lost its sbk_gla_step stub"
    doc_names = re.findall(r"#\s*([A-Za-z_0-9]+)", stub.group(1))
    assert doc_names == names, (doc_names, names)


def test_host_side_argument_errors_need_no_gpu(sb):
    """Argument validation happens before any CUDA call, so it can be exercised on the CPU."""
    from spikingbrain_7b_b200 import _abi
    lib = _abi.lib
    rc = lib.sbk_gla_step(None, None, None, None, 0, None, 4, None, 2, 28, 4, 96, 1.0, None, 0, 0, 0.0, None, 0.0, None, None)
    assert rc == _abi.SBK_E_ARG and b"D=96" in lib.sbk_last_error()
    rc = lib.sbk_swa_decode(None, 0, None, None, None, 4, None, 2, 36, 4, 128, 8, 16, 0, 63, 1.0, None, 0, 0,
                            None, None, 0, 0, 1, -1, None, None, 0, None, None)
    assert rc == _abi.SBK_E_ARG and b"unsupported shape" in lib.sbk_last_error()
    rc = lib.sbk_swa_decode(None, 0, None, None, None, 4, None, 2, 28, 4, 128, 8, 24, 0, 63, 1.0, None, 0, 0,
                            None, None, 0, 0, 1, -1, None, None, 0, None, None)
    rc2 = lib.sbk_swa_decode(None, 0, None, None, None, 4, None, 2, 28, 4, 128, 8, 16, 0, 63, 1.0, None, 0, 0,
                             None, None, 0, 0, 1, -1, None, None, 100, None, None)
    assert rc2 == _abi.SBK_E_ARG            # 100 sink tokens: not a multiple of 16, and no tensors
    assert rc == _abi.SBK_E_ARG and b"multiple of 16" in lib.sbk_last_error()
    assert lib.sbk_kv_append(None, None, None, None, None, 3, 4, 128, 2, 1024, 8, 16, 16384, None, 0, None,
                             None, 0, -1, None, 0, None, None) == _abi.SBK_E_ARG
    # empty work is a successful no-op
    assert lib.sbk_gla_step(None, None, None, None, 0, None, 0, None, 0, 28, 4, 128, 1.0, None, 0, 0, 0.0, None, 0.0, None, None) == 0
    assert lib.sbk_swa_workspace_bytes(256, 28, 128, 9) >= 256 * 9 * 28 * 130 * 4
    # GLA scan scratch: the hand-over positions of the tensor-core form (one int32 per sequence and head,
    # rounded to 256 bytes, for runs of 256 tokens or more) and, when the (sequence, head) chains would leave
    # the GPU mostly idle, the sub-chunk states of the chunk-parallel form
    assert lib.sbk_gla_scan_workspace_bytes(8, 8192, 28, 128) == 1792       # 224 chains: not cut; 2 x 224 int32
    assert lib.sbk_gla_scan_workspace_bytes(1, 255, 28, 128) == 0           # short runs: one chain, token by token
    assert lib.sbk_gla_scan_workspace_bytes(1, 8192, 28, 128) == 256 + 9 * 28 * (128 * 128 + 128) * 4   # 10 sub-chunks
    rc = lib.sbk_swa_prefill(None, 0, None, None, None, 4, None, None, 1, 16, 28, 4, 128, 8, 16, 0, 63, 1.0, None, 0,
                             None, None, 0, 7, None, None)
    assert rc == _abi.SBK_E_ARG and b"kernel=7" in lib.sbk_last_error()
    with pytest.raises(RuntimeError):
        from spikingbrain_7b_b200 import ops
        ops.gla_step(torch.zeros(1, 2, 64), torch.zeros(1, 2, 64), torch.zeros(1, 2, 64),
                     torch.zeros(1, 2, 64), torch.zeros(1, 2, 64, 64))   # CPU tensors: no CPU path


# ----------------------------------------------------------------------- block manager
@pytest.mark.parametrize("bs,wl", [(16, 40), (32, 63), (16, -1), (16, 0)])
def test_block_manager_matches_oracle_retirement(bs, wl):
    """Prompt + decode steps: slots, table and retired ids equal the oracle's rule applied to
    an independently tracked table."""
    from spikingbrain_7b_b200.block_pool import SlidingWindowBlockManager
    lens0 = [1, 15, 16, 17, 100, 333]
    B, steps = len(lens0), 80
    max_blocks = (max(lens0) + steps + bs) // bs + 1
    mgr = SlidingWindowBlockManager(B * (max_blocks + 1), bs, wl, B, max_blocks)
    for r in range(B):
        mgr.admit(r)
    shadow = torch.full((B, max_blocks), -1, dtype=torch.int32)
    lens = [0] * B
    for step in range(steps + 1):
        n_new = lens0 if step == 0 else [1] * B
        plan = mgr.advance(np.array(n_new))
        for r, j, pb in plan.new_entries.tolist():
            assert shadow[r, j] == -1
            shadow[r, j] = pb
        lens = [L + n for L, n in zip(lens, n_new)]
        assert plan.seq_lens.tolist() == lens
        # slots point at the right place of the right block
        off = 0
        for r, n in enumerate(n_new):
            for i in range(n):
                pos = lens[r] - n + i
                assert plan.slot_mapping[off + i] == int(shadow[r, pos // bs]) * bs + pos % bs
            off += n
        exp = ref_ops.retire_blocks(shadow, lens, n_new, wl, bs)
        assert plan.retired == exp, f"step {step}"
        assert np.array_equal(mgr.table, shadow.numpy())
        if wl >= 0 and step > 0:
            for r in range(B):   # after a decode step the resident blocks are bounded by the window
                assert mgr.resident_blocks(r) <= (wl + 1 + bs - 1) // bs + 1
    used = int((mgr.table >= 0).sum())
    assert used + mgr.pool.num_free == mgr.pool.num_blocks      # nothing leaked


def test_block_manager_churn_reuses_blocks_and_pads_inactive_rows():
    from spikingbrain_7b_b200.block_pool import OutOfBlocks, SlidingWindowBlockManager
    bs, wl, B = 16, 63, 8
    mgr = SlidingWindowBlockManager(64, bs, wl, B, 64)
    rng = np.random.default_rng(0)
    allocations = 0
    for r in range(B - 1):
        mgr.admit(r)
    mgr.advance(np.array([int(x) for x in rng.integers(1, 120, B - 1)] + [0]), pad_inactive=False)
    for step in range(200):
        plan = mgr.advance(mgr.active.astype(np.int64))
        assert plan.slot_mapping.shape == (B,) and (plan.slot_mapping[~mgr.active] == -1).all()
        live = plan.slot_mapping[mgr.active]
        assert len(set(live.tolist())) == len(live)              # no two sequences share a slot
        allocations += len(plan.new_entries)
        if step % 5 == 0:                                        # one sequence finishes, one arrives
            victim = int(rng.choice(np.nonzero(mgr.active)[0]))
            mgr.finish(victim)
            newcomer = int(np.nonzero(~mgr.active)[0][0])
            mgr.admit(newcomer)
            mgr.advance(np.where(np.arange(B) == newcomer, int(rng.integers(1, 200)), 0), pad_inactive=False)
    assert allocations > mgr.pool.num_blocks                     # retired blocks went round again
    small = SlidingWindowBlockManager(2, bs, -1, 1, 8)
    small.admit(0)
    with pytest.raises(OutOfBlocks):
        small.advance(np.array([100]))
    with pytest.raises(ValueError):
        SlidingWindowBlockManager(4, 24, 8, 1, 4)                # block size must be a multiple of 16


# ------------------------------------------------------------------------------ backend
def test_backend_static_surface():
    from spikingbrain_7b_b200.backend import (MetaAttentionBackend, MetaAttentionImpl, MetaAttentionMetadata,
                                               MetaAttentionMetadataBuilder)
    assert MetaAttentionBackend.get_name() == "META_FLASH_ATTN"
    assert MetaAttentionBackend.accept_output_buffer is True
    assert MetaAttentionBackend.get_supported_head_sizes() == [128]      # what the kernels are built for
    assert MetaAttentionBackend.get_kv_cache_shape(10, 16, 4, 128) == (2, 10, 16, 4, 128)
    with pytest.raises(ValueError):
        MetaAttentionBackend.get_kv_cache_shape(10, 8, 4, 128)
    assert MetaAttentionBackend.get_impl_cls() is MetaAttentionImpl
    assert MetaAttentionBackend.get_metadata_cls() is MetaAttentionMetadata
    assert MetaAttentionBackend.get_builder_cls() is MetaAttentionMetadataBuilder
    impl = MetaAttentionImpl(28, 128, 128 ** -0.5, 4, None, 4097, "auto")
    assert impl.sliding_window == (4096, 0) and impl.num_queries_per_kv == 7
    assert MetaAttentionImpl(28, 128, 1.0, 4, None, None, "auto").sliding_window == (-1, -1)
    with pytest.raises(NotImplementedError):
        MetaAttentionImpl(28, 128, 1.0, 4, None, 4097, "auto", kv_sharing_target_layer_name="x")
    with pytest.raises(ValueError):
        MetaAttentionImpl(28, 128, 1.0, 4, None, 4097, "auto", blocksparse_params={})
    with pytest.raises(ValueError):
        MetaAttentionImpl(28, 100, 1.0, 4, None, 4097, "auto")
    with pytest.raises(NotImplementedError):
        MetaAttentionImpl(28, 128, 1.0, 4, None, 4097, "fp8")
    # block copies are plain tensor moves
    kv = torch.arange(2 * 6 * 2, dtype=torch.float32).view(2, 6, 2)
    before = kv.clone()
    MetaAttentionBackend.copy_blocks([kv], torch.tensor([[0, 3], [1, 5]]))
    assert torch.equal(kv[:, 3], before[:, 0]) and torch.equal(kv[:, 5], before[:, 1])
    dst = torch.zeros_like(kv)
    MetaAttentionBackend.swap_blocks(kv, dst, torch.tensor([[2, 4]]))
    assert torch.equal(dst[:, 4], kv[:, 2]) and dst[:, :4].sum() == 0


class _Obj:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def _builder(inter, sliding_window, block_size=16, chunked=False):
    from spikingbrain_7b_b200.backend import MetaAttentionMetadataBuilder
    runner = _Obj(device="cpu", pin_memory=False, graph_block_tables=np.zeros((8, 6), dtype=np.int32))
    ib = _Obj(runner=runner, sliding_window=sliding_window, block_size=block_size, inter_data_list=inter,
              chunked_prefill_enabled=chunked)
    b = MetaAttentionMetadataBuilder(ib)
    b.prepare()
    return b


def test_metadata_builder_decode_window_truncates_tables():
    """Two decoding sequences under a window: trailing blocks only, slots at the last position,
    views split correctly (meta_attention.py:435-494, 521-608)."""
    tables = {7: list(range(100, 140)), 9: [5, 6]}
    inter = [
        _Obj(is_prompt=False, block_tables=tables, seq_ids=[7], input_tokens=[[1]], orig_seq_lens=[600],
             seq_lens=[72], query_lens=[1], context_lens=[599], curr_sliding_window_blocks=[5],
             multi_modal_placeholder_maps=None, prefix_cache_hit=False),
        _Obj(is_prompt=False, block_tables=tables, seq_ids=[9], input_tokens=[[2]], orig_seq_lens=[20],
             seq_lens=[20], query_lens=[1], context_lens=[19], curr_sliding_window_blocks=[0],
             multi_modal_placeholder_maps=None, prefix_cache_hit=False),
    ]
    b = _builder(inter, sliding_window=65)
    md = b.build(seq_lens=[72, 20], query_lens=[1, 1], cuda_graph_pad_size=-1, batch_size=2)
    assert md.num_prefills == 0 and md.num_decode_tokens == 2 and md.max_decode_seq_len == 72
    assert md.block_tables.tolist() == [[135, 136, 137, 138, 139], [5, 6, 0, 0, 0]]
    assert md.slot_mapping.tolist() == [tables[7][599 // 16] * 16 + 599 % 16, 6 * 16 + 3]
    assert md.seq_lens_tensor.dtype == torch.int32 and md.slot_mapping.dtype == torch.int64
    assert md.query_start_loc.tolist() == [0, 1, 2] and md.seq_start_loc.tolist() == [0, 72, 92]
    assert md.prefill_metadata is None
    dm = md.decode_metadata
    assert dm is md.decode_metadata and dm.num_decode_tokens == 2 and dm.block_tables.shape == (2, 5)


def test_metadata_builder_mixed_batch_and_graph_padding():
    """A chunked prompt followed by a decode, then the captured-graph padding path."""
    tables = {1: [3, 4, 8], 2: [9]}
    inter = [
        _Obj(is_prompt=True, block_tables=tables, seq_ids=[1], input_tokens=[[0] * 20], orig_seq_lens=[40],
             seq_lens=[40], query_lens=[20], context_lens=[20], curr_sliding_window_blocks=[0],
             multi_modal_placeholder_maps=None, prefix_cache_hit=False),
        _Obj(is_prompt=False, block_tables=tables, seq_ids=[2], input_tokens=[[5]], orig_seq_lens=[4],
             seq_lens=[4], query_lens=[1], context_lens=[3], curr_sliding_window_blocks=[0],
             multi_modal_placeholder_maps=None, prefix_cache_hit=False),
    ]
    b = _builder(inter, sliding_window=None, chunked=True)
    md = b.build(seq_lens=[40, 4], query_lens=[20, 1], cuda_graph_pad_size=-1, batch_size=21)
    assert (md.num_prefills, md.num_prefill_tokens, md.num_decode_tokens) == (1, 20, 1)
    exp = [tables[1][p // 16] * 16 + p % 16 for p in range(20, 40)] + [9 * 16 + 3]
    assert md.slot_mapping.tolist() == exp
    pm, dm = md.prefill_metadata, md.decode_metadata
    assert pm.slot_mapping.tolist() == exp[:20] and dm.slot_mapping.tolist() == exp[20:]
    assert pm.block_tables.tolist() == [[3, 4, 8]] and dm.block_tables.tolist() == [[9, 0, 0]]
    assert pm.context_lens_tensor.tolist() == [20] and dm.query_start_loc.tolist() == [0, 1]
    # a prompt longer than the window masks the tokens nothing will look at again
    from spikingbrain_7b_b200.backend import PAD_SLOT_ID, compute_slot_mapping, compute_slot_mapping_start_idx
    sm = []
    start = compute_slot_mapping_start_idx(True, 40, 0, 16)
    compute_slot_mapping(False, sm, 1, 40, 0, start, 16, {1: [3, 4, 8]})
    assert sm[:24] == [PAD_SLOT_ID] * 24 and sm[24:] == [4 * 16 + 8 + i for i in range(8)] + [8 * 16 + i for i in range(8)]
    sm = []
    compute_slot_mapping(True, sm, 1, 40, 0, 0, 16, None)      # profile run: nothing is written
    assert sm == [PAD_SLOT_ID] * 40
    # captured graph: batch padded from 1 to 4 sequences
    inter = [inter[1]]
    b = _builder(inter, sliding_window=None)
    md = b.build(seq_lens=[4, 1, 1, 1], query_lens=[1, 1, 1, 1], cuda_graph_pad_size=3, batch_size=4)
    assert md.use_cuda_graph and md.num_decode_tokens == 4
    assert md.slot_mapping.tolist() == [9 * 16 + 3, -1, -1, -1]
    assert md.block_tables.shape == (4, 6) and md.block_tables[0, 0] == 9


def test_metadata_advance_step_moves_slots_on_device_tensors():
    from spikingbrain_7b_b200.backend import MetaAttentionMetadata
    tables = torch.tensor([[3, 4, 8], [9, 2, 0]], dtype=torch.int32)
    md = MetaAttentionMetadata(
        num_prefills=0, num_prefill_tokens=0, num_decode_tokens=2,
        slot_mapping=torch.tensor([4 * 16 + 15, 9 * 16 + 3]), seq_lens=[32, 4],
        seq_lens_tensor=torch.tensor([32, 4], dtype=torch.int32), max_prefill_seq_len=0, max_decode_seq_len=32,
        context_lens_tensor=torch.tensor([31, 3], dtype=torch.int32), block_tables=tables, use_cuda_graph=False,
        max_query_len=1, max_decode_query_len=1, query_start_loc=torch.tensor([0, 1, 2], dtype=torch.int32),
        seq_start_loc=torch.tensor([0, 32, 36], dtype=torch.int32))
    mi = _Obj(input_tokens=torch.zeros(2, dtype=torch.long), input_positions=torch.zeros(2, dtype=torch.long))
    md.advance_step(mi, torch.tensor([[11], [12]]), block_size=16, num_seqs=2, num_queries=2)
    assert md.seq_lens == [33, 5] and md.seq_lens_tensor.tolist() == [33, 5] and md.max_decode_seq_len == 33
    assert md.slot_mapping.tolist() == [8 * 16 + 0, 9 * 16 + 4]     # first sequence moved into its next block
    assert mi.input_tokens.tolist() == [11, 12] and mi.input_positions.tolist() == [32, 4]


# ---------------------------------------------------------------------------- GLA slots
def test_gla_slot_manager_assigns_releases_and_forks():
    from spikingbrain_7b_b200.gla_slots import GLACacheManager, GLACacheParams
    mgr = GLACacheManager(torch.float32, (2, 4, 3, 8, 8), device="cpu")
    cache, idx = mgr.current_run_tensors({"a": [0], "b": [1]})
    assert cache.shape == (2, 4, 3, 8, 8) and idx.dtype == torch.int64 and len(set(idx.tolist())) == 2
    sa = int(idx[0])
    cache[:, sa] = 7.0
    _, idx2 = mgr.current_run_tensors({"a": [0, 5], "b": [1]}, pad_to=5)      # "a" forks a second sequence
    assert idx2.tolist()[0] == sa and idx2.tolist()[3:] == [-1, -1]
    fork = idx2.tolist()[1]
    assert torch.equal(cache[:, fork], cache[:, sa])            # the fork starts from its sibling's state
    _, idx3 = mgr.current_run_tensors({"c": [2]}, finished_requests_ids=["a"])
    assert int(idx3[0]) in (sa, fork) and cache[:, int(idx3[0])].abs().sum() == 0   # reused slot comes back zeroed
    p = GLACacheParams(cache, idx3).at_layer_idx(1)
    assert p.gla_cache.shape == (4, 3, 8, 8) and p.state_indices_tensor is idx3
    with pytest.raises(ValueError):
        GLACacheManager(torch.bfloat16, (2, 4, 3, 8, 8), device="cpu")
    with pytest.raises(RuntimeError):
        mgr.current_run_tensors({"d": [0], "e": [0], "f": [0], "g": [0]})    # more sequences than slots


# ----------------------------------------------------------------------------- HF cache
def test_hf_cache_surface_without_gpu():
    import transformers
    from spikingbrain_7b_b200.hf_cache import Cache
    c = Cache()
    assert isinstance(c, transformers.cache_utils.Cache)
    assert len(c) == 0 and c.get_seq_length() == 0 and c.get_max_length() is None and list(c) == []
    with pytest.raises(KeyError):
        c[0]
    rs = torch.zeros(2, 4, 8, 8)
    st = c.update(recurrent_state=rs, layer_idx=0, offset=5)
    assert st["recurrent_state"] is rs and st["attn_state"] is None and c.get_seq_length() == 5
    assert c.get_seq_length(1) == 0                              # layer 1 has no entry yet
    rs2 = torch.ones(2, 4, 8, 8)
    c.update(recurrent_state=rs2, layer_idx=0, offset=1)
    assert c[0]["recurrent_state"] is rs2 and c.get_seq_length() == 6
    with pytest.raises(ValueError):
        c.update(attn_state=[rs, rs], layer_idx=1, cache_kwargs={"window_size": 4})
    with pytest.raises(RuntimeError):                           # K/V must live on the GPU
        c.update(attn_state=(torch.zeros(1, 1, 2, 64), torch.zeros(1, 1, 2, 64)), layer_idx=1,
                 cache_kwargs={"window_size": 4})
    legacy = c.to_legacy_cache()
    assert isinstance(legacy, tuple) and legacy[0]["recurrent_state"] is rs2
    c2 = Cache.from_legacy_cache(legacy, seen_tokens=6)
    assert len(c2) == 1 and c2.get_seq_length() == 6 and c2[0]["recurrent_state"] is rs2


@pytest.mark.parametrize("name", ["bf16_d128_theta1e6", "bf16_d128_theta1e4", "f32_d64_theta1e4"])
def test_cos_sin_table_rows_equal_reference_rotary_embedding(sb, name):
    """ops.build_cos_sin_cache (the vLLM-side table layout: cos half | sin half) holds, row by row,
    the cos / sin the reference's HF RotaryEmbedding returns for that position (rope.npz)."""
    import numpy as np
    from spikingbrain_7b_b200 import ops
    from tests.test_oracle_golden import GOLD, ROPE_POSITIONS, rope_case
    gold = np.load(os.path.join(GOLD, "rope.npz"))
    (H, kvh, D, base, dtype), _, _, want = rope_case(gold, name)
    table = ops.build_cos_sin_cache(D, 131072, base, dtype, device="cpu")
    assert table.shape == (131072, D) and table.dtype == dtype
    rows = table[torch.tensor(ROPE_POSITIONS)]
    assert torch.equal(rows[:, :D // 2], want["cos"][:, :D // 2])
    assert torch.equal(rows[:, D // 2:], want["sin"][:, :D // 2])


# ------------------------------------------------------- CPU model of the device planner
def test_step_planner_model_agrees_with_host_manager_and_window_rule():
    """The planner model (FIFO ring) and the host block manager (LIFO pool) hand out different
    ids but must agree on everything the window rule fixes: lengths, which logical blocks are
    live, one slot per token inside the right logical block; and no id is ever owned twice."""
    from spikingbrain_7b_b200.block_pool import SlidingWindowBlockManager
    B, bs, wl, max_blocks, nb = 5, 16, 40, 64, 40
    ref = ref_ops.StepPlannerRef(nb, bs, B, max_blocks, wl)
    mgr = SlidingWindowBlockManager(nb, bs, wl, B, max_blocks)
    for r in range(B):
        mgr.admit(r)
    steps = [[33, 1, 64, 17, 48]] + [[1] * B] * 70 + [[16, 1, 1, 5, 1]] + [[1] * B] * 10
    for n_new in steps:
        want = ref.plan(n_new)
        plan = mgr.advance(np.array(n_new, dtype=np.int64), pad_inactive=False)
        assert ref.lens == mgr.lens.tolist() == plan.seq_lens.tolist()
        assert want["query_start_loc"] == plan.query_start_loc.tolist()
        live_ref = [[j for j, x in enumerate(row) if x >= 0] for row in ref.table]
        live_mgr = [[j for j, x in enumerate(row) if x >= 0] for row in mgr.table.tolist()]
        assert live_ref == live_mgr
        for t, (slot, pos) in enumerate(zip(want["slot_mapping"], want["positions"])):
            b = max(i for i in range(B) if want["query_start_loc"][i] <= t and n_new[i] > 0
                    and want["query_start_loc"][i] + n_new[i] > t)
            assert slot // bs == ref.table[b][pos // bs] and slot % bs == pos % bs
        owned = [x for row in ref.table for x in row if x >= 0]
        assert len(set(owned)) == len(owned) and not set(owned) & set(ref.ring)
        assert len(owned) + len(ref.ring) == nb
        for b in range(B):   # nothing visible was retired, nothing invisible is kept beyond one block
            t0 = ref_ops.first_visible(ref.lens[b], 1, wl)
            assert all(ref.table[b][j] >= 0 for j in range(t0 // bs, (ref.lens[b] - 1) // bs + 1))


def test_step_planner_model_refuses_without_side_effects():
    ref = ref_ops.StepPlannerRef(4, 16, 2, 8, -1)
    for _ in range(32):
        assert ref.plan() is not None
    state = (list(ref.lens), [list(r) for r in ref.table], list(ref.ring))
    assert ref.plan() is None
    assert state == (ref.lens, ref.table, ref.ring)
    held = [x for x in ref.table[1] if x >= 0]
    ref.release([1])
    assert ref.ring == held and ref.lens[1] == 0 and all(x < 0 for x in ref.table[1])
    assert ref.plan([1, 0]) is not None and ref.lens == [33, 0]
