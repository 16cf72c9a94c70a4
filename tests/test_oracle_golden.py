"""CPU: the oracle (oracle/ref_ops.py) against fixtures produced by the reference's own code
(tests/golden/make_golden.py). These pins are what lets the oracle judge the CUDA kernels."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import ref_ops

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def stream_kv(B, kvh, n, D, t_start, salt):
    """Same closed-form K/V stream as make_golden.py (no RNG involved)."""
    b = torch.arange(B).view(B, 1, 1, 1)
    h = torch.arange(kvh).view(1, kvh, 1, 1)
    t = (t_start + torch.arange(n)).view(1, 1, n, 1)
    d = torch.arange(D).view(1, 1, 1, D)
    k = ((b * 7919 + h * 613 + t * 131 + d * 17 + salt) % 8191).float() / 8191.0 - 0.5
    v = ((b * 6151 + h * 389 + t * 97 + d * 29 + salt * 3) % 8179).float() / 8179.0 - 0.5
    return k, v


def golden_state(slots, H, D):
    i = torch.arange(slots * H * D * D, dtype=torch.int64)
    return (((i * 2654435761) % 1000003).double() / 500001.5 - 1.0).float().view(slots, H, D, D)


def digest(t):
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


CACHE_CASES = ["prefill_gt_window", "prefill_lt_window", "prefill_eq_window", "chunks_on_full_window",
               "single_token_start"]


@pytest.fixture(scope="module")
def cache_gold():
    return np.load(os.path.join(GOLD, "cache_streams.npz"))


@pytest.mark.parametrize("name", CACHE_CASES)
def test_ref_window_cache_matches_reference_stream(cache_gold, name):
    """Every step of the K/V stream: cached tensors bit-identical to the reference class
    (hf_7B_model/cache.py), and the same get_seq_length on both layers."""
    meta = cache_gold[name + "/meta"].tolist()
    B, kvh, D, W, prefill = meta[:5]
    appends = meta[5:]
    cache = ref_ops.RefWindowCache()
    t = 0
    for step, n in enumerate([prefill] + appends):
        rs = torch.full((B, 2, 4, 4), float(step))
        cache.update(recurrent_state=rs, layer_idx=0, offset=n)
        assert cache[0]["recurrent_state"] is rs
        k, v = stream_kv(B, kvh, n, D, t, salt=len(name))
        kc, vc = cache.update(attn_state=(k, v), layer_idx=1, offset=n,
                              cache_kwargs={"window_size": W})["attn_state"]
        assert digest(kc) + digest(vc) == str(cache_gold[name + "/digests"][step]), f"step {step}"
        assert [cache.get_seq_length(0), cache.get_seq_length(1), kc.shape[-2]] == \
            cache_gold[name + "/seen"][step].tolist()
        t += n
    assert torch.equal(kc, torch.from_numpy(cache_gold[name + "/final_k"]))
    assert torch.equal(vc, torch.from_numpy(cache_gold[name + "/final_v"]))


def test_reference_edge_behaviour_recorded(cache_gold):
    """What the reference class does outside its working range, as recorded from it."""
    assert cache_gold["overshoot_len"].tolist() == [68]       # 60 cached + 8 new, window 64: never trims again
    assert cache_gold["oversize_chunk_raises"].tolist() == [1]  # 128 tokens onto a full 64-window: RuntimeError
    assert cache_gold["getitem_raises_keyerror"].tolist() == [1]
    c = ref_ops.RefWindowCache()
    k, v = stream_kv(1, 1, 60, 64, 0, 1)
    c.update(attn_state=(k, v), layer_idx=0, offset=60, cache_kwargs={"window_size": 64})
    k, v = stream_kv(1, 1, 8, 64, 60, 1)
    assert c.update(attn_state=(k, v), layer_idx=0, offset=8,
                    cache_kwargs={"window_size": 64})["attn_state"][0].shape[-2] == 68
    with pytest.raises(KeyError):
        ref_ops.RefWindowCache()[0]


@pytest.mark.parametrize("name", ["g7", "short"])
def test_swa_oracle_matches_reference_sdpa_layer(name):
    """swa_decode_ref on the window the cache holds == the reference's SDPA attention layer
    (hf_7B_model/window_attention_sdpa.py) run on the same injected q/k/v, decode steps."""
    gold = np.load(os.path.join(GOLD, "swa_sdpa.npz"))
    B, H, kvh, D, W, prefill, steps = gold[name + "/meta"].tolist()
    x = torch.from_numpy(gold[name + "/x_bf16"]).view(torch.bfloat16).float()
    q = x[..., :H * D].view(B, -1, H, D)
    k = x[..., H * D:(H + kvh) * D].view(B, -1, kvh, D)
    v = x[..., (H + kvh) * D:].view(B, -1, kvh, D)
    ref_out = torch.from_numpy(gold[name + "/decode_out"]).view(B, steps, H, D)
    for s in range(steps):
        pos = prefill + s
        lo = max(0, pos + 1 - W)   # the layer's mask keeps W keys, the query's own included
        for b in range(B):
            kw = k[b, lo:pos + 1].transpose(0, 1)
            vw = v[b, lo:pos + 1].transpose(0, 1)
            o = ref_ops.swa_decode_ref(q[b, pos], kw, vw, D ** -0.5)
            assert torch.allclose(o, ref_out[b, s], rtol=1e-5, atol=1e-6), f"step {s}"
            # the explicit mask over a longer key run gives the same answer
            o2 = ref_ops.swa_decode_ref(q[b, pos], k[b, :pos + 1].transpose(0, 1),
                                        v[b, :pos + 1].transpose(0, 1), D ** -0.5, window=W)
            assert torch.allclose(o2, ref_out[b, s], rtol=1e-5, atol=1e-6)


def test_swa_paged_oracle_equals_dense_oracle():
    """The paged form (block-table gather + window rule) reduces to the dense form."""
    from tests.helpers import make_paged_kv
    lens, wl, kvh, D, bs, H = [70, 5, 64, 65], 15, 2, 128, 16, 14
    kv, table, nb = make_paged_kv(lens, wl, kvh, D, bs, seed=3)
    g = torch.Generator().manual_seed(4)
    q = torch.randn(len(lens), H, D, generator=g).bfloat16()
    out = ref_ops.swa_paged_decode_ref(q, kv[0], kv[1], table, lens, wl, D ** -0.5)
    for b, L in enumerate(lens):
        toks = torch.arange(max(0, L - 1 - wl), L)
        kd = kv[0][table[b][toks // bs].long(), toks % bs].transpose(0, 1)
        vd = kv[1][table[b][toks // bs].long(), toks % bs].transpose(0, 1)
        assert torch.equal(out[b], ref_ops.swa_decode_ref(q[b], kd, vd, D ** -0.5))
        assert torch.isfinite(out[b]).all()


@pytest.mark.parametrize("name", ["f32_d128", "f32_d64", "f32_d128_g7"])
def test_gla_oracle_matches_reference_triton_kernel(name):
    """gla_step_ref == my_fused_recurrent_fwd_kernel (vllm_hymeta/model_for_7B/
    my_fused_recurrent.py) run under the Triton interpreter: two chained steps, a slot of -1,
    untouched slots. fp32 in and out, so only summation order differs."""
    gold = np.load(os.path.join(GOLD, "gla_triton.npz"))
    B, H, D, slots, _ = gold[name + "/meta"].tolist()
    q, k, v, g = (torch.from_numpy(gold[f"{name}/{n}"]) for n in "qkvg")
    slot = torch.from_numpy(gold[name + "/slot"])
    state = golden_state(slots, H, D)
    o1 = ref_ops.gla_step_ref(q, k, v, g, state, slot)
    o2 = ref_ops.gla_step_ref(q, k, v, g, state, slot)
    live = slot >= 0
    tol = dict(rtol=1e-5, atol=1e-5)
    assert torch.allclose(o1[live], torch.from_numpy(gold[name + "/out1"])[live], **tol)
    assert torch.allclose(o2[live], torch.from_numpy(gold[name + "/out2"])[live], **tol)
    assert torch.allclose(state, torch.from_numpy(gold[name + "/state2"]), **tol)
    untouched = [s for s in range(slots) if s not in slot.tolist()]
    assert torch.equal(state[untouched], golden_state(slots, H, D)[untouched])


def fused_case(gold, name):
    """Rebuilds the inputs of one gla_fused.npz case (formulas of the generator script)."""
    from tests.helpers import det_unit
    B, H, Hkv, D, slots, salt = gold[name + "/meta"].tolist()
    qp = det_unit((B, H, D), salt) * 2.0
    kp = det_unit((B, Hkv, D), salt + 1) * 2.0
    v = det_unit((B, Hkv, D), salt + 2)
    gl = det_unit((B, Hkv, D), salt + 3) * 4.0
    w = 1.0 + 0.5 * det_unit((D,), salt + 4)
    return (B, H, Hkv, D, slots), (qp, kp, v, gl, w), torch.from_numpy(gold[name + "/slot"])


@pytest.mark.parametrize("name", ["d128_h2_kv1", "d64_h8_kv8"])
def test_gla_layer_oracle_matches_reference_layer_pieces(name):
    """gla_layer_step_ref == relu / logsigmoid-gate / repeat_kv / Triton step kernel / rms_norm_ref
    chained by the generator script in the reference layer's order, two steps, a slot of -1."""
    gold = np.load(os.path.join(GOLD, "gla_fused.npz"))
    (B, H, Hkv, D, slots), (qp, kp, v, gl, w), slot = fused_case(gold, name)
    state = golden_state(slots, H, D)
    live = slot >= 0
    for step in (1, 2):
        o = ref_ops.gla_layer_step_ref(qp, kp, v, gl, state, slot, 16.0, w, 1e-5)
        want = torch.from_numpy(gold[f"{name}/out{step}"])
        assert torch.allclose(o[live], want[live], rtol=2e-5, atol=2e-5)
    assert torch.allclose(state, torch.from_numpy(gold[name + "/state2"]), rtol=1e-5, atol=1e-5)


def test_gate_expression_in_bf16_matches_fixture():
    """logsigmoid(gk) / 16 on a bf16 tensor, bit for bit (gla_prepare_inputs is that expression)."""
    from tests.helpers import det_unit
    gold = np.load(os.path.join(GOLD, "gla_fused.npz"))
    gl16 = (det_unit((4096,), 21) * 12.0).to(torch.bfloat16)
    _, _, g = ref_ops.gla_prepare_inputs(gl16, gl16, gl16, 16.0)
    assert g.dtype == torch.bfloat16
    assert torch.equal(g.float(), torch.from_numpy(gold["gate_bf16/g"]))


ROPE_POSITIONS = [0, 1, 2, 17, 255, 4095, 4096, 8191, 65535, 131071]
ROPE_CASES = ["bf16_d128_theta1e6", "bf16_d128_theta1e4", "f32_d64_theta1e4"]


def rope_case(gold, name):
    """Inputs (rebuilt from the generator's formulas) and reference outputs of one rope.npz case."""
    from tests.helpers import det_unit
    H, kvh, D, base, is_bf16, salt = gold[name + "/meta"].tolist()
    dtype = torch.bfloat16 if is_bf16 else torch.float32
    T = len(ROPE_POSITIONS)
    tm = lambda t: t[0].transpose(0, 1).contiguous()
    q = tm((det_unit((1, H, T, D), salt) * 3.0).to(dtype))
    k = tm((det_unit((1, kvh, T, D), salt + 10) * 3.0).to(dtype))
    load = lambda key: (torch.from_numpy(gold[f"{name}/{key}"]).view(torch.bfloat16) if is_bf16
                        else torch.from_numpy(gold[f"{name}/{key}"]))
    return (H, kvh, D, float(base), dtype), q, k, {n: load(n) for n in ("cos", "sin", "q", "k")}


@pytest.mark.parametrize("name", ROPE_CASES)
def test_rope_oracle_is_bit_exact_with_reference(name):
    """rope_cos_sin_ref / rope_ref == RotaryEmbedding + apply_rotary_pos_emb of the reference, bit
    for bit in bf16 and fp32, positions up to 131071."""
    gold = np.load(os.path.join(GOLD, "rope.npz"))
    (H, kvh, D, base, dtype), q, k, want = rope_case(gold, name)
    cos, sin = ref_ops.rope_cos_sin_ref(torch.tensor(ROPE_POSITIONS), D, base, dtype)
    assert torch.equal(cos, want["cos"]) and torch.equal(sin, want["sin"])
    assert torch.equal(ref_ops.rope_ref(q, cos, sin), want["q"])
    assert torch.equal(ref_ops.rope_ref(k, cos, sin), want["k"])


def test_gla_oracle_kv_head_sharing_equals_repeated_heads():
    """k, v, g given per kv head == the reference's repeat_kv'ed per-query-head inputs."""
    g = torch.Generator().manual_seed(9)
    B, H, Hkv, D = 2, 8, 2, 64
    q = torch.relu(torch.randn(B, H, D, generator=g))
    k, v, gk = (torch.randn(B, Hkv, D, generator=g) for _ in range(3))
    gk = torch.nn.functional.logsigmoid(gk) / 16
    s1, s2 = torch.randn(B, H, D, D, generator=g), None
    s2 = s1.clone()
    o1 = ref_ops.gla_step_ref(q, k, v, gk, s1)
    rep = lambda t: ref_ops.repeat_kv(t.unsqueeze(2), H // Hkv).squeeze(2)
    o2 = ref_ops.gla_step_ref(q, rep(k), rep(v), rep(gk), s2)
    assert torch.equal(o1, o2) and torch.equal(s1, s2)


def test_paged_append_and_retire_oracle():
    kc = torch.zeros(4, 16, 1, 8)
    vc = torch.zeros(4, 16, 1, 8)
    key = torch.arange(3 * 8, dtype=torch.float32).view(3, 1, 8)
    ref_ops.paged_append(key, -key, kc, vc, torch.tensor([17, -1, 63]))
    assert torch.equal(kc[1, 1], key[0]) and torch.equal(vc[3, 15], -key[2]) and kc.sum() == key[0].sum() + key[2].sum()
    table = torch.arange(8, dtype=torch.int32).view(1, 8)
    assert ref_ops.retire_blocks(table, [100], [1], 31, 16) == [[0, 1, 2, 3]]   # t0 = 68 -> blocks < 4
    assert table.tolist() == [[-1, -1, -1, -1, 4, 5, 6, 7]]
    assert ref_ops.retire_blocks(table, [101], [1], 31, 16) == [[]]
    assert ref_ops.retire_blocks(table, [200], [1], -1, 16) == [[]]            # no window: nothing retires
