"""Generates the golden fixtures in this directory by running the REFERENCE's own code.

Run it only in a container that holds the reference checkout (read-only):

    python tests/golden/make_golden.py /path/to/SpikingBrain-7B

It executes, on the CPU,
  * hf_7B_model/cache.py `Cache.update` on deterministic K/V streams          -> cache_*.npz
  * hf_7B_model/window_attention_sdpa.py `FlashAttention.forward` with the
    projections replaced by slicers (q/k/v injected, RoPE neutral at position 0)
    on top of that Cache                                                      -> swa_sdpa.npz
  * the Triton kernel of vllm_hymeta/model_for_7B/my_fused_recurrent.py under
    TRITON_INTERPRET=1 (fp32 inputs: the interpreter has no bf16)             -> gla_triton.npz
  * the element-wise neighbours of that kernel in the GLA layer (feature map, gate, repeat_kv,
    rms_norm_ref as g_norm) around the same Triton kernel                     -> gla_fused.npz
  * RotaryEmbedding + apply_rotary_pos_emb of hf_7B_model/window_attention_sdpa.py (the same
    two definitions as in window_attention.py) on bf16 and fp32 tensors       -> rope.npz
  * hf_7B_model GLAswaForCausalLM, two layers, prompt + 32 greedy steps (three third-party
    GPU-only ops swapped for PyTorch, see config1_hf_model)                   -> config1_hf.npz
The fixtures are what the oracle (oracle/ref_ops.py) and the CUDA kernels are pinned to;
the tests never import the reference.
"""
import hashlib
import importlib.util
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"  # must be set before triton is imported

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py /path/to/SpikingBrain-7B")
REF = sys.argv[1]


def load_ref(rel_path, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, rel_path))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def stream_kv(B, kvh, n, D, t_start, salt):
    """Deterministic, all-distinct K/V values: no RNG, so tests rebuild them exactly."""
    b = torch.arange(B).view(B, 1, 1, 1)
    h = torch.arange(kvh).view(1, kvh, 1, 1)
    t = (t_start + torch.arange(n)).view(1, 1, n, 1)
    d = torch.arange(D).view(1, 1, 1, D)
    k = ((b * 7919 + h * 613 + t * 131 + d * 17 + salt) % 8191).float() / 8191.0 - 0.5
    v = ((b * 6151 + h * 389 + t * 97 + d * 29 + salt * 3) % 8179).float() / 8179.0 - 0.5
    return k, v


# ------------------------------------------------------------------ 1. cache streams
def cache_streams():
    cache_mod = load_ref("hf_7B_model/cache.py", "ref_cache")
    cases = {
        # name: (B, kvh, D, window, prefill, [append sizes...])
        "prefill_gt_window": (2, 2, 64, 64, 128, [1] * 32),          # configs[0] shapes
        "prefill_lt_window": (2, 2, 64, 64, 40, [1] * 40),           # grows to exactly W, then rolls
        "prefill_eq_window": (1, 4, 128, 32, 32, [1] * 5),
        "chunks_on_full_window": (2, 2, 64, 64, 64, [16, 16, 1, 16, 64]),
        "single_token_start": (1, 1, 64, 16, 1, [1] * 20),
    }
    out = {}
    for name, (B, kvh, D, W, prefill, appends) in cases.items():
        cache = cache_mod.Cache()
        # layer 0 is a GLA layer (recurrent slot), layer 1 the SWA layer, as in configs[0]
        digests, seen = [], []
        t = 0
        for step, n in enumerate([prefill] + appends):
            rs = torch.full((B, 2, 4, 4), float(step))
            cache.update(recurrent_state=rs, layer_idx=0, offset=n)
            assert cache[0]["recurrent_state"] is rs  # a reference swap, not a copy
            k, v = stream_kv(B, kvh, n, D, t, salt=len(name))
            st = cache.update(attn_state=(k, v), layer_idx=1, offset=n, cache_kwargs={"window_size": W})
            kc, vc = st["attn_state"]
            digests.append(digest(kc) + digest(vc))
            seen.append((cache.get_seq_length(0), cache.get_seq_length(1), kc.shape[-2]))
            t += n
        out[name + "/meta"] = np.array([B, kvh, D, W, prefill] + appends, dtype=np.int64)
        out[name + "/digests"] = np.array(digests)
        out[name + "/seen"] = np.array(seen, dtype=np.int64)
        out[name + "/final_k"] = kc.numpy()
        out[name + "/final_v"] = vc.numpy()
    # behaviours at the edges of what the class supports (hf_7B_model/cache.py:96-107)
    c = cache_mod.Cache()
    k, v = stream_kv(1, 1, 60, 64, 0, 1)
    c.update(attn_state=(k, v), layer_idx=0, offset=60, cache_kwargs={"window_size": 64})
    k, v = stream_kv(1, 1, 8, 64, 60, 1)
    n68 = c.update(attn_state=(k, v), layer_idx=0, offset=8, cache_kwargs={"window_size": 64})["attn_state"][0].shape[-2]
    out["overshoot_len"] = np.array([n68])  # 68: the cat branch overshoots the window and never rolls again
    try:
        c2 = cache_mod.Cache()
        k, v = stream_kv(1, 1, 64, 64, 0, 1)
        c2.update(attn_state=(k, v), layer_idx=0, offset=64, cache_kwargs={"window_size": 64})
        k, v = stream_kv(1, 1, 128, 64, 64, 1)
        c2.update(attn_state=(k, v), layer_idx=0, offset=128, cache_kwargs={"window_size": 64})
        out["oversize_chunk_raises"] = np.array([0])
    except RuntimeError:
        out["oversize_chunk_raises"] = np.array([1])
    try:
        cache_mod.Cache()[0]
        out["getitem_raises_keyerror"] = np.array([0])
    except KeyError:
        out["getitem_raises_keyerror"] = np.array([1])
    np.savez_compressed(os.path.join(HERE, "cache_streams.npz"), **out)
    print("cache_streams.npz", {k: v.shape for k, v in out.items() if k.endswith("seen")})


# ---------------------------------------------------------------- 2. SWA decode (SDPA)
class _Slice(torch.nn.Module):
    def __init__(self, lo, hi):
        super().__init__()
        self.lo, self.hi = lo, hi

    def forward(self, x):
        return x[..., self.lo:self.hi]


def swa_sdpa():
    # the package __init__ pulls in fla-backed modules; load the two files it needs directly
    import types
    pkg = types.ModuleType("hf_7B_model")
    pkg.__path__ = [os.path.join(REF, "hf_7B_model")]
    sys.modules["hf_7B_model"] = pkg
    load_ref("hf_7B_model/cache.py", "hf_7B_model.cache")
    wa = load_ref("hf_7B_model/window_attention_sdpa.py", "hf_7B_model.window_attention_sdpa")
    cache_mod = sys.modules["hf_7B_model.cache"]
    out = {}
    for name, (B, H, kvh, D, W, prefill, steps) in {
        "g7": (1, 14, 2, 128, 64, 100, 6),       # 7 query heads per kv head, window crossed
        "short": (1, 4, 4, 128, 64, 5, 4),      # fewer tokens than the window
    }.items():
        torch.manual_seed(1234)
        attn = wa.FlashAttention(hidden_size=H * D, num_heads=H, num_key_value_heads=kvh,
                                 sliding_window=W, layer_idx=0)
        attn.q_proj = _Slice(0, H * D)
        attn.k_proj = _Slice(H * D, (H + kvh) * D)
        attn.v_proj = _Slice((H + kvh) * D, (H + 2 * kvh) * D)
        attn.o_proj = torch.nn.Identity()
        attn.eval()
        cache = cache_mod.Cache()
        total = prefill + steps
        x = (torch.randn(B, total, (H + 2 * kvh) * D) / D ** 0.5).bfloat16().float()  # bf16-representable
        outs = []
        with torch.no_grad():
            for (lo, hi) in [(0, prefill)] + [(prefill + i, prefill + i + 1) for i in range(steps)]:
                pos = torch.zeros(B, hi - lo, dtype=torch.long)  # cos=1, sin=0: RoPE is the identity
                o, _, _ = attn(x[:, lo:hi], position_ids=pos, past_key_values=cache, use_cache=True)
                # the reference counts tokens on layer 0 only; this one-layer harness IS layer 0
                outs.append(o)
        out[name + "/meta"] = np.array([B, H, kvh, D, W, prefill, steps], dtype=np.int64)
        out[name + "/x_bf16"] = x.bfloat16().view(torch.int16).numpy()
        out[name + "/prefill_out_tail"] = outs[0][:, -4:].numpy()
        out[name + "/decode_out"] = torch.cat(outs[1:], dim=1).numpy()
    np.savez_compressed(os.path.join(HERE, "swa_sdpa.npz"), **out)
    print("swa_sdpa.npz", {k: v.shape for k, v in out.items()})


# ------------------------------------------------------------------- 3. GLA (Triton)
def golden_state(slots, H, D):
    """Deterministic fp32 start state (no RNG): values in [-1, 1) with a different pattern
    per slot, head, row and column."""
    i = torch.arange(slots * H * D * D, dtype=torch.int64)
    return (((i * 2654435761) % 1000003).double() / 500001.5 - 1.0).float().view(slots, H, D, D)


def gla_triton():
    mfr = load_ref("vllm_hymeta/model_for_7B/my_fused_recurrent.py", "ref_mfr")
    out = {}
    for name, (B, H, D, slots, dtype) in {
        "f32_d128": (3, 2, 128, 4, torch.float32),
        "f32_d64": (2, 8, 64, 2, torch.float32),
        "f32_d128_g7": (1, 7, 128, 2, torch.float32),
    }.items():
        g = torch.Generator().manual_seed(77)
        q = torch.relu(torch.randn(B, H, 1, D, generator=g)).to(dtype)
        k = torch.relu(torch.randn(B, H, 1, D, generator=g)).to(dtype)
        v = torch.randn(B, H, 1, D, generator=g).to(dtype)
        gk = (torch.nn.functional.logsigmoid(torch.randn(B, H, 1, D, generator=g)) / 16).to(dtype)
        state = golden_state(slots, H, D)
        slot = torch.randperm(slots, generator=g)[:B].to(torch.int64)
        if B > 2:
            slot[1] = -1
        state0 = state.clone()
        o = torch.zeros_like(q)
        steps_out = []
        for _ in range(2):  # two chained steps on the same inputs: the state carries
            mfr.my_fused_recurrent_fwd_kernel[(B, H, D // 64)](
                q, k, v, gk, o, D, state, slot, D ** -0.5, q.stride(0), q.stride(1),
                state.stride(0), state.stride(1), state.stride(2), state.stride(3), 64)
            steps_out.append(o.float().clone())
        out[name + "/meta"] = np.array([B, H, D, slots, int(dtype == torch.bfloat16)], dtype=np.int64)
        for nm, t in (("q", q), ("k", k), ("v", v), ("g", gk)):
            out[f"{name}/{nm}"] = t.float().squeeze(2).numpy()
        out[name + "/slot"] = slot.numpy()
        out[name + "/state2"] = state.numpy()  # state0 is golden_state(): rebuilt by the tests
        assert torch.equal(state[[i for i in range(slots) if i not in slot.tolist()]],
                           state0[[i for i in range(slots) if i not in slot.tolist()]])
        out[name + "/out1"] = steps_out[0].squeeze(2).numpy()
        out[name + "/out2"] = steps_out[1].squeeze(2).numpy()
    np.savez_compressed(os.path.join(HERE, "gla_triton.npz"), **out)
    print("gla_triton.npz", {k: v.shape for k, v in out.items() if k.endswith("state2")})


def det_unit(shape, salt):
    """Deterministic values in [-1, 1) (no RNG); tests rebuild them with tests.helpers.det_unit."""
    n = 1
    for d in shape:
        n *= d
    i = torch.arange(n, dtype=torch.int64) + salt * 1000003
    return (((i * 2246822519) % 999983).double() / 499991.5 - 1.0).float().view(*shape)


def gla_fused():
    """The decode branch of the GLA layer around its kernel, in the reference's order
    (vllm_hymeta/model_for_7B/gla_attention.py:250-267, :232-233): relu(q), relu(k),
    logsigmoid(gk)/16, repeat_kv of k, v, gk, the Triton step kernel, then g_norm, for which the
    reference's own rms_norm_ref (hf_7B_model/layernorm.py:39-52) stands in for the vLLM layer.
    fp32 end to end (the interpreter has no bf16); the bf16 gate expression is recorded separately."""
    mfr = load_ref("vllm_hymeta/model_for_7B/my_fused_recurrent.py", "ref_mfr")
    sys.path.insert(0, REF)
    for k in [k for k in sys.modules if k.startswith("hf_7B_model")]:
        del sys.modules[k]
    lnmod = load_ref("hf_7B_model/layernorm.py", "ref_layernorm")
    out = {}
    for ci, (name, (B, H, Hkv, D, slots)) in enumerate({
        "d128_h2_kv1": (3, 2, 1, 128, 3),
        "d64_h8_kv8": (2, 8, 8, 64, 3),
    }.items()):
        qp = det_unit((B, H, D), 11 + ci) * 2.0
        kp = det_unit((B, Hkv, D), 12 + ci) * 2.0
        v = det_unit((B, Hkv, D), 13 + ci)
        gl = det_unit((B, Hkv, D), 14 + ci) * 4.0
        w = 1.0 + 0.5 * det_unit((D,), 15 + ci)
        rep = H // Hkv
        q = torch.relu(qp)
        k = torch.relu(kp)
        gk = torch.nn.functional.logsigmoid(gl) / 16
        rk = lambda t: t.repeat_interleave(rep, dim=1).unsqueeze(2).contiguous()
        q4, k4, v4, g4 = q.unsqueeze(2).contiguous(), rk(k), rk(v), rk(gk)
        state = golden_state(slots, H, D)
        slot = torch.arange(B, dtype=torch.int64)
        if B > 2:
            slot[1] = -1
        o = torch.zeros_like(q4)
        for step in range(2):
            mfr.my_fused_recurrent_fwd_kernel[(B, H, D // 64)](
                q4, k4, v4, g4, o, D, state, slot, D ** -0.5, q4.stride(0), q4.stride(1),
                state.stride(0), state.stride(1), state.stride(2), state.stride(3), 64)
            out[f"{name}/out{step + 1}"] = lnmod.rms_norm_ref(o.squeeze(2), w, None, eps=1e-5).numpy()
        out[name + "/meta"] = np.array([B, H, Hkv, D, slots, 11 + ci], dtype=np.int64)
        out[name + "/slot"] = slot.numpy()
        out[name + "/state2"] = state.numpy()
    # the gate expression on a bf16 tensor, as the layer evaluates it when the model runs in bf16
    gl16 = (det_unit((4096,), 21) * 12.0).to(torch.bfloat16)
    out["gate_bf16/g"] = (torch.nn.functional.logsigmoid(gl16) / 16).float().numpy()
    np.savez_compressed(os.path.join(HERE, "gla_fused.npz"), **out)
    print("gla_fused.npz", sorted(out))


ROPE_POSITIONS = [0, 1, 2, 17, 255, 4095, 4096, 8191, 65535, 131071]


def rope():
    """cos/sin and rotated q, k as the reference's HF attention computes them
    (hf_7B_model/window_attention.py:23-80 == window_attention_sdpa.py:23-80, used at :161-162)."""
    import types
    pkg = types.ModuleType("hf_7B_model")
    pkg.__path__ = [os.path.join(REF, "hf_7B_model")]
    sys.modules["hf_7B_model"] = pkg
    load_ref("hf_7B_model/cache.py", "hf_7B_model.cache")
    wa = load_ref("hf_7B_model/window_attention_sdpa.py", "hf_7B_model.window_attention_sdpa")
    out = {}
    for ci, (name, (H, kvh, D, base, dtype)) in enumerate({
        "bf16_d128_theta1e6": (4, 2, 128, 1000000.0, torch.bfloat16),
        "bf16_d128_theta1e4": (3, 1, 128, 10000.0, torch.bfloat16),
        "f32_d64_theta1e4": (4, 2, 64, 10000.0, torch.float32),
    }.items()):
        T = len(ROPE_POSITIONS)
        q = (det_unit((1, H, T, D), 31 + ci) * 3.0).to(dtype)
        k = (det_unit((1, kvh, T, D), 41 + ci) * 3.0).to(dtype)
        pos = torch.tensor([ROPE_POSITIONS], dtype=torch.long)
        emb = wa.RotaryEmbedding(D, max_position_embeddings=131072, base=base)
        cos, sin = emb(q, pos)
        qe, ke = wa.apply_rotary_pos_emb(q, k, cos, sin)
        assert qe.dtype == dtype and cos.dtype == dtype
        store = (lambda t: t.view(torch.int16).numpy()) if dtype == torch.bfloat16 else (lambda t: t.numpy())
        out[name + "/meta"] = np.array([H, kvh, D, int(base), int(dtype == torch.bfloat16), 31 + ci], dtype=np.int64)
        out[name + "/cos"] = store(cos[0].contiguous())          # [T, D] (the two halves are equal)
        out[name + "/sin"] = store(sin[0].contiguous())
        out[name + "/q"] = store(qe[0].transpose(0, 1).contiguous())   # token-major [T, H, D]
        out[name + "/k"] = store(ke[0].transpose(0, 1).contiguous())
    np.savez_compressed(os.path.join(HERE, "rope.npz"), **out)
    print("rope.npz", {k: v.shape for k, v in out.items()})


# ------------------------------------------------------- 4. the two-layer HF model (configs[0])
def config1_hf_model():
    """The reference GLAswaForCausalLM (2 layers: GLA then sliding window, hidden 512, 8/2 heads,
    head_dim 64, window 64, fp32) run on the CPU: batch 2, a 128-token prompt of uniform random ids
    over a 32k vocabulary, 32 greedy steps. Three GPU-only third-party pieces are swapped for PyTorch
    equivalents (nothing of the reference itself is changed):
      fla RMSNorm                  -> rms_norm_ref, the reference's own definition (hf_7B_model/layernorm.py:39-52)
      fla fused_recurrent/chunk GLA -> the recurrence in a loop (fp32, head-first layout, scale D^-1/2)
      flash_attn varlen + pad_input -> softmax attention with the same bottom-right causal window (W, 0)
    Weights are overwritten parameter by parameter with tests.helpers.det_param so that the GPU-side
    harness can rebuild them."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from tests.helpers import det_param
    for k in [k for k in sys.modules if k.startswith("hf_7B_model")]:
        del sys.modules[k]
    sys.path.insert(0, REF)
    import hf_7B_model.modeling_gla_swa as M
    import hf_7B_model.gla_attention as GA
    import hf_7B_model.window_attention as WA
    from hf_7B_model.layernorm import rms_norm_ref
    from hf_7B_model.configuration_gla_swa import GLAswaConfig

    class TorchRMSNorm(torch.nn.Module):
        def __init__(self, hidden_size, elementwise_affine=True, eps=1e-5):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.ones(hidden_size))
            self.eps = eps

        def forward(self, x, residual=None, prenorm=False, residual_in_fp32=False):
            return rms_norm_ref(x, self.weight, None, residual=residual, eps=self.eps, prenorm=prenorm)

    def torch_gla(q, k, v, gk, initial_state=None, output_final_state=False, scale=None, **kw):
        B, H, T, D = q.shape
        S = torch.zeros(B, H, D, v.shape[-1]) if initial_state is None else initial_state.float().clone()
        scale = D ** -0.5 if scale is None else scale
        out = []
        for t in range(T):
            S = torch.exp(gk[:, :, t].float())[..., None] * S + k[:, :, t].float()[..., None] * v[:, :, t].float()[..., None, :]
            out.append(torch.einsum("bhk,bhkv->bhv", q[:, :, t].float() * scale, S))
        return torch.stack(out, 2).to(q.dtype), (S if output_final_state else None)

    def varlen_attn(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, dropout_p=0.0,
                    softmax_scale=None, causal=True, window_size=(-1, -1)):
        outs = []
        for b in range(len(cu_seqlens_q) - 1):
            qb = q[cu_seqlens_q[b]:cu_seqlens_q[b + 1]].transpose(0, 1)
            kb = k[cu_seqlens_k[b]:cu_seqlens_k[b + 1]].transpose(0, 1)
            vb = v[cu_seqlens_k[b]:cu_seqlens_k[b + 1]].transpose(0, 1)
            sq, sk = qb.shape[1], kb.shape[1]
            qi = torch.arange(sq)[:, None] + (sk - sq)
            kj = torch.arange(sk)[None, :]
            mask = (kj <= qi + window_size[1]) & (kj >= qi - window_size[0])
            s = (qb @ kb.transpose(1, 2)) * softmax_scale
            outs.append((torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ vb).transpose(0, 1))
        return torch.cat(outs, 0)

    def pad_input(x, indices, batch, seqlen):
        out = torch.zeros(batch * seqlen, *x.shape[1:], dtype=x.dtype)
        out[indices] = x
        return out.view(batch, seqlen, *x.shape[1:])

    M.RMSNorm = GA.RMSNorm = TorchRMSNorm
    GA.fused_recurrent_gla = GA.chunk_gla = GA.fused_chunk_gla = torch_gla
    WA.flash_attn_varlen_func, WA.pad_input, WA.unpad_input = varlen_attn, pad_input, None

    torch.manual_seed(0)
    cfg = GLAswaConfig(vocab_size=32000, hidden_size=512, num_hidden_layers=2, num_attention_heads=8,
                       num_key_value_heads=2, sliding_window=64, intermediate_size=1024, fuse_cross_entropy=False)
    model = M.GLAswaForCausalLM(cfg).eval()
    names_shapes = []
    with torch.no_grad():
        for name, p in model.named_parameters():
            p.copy_(det_param(name, p.shape))
            names_shapes.append((name, tuple(p.shape)))
    ids = torch.randint(0, 32000, (2, 128))
    probe = torch.arange(0, 32000, 500)          # 64 vocabulary entries whose logits are recorded
    logits_probe, tokens, seen = [], [], []
    cache = None
    cur = ids
    with torch.no_grad():
        for step in range(33):
            out = model(input_ids=cur, past_key_values=cache, use_cache=True)
            cache = out.past_key_values
            last = out.logits[:, -1]
            logits_probe.append(last[:, probe])
            nxt = last.argmax(-1)
            tokens.append(nxt)
            seen.append([cache.get_seq_length(0), cache.get_seq_length(1), cache[1]["attn_state"][0].shape[-2]])
            cur = nxt[:, None]
    assert type(cache).__module__ == "hf_7B_model.cache"
    res = {
        "input_ids": ids.numpy(), "probe": probe.numpy(), "logits_probe": torch.stack(logits_probe).numpy(),
        "tokens": torch.stack(tokens, 1).numpy(), "seen": np.array(seen, dtype=np.int64),
        "final_k": cache[1]["attn_state"][0].numpy(), "final_v": cache[1]["attn_state"][1].numpy(),
        "final_state": cache[0]["recurrent_state"].numpy(),
        "param_names": np.array([n for n, _ in names_shapes]),
        "param_shapes": np.array([",".join(map(str, s)) for _, s in names_shapes]),
    }
    np.savez_compressed(os.path.join(HERE, "config1_hf.npz"), **res)
    print("config1_hf.npz tokens", res["tokens"][:, :8].tolist(), "seen", seen[0], seen[-1])


if __name__ == "__main__":
    config1_hf_model()
    cache_streams()
    swa_sdpa()
    gla_triton()
    gla_fused()
    rope()
