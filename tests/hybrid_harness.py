"""A small GLA + sliding-window decoder written for the tests: the dense parts (embedding, norms,
projections, rotary, GLU) in plain PyTorch, the cache path through the package's `Cache`
(paged K/V append + window gather, in-place GLA state step). It follows the layer arithmetic of
hf_7B_model/modeling_gla_swa.py:93-125, gla_attention.py:129-171 and window_attention.py:153-220 so
that its logits can be compared with the reference model's (fixture config1_hf.npz)."""
import math

import torch
import torch.nn.functional as F

from tests.helpers import det_param


def rms(x, w, eps):
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * w


class HybridHarness:
    def __init__(self, names_shapes, device, vocab=32000, hidden=512, layers=2, heads=8, kv_heads=2,
                 window=64, eps=1e-6, gla_eps=1e-5, rope_theta=1000000.0):
        self.p = {n: det_param(n, s).to(device) for n, s in names_shapes}
        self.dev, self.H, self.KVH, self.D, self.W = device, heads, kv_heads, hidden // heads, window
        self.layers, self.eps, self.gla_eps, self.theta = layers, eps, gla_eps, rope_theta

    def lin(self, x, prefix):
        return F.linear(x, self.p[prefix + ".weight"], self.p.get(prefix + ".bias"))

    def rope(self, x, pos):            # x [B, h, T, D], pos [T]
        D = self.D
        inv = 1.0 / (self.theta ** (torch.arange(0, D, 2, device=self.dev).float() / D))
        f = pos.float()[:, None] * inv[None, :]
        emb = torch.cat([f, f], -1)
        cos, sin = emb.cos()[None, None], emb.sin()[None, None]
        x1, x2 = x[..., :D // 2], x[..., D // 2:]
        return x * cos + torch.cat([-x2, x1], -1) * sin

    def forward(self, ids, cache):
        """ids [B, T] -> logits of the last position [B, vocab]; `cache` is updated in place."""
        B, T = ids.shape
        H, KVH, D, W = self.H, self.KVH, self.D, self.W
        past = cache.get_seq_length()
        pos = torch.arange(past, past + T, device=self.dev)
        x = self.p["model.embeddings.weight"][ids]
        for i in range(self.layers):
            pre = f"model.layers.{i}."
            residual = x
            h = rms(x, self.p[pre + "attn_norm.weight"], self.eps)
            if i % 2 == 0:                                     # gated linear attention
                q = torch.relu(self.lin(h, pre + "attn.q_proj")).view(B, T, H, D)
                k = torch.relu(self.lin(h, pre + "attn.k_proj")).view(B, T, KVH, D)
                v = self.lin(h, pre + "attn.v_proj").view(B, T, KVH, D)
                gk = self.lin(self.lin(h, pre + "attn.gk_proj.0"), pre + "attn.gk_proj.1").view(B, T, KVH, D)
                g = F.logsigmoid(gk) / 16
                if T > 1 and hasattr(cache, "gla_chunk"):      # a prompt: one scan with state carry
                    o = cache.gla_chunk(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), g.transpose(1, 2),
                                        i).transpose(1, 2)
                else:
                    outs = [cache.gla_step(q[:, t].contiguous(), k[:, t].contiguous(), v[:, t].contiguous(),
                                           g[:, t].contiguous(), i) for t in range(T)]
                    o = torch.stack(outs, 1)                   # [B, T, H, D]
                o = rms(o, self.p[pre + "attn.g_norm.weight"], self.gla_eps).reshape(B, T, H * D)
            else:                                              # sliding-window attention
                q = self.rope(self.lin(h, pre + "attn.q_proj").view(B, T, H, D).transpose(1, 2), pos)
                k = self.rope(self.lin(h, pre + "attn.k_proj").view(B, T, KVH, D).transpose(1, 2), pos)
                v = self.lin(h, pre + "attn.v_proj").view(B, T, KVH, D).transpose(1, 2)
                had_content = cache.get_seq_length(i) > 0
                st = cache.update(attn_state=(k.contiguous(), v.contiguous()), layer_idx=i, offset=T,
                                  cache_kwargs={"window_size": W})
                if had_content:
                    k, v = st["attn_state"]                    # gathered through the block table
                k = k.repeat_interleave(H // KVH, 1)
                v = v.repeat_interleave(H // KVH, 1)
                Tk = k.shape[2]
                qi = torch.arange(T, device=self.dev)[:, None] + (Tk - T)
                kj = torch.arange(Tk, device=self.dev)[None, :]
                mask = (kj <= qi) & (kj >= qi - W)             # flash-attn window (W, 0), bottom-right aligned
                s = torch.einsum("bhqd,bhkd->bhqk", q, k) * D ** -0.5
                o = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v
                o = o.transpose(1, 2).reshape(B, T, H * D)
            a = self.lin(o, pre + "attn.o_proj")
            residual = a + residual
            h = rms(residual, self.p[pre + "mlp_norm.weight"], self.eps)
            gate = self.lin(h, pre + "mlp.gate_proj")
            x = residual + self.lin(F.silu(gate) * self.lin(h, pre + "mlp.up_proj"), pre + "mlp.down_proj")
        x = rms(x[:, -1], self.p["model.norm.weight"], self.eps)
        return F.linear(x, self.p["lm_head.weight"])
