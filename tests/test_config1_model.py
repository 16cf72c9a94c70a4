"""The reference's CPU-runnable case (two-layer GLA + sliding-window model, batch 2, a 128-token
prompt, 32 greedy steps) against the reference model's own outputs (fixture config1_hf.npz, made by
tests/golden/make_golden.py from hf_7B_model.GLAswaForCausalLM).

The harness model (tests/hybrid_harness.py) is fed the reference's tokens step by step, so that a
rounding-level difference cannot send the two decodes down different paths; what is compared is
every step's logits, the argmax, the seen-token counters and the final cache contents.
  * on the CPU the harness runs over the oracle's cache classes  -> pins harness + oracle;
  * on the GPU it runs over the package's paged `Cache` and the GLA kernel -> the drop-in claim.
"""
import os

import numpy as np
import pytest
import torch

from oracle import ref_ops
from tests.hybrid_harness import HybridHarness

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "config1_hf.npz")


class OracleCache(ref_ops.RefWindowCache):
    """The oracle cache with the one-token GLA step the package's Cache offers as a fast path."""

    def gla_step(self, q, k, v, g, layer_idx, scale=None):
        B, H, D = q.shape
        S = self[layer_idx]["recurrent_state"] if layer_idx < len(self) else None
        if S is None:
            S = torch.zeros(B, H, D, D)
        o = ref_ops.gla_step_ref(q, k, v, g, S, scale=scale)
        self.update(recurrent_state=S, layer_idx=layer_idx, offset=1)
        return o


def _run(cache, device):
    gold = np.load(GOLD)
    names_shapes = [(str(n), tuple(int(x) for x in str(s).split(","))) for n, s in
                    zip(gold["param_names"], gold["param_shapes"])]
    model = HybridHarness(names_shapes, device)
    ids = torch.from_numpy(gold["input_ids"]).to(device)
    tokens = torch.from_numpy(gold["tokens"]).to(device)
    probe = torch.from_numpy(gold["probe"]).to(device)
    ref_logits = torch.from_numpy(gold["logits_probe"])
    cur = ids
    worst = 0.0
    with torch.no_grad():
        for step in range(33):
            logits = model.forward(cur, cache)
            worst = max(worst, float((logits[:, probe].cpu() - ref_logits[step]).abs().max()))
            assert torch.equal(logits.argmax(-1), tokens[:, step]), f"step {step}: greedy token differs"
            seen = [cache.get_seq_length(0), cache.get_seq_length(1), cache[1]["attn_state"][0].shape[-2]]
            assert seen == gold["seen"][step].tolist(), f"step {step}"
            cur = tokens[:, step:step + 1]          # teacher forcing with the reference's own tokens
    assert worst <= 5e-4, f"logits drift {worst}"
    k, v = cache[1]["attn_state"]
    assert torch.allclose(k.cpu(), torch.from_numpy(gold["final_k"]), rtol=1e-4, atol=1e-5)
    assert torch.allclose(v.cpu(), torch.from_numpy(gold["final_v"]), rtol=1e-4, atol=1e-5)
    S, S_ref = cache[0]["recurrent_state"].cpu(), torch.from_numpy(gold["final_state"])
    assert float((S - S_ref).abs().max() / S_ref.abs().max()) <= 1e-4
    return worst


def test_harness_over_oracle_cache_matches_reference_model():
    _run(OracleCache(), "cpu")


@pytest.mark.gpu
def test_harness_over_paged_cache_matches_reference_model(sb):
    from spikingbrain_7b_b200.hf_cache import Cache
    cache = Cache()
    _run(cache, "cuda:0")
    assert cache[1].paged.status.item() == 0
