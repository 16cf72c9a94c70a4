"""CPU oracle for the hybrid decode-time cache path of SpikingBrain-7B.

TEST INFRASTRUCTURE ONLY. This package restates, in plain PyTorch on the CPU,
the algorithms the reference runs on this path; it exists to check the CUDA
kernels and to serve as the timed CPU baseline. Only tests/, the smoke check of
__graft_entry__ and the `cpu_baseline` / `--impl reference` legs of bench.py may
import it. The product (the package next to it) never does.

Parity status: PINNED. Every function in ref_ops is checked against outputs of
the reference's own code, produced by tests/golden/make_golden.py in a container
that holds the reference (hf_7B_model/cache.py and window_attention_sdpa.py run
on the CPU; the Triton kernel of vllm_hymeta/model_for_7B/my_fused_recurrent.py
run under the Triton interpreter) and committed under tests/golden/.
"""
