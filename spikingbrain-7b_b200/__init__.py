"""B200-native hybrid decode-time cache path of SpikingBrain-7B.

Sub-modules
    build      -- compiles csrc/*.cu into libsbk.so (nvcc, sm_100a)
    _abi       -- ctypes binding of the C ABI declared in include/sbk.h
    ops        -- tensor-level wrappers of every libsbk entry point (append, decode, prefill, GLA
                  step and scan, step planner)
    block_pool -- host block allocator with sliding-window retirement
    hf_cache   -- the HF ``Cache`` surface of hf_7B_model/cache.py
    gla_slots  -- GLACacheParams / GLACacheManager / my_fused_recurrent_gla surface
    backend    -- MetaAttentionBackend / Metadata / Builder / Impl surface
    head_shard -- head-sharded (tensor-parallel) use: split rules, NCCL gather, fused peer-store gather
"""
__version__ = "0.1.0"
