"""Head-sharded (tensor-parallel) use of the cache path.

The reference splits attention heads over tensor-parallel ranks
(vllm_hymeta/model_for_7B/gla_attention.py:126-145, modeling_gla_swa.py:153-202): rank r owns
query heads [r*H/tp, (r+1)*H/tp) and the kv heads they read; when there are fewer kv heads than
ranks a kv head is replicated. Each rank then runs the same kernels on its slice -- the K/V pool
of a rank holds only its kv heads, the GLA state only its query heads -- and the per-rank head
outputs [T, H/tp, D] are all-gathered into [T, H, D] in rank order (NCCL over NVLink).
Block tables, sequence lengths and slot mappings are identical on all ranks.
"""
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_heads(num_heads: int, num_kv_heads: int, tp_size: int, tp_rank: int) -> Tuple[range, range]:
    """(query heads, kv heads) owned by `tp_rank`, with the reference's divisibility rules."""
    if num_heads % tp_size != 0:
        raise ValueError(f"num_heads {num_heads} must be divisible by tensor model parallel size {tp_size}")
    hq = num_heads // tp_size
    if num_kv_heads >= tp_size:
        if num_kv_heads % tp_size != 0:
            raise ValueError(f"{num_kv_heads} kv heads cannot be split over {tp_size} ranks")
        hk = num_kv_heads // tp_size
        kv = range(tp_rank * hk, (tp_rank + 1) * hk)
    else:
        if tp_size % num_kv_heads != 0:
            raise ValueError(f"{tp_size} ranks cannot share {num_kv_heads} kv heads evenly")
        owner = tp_rank // (tp_size // num_kv_heads)      # several ranks read the same kv head
        kv = range(owner, owner + 1)
    return range(tp_rank * hq, (tp_rank + 1) * hq), kv


def all_gather_heads(local: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """local [T, Hl, D] (this rank's heads) -> [T, tp*Hl, D] with rank r's heads at [r*Hl, (r+1)*Hl).
    One collective into a rank-major [tp*T, Hl, D] staging buffer, then one strided copy into head order."""
    tp = dist.get_world_size(group)
    T, Hl, D = local.shape
    if tp == 1:
        return local
    stage = torch.empty((tp * T, Hl, D), dtype=local.dtype, device=local.device)   # rank-major
    dist.all_gather_into_tensor(stage, local.contiguous(), group=group)
    if out is None:
        out = torch.empty((T, tp * Hl, D), dtype=local.dtype, device=local.device)
    out.view(T, tp, Hl, D).copy_(stage.view(tp, T, Hl, D).permute(1, 0, 2, 3))
    return out
