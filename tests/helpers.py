"""Shared builders of seeded synthetic inputs for the parity tests."""
import math
from typing import List, Tuple

import torch


def make_paged_kv(seq_lens: List[int], window_left: int, kvh: int, D: int, block_size: int,
                  dtype=torch.bfloat16, seed: int = 0, slack_blocks: int = 7,
                  full_retention: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]:
    """A paged pool holding K/V ~ N(0,1)/sqrt(D) for every visible token of every sequence,
    reached through a randomly permuted block table (logical blocks that lie wholly before
    the window are -1 unless `full_retention`). Returns (kv_cache [2,NB,bs,kvh,D], table
    [B,max_blocks] int32, num_blocks)."""
    g = torch.Generator().manual_seed(seed)
    B = len(seq_lens)
    max_blocks = max(1, max((L + block_size - 1) // block_size for L in seq_lens))
    need = []
    for L in seq_lens:
        t0 = 0 if (window_left < 0 or full_retention) else max(0, L - 1 - window_left)
        first = t0 // block_size
        last = (L - 1) // block_size if L > 0 else -1
        need.append((first, last))
    total = sum(max(0, l - f + 1) for f, l in need)
    nb = total + slack_blocks
    perm = torch.randperm(nb, generator=g)
    table = torch.full((B, max_blocks), -1, dtype=torch.int32)
    kv = torch.zeros(2, nb, block_size, kvh, D, dtype=dtype)
    # unowned blocks carry a poison pattern so that a stray read shows up
    kv.fill_(float("nan"))
    cur = 0
    for b, (f, l) in enumerate(need):
        for j in range(f, l + 1):
            pb = int(perm[cur]); cur += 1
            table[b, j] = pb
            kv[:, pb] = (torch.randn(2, block_size, kvh, D, generator=g) / math.sqrt(D)).to(dtype)
        # rows of the newest block that no token has reached yet are uninitialised memory
        L = seq_lens[b]
        if L > 0 and L % block_size:
            kv[:, int(table[b, l]), L % block_size:] = float("nan")
    return kv, table, nb


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a-b| relative to max |b|."""
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


def mean_rel(a: torch.Tensor, b: torch.Tensor) -> float:
    """sum |a-b| / sum |b|."""
    return float((a.double() - b.double()).abs().sum() / b.double().abs().sum().clamp_min(1e-30))


# --------------------------------------------------------------- deterministic weights
def det_param(name: str, shape) -> torch.Tensor:
    """Weights of the two-layer plumbing model, rebuilt identically wherever they are needed:
    one seeded CPU generator per parameter name. Norm weights sit around 1, everything else is
    N(0, 0.05) (biases included, so that they matter)."""
    import zlib
    g = torch.Generator().manual_seed(zlib.crc32(name.encode()) & 0x7FFFFFFF)
    t = torch.randn(tuple(shape), generator=g)
    if name.endswith("norm.weight"):
        return 1.0 + 0.1 * t
    return 0.05 * t


def det_unit(shape, salt):
    """Deterministic values in [-1, 1) without an RNG: the inputs of tests/golden/gla_fused.npz
    (the generator script holds the same formula)."""
    n = 1
    for d in shape:
        n *= d
    i = torch.arange(n, dtype=torch.int64) + salt * 1000003
    return (((i * 2246822519) % 999983).double() / 499991.5 - 1.0).float().view(*shape)
