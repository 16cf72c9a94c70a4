"""Head-sharded (tensor-parallel) use of the cache path.

The reference splits attention heads over tensor-parallel ranks
(vllm_hymeta/model_for_7B/gla_attention.py:126-145, modeling_gla_swa.py:153-202): rank r owns
query heads [r*H/tp, (r+1)*H/tp) and the kv heads they read; when there are fewer kv heads than
ranks a kv head is replicated. Each rank then runs the same kernels on its slice -- the K/V pool
of a rank holds only its kv heads, the GLA state only its query heads -- and the per-rank head
outputs [T, H/tp, D] are all-gathered into [T, H, D] in rank order (NCCL over NVLink).
Block tables, sequence lengths and slot mappings are identical on all ranks.
"""
import ctypes
from typing import List, Optional, Sequence, Tuple

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


class HybridLayout:
    """Ranks of one node as `n_seq_groups` groups of `tp_size` head shards: rank = group * tp_size +
    tp_rank. Heads are split inside a group (one gather per attention layer, among its tp_size
    ranks only), sequences across groups (no traffic between groups). This is how 8 GPUs run the
    28-head model: 28 heads do not split 8 ways (the reference asserts against it,
    vllm_hymeta/model_for_7B/gla_attention.py:128), 4 head shards x 2 sequence groups do."""

    def __init__(self, tp_size: int, world_size: int, rank: int, tp_group: Optional[dist.ProcessGroup]):
        self.tp_size, self.world_size, self.rank = tp_size, world_size, rank
        self.n_seq_groups = world_size // tp_size
        self.seq_group = rank // tp_size
        self.tp_rank = rank % tp_size
        self.tp_group = tp_group

    def my_sequences(self, n_sequences: int) -> range:
        """Contiguous share of `n_sequences` owned by this rank's sequence group."""
        return split_sequences(n_sequences, self.n_seq_groups, self.seq_group)


def split_sequences(n_sequences: int, n_groups: int, group: int) -> range:
    """Group g of n takes sequences [g * ceil-balanced share): sizes differ by at most one."""
    base, extra = divmod(n_sequences, n_groups)
    start = group * base + min(group, extra)
    return range(start, start + base + (1 if group < extra else 0))


def make_hybrid_layout(tp_size: int) -> HybridLayout:
    """Collective over the default process group: every rank must call it. Creates one process
    group per head-shard group and returns this rank's view."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if tp_size < 1 or world % tp_size != 0:
        raise ValueError(f"{world} ranks do not form groups of {tp_size} head shards")
    mine = None
    for g in range(world // tp_size):
        ranks = list(range(g * tp_size, (g + 1) * tp_size))
        grp = dist.new_group(ranks)          # every rank takes part in every creation
        if rank in ranks:
            mine = grp
    return HybridLayout(tp_size, world, rank, mine)


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


# ---------------------------------------------------------------------------------------------
# The all-gather fused into the decode kernel: peers are reached by stores, not by a collective.
# ---------------------------------------------------------------------------------------------
def gather_layout(max_tokens: int, num_heads: int, head_dim: int, tp_size: int) -> dict:
    """Byte layout of one rank's peer-visible allocation: two gathered buffers
    [max_tokens, num_heads, head_dim] bf16 (steps alternate between them, so a peer that is one
    step ahead never stores into rows still being read) and one int32 flag per rank."""
    if num_heads % tp_size != 0:
        raise ValueError(f"num_heads {num_heads} must be divisible by tensor model parallel size {tp_size}")
    if tp_size < 1 or tp_size > 8:
        raise ValueError("a head-sharded group has 1 to 8 ranks")
    row = num_heads * head_dim * 2
    if row % 16 != 0 or (num_heads // tp_size * head_dim * 2) % 16 != 0:
        raise ValueError("a rank's head slice must be a multiple of 16 bytes")
    buf = (max_tokens * row + 255) // 256 * 256
    return {"row_bytes": row, "slice_bytes": num_heads // tp_size * head_dim * 2, "buffer_bytes": buf,
            "buffer_offsets": (0, buf), "flag_offset": 2 * buf, "total_bytes": 2 * buf + 256}


def peer_addresses(layout: dict, bases: Sequence[int], rank: int, parity: int) -> Tuple[List[int], List[int]]:
    """For the writer `rank`: per other rank p (in rank order) the address of `rank`'s head slice
    in p's buffer `parity`, and of flag[rank] in p's flag array. `bases[p]` is p's allocation as
    mapped into this process."""
    outs, flags = [], []
    for p, base in enumerate(bases):
        if p == rank:
            continue
        outs.append(base + layout["buffer_offsets"][parity] + rank * layout["slice_bytes"])
        flags.append(base + layout["flag_offset"] + 4 * rank)
    return outs, flags


class _DeviceBytes:
    """Device memory owned by libsbk, seen by torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class FusedHeadGather:
    """Head-sharded sliding-window decode whose kernel also delivers the head outputs to the other
    ranks (sbk_swa_decode_gather), in place of the collective the reference issues after its
    attention (vllm_hymeta/model_for_7B/modeling_gla_swa.py:228-231 gathers through the
    row-parallel output projection's input). One instance per layer stack is enough: steps alternate
    between its two buffers, and a rank enters step s + 1 only after it has seen every peer's flag of
    step s, so a buffer is rewritten only once all of its readers are a full step past it.

    `group` carries the one-off exchange of memory handles (and a barrier at close); the data path
    uses no collective."""

    def __init__(self, max_tokens: int, num_heads: int, head_dim: int,
                 group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None,
                 timeout_ms: int = 2000):
        from . import _abi
        self._abi = _abi
        self.group = group
        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device if device is not None else torch.device("cuda", torch.cuda.current_device()))
        self.H, self.D, self.max_tokens = num_heads, head_dim, max_tokens
        self.Hl = num_heads // self.tp
        self.timeout_ms = timeout_ms
        self.layout = gather_layout(max_tokens, num_heads, head_dim, self.tp)
        self._closed = False
        lib = _abi.lib
        with torch.cuda.device(self.device):
            base = ctypes.c_void_p()
            _abi.check("sbk_peer_alloc", lib.sbk_peer_alloc(self.layout["total_bytes"], ctypes.byref(base)))
            self._base = base.value
            hb = lib.sbk_peer_handle_bytes()
            handle = ctypes.create_string_buffer(hb)
            _abi.check("sbk_peer_export", lib.sbk_peer_export(self._base, handle, hb))
            handles: List[Optional[bytes]] = [None] * self.tp
            dist.all_gather_object(handles, handle.raw, group=group)
            self.bases: List[int] = []
            for p, h in enumerate(handles):
                if p == self.rank:
                    self.bases.append(self._base)
                    continue
                mapped = ctypes.c_void_p()
                _abi.check("sbk_peer_open", lib.sbk_peer_open(ctypes.create_string_buffer(h, hb), hb,
                                                              ctypes.byref(mapped)))
                self.bases.append(mapped.value)
        raw = torch.as_tensor(_DeviceBytes(self._base, self.layout["total_bytes"]), device=self.device)
        self._raw = raw
        n = max_tokens * self.layout["row_bytes"]
        self.buffers = [raw[o:o + n].view(torch.bfloat16).view(max_tokens, num_heads, head_dim)
                        for o in self.layout["buffer_offsets"]]
        fo = self.layout["flag_offset"]
        self.flags = raw[fo:fo + 4 * self.tp].view(torch.int32)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # Steps are counted on the device: every decode raises the peers' flags to base + 1 and
        # every wait moves the base on by one, so the calls carry no host-side step number and a
        # captured CUDA graph replays them unchanged.
        self.base = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.calls = 0
        self._counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        from .ops import PeerTargets
        self._targets = []
        for parity in (0, 1):
            outs, flags = peer_addresses(self.layout, self.bases, self.rank, parity)
            self._targets.append(PeerTargets(outs, flags, 1, self.base))
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)     # every rank has mapped every buffer before anyone stores

    def local_slice(self, gathered: torch.Tensor) -> torch.Tensor:
        return gathered[:, self.rank * self.Hl:(self.rank + 1) * self.Hl]

    def decode(self, q_local: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
               block_tables: torch.Tensor, seq_lens: torch.Tensor, *, window_left: int, **kw) -> torch.Tensor:
        """q_local [B, H/tp, D]; returns [B, H, D] with every rank's heads, valid for whatever is
        enqueued on the current stream after this call, until the next-but-one call. Readers of
        the result must be ordered before this rank's next call (same stream, or an event).
        Check `status` (SBK_ST_WAIT_TIMEOUT) when the step is synchronised: a peer that never
        delivered leaves its slice stale. Calls alternate between the two buffers; a captured
        graph must therefore hold an even number of calls."""
        from . import ops
        B = q_local.shape[0]
        if B > self.max_tokens or q_local.shape[1] != self.Hl:
            raise ValueError(f"q_local must be [<= {self.max_tokens}, {self.Hl}, {self.D}]")
        parity = self.calls & 1
        self.calls += 1
        gathered = self.buffers[parity][:B]
        ops.swa_decode(q_local, k_cache, v_cache, block_tables, seq_lens, window_left=window_left,
                       out=self.local_slice(gathered), peers=self._targets[parity], status=self.status, **kw)
        self.wait()
        return gathered

    def gla_step(self, q_local: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
                 state: torch.Tensor, slot_idx: Optional[torch.Tensor] = None, **kw) -> torch.Tensor:
        """The GLA layer's counterpart of `decode`: q_local [B, H/tp, D], k/v/g [B, kv heads of this
        rank, D], state [slots, H/tp, D, D]; returns [B, H, D] with every rank's head outputs."""
        from . import ops
        B = q_local.shape[0]
        if B > self.max_tokens or q_local.shape[1] != self.Hl:
            raise ValueError(f"q_local must be [<= {self.max_tokens}, {self.Hl}, {self.D}]")
        parity = self.calls & 1
        self.calls += 1
        gathered = self.buffers[parity][:B]
        ops.gla_step(q_local, k, v, g, state, slot_idx, out=self.local_slice(gathered), peers=self._targets[parity],
                     peer_counter=self._counter, status=self.status, **kw)
        self.wait()
        return gathered

    def wait(self) -> None:
        """Enqueue the bounded wait for every peer's flag of the current step; it also moves the
        device-side step counter on."""
        from . import ops
        rc = self._abi.lib.sbk_peer_wait(self.flags.data_ptr(), self.tp, self.rank, 1, self.base.data_ptr(), 1,
                                         self.timeout_ms, self.status.data_ptr(), ops._stream())
        self._abi.check("sbk_peer_wait", rc)

    def resync(self) -> None:
        """After a step that some rank did not take part in (its peers saw SBK_ST_WAIT_TIMEOUT): bring
        every rank's step counter, flags and buffer turn back to the start. Collective over the group;
        call it on every rank, between steps."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)          # nobody is storing into a peer any more
        self.flags.zero_()
        self.base.zero_()
        self.status.zero_()
        self._counter.zero_()
        self.calls = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)          # every rank starts from zero before the next stores arrive

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)      # nobody stores into memory that is about to go
        lib = self._abi.lib
        with torch.cuda.device(self.device):
            for p, b in enumerate(self.bases):
                if p != self.rank:
                    self._abi.check("sbk_peer_close", lib.sbk_peer_close(b))
            self.buffers, self.flags, self._raw = [], None, None
            self._abi.check("sbk_peer_free", lib.sbk_peer_free(self._base))
