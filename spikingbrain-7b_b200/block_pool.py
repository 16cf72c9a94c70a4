"""Host-side block allocator with sliding-window retirement.

Stands in for the block manager the reference leaves to vLLM: it decides which
physical block holds which 16-token span of which sequence, hands out the flat
slot ids the append kernel writes to (the `slot_mapping` of
vllm_hymeta/attention/meta_attention.py:487-494), and recycles blocks that fall
wholly before the sliding window (the window-truncated tables of :479-485).

The retirement rule is the one the device applies inside `sbk_kv_append`, so the
host mirror and the device table stay identical without reading anything back:
    first token still needed  t0 = max(0, seq_len - n_new - window_left)
    logical blocks            j < t0 // block_size   are released.
Pure numpy: no tensor maths happens here.
"""
from dataclasses import dataclass
from typing import List, Sequence, Optional

import numpy as np


class OutOfBlocks(MemoryError):
    """The pool has no free block left."""


class BlockPool:
    """LIFO free list over ``num_blocks`` physical blocks: the block retired last is
    handed out first, so a churning batch fragments the pool the way a serving engine does."""

    def __init__(self, num_blocks: int):
        if num_blocks <= 0:
            raise ValueError("num_blocks must be positive")
        self.num_blocks = num_blocks
        self._free: List[int] = list(range(num_blocks - 1, -1, -1))
        self._is_free = np.ones(num_blocks, dtype=bool)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfBlocks(f"all {self.num_blocks} KV blocks are in use")
        b = self._free.pop()
        self._is_free[b] = False
        return b

    def release(self, ids: Sequence[int]) -> None:
        for b in ids:
            b = int(b)
            if not 0 <= b < self.num_blocks:
                raise ValueError(f"block id {b} outside the pool")
            if self._is_free[b]:
                raise ValueError(f"block {b} released twice")
            self._is_free[b] = True
            self._free.append(b)


def first_visible(seq_len: int, n_new: int, window_left: int) -> int:
    if window_left < 0:
        return 0
    return max(0, seq_len - n_new - window_left)


@dataclass
class StepPlan:
    """What one call of ``SlidingWindowBlockManager.advance`` decided."""
    slot_mapping: np.ndarray       # int64 [T]  flat slot per new token, rows in order, -1 = padding
    seq_lens: np.ndarray           # int32 [rows] lengths AFTER the append (0 = inactive row)
    query_start_loc: np.ndarray    # int32 [rows+1]
    new_entries: np.ndarray        # int32 [n, 3] (row, logical block, physical block) allocated now
    retired: List[List[int]]       # per row, ids released now, in logical order


class SlidingWindowBlockManager:
    """Block tables of up to ``max_seqs`` sequences over one pool.

    Rows are stable: a sequence keeps its row from ``admit`` to ``finish``; an inactive row
    has length 0 and takes no part in a step. ``table`` is the host mirror of the device
    block table ([max_seqs, max_blocks] int32, -1 = no block)."""

    def __init__(self, num_blocks: int, block_size: int, window_left: int, max_seqs: int,
                 max_blocks_per_seq: int):
        if block_size <= 0 or block_size % 16:
            raise ValueError(f"Invalid block size {block_size}. Must be a multiple of 16 and at least 16.")
        self.pool = BlockPool(num_blocks)
        self.block_size = block_size
        self.window_left = window_left
        self.max_seqs = max_seqs
        self.max_blocks = max_blocks_per_seq
        self.table = np.full((max_seqs, max_blocks_per_seq), -1, dtype=np.int32)
        self.lens = np.zeros(max_seqs, dtype=np.int32)
        self.active = np.zeros(max_seqs, dtype=bool)
        self._first_live = np.zeros(max_seqs, dtype=np.int64)  # first logical block not yet retired

    # ---------------------------------------------------------------- sequences
    def admit(self, row: int) -> None:
        if self.active[row]:
            raise ValueError(f"row {row} already holds a sequence")
        self.active[row] = True
        self.lens[row] = 0
        self._first_live[row] = 0

    def finish(self, row: int) -> List[int]:
        """Release every block of the sequence in ``row``; returns the released ids."""
        if not self.active[row]:
            raise ValueError(f"row {row} holds no sequence")
        ids = [int(b) for b in self.table[row] if b >= 0]
        self.pool.release(ids)
        self.table[row] = -1
        self.lens[row] = 0
        self.active[row] = False
        self._first_live[row] = 0
        return ids

    def resident_blocks(self, row: int) -> int:
        return int((self.table[row] >= 0).sum())

    # --------------------------------------------------------------------- step
    def advance(self, n_new: Sequence[int], pad_inactive: bool = True) -> StepPlan:
        """Append ``n_new[row]`` tokens to every active row: release the blocks this step's queries
        can no longer see, allocate the blocks the new tokens need, compute their slots. With ``pad_inactive`` an
        inactive row contributes one -1 slot when every active row appends one token
        (the static decode batch: token i belongs to row i)."""
        n_new = np.asarray(n_new, dtype=np.int64)
        if n_new.shape != (self.max_seqs,):
            raise ValueError("n_new needs one entry per row")
        if (n_new[~self.active] != 0).any():
            raise ValueError("inactive rows cannot take tokens")
        bs = self.block_size
        if pad_inactive and bool((n_new[self.active] == 1).all()):
            return self._advance_decode()
        if ((self.lens.astype(np.int64) + n_new + bs - 1) // bs > self.max_blocks).any():
            raise ValueError(f"a sequence exceeds max_blocks_per_seq={self.max_blocks}")
        old_lens = self.lens.copy()
        self.lens = (self.lens.astype(np.int64) + n_new).astype(np.int32)
        # Blocks that this step's queries can no longer see go back to the pool BEFORE the new
        # tokens take theirs: nothing reads them in this step, so they may be reused at once.
        retired = self._retire(n_new)
        slots: List[np.ndarray] = []
        new_entries: List[List[int]] = []
        qsl = np.zeros(self.max_seqs + 1, dtype=np.int32)
        for row in range(self.max_seqs):
            n = int(n_new[row])
            qsl[row + 1] = qsl[row] + n
            if n == 0:
                continue
            L0 = int(old_lens[row])
            pos = np.arange(L0, L0 + n, dtype=np.int64)
            lb = pos // bs
            for j in range(int(lb[0]), int(lb[-1]) + 1):
                if self.table[row, j] < 0:
                    if j < self._first_live[row]:
                        continue   # a prompt longer than the window: its oldest tokens are never stored
                    pb = self.pool.allocate()
                    self.table[row, j] = pb
                    new_entries.append([row, j, pb])
            blk = self.table[row, lb].astype(np.int64)
            slots.append(np.where(blk >= 0, blk * bs + pos % bs, -1))
        return StepPlan(
            slot_mapping=np.concatenate(slots) if slots else np.zeros(0, dtype=np.int64),
            seq_lens=self.lens.copy(), query_start_loc=qsl,
            new_entries=np.asarray(new_entries, dtype=np.int32).reshape(-1, 3), retired=retired)

    def _advance_decode(self) -> StepPlan:
        """The decode step (one token per active row, token i <-> row i) without a Python
        loop over rows: only rows that cross a block edge are visited one by one."""
        bs = self.block_size
        rows = np.nonzero(self.active)[0]
        pos = self.lens[rows].astype(np.int64)
        lb = pos // bs
        if rows.size and lb.max() >= self.max_blocks:
            raise ValueError(f"a sequence exceeds max_blocks_per_seq={self.max_blocks}")
        self.lens[rows] += 1
        retired: List[List[int]] = [[] for _ in range(self.max_seqs)]
        if self.window_left >= 0 and rows.size:   # retire first: the freed blocks can be reused at once
            t0 = np.maximum(self.lens[rows].astype(np.int64) - 1 - self.window_left, 0)
            first_live = np.minimum(t0 // bs, self.max_blocks)
            for i in np.nonzero(first_live > self._first_live[rows])[0]:
                row = int(rows[i])
                ids = []
                for j in range(int(self._first_live[row]), int(first_live[i])):
                    if self.table[row, j] >= 0:
                        ids.append(int(self.table[row, j]))
                        self.table[row, j] = -1
                self._first_live[row] = int(first_live[i])
                self.pool.release(ids)
                retired[row] = ids
        new_entries: List[List[int]] = []
        for i in np.nonzero(self.table[rows, lb] < 0)[0]:
            row, j = int(rows[i]), int(lb[i])
            if j < self._first_live[row]:
                raise RuntimeError("append into a block that was already retired")
            pb = self.pool.allocate()
            self.table[row, j] = pb
            new_entries.append([row, j, pb])
        slot_mapping = np.full(self.max_seqs, -1, dtype=np.int64)
        slot_mapping[rows] = self.table[rows, lb].astype(np.int64) * bs + pos % bs
        return StepPlan(slot_mapping=slot_mapping, seq_lens=self.lens.copy(),
                        query_start_loc=np.arange(self.max_seqs + 1, dtype=np.int32),
                        new_entries=np.asarray(new_entries, dtype=np.int32).reshape(-1, 3),
                        retired=retired)

    def _retire(self, n_new: np.ndarray) -> List[List[int]]:
        out: List[List[int]] = [[] for _ in range(self.max_seqs)]
        if self.window_left < 0:
            return out
        for row in np.nonzero(self.active)[0]:
            n = int(n_new[row]) if n_new[row] > 0 else 1
            t0 = first_visible(int(self.lens[row]), n, self.window_left)
            first_live = min(t0 // self.block_size, self.max_blocks)
            ids = []
            for j in range(int(self._first_live[row]), first_live):
                if self.table[row, j] >= 0:
                    ids.append(int(self.table[row, j]))
                    self.table[row, j] = -1
            if first_live > self._first_live[row]:
                self._first_live[row] = first_live
            self.pool.release(ids)
            out[int(row)] = ids
        return out


class DeviceStepPlanner:
    """The sliding-window block manager with its state on the GPU: lengths, block tables, the
    ring of free block ids and the per-step metadata (slot mapping, positions, context lengths,
    query starts) are device tensors that one `sbk_plan_step` launch advances, so a decode loop
    needs no host work and no host-to-device copy per step, and the launch can sit in a CUDA
    graph. It stands in for the per-step work of MetaAttentionMetadataBuilder
    (vllm_hymeta/attention/meta_attention.py:435-494, 532-583), MetaAttentionMetadata.advance_step
    (:338-409) and the engine's block manager. The host keeps no copy of the lengths;
    `snapshot()` reads the state back when it is wanted (tests, debugging)."""

    def __init__(self, num_blocks: int, block_size: int, window_left: int, max_seqs: int,
                 max_blocks_per_seq: int, device, max_tokens: Optional[int] = None):
        import torch
        from . import ops
        self._ops = ops
        self.num_blocks, self.block_size, self.window_left = num_blocks, block_size, window_left
        self.max_seqs, self.max_blocks = max_seqs, max_blocks_per_seq
        T = max_tokens or max_seqs
        i32 = dict(dtype=torch.int32, device=device)
        self.ring = torch.empty(num_blocks, **i32)
        self.ctrl = torch.zeros(4, dtype=torch.int64, device=device)
        self.seq_lens = torch.empty(max_seqs, **i32)
        self.block_tables = torch.empty(max_seqs, max_blocks_per_seq, **i32)
        self.slot_mapping = torch.full((T,), -1, dtype=torch.int64, device=device)
        self.positions = torch.zeros(T, dtype=torch.int64, device=device)
        self.context_lens = torch.zeros(max_seqs, **i32)
        self.query_start_loc = torch.zeros(max_seqs + 1, **i32)
        self.status = torch.zeros(1, **i32)
        ops.pool_init(self.ring, self.ctrl, self.seq_lens, self.block_tables)

    def load_state(self, lens, table, free_ids) -> None:
        """Adopt an existing state (host arrays): per-row lengths, the block table, and the ids of
        the free blocks in the order they are to be handed out."""
        import numpy as np
        import torch
        lens = np.ascontiguousarray(lens, dtype=np.int32)
        table = np.ascontiguousarray(table, dtype=np.int32)
        free_ids = np.ascontiguousarray(free_ids, dtype=np.int32)
        if lens.shape != (self.max_seqs,) or table.shape != (self.max_seqs, self.max_blocks):
            raise ValueError("lens / table do not match the planner's shape")
        live = table[table >= 0]
        if len(live) + len(free_ids) > self.num_blocks or len(np.unique(np.concatenate([live, free_ids]))) != len(live) + len(free_ids):
            raise ValueError("a block id is owned twice (or the pool is over-subscribed)")
        self.seq_lens.copy_(torch.from_numpy(lens))
        self.block_tables.copy_(torch.from_numpy(table))
        ring = np.zeros(self.num_blocks, dtype=np.int32)
        ring[:len(free_ids)] = free_ids
        self.ring.copy_(torch.from_numpy(ring))
        self.ctrl.copy_(torch.tensor([0, len(free_ids), len(free_ids), 0], dtype=torch.int64))

    def plan(self, n_new=None, retire: bool = True) -> None:
        """Advance every row by n_new[b] tokens (device int32 [max_seqs]; None: one token each).
        Results are in slot_mapping / positions / context_lens / query_start_loc / seq_lens /
        block_tables; nothing is returned and nothing is synchronised."""
        self._ops.plan_step(self.seq_lens, self.block_tables, self.slot_mapping,
                            block_size=self.block_size, num_blocks=self.num_blocks,
                            window_left=self.window_left, retire=retire, n_new=n_new, ring=self.ring,
                            ctrl=self.ctrl, positions=self.positions, context_lens=self.context_lens,
                            query_start_loc=self.query_start_loc, status=self.status)

    def trim(self) -> None:
        """Give back, for every row, the blocks its next token will not see. A planner launch with no
        new tokens: after a prompt chunk the rows still hold the chunk's look-back window (the first
        token of the chunk saw window_left tokens behind it); this returns the resident set to the
        window at once, so the blocks can serve other sequences before the row's next step."""
        import torch
        if not hasattr(self, "_zeros"):
            self._zeros = torch.zeros(self.max_seqs, dtype=torch.int32, device=self.seq_lens.device)
        self._ops.plan_step(self.seq_lens, self.block_tables, self.slot_mapping,
                            block_size=self.block_size, num_blocks=self.num_blocks,
                            window_left=self.window_left, retire=True, trim=True, n_new=self._zeros,
                            ring=self.ring, ctrl=self.ctrl, positions=self.positions,
                            context_lens=self.context_lens, query_start_loc=self.query_start_loc,
                            status=self.status)

    def release(self, rows) -> None:
        """rows: device int32 tensor of finished table rows; their blocks return to the ring."""
        self._ops.release_rows(rows, self.seq_lens, self.block_tables, block_size=self.block_size,
                               num_blocks=self.num_blocks, ring=self.ring, ctrl=self.ctrl,
                               status=self.status)

    def snapshot(self) -> dict:
        """Host copy of the state (synchronises): lens, table, free ids in ring order, counters."""
        head, tail, min_free, steps = (int(x) for x in self.ctrl.tolist())
        ring = self.ring.tolist()
        free = [ring[i % self.num_blocks] for i in range(head, tail)]
        return dict(lens=self.seq_lens.tolist(), table=self.block_tables.tolist(), free=free,
                    min_free=min_free, steps=steps, status=int(self.status.item()))
