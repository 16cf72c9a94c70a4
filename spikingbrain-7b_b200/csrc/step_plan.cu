// Device-resident step planner and block allocator for the paged sliding-window cache.
//
// The reference prepares every step on the host: a Python loop per sequence builds the block
// table row, the slot of each new token, the lengths (MetaAttentionMetadataBuilder,
// vllm_hymeta/attention/meta_attention.py:435-494, 532-583), the engine's block manager hands out
// and takes back blocks, and only multi-step decode advances lengths and slots on the device
// (MetaAttentionMetadata.advance_step, :338-409). Here the whole of it is one launch on state
// that never leaves the GPU:
//     seq_lens[B], block_tables[B, max_blocks], a ring of free block ids, head/tail counters.
// sbk_plan_step, for every row b with n_new[b] > 0 new tokens:
//   1. retires the blocks that no token of this step can see (wholly before
//      t0 = max(0, seq_len - window_left), seq_len before the step): ids pushed on the ring,
//      table entries -> -1
//   2. allocates the blocks the new tokens land in (missing entries of logical blocks
//      seq_len / bs .. (seq_len + n_new - 1) / bs) : ids popped from the ring
//   3. writes slot_mapping / positions of every new token, context_lens, query_start_loc,
//      and advances seq_lens.
// One CTA of 1024 threads does it all (rows are few: hundreds to thousands), which makes the
// allocator DETERMINISTIC: pushes and pops are placed by block-wide prefix sums in row order, so
// a CPU model of the same policy predicts every block id. Retirement comes before allocation
// (a __syncthreads apart), so a pool with no slack beyond the windows still works. A step that
// cannot be served (ring empty, table row full, more tokens than slot_mapping holds) changes
// NOTHING: it raises a status bit and fills slot_mapping with -1, so the append that follows
// writes nothing either.
#include "sbk_common.cuh"

namespace sbk {

constexpr int kPlanThreads = 1024;

struct PlanParams {
  const int32_t* n_new;        // [B] or NULL (one token per row)
  int32_t* seq_lens;           // [B]
  int32_t* block_tables;       // [B, max_blocks]
  int max_blocks, B, block_size, window_left, retire;
  int32_t* ring;               // [num_blocks] free ids, or NULL (tables are filled by someone else)
  unsigned long long* ctrl;    // [4]: head, tail, lowest free count seen, steps planned
  int num_blocks;
  int64_t* slot_mapping;       // [T]
  int64_t* positions;          // [T] or NULL
  int32_t* context_lens;       // [B] or NULL
  int32_t* query_start_loc;    // [B+1] (written); may be NULL only when n_new is NULL
  int T;
  int32_t* status;
};

// exclusive prefix sums of three per-thread counts over the CTA; totals returned through tot[]
__device__ __forceinline__ void block_scan3(int (&v)[3], int (&tot)[3], int (*s_warp)[3]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl[3];
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    int x = v[c];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, off);
      if (lane >= off) x += y;
    }
    incl[c] = x;
    if (lane == 31) s_warp[warp][c] = x;
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      int x = s_warp[lane][c];
      const int own = x;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, off);
        if (lane >= off) x += y;
      }
      s_warp[lane][c] = x - own;                  // exclusive prefix of the warp totals
      if (lane == 31) s_warp[32][c] = x;          // grand total
    }
  }
  __syncthreads();
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    tot[c] = s_warp[32][c];
    v[c] = incl[c] - v[c] + s_warp[warp][c];
  }
}

struct RowPlan {
  int L, n, need, nret, first_live, lb0, lb1;
  bool overflow;
};

__device__ __forceinline__ RowPlan plan_row(const PlanParams& p, int b) {
  RowPlan r;
  r.L = p.seq_lens[b];
  r.n = p.n_new ? p.n_new[b] : 1;
  if (r.n < 0) r.n = 0;
  r.need = r.nret = 0;
  r.first_live = r.lb0 = 0;
  r.lb1 = -1;
  r.overflow = false;
  // a row without new tokens is left alone, except in trim mode (retire == 2), where it gives up
  // what its NEXT token will not see: blocks wholly before seq_len - window_left
  if (r.n == 0 && p.retire != 2) return r;
  const int32_t* row = p.block_tables + (int64_t)b * p.max_blocks;
  if (r.n > 0) {
    r.lb0 = r.L / p.block_size;
    r.lb1 = (r.L + r.n - 1) / p.block_size;
    if (r.lb1 >= p.max_blocks) {
      r.overflow = true;
      return r;
    }
    for (int lb = r.lb0; lb <= r.lb1; ++lb) r.need += row[lb] < 0;
  }
  if (p.retire) {
    const int t0 = first_visible(r.L + r.n, r.n, p.window_left);
    r.first_live = t0 / p.block_size;   // <= lb0, so never one of the blocks counted above
    if (r.first_live > p.max_blocks) r.first_live = p.max_blocks;
    for (int j = r.first_live - 1; j >= 0 && row[j] >= 0; --j) ++r.nret;
  }
  return r;
}

__global__ void __launch_bounds__(kPlanThreads) plan_step_kernel(const PlanParams p) {
  __shared__ int s_warp[33][3];
  __shared__ int s_abort;
  const int tid = threadIdx.x;
  const int rpt = (p.B + kPlanThreads - 1) / kPlanThreads;   // consecutive rows per thread
  const int r_begin = min(tid * rpt, p.B), r_end = min(r_begin + rpt, p.B);
  if (tid == 0) s_abort = 0;
  __syncthreads();

  // ---- phase A: what every row needs ----
  int v[3] = {0, 0, 0};   // blocks to allocate, blocks to retire, new tokens
  bool overflow = false;
  for (int b = r_begin; b < r_end; ++b) {
    const RowPlan r = plan_row(p, b);
    v[0] += r.need;
    v[1] += r.nret;
    v[2] += r.n;
    overflow |= r.overflow;
  }
  int tot[3];
  block_scan3(v, tot, s_warp);
  const unsigned long long head = p.ring ? p.ctrl[0] : 0ull, tail = p.ring ? p.ctrl[1] : 0ull;
  const long long avail = (long long)(tail - head);
  if (overflow) {
    raise_status(p.status, SBK_ST_TABLE_FULL);
    s_abort = 1;
  }
  if (tid == 0) {
    if (tot[0] > (p.ring ? avail + tot[1] : 0)) {
      raise_status(p.status, SBK_ST_OUT_OF_BLOCKS);
      s_abort = 1;
    }
    if (tot[2] > p.T) {
      raise_status(p.status, SBK_ST_TABLE_FULL);
      s_abort = 1;
    }
  }
  __syncthreads();
  if (s_abort) {   // nothing was changed; the append that follows must not write either
    for (int t = tid; t < p.T; t += kPlanThreads) p.slot_mapping[t] = -1;
    return;
  }

  // ---- phase B: retire (push), in row order ----
  if (p.retire && p.ring) {
    unsigned long long at = tail + (unsigned long long)v[1];
    for (int b = r_begin; b < r_end; ++b) {
      const RowPlan r = plan_row(p, b);
      int32_t* row = p.block_tables + (int64_t)b * p.max_blocks;
      // oldest block first, as the host-side manager lists them
      for (int j = r.first_live - r.nret; j < r.first_live; ++j) {
        p.ring[at % (unsigned long long)p.num_blocks] = row[j];
        row[j] = -1;
        ++at;
      }
    }
  } else if (p.retire) {
    for (int b = r_begin; b < r_end; ++b) {
      const RowPlan r = plan_row(p, b);
      int32_t* row = p.block_tables + (int64_t)b * p.max_blocks;
      for (int j = r.first_live - r.nret; j < r.first_live; ++j) row[j] = -1;
    }
  }
  __syncthreads();   // pushes of this step may be popped by it

  // ---- phase C: allocate (pop) in row order, advance the lengths, per-row outputs ----
  {
    unsigned long long at = head + (unsigned long long)v[0];
    int tok = v[2];
    for (int b = r_begin; b < r_end; ++b) {
      const int L = p.seq_lens[b];
      int n = p.n_new ? p.n_new[b] : 1;
      if (n < 0) n = 0;
      if (p.query_start_loc) p.query_start_loc[b] = tok;
      if (p.context_lens) p.context_lens[b] = L;
      tok += n;
      if (n == 0) continue;
      int32_t* row = p.block_tables + (int64_t)b * p.max_blocks;
      const int lb1 = (L + n - 1) / p.block_size;
      for (int lb = L / p.block_size; lb <= lb1; ++lb) {
        if (row[lb] < 0) {
          row[lb] = p.ring[at % (unsigned long long)p.num_blocks];
          ++at;
        }
      }
      p.seq_lens[b] = L + n;
    }
    if (tid == kPlanThreads - 1 && p.query_start_loc) p.query_start_loc[p.B] = tot[2];
  }
  if (tid == 0 && p.ring) {
    p.ctrl[0] = head + (unsigned long long)tot[0];
    p.ctrl[1] = tail + (unsigned long long)tot[1];
    const unsigned long long free_now = (tail + tot[1]) - (head + tot[0]);
    if (free_now < p.ctrl[2]) p.ctrl[2] = free_now;
    p.ctrl[3] += 1;
  }
  __syncthreads();

  // ---- phase D: one slot and position per new token, all threads ----
  for (int t = tid; t < p.T; t += kPlanThreads) {
    int64_t slot = -1, pos = 0;
    if (t < tot[2]) {
      int b = t;
      if (p.n_new) {   // last row whose first token is <= t (rows without tokens share a start)
        int lo = 0, hi = p.B;
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (p.query_start_loc[mid] <= t) lo = mid; else hi = mid;
        }
        b = lo;
      }
      const int first = p.n_new ? p.query_start_loc[b] : b;
      const int n = p.n_new ? p.n_new[b] : 1;
      pos = (int64_t)p.seq_lens[b] - n + (t - first);
      const int lb = (int)(pos / p.block_size);
      const int32_t blk = p.block_tables[(int64_t)b * p.max_blocks + lb];
      if (blk < 0 || blk >= p.num_blocks) raise_status(p.status, SBK_ST_BAD_BLOCK);
      else slot = (int64_t)blk * p.block_size + (pos - (int64_t)lb * p.block_size);
    }
    p.slot_mapping[t] = slot;
    if (p.positions) p.positions[t] = pos;
  }
}

// ring <- 0 .. num_blocks-1, counters reset; tables and lengths cleared when given
__global__ void pool_init_kernel(int32_t* ring, unsigned long long* ctrl, int num_blocks,
                                 int32_t* seq_lens, int32_t* block_tables, int64_t table_elems, int B) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t j = i; j < num_blocks; j += stride) ring[j] = (int32_t)j;
  if (block_tables)
    for (int64_t j = i; j < table_elems; j += stride) block_tables[j] = -1;
  if (seq_lens)
    for (int64_t j = i; j < B; j += stride) seq_lens[j] = 0;
  if (i == 0) {
    ctrl[0] = 0ull;
    ctrl[1] = (unsigned long long)num_blocks;
    ctrl[2] = (unsigned long long)num_blocks;
    ctrl[3] = 0ull;
  }
}

// Finished sequences give their blocks back: rows[i] names a table row; its live blocks (a
// contiguous run ending at the block of its last token) are pushed on the ring in logical
// order, its entries become -1 and its length 0. One CTA, pushes placed by a prefix sum in the
// order of `rows`, so the ring contents are deterministic. A row named more than once is released
// once, at its first mention (a repeat would otherwise count its blocks twice and hand the same
// physical block to two sequences later on): every entry is checked against the ones before it.
__global__ void __launch_bounds__(kPlanThreads)
release_rows_kernel(const int32_t* __restrict__ rows, int n_rows, int32_t* seq_lens,
                    int32_t* block_tables, int max_blocks, int B, int block_size, int32_t* ring,
                    unsigned long long* ctrl, int num_blocks, int32_t* status) {
  __shared__ int s_warp[33][3];
  const int tid = threadIdx.x;
  const int rpt = (n_rows + kPlanThreads - 1) / kPlanThreads;
  const int i_begin = min(tid * rpt, n_rows), i_end = min(i_begin + rpt, n_rows);
  auto live_run = [&](int b, int& first) {   // -> number of live blocks, first logical index
    const int L = seq_lens[b];
    int last = L > 0 ? (L - 1) / block_size : -1;
    if (last >= max_blocks) last = max_blocks - 1;
    const int32_t* row = block_tables + (int64_t)b * max_blocks;
    int j = last;
    while (j >= 0 && row[j] >= 0) --j;
    first = j + 1;
    return last - j;
  };
  auto repeated = [&](int i, int b) {
    for (int j = 0; j < i; ++j)
      if (rows[j] == b) return true;
    return false;
  };
  int v[3] = {0, 0, 0};
  for (int i = i_begin; i < i_end; ++i) {
    const int b = rows[i];
    if (b < 0 || b >= B) {
      raise_status(status, SBK_ST_BAD_SLOT);
      continue;
    }
    if (repeated(i, b)) continue;
    int first;
    v[0] += live_run(b, first);
  }
  int tot[3];
  block_scan3(v, tot, s_warp);
  const unsigned long long tail = ring ? ctrl[1] : 0ull;
  unsigned long long at = tail + (unsigned long long)v[0];
  for (int i = i_begin; i < i_end; ++i) {
    const int b = rows[i];
    if (b < 0 || b >= B || repeated(i, b)) continue;
    int first;
    const int cnt = live_run(b, first);
    int32_t* row = block_tables + (int64_t)b * max_blocks;
    for (int j = first; j < first + cnt; ++j) {
      if (ring) ring[(at++) % (unsigned long long)num_blocks] = row[j];
      row[j] = -1;
    }
    seq_lens[b] = 0;
  }
  if (tid == 0 && ring) ctrl[1] = tail + (unsigned long long)tot[0];
}

}  // namespace sbk

extern "C" int sbk_pool_init(int32_t* ring, uint64_t* ctrl, int num_blocks, int32_t* seq_lens,
                             int32_t* block_tables, int max_blocks, int B, void* stream) {
  using namespace sbk;
  if (!ring || !ctrl || num_blocks <= 0 || B < 0 || (block_tables && max_blocks <= 0)) {
    set_error("sbk_pool_init: ring, ctrl and num_blocks > 0 are required");
    return SBK_E_ARG;
  }
  if (reinterpret_cast<uintptr_t>(ctrl) & 7u) {
    set_error("sbk_pool_init: ctrl must be 8-byte aligned");
    return SBK_E_ALIGN;
  }
  pool_init_kernel<<<64, 256, 0, (cudaStream_t)stream>>>(
      ring, reinterpret_cast<unsigned long long*>(ctrl), num_blocks, seq_lens, block_tables,
      (int64_t)B * max_blocks, B);
  return check_launch("sbk_pool_init");
}

extern "C" int sbk_plan_step(const int32_t* n_new, int32_t* seq_lens, int32_t* block_tables,
                             int max_blocks, int B, int block_size, int window_left, int retire,
                             int32_t* ring, uint64_t* ctrl, int num_blocks, int64_t* slot_mapping,
                             int64_t* positions, int32_t* context_lens, int32_t* query_start_loc,
                             int T, int32_t* status, void* stream) {
  using namespace sbk;
  if (B < 0 || T < 0 || max_blocks <= 0 || block_size <= 0 || num_blocks <= 0) {
    set_error("sbk_plan_step: negative or zero dimension");
    return SBK_E_ARG;
  }
  if (retire < 0 || retire > 2) {
    set_error("sbk_plan_step: retire=%d is none of 0 (keep), 1 (retire), 2 (retire and trim idle rows)", retire);
    return SBK_E_ARG;
  }
  if (B == 0 && T == 0) return SBK_OK;
  if ((B > 0 && (!seq_lens || !block_tables)) || (T > 0 && !slot_mapping)) {
    set_error("sbk_plan_step: null pointer");
    return SBK_E_ARG;
  }
  if ((ring == nullptr) != (ctrl == nullptr)) {
    set_error("sbk_plan_step: ring and ctrl come together");
    return SBK_E_ARG;
  }
  if (n_new && !query_start_loc) {
    set_error("sbk_plan_step: n_new needs query_start_loc (it is written, and read back for the slots)");
    return SBK_E_ARG;
  }
  if (ctrl && (reinterpret_cast<uintptr_t>(ctrl) & 7u)) {
    set_error("sbk_plan_step: ctrl must be 8-byte aligned");
    return SBK_E_ALIGN;
  }
  PlanParams p;
  p.n_new = n_new;
  p.seq_lens = seq_lens;
  p.block_tables = block_tables;
  p.max_blocks = max_blocks;
  p.B = B;
  p.block_size = block_size;
  p.window_left = window_left;
  p.retire = retire;
  p.ring = ring;
  p.ctrl = reinterpret_cast<unsigned long long*>(ctrl);
  p.num_blocks = num_blocks;
  p.slot_mapping = slot_mapping;
  p.positions = positions;
  p.context_lens = context_lens;
  p.query_start_loc = query_start_loc;
  p.T = T;
  p.status = status;
  plan_step_kernel<<<1, kPlanThreads, 0, (cudaStream_t)stream>>>(p);
  return check_launch("sbk_plan_step");
}

extern "C" int sbk_release_rows(const int32_t* rows, int n_rows, int32_t* seq_lens,
                                int32_t* block_tables, int max_blocks, int B, int block_size,
                                int32_t* ring, uint64_t* ctrl, int num_blocks, int32_t* status,
                                void* stream) {
  using namespace sbk;
  if (n_rows < 0 || B < 0 || max_blocks <= 0 || block_size <= 0 || num_blocks <= 0) {
    set_error("sbk_release_rows: negative or zero dimension");
    return SBK_E_ARG;
  }
  if (n_rows == 0) return SBK_OK;
  if (!rows || !seq_lens || !block_tables || (ring == nullptr) != (ctrl == nullptr)) {
    set_error("sbk_release_rows: null pointer (ring and ctrl come together)");
    return SBK_E_ARG;
  }
  release_rows_kernel<<<1, kPlanThreads, 0, (cudaStream_t)stream>>>(
      rows, n_rows, seq_lens, block_tables, max_blocks, B, block_size, ring,
      reinterpret_cast<unsigned long long*>(ctrl), num_blocks, status);
  return check_launch("sbk_release_rows");
}
