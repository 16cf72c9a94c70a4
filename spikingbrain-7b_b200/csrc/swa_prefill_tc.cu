// Sliding-window attention for runs of query tokens over the paged K/V cache on the 5th-generation
// tensor cores: tcgen05.mma with both GEMMs' accumulators in tensor memory (TMEM), operands staged
// in shared memory by TMA tensor copies.
//
// A CTA owns 128 / G consecutive query tokens of one sequence and one kv head, G being the query
// heads per kv head: those queries times the G heads form the 128 rows of an MMA tile
// (row = query * G + head; 18 queries x 7 heads fill 126 of the 128 rows, where 16 queries x 8 head
// slots with one slot empty would fill 112), so one K/V tile in shared memory serves all of them.
// Keys are taken 128 at a time:
//     S[128 rows, 128 keys]  = Q . K^T      8 x tcgen05.mma (M128 N128 K16), accumulator in TMEM
//     softmax on S straight from TMEM; P -> bf16 head + bf16 remainder -> shared memory
//     O_t[128 rows, 128 dims] = P . V       16 x tcgen05.mma, fresh accumulator in TMEM
//     O += O_t (registers; rescaled by exp2(m_old - m_new) beforehand)
// Roles (608 threads):
//   warps 0-15 softmax / accumulate / epilogue. A TMEM lane (= row) can only be read by warps with
//              the same index mod 4, so warps w, w + 4, w + 8, w + 12 share the rows 32 (w mod 4) ... + 31:
//              each takes 32 keys of a tile and 32 dims of the output; they exchange their partial
//              row maxima through shared memory once a tile.
//   warps 16, 17  TMA producers of the K and of the V ring: walk the block table; a 128-key tile of K or V is 16 copies of 2 KiB
//              (one per 16-token block piece and 64-dim half), landing as two [128 keys][128 B]
//              panels with the 128-byte swizzle -- the canonical K-major layout for K in S = Q.K^T
//              and at once the canonical MN-major layout for V in O = P.V. K and V have rings of
//              their own (two slots each): a K slot is free as soon as its S is computed.
//   warp 18    allocates TMEM and issues the MMAs (one thread). S is double-buffered in TMEM, so
//              Q.K^T of tile t+1 runs while the softmax threads work on tile t, and P.V of tile t
//              runs while they compute the exponentials of tile t+1.
// Hand-offs are mbarriers; the tensor core signals them through tcgen05.commit. Every wait is bounded.
// The query at position p sees keys [p - window_left, p]; only tiles at the two ends of that range
// are masked. Sink (meta) keys, if any, come first as always-visible tiles.
#include "sbk_common.cuh"
#include "sbk_tma.cuh"
#include "sbk_tcgen05.cuh"
#include "swa_prefill_tc.cuh"

namespace sbk {
namespace prefill_tc {

constexpr int kD = 128;
constexpr int kChunk = 16;                    // keys per cache-block piece
constexpr int kTileKeys = 128;                // keys per MMA tile
constexpr int kTileChunks = kTileKeys / kChunk;
constexpr int kPanelBytes = 128 * 128;        // [128 rows][128 B]: 64 bf16 of every row
constexpr int kOperandBytes = 2 * kPanelBytes;   // a [128 x 128] bf16 operand: two panels
constexpr int kStages = 3;                    // slots of the K ring and of the V ring
constexpr int kQOff = 0;
constexpr int kKOff = kOperandBytes;                         // K ring
constexpr int kVOff = kKOff + kStages * kOperandBytes;       // V ring
constexpr int kBarOff = kVOff + kStages * kOperandBytes;     // 229376
constexpr int kXchOff = kBarOff + 128;                       // 4 x 128 floats: partial row maxima / sums
constexpr int kSmemBytes = kXchOff + 2048 + 64 + 768;        // + TMEM slot and flags; + alignment slack
constexpr int kSplit = 4;                     // softmax threads per row
constexpr int kCols = 128 / kSplit;           // keys of a tile / dims of the output per softmax thread
constexpr int kSoftmaxWarps = 4 * kSplit;
constexpr int kSoftmaxThreads = 32 * kSoftmaxWarps;
constexpr int kThreads = kSoftmaxThreads + 96;   // + K producer, V producer, MMA issuer
static_assert(kCols == 32, "a softmax thread reads its columns with one 32-column TMEM load");
constexpr int kTmemCols = 512;                // S0 / P0: columns [0,128), S1 / P1: [128,256), O: [256,384)
constexpr int kOCol = 256;
constexpr float kNegBig = -1.0e30f;

using namespace tc5;

// barrier among the kSplit warps that share the rows 32 q ... 32 q + 31 (named barriers 1..4)
__device__ __forceinline__ void row_bar(int q) {
  asm volatile("bar.sync %0, %1;" ::"r"(q + 1), "n"(32 * kSplit) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
swa_prefill_tc_kernel(const Params P, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_k2,
                      const __grid_constant__ CUtensorMap map_v2) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* const smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  if (sbase - smem_u32(smem_raw) > 768u) {   // the launch leaves room for this much padding only
    if (threadIdx.x == 0) raise_status(P.status, SBK_ST_WAIT_TIMEOUT);
    return;
  }
  // barriers: K ring full/empty, V ring full/empty; S ready, P ready and O ready, each one per S
  // buffer (tile t uses the barriers t & 1, phase t >> 1: with two barriers taking turns no waiter
  // can be two phases away from the phase it waits for, whatever the timing of the other side);
  // Q staged
  const uint32_t bar_kf = sbase + kBarOff, bar_ke = bar_kf + 8 * kStages;
  const uint32_t bar_vf = bar_ke + 8 * kStages, bar_ve = bar_vf + 8 * kStages;
  const uint32_t bar_s = bar_ve + 8 * kStages, bar_p = bar_s + 16;
  const uint32_t bar_q = sbase + kXchOff + 2048 + 8, bar_o = bar_q + 8;   // between the TMEM slot and the flags
  float* xch = reinterpret_cast<float*>(smem + kXchOff);                       // [2][128]
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kXchOff + 2048);
  volatile uint8_t* flags = smem + kXchOff + 2048 + 32;   // [0..7] tile t & 7 bad, [8] abort

  const int s = blockIdx.x / P.tiles_per_seq;
  // later query tiles see more keys: they are launched first, so the long items do not start last
  const int j = P.tiles_per_seq - 1 - (int)(blockIdx.x - s * P.tiles_per_seq);
  const int hk = blockIdx.y;
  const int qs = P.query_start_loc[s];
  const int n_q = P.query_start_loc[s + 1] - qs;
  const int kBQ = P.bq;         // queries per CTA
  if (j * kBQ >= n_q) return;   // whole CTA, before anything is allocated
  const int nq_tile = n_q - j * kBQ < kBQ ? n_q - j * kBQ : kBQ;
  const bool dense = P.k_start_loc != nullptr;
  const int k_start = dense ? P.k_start_loc[s] : 0;
  const int ctx = dense ? (P.k_start_loc[s + 1] - k_start) - n_q : P.context_lens[s];
  const bool full_attn = dense && P.noncausal;                // every key of the sequence, no window
  const int p0 = full_attn ? ctx + n_q - 1 : ctx + j * kBQ;   // position of the tile's first query
  const int key_lo = (P.window_left < 0 || full_attn) ? 0 : (p0 - P.window_left > 0 ? p0 - P.window_left : 0);
  const int key_hi = full_attn ? ctx + n_q : p0 + nq_tile;    // exclusive
  const int c_lo = key_lo / kChunk, c_hi = (key_hi - 1) / kChunk;
  const int n_chunks = c_hi - c_lo + 1;
  const int n_mt = (P.n_meta_chunks + kTileChunks - 1) / kTileChunks;   // sink-token tiles come first
  const int n_tiles = n_mt + (n_chunks + kTileChunks - 1) / kTileChunks;
  const int G = P.G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar_kf + 8 * i, 1);
      mbar_init(bar_ke + 8 * i, 1);
      mbar_init(bar_vf + 8 * i, 1);
      mbar_init(bar_ve + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s + 8 * i, 1);
      mbar_init(bar_p + 8 * i, kSoftmaxThreads);
      mbar_init(bar_o + 8 * i, 1);
    }
    mbar_init(bar_q, kSoftmaxThreads);
    for (int i = 0; i < 9; ++i) flags[i] = 0;
    fence_mbar_init();
  }
  // V panels start finite: a tile may be filled only in part (its other keys are masked, and a
  // zero probability must not meet a NaN), and what a slot holds later is older, finite data
  for (int i = threadIdx.x; i < kStages * kOperandBytes / 16; i += kThreads)
    *reinterpret_cast<uint4*>(smem + kVOff + i * 16) = make_uint4(0, 0, 0, 0);
  if (warp == kSoftmaxWarps + 2) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == kSoftmaxWarps || warp == kSoftmaxWarps + 1) {
    // ===== TMA producers: one warp per ring (K, V), so that a K tile never queues behind a V slot =====
    const int kind = warp - kSoftmaxWarps;   // 0: K ring, 1: V ring
    const int32_t* table = dense ? nullptr : P.block_tables + (int64_t)s * P.max_blocks;
    int64_t pb_lane = -1;
    int batch_c0 = 0;
    bool ok = true;
    for (int t = 0; ok && t < n_tiles; ++t) {
      const bool meta = t < n_mt;
      const int c0 = meta ? t * kTileChunks : c_lo + (t - n_mt) * kTileChunks;
      const int c_end = meta ? P.n_meta_chunks - 1 : c_hi;     // last chunk of this kind
      if (!meta && (t == n_mt || c0 + kTileChunks > batch_c0 + 32)) {      // one table read per 32 chunks
        batch_c0 = c0;
        const int c = c0 + lane;
        const int lb = (c * kChunk) / P.block_size;
        pb_lane = dense ? 0 : ((c <= c_hi && lb < P.max_blocks) ? (int64_t)table[lb] : -1);
      }
      const int slot = t % kStages, use = t / kStages;
      // lane -> one copy of 2 KiB: chunk (lane >> 1), 64-dim half (lane & 1); lanes 16-31 idle
      const int i = (lane >> 1) & 7, half = lane & 1;
      const int c = c0 + i;
      const bool active = lane < 16 && c <= c_end;
      int src_lane = c - batch_c0;
      src_lane = src_lane < 0 ? 0 : (src_lane > 31 ? 31 : src_lane);
      const int64_t pb_tab = __shfl_sync(0xffffffffu, pb_lane, src_lane);
      const int64_t pb = meta ? (int64_t)c : pb_tab;           // the sink tensors are their own block table
      bool bad = !meta && !dense && active && (pb < 0 || pb >= P.num_blocks);
      bad = __any_sync(0xffffffffu, bad);
      const int nvalid = c_end - c0 + 1 < kTileChunks ? c_end - c0 + 1 : kTileChunks;
      const int tin = meta ? 0 : (dense ? k_start + c * kChunk : (c * kChunk) % P.block_size);
      const uint32_t dst = sbase + (kind ? kVOff : kKOff) + slot * kOperandBytes + half * kPanelBytes + i * 2048;
      const CUtensorMap* map = meta ? (kind ? &map_v2 : &map_k2) : (kind ? &map_v : &map_k);
      const uint32_t bar_e = (kind ? bar_ve : bar_ke) + 8 * slot, bar_f = (kind ? bar_vf : bar_kf) + 8 * slot;
      if (use > 0 && !mbar_wait_bounded(bar_e, (use - 1) & 1)) ok = false;
      if (flags[8]) ok = false;
      if (!ok) break;
      if (lane == 0) {
        if (kind == 0) {
          flags[t & 7] = bad ? 1 : 0;
          if (bad) raise_status(P.status, SBK_ST_BAD_BLOCK);
        }
        mbar_arrive_expect_tx(bar_f, bad ? 0u : (uint32_t)nvalid * 2u * 2048u);
      }
      __syncwarp();
      if (!bad && active) {
        if (P.tile_copy) tma_load_4d(dst, map, 0, tin, hk * 2 + half, (int)pb, bar_f);
        else tma_load_4d(dst, map, 0, hk * 2 + half, tin, (int)pb, bar_f);
      }
    }
    if (!ok && lane == 0 && !flags[8]) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); flags[8] = 1; }
  } else if (warp == kSoftmaxWarps + 2) {
    // ================================= MMA issuer =================================
    const uint32_t idesc_qk = instr_desc(0), idesc_pv = instr_desc(1);
    const uint32_t q_addr = sbase + kQOff;
    // S(t) = Q . K(t)^T into S buffer t & 1; frees the K slot
    auto issue_qk = [&](int t) -> bool {
      const int slot = t % kStages;
      if (!mbar_wait_bounded(bar_kf + 8 * slot, (t / kStages) & 1) || flags[8]) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t k_addr = sbase + kKOff + slot * kOperandBytes;
#pragma unroll
        for (int k = 0; k < 8; ++k) {   // 8 steps of 16 dims: 0-3 in the first 64-dim panel, 4-7 in the second
          const uint32_t off = (k >> 2) * kPanelBytes + (k & 3) * 32;
          umma_bf16(tmem + (t & 1) * 128, smem_desc(q_addr + off, 16), smem_desc(k_addr + off, 16), idesc_qk, k > 0);
        }
        umma_commit(bar_s + 8 * (t & 1));
        umma_commit(bar_ke + 8 * slot);
      }
      __syncwarp();
      return true;
    };
    // Q is written by the softmax threads
    bool ok = mbar_wait_bounded(bar_q, 0);
    tc_fence_after();
    ok = ok && issue_qk(0);
    for (int t = 0; ok && t < n_tiles; ++t) {
      // the next tile's scores are computed while the softmax threads work on this one
      if (t + 1 < n_tiles) ok = issue_qk(t + 1);
      if (!ok) break;
      // P of this tile (and with it: S(t) read, O_t of the previous tile read)
      const int slot = t % kStages;
      ok = mbar_wait_bounded(bar_p + 8 * (t & 1), (t >> 1) & 1) && mbar_wait_bounded(bar_vf + 8 * slot, (t / kStages) & 1);
      if (!ok || flags[8]) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v_addr = sbase + kVOff + slot * kOperandBytes;
#pragma unroll
        for (int k = 0; k < 8; ++k) {   // 8 steps of 16 keys: 8 TMEM columns of P (head, then remainder), 16 rows of V
          const uint64_t vd = smem_desc(v_addr + k * 2048, kPanelBytes);
          umma_bf16_ts(tmem + kOCol, tmem + (t & 1) * 128 + k * 8, vd, idesc_pv, (t > 0) || (k > 0));
          umma_bf16_ts(tmem + kOCol, tmem + (t & 1) * 128 + 64 + k * 8, vd, idesc_pv, 1);
        }
        umma_commit(bar_ve + 8 * slot);
        umma_commit(bar_o + 8 * (t & 1));
      }
      __syncwarp();
    }
    if (!ok && lane == 0 && !flags[8]) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); flags[8] = 1; }
  } else {
    // ====================== softmax / accumulate / epilogue ======================
    constexpr int kCh = kCols / 8;         // 16-byte chunks of bf16 per thread and row
    const int r = (warp & 3) * 32 + lane;  // row of the MMA tile = TMEM lane
    const int part = warp >> 2;            // which kCols keys of a tile / which kCols dims of the output
    const int panel = (part * kCols) >> 6, ch0 = ((part * kCols) & 63) >> 3;
    const int ql = r / G, slot_h = r - ql * G;   // rows past bq * G land on ql == bq: never a query of the tile
    const bool row_ok = ql < nq_tile;
    const int p_row = full_attn ? p0 : p0 + ql;   // position of this row's query (its last visible key)
    const int lo_row = (P.window_left < 0 || full_attn) ? 0 : (p_row - P.window_left > 0 ? p_row - P.window_left : 0);
    // ---- Q rows into the swizzled K-major panels (this thread: its kCols dims) ----
    {
      const uint4* qp = reinterpret_cast<const uint4*>(
          P.q + (int64_t)(qs + j * kBQ + ql) * P.q_tok_stride + (int64_t)(hk * G + slot_h) * kD + part * kCols);
#pragma unroll
      for (int c = 0; c < kCh; ++c) {
        const uint4 v = row_ok ? qp[c] : make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(smem + kQOff + panel * kPanelBytes + swz(r, ch0 + c)) = v;
      }
      fence_proxy_async_smem();
      mbar_arrive(bar_q);                  // Q is in place
    }
    float m_run = -INFINITY, l_run = 0.f;
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    __nv_bfloat16* xm = reinterpret_cast<__nv_bfloat16*>(xch);   // [kSplit][128] partial row maxima
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      ok = mbar_wait_bounded(bar_s + 8 * (t & 1), (t >> 1) & 1);
      if (!ok || flags[8]) break;
      tc_fence_after();
      // ---- my kCols scores of this row ----
      uint32_t sr[32];
      tmem_ld32_issue(t_lane + (t & 1) * 128 + part * kCols, sr);
      const bool meta = t < n_mt;
      const int tb = meta ? t * kTileKeys : (c_lo + (t - n_mt) * kTileChunks) * kChunk;   // first key of the tile
      // columns (of my part) this row may see: [v_lo, v_hi)
      int v_lo, v_hi;
      if (meta) { v_lo = 0; v_hi = P.n_meta_chunks * kChunk - tb; }
      else { v_lo = lo_row - tb; v_hi = p_row + 1 - tb; }
      v_lo -= part * kCols; v_hi -= part * kCols;
      v_lo = v_lo < 0 ? 0 : v_lo;
      v_hi = v_hi > kCols ? kCols : v_hi;
      if (flags[t & 7]) v_hi = 0;
      const bool full = v_lo == 0 && v_hi == kCols;
      tmem_ld_fence(sr);
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (full) {
#pragma unroll
        for (int i = 0; i < kCols; i += 2)
          mx[(i >> 1) & 3] = fmax3(mx[(i >> 1) & 3], __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
      } else {
#pragma unroll
        for (int i = 0; i < kCols; ++i)
          if (i >= v_lo && i < v_hi) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(sr[i]));
      }
      // The threads of a row must agree on the offset m exactly, but m only has to be an upper
      // bound of the row's scores, not the maximum itself: the partial maxima are exchanged rounded
      // UP to bf16 (every side uses the rounded values).
      row_bar(warp & 3);                   // everyone has read the previous tile's maxima
      xm[part * 128 + r] = __float2bfloat16_ru(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])));
      row_bar(warp & 3);
      float both = -INFINITY;
#pragma unroll
      for (int q2 = 0; q2 < kSplit; ++q2) both = fmaxf(both, __bfloat162float(xm[q2 * 128 + r]));
      // The offset in use moves only when the row maximum has grown by more than 2^8 (the
      // probabilities then stay below 256, far inside fp32 and bf16 range): O, which accumulates in
      // tensor memory, has to be rescaled only then, which after the first tile is rare.
      const float cand = fmaxf(m_run, both * P.scale_log2);
      const bool move = cand > m_run + 8.f;   // also the first visible key of a row (m_run = -inf)
      const float m_new = move ? cand : m_run;
      const float m_s = fmaxf(m_new, kNegBig);
      const float alpha = move ? fast_exp2(m_run - m_s) : 1.f;
      m_run = m_new;
      // ---- probabilities, in place of the scores ----
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t hi[16], lo[16];
      if (full) {
        const f32x2 sc2 = pack2(P.scale_log2, P.scale_log2), nm2 = pack2(-m_s, -m_s);
        f32x2 la = 0ull, lb = 0ull;
#pragma unroll
        for (int i = 0; i < kCols; i += 4) {
          float x0, x1, x2, x3;
          unpack2(ffma2(pack2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), sc2, nm2), x0, x1);
          unpack2(ffma2(pack2(__uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3])), sc2, nm2), x2, x3);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1), p2 = fast_exp2(x2), p3 = fast_exp2(x3);
          la = fadd2(la, pack2(p0, p1));
          lb = fadd2(lb, pack2(p2, p3));
          // split here, among the exponentials: the special-function unit paces those, and the
          // conversions fill the issue slots it leaves
          split_bf16x2(p0, p1, hi[i >> 1], lo[i >> 1]);
          split_bf16x2(p2, p3, hi[(i >> 1) + 1], lo[(i >> 1) + 1]);
        }
        unpack2(la, ls[0], ls[1]);
        unpack2(lb, ls[2], ls[3]);
      } else {
#pragma unroll
        for (int i = 0; i < kCols; ++i) {
          float pv = fast_exp2(__uint_as_float(sr[i]) * P.scale_log2 - m_s);
          if (i < v_lo || i >= v_hi) pv = 0.f;
          sr[i] = __float_as_uint(pv);
          ls[i & 3] += pv;
        }
#pragma unroll
        for (int e = 0; e < 16; ++e)
          split_bf16x2(__uint_as_float(sr[2 * e]), __uint_as_float(sr[2 * e + 1]), hi[e], lo[e]);
      }
      l_run = l_run * alpha + (ls[0] + ls[1]) + (ls[2] + ls[3]);
      // ---- rescale O (my kCols dims of this row) where the offset moved; the GEMMs that wrote it must be done ----
      if (__any_sync(0xffffffffu, t > 0 && alpha != 1.f)) {
        ok = mbar_wait_bounded(bar_o + 8 * ((t - 1) & 1), ((t - 1) >> 1) & 1);
        if (!ok || flags[8]) break;
        tc_fence_after();
        uint32_t orr[32];
        tmem_ld32_issue(t_lane + kOCol + part * kCols, orr);
        tmem_ld_fence(orr);
#pragma unroll
        for (int i = 0; i < kCols; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
        tmem_st32(t_lane + kOCol + part * kCols, orr);
      }
      // The cache block that holds the newest key also holds slots nobody has written yet; their V
      // bits may be anything, and a zero probability times a NaN is a NaN. Clear those rows of the
      // tile (at most 15, in the chunk of the last key) before the second GEMM reads them.
      if (!meta && tb + kTileKeys > key_hi) {
        if (!mbar_wait_bounded(bar_vf + 8 * (t % kStages), (t / kStages) & 1)) { ok = false; break; }
        const int row0 = key_hi - tb;
        const int row1 = ((key_hi + kChunk - 1) / kChunk) * kChunk - tb;
        uint8_t* vbase = smem + kVOff + (t % kStages) * kOperandBytes;
        for (int i = threadIdx.x; i < (row1 - row0) * 16; i += kSoftmaxThreads) {
          const int row = row0 + (i >> 4), c = i & 15;
          *reinterpret_cast<uint4*>(vbase + (c >> 3) * kPanelBytes + row * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
      }
      // ---- P to tensor memory, where the second GEMM reads its A operand: packed bf16 pairs (key 2c in
      //      the low half of column c), as a bf16 head plus a bf16 remainder (two MMAs per step): with the
      //      head alone the rounding of the probabilities shows in the output (mean relative error
      //      against an fp32 softmax just over 1e-3) ----
      {
        // P takes the place of S in the same TMEM buffer (every thread of the row has its scores in
        // registers since the exchange of the maxima): head in columns [0,64), remainder in [64,128)
        tmem_st16(t_lane + (t & 1) * 128 + part * (kCols / 2), hi);
        tmem_st16(t_lane + (t & 1) * 128 + 64 + part * (kCols / 2), lo);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_p + 8 * (t & 1));    // tile t
    }
    if (ok && !flags[8]) {
      ok = mbar_wait_bounded(bar_o + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1);
      if (ok) {
        tc_fence_after();
        uint32_t orr[32];
        tmem_ld32_issue(t_lane + kOCol + part * kCols, orr);
        tmem_ld_fence(orr);
        float acc[kCols];
#pragma unroll
        for (int i = 0; i < kCols; ++i) acc[i] = __uint_as_float(orr[i]);
        // the threads of a row hold partial sums of the probabilities
        row_bar(warp & 3);                 // the last exchange of maxima has been read by everyone
        float* xl = xch;                                         // [kSplit][128]
        xl[part * 128 + r] = l_run;
        row_bar(warp & 3);
        float l_tot = 0.f;
#pragma unroll
        for (int q2 = 0; q2 < kSplit; ++q2) l_tot += xl[q2 * 128 + r];
        if (row_ok) {
          const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
          uint4* op = reinterpret_cast<uint4*>(
              P.out + (int64_t)(qs + j * kBQ + ql) * P.out_tok_stride + (int64_t)(hk * G + slot_h) * kD + part * kCols);
#pragma unroll
          for (int c = 0; c < kCh; ++c) {
            uint4 w;
            w.x = pack_bf16x2(acc[c * 8 + 0] * inv, acc[c * 8 + 1] * inv);
            w.y = pack_bf16x2(acc[c * 8 + 2] * inv, acc[c * 8 + 3] * inv);
            w.z = pack_bf16x2(acc[c * 8 + 4] * inv, acc[c * 8 + 5] * inv);
            w.w = pack_bf16x2(acc[c * 8 + 6] * inv, acc[c * 8 + 7] * inv);
            op[c] = w;
          }
        }
      }
    }
    if (!ok && lane == 0 && !flags[8]) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); flags[8] = 1; }
  }

  // ---- teardown: everyone meets here, then the allocating warp returns the TMEM columns ----
  if (flags[8]) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);   // let copies and MMAs in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kSoftmaxWarps + 2) tmem_dealloc(tmem, kTmemCols);
}

int launch(const Params& P, int kvh, const CUtensorMap& map_k, const CUtensorMap& map_v,
           const CUtensorMap& map_k2, const CUtensorMap& map_v2, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(swa_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) {
      set_error("sbk_swa_prefill: cannot opt in to %d bytes of shared memory: %s", kSmemBytes, cudaGetErrorString(e));
      return SBK_E_LAUNCH;
    }
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid(P.n_seqs * P.tiles_per_seq, kvh);
  swa_prefill_tc_kernel<<<grid, kThreads, kSmemBytes, stream>>>(P, map_k, map_v, map_k2, map_v2);
  return check_launch("sbk_swa_prefill");
}

}  // namespace prefill_tc
}  // namespace sbk
