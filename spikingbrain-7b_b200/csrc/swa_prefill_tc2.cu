// Sliding-window attention for runs of query tokens over the paged K/V cache on the 5th-generation
// tensor cores, two query tiles per CTA taking turns.
//
// A CTA owns 2 x (128 / G) consecutive query tokens of one sequence and one kv head, as two MMA
// tiles A and B of 128 rows each (row = query * G + head, as in the one-tile kernel). Both read the
// same K/V tiles in shared memory. One thread owns one row: no exchange between threads anywhere in
// the softmax, and while the four warps of tile A work on their scores the tensor core computes for
// tile B and the other way round:
//     tensor core:  S_A(0) S_B(0) | P_A(0).V S_A(1) | P_B(0).V S_B(1) | P_A(1).V S_A(2) | ...
//     warps 0-3  :  softmax A(0)  |                 | softmax A(1)    |                 ...
//     warps 4-7  :                | softmax B(0)    |                 | softmax B(1)    ...
// so the latencies inside a softmax pass (tensor-memory loads and stores, the dependent chains
// around the row maximum) are covered by the other tile's work instead of by more threads per row.
// Tensor memory (512 columns): S_A / P_A [0,128), S_B / P_B [128,256), O_A [256,384), O_B [384,512).
// The second GEMM runs in fp16: P takes the place of S chunk by chunk as packed fp16 pairs (the 32
// scores in columns [32c, 32c+32) become the 16 columns [32c, 32c+16)), eleven significant bits where
// bf16 has eight -- one MMA per step where a bf16 P needs a head and a remainder to hold the 1e-3
// bar -- and the V tile, bf16 in the cache, is converted to fp16 in shared memory once it has landed
// (exact for magnitudes in [2^-14, 65504]; smaller ones lose bits no output shows; a larger one
// raises SBK_ST_VALUE_RANGE, its row of the output is not finite, and the one-tile kernel serves
// such a cache). Both tiles read the converted V.
// Roles (512 threads): warps 0-3 softmax / epilogue of tile A, warps 4-7 of tile B, warp 8 TMA
// producer of the K ring, warp 9 of the V ring, warp 10 allocates tensor memory and issues the MMAs,
// warps 11-15 convert V.
// Every wait is bounded. Masks, sink tiles, dense and non-causal modes as in the one-tile kernel.
#include "sbk_common.cuh"
#include "sbk_tma.cuh"
#include "sbk_tcgen05.cuh"
#include "swa_prefill_tc.cuh"

namespace sbk {
namespace prefill_tc2 {

using prefill_tc::Params;

constexpr int kD = 128;
constexpr int kChunk = 16;                    // keys per cache-block piece
constexpr int kTileKeys = 128;                // keys per MMA tile
constexpr int kTileChunks = kTileKeys / kChunk;
constexpr int kPanelBytes = 128 * 128;        // [128 rows][128 B]: 64 bf16 of every row
constexpr int kOperandBytes = 2 * kPanelBytes;   // a [128 x 128] bf16 operand: two panels
constexpr int kStagesK = 2, kStagesV = 3;     // slots of the K ring and of the V ring
constexpr int kQOff = 0;                                     // Q_A, Q_B
constexpr int kKOff = 2 * kOperandBytes;
constexpr int kVOff = kKOff + kStagesK * kOperandBytes;
constexpr int kBarOff = kVOff + kStagesV * kOperandBytes;    // 229376
constexpr int kSmemBytes = kBarOff + 256 + 1024;             // barriers, TMEM slot, flags; + alignment slack
constexpr int kSoftmaxWarps = 8;
constexpr int kConvWarps = 5;   // (2: 5.09 ms, 4: 4.42, 5: 4.37, 6 and its spills: 4.65 on 8 x 8192 tokens)
constexpr int kThreads = 32 * (kSoftmaxWarps + 3 + kConvWarps);
constexpr int kTmemCols = 512;
constexpr int kOCol = 256;
constexpr float kNegBig = -1.0e30f;

using namespace tc5;

__global__ void __launch_bounds__(kThreads, 1)
swa_prefill_pair_kernel(const Params P, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_k2,
                        const __grid_constant__ CUtensorMap map_v2) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* const smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  // barriers: K ring full/empty, V ring full/empty; per tile (A, B): S ready, P ready; Q staged; all
  // MMAs done. The S and P barriers of a tile take turns strictly (S(t+1) is issued only after P(t)
  // was seen, P(t+1) written only after S(t+1) was seen), so one barrier each and phase t & 1.
  const uint32_t bar_kf = sbase + kBarOff, bar_ke = bar_kf + 8 * kStagesK;
  const uint32_t bar_vf = bar_ke + 8 * kStagesK, bar_ve = bar_vf + 8 * kStagesV;
  const uint32_t bar_s = bar_ve + 8 * kStagesV, bar_p = bar_s + 16;   // bar_p: [tile][half of the keys]
  const uint32_t bar_q = bar_p + 32, bar_done = bar_q + 8;
  const uint32_t bar_vc = bar_done + 8;                               // V converted, per slot of the ring
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kBarOff + 192);
  volatile uint8_t* flags = smem + kBarOff + 208;   // [0..7] tile t & 7 bad, [8] abort, [16..23] the same from the V producer

  const int s = blockIdx.x / P.tiles_per_seq;
  // later query tiles see more keys: they are launched first, so the long items do not start last
  const int j = P.tiles_per_seq - 1 - (int)(blockIdx.x - s * P.tiles_per_seq);
  const int hk = blockIdx.y;
  const int qs = P.query_start_loc[s];
  const int n_q = P.query_start_loc[s + 1] - qs;
  const int kBQ = P.bq;             // queries per tile; the CTA owns two tiles
  if (j * 2 * kBQ >= n_q) return;   // whole CTA, before anything is allocated
  const int nq_pair = n_q - j * 2 * kBQ < 2 * kBQ ? n_q - j * 2 * kBQ : 2 * kBQ;
  const bool has_b = nq_pair > kBQ;   // a run's last pair may have tile A only
  const bool dense = P.k_start_loc != nullptr;
  const int k_start = dense ? P.k_start_loc[s] : 0;
  const int ctx = dense ? (P.k_start_loc[s + 1] - k_start) - n_q : P.context_lens[s];
  const bool full_attn = dense && P.noncausal;                    // every key of the sequence, no window
  const int p0 = full_attn ? ctx + n_q - 1 : ctx + j * 2 * kBQ;   // position of the pair's first query
  const int key_lo = (P.window_left < 0 || full_attn) ? 0 : (p0 - P.window_left > 0 ? p0 - P.window_left : 0);
  const int key_hi = full_attn ? ctx + n_q : p0 + nq_pair;        // exclusive
  const int c_lo = key_lo / kChunk, c_hi = (key_hi - 1) / kChunk;
  const int n_chunks = c_hi - c_lo + 1;
  const int n_mt = (P.n_meta_chunks + kTileChunks - 1) / kTileChunks;   // sink-token tiles come first
  const int n_tiles = n_mt + (n_chunks + kTileChunks - 1) / kTileChunks;
  const int G = P.G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStagesK; ++i) {
      mbar_init(bar_kf + 8 * i, 1);
      mbar_init(bar_ke + 8 * i, 1);
    }
    for (int i = 0; i < kStagesV; ++i) {
      mbar_init(bar_vf + 8 * i, 1);
      mbar_init(bar_ve + 8 * i, 1);
      mbar_init(bar_vc + 8 * i, kConvWarps);
    }
    for (int i = 0; i < 2; ++i) mbar_init(bar_s + 8 * i, 1);
    for (int i = 0; i < 4; ++i) mbar_init(bar_p + 8 * i, 4);      // one arrival per warp of the tile
    mbar_init(bar_q, kSoftmaxWarps);
    mbar_init(bar_done, 1);
    for (int i = 0; i < 24; ++i) flags[i] = 0;
    fence_mbar_init();
  }
  // V panels start finite: a tile may be filled only in part (its other keys are masked, and a
  // zero probability must not meet a NaN), and what a slot holds later is older, finite data
  for (int i = threadIdx.x; i < kStagesV * kOperandBytes / 16; i += kThreads)
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
    const int stages = kind ? kStagesV : kStagesK;
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
      const int slot = t % stages, use = t / stages;
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
        } else {
          flags[16 + (t & 7)] = bad ? 1 : 0;     // for the converters: nothing lands in this slot
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
    const uint32_t idesc_qk = instr_desc(0), idesc_pv = instr_desc_f16(1);
    // S_X(t) = Q_X . K(t)^T
    auto issue_s = [&](int X, int t) {
      if (lane == 0) {
        const uint32_t q_addr = sbase + kQOff + X * kOperandBytes;
        const uint32_t k_addr = sbase + kKOff + (t % kStagesK) * kOperandBytes;
#pragma unroll
        for (int k = 0; k < 8; ++k) {   // 8 steps of 16 dims: 0-3 in the first 64-dim panel, 4-7 in the second
          const uint32_t off = (k >> 2) * kPanelBytes + (k & 3) * 32;
          umma_bf16(tmem + X * 128, smem_desc(q_addr + off, 16), smem_desc(k_addr + off, 16), idesc_qk, k > 0);
        }
        umma_commit(bar_s + 8 * X);
      }
      __syncwarp();
    };
    // O_X += P_X(t) . V(t): 8 steps of 16 keys; a step's P is 8 columns of packed fp16 pairs at the
    // head of the 32 columns its scores came from
    auto issue_pv = [&](int X, int t, int half) {
      if (lane == 0) {
        const uint32_t v_addr = sbase + kVOff + (t % kStagesV) * kOperandBytes;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const int k = 4 * half + k4;
          const uint64_t vd = smem_desc(v_addr + k * 2048, kPanelBytes);
          const uint32_t a = tmem + X * 128 + 32 * (k >> 1) + 8 * (k & 1);
          umma_bf16_ts(tmem + kOCol + X * 128, a, vd, idesc_pv, (t > 0) || (k > 0));
        }
      }
      __syncwarp();
    };
    auto commit = [&](uint32_t bar) {
      if (lane == 0) umma_commit(bar);
      __syncwarp();
    };
    auto k_full = [&](int t) { return mbar_wait_bounded(bar_kf + 8 * (t % kStagesK), (t / kStagesK) & 1) && !flags[8]; };
    bool ok = mbar_wait_bounded(bar_q, 0) && k_full(0);   // Q is written by the softmax threads
    if (ok) {
      tc_fence_after();
      issue_s(0, 0);
      if (has_b) issue_s(1, 0);
      commit(bar_ke);
    }
    for (int t = 0; ok && t < n_tiles; ++t) {
      const int vslot = t % kStagesV;
      const bool more = t + 1 < n_tiles;
      // P_A(t), the first 64 keys and then the rest (the product of the first half runs while the
      // softmax threads still work on the second): with it S_A(t) is read, so S_A(t+1) may follow
      ok = mbar_wait_bounded(bar_p, t & 1) && mbar_wait_bounded(bar_vc + 8 * vslot, (t / kStagesV) & 1);
      if (!ok || flags[8]) break;
      tc_fence_after();
      issue_pv(0, t, 0);
      ok = mbar_wait_bounded(bar_p + 8, t & 1);
      if (!ok || flags[8]) break;
      tc_fence_after();
      issue_pv(0, t, 1);
      if (!has_b) commit(bar_ve + 8 * vslot);
      if (more) {
        ok = k_full(t + 1);
        if (!ok) break;
        tc_fence_after();
        issue_s(0, t + 1);
        if (!has_b) commit(bar_ke + 8 * ((t + 1) % kStagesK));
      }
      if (has_b) {
        ok = mbar_wait_bounded(bar_p + 16, t & 1);
        if (!ok || flags[8]) break;
        tc_fence_after();
        issue_pv(1, t, 0);
        ok = mbar_wait_bounded(bar_p + 24, t & 1);
        if (!ok || flags[8]) break;
        tc_fence_after();
        issue_pv(1, t, 1);
        commit(bar_ve + 8 * vslot);
        if (more) {
          issue_s(1, t + 1);
          commit(bar_ke + 8 * ((t + 1) % kStagesK));
        }
      }
    }
    if (ok) commit(bar_done);
    if (!ok && lane == 0 && !flags[8]) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); flags[8] = 1; }
  } else if (warp > kSoftmaxWarps + 2) {
    // ===== V converters: the tile that landed as bf16 becomes fp16 in place (the layout stays: the
    //       conversion is element by element), then the rows past the newest key are cleared =====
    const int ct = threadIdx.x - 32 * (kSoftmaxWarps + 3);     // 0 .. 32 * kConvWarps - 1
    bool ok = true;
    uint32_t top = 0;                                          // largest magnitude seen (bf16 bits, per half)
    for (int t = 0; t < n_tiles; ++t) {
      const int slot = t % kStagesV;
      ok = mbar_wait_bounded(bar_vf + 8 * slot, (t / kStagesV) & 1);
      if (!ok || flags[8]) break;
      const bool meta = t < n_mt;
      const int c0 = meta ? t * kTileChunks : c_lo + (t - n_mt) * kTileChunks;
      const int c_end = meta ? P.n_meta_chunks - 1 : c_hi;
      const int nvalid = c_end - c0 + 1 < kTileChunks ? c_end - c0 + 1 : kTileChunks;
      uint8_t* const vbase = smem + kVOff + slot * kOperandBytes;
      if (!flags[16 + (t & 7)]) {
        // The chunks that landed: rows [0, 16 nvalid) of both panels, 128 B per row (what the slot
        // holds beyond them is older, already converted data). The cache block that holds the newest
        // key also holds slots nobody has written yet; their bits may be anything, and a zero
        // probability times a NaN is a NaN: those rows (at most 15, in the chunk of the last key) are
        // cleared instead of converted.
        const int tb = c0 * kChunk;
        const bool tail = !meta && tb + kTileKeys > key_hi;
        const int rows = tail ? key_hi - tb : nvalid * kChunk;
        const int n16 = rows * 8;                              // 16-byte pieces per panel
        for (int i = ct; i < 2 * n16; i += 32 * kConvWarps) {
          uint4* const ptr = reinterpret_cast<uint4*>(vbase + (i >= n16 ? kPanelBytes + (i - n16) * 16 : i * 16));
          uint4 w = *ptr;
          uint32_t x[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            top = __vmaxu2(top, x[e] & 0x7fff7fffu);
            x[e] = bf16x2_to_f16x2(x[e]);
          }
          *ptr = make_uint4(x[0], x[1], x[2], x[3]);
        }
        if (tail) {
          const int row1 = ((key_hi + kChunk - 1) / kChunk) * kChunk - tb;
          for (int i = ct; i < (row1 - rows) * 16; i += 32 * kConvWarps) {
            const int row = rows + (i >> 4), c = i & 15;
            *reinterpret_cast<uint4*>(vbase + (c >> 3) * kPanelBytes + row * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_vc + 8 * slot);
    }
    // bf16 bits of 0x4780 or more: a magnitude of 2^16 or more (or inf / NaN), which fp16 does not hold
    if (__any_sync(0xffffffffu, (top & 0xffffu) >= 0x4780u || (top >> 16) >= 0x4780u) && lane == 0)
      raise_status(P.status, SBK_ST_VALUE_RANGE);
    if (!ok && lane == 0 && !flags[8]) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); flags[8] = 1; }
  } else {
    // ====================== softmax / epilogue: one thread per row ======================
    const int X = warp >> 2;               // tile A or B
    const int r = (warp & 3) * 32 + lane;  // row of the MMA tile = TMEM lane
    const int ql = r / G, slot_h = r - ql * G;   // rows past bq * G land on ql == bq: never a query of the tile
    const int nq_tile = X ? nq_pair - kBQ : (nq_pair < kBQ ? nq_pair : kBQ);
    const bool row_ok = ql < nq_tile;      // (nq_tile <= 0 for an absent tile B)
    const int q_tok = j * 2 * kBQ + X * kBQ + ql;   // of the run
    const int p_row = full_attn ? p0 : p0 + X * kBQ + ql;   // position of this row's query (its last visible key)
    const int lo_row = (P.window_left < 0 || full_attn) ? 0 : (p_row - P.window_left > 0 ? p_row - P.window_left : 0);
    // ---- the Q row into the swizzled K-major panels of its tile ----
    {
      const uint4* qp = reinterpret_cast<const uint4*>(P.q + (int64_t)(qs + q_tok) * P.q_tok_stride +
                                                       (int64_t)(hk * G + slot_h) * kD);
      uint4 v[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) v[c] = row_ok ? qp[c] : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int c = 0; c < 16; ++c)
        *reinterpret_cast<uint4*>(smem + kQOff + X * kOperandBytes + (c >> 3) * kPanelBytes + swz(r, c & 7)) = v[c];
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_q);   // this warp's rows are in place
    }
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t s_col = t_lane + X * 128, o_col = t_lane + kOCol + X * 128;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    if (X == 0 || has_b) {
      for (int t = 0; t < n_tiles; ++t) {
        ok = mbar_wait_bounded(bar_s + 8 * X, t & 1);
        if (!ok || flags[8]) break;
        tc_fence_after();
        const bool meta = t < n_mt;
        const int tb = meta ? t * kTileKeys : (c_lo + (t - n_mt) * kTileChunks) * kChunk;   // first key of the tile
        // columns this row may see: [v_lo, v_hi)
        int v_lo, v_hi;
        if (meta) { v_lo = 0; v_hi = P.n_meta_chunks * kChunk - tb; }
        else { v_lo = lo_row - tb; v_hi = p_row + 1 - tb; }
        v_lo = v_lo < 0 ? 0 : v_lo;
        v_hi = v_hi > kTileKeys ? kTileKeys : v_hi;
        if (flags[t & 7]) v_hi = 0;
        const bool full = __all_sync(0xffffffffu, v_lo == 0 && v_hi == kTileKeys);   // the warp takes one path
        // ---- first pass: the row maximum, 64 columns at a time ----
        float both;
        {
          float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            uint32_t s0[32], s1[32];
            tmem_ld32_issue(s_col + 64 * hf, s0);
            tmem_ld32_issue(s_col + 64 * hf + 32, s1);
            tmem_ld_fence(s0); tmem_ld_fence(s1);
            if (full) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                mx[0] = fmax3(mx[0], __uint_as_float(s0[i]), __uint_as_float(s0[i + 1]));
                mx[1] = fmax3(mx[1], __uint_as_float(s0[i + 2]), __uint_as_float(s0[i + 3]));
                mx[2] = fmax3(mx[2], __uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
                mx[3] = fmax3(mx[3], __uint_as_float(s1[i + 2]), __uint_as_float(s1[i + 3]));
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int col = 64 * hf + i;
                if (col >= v_lo && col < v_hi) mx[i & 1] = fmaxf(mx[i & 1], __uint_as_float(s0[i]));
                if (col + 32 >= v_lo && col + 32 < v_hi) mx[2 + (i & 1)] = fmaxf(mx[2 + (i & 1)], __uint_as_float(s1[i]));
              }
            }
          }
          both = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        }
        // The offset in use moves only when the row maximum has grown by more than 2^8 (the
        // probabilities then stay below 256, far inside fp32 and bf16 range): O, which accumulates in
        // tensor memory, has to be rescaled only then, which after the first tile is rare.
        const float cand = fmaxf(m_run, both * P.scale_log2);
        const bool move = cand > m_run + 8.f;   // also the first visible key of a row (m_run = -inf)
        const float m_new = move ? cand : m_run;
        const float m_s = fmaxf(m_new, kNegBig);
        const float alpha = move ? fast_exp2(m_run - m_s) : 1.f;
        m_run = m_new;
        // ---- rescale O where the offset moved. The products that wrote it are done: S_X(t) was
        //      issued behind P_X(t-1).V and its completion has been seen above. ----
        if (__any_sync(0xffffffffu, t > 0 && alpha != 1.f)) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t orr[32];
            tmem_ld32_issue(o_col + 32 * c, orr);
            tmem_ld_fence(orr);
#pragma unroll
            for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
            tmem_st32(o_col + 32 * c, orr);
          }
        }
        // ---- second pass: probabilities in place of the scores, 64 columns at a time, each half
        //      reported as soon as it is stored (its product runs while the other half is worked on) ----
        float ls[4] = {0.f, 0.f, 0.f, 0.f};
        const f32x2 sc2 = pack2(P.scale_log2, P.scale_log2), nm2 = pack2(-m_s, -m_s);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t sa[32], sb[32];
          tmem_ld32_issue(s_col + 64 * hf, sa);
          tmem_ld32_issue(s_col + 64 * hf + 32, sb);
          tmem_ld_fence(sa); tmem_ld_fence(sb);
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            uint32_t (&sr)[32] = cc ? sb : sa;
            const int col0 = 64 * hf + 32 * cc;
            uint32_t ph[16];               // packed fp16 pairs, key 2e in the low half
            if (full) {
              f32x2 la = 0ull, lb = 0ull;
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float x0, x1, x2, x3;
                unpack2(ffma2(pack2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), sc2, nm2), x0, x1);
                unpack2(ffma2(pack2(__uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3])), sc2, nm2), x2, x3);
                const float p0 = fast_exp2(x0), p1 = fast_exp2(x1), p2 = fast_exp2(x2), p3 = fast_exp2(x3);
                la = fadd2(la, pack2(p0, p1));
                lb = fadd2(lb, pack2(p2, p3));
                ph[i >> 1] = pack_f16x2(p0, p1);
                ph[(i >> 1) + 1] = pack_f16x2(p2, p3);
              }
              float a0, a1, b0, b1;
              unpack2(la, a0, a1);
              unpack2(lb, b0, b1);
              ls[0] += a0; ls[1] += a1; ls[2] += b0; ls[3] += b1;
            } else {
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                float pa = fast_exp2(__uint_as_float(sr[i]) * P.scale_log2 - m_s);
                float pb = fast_exp2(__uint_as_float(sr[i + 1]) * P.scale_log2 - m_s);
                if (col0 + i < v_lo || col0 + i >= v_hi) pa = 0.f;
                if (col0 + i + 1 < v_lo || col0 + i + 1 >= v_hi) pb = 0.f;
                ls[i & 3] += pa;
                ls[(i + 1) & 3] += pb;
                ph[i >> 1] = pack_f16x2(pa, pb);
              }
            }
            tmem_st16(s_col + col0, ph);
          }
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_p + 16 * X + 8 * hf);
        }
        l_run = l_run * alpha + (ls[0] + ls[1]) + (ls[2] + ls[3]);
      }
      if (ok && !flags[8]) {
        ok = mbar_wait_bounded(bar_done, 0);
        if (ok) {
          tc_fence_after();
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
          uint4* op = reinterpret_cast<uint4*>(P.out + (int64_t)(qs + q_tok) * P.out_tok_stride +
                                               (int64_t)(hk * G + slot_h) * kD);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t orr[32];
            tmem_ld32_issue(o_col + 32 * c, orr);
            tmem_ld_fence(orr);
            if (row_ok) {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                uint4 w;
                w.x = pack_bf16x2(__uint_as_float(orr[e * 8 + 0]) * inv, __uint_as_float(orr[e * 8 + 1]) * inv);
                w.y = pack_bf16x2(__uint_as_float(orr[e * 8 + 2]) * inv, __uint_as_float(orr[e * 8 + 3]) * inv);
                w.z = pack_bf16x2(__uint_as_float(orr[e * 8 + 4]) * inv, __uint_as_float(orr[e * 8 + 5]) * inv);
                w.w = pack_bf16x2(__uint_as_float(orr[e * 8 + 6]) * inv, __uint_as_float(orr[e * 8 + 7]) * inv);
                op[c * 4 + e] = w;
              }
            }
          }
        }
      }
      if (!ok && lane == 0 && !flags[8]) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); flags[8] = 1; }
    }
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
    cudaError_t e = cudaFuncSetAttribute(swa_prefill_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) {
      set_error("sbk_swa_prefill: cannot opt in to %d bytes of shared memory: %s", kSmemBytes, cudaGetErrorString(e));
      return SBK_E_LAUNCH;
    }
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid(P.n_seqs * P.tiles_per_seq, kvh);
  swa_prefill_pair_kernel<<<grid, kThreads, kSmemBytes, stream>>>(P, map_k, map_v, map_k2, map_v2);
  return check_launch("sbk_swa_prefill");
}

}  // namespace prefill_tc2
}  // namespace sbk
