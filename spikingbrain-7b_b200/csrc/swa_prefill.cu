// Sliding-window attention for runs of query tokens (prefill / chunked prefill) over the paged
// K/V cache, sm_100a.
//
// A CTA owns 16 consecutive query tokens of one sequence and one kv head: the G query heads of
// that kv group give G consumer warps, each holding a 16-query x 128-dim tile of ONE head, and
// all of them read the same K/V tiles -- a 16-key tile of one kv head is fetched once per CTA
// (TMA tensor copy through the block table, 128-byte swizzle, ring of 3 stages of 64 keys) and
// used by 16 x G queries. One extra warp is the producer. The query at position p sees keys
// [p - window_left, p]; only the chunks at the two ends of that range need a mask.
// Math per warp and 16 keys: S = Q K^T (16 mma.sync m16n8k16), online softmax on the accumulator
// rows, O += P V with P as bf16 head + bf16 remainder (32 mma.sync), fp32 accumulation.
// The new tokens' K/V must already be in the cache (the append runs first).
#include "sbk_common.cuh"

#include "sbk_tma.cuh"
#include "swa_prefill_tc.cuh"

namespace sbk {
namespace prefill {

constexpr int kD = 128;
constexpr int kChunk = 16;          // keys per tile
constexpr int kBQ = 16;             // queries per CTA
constexpr int kStageChunks = 4;     // 64 keys per stage
constexpr int kTileBytes = kChunk * 2 * 128;              // one kv head: [half][key][128 B] = 4 KiB
constexpr int kVOffset = kStageChunks * kTileBytes;       // 16 KiB of K, then 16 KiB of V
constexpr int kStageBytes = 2 * kVOffset;
constexpr int kStages = 3;
constexpr int kRingBytes = kStages * kStageBytes;
constexpr int kBarOff = kRingBytes;
constexpr int kFlagOff = kBarOff + 2 * kStages * 8;
constexpr int kSmemBytes = kFlagOff + 32 + 1024;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegBig = -1.0e30f;

struct Params {
  const __nv_bfloat16* q; int64_t q_tok_stride;
  const int32_t* block_tables; int max_blocks;
  const int32_t* query_start_loc; const int32_t* context_lens;
  int n_seqs; int tiles_per_seq; int H; int G; int64_t num_blocks; int block_size;
  int window_left; float scale_log2;
  __nv_bfloat16* out; int64_t out_tok_stride;
  int32_t* status; int tile_copy;
  int n_meta_chunks;   // 16-token chunks of always-visible sink keys, streamed ahead of the window
};

__global__ void __launch_bounds__(288, 1)
swa_prefill_kernel(const Params P, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_k2,
                   const __grid_constant__ CUtensorMap map_v2) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* const smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t ring = smem_u32(smem);
  const uint32_t bar_full = ring + kBarOff, bar_empty = bar_full + kStages * 8;
  volatile int* flags = reinterpret_cast<volatile int*>(smem + kFlagOff);   // [0..2] stage bad, [3] abort

  const int s = blockIdx.x / P.tiles_per_seq;
  // later query tiles see more keys: they are launched first, so the long items do not start last
  const int j = P.tiles_per_seq - 1 - (int)(blockIdx.x - s * P.tiles_per_seq);
  const int hk = blockIdx.y;
  const int qs = P.query_start_loc[s];
  const int n_q = P.query_start_loc[s + 1] - qs;
  if (j * kBQ >= n_q) return;
  const int nq_tile = n_q - j * kBQ < kBQ ? n_q - j * kBQ : kBQ;
  const int p0 = P.context_lens[s] + j * kBQ;                 // position of the tile's first query
  const int key_lo = P.window_left < 0 ? 0 : (p0 - P.window_left > 0 ? p0 - P.window_left : 0);
  const int key_hi = p0 + nq_tile;                            // exclusive
  const int c_lo = key_lo / kChunk, c_hi = (key_hi - 1) / kChunk;
  const int n_chunks = c_hi - c_lo + 1;
  const int n_ms = (P.n_meta_chunks + kStageChunks - 1) / kStageChunks;    // sink-token stages come first
  const int n_stages = n_ms + (n_chunks + kStageChunks - 1) / kStageChunks;
  const int G = P.G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, G);
    }
    flags[3] = 0;
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == G) {
    // ================================= producer =================================
    const int32_t* table = P.block_tables + (int64_t)s * P.max_blocks;
    int64_t pb_lane = -1;
    int batch_c0 = 0;
    for (int st = 0; st < n_stages; ++st) {
      const bool meta = st < n_ms;
      const int c0 = meta ? st * kStageChunks : c_lo + (st - n_ms) * kStageChunks;
      const int c_end = meta ? P.n_meta_chunks - 1 : c_hi;     // last chunk of this kind
      if (!meta && (st == n_ms || c0 + kStageChunks > batch_c0 + 32)) {      // one table read per 32 chunks
        batch_c0 = c0;
        const int c = c0 + lane;
        const int lb = (c * kChunk) / P.block_size;
        pb_lane = (c <= c_hi && lb < P.max_blocks) ? (int64_t)table[lb] : -1;
      }
      const int slot = st % kStages, use = st / kStages;
      if (use > 0 && !mbar_wait_bounded(bar_empty + 8 * slot, (use - 1) & 1)) {
        if (lane == 0) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); flags[3] = 1; }
        break;
      }
      if (flags[3]) break;
      // lane -> one copy: chunk of the stage, K or V, and (row-wise mode) which 128-byte half
      const int n_copies = P.tile_copy ? 2 * kStageChunks : 4 * kStageChunks;
      const int i = P.tile_copy ? lane >> 1 : lane >> 2;
      const int is_v = P.tile_copy ? lane & 1 : (lane >> 1) & 1;
      const int half = P.tile_copy ? 0 : lane & 1;
      const int c = c0 + (lane < n_copies ? i : 0);
      const bool active = lane < n_copies && c <= c_end;
      int src_lane = c - batch_c0;
      src_lane = src_lane < 0 ? 0 : (src_lane > 31 ? 31 : src_lane);
      const int64_t pb_tab = __shfl_sync(0xffffffffu, pb_lane, src_lane);
      const int64_t pb = meta ? (int64_t)c : pb_tab;           // the sink tensors are their own block table
      bool bad = !meta && active && (pb < 0 || pb >= P.num_blocks);
      bad = __any_sync(0xffffffffu, bad);
      const int nvalid = c_end - c0 + 1 < kStageChunks ? c_end - c0 + 1 : kStageChunks;
      if (lane == 0) {
        flags[slot] = bad ? 1 : 0;
        if (bad) raise_status(P.status, SBK_ST_BAD_BLOCK);
        mbar_arrive_expect_tx(bar_full + 8 * slot, bad ? 0u : (uint32_t)nvalid * 2u * kTileBytes);
      }
      __syncwarp();
      if (!bad && active) {
        const uint32_t dst = ring + slot * kStageBytes + is_v * kVOffset + i * kTileBytes + half * 2048;
        const int tin = meta ? 0 : (c * kChunk) % P.block_size;
        const CUtensorMap* map = meta ? (is_v ? &map_v2 : &map_k2) : (is_v ? &map_v : &map_k);
        if (P.tile_copy) tma_load_4d(dst, map, 0, tin, hk * 2, (int)pb, bar_full + 8 * slot);
        else tma_load_4d(dst, map, 0, hk * 2 + half, tin, (int)pb, bar_full + 8 * slot);
      }
    }
    return;
  }
  if (warp > G) return;

  // ================================== consumers ==================================
  const int h = hk * G + warp;              // this warp's query head
  const int gq = lane >> 2, tq = lane & 3;  // fragment row (query / key) and column pair
  const int qpos_lo = p0 + gq, qpos_hi = p0 + gq + 8;
  const bool row_lo_ok = gq < nq_tile, row_hi_ok = gq + 8 < nq_tile;

  // Q as the A operand: a0 (row gq, dims 2tq..), a1 (row gq+8), a2 (row gq, dims +8), a3 (row gq+8, dims +8)
  uint32_t qa[kD / 16][4];
  {
    const __nv_bfloat16* q_lo = P.q + (int64_t)(qs + j * kBQ + gq) * P.q_tok_stride + (int64_t)h * kD + tq * 2;
    const __nv_bfloat16* q_hi = q_lo + 8 * P.q_tok_stride;
#pragma unroll
    for (int kk = 0; kk < kD / 16; ++kk) {
      qa[kk][0] = row_lo_ok ? *reinterpret_cast<const uint32_t*>(q_lo + kk * 16) : 0u;
      qa[kk][1] = row_hi_ok ? *reinterpret_cast<const uint32_t*>(q_hi + kk * 16) : 0u;
      qa[kk][2] = row_lo_ok ? *reinterpret_cast<const uint32_t*>(q_lo + kk * 16 + 8) : 0u;
      qa[kk][3] = row_hi_ok ? *reinterpret_cast<const uint32_t*>(q_hi + kk * 16 + 8) : 0u;
    }
  }
  float acc[kD / 8][4];
#pragma unroll
  for (int n = 0; n < kD / 8; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  // ldmatrix lane addressing inside a 16-key tile [half][key][128 B], chunk index XOR (key & 7)
  const int mi = lane >> 3, lr = lane & 7;
  const int key_k = lr + ((mi >> 1) ? 8 : 0), cj_k = mi & 1;     // K: matrices (keys, dim chunk)
  const int key_v = lr + ((mi & 1) ? 8 : 0), cj_v = mi >> 1;     // V (transposed load)
  const uint32_t k_off = key_k * 128, v_off = key_v * 128;
  const int xk = key_k & 7, xv = key_v & 7;

  for (int st = 0; st < n_stages; ++st) {
    const int slot = st % kStages;
    if (!mbar_wait_bounded(bar_full + 8 * slot, (st / kStages) & 1)) {
      if (lane == 0) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); flags[3] = 1; }
      break;
    }
    const bool bad = flags[slot] != 0;
    const bool meta = st < n_ms;
    const int c0 = meta ? st * kStageChunks : c_lo + (st - n_ms) * kStageChunks;
    const int c_end = meta ? P.n_meta_chunks - 1 : c_hi;
    const int nch = c_end - c0 + 1 < kStageChunks ? c_end - c0 + 1 : kStageChunks;
    bool wrote = false;
    for (int i = 0; i < nch && !bad; ++i) {
      const int kbase = (c0 + i) * kChunk;                    // position of the tile's first key
      const uint32_t ktile = ring + slot * kStageBytes + i * kTileBytes;
      const uint32_t vtile = ktile + kVOffset;
      if (!meta && kbase + kChunk > key_hi) {
        // keys past the last query of the tile may be memory no token has reached: their V must
        // be finite before it meets a zero probability (every warp writes the same zeros)
        for (int r = lane >> 4; r < kChunk; r += 2) {
          if (kbase + r >= key_hi)
            *reinterpret_cast<uint4*>(smem + slot * kStageBytes + kVOffset + i * kTileBytes +
                                      (((lane >> 3) & 1) * 16 + r) * 128 + (lane & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
        wrote = true;
      }
      // ---- S[16 queries, 16 keys] ----
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < kD / 16; ++kk) {
        uint32_t b[4];
        ldmatrix_x4(b, ktile + (kk >> 2) * 2048 + k_off + (((((kk & 3) << 1) + cj_k) ^ xk) << 4));
        mma_bf16_16816(s0, qa[kk], b[0], b[1]);
        mma_bf16_16816(s1, qa[kk], b[2], b[3]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) { s0[e] *= P.scale_log2; s1[e] *= P.scale_log2; }
      const bool interior = meta || (kbase + kChunk - 1 <= p0 &&
                            (P.window_left < 0 || kbase >= p0 + nq_tile - 1 - P.window_left) && nq_tile == kBQ);
      if (!interior) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int qp = (e & 2) ? qpos_hi : qpos_lo;
          const bool rok = (e & 2) ? row_hi_ok : row_lo_ok;
          const int kp0 = kbase + 2 * tq + (e & 1), kp1 = kp0 + 8;
          const bool v0 = rok && kp0 <= qp && (P.window_left < 0 || kp0 >= qp - P.window_left);
          const bool v1 = rok && kp1 <= qp && (P.window_left < 0 || kp1 >= qp - P.window_left);
          if (!v0) s0[e] = -INFINITY;
          if (!v1) s1[e] = -INFINITY;
        }
      }
      // ---- online softmax per query row (a row lives in the four lanes of equal gq) ----
      float mx_lo = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
      float mx_hi = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
#pragma unroll
      for (int off = 1; off < 4; off <<= 1) {
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, off));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, off));
      }
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float ms_lo = fmaxf(mn_lo, kNegBig), ms_hi = fmaxf(mn_hi, kNegBig);
      const float al_lo = fast_exp2(m_lo - ms_lo), al_hi = fast_exp2(m_hi - ms_hi);
      m_lo = mn_lo; m_hi = mn_hi;
      float p0v[4], p1v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float ms = (e & 2) ? ms_hi : ms_lo;
        p0v[e] = fast_exp2(s0[e] - ms);
        p1v[e] = fast_exp2(s1[e] - ms);
      }
      l_lo = l_lo * al_lo + p0v[0] + p0v[1] + p1v[0] + p1v[1];
      l_hi = l_hi * al_hi + p0v[2] + p0v[3] + p1v[2] + p1v[3];
#pragma unroll
      for (int n = 0; n < kD / 8; ++n) {
        acc[n][0] *= al_lo; acc[n][1] *= al_lo; acc[n][2] *= al_hi; acc[n][3] *= al_hi;
      }
      // P as the A operand (16 queries x 16 keys), bf16 head + bf16 remainder
      uint32_t ph[4], pl[4];
      {
        float hi_[8], lo_[8];
        const float src[8] = {p0v[0], p0v[1], p0v[2], p0v[3], p1v[0], p1v[1], p1v[2], p1v[3]};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          hi_[e] = __bfloat162float(__float2bfloat16_rn(src[e]));
          lo_[e] = src[e] - hi_[e];
        }
        ph[0] = pack_bf16x2(hi_[0], hi_[1]); ph[1] = pack_bf16x2(hi_[2], hi_[3]);
        ph[2] = pack_bf16x2(hi_[4], hi_[5]); ph[3] = pack_bf16x2(hi_[6], hi_[7]);
        pl[0] = pack_bf16x2(lo_[0], lo_[1]); pl[1] = pack_bf16x2(lo_[2], lo_[3]);
        pl[2] = pack_bf16x2(lo_[4], lo_[5]); pl[3] = pack_bf16x2(lo_[6], lo_[7]);
      }
      // ---- O[16 queries, 128 dims] += P V ----
#pragma unroll
      for (int nd = 0; nd < kD / 16; ++nd) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vtile + (nd >> 2) * 2048 + v_off + (((((nd & 3) << 1) + cj_v) ^ xv) << 4));
        mma_bf16_16816(acc[2 * nd], ph, b[0], b[1]);
        mma_bf16_16816(acc[2 * nd], pl, b[0], b[1]);
        mma_bf16_16816(acc[2 * nd + 1], ph, b[2], b[3]);
        mma_bf16_16816(acc[2 * nd + 1], pl, b[2], b[3]);
      }
    }
    if (wrote) fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
  }

#pragma unroll
  for (int off = 1; off < 4; off <<= 1) {
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, off);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, off);
  }
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
  __nv_bfloat16* o_lo = P.out + (int64_t)(qs + j * kBQ + gq) * P.out_tok_stride + (int64_t)h * kD + tq * 2;
  __nv_bfloat16* o_hi = o_lo + 8 * P.out_tok_stride;
#pragma unroll
  for (int n = 0; n < kD / 8; ++n) {
    if (row_lo_ok) *reinterpret_cast<uint32_t*>(o_lo + n * 8) = pack_bf16x2(acc[n][0] * inv_lo, acc[n][1] * inv_lo);
    if (row_hi_ok) *reinterpret_cast<uint32_t*>(o_hi + n * 8) = pack_bf16x2(acc[n][2] * inv_hi, acc[n][3] * inv_hi);
  }
  if (flags[3]) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
}

}  // namespace prefill
}  // namespace sbk

extern "C" int sbk_swa_prefill(const void* q, int64_t q_tok_stride, const void* k_cache, const void* v_cache,
                               const int32_t* block_tables, int max_blocks, const int32_t* query_start_loc,
                               const int32_t* context_lens, int n_seqs, int max_query_len, int H, int kvh,
                               int D, int64_t num_blocks, int block_size, int64_t cache_block_stride_bytes,
                               int window_left, float scale, void* out, int64_t out_tok_stride,
                               const void* key2, const void* value2, int num_meta, int kernel,
                               int32_t* status, void* stream) {
  using namespace sbk;
  using namespace sbk::prefill;
  if (kernel != SBK_PREFILL_AUTO && kernel != SBK_PREFILL_TCGEN05 && kernel != SBK_PREFILL_MMA_SYNC &&
      kernel != SBK_PREFILL_TCGEN05_PAIR) {
    set_error("sbk_swa_prefill: kernel=%d is none of SBK_PREFILL_AUTO / _TCGEN05 / _MMA_SYNC / _TCGEN05_PAIR", kernel);
    return SBK_E_ARG;
  }
  if (num_meta < 0 || num_meta % 16 != 0 || (num_meta > 0 && (!key2 || !value2 || !aligned16(key2) || !aligned16(value2)))) {
    set_error("sbk_swa_prefill: sink tokens need 16-byte aligned key2/value2 and a count that is a multiple of 16 (got %d)",
              num_meta);
    return SBK_E_ARG;
  }
  if (n_seqs < 0 || max_query_len < 0 || H <= 0 || kvh <= 0 || H % kvh != 0 || max_blocks <= 0 || num_blocks < 0) {
    set_error("sbk_swa_prefill: bad sizes n_seqs=%d H=%d kvh=%d max_blocks=%d", n_seqs, H, kvh, max_blocks);
    return SBK_E_ARG;
  }
  if (D != kD || H / kvh > 8) {
    set_error("sbk_swa_prefill: unsupported shape D=%d H/kvh=%d (need D=128, at most 8 query heads per kv head)",
              D, H / kvh);
    return SBK_E_ARG;
  }
  if (block_size <= 0 || block_size % 16 != 0) {
    set_error("sbk_swa_prefill: block_size=%d must be a positive multiple of 16", block_size);
    return SBK_E_ARG;
  }
  if (n_seqs == 0 || max_query_len == 0) return SBK_OK;
  if (!q || !k_cache || !v_cache || !block_tables || !query_start_loc || !context_lens || !out) {
    set_error("sbk_swa_prefill: null pointer");
    return SBK_E_ARG;
  }
  if (!aligned16(k_cache) || !aligned16(v_cache) || cache_block_stride_bytes % 16 ||
      (reinterpret_cast<uintptr_t>(q) & 3u) || (reinterpret_cast<uintptr_t>(out) & 3u) || (q_tok_stride & 1) ||
      (out_tok_stride & 1)) {
    set_error("sbk_swa_prefill: cache base/stride must be 16-byte multiples, q/out 4-byte aligned with even strides");
    return SBK_E_ALIGN;
  }
  const int tiles = (max_query_len + kBQ - 1) / kBQ;
  if ((int64_t)n_seqs * tiles > 2147483647LL || kvh > 65535) {
    set_error("sbk_swa_prefill: grid too large");
    return SBK_E_ARG;
  }
  const int bq_tc = prefill_tc::queries_per_tile(H / kvh);
  // Three kernels serve this entry point: tcgen05 with two query tiles per CTA taking turns (what
  // `kernel` AUTO picks when a run has more queries than one tile), tcgen05 with one tile per CTA
  // (AUTO for shorter runs), and mma.sync (on request, or under AUTO when q / out cannot be moved
  // as 16-byte vectors).
  const bool vec_ok = aligned16(q) && aligned16(out) && q_tok_stride % 8 == 0 && out_tok_stride % 8 == 0;
  if ((kernel == SBK_PREFILL_TCGEN05 || kernel == SBK_PREFILL_TCGEN05_PAIR) && !vec_ok) {
    set_error("sbk_swa_prefill: the tcgen05 kernel needs q and out 16-byte aligned with token strides that are "
              "multiples of 8 elements");
    return SBK_E_ALIGN;
  }
  const bool use_tc = vec_ok && kernel != SBK_PREFILL_MMA_SYNC;
  const int64_t mstride = (int64_t)16 * kvh * D * 2;   // the sink tensors as blocks of 16 tokens
  if (use_tc) {
    const MapKey keys[4] = {MapKey{k_cache, kvh, num_blocks, block_size, cache_block_stride_bytes, 1},
                            MapKey{v_cache, kvh, num_blocks, block_size, cache_block_stride_bytes, 1},
                            MapKey{key2, kvh, num_meta / 16, 16, mstride, 1},
                            MapKey{value2, kvh, num_meta / 16, 16, mstride, 1}};
    CUtensorMap maps[4];
    int tc_mode = 0;
    if (!get_maps(maps, keys, num_meta > 0 ? 4 : 2, &tc_mode)) {
      set_error("sbk_swa_prefill: cuTensorMapEncodeTiled rejected the cache geometry or the sink-token tensors");
      return SBK_E_ARG;
    }
    const CUtensorMap &mk = maps[0], &mv = maps[1];
    const CUtensorMap &mk2 = num_meta > 0 ? maps[2] : maps[0], &mv2 = num_meta > 0 ? maps[3] : maps[1];
    prefill_tc::Params T;
    T.q = (const __nv_bfloat16*)q; T.q_tok_stride = q_tok_stride;
    T.block_tables = block_tables; T.max_blocks = max_blocks;
    T.query_start_loc = query_start_loc; T.context_lens = context_lens;
    const bool pair = kernel == SBK_PREFILL_TCGEN05_PAIR || (kernel == SBK_PREFILL_AUTO && max_query_len > bq_tc);
    const int per_cta = pair ? 2 * bq_tc : bq_tc;
    T.n_seqs = n_seqs; T.bq = bq_tc; T.tiles_per_seq = (max_query_len + per_cta - 1) / per_cta; T.H = H; T.G = H / kvh;
    T.num_blocks = num_blocks;
    T.block_size = block_size; T.window_left = window_left; T.scale_log2 = scale * kLog2e;
    T.out = (__nv_bfloat16*)out; T.out_tok_stride = out_tok_stride; T.status = status;
    T.n_meta_chunks = num_meta / 16;
    T.k_start_loc = nullptr;
    T.noncausal = 0;
    T.tile_copy = tc_mode;
    if (pair) return prefill_tc2::launch(T, kvh, mk, mv, mk2, mv2, (cudaStream_t)stream);
    return prefill_tc::launch(T, kvh, mk, mv, mk2, mv2, (cudaStream_t)stream);
  }
  const MapKey keys[4] = {MapKey{k_cache, kvh, num_blocks, block_size, cache_block_stride_bytes, 2},
                          MapKey{v_cache, kvh, num_blocks, block_size, cache_block_stride_bytes, 2},
                          MapKey{key2, kvh, num_meta / 16, 16, mstride, 2},
                          MapKey{value2, kvh, num_meta / 16, 16, mstride, 2}};
  CUtensorMap maps[4];
  int tile_copy = 0;
  if (!get_maps(maps, keys, num_meta > 0 ? 4 : 2, &tile_copy)) {
    set_error("sbk_swa_prefill: cuTensorMapEncodeTiled rejected the cache geometry or the sink-token tensors");
    return SBK_E_ARG;
  }
  const CUtensorMap &map_k = maps[0], &map_v = maps[1];
  const CUtensorMap &map_k2 = num_meta > 0 ? maps[2] : maps[0], &map_v2 = num_meta > 0 ? maps[3] : maps[1];
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(swa_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) {
      set_error("sbk_swa_prefill: cannot opt in to %d bytes of shared memory: %s", kSmemBytes, cudaGetErrorString(e));
      return SBK_E_LAUNCH;
    }
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  Params P;
  P.q = (const __nv_bfloat16*)q; P.q_tok_stride = q_tok_stride;
  P.block_tables = block_tables; P.max_blocks = max_blocks;
  P.query_start_loc = query_start_loc; P.context_lens = context_lens;
  P.n_seqs = n_seqs; P.tiles_per_seq = tiles; P.H = H; P.G = H / kvh; P.num_blocks = num_blocks;
  P.block_size = block_size; P.window_left = window_left; P.scale_log2 = scale * kLog2e;
  P.out = (__nv_bfloat16*)out; P.out_tok_stride = out_tok_stride; P.status = status;
  P.n_meta_chunks = num_meta / 16;
  P.tile_copy = tile_copy;
  dim3 grid(n_seqs * tiles, kvh);
  swa_prefill_kernel<<<grid, (P.G + 1) * 32, kSmemBytes, (cudaStream_t)stream>>>(P, map_k, map_v, map_k2, map_v2);
  return check_launch("sbk_swa_prefill");
}

extern "C" int sbk_swa_prefill_dense(const void* q, int64_t q_tok_stride, const void* key, const void* value,
                                     int64_t kv_tok_stride, int64_t n_kv_tokens, const int32_t* query_start_loc,
                                     const int32_t* k_start_loc, int n_seqs, int max_query_len, int H, int kvh,
                                     int D, int window_left, int causal, float scale, void* out,
                                     int64_t out_tok_stride, const void* key2, const void* value2, int num_meta,
                                     int32_t* status, void* stream) {
  using namespace sbk;
  using namespace sbk::prefill;
  if (num_meta < 0 || num_meta % 16 != 0 || (num_meta > 0 && (!key2 || !value2 || !aligned16(key2) || !aligned16(value2)))) {
    set_error("sbk_swa_prefill_dense: sink tokens need 16-byte aligned key2/value2 and a count that is a multiple of 16 (got %d)",
              num_meta);
    return SBK_E_ARG;
  }
  if (n_seqs < 0 || max_query_len < 0 || n_kv_tokens < 0 || H <= 0 || kvh <= 0 || H % kvh != 0) {
    set_error("sbk_swa_prefill_dense: bad sizes n_seqs=%d H=%d kvh=%d", n_seqs, H, kvh);
    return SBK_E_ARG;
  }
  if (D != kD || H / kvh > 8) {
    set_error("sbk_swa_prefill_dense: unsupported shape D=%d H/kvh=%d (need D=128, at most 8 query heads per kv head)",
              D, H / kvh);
    return SBK_E_ARG;
  }
  if (n_seqs == 0 || max_query_len == 0) return SBK_OK;
  if (!q || !key || !value || !query_start_loc || !k_start_loc || !out || n_kv_tokens == 0) {
    set_error("sbk_swa_prefill_dense: null pointer or no key tokens");
    return SBK_E_ARG;
  }
  if (!aligned16(q) || !aligned16(out) || q_tok_stride % 8 || out_tok_stride % 8 || !aligned16(key) ||
      !aligned16(value) || kv_tok_stride % 8 || kv_tok_stride < (int64_t)kvh * D) {
    set_error("sbk_swa_prefill_dense: q, out, key, value must be 16-byte aligned with token strides that are "
              "multiples of 8 elements (key/value at least kvh*D)");
    return SBK_E_ALIGN;
  }
  const int bq_tc = prefill_tc::queries_per_tile(H / kvh);
  const int tiles = (max_query_len + bq_tc - 1) / bq_tc;
  if ((int64_t)n_seqs * tiles > 2147483647LL || kvh > 65535) {
    set_error("sbk_swa_prefill_dense: grid too large");
    return SBK_E_ARG;
  }
  // the tensors as one block of n_kv_tokens tokens with their own token stride
  const int64_t bstride = n_kv_tokens * kv_tok_stride * 2;
  const int64_t mstride = (int64_t)16 * kvh * D * 2;
  const int kv_tokens32 = n_kv_tokens > 2147483647LL ? 0 : (int)n_kv_tokens;
  const MapKey keys[4] = {MapKey{key, kvh, 1, kv_tokens32, bstride, 1, kv_tok_stride * 2},
                          MapKey{value, kvh, 1, kv_tokens32, bstride, 1, kv_tok_stride * 2},
                          MapKey{key2, kvh, num_meta / 16, 16, mstride, 1},
                          MapKey{value2, kvh, num_meta / 16, 16, mstride, 1}};
  CUtensorMap maps[4];
  int tc_mode = 0;
  if (kv_tokens32 == 0 || !get_maps(maps, keys, num_meta > 0 ? 4 : 2, &tc_mode)) {
    set_error("sbk_swa_prefill_dense: cuTensorMapEncodeTiled rejected the key/value geometry or the sink-token tensors");
    return SBK_E_ARG;
  }
  const CUtensorMap &mk = maps[0], &mv = maps[1];
  const CUtensorMap &mk2 = num_meta > 0 ? maps[2] : maps[0], &mv2 = num_meta > 0 ? maps[3] : maps[1];
  prefill_tc::Params T;
  T.q = (const __nv_bfloat16*)q; T.q_tok_stride = q_tok_stride;
  T.block_tables = nullptr; T.max_blocks = 0;
  T.query_start_loc = query_start_loc; T.context_lens = nullptr; T.k_start_loc = k_start_loc;
  T.noncausal = causal ? 0 : 1;
  const bool pair = max_query_len > bq_tc;     // as under SBK_PREFILL_AUTO in the paged entry point
  T.n_seqs = n_seqs; T.bq = bq_tc; T.tiles_per_seq = pair ? (tiles + 1) / 2 : tiles; T.H = H; T.G = H / kvh; T.num_blocks = 1;
  T.block_size = 16; T.window_left = window_left; T.scale_log2 = scale * kLog2e;
  T.out = (__nv_bfloat16*)out; T.out_tok_stride = out_tok_stride; T.status = status;
  T.n_meta_chunks = num_meta / 16;
  T.tile_copy = tc_mode;
  if (pair) return prefill_tc2::launch(T, kvh, mk, mv, mk2, mv2, (cudaStream_t)stream);
  return prefill_tc::launch(T, kvh, mk, mv, mk2, mv2, (cudaStream_t)stream);
}
