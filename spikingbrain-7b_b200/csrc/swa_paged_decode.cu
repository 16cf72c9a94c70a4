// Sliding-window paged-attention decode for sm_100a.
//
// Work decomposition
//   grid = (max_pieces, B). A CTA owns one split ("piece") of one sequence: a
//   run of 16-token chunks inside the visible window [t0, seq_len). It streams
//   those chunks for ALL kv heads, so every token it touches is one contiguous
//   kvh*D*2-byte row of K and one of V.
// Data movement
//   One producer warp walks the block table and issues one bulk async copy
//   (TMA engine, untiled form) per token row into a ring of shared-memory
//   stages; completion is counted in bytes on an mbarrier per stage. Rows are
//   laid down with a 16-byte skew so that ldmatrix reads of 8 tokens at a
//   fixed head/dim offset hit 8 different bank groups.
// Math
//   4 consumer warps; warp w serves kv head w % kvh and every (4/kvh)-th chunk.
//   Warps that take the same chunks form a group with a private ring of stages
//   and private barriers, so every waiter sees every phase of its barriers in
//   order (a parity wait cannot tell phase n from phase n+2).
//   Scores are formed TRANSPOSED, S^T[token, head] = K[token, :] . Q^T, with
//   mma.sync m16n8k16 (16 tokens x 8 query heads of the kv group), so the
//   7-of-8 head padding wastes 1/8 of the tile instead of 9/16; softmax runs
//   on the accumulator fragment with warp shuffles over the token axis;
//   P^T is turned into the B fragment with movmatrix; O^T[d, head] += V^T . P^T,
//   with P split into a bf16 head and a bf16 remainder (two MMAs) so that the
//   rounding of the probabilities stays below the bf16 rounding of the output.
//   Warps that share a kv head merge their (m, l, O) through shared memory.
// Split-K
//   A sequence with more than one piece writes un-normalised partials to the
//   workspace; swa_reduce_kernel folds them. One piece writes `out` directly.
// HBM-bound: min(seq_len, window_left+1) * kvh*D*2*2 bytes read per sequence.
#include "sbk_common.cuh"

namespace sbk {

constexpr int kChunk = 16;          // tokens per pipeline stage
constexpr int kD = 128;             // head dim
constexpr int kConsumerWarps = 4;
constexpr int kStagesPerGroup = 3;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kHeadStride = 132;    // floats per head row in the merge buffer (bank skew)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kNegBig = -1.0e30f;

struct Plan {
  int t0, c_first, n_chunks, n_pieces, chunks_per_piece;
};

// The split of a sequence into pieces; the main and the reduce kernel must agree on it.
__device__ __forceinline__ Plan make_plan(int L, int window_left, int split_chunks,
                                          int max_pieces) {
  Plan p;
  if (L <= 0) {
    p.t0 = 0; p.c_first = 0; p.n_chunks = 0; p.n_pieces = 1; p.chunks_per_piece = 0;
    return p;
  }
  p.t0 = first_visible(L, 1, window_left);
  p.c_first = p.t0 / kChunk;
  p.n_chunks = (L - 1) / kChunk - p.c_first + 1;
  int np = (p.n_chunks + split_chunks - 1) / split_chunks;
  if (np > max_pieces) np = max_pieces;
  p.chunks_per_piece = (p.n_chunks + np - 1) / np;
  p.n_pieces = (p.n_chunks + p.chunks_per_piece - 1) / p.chunks_per_piece;
  return p;
}

template <int KVH>
struct Cfg {
  static constexpr int kRowBytes = KVH * kD * 2;
  static constexpr int kRowStride = kRowBytes + 16;
  static constexpr int kStageBytes = 2 * kChunk * kRowStride;   // K rows then V rows
  static constexpr int kWarpsPerHead = kConsumerWarps / KVH;   // = number of chunk groups
  static constexpr int kStages = kWarpsPerHead * kStagesPerGroup;
  static constexpr int kMergeBytes = kConsumerWarps * (8 * kHeadStride * 4 + 64);
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kSmemBytes = (kRingBytes > kMergeBytes ? kRingBytes : kMergeBytes) +
                                    2 * kStages * 8 + 16;
  static_assert(kConsumerWarps % KVH == 0, "warps must split evenly over kv heads");
};

template <typename TO>
__device__ __forceinline__ void store_out(TO* p, float x);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float x) { *p = x; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float x) {
  *p = __float2bfloat16_rn(x);
}

template <int KVH, typename TO>
__global__ void __launch_bounds__(kThreads, 2)
swa_decode_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_seq_stride,
                  const uint8_t* __restrict__ k_cache, const uint8_t* __restrict__ v_cache,
                  const int32_t* __restrict__ block_tables, int max_blocks,
                  const int32_t* __restrict__ seq_lens, int H, int64_t num_blocks,
                  int block_size, int64_t block_stride, int window_left, float scale_log2,
                  TO* __restrict__ out, int64_t out_seq_stride, float* __restrict__ lse_out,
                  float* __restrict__ ws_o, float* __restrict__ ws_ml, int split_chunks,
                  int max_pieces, int32_t* status) {
  using C = Cfg<KVH>;
  extern __shared__ __align__(128) uint8_t smem[];
  const int b = blockIdx.y;
  const int piece = blockIdx.x;
  const int L = seq_lens[b];
  const Plan plan = make_plan(L, window_left, split_chunks, max_pieces);
  if (piece >= plan.n_pieces) return;
  const int G = H / KVH;

  int cb = plan.c_first + piece * plan.chunks_per_piece;
  int n = plan.n_chunks - piece * plan.chunks_per_piece;
  if (n > plan.chunks_per_piece) n = plan.chunks_per_piece;
  if (n < 0) n = 0;
  const int t0 = plan.t0;
  const int32_t* table = block_tables + (int64_t)b * max_blocks;

  // ---- every block id this piece will dereference must lie inside the pool ----
  {
    int bad = 0;
    if (n > 0) {
      int tb = cb * kChunk; if (tb < t0) tb = t0;
      int te = (cb + n) * kChunk; if (te > L) te = L;
      const int lb0 = tb / block_size, lb1 = (te - 1) / block_size;
      for (int lb = lb0 + threadIdx.x; lb <= lb1; lb += kThreads) {
        if (lb >= max_blocks) { bad = 1; break; }
        const int32_t pb = table[lb];
        if (pb < 0 || pb >= num_blocks) { bad = 1; break; }
      }
    }
    if (__syncthreads_or(bad)) {
      if (threadIdx.x == 0) raise_status(status, SBK_ST_BAD_BLOCK);
      n = 0;  // contribute nothing; the output stays finite
    }
  }

  const uint32_t ring = smem_u32(smem);
  const uint32_t bar_full = ring + (C::kSmemBytes - 2 * C::kStages * 8 - 16);
  const uint32_t bar_empty = bar_full + C::kStages * 8;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::kSmemBytes - 16);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, KVH);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  // V rows that a ragged first or last chunk never fills must still hold finite values,
  // since a zero probability times a NaN would poison the accumulator.
  for (int s = 0; s < C::kStages; ++s) {
    uint4* vreg = reinterpret_cast<uint4*>(smem + s * C::kStageBytes + kChunk * C::kRowStride);
    for (int i = threadIdx.x; i < kChunk * C::kRowStride / 16; i += kThreads)
      vreg[i] = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async_smem();
  __syncthreads();

  if (warp == kConsumerWarps) {
    // =============================== producer ===============================
    const int r = lane & 15;
    const int is_v = lane >> 4;
    const uint8_t* base = is_v ? v_cache : k_cache;
    for (int i = 0; i < n; ++i) {
      const int grp = i % C::kWarpsPerHead, j = i / C::kWarpsPerHead;
      const int s = grp * kStagesPerGroup + j % kStagesPerGroup;
      const int use = j / kStagesPerGroup;
      if (use > 0) {
        if (!mbar_wait_bounded(bar_empty + 8 * s, (use - 1) & 1)) {
          if (lane == 0) { raise_status(status, SBK_ST_WAIT_TIMEOUT); *abort_flag = 1; }
          break;
        }
      }
      if (*abort_flag) break;
      const int tok_base = (cb + i) * kChunk;
      int lo = tok_base > t0 ? tok_base : t0;
      int hi = tok_base + kChunk < L ? tok_base + kChunk : L;
      int nvalid = hi - lo; if (nvalid < 0) nvalid = 0;
      if (lane == 0) mbar_arrive_expect_tx(bar_full + 8 * s, 2u * nvalid * C::kRowBytes);
      __syncwarp();
      const int tok = tok_base + r;
      if (tok >= t0 && tok < L) {
        const int lb = tok / block_size;
        const int64_t pb = table[lb];
        const uint8_t* src = base + pb * block_stride + (int64_t)(tok - lb * block_size) * C::kRowBytes;
        const uint32_t dst = ring + s * C::kStageBytes + is_v * (kChunk * C::kRowStride) + r * C::kRowStride;
        bulk_g2s(dst, src, C::kRowBytes, bar_full + 8 * s);
      }
    }
    return;
  }

  // ================================ consumers ================================
  const int hk = warp % KVH;
  const int phase = warp / KVH;
  const int gq = lane >> 2;   // B-fragment column: query head inside the kv group
  const int tq = lane & 3;

  // Q^T as the B operand of S^T = K . Q^T : b0 = dims 2tq,2tq+1 of step kk, b1 = +8
  uint32_t qf[kD / 16][2];
  {
    const __nv_bfloat16* qp = q + (int64_t)b * q_seq_stride + (int64_t)(hk * G + gq) * kD + tq * 2;
#pragma unroll
    for (int kk = 0; kk < kD / 16; ++kk) {
      if (gq < G) {
        qf[kk][0] = *reinterpret_cast<const uint32_t*>(qp + kk * 16);
        qf[kk][1] = *reinterpret_cast<const uint32_t*>(qp + kk * 16 + 8);
      } else {
        qf[kk][0] = 0u; qf[kk][1] = 0u;
      }
    }
  }
  float acc[kD / 16][4];
#pragma unroll
  for (int mt = 0; mt < kD / 16; ++mt) { acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  // per-lane ldmatrix row addresses inside a stage
  const int lj = lane >> 3, lr = lane & 7;
  const uint32_t k_lane_off = (lr + ((lj & 1) ? 8 : 0)) * C::kRowStride + hk * (kD * 2) + ((lj >> 1) ? 16 : 0);
  const uint32_t v_lane_off = kChunk * C::kRowStride + (lr + ((lj >> 1) ? 8 : 0)) * C::kRowStride +
                              hk * (kD * 2) + ((lj & 1) ? 16 : 0);

  for (int i = phase, j = 0; i < n; i += C::kWarpsPerHead, ++j) {
    const int s = phase * kStagesPerGroup + j % kStagesPerGroup;
    if (!mbar_wait_bounded(bar_full + 8 * s, (j / kStagesPerGroup) & 1)) {
      if (lane == 0) { raise_status(status, SBK_ST_WAIT_TIMEOUT); *abort_flag = 1; }
      break;
    }
    const uint32_t stage = ring + s * C::kStageBytes;

    // ---- S^T[16 tokens, 8 heads] ----
    float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < kD / 16; kk += 2) {
      uint32_t a[4];
      ldmatrix_x4(a, stage + k_lane_off + kk * 32);
      mma_bf16_16816(sa, a, qf[kk][0], qf[kk][1]);
      ldmatrix_x4(a, stage + k_lane_off + (kk + 1) * 32);
      mma_bf16_16816(sb, a, qf[kk + 1][0], qf[kk + 1][1]);
    }
    float sc[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) sc[e] = (sa[e] + sb[e]) * scale_log2;

    const int tok_base = (cb + i) * kChunk;
    if (tok_base < t0 || tok_base + kChunk > L) {
      const int ta = tok_base + gq, tb2 = ta + 8;
      if (ta < t0 || ta >= L) { sc[0] = -INFINITY; sc[1] = -INFINITY; }
      if (tb2 < t0 || tb2 >= L) { sc[2] = -INFINITY; sc[3] = -INFINITY; }
    }

    // ---- online softmax over the token axis (lanes with equal tq share heads) ----
    float mx0 = fmaxf(sc[0], sc[2]), mx1 = fmaxf(sc[1], sc[3]);
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float ms0 = fmaxf(mn0, kNegBig), ms1 = fmaxf(mn1, kNegBig);
    const float al0 = fast_exp2(m0 - ms0), al1 = fast_exp2(m1 - ms1);
    m0 = mn0; m1 = mn1;
    float p[4];
    p[0] = fast_exp2(sc[0] - ms0);
    p[1] = fast_exp2(sc[1] - ms1);
    p[2] = fast_exp2(sc[2] - ms0);
    p[3] = fast_exp2(sc[3] - ms1);
    l0 = l0 * al0 + p[0] + p[2];
    l1 = l1 * al1 + p[1] + p[3];
#pragma unroll
    for (int mt = 0; mt < kD / 16; ++mt) {
      acc[mt][0] *= al0; acc[mt][1] *= al1; acc[mt][2] *= al0; acc[mt][3] *= al1;
    }
    // P^T as the B operand of O^T = V^T . P^T; p = head + remainder, both bf16
    float ph[4], pl[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      ph[e] = __bfloat162float(__float2bfloat16_rn(p[e]));
      pl[e] = p[e] - ph[e];
    }
    const uint32_t pb0 = movmatrix_trans(pack_bf16x2(ph[0], ph[1]));
    const uint32_t pb1 = movmatrix_trans(pack_bf16x2(ph[2], ph[3]));
    const uint32_t pc0 = movmatrix_trans(pack_bf16x2(pl[0], pl[1]));
    const uint32_t pc1 = movmatrix_trans(pack_bf16x2(pl[2], pl[3]));
#pragma unroll
    for (int mt = 0; mt < kD / 16; ++mt) {
      uint32_t a[4];
      ldmatrix_x4_trans(a, stage + v_lane_off + mt * 32);
      mma_bf16_16816(acc[mt], a, pb0, pb1);
      mma_bf16_16816(acc[mt], a, pc0, pc1);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_empty + 8 * s);
  }

  // l: sum over the 8 token lanes that share this thread's heads
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, off);
    l1 += __shfl_xor_sync(0xffffffffu, l1, off);
  }

  // A wait that ran out may have left copies in flight: give them time to land before the
  // ring is reused or the CTA retires (bounded; the result is already flagged invalid).
  if (*abort_flag) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  // ---- merge the warps of a kv head through shared memory (the ring is idle now) ----
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
  {
    float* wo = reinterpret_cast<float*>(smem + warp * (8 * kHeadStride * 4 + 64));
    float* wml = wo + 8 * kHeadStride;
#pragma unroll
    for (int mt = 0; mt < kD / 16; ++mt) {
      const int d = mt * 16 + gq;
      wo[(2 * tq) * kHeadStride + d] = acc[mt][0];
      wo[(2 * tq + 1) * kHeadStride + d] = acc[mt][1];
      wo[(2 * tq) * kHeadStride + d + 8] = acc[mt][2];
      wo[(2 * tq + 1) * kHeadStride + d + 8] = acc[mt][3];
    }
    if (gq == 0) {
      wml[2 * tq] = m0; wml[2 * tq + 1] = m1;
      wml[8 + 2 * tq] = l0; wml[8 + 2 * tq + 1] = l1;
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");

  const int d = threadIdx.x & (kD - 1);
  const bool direct = plan.n_pieces == 1;
  for (int h = threadIdx.x >> 7; h < H; h += (kConsumerWarps * 32) / kD) {
    const int kvhd = h / G, nq = h - kvhd * G;
    float M = -INFINITY;
#pragma unroll
    for (int ph = 0; ph < C::kWarpsPerHead; ++ph) {
      const float* wml = reinterpret_cast<const float*>(smem + (kvhd + KVH * ph) * (8 * kHeadStride * 4 + 64)) + 8 * kHeadStride;
      M = fmaxf(M, wml[nq]);
    }
    const float Ms = fmaxf(M, kNegBig);
    float Lsum = 0.f, O = 0.f;
#pragma unroll
    for (int ph = 0; ph < C::kWarpsPerHead; ++ph) {
      const float* wo = reinterpret_cast<const float*>(smem + (kvhd + KVH * ph) * (8 * kHeadStride * 4 + 64));
      const float* wml = wo + 8 * kHeadStride;
      const float w = fast_exp2(wml[nq] - Ms);
      Lsum += wml[8 + nq] * w;
      O += wo[nq * kHeadStride + d] * w;
    }
    if (direct) {
      const float inv = Lsum > 0.f ? 1.f / Lsum : 0.f;
      store_out<TO>(out + (int64_t)b * out_seq_stride + (int64_t)h * kD + d, O * inv);
      if (lse_out && d == 0)
        lse_out[(int64_t)b * H + h] = Lsum > 0.f ? (M + log2f(Lsum)) * kLn2 : -INFINITY;
    } else {
      const int64_t pi = ((int64_t)b * max_pieces + piece) * H + h;
      ws_o[pi * kD + d] = O;
      if (d == 0) { ws_ml[pi * 2] = M; ws_ml[pi * 2 + 1] = Lsum; }
    }
  }
}

// Folds the partials of sequences that were split; one CTA per sequence.
template <typename TO>
__global__ void __launch_bounds__(256)
swa_reduce_kernel(const int32_t* __restrict__ seq_lens, int H, int window_left, int split_chunks,
                  int max_pieces, const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                  TO* __restrict__ out, int64_t out_seq_stride, float* __restrict__ lse_out) {
  const int b = blockIdx.x;
  const Plan plan = make_plan(seq_lens[b], window_left, split_chunks, max_pieces);
  if (plan.n_pieces <= 1) return;
  const int d = threadIdx.x & (kD - 1);
  for (int h = threadIdx.x >> 7; h < H; h += 256 / kD) {
    float M = -INFINITY;
    for (int p = 0; p < plan.n_pieces; ++p)
      M = fmaxf(M, ws_ml[(((int64_t)b * max_pieces + p) * H + h) * 2]);
    const float Ms = fmaxf(M, kNegBig);
    float Lsum = 0.f, O = 0.f;
    for (int p = 0; p < plan.n_pieces; ++p) {
      const int64_t pi = ((int64_t)b * max_pieces + p) * H + h;
      const float w = fast_exp2(ws_ml[pi * 2] - Ms);
      Lsum += ws_ml[pi * 2 + 1] * w;
      O += ws_o[pi * kD + d] * w;
    }
    const float inv = Lsum > 0.f ? 1.f / Lsum : 0.f;
    store_out<TO>(out + (int64_t)b * out_seq_stride + (int64_t)h * kD + d, O * inv);
    if (lse_out && d == 0)
      lse_out[(int64_t)b * H + h] = Lsum > 0.f ? (M + log2f(Lsum)) * kLn2 : -INFINITY;
  }
}

template <int KVH, typename TO>
int launch_swa(const void* q, int64_t q_seq_stride, const void* k_cache, const void* v_cache,
               const int32_t* block_tables, int max_blocks, const int32_t* seq_lens, int B, int H,
               int64_t num_blocks, int block_size, int64_t block_stride, int window_left,
               float scale, void* out, int64_t out_seq_stride, float* lse_out, float* ws_o,
               float* ws_ml, int split_chunks, int max_pieces, int32_t* status, cudaStream_t st) {
  using C = Cfg<KVH>;
  auto kern = swa_decode_kernel<KVH, TO>;
  // The opt-in to large dynamic shared memory is per device; remember which devices have it.
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) {
      set_error("sbk_swa_decode: cannot opt in to %d bytes of shared memory: %s", C::kSmemBytes,
                cudaGetErrorString(e));
      return SBK_E_LAUNCH;
    }
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid(max_pieces, B);
  kern<<<grid, kThreads, C::kSmemBytes, st>>>(
      (const __nv_bfloat16*)q, q_seq_stride, (const uint8_t*)k_cache, (const uint8_t*)v_cache,
      block_tables, max_blocks, seq_lens, H, num_blocks, block_size, block_stride, window_left,
      scale * kLog2e, (TO*)out, out_seq_stride, lse_out, ws_o, ws_ml, split_chunks, max_pieces,
      status);
  int rc = check_launch("sbk_swa_decode");
  if (rc != SBK_OK || max_pieces == 1) return rc;
  swa_reduce_kernel<TO><<<B, 256, 0, st>>>(seq_lens, H, window_left, split_chunks, max_pieces, ws_o,
                                           ws_ml, (TO*)out, out_seq_stride, lse_out);
  return check_launch("sbk_swa_decode(reduce)");
}

}  // namespace sbk

extern "C" size_t sbk_swa_workspace_bytes(int B, int H, int D, int max_pieces) {
  if (B <= 0 || H <= 0 || D <= 0 || max_pieces <= 1) return 0;
  return (size_t)B * max_pieces * H * ((size_t)D + 2) * sizeof(float);
}

extern "C" int sbk_swa_decode(const void* q, int64_t q_seq_stride, const void* k_cache,
                              const void* v_cache, const int32_t* block_tables, int max_blocks,
                              const int32_t* seq_lens, int B, int H, int kvh, int D,
                              int64_t num_blocks, int block_size, int64_t cache_block_stride_bytes,
                              int window_left, float scale, void* out, int out_dtype,
                              int64_t out_seq_stride, float* lse_out, void* workspace,
                              size_t workspace_bytes, int split_chunks, int max_pieces,
                              int32_t* status, void* stream) {
  using namespace sbk;
  if (B < 0 || H <= 0 || kvh <= 0 || H % kvh != 0 || max_blocks <= 0 || num_blocks < 0) {
    set_error("sbk_swa_decode: bad sizes B=%d H=%d kvh=%d max_blocks=%d", B, H, kvh, max_blocks);
    return SBK_E_ARG;
  }
  if (D != kD || H / kvh > 8 || !(kvh == 1 || kvh == 2 || kvh == 4)) {
    set_error("sbk_swa_decode: unsupported shape D=%d H/kvh=%d kvh=%d (need D=128, group<=8, kvh in 1,2,4)",
              D, H / kvh, kvh);
    return SBK_E_ARG;
  }
  if (block_size <= 0 || block_size % 16 != 0) {
    set_error("sbk_swa_decode: block_size=%d must be a positive multiple of 16", block_size);
    return SBK_E_ARG;
  }
  if (out_dtype != SBK_BF16 && out_dtype != SBK_F32) {
    set_error("sbk_swa_decode: out_dtype=%d unsupported", out_dtype);
    return SBK_E_ARG;
  }
  if (max_pieces < 1 || max_pieces > 65535 || B > 65535) {
    set_error("sbk_swa_decode: max_pieces=%d / B=%d outside [1,65535]", max_pieces, B);
    return SBK_E_ARG;
  }
  if (B == 0) return SBK_OK;
  if (!q || !k_cache || !v_cache || !block_tables || !seq_lens || !out) {
    set_error("sbk_swa_decode: null pointer");
    return SBK_E_ARG;
  }
  const int64_t row_bytes = (int64_t)kvh * D * 2;
  if (!aligned16(k_cache) || !aligned16(v_cache) || cache_block_stride_bytes % 16 ||
      (reinterpret_cast<uintptr_t>(q) & 3u) || (q_seq_stride & 1)) {
    set_error("sbk_swa_decode: cache base/stride must be 16-byte multiples and q 4-byte aligned");
    return SBK_E_ALIGN;
  }
  if (cache_block_stride_bytes < row_bytes * block_size) {
    set_error("sbk_swa_decode: cache block stride smaller than a block");
    return SBK_E_ARG;
  }
  if (split_chunks <= 0) split_chunks = 32;
  float* ws_o = nullptr;
  float* ws_ml = nullptr;
  if (max_pieces > 1) {
    const size_t need = sbk_swa_workspace_bytes(B, H, D, max_pieces);
    if (!workspace || workspace_bytes < need) {
      set_error("sbk_swa_decode: workspace of %zu bytes given, %zu needed", workspace_bytes, need);
      return SBK_E_WORKSPACE;
    }
    if (!aligned16(workspace)) {
      set_error("sbk_swa_decode: workspace must be 16-byte aligned");
      return SBK_E_ALIGN;
    }
    ws_o = (float*)workspace;
    ws_ml = ws_o + (size_t)B * max_pieces * H * D;
  }
  cudaStream_t st = (cudaStream_t)stream;
#define SBK_SWA_CALL(KVH, TO)                                                                     \
  return launch_swa<KVH, TO>(q, q_seq_stride, k_cache, v_cache, block_tables, max_blocks, seq_lens, \
                             B, H, num_blocks, block_size, cache_block_stride_bytes, window_left,  \
                             scale, out, out_seq_stride, lse_out, ws_o, ws_ml, split_chunks,       \
                             max_pieces, status, st)
#define SBK_SWA_KVH(TO)                 \
  switch (kvh) {                        \
    case 1: SBK_SWA_CALL(1, TO);        \
    case 2: SBK_SWA_CALL(2, TO);        \
    default: SBK_SWA_CALL(4, TO);       \
  }
  if (out_dtype == SBK_BF16) { SBK_SWA_KVH(__nv_bfloat16) } else { SBK_SWA_KVH(float) }
#undef SBK_SWA_KVH
#undef SBK_SWA_CALL
}
