// Sliding-window paged-attention decode for sm_100a: a persistent, warp-specialised,
// HBM-streaming kernel.
//
// Work decomposition
//   A work item is one split ("piece") of one sequence: a run of 16-token chunks of the
//   visible window [t0, seq_len). The grid is two CTAs per SM; each CTA draws items from a
//   global ticket counter until none is left, so ragged batches balance themselves and the
//   copy pipeline never drains between items.
//   Balanced mode (split_chunks < 0) drops the tickets: the chunks of all sequences, laid end to
//   end, are cut into one equal run per CTA (a run may cross sequence boundaries; each
//   sequence it touches is one item), so every CTA streams the same number of bytes whatever
//   the batch size or the spread of lengths, in a single wave.
// Data movement
//   One producer warp per CTA walks the block table and issues TMA tensor copies
//   (cp.async.bulk.tensor, no multicast) of 16-token tiles -- all kv heads of a token are one
//   contiguous kvh*256-byte row of K and one of V -- into a ring of 32 KiB shared-memory
//   stages; completion is counted in bytes on an mbarrier per stage. The tensor map views a
//   cache as [block][128-byte row of a token][token in block][64 elements] and lands a tile as
//   [128-byte row][token][128 B] with the 128-byte swizzle, so ldmatrix reads of 8 tokens at one
//   head/dim offset hit 8 different bank groups. Where the driver accepts the permuted strides
//   a whole tile is ONE copy of kvh*4 KiB; otherwise one copy per 128-byte row (2 KiB each).
//   A stage also carries a small descriptor (sequence, piece, token range, first/last flags),
//   so the consumers learn about items from the stream itself.
// Math
//   4 consumer warps. A stage holds 64/kvh tokens; warp w serves kv head w % kvh and the
//   16-token sub-chunk w / kvh of every stage. Scores are formed TRANSPOSED,
//   S^T[token, head] = K[token, :] . Q^T, with mma.sync m16n8k16 (16 tokens x the 8 query
//   heads of a kv group), so padding 7 heads to 8 wastes 1/8 of the tile; softmax runs on
//   the accumulator fragment with warp shuffles over the token axis; P^T becomes the B
//   fragment through movmatrix; O^T[d, head] += V^T . P^T with P split into a bf16 head and
//   a bf16 remainder (two MMAs), which keeps the rounding of the probabilities below the
//   bf16 rounding of the output.
// Split-K
//   A sequence with several pieces writes un-normalised partials (m, l, O) to the workspace and
//   counts them (a counter per sequence); there is no second kernel. Few pieces: the CTA that
//   counts last folds them (out of its idle ring when the piece was its last item, else through
//   registers). Many pieces (at most four heads per piece): head by head, and in balanced mode
//   shared out over the CTAs that hold the pieces, which wait for one another -- balanced-mode
//   launches are cooperative launches. A single piece writes `out` directly.
// HBM-bound: min(seq_len, window_left+1) * kvh*128*2*2 bytes read per sequence.
#include "sbk_common.cuh"
#include "sbk_tma.cuh"

namespace sbk {

constexpr int kChunk = 16;            // tokens per MMA tile
constexpr int kD = 128;               // head dim
constexpr int kConsumerWarps = 4;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;
constexpr int kMaxPeers = kPeerTableSize;
// Balanced mode charges every sequence this many chunks on top of its own. Measured on 1024 sequences
// with Zipf(1.2) lengths: 0 -> 8 takes the launch from 215 to 176 us with 2 kv heads per GPU, from
// 119 to 96 us with one, from 334 to 328 us with four; 4 and 16 are within a few percent of 8.
constexpr int kItemCostChunks = 8;
constexpr int kMaxSeqs = 1024;        // sequences per launch (prefix and length tables in shared memory)
constexpr int kHeadStride = 132;      // floats per head row in the merge buffer (bank skew)
constexpr int kMergeWarpBytes = 8 * kHeadStride * 4 + 64;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kNegBig = -1.0e30f;

enum : int { kFlagFirst = 1, kFlagLast = 2, kFlagBad = 4, kFlagEnd = 8, kFlagFinal = 16 };   // Final: the CTA's last item

struct Plan {
  int t0, c_first, n_chunks, n_pieces, chunks_per_piece;
};

// The split of a sequence into pieces.
__device__ __forceinline__ Plan make_plan(int L, int window_left, int split_chunks, int max_pieces) {
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

struct StageInfo {   // written by the producer before it arms the stage's barrier
  int b, piece, n_pieces, tok_base, lo, hi, flags;
  int next_b;        // on an item's first stage: the sequence this CTA will take next, or -1
};

__device__ __forceinline__ void prefetch_l1(const void* p) {
  asm volatile("prefetch.global.L1 [%0];" ::"l"(p));
}

template <int KVH>
struct Cfg {
  static constexpr int kSub = kConsumerWarps / KVH;            // 16-token sub-chunks per stage
  static constexpr int kStageTokens = kSub * kChunk;
  static constexpr int kRows128 = 2 * KVH;                     // 128-byte rows per token (K or V)
  static constexpr int kTileBytes = kChunk * kRows128 * 128;   // one sub-chunk of K or of V
  static constexpr int kVOffset = kSub * kTileBytes;           // = 16 KiB: K tiles, then V tiles
  static constexpr int kStageBytes = 2 * kVOffset;             // = 32 KiB
  static constexpr int kStages = 3;
  static constexpr int kRingBytes = kStages * kStageBytes;
  // warps that share a kv head (kSub > 1) merge their partial results at the end of an item in the
  // stage they have just consumed, before handing it back: no buffer of its own, so the ring has
  // three stages for every head layout
  static constexpr int kMergeBytes = kSub > 1 ? kConsumerWarps * kMergeWarpBytes : 0;
  static_assert(kMergeBytes <= kStageBytes, "the merge scratch lives inside one stage");
  static constexpr int kInfoOff = kRingBytes;
  static constexpr int kPreOff = kInfoOff + kStages * (int)sizeof(StageInfo);
  static constexpr int kLensOff = kPreOff + (kMaxSeqs + 4) * 4;
  static constexpr int kBarOff = kLensOff + kMaxSeqs * 4;
  static constexpr int kMiscOff = kBarOff + 2 * kStages * 8;
  static constexpr int kFoldBarOff = kMiscOff + 48;            // barrier of the fold's bulk copies
  static constexpr int kFoldOff = kFoldBarOff + 16;            // scratch of the shared fold: 4 x 32 x 6 floats
  static constexpr int kSmemBytes = kFoldOff + 3072 + 1024;    // + slack to align the ring to 1 KiB
  static_assert(kConsumerWarps % KVH == 0, "warps must split evenly over kv heads");
  static_assert(kVOffset == 16384, "a stage holds 16 KiB of K and 16 KiB of V");
  static_assert(kSmemBytes <= 115200, "two CTAs must fit one SM");
};

template <typename TO>
__device__ __forceinline__ void store_out(TO* p, float x);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float x) { *p = x; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float x) {
  *p = __float2bfloat16_rn(x);
}

// four consecutive outputs: one vector store where the address allows it
__device__ __forceinline__ void store_out4(float* p, float a, float b, float c, float d) {
  if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
  } else {
    p[0] = a; p[1] = b; p[2] = c; p[3] = d;
  }
}
__device__ __forceinline__ void store_out4(__nv_bfloat16* p, float a, float b, float c, float d) {
  if ((reinterpret_cast<uintptr_t>(p) & 7u) == 0) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 w;
    w.x = *reinterpret_cast<uint32_t*>(&lo);
    w.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = w;
  } else {
    p[0] = __float2bfloat16_rn(a); p[1] = __float2bfloat16_rn(b);
    p[2] = __float2bfloat16_rn(c); p[3] = __float2bfloat16_rn(d);
  }
}

__device__ __forceinline__ void consumer_bar() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
}

struct Params {
  const __nv_bfloat16* q; int64_t q_seq_stride;
  const uint8_t* k_cache; const uint8_t* v_cache;
  const int32_t* block_tables; int max_blocks;
  const int32_t* seq_lens; int B; int H; int64_t num_blocks;
  int block_size; int64_t block_stride; int window_left; float scale_log2;
  void* out; int64_t out_seq_stride; float* lse_out;
  int32_t* ctrl;      // [0] next ticket, [1] CTAs that ran out of tickets, [2] CTAs through and [3] aborts
                      // (gather), [4] set for good by a CTA whose wait ran out: the counters are then stale
  int32_t* done;      // [B] pieces finished per sequence
  float* ws_o; float* ws_ml; int split_chunks; int max_pieces; int32_t* status;
  int tile_copy;      // 1: one copy per tile (permuted-stride map), 0: one copy per 128-byte row
  int n_meta_chunks;  // 16-token chunks of always-visible sink keys (key2/value2), 0 = none
  int balanced;       // 1: equal runs of chunks per CTA; split_chunks is then the shortest run allowed
  int item_cost;      // balanced mode: what starting and finishing a sequence costs a CTA, in chunks (< 0: default)
  // Head-sharded use (kernel instantiated with PEER): every finished output row is also stored
  // into the same place of each peer GPU's gathered buffer, and the last CTA to finish raises
  // this rank's flag on every peer. ctrl[2] counts finished CTAs, ctrl[3] collects their aborts.
  void* peer_out[kMaxPeers];        // peer p's address of this rank's (sequence 0, head 0) element
  int32_t* peer_flag[kMaxPeers];    // this rank's slot in peer p's flag array
  int n_peer; int32_t flag_value; int signal;
  const int32_t* flag_base;         // device word added to flag_value when the flags are raised (may be null)
};

// Copies the finished output row of sequence b (this rank's H heads, contiguous) to every peer
// with 16-byte stores. Called by the 128 consumer threads after a consumer_bar that follows the
// row's last store, so the row is read back from this GPU's L2.
template <typename TO>
__device__ __forceinline__ void mirror_row(const Params& P, int b) {
  const int n16 = (int)(P.H * kD * sizeof(TO) / 16);
  const int64_t row = (int64_t)b * P.out_seq_stride;
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const TO*>(P.out) + row);
  for (int i = threadIdx.x; i < n16; i += kConsumers) {
    const uint4 v = __ldcg(src + i);
#pragma unroll
    for (int p = 0; p < kMaxPeers; ++p)
      if (p < P.n_peer) reinterpret_cast<uint4*>(reinterpret_cast<TO*>(P.peer_out[p]) + row)[i] = v;
  }
}

// Folds the partials (m, l, O) of a split sequence into its output row; called by the 128
// consumer threads of the CTA that completed the sequence's last piece. Thread = a float4 of dims
// of the heads warp, warp + 4, ...; the loads of four heads x four pieces are issued together, so
// a fold of up to four pieces costs two trips to L2 per thread instead of one per head and piece
// (this sits at the very end of the kernel in balanced mode, where every CTA ends at once).
// Inlined on purpose: as a separate function the call alone cost tens of microseconds.
template <typename TO>
__device__ __forceinline__ void fold_pieces(const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                         float* lse_out, int H, int max_pieces, int64_t out_seq_stride,
                                         int b, int n_pieces, TO* out) {
  const int d4 = threadIdx.x & 31;
  const int w = threadIdx.x >> 5;
  for (int h0 = w; h0 < H; h0 += 4 * kConsumerWarps) {
    float M[4], Ls[4];
    float4 O[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { M[j] = -INFINITY; Ls[j] = 0.f; O[j] = make_float4(0.f, 0.f, 0.f, 0.f); }
    for (int pc0 = 0; pc0 < n_pieces; pc0 += 4) {
      float2 ml[4][4];
      float4 o[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int h = h0 + j * kConsumerWarps < H ? h0 + j * kConsumerWarps : h0;
        const int64_t hb = (int64_t)b * max_pieces * H + h;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int64_t pi = hb + (int64_t)(pc0 + i < n_pieces ? pc0 + i : pc0) * H;
          ml[j][i] = __ldcg(reinterpret_cast<const float2*>(ws_ml + pi * 2));
          o[j][i] = __ldcg(reinterpret_cast<const float4*>(ws_o + pi * kD) + d4);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float Mn = M[j];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (pc0 + i >= n_pieces) { ml[j][i].x = -INFINITY; ml[j][i].y = 0.f; }
          Mn = fmaxf(Mn, ml[j][i].x);
        }
        const float Ms = fmaxf(Mn, kNegBig);
        const float resc = fast_exp2(M[j] - Ms);
        Ls[j] *= resc; O[j].x *= resc; O[j].y *= resc; O[j].z *= resc; O[j].w *= resc;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float wgt = fast_exp2(ml[j][i].x - Ms);
          Ls[j] += ml[j][i].y * wgt;
          O[j].x += o[j][i].x * wgt; O[j].y += o[j][i].y * wgt;
          O[j].z += o[j][i].z * wgt; O[j].w += o[j][i].w * wgt;
        }
        M[j] = Mn;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int h = h0 + j * kConsumerWarps;
      if (h >= H) break;
      const float inv = Ls[j] > 0.f ? 1.f / Ls[j] : 0.f;
      TO* op = out + (int64_t)b * out_seq_stride + (int64_t)h * kD + d4 * 4;
      store_out<TO>(op, O[j].x * inv); store_out<TO>(op + 1, O[j].y * inv);
      store_out<TO>(op + 2, O[j].z * inv); store_out<TO>(op + 3, O[j].w * inv);
      if (lse_out && d4 == 0)
        lse_out[(int64_t)b * H + h] = Ls[j] > 0.f ? (M[j] + log2f(Ls[j])) * kLn2 : -INFINITY;
    }
  }
}

// The same fold out of shared memory: `land` holds the O partials of the n_pieces pieces, [piece][H][D]
// floats, then their (m, l) pairs, [piece][H][2]. `write` false: a dry run on whatever the memory
// holds, for the sake of the instruction cache (this code runs once per CTA, at the very end of
// the kernel, and fetching it cold costs more than running it).
template <typename TO>
__device__ __noinline__ void fold_landed(const float* land, float* lse_out, int H, int64_t out_seq_stride,
                                      int b, int n_pieces, TO* out, bool write) {
  const int d4 = threadIdx.x & 31;
  const int w = threadIdx.x >> 5;
  const float2* const ml = reinterpret_cast<const float2*>(land + (int64_t)n_pieces * H * kD);
  constexpr int kU = 8;   // pieces whose loads are in flight together (the loops below are short chains otherwise)
  for (int h = w; h < H; h += kConsumerWarps) {
    float M = -INFINITY;
    for (int i0 = 0; i0 < n_pieces; i0 += kU) {
      float2 v[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) v[u] = ml[(i0 + u < n_pieces ? i0 + u : i0) * H + h];
#pragma unroll
      for (int u = 0; u < kU; ++u) M = fmaxf(M, v[u].x);
    }
    const float Ms = fmaxf(M, kNegBig);
    float Ls = 0.f;
    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i0 = 0; i0 < n_pieces; i0 += kU) {
      float2 v[kU];
      float4 o[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int i = i0 + u < n_pieces ? i0 + u : i0;
        v[u] = ml[i * H + h];
        o[u] = *reinterpret_cast<const float4*>(land + ((int64_t)i * H + h) * kD + d4 * 4);
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const float wgt = i0 + u < n_pieces ? fast_exp2(v[u].x - Ms) : 0.f;
        Ls += v[u].y * wgt;
        O.x += o[u].x * wgt; O.y += o[u].y * wgt; O.z += o[u].z * wgt; O.w += o[u].w * wgt;
      }
    }
    const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
    if (write) {
      TO* op = out + (int64_t)b * out_seq_stride + (int64_t)h * kD + d4 * 4;
      store_out4(op, O.x * inv, O.y * inv, O.z * inv, O.w * inv);
      if (lse_out && d4 == 0)
        lse_out[(int64_t)b * H + h] = Ls > 0.f ? (M + log2f(Ls)) * kLn2 : -INFINITY;
    }
  }
}

// The fold of a split sequence shared out over the CTAs that hold its pieces (balanced mode): every
// piece but the sequence's last is the last item of its CTA, which then has nothing else to do,
// so those n_pieces - 1 CTAs wait for all pieces to be counted and fold the heads between them,
// participant p the heads p, p + (n_pieces - 1), ... -- about one head each at one sequence per
// launch, where a single CTA folding 33 pieces of 28 heads took 18 us of a 30 us kernel. Within a
// CTA the four warps take every fourth piece of a head (a lane one float4 of dims, a warp's loads
// issued together: one trip to L2), leave their (m, l, O) in `scratch` (shared memory, 4 x 32 x 6
// floats) and warp 0 combines them and writes the head's output. `write` false: a dry run without
// loads from the workspace or stores, for the sake of the instruction cache (this code runs once
// per CTA, at the very end of the kernel, and fetching it cold costs more than running it).
template <typename TO>
__device__ __noinline__ void fold_heads(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, float* scratch,
                                     float* lse_out, int H, int max_pieces, int64_t out_seq_stride, int b,
                                     int n_pieces, int part, int n_part, TO* out, bool write) {
  constexpr int kB = 8;                                   // pieces of a warp whose loads are in flight together
  const int lane = threadIdx.x & 31;
  const int w = threadIdx.x >> 5;
  const int64_t seq_base = (int64_t)b * max_pieces * H;
  for (int h = part; h < H; h += n_part) {
    float M = -INFINITY, Ls = 0.f;
    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i0 = w; i0 < n_pieces; i0 += kB * kConsumerWarps) {
      float2 ml[kB];
      float4 o[kB];
#pragma unroll
      for (int u = 0; u < kB; ++u) {
        const int i = i0 + u * kConsumerWarps;
        const int64_t pi = seq_base + (int64_t)(i < n_pieces ? i : i0) * H + h;   // a piece that exists; dropped below
        if (write) {
          ml[u] = __ldcg(reinterpret_cast<const float2*>(ws_ml + pi * 2));
          o[u] = __ldcg(reinterpret_cast<const float4*>(ws_o + pi * kD) + lane);
        } else {
          ml[u] = make_float2(scratch[u], scratch[u + 1]);
          o[u] = make_float4(scratch[u], scratch[u + 1], scratch[u + 2], scratch[u + 3]);
        }
        if (i >= n_pieces) { ml[u].x = -INFINITY; ml[u].y = 0.f; }
      }
      float Mn = M;
#pragma unroll
      for (int u = 0; u < kB; ++u) Mn = fmaxf(Mn, ml[u].x);
      const float Ms = fmaxf(Mn, kNegBig);
      const float resc = fast_exp2(M - Ms);
      Ls *= resc; O.x *= resc; O.y *= resc; O.z *= resc; O.w *= resc;
#pragma unroll
      for (int u = 0; u < kB; ++u) {
        const float wgt = fast_exp2(ml[u].x - Ms);
        Ls += ml[u].y * wgt;
        O.x += o[u].x * wgt; O.y += o[u].y * wgt; O.z += o[u].z * wgt; O.w += o[u].w * wgt;
      }
      M = Mn;
    }
    consumer_bar();                                       // the scratch of the head before has been read
    if (write) {
      float* sp = scratch + (w * 32 + lane) * 6;
      sp[0] = M; sp[1] = Ls; sp[2] = O.x; sp[3] = O.y; sp[4] = O.z; sp[5] = O.w;
    }
    consumer_bar();
    if (w == 0) {
      float Mt = -INFINITY;
#pragma unroll
      for (int q = 0; q < kConsumerWarps; ++q) Mt = fmaxf(Mt, scratch[(q * 32 + lane) * 6]);
      const float Ms = fmaxf(Mt, kNegBig);
      float Lt = 0.f;
      float4 Ot = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int q = 0; q < kConsumerWarps; ++q) {
        const float* sq = scratch + (q * 32 + lane) * 6;
        const float wgt = fast_exp2(sq[0] - Ms);
        Lt += sq[1] * wgt;
        Ot.x += sq[2] * wgt; Ot.y += sq[3] * wgt; Ot.z += sq[4] * wgt; Ot.w += sq[5] * wgt;
      }
      if (write) {
        const float inv = Lt > 0.f ? 1.f / Lt : 0.f;
        TO* op = out + (int64_t)b * out_seq_stride + (int64_t)h * kD + lane * 4;
        store_out4(op, Ot.x * inv, Ot.y * inv, Ot.z * inv, Ot.w * inv);
        if (lse_out && lane == 0)
          lse_out[(int64_t)b * H + h] = Lt > 0.f ? (Mt + log2f(Lt)) * kLn2 : -INFINITY;
      }
    }
  }
}

template <int KVH, typename TO, bool PEER>
__global__ void __launch_bounds__(kThreads, 2)
swa_decode_kernel(const Params P, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_k2,
                  const __grid_constant__ CUtensorMap map_v2) {
  using C = Cfg<KVH>;
  extern __shared__ uint8_t smem_raw[];
  // the swizzle pattern is a function of the shared-memory address: tiles sit on 1 KiB boundaries
  uint8_t* const smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t ring = smem_u32(smem);
  StageInfo* info = reinterpret_cast<StageInfo*>(smem + C::kInfoOff);
  int* pre = reinterpret_cast<int*>(smem + C::kPreOff);
  int* lens_s = reinterpret_cast<int*>(smem + C::kLensOff);
  const uint32_t bar_full = ring + C::kBarOff;
  const uint32_t bar_empty = bar_full + C::kStages * 8;
  const uint32_t bar_fold = ring + C::kFoldBarOff;
  // [0] abort, [1] fold flag, [2..6] scan, [7] longest sequence in chunks, [8] workspace marked stale
  volatile int* misc = reinterpret_cast<volatile int*>(smem + C::kMiscOff);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = P.H / KVH;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, kConsumerWarps);
    }
    mbar_init(bar_fold, 1);
    misc[0] = 0;
    misc[7] = 0;
    misc[8] = __ldcg(P.ctrl + 4);
    pre[0] = 0;
    fence_mbar_init();
  }
  __syncthreads();
  // An earlier launch on this workspace gave up on a wait: its ticket and completion counters
  // were left where they stood, so nothing computed with them can be trusted. Say so again and
  // compute nothing (in the gathering form the flags stay down and the peers' wait reports the
  // step) until the caller has zeroed the head of the workspace.
  if (misc[8]) {
    if (threadIdx.x == 0) raise_status(P.status, SBK_ST_WAIT_TIMEOUT);
    return;
  }
  const int item_cost = !P.balanced ? 0 : (P.item_cost >= 0 ? P.item_cost : kItemCostChunks);
  // ---- number of pieces of every sequence, as an exclusive prefix: item w belongs to the
  //      sequence b with pre[b] <= w < pre[b+1] ----
  //      One round whatever the batch: a thread takes a run of consecutive sequences (all its
  //      loads in flight at once), the block scans the per-thread sums, and every thread writes the
  //      prefixes of its own run. (A round per kThreads sequences cost a load latency and two
  //      block barriers each, in every CTA: about 10 us ahead of the first copy at 1024 sequences.)
  {
    constexpr int kRun = (kMaxSeqs + kThreads - 1) / kThreads;
    const int run_len = (P.B + kThreads - 1) / kThreads;      // <= kRun
    const int b_lo = threadIdx.x * run_len;
    int cnt[kRun];
    int sum = 0, mx = 0;
#pragma unroll
    for (int i = 0; i < kRun; ++i) {
      const int b = b_lo + i;
      int c = 0;
      if (i < run_len && b < P.B) {
        const int Lb = P.seq_lens[b];
        lens_s[b] = Lb;
        const Plan pl = make_plan(Lb, P.window_left, P.split_chunks, P.max_pieces);
        // balanced mode counts chunks (sink chunks included; an empty sequence keeps one, so that
        // somebody writes its zero output), ticket mode counts pieces
        c = P.balanced ? (Lb > 0 ? P.n_meta_chunks + pl.n_chunks : 1) : pl.n_pieces;
        mx = max(mx, c);
        // Balanced runs are equal in cost, not in chunks: a sequence also costs its CTA a fixed
        // time (first loads, merge of the warps' partials, output), counted as `item_cost` slots
        // after its chunks that no run streams. Without them a CTA handed thirty short sequences
        // finishes long after one handed a single long sequence of the same number of chunks.
        if (P.balanced) c += item_cost;
      }
      cnt[i] = c;
      sum += c;
    }
    if (P.balanced) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      if (lane == 0) atomicMax(const_cast<int*>(&misc[7]), mx);
    }
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    if (lane == 31) misc[2 + warp] = incl;
    __syncthreads();
    int run = incl - sum;
#pragma unroll
    for (int w2 = 0; w2 < kThreads / 32; ++w2)
      if (w2 < warp) run += misc[2 + w2];
#pragma unroll
    for (int i = 0; i < kRun; ++i) {
      const int b = b_lo + i;
      if (i < run_len && b < P.B) {
        run += cnt[i];
        pre[b + 1] = run;
      }
    }
    __syncthreads();
  }
  const int total = pre[P.B];

  if (warp == kConsumerWarps) {
    // ================================= producer =================================
    int it = 0;
    bool aborted = false;

    // Streams one item: sink chunks [meta_a, meta_b) of the [n_meta, kvh, D] tensors, as stages of
    // their own, then window chunks [cb, cb + n) of sequence b (n == 0 with no sink chunk still
    // sends one empty stage, so that an empty sequence gets its zero output written).
    // `next_b`: the sequence whose item follows on this CTA (-1: none or unknown). Its block-table
    // entries are asked for now, and the consumers ask for its q row, so that neither side meets
    // a trip to L2 at the start of the next item: with short sequences those trips are most of an
    // item's time.
    auto stream_item = [&](int b, int piece, int n_pieces, int meta_a, int meta_b, int cb, int n, int next_b,
                           bool final_item = false) {
      if (next_b >= 0 && lane < 2) {
        const Plan np = make_plan(lens_s[next_b], P.window_left, P.split_chunks, P.max_pieces);
        const int lb = (np.c_first * kChunk) / P.block_size + lane * 32;
        if (lb < P.max_blocks) prefetch_l1(P.block_tables + (int64_t)next_b * P.max_blocks + lb);
      }
      const int L = lens_s[b];
      const int t0 = first_visible(L, 1, P.window_left);
      const int n_ms = (meta_b - meta_a + C::kSub - 1) / C::kSub;
      int nst = (n + C::kSub - 1) / C::kSub;
      if (nst < 1 && n_ms < 1) nst = 1;
      const int item_end = (cb + n) * kChunk;
      const int32_t* table = P.block_tables + (int64_t)b * P.max_blocks;
      int64_t pb_lane = -1;   // physical block of chunk (batch_c0 + lane): one table read per 32 chunks
      int batch_c0 = 0;
      for (int jj = -n_ms; jj < nst; ++jj, ++it) {
        const bool meta = jj < 0;
        const int j = meta ? jj + n_ms : jj;
        const int c0 = meta ? meta_a + j * C::kSub : cb + j * C::kSub;       // first chunk of this stage
        if (!meta && (j == 0 || c0 + C::kSub > batch_c0 + 32)) {
          batch_c0 = c0;
          const int c = c0 + lane;
          const int lb = (c * kChunk) / P.block_size;
          pb_lane = (c < cb + n && lb < P.max_blocks) ? (int64_t)table[lb] : -1;
        }
        const int s = it % C::kStages;
        const int use = it / C::kStages;
        if (use > 0 && !mbar_wait_bounded(bar_empty + 8 * s, (use - 1) & 1)) {
          if (lane == 0) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); P.ctrl[4] = 1; misc[0] = 1; }
          aborted = true;
          return;
        }
        if (misc[0]) { aborted = true; return; }
        const int tok_base = c0 * kChunk;
        int lo, hi;
        if (meta) {
          lo = tok_base;
          hi = tok_base + C::kStageTokens;
          if (hi > meta_b * kChunk) hi = meta_b * kChunk;
        } else {
          lo = tok_base > t0 ? tok_base : t0;
          hi = tok_base + C::kStageTokens;
          if (hi > L) hi = L;
          if (hi > item_end) hi = item_end;
          if (hi < lo) hi = lo;
        }
        // lane -> one copy of this stage: K or V, sub-chunk, and (row-wise mode) 128-byte row
        const int n_copies = P.tile_copy ? 2 * C::kSub : 2 * C::kSub * C::kRows128;
        const int is_v = lane & 1;
        const int r2 = lane >> 1;
        const int sc = P.tile_copy ? r2 : r2 / C::kRows128;
        const int row = P.tile_copy ? 0 : r2 % C::kRows128;
        const bool active = lane < n_copies;
        const int my_c = c0 + (active ? sc : 0);
        int src_lane = my_c - batch_c0;
        src_lane = src_lane < 0 ? 0 : (src_lane > 31 ? 31 : src_lane);
        const int64_t pb_tab = __shfl_sync(0xffffffffu, pb_lane, src_lane);
        const int64_t pb = meta ? (int64_t)my_c : pb_tab;      // the sink tensors are their own block table
        const int tbl = my_c * kChunk;
        const bool has_tok = (tbl > lo ? tbl : lo) < (tbl + kChunk < hi ? tbl + kChunk : hi);
        bool bad = !meta && active && has_tok && (pb < 0 || pb >= P.num_blocks);
        bad = __any_sync(0xffffffffu, bad);
        int n_sub = 0;   // sub-chunks of this stage that carry tokens
#pragma unroll
        for (int q2 = 0; q2 < C::kSub; ++q2) {
          const int t2 = tok_base + q2 * kChunk;
          n_sub += ((t2 > lo ? t2 : lo) < (t2 + kChunk < hi ? t2 + kChunk : hi)) ? 1 : 0;
        }
        if (lane == 0) {
          StageInfo si;
          si.b = b; si.piece = piece; si.n_pieces = n_pieces; si.tok_base = tok_base;
          si.lo = lo; si.hi = hi; si.next_b = next_b;
          si.flags = (jj == -n_ms ? kFlagFirst : 0) | (jj == nst - 1 ? kFlagLast : 0) | (bad ? kFlagBad : 0) |
                     (final_item && jj == nst - 1 ? kFlagFinal : 0);
          info[s] = si;
          if (bad) raise_status(P.status, SBK_ST_BAD_BLOCK);
          mbar_arrive_expect_tx(bar_full + 8 * s, bad ? 0u : (uint32_t)n_sub * 2u * C::kTileBytes);
        }
        __syncwarp();
        if (!bad && active && has_tok) {
          const uint32_t dst = ring + s * C::kStageBytes + is_v * C::kVOffset + sc * C::kTileBytes + row * 2048;
          const int tin = meta ? 0 : tbl % P.block_size;
          const CUtensorMap* map = meta ? (is_v ? &map_v2 : &map_k2) : (is_v ? &map_v : &map_k);
          if (P.tile_copy) tma_load_4d(dst, map, 0, tin, 0, (int)pb, bar_full + 8 * s);
          else tma_load_4d(dst, map, 0, row, tin, (int)pb, bar_full + 8 * s);
        }
      }
    };

    if (P.balanced) {
      // ---- equal runs of chunks: CTA g streams global chunks [g * per, (g + 1) * per) ----
      const int n_cta = (int)gridDim.x;
      int per = (total + n_cta - 1) / n_cta;
      if (per < P.split_chunks) per = P.split_chunks;
      // a sequence of C chunks meets at most ceil(C / per) + 1 runs: keep that within max_pieces
      if (P.max_pieces > 1) {
        const int need = (misc[7] + P.max_pieces - 2) / (P.max_pieces - 1);
        if (per < need) per = need;
      } else if (per < misc[7]) {
        per = misc[7];
      }
      if (per < 1) per = 1;
      const int64_t g0 = (int64_t)blockIdx.x * per;
      const int64_t g1 = g0 + per < total ? g0 + per : total;
      // A batch of near-equal sequences that already fills at least half of the CTAs streams
      // fastest as whole sequences (no partials to write and fold): sequence b goes to CTA
      // b mod n_cta. The kernel is bound by HBM, not by the busiest CTA, as long as enough CTAs
      // keep copies in flight.
      const int64_t total_chunks = (int64_t)total - (int64_t)item_cost * P.B;
      const bool whole = 2 * P.B >= n_cta && (int64_t)misc[7] * P.B <= total_chunks + total_chunks / 8;
      if (whole) {
        for (int b = (int)blockIdx.x; b < P.B && !aborted; b += n_cta) {
          const int L = lens_s[b];
          const Plan plan = make_plan(L, P.window_left, P.split_chunks, P.max_pieces);
          stream_item(b, 0, 1, 0, L > 0 ? P.n_meta_chunks : 0, plan.c_first, plan.n_chunks,
                      b + n_cta < P.B ? b + n_cta : -1);
        }
      } else if (g0 < total) {
        int lo_b = 0, hi_b = P.B;   // largest b with pre[b] <= g0
        while (hi_b - lo_b > 1) {
          const int mid = (lo_b + hi_b) >> 1;
          if (pre[mid] <= g0) lo_b = mid; else hi_b = mid;
        }
        for (int b = lo_b; b < P.B && pre[b] < g1 && !aborted; ++b) {
          const int L = lens_s[b];
          const Plan plan = make_plan(L, P.window_left, P.split_chunks, P.max_pieces);
          const int nm = L > 0 ? P.n_meta_chunks : 0;
          const int cr = L > 0 ? nm + plan.n_chunks : 1;       // the sequence's chunks; its cost slots follow them
          const int va = (int)(g0 > pre[b] ? g0 - pre[b] : 0);
          if (va >= cr) continue;                               // only cost slots of b fall into this run
          int vb = (int)((g1 < pre[b + 1] ? g1 : pre[b + 1]) - pre[b]);
          if (vb > cr) vb = cr;
          const int first_run = pre[b] / per;
          const int n_pieces = (pre[b] + cr - 1) / per - first_run + 1;
          const int ma = va < nm ? va : nm, mb = vb < nm ? vb : nm;
          const int wa = (va > nm ? va : nm) - nm, wb = (vb > nm ? vb : nm) - nm;
          const int nb = (b + 1 < P.B && pre[b + 1] < g1) ? b + 1 : -1;
          stream_item(b, (int)blockIdx.x - first_run, n_pieces, ma, mb, plan.c_first + wa,
                      L > 0 ? wb - wa : 0, nb, nb < 0);
        }
      }
    } else {
      int w_next = 0;
      if (lane == 0) w_next = atomicAdd(&P.ctrl[0], 1);
      while (!aborted) {
        const int w = __shfl_sync(0xffffffffu, w_next, 0);
        if (w >= total) break;
        if (lane == 0) w_next = atomicAdd(&P.ctrl[0], 1);   // the next ticket is on its way while this item streams
        int lo_b = 0, hi_b = P.B;   // largest b with pre[b] <= w
        while (hi_b - lo_b > 1) {
          const int mid = (lo_b + hi_b) >> 1;
          if (pre[mid] <= w) lo_b = mid; else hi_b = mid;
        }
        const int b = lo_b;
        const int piece = w - pre[b];
        const int L = lens_s[b];
        const Plan plan = make_plan(L, P.window_left, P.split_chunks, P.max_pieces);
        const int cb = plan.c_first + piece * plan.chunks_per_piece;
        int n = plan.n_chunks - piece * plan.chunks_per_piece;
        if (n > plan.chunks_per_piece) n = plan.chunks_per_piece;
        if (n < 0) n = 0;
        // sink keys are visible to every query: the first piece of a sequence streams them
        stream_item(b, piece, plan.n_pieces, 0, (piece == 0 && L > 0) ? P.n_meta_chunks : 0, cb, n, -1);
      }
    }
    if (!aborted) {
      // the end marker travels through the ring like any stage
      const int s = it % C::kStages;
      const int use = it / C::kStages;
      if (use == 0 || mbar_wait_bounded(bar_empty + 8 * s, (use - 1) & 1)) {
        if (lane == 0) {
          StageInfo si = {};
          si.flags = kFlagEnd;
          info[s] = si;
          mbar_arrive_expect_tx(bar_full + 8 * s, 0u);
        }
      } else if (lane == 0) {
        raise_status(P.status, SBK_ST_WAIT_TIMEOUT);
        P.ctrl[4] = 1;
        misc[0] = 1;
      }
      // the CTA that draws the last losing ticket rewinds the counters for the next launch
      if (lane == 0 && !P.balanced) {
        const int f = atomicAdd(&P.ctrl[1], 1);
        if (f == (int)gridDim.x - 1) { P.ctrl[0] = 0; P.ctrl[1] = 0; __threadfence(); }
      }
    }
    return;
  }

  // ================================== consumers ==================================
  const int hk = warp % KVH;     // kv head
  const int sub = warp / KVH;    // 16-token sub-chunk of a stage
  const int gq = lane >> 2;      // fragment row: token (scores) / head (B operand) / dim (output)
  const int tq = lane & 3;
  TO* const out = reinterpret_cast<TO*>(P.out);

  uint32_t qf[kD / 16][2];
  float acc[kD / 16][4];
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  // ldmatrix row addresses inside a stage. A tile is [128-byte row = head*2 + half][token][128 B] with
  // the 16-byte chunk index XOR-ed by (token & 7) (the 128-byte swizzle of the tensor copy).
  const int lj = lane >> 3, lr = lane & 7;
  const int tok_k = lr + ((lj & 1) ? 8 : 0), cj_k = lj >> 1;
  const int tok_v = lr + ((lj >> 1) ? 8 : 0), cj_v = lj & 1;
  const uint32_t k_lane_off = sub * C::kTileBytes + (hk * 32 + tok_k) * 128;
  const uint32_t v_lane_off = C::kVOffset + sub * C::kTileBytes + (hk * 32 + tok_v) * 128;
  const int xk = tok_k & 7, xv = tok_v & 7;
  // dims [16*i, 16*i+16) of a head: half = i/4 (2 KiB apart), chunks 2*(i%4) and 2*(i%4)+1
#define SBK_K_ADDR(i) (stage + k_lane_off + ((i) >> 2) * 2048 + ((((((i) & 3) << 1) + cj_k) ^ xk) << 4))
#define SBK_V_ADDR(i) (stage + v_lane_off + ((i) >> 2) * 2048 + ((((((i) & 3) << 1) + cj_v) ^ xv) << 4))

  // the fold's code, once, while the first copies are on their way (two pieces of whatever the ring holds)
  if (P.max_pieces > 1) {
    fold_landed<TO>(reinterpret_cast<const float*>(smem), nullptr, P.H, 0, 0, 2, out, false);
    fold_heads<TO>(nullptr, nullptr, reinterpret_cast<float*>(smem + C::kFoldOff), nullptr, 1, 1, 0, 0, 4, 0, 1, out, false);
  }
  for (int it = 0;; ++it) {
    const int s = it % C::kStages;
    if (!mbar_wait_bounded(bar_full + 8 * s, (it / C::kStages) & 1)) {
      if (lane == 0) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); P.ctrl[4] = 1; misc[0] = 1; }
      break;
    }
    const StageInfo si = info[s];
    if (si.flags & kFlagEnd) break;
    const uint32_t stage = ring + s * C::kStageBytes;

    if (si.flags & kFlagFirst) {
      // Q^T as the B operand of S^T = K . Q^T : b0 = dims 2tq,2tq+1 of k-step kk, b1 = +8
      const __nv_bfloat16* qp = P.q + (int64_t)si.b * P.q_seq_stride + (int64_t)(hk * G + gq) * kD + tq * 2;
#pragma unroll
      for (int kk = 0; kk < kD / 16; ++kk) {
        if (gq < G) {
          qf[kk][0] = *reinterpret_cast<const uint32_t*>(qp + kk * 16);
          qf[kk][1] = *reinterpret_cast<const uint32_t*>(qp + kk * 16 + 8);
        } else {
          qf[kk][0] = 0u; qf[kk][1] = 0u;
        }
      }
#pragma unroll
      for (int mt = 0; mt < kD / 16; ++mt) { acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f; }
      m0 = m1 = -INFINITY; l0 = l1 = 0.f;
      // the q rows of this warp's heads in the next item: G * 256 bytes, one line per lane
      if (si.next_b >= 0) {
        const uint8_t* nq = reinterpret_cast<const uint8_t*>(P.q + (int64_t)si.next_b * P.q_seq_stride + (int64_t)hk * G * kD);
        const int off = lane * 128 < G * kD * 2 ? lane * 128 : G * kD * 2 - 1;
        if (lane <= 2 * G) prefetch_l1(nq + off);
      }
    }

    const int tb = si.tok_base + sub * kChunk;            // my 16 tokens: [tb, tb+16)
    const int vlo = si.lo > tb ? si.lo : tb;
    const int vhi = si.hi < tb + kChunk ? si.hi : tb + kChunk;
    const bool ragged = vlo > tb || vhi < tb + kChunk;
    if (!(si.flags & kFlagBad) && vhi > vlo) {
      if (ragged) {
        // A tile always brings 16 token rows; those outside the visible range may hold anything.
        // Their V must be finite (a zero probability times a NaN would poison the accumulator):
        // each warp clears its own head's 256 bytes of those rows.
#pragma unroll
        for (int r0 = 0; r0 < kChunk; r0 += 2) {
          const int r = r0 + (lane >> 4);
          const int tok = tb + r;
          if (tok < vlo || tok >= vhi) {   // both 128-byte rows of my head for this token
            *reinterpret_cast<uint4*>(smem + s * C::kStageBytes + C::kVOffset + sub * C::kTileBytes +
                                      ((hk * 2 + ((lane >> 3) & 1)) * 16 + r) * 128 + (lane & 7) * 16) =
                make_uint4(0, 0, 0, 0);
          }
        }
        __syncwarp();
      }
      // ---- S^T[16 tokens, 8 heads] ----
      float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < kD / 16; kk += 2) {
        uint32_t a[4];
        ldmatrix_x4(a, SBK_K_ADDR(kk));
        mma_bf16_16816(sa, a, qf[kk][0], qf[kk][1]);
        ldmatrix_x4(a, SBK_K_ADDR(kk + 1));
        mma_bf16_16816(sb, a, qf[kk + 1][0], qf[kk + 1][1]);
      }
      float sc[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[e] = (sa[e] + sb[e]) * P.scale_log2;
      if (ragged) {
        const int ta = tb + gq, tb2 = ta + 8;
        if (ta < vlo || ta >= vhi) { sc[0] = -INFINITY; sc[1] = -INFINITY; }
        if (tb2 < vlo || tb2 >= vhi) { sc[2] = -INFINITY; sc[3] = -INFINITY; }
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
        ldmatrix_x4_trans(a, SBK_V_ADDR(mt));
        mma_bf16_16816(acc[mt], a, pb0, pb1);
        mma_bf16_16816(acc[mt], a, pc0, pc1);
      }
      if (ragged) fence_proxy_async_smem();   // my zero fill precedes the next tensor copy into these rows
    }
    __syncwarp();
    // the last stage of an item doubles as the merge scratch when warps share a kv head: it goes
    // back to the producer after the merge
    const bool keep_stage = C::kSub > 1 && (si.flags & kFlagLast);
    if (lane == 0 && !keep_stage) mbar_arrive(bar_empty + 8 * s);
    if (!(si.flags & kFlagLast)) continue;

    // ================= end of an item: write its partial or the output =================
    float ls0 = l0, ls1 = l1;   // l: sum over the 8 token lanes that share this thread's heads
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      ls0 += __shfl_xor_sync(0xffffffffu, ls0, off);
      ls1 += __shfl_xor_sync(0xffffffffu, ls1, off);
    }
    const bool direct = si.n_pieces == 1;
    const int64_t pbase = ((int64_t)si.b * P.max_pieces + si.piece) * P.H;
    if constexpr (C::kSub == 1) {
      // one warp owns a kv head outright: straight from the accumulator fragments
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int nq = 2 * tq + e;
        if (nq < G) {
          const int h = hk * G + nq;
          const float M = e ? m1 : m0, Ls = e ? ls1 : ls0;
          if (direct) {
            const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
            TO* op = out + (int64_t)si.b * P.out_seq_stride + (int64_t)h * kD;
#pragma unroll
            for (int mt = 0; mt < kD / 16; ++mt) {
              store_out<TO>(op + mt * 16 + gq, acc[mt][e] * inv);
              store_out<TO>(op + mt * 16 + gq + 8, acc[mt][2 + e] * inv);
            }
            if (P.lse_out && gq == 0)
              P.lse_out[(int64_t)si.b * P.H + h] = Ls > 0.f ? (M + log2f(Ls)) * kLn2 : -INFINITY;
          } else {
            float* wp = P.ws_o + (pbase + h) * kD;
#pragma unroll
            for (int mt = 0; mt < kD / 16; ++mt) {
              wp[mt * 16 + gq] = acc[mt][e];
              wp[mt * 16 + gq + 8] = acc[mt][2 + e];
            }
            if (gq == 0) { P.ws_ml[(pbase + h) * 2] = M; P.ws_ml[(pbase + h) * 2 + 1] = Ls; }
          }
        }
      }
      if constexpr (PEER) {
        if (direct) consumer_bar();   // the row's stores came from all four warps
      }
    } else {
      // several warps share a kv head (each took other tokens): merge through shared memory
      uint8_t* mbuf = smem + s * C::kStageBytes;
      float* wo = reinterpret_cast<float*>(mbuf + warp * kMergeWarpBytes);
      float* wml = wo + 8 * kHeadStride;
      consumer_bar();   // every warp is done reading this stage's K and V
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
        wml[8 + 2 * tq] = ls0; wml[8 + 2 * tq + 1] = ls1;
      }
      consumer_bar();
      // heads go round the four warps, a lane takes four dims of a head (one 128-bit read per
      // partial): at most H / 4 trips, two in flight, instead of H dependent ones
      const int d4 = lane * 4;
#pragma unroll 2
      for (int h = warp; h < P.H; h += kConsumerWarps) {
        const int kvhd = h / G, nq = h - kvhd * G;
        float M = -INFINITY;
#pragma unroll
        for (int sw = 0; sw < C::kSub; ++sw)
          M = fmaxf(M, reinterpret_cast<const float*>(mbuf + (kvhd + KVH * sw) * kMergeWarpBytes)[8 * kHeadStride + nq]);
        const float Ms = fmaxf(M, kNegBig);
        float Ls = 0.f;
        float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int sw = 0; sw < C::kSub; ++sw) {
          const float* po = reinterpret_cast<const float*>(mbuf + (kvhd + KVH * sw) * kMergeWarpBytes);
          const float wgt = fast_exp2(po[8 * kHeadStride + nq] - Ms);
          Ls += po[8 * kHeadStride + 8 + nq] * wgt;
          const float4 o = *reinterpret_cast<const float4*>(po + nq * kHeadStride + d4);
          O.x += o.x * wgt; O.y += o.y * wgt; O.z += o.z * wgt; O.w += o.w * wgt;
        }
        if (direct) {
          const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
          TO* op = out + (int64_t)si.b * P.out_seq_stride + (int64_t)h * kD + d4;
          store_out4(op, O.x * inv, O.y * inv, O.z * inv, O.w * inv);
          if (P.lse_out && lane == 0)
            P.lse_out[(int64_t)si.b * P.H + h] = Ls > 0.f ? (M + log2f(Ls)) * kLn2 : -INFINITY;
        } else {
          *reinterpret_cast<float4*>(P.ws_o + (pbase + h) * kD + d4) = O;
          if (lane == 0) { P.ws_ml[(pbase + h) * 2] = M; P.ws_ml[(pbase + h) * 2 + 1] = Ls; }
        }
      }
      // every reader of the scratch is done; these generic writes precede the tensor copies that
      // will refill the stage
      fence_proxy_async_smem();
      consumer_bar();
      if (lane == 0) mbar_arrive(bar_empty + 8 * s);
    }
    if (direct) {
      if constexpr (PEER) mirror_row<TO>(P, si.b);
      continue;
    }

    // ---- split sequence ----
    __threadfence();
    consumer_bar();
    // Many pieces (at most four heads per piece; measured: 24 sequences 49.7 -> 43.9 us, 32 sequences
    // 58.6 -> 55.1 us against two heads per piece, 64 and more unchanged): the fold goes head by head (fold_heads), and in
    // balanced mode it is shared out. A piece that is not the sequence's last one ends its CTA's
    // run (the sequence goes on in the next CTA's), so its CTA has nothing left to do: it counts
    // its piece, waits until all pieces are counted and folds its share of the heads. The CTA of
    // the last piece only counts. A second count by every participant tells the last one to
    // finish to put the counter back to zero for the next launch. (The grid is a cooperative
    // launch: every CTA is resident, so the wait ends.)
    const bool by_heads = 4 * (si.n_pieces - 1) >= P.H;     // the same answer for every piece of the sequence
    if (!PEER && P.balanced && by_heads) {
      const bool takes_part = si.piece < si.n_pieces - 1;
      if (threadIdx.x == 0) {
        atomicAdd(&P.done[si.b], 1);
        int ok = 1;
        if (takes_part) {
          ok = 0;
          for (uint32_t i = 0; i < (1u << 21); ++i) {
            if (*reinterpret_cast<volatile int32_t*>(&P.done[si.b]) >= si.n_pieces) { ok = 1; break; }
            __nanosleep(200);   // (polls of many CTAs on one counter get in the way of the counting)
          }
        }
        misc[1] = ok;
      }
      consumer_bar();
      const int ok = misc[1];
      consumer_bar();   // misc[1] may be rewritten by the next item only after everyone has read it
      if (!takes_part) continue;
      if (!ok) {
        if (lane == 0) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); P.ctrl[4] = 1; misc[0] = 1; }
        break;
      }
      __threadfence();
      fold_heads<TO>(P.ws_o, P.ws_ml, reinterpret_cast<float*>(smem + C::kFoldOff), P.lse_out, P.H, P.max_pieces,
                     P.out_seq_stride, si.b, si.n_pieces, si.piece, si.n_pieces - 1, out, true);
      if (threadIdx.x == 0) {
        const int prev = atomicAdd(&P.done[si.b], 1);
        if (prev == 2 * si.n_pieces - 2) P.done[si.b] = 0;   // ready for the next launch
      }
      continue;
    }
    // ---- otherwise whoever completes the last piece folds all of them ----
    if (threadIdx.x == 0) {
      const int prev = atomicAdd(&P.done[si.b], 1);
      const int last = prev == si.n_pieces - 1;
      if (last) P.done[si.b] = 0;   // ready for the next launch
      misc[1] = last;
    }
    consumer_bar();
    const int fold = misc[1];
    consumer_bar();   // misc[1] may be rewritten by the next item only after everyone has read it
    if (!fold) continue;
    __threadfence();
    // After its last item a CTA's ring is idle (only the end marker follows, which carries no data, and
    // every warp is past the barriers above): the partials of all pieces land there by bulk copies
    // issued together and are combined out of shared memory by code that has been run once already
    // (see the warm-up in front of the loop). In balanced mode this sits at the very end of the
    // kernel on every CTA at once.
    const uint32_t o_bytes = (uint32_t)P.H * kD * 4u, ml_bytes = (uint32_t)P.H * 8u;
    const float* const src_o = P.ws_o + (int64_t)si.b * P.max_pieces * P.H * kD;
    const float* const src_ml = P.ws_ml + (int64_t)si.b * P.max_pieces * P.H * 2;
    const bool land = !by_heads && (si.flags & kFlagFinal) && (ml_bytes & 15u) == 0 &&
                      (uint32_t)si.n_pieces * (o_bytes + ml_bytes) <= (uint32_t)C::kRingBytes &&
                      ((reinterpret_cast<uintptr_t>(src_o) | reinterpret_cast<uintptr_t>(src_ml)) & 15) == 0;
    if (land) {
      if (threadIdx.x == 0) {
        fence_proxy_async_all();   // the partials were written through the generic proxy (by other CTAs)
        mbar_arrive_expect_tx(bar_fold, (uint32_t)si.n_pieces * (o_bytes + ml_bytes));
        for (int i = 0; i < si.n_pieces; ++i) {
          bulk_g2s(ring + i * o_bytes, src_o + (int64_t)i * P.H * kD, o_bytes, bar_fold);
          bulk_g2s(ring + si.n_pieces * o_bytes + i * ml_bytes, src_ml + (int64_t)i * P.H * 2, ml_bytes, bar_fold);
        }
      }
      if (!mbar_wait_bounded(bar_fold, 0)) {
        if (lane == 0) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); P.ctrl[4] = 1; misc[0] = 1; }
        break;
      }
      fold_landed<TO>(reinterpret_cast<const float*>(smem), P.lse_out, P.H, P.out_seq_stride, si.b, si.n_pieces, out, true);
    } else if (by_heads) {
      // (ticket mode and the gathering form with many pieces: head by head, the shared form's arithmetic)
      fold_heads<TO>(P.ws_o, P.ws_ml, reinterpret_cast<float*>(smem + C::kFoldOff), P.lse_out, P.H, P.max_pieces,
                     P.out_seq_stride, si.b, si.n_pieces, 0, 1, out, true);
    } else {
      fold_pieces<TO>(P.ws_o, P.ws_ml, P.lse_out, P.H, P.max_pieces, P.out_seq_stride, si.b, si.n_pieces, out);
    }
    if constexpr (PEER) {
      consumer_bar();
      mirror_row<TO>(P, si.b);
    }
  }
  if constexpr (PEER) {
    // Every CTA: its peer stores are ordered before its count (the consumers' barrier, then one
    // thread's fence at system scope, which is cumulative over what the barrier ordered before it,
    // then one atomic). The CTA that counts last has therefore every row of this launch behind
    // it; it raises this rank's flag on each peer, unless some CTA gave up on a wait -- the
    // peers' own bounded wait then reports the step as failed on every rank. (A batch of more than
    // kMaxSeqs sequences is several launches of which the last one signals: a CTA that gives up in
    // an earlier one also marks the workspace, ctrl[4], so the later ones compute and signal nothing.)
    consumer_bar();
    if (threadIdx.x == 0) {
      if (misc[0]) atomicOr(&P.ctrl[3], 1);
      __threadfence_system();
      const int f = atomicAdd(&P.ctrl[2], 1);
      if (f == (int)gridDim.x - 1) {
        __threadfence_system();
        const int failed = atomicExch(&P.ctrl[3], 0);
        P.ctrl[2] = 0;
        if (P.signal && !failed) {
          const int32_t value = P.flag_value + (P.flag_base ? __ldcg(P.flag_base) : 0);
#pragma unroll
          for (int p = 0; p < kMaxPeers; ++p)
            if (p < P.n_peer)
              asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(P.peer_flag[p]), "r"(value) : "memory");
        }
      }
    }
  }
  // A wait that ran out may have left copies in flight: give them time to land before the
  // CTA retires (bounded; the result is already flagged invalid).
  if (misc[0]) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
}

template <int KVH, typename TO, bool PEER = false>
int launch_swa(const Params& P0, int B_total, int n_ctas, const CUtensorMap& map_k, const CUtensorMap& map_v,
               const CUtensorMap& map_k2, const CUtensorMap& map_v2, cudaStream_t st) {
  using C = Cfg<KVH>;
  auto kern = swa_decode_kernel<KVH, TO, PEER>;
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
  // at most kMaxSeqs sequences per launch; consecutive launches reuse the ticket counters,
  // which every launch leaves at zero
  for (int b0 = 0; b0 < B_total; b0 += kMaxSeqs) {
    Params P = P0;
    P.B = B_total - b0 < kMaxSeqs ? B_total - b0 : kMaxSeqs;
    P.q = P0.q + (int64_t)b0 * P0.q_seq_stride;
    P.block_tables = P0.block_tables + (int64_t)b0 * P0.max_blocks;
    P.seq_lens = P0.seq_lens + b0;
    P.out = (uint8_t*)P0.out + (int64_t)b0 * P0.out_seq_stride * sizeof(TO);
    if (P0.lse_out) P.lse_out = P0.lse_out + (int64_t)b0 * P0.H;
    P.done = P0.done + b0;
    if constexpr (PEER) {
      for (int p = 0; p < P0.n_peer; ++p)
        P.peer_out[p] = (uint8_t*)P0.peer_out[p] + (int64_t)b0 * P0.out_seq_stride * sizeof(TO);
      P.signal = b0 + kMaxSeqs >= B_total;   // launches of one stream finish in order: the last one tells the peers
    }
    if (P0.ws_o) {
      P.ws_o = P0.ws_o + (int64_t)b0 * P0.max_pieces * P0.H * kD;
      P.ws_ml = P0.ws_ml + (int64_t)b0 * P0.max_pieces * P0.H * 2;
    }
    int64_t items = (int64_t)P.B * P0.max_pieces;
    int grid = (int)(items < n_ctas ? items : n_ctas);
    // Balanced mode with a batch between one and two CTAs per SM: one CTA per sequence. Every
    // CTA then has work in either of the kernel's two partitions (whole sequences or equal
    // runs); idle CTAs would otherwise be left to the block scheduler's placement, and an SM
    // whose two CTAs are both idle streams nothing.
    if (P0.balanced && 2 * P.B >= n_ctas && P.B < n_ctas) grid = P.B;
    if (P0.balanced && !PEER) {
      // In balanced mode the CTAs of a sequence cut into many pieces wait for one another at the end
      // (the shared fold): the grid is launched as a cooperative one, which the driver runs only
      // with every CTA resident -- whatever else shares the GPU -- or not at all.
      void* args[] = {(void*)&P, (void*)&map_k, (void*)&map_v, (void*)&map_k2, (void*)&map_v2};
      const cudaError_t e = cudaLaunchCooperativeKernel((const void*)kern, dim3(grid), dim3(kThreads), args,
                                                        (size_t)C::kSmemBytes, st);
      if (e != cudaSuccess) {
        set_error("sbk_swa_decode: cooperative launch of %d CTAs failed: %s", grid, cudaGetErrorString(e));
        return SBK_E_LAUNCH;
      }
    } else {
      kern<<<grid, kThreads, C::kSmemBytes, st>>>(P, map_k, map_v, map_k2, map_v2);
    }
    int rc = check_launch("sbk_swa_decode");
    if (rc != SBK_OK) return rc;
  }
  return SBK_OK;
}

static size_t ctrl_bytes(int B) { return 32 + (size_t)((B + 3) / 4 * 4) * 4; }

}  // namespace sbk

extern "C" int sbk_swa_copy_mode(void) { return sbk::copy_mode(); }

extern "C" size_t sbk_swa_workspace_bytes(int B, int H, int D, int max_pieces) {
  if (B <= 0 || H <= 0 || D <= 0 || max_pieces < 1) return 0;
  size_t n = sbk::ctrl_bytes(B);
  if (max_pieces > 1) n += (size_t)B * max_pieces * H * ((size_t)D + 2) * sizeof(float);
  return n;
}

namespace sbk {
struct PeerTargets {
  void* const* out; int32_t* const* flag; int n; int32_t value; const int32_t* base;
};

static int swa_decode_impl(const void* q, int64_t q_seq_stride, const void* k_cache,
                           const void* v_cache, const int32_t* block_tables, int max_blocks,
                           const int32_t* seq_lens, int B, int H, int kvh, int D,
                           int64_t num_blocks, int block_size, int64_t cache_block_stride_bytes,
                           int window_left, float scale, void* out, int out_dtype,
                           int64_t out_seq_stride, float* lse_out, void* workspace,
                           size_t workspace_bytes, int split_chunks, int max_pieces, int item_cost,
                           const void* key2, const void* value2, int num_meta,
                           int32_t* status, void* stream, const PeerTargets* peers) {
  if (num_meta < 0 || num_meta % 16 != 0 || (num_meta > 0 && (!key2 || !value2 || !aligned16(key2) || !aligned16(value2)))) {
    set_error("sbk_swa_decode: sink tokens need 16-byte aligned key2/value2 and a count that is a multiple of 16 (got %d)",
              num_meta);
    return SBK_E_ARG;
  }
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
  if (max_pieces < 1 || max_pieces > 65535) {
    set_error("sbk_swa_decode: max_pieces=%d outside [1,65535]", max_pieces);
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
  // balanced runs cross sequence boundaries, so a sequence may always end up in two pieces
  const int balanced = split_chunks < 0 && max_pieces > 1;
  if (split_chunks < 0) split_chunks = -split_chunks;
  if (split_chunks == 0) split_chunks = 32;
  const size_t need = sbk_swa_workspace_bytes(B, H, D, max_pieces);
  if (!workspace || workspace_bytes < need) {
    set_error("sbk_swa_decode: workspace of %zu bytes given, %zu needed", workspace_bytes, need);
    return SBK_E_WORKSPACE;
  }
  if (!aligned16(workspace)) {
    set_error("sbk_swa_decode: workspace must be 16-byte aligned");
    return SBK_E_ALIGN;
  }
  Params P;
  P.q = (const __nv_bfloat16*)q; P.q_seq_stride = q_seq_stride;
  P.k_cache = (const uint8_t*)k_cache; P.v_cache = (const uint8_t*)v_cache;
  P.block_tables = block_tables; P.max_blocks = max_blocks; P.seq_lens = seq_lens;
  P.B = B; P.H = H; P.num_blocks = num_blocks; P.block_size = block_size;
  P.block_stride = cache_block_stride_bytes; P.window_left = window_left;
  P.scale_log2 = scale * kLog2e; P.out = out; P.out_seq_stride = out_seq_stride; P.lse_out = lse_out;
  P.ctrl = (int32_t*)workspace; P.done = P.ctrl + 8;
  P.ws_o = nullptr; P.ws_ml = nullptr;
  if (max_pieces > 1) {
    P.ws_o = (float*)((uint8_t*)workspace + ctrl_bytes(B));
    P.ws_ml = P.ws_o + (size_t)B * max_pieces * H * D;
  }
  P.split_chunks = split_chunks; P.max_pieces = max_pieces; P.status = status;
  P.balanced = balanced;
  P.item_cost = item_cost;
  P.n_peer = 0; P.flag_value = 0; P.signal = 0; P.flag_base = nullptr;
  for (int p = 0; p < kMaxPeers; ++p) { P.peer_out[p] = nullptr; P.peer_flag[p] = nullptr; }
  if (peers) {
    for (int p = 0; p < peers->n; ++p) { P.peer_out[p] = peers->out[p]; P.peer_flag[p] = peers->flag[p]; }
    P.n_peer = peers->n; P.flag_value = peers->value; P.flag_base = peers->base;
  }

  static int sm_count[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int sms = (dev >= 0 && dev < 64) ? sm_count[dev] : 0;
  if (sms == 0) {
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    if (dev >= 0 && dev < 64) sm_count[dev] = sms;
  }
  const int n_ctas = 2 * sms;
  // the sink tensors [num_meta, kvh, D] read as a cache of num_meta/16 blocks of 16 tokens
  const int64_t mstride = (int64_t)16 * kvh * D * 2;
  const MapKey keys[4] = {MapKey{k_cache, kvh, num_blocks, block_size, cache_block_stride_bytes, 2 * kvh},
                          MapKey{v_cache, kvh, num_blocks, block_size, cache_block_stride_bytes, 2 * kvh},
                          MapKey{key2, kvh, num_meta / 16, 16, mstride, 2 * kvh},
                          MapKey{value2, kvh, num_meta / 16, 16, mstride, 2 * kvh}};
  CUtensorMap maps[4];
  int tile_copy = 0;
  if (!get_maps(maps, keys, num_meta > 0 ? 4 : 2, &tile_copy)) {
    set_error("sbk_swa_decode: cuTensorMapEncodeTiled rejected the cache geometry (blocks=%lld block=%d kvh=%d) "
              "or the sink-token tensors", (long long)num_blocks, block_size, kvh);
    return SBK_E_ARG;
  }
  const CUtensorMap &map_k = maps[0], &map_v = maps[1];
  const CUtensorMap &map_k2 = num_meta > 0 ? maps[2] : maps[0], &map_v2 = num_meta > 0 ? maps[3] : maps[1];
  P.tile_copy = tile_copy;
  P.n_meta_chunks = num_meta / 16;
  cudaStream_t st = (cudaStream_t)stream;
#define SBK_SWA_KVH(TO)                                                            \
  switch (kvh) {                                                                   \
    case 1: return launch_swa<1, TO>(P, B, n_ctas, map_k, map_v, map_k2, map_v2, st);  \
    case 2: return launch_swa<2, TO>(P, B, n_ctas, map_k, map_v, map_k2, map_v2, st);  \
    default: return launch_swa<4, TO>(P, B, n_ctas, map_k, map_v, map_k2, map_v2, st); \
  }
  if (peers) {
    // gathered head outputs are bf16 (checked by the caller of this path)
    switch (kvh) {
      case 1: return launch_swa<1, __nv_bfloat16, true>(P, B, n_ctas, map_k, map_v, map_k2, map_v2, st);
      case 2: return launch_swa<2, __nv_bfloat16, true>(P, B, n_ctas, map_k, map_v, map_k2, map_v2, st);
      default: return launch_swa<4, __nv_bfloat16, true>(P, B, n_ctas, map_k, map_v, map_k2, map_v2, st);
    }
  }
  if (out_dtype == SBK_BF16) { SBK_SWA_KVH(__nv_bfloat16) } else { SBK_SWA_KVH(float) }
#undef SBK_SWA_KVH
}
}  // namespace sbk

extern "C" int sbk_swa_decode(const void* q, int64_t q_seq_stride, const void* k_cache,
                              const void* v_cache, const int32_t* block_tables, int max_blocks,
                              const int32_t* seq_lens, int B, int H, int kvh, int D,
                              int64_t num_blocks, int block_size, int64_t cache_block_stride_bytes,
                              int window_left, float scale, void* out, int out_dtype,
                              int64_t out_seq_stride, float* lse_out, void* workspace,
                              size_t workspace_bytes, int split_chunks, int max_pieces, int item_cost,
                              const void* key2, const void* value2, int num_meta,
                              int32_t* status, void* stream) {
  return sbk::swa_decode_impl(q, q_seq_stride, k_cache, v_cache, block_tables, max_blocks, seq_lens, B, H, kvh,
                              D, num_blocks, block_size, cache_block_stride_bytes, window_left, scale, out,
                              out_dtype, out_seq_stride, lse_out, workspace, workspace_bytes, split_chunks,
                              max_pieces, item_cost, key2, value2, num_meta, status, stream, nullptr);
}

extern "C" int sbk_swa_decode_gather(const void* q, int64_t q_seq_stride, const void* k_cache,
                                     const void* v_cache, const int32_t* block_tables, int max_blocks,
                                     const int32_t* seq_lens, int B, int H, int kvh, int D,
                                     int64_t num_blocks, int block_size, int64_t cache_block_stride_bytes,
                                     int window_left, float scale, void* out, int64_t out_seq_stride,
                                     void* workspace, size_t workspace_bytes, int split_chunks,
                                     int max_pieces, int item_cost, const void* key2, const void* value2, int num_meta,
                                     void* const* peer_out, int32_t* const* peer_flag, int n_peer,
                                     int32_t flag_value, const int32_t* flag_base, int32_t* status,
                                     void* stream) {
  using namespace sbk;
  if (n_peer < 0 || n_peer > kMaxPeers || (n_peer > 0 && (!peer_out || !peer_flag))) {
    set_error("sbk_swa_decode_gather: n_peer=%d outside [0,%d] or null peer tables", n_peer, kMaxPeers);
    return SBK_E_ARG;
  }
  if (B < 0) {
    set_error("sbk_swa_decode_gather: bad size B=%d", B);
    return SBK_E_ARG;
  }
  // rows travel as 16-byte vectors: H * D bf16 is a multiple of 16 bytes for D = 128, the bases
  // and the row stride have to be as well
  if (!aligned16(out) || (out_seq_stride * 2) % 16 != 0) {
    set_error("sbk_swa_decode_gather: out and its row stride must be 16-byte multiples");
    return SBK_E_ALIGN;
  }
  for (int p = 0; p < n_peer; ++p) {
    if (!peer_out[p] || !peer_flag[p] || !aligned16(peer_out[p]) || (reinterpret_cast<uintptr_t>(peer_flag[p]) & 3u)) {
      set_error("sbk_swa_decode_gather: peer %d: null or misaligned buffer / flag address", p);
      return SBK_E_ALIGN;
    }
  }
  if (B == 0 && n_peer > 0) {
    // nothing to compute, but the peers still wait for this step's flag
    return sbk_peer_signal(peer_flag, n_peer, flag_value, flag_base, stream);
  }
  PeerTargets pt{peer_out, peer_flag, n_peer, flag_value, flag_base};
  return swa_decode_impl(q, q_seq_stride, k_cache, v_cache, block_tables, max_blocks, seq_lens, B, H, kvh, D,
                         num_blocks, block_size, cache_block_stride_bytes, window_left, scale, out, SBK_BF16,
                         out_seq_stride, nullptr, workspace, workspace_bytes, split_chunks, max_pieces, item_cost,
                         key2, value2, num_meta, status, stream, &pt);
}

// ---------------------------------------------------------------------------------------------
// sbk_swa_decode_static: the same decode, for callers that must not allocate device memory.
//
// A serving process often hands every spare byte of HBM to its KV-cache pool when it starts, a
// real-time loop may forbid allocator calls once it is running, and a binding written in a
// language without a tensor library has no allocator to ask at all. For them the scratch of
// the decode kernel (work tickets, per-sequence completion counters, split partials) lives in
// a fixed array inside the library's own device image instead of a caller-supplied buffer.
// The price: kStaticScratchBytes of HBM on every GPU that loads the library, held until the
// process exits, and an upper limit on B * max_pieces.
namespace sbk {
constexpr size_t kStaticScratchBytes = 16u << 20;   // 16 MiB
static __device__ __align__(256) unsigned char g_swa_static_scratch[kStaticScratchBytes];
}  // namespace sbk

extern "C" size_t sbk_swa_static_scratch_bytes(void) { return sbk::kStaticScratchBytes; }

extern "C" int sbk_swa_decode_static(const void* q, int64_t q_seq_stride, const void* k_cache,
                                     const void* v_cache, const int32_t* block_tables, int max_blocks,
                                     const int32_t* seq_lens, int B, int H, int kvh, int D,
                                     int64_t num_blocks, int block_size,
                                     int64_t cache_block_stride_bytes, int window_left, float scale,
                                     void* out, int out_dtype, int64_t out_seq_stride, float* lse_out,
                                     int split_chunks, int max_pieces, int32_t* status, void* stream) {
  using namespace sbk;
  if (B < 0 || H <= 0 || D <= 0 || max_pieces < 1) {
    set_error("sbk_swa_decode_static: bad sizes B=%d H=%d D=%d max_pieces=%d", B, H, D, max_pieces);
    return SBK_E_ARG;
  }
  if (B == 0) return SBK_OK;
  const size_t need = sbk_swa_workspace_bytes(B, H, D, max_pieces);
  if (need > kStaticScratchBytes) {
    set_error("sbk_swa_decode_static: B=%d x max_pieces=%d needs %zu bytes of scratch, the built-in array "
              "holds %zu; lower max_pieces or use sbk_swa_decode with a workspace of your own",
              B, max_pieces, need, kStaticScratchBytes);
    return SBK_E_WORKSPACE;
  }
  // Inside host code the array's name is only a handle: the address a kernel can use has to be
  // asked for, once per device, while that device is current.
  static void* scratch_of_device[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("sbk_swa_decode_static: no current CUDA device (or index above 63)");
    return SBK_E_ARG;
  }
  void* scratch = scratch_of_device[dev];
  if (scratch == nullptr) {
    cudaError_t e = cudaGetSymbolAddress(&scratch, g_swa_static_scratch);
    if (e != cudaSuccess || scratch == nullptr) {
      set_error("sbk_swa_decode_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                cudaGetErrorString(e));
      return SBK_E_LAUNCH;
    }
    scratch_of_device[dev] = scratch;
  }
  // The array keeps whatever the previous call left in it. The partials are rewritten before
  // they are read; the counters at its head have to start from zero.
  cudaError_t e = cudaMemsetAsync(scratch, 0, ctrl_bytes(B), (cudaStream_t)stream);
  if (e != cudaSuccess) {
    set_error("sbk_swa_decode_static: clearing the counters failed: %s", cudaGetErrorString(e));
    return SBK_E_LAUNCH;
  }
  return sbk_swa_decode(q, q_seq_stride, k_cache, v_cache, block_tables, max_blocks, seq_lens, B, H, kvh, D,
                        num_blocks, block_size, cache_block_stride_bytes, window_left, scale, out, out_dtype,
                        out_seq_stride, lse_out, scratch, kStaticScratchBytes, split_chunks, max_pieces, -1, nullptr,
                        nullptr, 0, status, stream);
}
