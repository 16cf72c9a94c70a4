// GLA scan over a run of tokens per sequence (prefill / chunked prefill), carrying the fp32
// state: the multi-token form of gla_step.cu. For every sequence s with tokens [t0, t1):
//     S <- state[slot[s]]  (or zero when reset[s])
//     for t in t0..t1-1:   S <- diag(exp(g_t)) . S + k_t^T v_t ;   o_t = (q_t * scale) . S
//     state[slot[s]] <- S
// One CTA of 256 threads per (sequence, head). The 64 KiB state tile lives in REGISTERS for the
// whole run (thread = float4 of v columns x 16 k rows), so it crosses HBM twice per chunk instead
// of twice per token; per token only the four 128-vectors q, k, g, v are read and o written. The
// work is fp32 arithmetic on the CUDA cores (the state and read-out must hold 1e-4 against an fp32
// recurrence), so the count of operations per state element is what matters: see the round below.
// Tokens are staged eight at a time through shared memory; the read-out's sum over k rows is
// finished across the 8 row groups once per eight tokens. The same optional fused neighbours as
// the single-token step (GlaFusion): ReLU on q/k, gate logits -> log-decay, per-head RMS norm.
//
// Chunk-parallel form (a few long sequences, e.g. one 8192-token prompt chunk per GPU, which as
// one chain per (sequence, head) would occupy 28 of 296 CTA slots): a run is cut into sub-chunks
// of `sub_len` tokens that different CTAs own.
//   pass 1  (kScanLocal)  every sub-chunk but a sequence's last one is scanned WITHOUT read-out
//           (one multiply-add per state element and token instead of two): sub-chunk 0 from the
//           sequence's true incoming state, the others from zero. It leaves its end state L_j and
//           the product of its decays per key row, P_j = exp(sum_t g_t), in the workspace.
//   carry   S_in(1) = L_0;  S_in(j+1) = diag(P_j) S_in(j) + L_j  -- element-wise, in place over L_j.
//   pass 2  (kScanFull)   every sub-chunk is scanned with read-out from its true incoming state;
//           the last one writes the sequence's state back.
// The recurrence is linear in the state, so this is the same sum in another association: results
// agree with the one-chain scan to fp32 rounding (a few 1e-7 relative), not bit for bit.
#include <math.h>

#include "gla_scan_tc.cuh"
#include "sbk_common.cuh"

namespace sbk {

template <typename T>
__device__ __forceinline__ float scan_to_f32(T x);
template <>
__device__ __forceinline__ float scan_to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float scan_to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T>
__device__ __forceinline__ T scan_from_f32(float x);
template <>
__device__ __forceinline__ float scan_from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 scan_from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// four consecutive outputs: one vector store where the address allows it
__device__ __forceinline__ void scan_store4(float* p, float4 a) {
  if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
    *reinterpret_cast<float4*>(p) = a;
  } else {
    p[0] = a.x; p[1] = a.y; p[2] = a.z; p[3] = a.w;
  }
}
__device__ __forceinline__ void scan_store4(__nv_bfloat16* p, float4 a) {
  if ((reinterpret_cast<uintptr_t>(p) & 7u) == 0) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
    uint2 w;
    w.x = *reinterpret_cast<uint32_t*>(&lo);
    w.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = w;
  } else {
    p[0] = __float2bfloat16_rn(a.x); p[1] = __float2bfloat16_rn(a.y);
    p[2] = __float2bfloat16_rn(a.z); p[3] = __float2bfloat16_rn(a.w);
  }
}

constexpr int kScanTokens = 8;   // tokens staged per round

// Two fp32 values in one 64-bit register, for the packed fp32 instructions of sm_100
// (fma.rn.f32x2 / mul.rn.f32x2: two IEEE operations per instruction, same results as the scalar
// ones). The scan is bound by instructions issued per token, not by the FMA units.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 p, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}
__device__ __forceinline__ f32x2 ffma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 fmul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

enum : int { kScanFull = 0, kScanLocal = 1 };

// Where the sub-chunks of the chunk-parallel form keep their states: tiles [n_seqs][n_sub-1][H][D*D]
// then decay products [n_seqs][n_sub-1][H][D]; n_sub == 1: one chain per (sequence, head), unused.
struct ScanSplit {
  float* tiles; float* decays; int n_sub; int sub_len;
  // [n_seqs * H] or NULL: the token each (sequence, head) chain starts from when another kernel has
  // already taken the run that far (and left the state in the slot); only with n_sub == 1
  const int32_t* resume;
};

template <typename T, typename TO, int D, int MODE>
__global__ void __launch_bounds__(256, 2)
gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                const T* __restrict__ g, const int32_t* __restrict__ query_start_loc,
                float* __restrict__ state, int64_t num_slots, const int64_t* __restrict__ slot_idx,
                const uint8_t* __restrict__ reset, int H, int Hkv, float scale, TO* __restrict__ out,
                int32_t* status, const GlaFusion fu, const ScanSplit sp) {
  constexpr int TPR = D / 4;          // threads per state row
  constexpr int GROUPS = 256 / TPR;   // row groups
  constexpr int RPT = D / GROUPS;     // rows per thread
  constexpr int PPT = RPT / 2;        // ... held as pairs of adjacent rows: 2 (r0 + i GROUPS), + 1
  static_assert(RPT % 2 == 0, "rows are paired");
  const int h = blockIdx.x;
  const int s = blockIdx.y / sp.n_sub;
  const int sub = blockIdx.y - s * sp.n_sub;       // sub-chunk of the run (0 when runs are not cut)
  const int run0 = query_start_loc[s], run1 = query_start_loc[s + 1];
  const int64_t slot = slot_idx ? slot_idx[s] : (int64_t)s;
  if (slot < 0 || run1 <= run0) return;
  if (slot >= num_slots) {
    if (threadIdx.x == 0 && sub == 0 && MODE == kScanFull) raise_status(status, SBK_ST_BAD_SLOT);
    return;
  }
  int t0 = sp.n_sub > 1 ? run0 + sub * sp.sub_len : run0;
  if (sp.resume != nullptr) {
    const int done = sp.resume[(int64_t)s * H + h];
    if (done > t0) t0 = done;
  }
  // a run longer than the caller said: its last sub-chunk takes the rest
  const int t1 = sub + 1 < sp.n_sub && t0 + sp.sub_len < run1 ? t0 + sp.sub_len : run1;
  if (t0 >= run1) return;                           // the run is shorter than this sub-chunk's start
  const bool last_sub = t1 == run1;
  if (MODE == kScanLocal && last_sub) return;       // nobody needs the local state of the last sub-chunk
  // tile of this (sequence, sub-chunk, head) in the workspace, and the one before it
  const int64_t ws_idx = ((int64_t)s * (sp.n_sub - 1) + sub) * H + h;
  const int hk = h / (H / Hkv);
  const int tid = threadIdx.x;
  const int c4 = tid % TPR, r0 = tid / TPR;

  // Within a round of up to eight tokens the decays are factored out of the state: with
  // G_t[r] = g_1[r] + ... + g_t[r] (per key row r) and St = diag(exp(-G_t)) S_t,
  //     St_t = St_(t-1) + (k_t exp(-G_t)) v_t^T ,   o_t = (q_t scale exp(G_t)) . St_t ,
  // and the true state comes back at the end of the round as diag(exp(G_R)) St_R: two fused
  // multiply-adds per state element and token instead of three operations. A row whose decay
  // within a round is too strong for that (exp(-G) would leave fp32 range; gate logits far below
  // -500) makes the whole CTA keep the plain recurrence for that round.
  __shared__ __align__(16) float s_q[kScanTokens][D];   // read two rows at a time (64-bit loads)
  __shared__ __align__(16) float s_k[kScanTokens][D];
  __shared__ __align__(16) float s_end[D];        // what the row is multiplied by at the end of the round
  __shared__ int s_plain[1];        // 1: this round runs the plain recurrence
  __shared__ float4 s_v[kScanTokens][TPR];
  __shared__ float4 s_o[kScanTokens][GROUPS][TPR];

  float4* tile = reinterpret_cast<float4*>(state + ((slot * H + h) * (int64_t)D) * D);
  // incoming state: the slot (or zero on reset) for the head of the run; for a later sub-chunk the
  // carried state the pass before left in the workspace (full scan) or zero (local scan)
  const float4* tile_in = sub == 0 ? tile : reinterpret_cast<const float4*>(sp.tiles + (ws_idx - H) * (int64_t)D * D);
  const bool from_zero = sub == 0 ? (reset && reset[s] && t0 == run0) : MODE == kScanLocal;
  // SP[i][c] = (S[row, col c], S[row + 1, col c]) for row = 2 (r0 + i GROUPS) and the thread's four
  // columns: the two rows of a pair go through one packed FMA, their k (and q) values come as one
  // 64-bit shared-memory load
  f32x2 SP[PPT][4];
  if (from_zero) {
#pragma unroll
    for (int i = 0; i < PPT; ++i) SP[i][0] = SP[i][1] = SP[i][2] = SP[i][3] = 0ull;
  } else {
#pragma unroll
    for (int i = 0; i < PPT; ++i) {
      const int r = 2 * (r0 + i * GROUPS);
      const float4 a = ld_stream_f4(tile_in + (int64_t)r * TPR + c4);
      const float4 b = ld_stream_f4(tile_in + (int64_t)(r + 1) * TPR + c4);
      SP[i][0] = pack2(a.x, b.x); SP[i][1] = pack2(a.y, b.y);
      SP[i][2] = pack2(a.z, b.z); SP[i][3] = pack2(a.w, b.w);
    }
  }

  // The inputs of a round are fetched into registers one round ahead (thread -> key row d = tid % D
  // and the tokens tt = tid / D, tid / D + 256 / D, ...; every thread also takes the row's eight gate
  // values, to sum the log-decays itself), so that their latency hides behind the previous round.
  constexpr int TSTEP = 256 / D;           // 2 for D = 128, 4 for D = 64
  constexpr int TPT = kScanTokens / TSTEP; // tokens per thread and round
  const int sd = tid % D, st0 = tid / D;
  T pg[kScanTokens], pq[TPT], pk[TPT], pv[TPT];
  auto prefetch = [&](int tb2) {
#pragma unroll
    for (int tt = 0; tt < kScanTokens; ++tt)
      if (tb2 + tt < t1) pg[tt] = g[((int64_t)(tb2 + tt) * Hkv + hk) * D + sd];
#pragma unroll
    for (int u = 0; u < TPT; ++u) {
      const int64_t tok = tb2 + st0 + u * TSTEP;
      if (tok < t1) {
        const int64_t kv_off = (tok * Hkv + hk) * D + sd;
        if (MODE == kScanFull) pq[u] = q[(tok * H + h) * D + sd];
        pk[u] = k[kv_off];
        pv[u] = v[kv_off];
      }
    }
  };
  prefetch(t0);
  float g_run = 0.f;   // local scan: sum of this key row's log-decays over the sub-chunk (threads < D)

  for (int tb = t0; tb < t1; tb += kScanTokens) {
    const int nt = t1 - tb < kScanTokens ? t1 - tb : kScanTokens;
    // ---- stage the round from the registers ----
    {
      float gl[kScanTokens];
      float G = 0.f;
#pragma unroll
      for (int tt = 0; tt < kScanTokens; ++tt) {
        gl[tt] = tt < nt ? gla_gate<T>(scan_to_f32(pg[tt]), fu) : 0.f;
        G += gl[tt];
      }
      // exp(60) keeps every product well inside fp32 range (a NaN also lands on the plain side); the
      // choice is made for the whole CTA, so that the common case runs without a branch per row
      const bool plain = __syncthreads_or(!(G > -60.f)) != 0;
      if (tid == 0) s_plain[0] = plain ? 1 : 0;
      if (tid < D) s_end[sd] = plain ? 1.f : __expf(G);
      if (MODE == kScanLocal) g_run += G;
      float Gt = 0.f;
#pragma unroll
      for (int tt = 0; tt < kScanTokens; ++tt) {
        Gt += gl[tt];
        if (tt < nt && tt % TSTEP == st0) {
          float kv = scan_to_f32(pk[tt / TSTEP]);
          if (fu.relu_qk) kv = fmaxf(kv, 0.f);
          s_k[tt][sd] = plain ? kv : kv * __expf(-Gt);
          if (MODE == kScanFull) {
            float qv = scan_to_f32(pq[tt / TSTEP]);
            if (fu.relu_qk) qv = fmaxf(qv, 0.f);
            s_q[tt][sd] = plain ? qv * scale : qv * scale * __expf(Gt);
          }
          reinterpret_cast<float*>(&s_v[tt][0])[sd] = scan_to_f32(pv[tt / TSTEP]);
        }
      }
    }
    if (tb + kScanTokens < t1) prefetch(tb + kScanTokens);
    __syncthreads();
    if (!s_plain[0]) {
      // one token of the round: the state update and the read-out of this thread's rows and columns
      auto token = [&](int tt) {
        const float4 vv = s_v[tt][c4];
        const f32x2 v0 = pack2(vv.x, vv.x), v1 = pack2(vv.y, vv.y), v2 = pack2(vv.z, vv.z), v3 = pack2(vv.w, vv.w);
        f32x2 o0 = 0ull, o1 = 0ull, o2 = 0ull, o3 = 0ull;   // per column: (sum over even rows, sum over odd rows)
#pragma unroll
        for (int i = 0; i < PPT; ++i) {
          const int r = 2 * (r0 + i * GROUPS);
          const f32x2 kk = *reinterpret_cast<const f32x2*>(&s_k[tt][r]);
          SP[i][0] = ffma2(kk, v0, SP[i][0]);
          SP[i][1] = ffma2(kk, v1, SP[i][1]);
          SP[i][2] = ffma2(kk, v2, SP[i][2]);
          SP[i][3] = ffma2(kk, v3, SP[i][3]);
          if (MODE == kScanFull) {
            const f32x2 qq = *reinterpret_cast<const f32x2*>(&s_q[tt][r]);
            o0 = ffma2(qq, SP[i][0], o0);
            o1 = ffma2(qq, SP[i][1], o1);
            o2 = ffma2(qq, SP[i][2], o2);
            o3 = ffma2(qq, SP[i][3], o3);
          }
        }
        if (MODE == kScanLocal) return;
        float4 o;
        float lo, hi;
        unpack2(o0, lo, hi); o.x = lo + hi;
        unpack2(o1, lo, hi); o.y = lo + hi;
        unpack2(o2, lo, hi); o.z = lo + hi;
        unpack2(o3, lo, hi); o.w = lo + hi;
        s_o[tt][r0][c4] = o;
      };
      if (nt == kScanTokens) {
        // a full round, unrolled: the loads of the next token overlap the arithmetic of this one
#pragma unroll
        for (int tt = 0; tt < kScanTokens; ++tt) token(tt);
      } else {
        for (int tt = 0; tt < nt; ++tt) token(tt);
      }
#pragma unroll
      for (int i = 0; i < PPT; ++i) {
        const f32x2 e = *reinterpret_cast<const f32x2*>(&s_end[2 * (r0 + i * GROUPS)]);
        SP[i][0] = fmul2(SP[i][0], e); SP[i][1] = fmul2(SP[i][1], e);
        SP[i][2] = fmul2(SP[i][2], e); SP[i][3] = fmul2(SP[i][3], e);
      }
    } else {
      // (rare path: the decay is recomputed from the gate instead of being staged; scalar arithmetic)
      for (int tt = 0; tt < nt; ++tt) {
        const float4 vv = s_v[tt][c4];
        const float vc[4] = {vv.x, vv.y, vv.z, vv.w};
        float oc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < PPT; ++i) {
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int r = 2 * (r0 + i * GROUPS) + hf;
            const float d = expf(gla_gate<T>(scan_to_f32(g[((int64_t)(tb + tt) * Hkv + hk) * D + r]), fu));
            const float kk = s_k[tt][r], qq = MODE == kScanFull ? s_q[tt][r] : 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              float lo, hi;
              unpack2(SP[i][c], lo, hi);
              float& x = hf ? hi : lo;
              x = fmaf(d, x, kk * vc[c]);
              oc[c] = fmaf(qq, x, oc[c]);
              SP[i][c] = pack2(lo, hi);
            }
          }
        }
        if (MODE == kScanFull) s_o[tt][r0][c4] = make_float4(oc[0], oc[1], oc[2], oc[3]);
      }
    }
    __syncthreads();
    // ---- finish the read-out: sum the row groups; a thread takes four outputs of one token ----
    // (a token's D outputs sit in TPR consecutive lanes: one warp for D = 128, half a warp for
    // D = 64, so the sum of squares of the fused norm is a shuffle reduction, no barrier)
    // (a local scan has no read-out; the barrier above guards its staging buffers)
    for (int base = 0; MODE == kScanFull && base < nt * TPR; base += 256) {
      const int idx = base + tid;
      const bool valid = idx < nt * TPR;
      const int tt = valid ? idx / TPR : 0, c = valid ? idx - tt * TPR : 0;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (valid) {
#pragma unroll
        for (int gi = 0; gi < GROUPS; ++gi) {
          const float4 p = s_o[tt][gi][c];
          acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
      }
      if (fu.norm_weight != nullptr) {
        float sq = acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
#pragma unroll
        for (int off = TPR / 2; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
        const float rs = rsqrtf(sq / D + fu.norm_eps);
        const T* w = reinterpret_cast<const T*>(fu.norm_weight) + 4 * c;
        acc.x = acc.x * rs * scan_to_f32(w[0]);
        acc.y = acc.y * rs * scan_to_f32(w[1]);
        acc.z = acc.z * rs * scan_to_f32(w[2]);
        acc.w = acc.w * rs * scan_to_f32(w[3]);
      }
      if (valid) {
        TO* op = out + ((int64_t)(tb + tt) * H + h) * D + 4 * c;
        scan_store4(op, acc);
      }
    }
    // the next round's staging only touches s_q/s_k/s_d/s_v, and its first barrier orders the
    // reads of s_o above before the next writes to s_o
  }
  // the end state goes to the slot (end of the run), to the workspace (local scan), or nowhere (a
  // full scan of an inner sub-chunk: the carried states are already in the workspace)
  float4* tile_out = tile;
  if (MODE == kScanLocal) {
    tile_out = reinterpret_cast<float4*>(sp.tiles + ws_idx * (int64_t)D * D);
    if (tid < D) sp.decays[ws_idx * D + sd] = expf(g_run);
  } else if (!last_sub) {
    return;
  }
#pragma unroll
  for (int i = 0; i < PPT; ++i) {
    const int r = 2 * (r0 + i * GROUPS);
    float4 a, b;
    unpack2(SP[i][0], a.x, b.x); unpack2(SP[i][1], a.y, b.y);
    unpack2(SP[i][2], a.z, b.z); unpack2(SP[i][3], a.w, b.w);
    st_stream_f4(tile_out + (int64_t)r * TPR + c4, a);
    st_stream_f4(tile_out + (int64_t)(r + 1) * TPR + c4, b);
  }
}

// The carry between the two passes: for every (sequence, head), S_in(1) = L_0 stays where it is and
// S_in(j+1) = diag(P_j) S_in(j) + L_j replaces L_j for j = 1 .. n_sub-2, in order. Element-wise: a CTA
// takes D*D/kCarrySplit elements of a tile, a thread one float4 of them per trip.
constexpr int kCarrySplit = 8;
template <int D>
__global__ void __launch_bounds__(256)
gla_scan_carry_kernel(const int32_t* __restrict__ query_start_loc, const int64_t* __restrict__ slot_idx,
                      int64_t num_slots, int H, const ScanSplit sp) {
  const int h = blockIdx.x / kCarrySplit, part = blockIdx.x % kCarrySplit;
  const int s = blockIdx.y;
  const int n_tok = query_start_loc[s + 1] - query_start_loc[s];
  const int64_t slot = slot_idx ? slot_idx[s] : (int64_t)s;
  if (slot < 0 || slot >= num_slots || n_tok <= 0) return;
  int n_used = (n_tok + sp.sub_len - 1) / sp.sub_len;         // sub-chunks this run really has
  n_used = n_used < sp.n_sub ? n_used : sp.n_sub;
  constexpr int kPer = D * D / 4 / kCarrySplit;               // float4s per CTA
  for (int e = threadIdx.x; e < kPer; e += 256) {
    const int e4 = part * kPer + e;
    const int row = e4 / (D / 4);
    const int64_t base = ((int64_t)s * (sp.n_sub - 1)) * H + h;
    float4 S = reinterpret_cast<const float4*>(sp.tiles + base * (int64_t)D * D)[e4];
    for (int j = 1; j + 1 < n_used; ++j) {
      const int64_t idx = base + (int64_t)j * H;
      float4* lp = reinterpret_cast<float4*>(sp.tiles + idx * (int64_t)D * D) + e4;
      const float4 L = *lp;
      const float pj = sp.decays[idx * D + row];
      S.x = fmaf(pj, S.x, L.x); S.y = fmaf(pj, S.y, L.y);
      S.z = fmaf(pj, S.z, L.z); S.w = fmaf(pj, S.w, L.w);
      *lp = S;
    }
  }
}

// How a call is cut into sub-chunks: only when the (sequence, head) chains would leave at least
// half of the machine's CTA slots (two per SM, 148 SMs) empty, into as many sub-chunks as fill
// them, none shorter than 256 tokens (a sub-chunk costs a state tile in and out on top of its
// tokens). Returns n_sub (1: do not cut) and sets *sub_len (a multiple of the staging round).
// Head of the workspace for the tensor-core form: per (sequence, head) the hand-over position, then
// the flag "a piece of this run cannot be taken" of the chunk-parallel use.
static size_t resume_bytes(int n_seqs, int max_query_len, int H) {
  if (max_query_len < gla_tc::kMinRun) return 0;
  return ((size_t)2 * n_seqs * H * sizeof(int32_t) + 255) / 256 * 256;
}

// How the tensor-core form cuts its runs: one CTA per SM (its operands fill the shared memory), so
// 148 slots; only when the chains fill at most half of them, and into pieces of at least two chunks.
static int tc_split_plan(int n_seqs, int max_query_len, int H, int* sub_chunks) {
  constexpr int kSlots = 148;
  const int n_chunks = (max_query_len + gla_tc::kChunkTokens - 1) / gla_tc::kChunkTokens;
  *sub_chunks = n_chunks;
  const int64_t chains = (int64_t)n_seqs * H;
  if (chains <= 0 || n_chunks < 4 || 2 * chains > kSlots) return 1;
  int n_sub = (int)(kSlots / chains);
  int per = (n_chunks + n_sub - 1) / n_sub;
  if (per < 2) per = 2;
  n_sub = (n_chunks + per - 1) / per;
  if (n_sub < 2) return 1;
  *sub_chunks = per;
  return n_sub;
}

static int scan_split_plan(int n_seqs, int max_query_len, int H, int* sub_len) {
  constexpr int kSlots = 2 * 148;
  *sub_len = max_query_len;
  const int64_t chains = (int64_t)n_seqs * H;
  if (chains <= 0 || max_query_len < 512 || 2 * chains > kSlots) return 1;
  int n_sub = (int)(kSlots / chains);
  if (n_sub > max_query_len / 256) n_sub = max_query_len / 256;
  if (n_sub > 64) n_sub = 64;
  if (n_sub < 2) return 1;
  int len = (max_query_len + n_sub - 1) / n_sub;
  len = (len + kScanTokens - 1) / kScanTokens * kScanTokens;
  *sub_len = len;
  return (max_query_len + len - 1) / len;
}

}  // namespace sbk

extern "C" size_t sbk_gla_scan_workspace_bytes(int n_seqs, int max_query_len, int H, int D) {
  if (n_seqs <= 0 || H <= 0 || D <= 0) return 0;
  int sub_len = 0;
  const int n_sub = sbk::scan_split_plan(n_seqs, max_query_len, H, &sub_len);
  // the hand-over positions of the tensor-core form come first, the sub-chunk states after them
  size_t n = sbk::resume_bytes(n_seqs, max_query_len, H);
  int per = 0;
  const int n_sub_tc = n > 0 ? sbk::tc_split_plan(n_seqs, max_query_len, H, &per) : 1;
  const int most = n_sub > n_sub_tc ? n_sub : n_sub_tc;     // whichever form the call takes
  if (most >= 2) n += (size_t)n_seqs * (most - 1) * H * ((size_t)D * D + D) * sizeof(float);
  return n;
}

extern "C" int sbk_gla_scan(const void* q, const void* k, const void* v, const void* g, int in_dtype,
                            const int32_t* query_start_loc, int n_seqs, float* state,
                            int64_t num_slots, const int64_t* slot_idx, const uint8_t* reset, int H,
                            int Hkv, int D, float scale, void* out, int out_dtype, int fuse_flags,
                            float gate_normalizer, const void* norm_weight, float norm_eps,
                            int max_query_len, void* workspace, size_t workspace_bytes,
                            int32_t* status, void* stream) {
  using namespace sbk;
  GlaFusion fu;
  if (!make_gla_fusion(&fu, "sbk_gla_scan", fuse_flags, gate_normalizer, norm_weight, norm_eps)) return SBK_E_ARG;
  if (n_seqs < 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || num_slots < 0) {
    set_error("sbk_gla_scan: bad head counts H=%d Hkv=%d or negative size", H, Hkv);
    return SBK_E_ARG;
  }
  if (D != 64 && D != 128) {
    set_error("sbk_gla_scan: D=%d unsupported (64 or 128)", D);
    return SBK_E_ARG;
  }
  if ((in_dtype != SBK_BF16 && in_dtype != SBK_F32) || (out_dtype != SBK_BF16 && out_dtype != SBK_F32)) {
    set_error("sbk_gla_scan: in_dtype=%d / out_dtype=%d unsupported", in_dtype, out_dtype);
    return SBK_E_ARG;
  }
  if (n_seqs == 0) return SBK_OK;
  if (!q || !k || !v || !g || !state || !out || !query_start_loc) {
    set_error("sbk_gla_scan: null pointer");
    return SBK_E_ARG;
  }
  if (!aligned16(state)) {
    set_error("sbk_gla_scan: state must be 16-byte aligned");
    return SBK_E_ALIGN;
  }
  if (n_seqs > 65535) {
    set_error("sbk_gla_scan: n_seqs=%d exceeds 65535", n_seqs);
    return SBK_E_ARG;
  }
  // One chain per (sequence, head), or -- given a workspace and the longest run -- the
  // chunk-parallel form when the chains alone would leave most of the GPU idle.
  ScanSplit sp{nullptr, nullptr, 1, 0, nullptr};
  cudaStream_t st = (cudaStream_t)stream;
  if (workspace != nullptr && max_query_len > 0) {
    const size_t need = sbk_gla_scan_workspace_bytes(n_seqs, max_query_len, H, D);
    if (workspace_bytes < need) {
      set_error("sbk_gla_scan: workspace of %zu bytes given, %zu needed (sbk_gla_scan_workspace_bytes)",
                workspace_bytes, need);
      return SBK_E_WORKSPACE;
    }
    if (need > 0 && !aligned16(workspace)) {
      set_error("sbk_gla_scan: workspace must be 16-byte aligned");
      return SBK_E_ALIGN;
    }
    const size_t rb = resume_bytes(n_seqs, max_query_len, H);
    if (rb > 0 && in_dtype == SBK_BF16 && D == 128 && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(g) &&
        aligned16(out)) {
      // Long runs of bf16 tokens at head dim 128: the chunked form on the tensor cores takes every run as
      // far as its gates allow; the token-by-token kernel below finishes what it left (normally nothing).
      gla_tc::Params T;
      T.q = (const __nv_bfloat16*)q; T.k = (const __nv_bfloat16*)k; T.v = (const __nv_bfloat16*)v;
      T.g = (const __nv_bfloat16*)g; T.query_start_loc = query_start_loc; T.state = state; T.num_slots = num_slots;
      T.slot_idx = slot_idx; T.reset = reset; T.H = H; T.Hkv = Hkv; T.scale = scale; T.out = out;
      T.out_f32 = out_dtype == SBK_F32; T.status = status; T.fu = fu; T.resume = (int32_t*)workspace;
      T.tiles = nullptr; T.decays = nullptr; T.n_sub = 1; T.sub_chunks = 0; T.bail = nullptr;
      int per = 0;
      const int n_sub_tc = tc_split_plan(n_seqs, max_query_len, H, &per);
      if (n_sub_tc > 1 && D == 128) {
        // few long runs: every run in pieces that different CTAs own -- local pass, carry, full pass
        T.n_sub = n_sub_tc; T.sub_chunks = per;
        T.bail = T.resume + (size_t)n_seqs * H;
        T.tiles = (float*)((uint8_t*)workspace + rb);
        T.decays = T.tiles + (size_t)n_seqs * (n_sub_tc - 1) * H * D * D;
        if (cudaMemsetAsync(T.bail, 0, (size_t)n_seqs * H * sizeof(int32_t), st) != cudaSuccess) {
          set_error("sbk_gla_scan: clearing the workspace head failed");
          return SBK_E_LAUNCH;
        }
        int rc = gla_tc::launch(T, n_seqs, true, st);
        if (rc != SBK_OK) return rc;
        if (n_sub_tc > 2) {
          const ScanSplit cs{T.tiles, T.decays, n_sub_tc, per * gla_tc::kChunkTokens, nullptr};
          gla_scan_carry_kernel<128><<<dim3(H * kCarrySplit, n_seqs), 256, 0, st>>>(query_start_loc, slot_idx, num_slots, H, cs);
          rc = check_launch("sbk_gla_scan");
          if (rc != SBK_OK) return rc;
        }
      }
      const int rc = gla_tc::launch(T, n_seqs, false, st);
      if (rc != SBK_OK) return rc;
      sp.resume = (const int32_t*)workspace;
    } else {
      int sub_len = 0;
      const int n_sub = scan_split_plan(n_seqs, max_query_len, H, &sub_len);
      if (n_sub > 1) {
        sp.tiles = (float*)((uint8_t*)workspace + rb);
        sp.decays = sp.tiles + (size_t)n_seqs * (n_sub - 1) * H * D * D;
        sp.n_sub = n_sub;
        sp.sub_len = sub_len;
      }
    }
  }
  if ((int64_t)n_seqs * sp.n_sub > 65535) {
    set_error("sbk_gla_scan: n_seqs=%d x %d sub-chunks exceeds 65535", n_seqs, sp.n_sub);
    return SBK_E_ARG;
  }
  dim3 grid(H, n_seqs * sp.n_sub);
#define SBK_SCAN_LAUNCH(T, TO, DD)                                                                      \
  do {                                                                                                  \
    if (sp.n_sub > 1) {                                                                                 \
      gla_scan_kernel<T, TO, DD, kScanLocal><<<grid, 256, 0, st>>>(                                     \
          (const T*)q, (const T*)k, (const T*)v, (const T*)g, query_start_loc, state, num_slots,        \
          slot_idx, reset, H, Hkv, scale, (TO*)out, status, fu, sp);                                    \
      if (sp.n_sub > 2)                                                                                 \
        gla_scan_carry_kernel<DD><<<dim3(H * kCarrySplit, n_seqs), 256, 0, st>>>(query_start_loc,       \
                                                                                 slot_idx, num_slots, H, sp); \
    }                                                                                                   \
    gla_scan_kernel<T, TO, DD, kScanFull><<<grid, 256, 0, st>>>(                                        \
        (const T*)q, (const T*)k, (const T*)v, (const T*)g, query_start_loc, state, num_slots,          \
        slot_idx, reset, H, Hkv, scale, (TO*)out, status, fu, sp);                                      \
  } while (0)
#define SBK_SCAN_D(T, TO)                     \
  do {                                        \
    if (D == 128) SBK_SCAN_LAUNCH(T, TO, 128); \
    else SBK_SCAN_LAUNCH(T, TO, 64);          \
  } while (0)
  if (in_dtype == SBK_BF16) {
    if (out_dtype == SBK_BF16) SBK_SCAN_D(__nv_bfloat16, __nv_bfloat16);
    else SBK_SCAN_D(__nv_bfloat16, float);
  } else {
    if (out_dtype == SBK_BF16) SBK_SCAN_D(float, __nv_bfloat16);
    else SBK_SCAN_D(float, float);
  }
#undef SBK_SCAN_D
#undef SBK_SCAN_LAUNCH
  return check_launch("sbk_gla_scan");
}
