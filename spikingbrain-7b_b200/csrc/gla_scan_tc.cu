// GLA scan over runs of tokens on the 5th-generation tensor cores (tcgen05, accumulators in TMEM):
// the chunked form of the recurrence   S <- diag(exp g_t) S + k_t^T v_t ,  o_t = (q_t scale) S .
//
// One CTA per (sequence, head) walks its run in chunks of 128 tokens. With G_t = g_1 + ... + g_t the
// log-decay summed from the start of the chunk (per key dim), qs_t = q_t scale exp(G_t) and
// ks_t = k_t exp(-G_t), a chunk is four matrix products:
//     A   = Qs . Ks^T , keeping s <= t            [128 tokens x 128 tokens]   (inside the chunk)
//     O   = A . V + Qs . S_in                     [128 tokens x 128 dims]     (+ what came before it)
//     S'  = S_in + Ks^T . V ;  S_out = diag(exp G_C) S'                       (state carry)
// The state and the read-out must hold 1e-4 against an fp32 recurrence, which one bf16 operand
// (2^-9) cannot: every fp32 operand is split into a bf16 head and a bf16 remainder (2^-17 together)
// and a product of two split operands is three MMAs (head.head + head.rem + rem.head); V comes as bf16
// and is exact. 10 x 8 MMAs of M128 N128 K16 per chunk, 42 MFLOP, against 65 kFLOP per token of fp32
// arithmetic on the CUDA cores for the token-by-token form.
// Roles (544 threads): warps 0-15 prepare the operands (cumulative gates, exponentials, splits into
//   swizzled shared-memory panels), mask and split A in tensor memory, rescale the state, write the
//   outputs; warp 16 allocates TMEM and issues the MMAs. Hand-offs are mbarriers (tcgen05.commit on the
//   tensor side); every wait is bounded.
// Tensor memory: S [0,128) fp32, O [128,256) fp32, A [256,384) fp32 -> packed bf16 head / remainder.
// Shared memory: Qs head/rem, Ks head/rem, V, S head/rem: seven [128 x 128] bf16 operands of 32 KiB,
//   each two [128 rows][128 B] panels with the 128-byte swizzle. Read K-major (rows = tokens, K =
//   dims) in Qs.Ks^T and Qs.S, MN-major (rows = the contraction index) for V, S and Ks in Ks^T.V.
// exp(-G_t) grows with the decay inside a chunk: a chunk whose summed log-decay leaves [-80, 0] in
// any key dim is not taken. The CTA then stores its state and the position in `resume`, and the
// token-by-token kernel, launched behind this one, finishes the run from there.
#include "gla_scan_tc.cuh"

#include "sbk_tcgen05.cuh"

namespace sbk {
namespace gla_tc {

using namespace tc5;

constexpr int kD = 128;
constexpr int kC = 128;                        // tokens per chunk
constexpr int kPanelBytes = 128 * 128;
constexpr int kOperandBytes = 2 * kPanelBytes;
constexpr int kQH = 0, kQL = kOperandBytes, kKH = 2 * kOperandBytes, kKL = 3 * kOperandBytes;
constexpr int kV = 4 * kOperandBytes, kSH = 5 * kOperandBytes, kSL = 6 * kOperandBytes;
constexpr int kMiscOff = 7 * kOperandBytes;    // exp(G_C) [128] f32, barriers, TMEM slot, flags
constexpr int kSmemBytes = kMiscOff + 768 + 1024;
constexpr int kWorkers = 512;
constexpr int kThreads = kWorkers + 32;
constexpr int kSCol = 0, kOCol = 128, kACol = 256;
constexpr int kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kMaxDecay = 80.f;              // |G_C| beyond this: the chunk goes to the other kernel
// scratch that lives in the V operand's bytes while V itself is not there
constexpr int kPartOff = kV;                   // [32][128] f32: per token group, the sum of its four gates
constexpr int kXchOff = kV + 16384;            // [4][128] f32: partial sums of squares of the fused norm
constexpr int kStageOff = kQH;                 // output rows of a chunk on their way out: 128 x (512 + 16) bytes at most

__device__ __forceinline__ void workers_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kWorkers) : "memory"); }
// the four warps that share the TMEM lanes (rows) 32 q ... 32 q + 31
__device__ __forceinline__ void row_bar(int q) { asm volatile("bar.sync %0, 128;" ::"r"(q + 2) : "memory"); }

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// F: which element-wise neighbours are compiled in -- bit 0 ReLU on q/k, bit 1 gate logits ->
// log-decay, bit 2 per-head RMS norm; -1: whatever the call's flags say, decided at run time.
// Instantiated for 0 (plain), 7 (the reference layer's three) and -1 (any other mix): without
// run-time branches inside its unrolled loops the compiler keeps the global loads of a chunk ahead
// of their uses (0.76 -> 0.62 ms on one 8192-token run for the plain one).
// LOCAL: the first pass of the chunk-parallel form: no queries, no read-out (of the five products
// only S += Ks^T . V), the end state and the product of the decays go to the workspace.
template <int F, bool LOCAL>
__global__ void __launch_bounds__(kThreads, 1) gla_scan_tc_kernel(const Params P) {
  const bool f_relu = F < 0 ? P.fu.relu_qk != 0 : (F & 1) != 0;
  const bool f_gate = F < 0 ? P.fu.gate_logits != 0 : (F & 2) != 0;
  const bool f_norm = F < 0 ? P.fu.norm_weight != nullptr : (F & 4) != 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* const smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  const int h = blockIdx.x;
  const int s = blockIdx.y / P.n_sub, sub = blockIdx.y - s * P.n_sub;   // sub: this CTA's piece of the run
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int run0 = P.query_start_loc[s], run1 = P.query_start_loc[s + 1];
  const int64_t slot = P.slot_idx ? P.slot_idx[s] : (int64_t)s;
  int32_t* const my_resume = P.resume + (int64_t)s * P.H + h;
  if (slot < 0 || run1 <= run0 || slot >= P.num_slots) {   // whole CTA, before anything is allocated
    if (tid == 0 && sub == 0 && !LOCAL) {
      *my_resume = run1;
      if (slot >= P.num_slots) raise_status(P.status, SBK_ST_BAD_SLOT);
    }
    return;
  }
  const int n_chunks = (run1 - run0 + kC - 1) / kC;                       // of the run
  const int c_lo = P.n_sub > 1 ? sub * P.sub_chunks : 0;                  // of this CTA: [c_lo, c_hi)
  // a run longer than the caller said: its last piece takes the rest
  const int c_hi = sub + 1 < P.n_sub && c_lo + P.sub_chunks < n_chunks ? c_lo + P.sub_chunks : n_chunks;
  const bool is_last = c_hi == n_chunks;
  if (c_lo >= n_chunks) return;          // the run is shorter than this piece's start
  if (LOCAL && is_last) return;          // nobody needs the local state of a run's last piece
  int32_t* const my_bail = P.bail ? P.bail + (int64_t)s * P.H + h : nullptr;
  if (!LOCAL && my_bail != nullptr && *my_bail != 0) {   // the local pass met a chunk it does not take
    if (is_last && tid == 0) *my_resume = run0;          // the whole run goes to the other kernel
    return;
  }
  if (sbase - smem_u32(smem_raw) > 1023u) {   // the launch leaves room for this much padding only
    if (tid == 0) {
      raise_status(P.status, SBK_ST_WAIT_TIMEOUT);
      if (is_last && !LOCAL) *my_resume = run1;
    }
    return;
  }
  // tile of this (sequence, piece, head) in the workspace; the piece before it is H tiles back
  const int64_t ws_idx = ((int64_t)s * (P.n_sub - 1) + sub) * P.H + h;
  float* const egc = reinterpret_cast<float*>(smem + kMiscOff);                 // exp(G_C) per key dim
  const uint32_t bar_prep = sbase + kMiscOff + 512, bar_a = bar_prep + 8, bar_p = bar_a + 8;
  const uint32_t bar_s = bar_p + 8, bar_o = bar_s + 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kMiscOff + 512 + 64);
  volatile int* flags = reinterpret_cast<volatile int*>(smem + kMiscOff + 512 + 96);   // [0] abort, [1] stop here, [2] scan says stop

  if (tid == 0) {
    mbar_init(bar_prep, kWorkers);
    mbar_init(bar_a, 1);
    mbar_init(bar_p, kWorkers);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    flags[0] = 0; flags[1] = 0; flags[2] = 0;
    fence_mbar_init();
  }
  if (warp == kWorkers / 32) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int hk = h / (P.H / P.Hkv);

  if (warp == kWorkers / 32) {
    // ================================= MMA issuer =================================
    const uint32_t id_kk = instr_desc(0, 0), id_kmn = instr_desc(1, 0), id_mnmn = instr_desc(1, 1);
    bool ok = true;
    for (int c = c_lo; ok && c < c_hi; ++c) {
      const uint32_t ph = (c - c_lo) & 1;
      ok = mbar_wait_bounded(bar_prep, ph);
      if (!ok || flags[0] || flags[1]) break;
      tc_fence_after();
      if (LOCAL) {
        if (lane == 0) {
#pragma unroll
          for (int pr = 0; pr < 2; ++pr) {
            const uint32_t ka = sbase + (pr ? kKL : kKH);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_bf16(tmem + kSCol, smem_desc(ka + k * 2048, kPanelBytes), smem_desc(sbase + kV + k * 2048, kPanelBytes),
                        id_mnmn, 1);
          }
          umma_commit(bar_s);
        }
        __syncwarp();
        continue;
      }
      if (lane == 0) {
        // A = Qs . Ks^T : both K-major, 8 steps of 16 dims (4 per 64-dim panel)
#pragma unroll
        for (int pr = 0; pr < 3; ++pr) {
          const uint32_t qa = sbase + (pr == 2 ? kQL : kQH), ka = sbase + (pr == 1 ? kKL : kKH);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = (k >> 2) * kPanelBytes + (k & 3) * 32;
            umma_bf16(tmem + kACol, smem_desc(qa + off, 16), smem_desc(ka + off, 16), id_kk, (pr > 0) || (k > 0));
          }
        }
        umma_commit(bar_a);
        // O = Qs . S_in : Qs K-major; S as B with the key dim as K and the value dim contiguous (MN-major)
#pragma unroll
        for (int pr = 0; pr < 3; ++pr) {
          const uint32_t qa = sbase + (pr == 2 ? kQL : kQH), sa = sbase + (pr == 1 ? kSL : kSH);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = (k >> 2) * kPanelBytes + (k & 3) * 32;
            umma_bf16(tmem + kOCol, smem_desc(qa + off, 16), smem_desc(sa + k * 2048, kPanelBytes), id_kmn,
                      (pr > 0) || (k > 0));
          }
        }
        // S += Ks^T . V : both MN-major (rows = tokens = the contraction index), 8 steps of 16 tokens
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {
          const uint32_t ka = sbase + (pr ? kKL : kKH);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_bf16(tmem + kSCol, smem_desc(ka + k * 2048, kPanelBytes), smem_desc(sbase + kV + k * 2048, kPanelBytes),
                      id_mnmn, 1);
        }
        umma_commit(bar_s);
      }
      __syncwarp();
      // O += A . V once the masked A is back in tensor memory as bf16 head / remainder
      ok = mbar_wait_bounded(bar_p, ph);
      if (!ok || flags[0]) break;
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t vd = smem_desc(sbase + kV + k * 2048, kPanelBytes);
          umma_bf16_ts(tmem + kOCol, tmem + kACol + k * 8, vd, id_kmn, 1);
          umma_bf16_ts(tmem + kOCol, tmem + kACol + 64 + k * 8, vd, id_kmn, 1);
        }
        umma_commit(bar_o);
      }
      __syncwarp();
    }
    if (!ok && lane == 0 && !flags[0]) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); flags[0] = 1; }
  } else {
    // ================================== workers ==================================
    // TMEM-side layout: row r = TMEM lane, this thread's 32 columns [32 part, 32 part + 32)
    const int r = (warp & 3) * 32 + lane, part = warp >> 2;
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int s_panel = part >> 1, s_c0 = (part & 1) * 4;     // where those columns sit in a bf16 operand
    // prepare-side layout: four consecutive tokens, eight consecutive dims
    const int tg = tid >> 4, dg = tid & 15, d0 = dg * 8;
    const uint32_t p_off = (uint32_t)((dg >> 3) * kPanelBytes);
    float* const tile = P.state + ((slot * P.H + h) * (int64_t)kD) * kD;
    float* const part_s = reinterpret_cast<float*>(smem + kPartOff);
    float* const xch = reinterpret_cast<float*>(smem + kXchOff);
    bool ok = true;

    // split 32 fp32 values (this thread's columns of row r) into the bf16 head / remainder operands
    auto store_state_split = [&](const uint32_t (&x)[32]) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          split_bf16x2(__uint_as_float(x[c * 8 + 2 * e]), __uint_as_float(x[c * 8 + 2 * e + 1]), hi[e], lo[e]);
        const uint32_t o = (uint32_t)(s_panel * kPanelBytes) + swz(r, s_c0 + c);
        *reinterpret_cast<uint4*>(smem + kSH + o) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(smem + kSL + o) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      }
    };
    auto store_state_global = [&](const uint32_t (&x)[32], float* to) {
      float4* dst = reinterpret_cast<float4*>(to + (int64_t)r * kD + part * 32);
#pragma unroll
      for (int c = 0; c < 8; ++c)
        st_stream_f4(dst + c, make_float4(__uint_as_float(x[4 * c]), __uint_as_float(x[4 * c + 1]),
                                          __uint_as_float(x[4 * c + 2]), __uint_as_float(x[4 * c + 3])));
    };

    // ---- incoming state: the slot (or zero) -> tensor memory and the split operands ----
    {
      uint32_t sv[32];
      // the run's slot (or zero) for its first piece; for a later piece the carried state of the pass
      // before (full pass) or zero (local pass)
      const bool from_zero = sub == 0 ? (P.reset && P.reset[s]) : LOCAL;
      const float* src_tile = sub == 0 ? tile : P.tiles + (ws_idx - P.H) * (int64_t)kD * kD;
      if (from_zero) {
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[i] = 0u;
      } else {
        const float4* src = reinterpret_cast<const float4*>(src_tile + (int64_t)r * kD + part * 32);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float4 x = ld_stream_f4(src + c);
          sv[4 * c] = __float_as_uint(x.x); sv[4 * c + 1] = __float_as_uint(x.y);
          sv[4 * c + 2] = __float_as_uint(x.z); sv[4 * c + 3] = __float_as_uint(x.w);
        }
      }
      tmem_st32(t_lane + kSCol + part * 32, sv);
      store_state_split(sv);
      tmem_st_wait();
    }

    float g_piece = 0.f;   // local pass, threads < 128: log-decay of key dim `tid` summed over the piece
    int c = c_lo;
    for (; c < c_hi; ++c) {
      const uint32_t ph = (c - c_lo) & 1;
      const int tb = run0 + c * kC;
      const int nt = run1 - tb < kC ? run1 - tb : kC;
      bulk_wait_read<0>();   // (the threads that sent the previous chunk's rows off: the staging bytes are free)
      // ============ prepare: cumulative gates, Qs / Ks split, V ============
      float cum[4][8];
      {
        float run[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) run[j] = 0.f;
        // (all four loads are issued before the first is used: one trip to L2, not four)
        uint4 gw4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tl = tg * 4 + i;
          const int tc = tl < nt ? tl : 0;   // a row that exists; its value is dropped below
          gw4[i] = *reinterpret_cast<const uint4*>(P.g + ((int64_t)(tb + tc) * P.Hkv + hk) * kD + d0);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tl = tg * 4 + i;
          const uint32_t w[4] = {gw4[i].x, gw4[i].y, gw4[i].z, gw4[i].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float g0 = tl < nt ? (f_gate ? gla_gate_logit<__nv_bfloat16>(bf_lo(w[e]), P.fu.gate_normalizer) : bf_lo(w[e])) : 0.f;
            const float g1 = tl < nt ? (f_gate ? gla_gate_logit<__nv_bfloat16>(bf_hi(w[e]), P.fu.gate_normalizer) : bf_hi(w[e])) : 0.f;
            run[2 * e] += g0; run[2 * e + 1] += g1;
            cum[i][2 * e] = run[2 * e]; cum[i][2 * e + 1] = run[2 * e + 1];
          }
        }
        *reinterpret_cast<float4*>(part_s + tg * kD + d0) = make_float4(run[0], run[1], run[2], run[3]);
        *reinterpret_cast<float4*>(part_s + tg * kD + d0 + 4) = make_float4(run[4], run[5], run[6], run[7]);
      }
      // the next chunk's rows on their way into L2 meanwhile (its loads then meet L2, not HBM, latency):
      // one request per 128-byte line
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tn = tb + kC + tg * 4 + i;
        if (tn < run1 && (dg & 7) == 0) {
          const int64_t kv_n = ((int64_t)tn * P.Hkv + hk) * kD + d0;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(P.g + kv_n));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(P.k + kv_n));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(P.v + kv_n));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(P.q + ((int64_t)tn * P.H + h) * kD + d0));
        }
      }
      workers_bar();
      if (tid < kD) {   // one thread per key dim: exclusive prefix over the 32 token groups
        float acc = 0.f;
#pragma unroll 8
        for (int t2 = 0; t2 < kC / 4; ++t2) {
          const float x = part_s[t2 * kD + tid];
          part_s[t2 * kD + tid] = acc;
          acc += x;
        }
        egc[tid] = fast_exp2(acc * kLog2e);
        g_piece += acc;
        if (!(acc >= -kMaxDecay && acc <= 0.f)) flags[2] = 1;   // too strong a decay (or not a decay, or NaN)
      }
      workers_bar();
      const bool stop = flags[2] != 0;
      float base[8];
      {
        const float4 b0 = *reinterpret_cast<const float4*>(part_s + tg * kD + d0);
        const float4 b1 = *reinterpret_cast<const float4*>(part_s + tg * kD + d0 + 4);
        base[0] = b0.x; base[1] = b0.y; base[2] = b0.z; base[3] = b0.w;
        base[4] = b1.x; base[5] = b1.y; base[6] = b1.z; base[7] = b1.w;
      }
      workers_bar();   // the scratch is read; V may land on it (and flags[2] is read by everyone)
      if (stop) break;
#pragma unroll
      for (int i2 = 0; i2 < 4; i2 += 2) {
      // (two tokens' loads are issued together: two trips to L2 per chunk instead of four)
      uint4 qw2[2], kw2[2], vw2[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int tl = tg * 4 + i2 + u;
        const int tc = tl < nt ? tl : 0;
        const int64_t kv_off = ((int64_t)(tb + tc) * P.Hkv + hk) * kD + d0;
        if (!LOCAL) qw2[u] = *reinterpret_cast<const uint4*>(P.q + ((int64_t)(tb + tc) * P.H + h) * kD + d0);
        else qw2[u] = make_uint4(0, 0, 0, 0);
        kw2[u] = *reinterpret_cast<const uint4*>(P.k + kv_off);
        vw2[u] = *reinterpret_cast<const uint4*>(P.v + kv_off);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = i2 + u;
        const int tl = tg * 4 + i;
        uint4 qw = qw2[u], kw = kw2[u], vw = vw2[u];
        if (tl >= nt) qw = kw = vw = make_uint4(0, 0, 0, 0);
        const uint32_t qx[4] = {qw.x, qw.y, qw.z, qw.w}, kx[4] = {kw.x, kw.y, kw.z, kw.w};
        uint32_t qh[4], ql[4], kh[4], kl[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float G0 = (base[2 * e] + cum[i][2 * e]) * kLog2e, G1 = (base[2 * e + 1] + cum[i][2 * e + 1]) * kLog2e;
          float q0 = bf_lo(qx[e]), q1 = bf_hi(qx[e]), k0 = bf_lo(kx[e]), k1 = bf_hi(kx[e]);
          if (f_relu) { q0 = fmaxf(q0, 0.f); q1 = fmaxf(q1, 0.f); k0 = fmaxf(k0, 0.f); k1 = fmaxf(k1, 0.f); }
          if (!LOCAL) split_bf16x2(q0 * P.scale * fast_exp2(G0), q1 * P.scale * fast_exp2(G1), qh[e], ql[e]);
          split_bf16x2(k0 * fast_exp2(-G0), k1 * fast_exp2(-G1), kh[e], kl[e]);
        }
        const uint32_t o = p_off + swz(tl, dg & 7);
        if (!LOCAL) {
          *reinterpret_cast<uint4*>(smem + kQH + o) = make_uint4(qh[0], qh[1], qh[2], qh[3]);
          *reinterpret_cast<uint4*>(smem + kQL + o) = make_uint4(ql[0], ql[1], ql[2], ql[3]);
        }
        *reinterpret_cast<uint4*>(smem + kKH + o) = make_uint4(kh[0], kh[1], kh[2], kh[3]);
        *reinterpret_cast<uint4*>(smem + kKL + o) = make_uint4(kl[0], kl[1], kl[2], kl[3]);
        *reinterpret_cast<uint4*>(smem + kV + o) = vw;
      }
      }
      fence_proxy_async_smem();   // these generic writes (and the state operands) precede the MMAs' reads
      tc_fence_before();
      mbar_arrive(bar_prep);

      // ============ A: keep s <= t, split, back into tensor memory ============
      if (!LOCAL) {
      ok = mbar_wait_bounded(bar_a, ph);
      if (!ok || flags[0]) break;
      tc_fence_after();
      {
        uint32_t ar[32];
        tmem_ld32_issue(t_lane + kACol + part * 32, ar);
        tmem_ld_fence(ar);
        row_bar(warp & 3);   // every thread of the row holds its scores: the packed halves may overwrite them
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int col = part * 32 + 2 * e;
          const float a0 = col <= r ? __uint_as_float(ar[2 * e]) : 0.f;
          const float a1 = col + 1 <= r ? __uint_as_float(ar[2 * e + 1]) : 0.f;
          split_bf16x2(a0, a1, hi[e], lo[e]);
        }
        tmem_st16(t_lane + kACol + part * 16, hi);
        tmem_st16(t_lane + kACol + 64 + part * 16, lo);
        tmem_st_wait();
      }
      tc_fence_before();
      mbar_arrive(bar_p);
      }

      // ============ state: S_out = diag(exp G_C) (S_in + Ks^T V) ============
      ok = mbar_wait_bounded(bar_s, ph);
      if (!ok || flags[0]) break;
      tc_fence_after();
      {
        uint32_t sr[32];
        tmem_ld32_issue(t_lane + kSCol + part * 32, sr);
        const float e = egc[r];
        tmem_ld_fence(sr);
#pragma unroll
        for (int i = 0; i < 32; ++i) sr[i] = __float_as_uint(__uint_as_float(sr[i]) * e);
        tmem_st32(t_lane + kSCol + part * 32, sr);
        store_state_split(sr);
        if (c + 1 == c_hi) {   // end of this CTA's piece: the run's slot, or the workspace (local pass)
          if (LOCAL) store_state_global(sr, P.tiles + ws_idx * (int64_t)kD * kD);
          else if (is_last) store_state_global(sr, tile);
        }
        tmem_st_wait();
      }

      // ============ outputs of the chunk ============
      if (LOCAL) continue;
      ok = mbar_wait_bounded(bar_o, ph);
      if (!ok || flags[0]) break;
      tc_fence_after();
      {
        uint32_t orr[32];
        tmem_ld32_issue(t_lane + kOCol + part * 32, orr);
        tmem_ld_fence(orr);
        float rs = 1.f;
        if (f_norm) {   // the layer's per-head RMS norm on the fp32 read-out
          float sq = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) sq = fmaf(__uint_as_float(orr[i]), __uint_as_float(orr[i]), sq);
          xch[part * kD + r] = sq;
          row_bar(warp & 3);
          const float tot = xch[r] + xch[kD + r] + xch[2 * kD + r] + xch[3 * kD + r];
          rs = rsqrtf(tot / kD + P.fu.norm_eps);
          const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(P.fu.norm_weight) + part * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            orr[i] = __float_as_uint(__uint_as_float(orr[i]) * rs * __bfloat162float(w[i]));
        }
        // A thread holds 64 (or 128) bytes of a token's row, and the 32 lanes of a warp hold 32 different
        // rows: stored from here they would be 32 separate sectors per instruction, and the loads of the
        // next chunk would queue behind them. The rows are put together in shared memory (in the
        // operands' bytes, free now: every MMA of the chunk is done; rows 16 bytes apart from a multiple
        // of 128, so the lanes do not collide) and leave as one bulk copy per row.
        const int row_bytes = P.out_f32 ? kD * 4 : kD * 2;
        uint8_t* const srow = smem + kStageOff + r * (row_bytes + 16);
        if (P.out_f32) {
          float4* op = reinterpret_cast<float4*>(srow + part * 128);
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4)
            op[c4] = make_float4(__uint_as_float(orr[4 * c4]), __uint_as_float(orr[4 * c4 + 1]),
                                 __uint_as_float(orr[4 * c4 + 2]), __uint_as_float(orr[4 * c4 + 3]));
        } else {
          uint4* op = reinterpret_cast<uint4*>(srow + part * 64);
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            uint4 w4;
            w4.x = pack_bf16x2(__uint_as_float(orr[8 * c4]), __uint_as_float(orr[8 * c4 + 1]));
            w4.y = pack_bf16x2(__uint_as_float(orr[8 * c4 + 2]), __uint_as_float(orr[8 * c4 + 3]));
            w4.z = pack_bf16x2(__uint_as_float(orr[8 * c4 + 4]), __uint_as_float(orr[8 * c4 + 5]));
            w4.w = pack_bf16x2(__uint_as_float(orr[8 * c4 + 6]), __uint_as_float(orr[8 * c4 + 7]));
            op[c4] = w4;
          }
        }
        fence_proxy_async_smem();
        workers_bar();
        if (part == 0 && r < nt) {
          uint8_t* dst = reinterpret_cast<uint8_t*>(P.out) + (((int64_t)(tb + r) * P.H + h) * kD) * (P.out_f32 ? 4 : 2);
          bulk_s2g(dst, smem_u32(srow), (uint32_t)row_bytes);
          bulk_commit();
        }
      }
      // (the next chunk's first barrier orders the reads of the exchange buffer before its scratch
      // writes; the copies out of the staging rows are waited for at the top of the loop)
    }
    bulk_wait_all<0>();   // the last rows have left shared memory and are written
    if (!ok) {
      if (lane == 0 && !flags[0]) { raise_status(P.status, SBK_ST_WAIT_TIMEOUT); flags[0] = 1; }
      if (tid == 0 && is_last && !LOCAL) *my_resume = run1;   // the status word says the result is void; nobody resumes it
    } else if (c < c_hi) {
      // Stopped ahead of chunk c; the MMA warp is let out of its wait.
      if (LOCAL) {
        // a piece of the run cannot be taken: the full pass leaves the whole run to the other kernel
        if (tid == 0) atomicExch(my_bail, 1);
      } else if (is_last) {
        // Hand the rest of the run over. The state as of chunk c's first token goes back to the slot
        // (nothing to store if the run has not been touched at all: the other kernel then starts from
        // the slot, or from zero, by itself).
        if (c > c_lo || sub > 0) {
          uint32_t sr[32];
          tmem_ld32_issue(t_lane + kSCol + part * 32, sr);
          tmem_ld_fence(sr);
          store_state_global(sr, tile);
        }
        if (tid == 0) *my_resume = run0 + c * kC;
      } else if (tid == 0) {
        // an inner piece the local pass went through without complaint: cannot happen (same gates,
        // same arithmetic); if it does, the run's result is void and the status word says so
        raise_status(P.status, SBK_ST_WAIT_TIMEOUT);
      }
      if (tid == 0) flags[1] = 1;
      __threadfence_block();
      mbar_arrive(bar_prep);
    } else if (LOCAL) {
      if (tid < kD) P.decays[ws_idx * kD + tid] = expf(g_piece);
    } else if (tid == 0 && is_last) {
      *my_resume = run1;
    }
  }

  // ---- teardown: everyone meets here, then the allocating warp returns the TMEM columns ----
  if (flags[0]) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);   // let MMAs in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kWorkers / 32) tmem_dealloc(tmem, kTmemCols);
}

template <int F, bool LOCAL>
static cudaError_t opt_in() {
  return cudaFuncSetAttribute(gla_scan_tc_kernel<F, LOCAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
}

int launch(const Params& P, int n_seqs, bool local, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = opt_in<0, false>();
    if (e == cudaSuccess) e = opt_in<7, false>();
    if (e == cudaSuccess) e = opt_in<-1, false>();
    if (e == cudaSuccess) e = opt_in<0, true>();
    if (e == cudaSuccess) e = opt_in<7, true>();
    if (e == cudaSuccess) e = opt_in<-1, true>();
    if (e != cudaSuccess) {
      set_error("sbk_gla_scan: cannot opt in to %d bytes of shared memory: %s", kSmemBytes, cudaGetErrorString(e));
      return SBK_E_LAUNCH;
    }
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid(P.H, n_seqs * P.n_sub);
  const int mix = (P.fu.relu_qk ? 1 : 0) | (P.fu.gate_logits ? 2 : 0) | (P.fu.norm_weight != nullptr ? 4 : 0);
#define SBK_TC_LAUNCH(FF)                                                                        \
  do {                                                                                           \
    if (local) gla_scan_tc_kernel<FF, true><<<grid, kThreads, kSmemBytes, stream>>>(P);          \
    else gla_scan_tc_kernel<FF, false><<<grid, kThreads, kSmemBytes, stream>>>(P);               \
  } while (0)
  if (mix == 0) SBK_TC_LAUNCH(0);
  else if (mix == 7) SBK_TC_LAUNCH(7);
  else SBK_TC_LAUNCH(-1);
#undef SBK_TC_LAUNCH
  return check_launch("sbk_gla_scan");
}

}  // namespace gla_tc
}  // namespace sbk
