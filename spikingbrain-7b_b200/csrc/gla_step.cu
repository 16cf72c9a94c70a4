// Fused GLA recurrent-state step: one pass over the fp32 state tile of a
// (sequence, head) pair updates it in place and reads the output out of the
// NEW state, in the order of vllm_hymeta/model_for_7B/my_fused_recurrent.py:60-80:
//   S[k,v] <- exp(g[k]) * S[k,v] + k[k] * v[v];   o[v] = sum_k (q[k]*scale) * S[k,v]
// Every v column is independent, so a thread owns four v columns (one float4)
// and strides over k rows; the tile is read and written exactly once with
// 128-bit streaming accesses. HBM-bound: 2*D*D*4 bytes per (sequence, head).
#include <math.h>

#include "sbk_common.cuh"

namespace sbk {

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// The element-wise neighbours of the step in the reference model can ride along (GlaFusion,
// sbk_common.cuh): ReLU on q and k, g = logsigmoid(gate logits) / normalizer, and the per-head
// RMS norm of the output (vllm_hymeta/model_for_7B/gla_attention.py:250-262 and :233).
//
// D = 128: 32 threads span a row (float4 each), 8 row groups, 16 rows per thread.
// D = 64 : 16 threads span a row, 16 row groups, 4 rows per thread.
//
// Head-sharded use (PEER): the output row of a (sequence, head) pair goes into a gathered
// buffer [tokens, all heads, D] (row stride given) and, with the same values, into the same
// place of every peer GPU's buffer; the CTA that finishes last raises this rank's flag on the
// peers (the protocol of sbk_swa_decode_gather).
struct GlaPeer {
  void* out[kPeerTableSize];        // peer p's address of this rank's (sequence 0, head 0) element
  int32_t* flag[kPeerTableSize];    // this rank's slot in peer p's flag array
  int n; int32_t value; const int32_t* base;
  int32_t* counter;                 // one zeroed word: CTAs that are through
  int64_t out_seq_stride;           // elements between the rows of consecutive sequences
};

__device__ __forceinline__ void gla_peer_tail(const GlaPeer& pp) {
  // peer stores -> the CTA's barrier -> ONE thread's fence at GPU scope (cumulative: it covers what
  // the barrier ordered before it) -> one count. The count is a release towards the CTA that counts
  // last; that CTA's fence at system scope and its release store of the flag carry every CTA's rows
  // on to the peer that acquires the flag. A system fence in every thread waits out each thread's
  // 64 KB of state stores and doubled the kernel's time; one per CTA still cost 15 %.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();   // release at GPU scope towards the CTA that counts last; its system fence carries it on
    const int total = (int)(gridDim.x * gridDim.y);
    const int f = atomicAdd(pp.counter, 1);
    if (f == total - 1) {
      __threadfence_system();
      *pp.counter = 0;
      const int32_t value = pp.value + (pp.base ? __ldcg(pp.base) : 0);
#pragma unroll
      for (int p = 0; p < kPeerTableSize; ++p)
        if (p < pp.n) asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(pp.flag[p]), "r"(value) : "memory");
    }
  }
}

template <typename T, typename TO, int D, bool FUSED, bool PEER>
__global__ void __launch_bounds__(256)
gla_step_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                const T* __restrict__ g, float* __restrict__ state, int64_t num_slots,
                const int64_t* __restrict__ slot_idx, int H, int Hkv, float scale,
                TO* __restrict__ out, int32_t* status, const GlaFusion fu, const GlaPeer pp) {
  constexpr int TPR = D / 4;          // threads per state row
  constexpr int GROUPS = 256 / TPR;   // row groups
  constexpr int RPT = D / GROUPS;     // rows per thread
  const int h = blockIdx.x;
  const int b = blockIdx.y;
  const int64_t slot = slot_idx ? slot_idx[b] : (int64_t)b;
  if (slot < 0) {          // padded sequence: state row untouched, output row not written
    if constexpr (PEER) gla_peer_tail(pp);
    return;
  }
  if (slot >= num_slots) {
    if (threadIdx.x == 0) raise_status(status, SBK_ST_BAD_SLOT);
    if constexpr (PEER) gla_peer_tail(pp);
    return;
  }
  const int hk = h / (H / Hkv);

  __shared__ float s_q[D], s_k[D], s_decay[D];
  __shared__ float4 s_o[GROUPS][TPR];

  const int tid = threadIdx.x;
  if (tid < D) {
    float qv = to_f32(q[((int64_t)b * H + h) * D + tid]);
    const int64_t kv_off = ((int64_t)b * Hkv + hk) * D + tid;
    float kv = to_f32(k[kv_off]);
    if (FUSED && fu.relu_qk) { qv = fmaxf(qv, 0.f); kv = fmaxf(kv, 0.f); }
    s_q[tid] = qv * scale;
    s_k[tid] = kv;
    s_decay[tid] = expf(FUSED ? gla_gate<T>(to_f32(g[kv_off]), fu) : to_f32(g[kv_off]));
  }
  const int c4 = tid % TPR;
  const int r0 = tid / TPR;
  float4 vv;
  {
    const T* vp = v + ((int64_t)b * Hkv + hk) * D + c4 * 4;
    vv = make_float4(to_f32(vp[0]), to_f32(vp[1]), to_f32(vp[2]), to_f32(vp[3]));
  }
  float4* tile = reinterpret_cast<float4*>(state + ((slot * H + h) * (int64_t)D) * D);

  float4 s[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) s[i] = ld_stream_f4(tile + (int64_t)(r0 + i * GROUPS) * TPR + c4);
  __syncthreads();

  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = r0 + i * GROUPS;
    const float d = s_decay[r], kk = s_k[r], qq = s_q[r];
    float4 n;
    n.x = fmaf(d, s[i].x, kk * vv.x);
    n.y = fmaf(d, s[i].y, kk * vv.y);
    n.z = fmaf(d, s[i].z, kk * vv.z);
    n.w = fmaf(d, s[i].w, kk * vv.w);
    st_stream_f4(tile + (int64_t)r * TPR + c4, n);
    o.x = fmaf(qq, n.x, o.x);
    o.y = fmaf(qq, n.y, o.y);
    o.z = fmaf(qq, n.z, o.z);
    o.w = fmaf(qq, n.w, o.w);
  }
  s_o[r0][c4] = o;
  __syncthreads();
  float acc = 0.f;
  if (tid < D) {
    const float* so = reinterpret_cast<const float*>(&s_o[0][0]);
#pragma unroll
    for (int gi = 0; gi < GROUPS; ++gi) acc += so[gi * D + tid];
  }
  if (FUSED && fu.norm_weight != nullptr) {
    // per-head RMS norm of the D outputs (they sit in threads 0..D-1)
    float sq = tid < D ? acc * acc : 0.f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
    __syncthreads();               // everyone is done reading s_q
    if ((tid & 31) == 0) s_q[tid >> 5] = sq;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < D / 32; ++w) tot += s_q[w];
    if (tid < D) acc = acc * rsqrtf(tot / D + fu.norm_eps) * to_f32(reinterpret_cast<const T*>(fu.norm_weight)[tid]);
  }
  if constexpr (PEER) {
    if (tid < D) {
      const TO o = from_f32<TO>(acc);
      const int64_t at = (int64_t)b * pp.out_seq_stride + (int64_t)h * D + tid;
      out[at] = o;
#pragma unroll
      for (int p = 0; p < kPeerTableSize; ++p)
        if (p < pp.n) reinterpret_cast<TO*>(pp.out[p])[at] = o;
    }
    gla_peer_tail(pp);
  } else {
    if (tid < D) out[((int64_t)b * H + h) * D + tid] = from_f32<TO>(acc);
  }
}

}  // namespace sbk

namespace sbk {
static int gla_step_impl(const void* q, const void* k, const void* v, const void* g,
                         int in_dtype, float* state, int64_t num_slots,
                         const int64_t* slot_idx, int B, int H, int Hkv, int D, float scale,
                         void* out, int out_dtype, int fuse_flags, float gate_normalizer,
                         const void* norm_weight, float norm_eps, int32_t* status, void* stream,
                         const GlaPeer* peer) {
  GlaFusion fu;
  if (!make_gla_fusion(&fu, "sbk_gla_step", fuse_flags, gate_normalizer, norm_weight, norm_eps)) return SBK_E_ARG;
  if (B < 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || num_slots < 0) {
    set_error("sbk_gla_step: bad head counts H=%d Hkv=%d or negative size", H, Hkv);
    return SBK_E_ARG;
  }
  if (D != 64 && D != 128) {
    set_error("sbk_gla_step: D=%d unsupported (64 or 128)", D);
    return SBK_E_ARG;
  }
  if ((in_dtype != SBK_BF16 && in_dtype != SBK_F32) || (out_dtype != SBK_BF16 && out_dtype != SBK_F32)) {
    set_error("sbk_gla_step: in_dtype=%d / out_dtype=%d unsupported", in_dtype, out_dtype);
    return SBK_E_ARG;
  }
  if (B == 0) return SBK_OK;
  if (!q || !k || !v || !g || !state || !out) {
    set_error("sbk_gla_step: null pointer");
    return SBK_E_ARG;
  }
  if (!aligned16(state)) {
    set_error("sbk_gla_step: state must be 16-byte aligned");
    return SBK_E_ALIGN;
  }
  if (B > 65535) {
    set_error("sbk_gla_step: B=%d exceeds 65535", B);
    return SBK_E_ARG;
  }
  dim3 grid(H, B);
  cudaStream_t st = (cudaStream_t)stream;
  // the plain step keeps its own instantiation: nothing of the fused neighbours is compiled in
  const bool fused = fuse_flags != 0 || norm_weight != nullptr;
  GlaPeer pp = {};
  if (peer) {
    // head-sharded layers hand bf16 in and out; the neighbours ride along or not (one instantiation)
    pp = *peer;
#define SBK_GLA_PEER(DD)                                                                                   \
  gla_step_kernel<__nv_bfloat16, __nv_bfloat16, DD, true, true><<<grid, 256, 0, st>>>(                     \
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)g,  \
      state, num_slots, slot_idx, H, Hkv, scale, (__nv_bfloat16*)out, status, fu, pp)
    if (D == 128) SBK_GLA_PEER(128);
    else SBK_GLA_PEER(64);
#undef SBK_GLA_PEER
    return check_launch("sbk_gla_step_gather");
  }
#define SBK_GLA_LAUNCH_F(T, TO, DD, F)                                                          \
  gla_step_kernel<T, TO, DD, F, false><<<grid, 256, 0, st>>>((const T*)q, (const T*)k, (const T*)v, \
                                                      (const T*)g, state, num_slots, slot_idx,  \
                                                      H, Hkv, scale, (TO*)out, status, fu, pp)
#define SBK_GLA_LAUNCH(T, TO, DD)            \
  do {                                       \
    if (fused) SBK_GLA_LAUNCH_F(T, TO, DD, true); \
    else SBK_GLA_LAUNCH_F(T, TO, DD, false); \
  } while (0)
#define SBK_GLA_DISPATCH_D(T, TO)         \
  do {                                    \
    if (D == 128) SBK_GLA_LAUNCH(T, TO, 128); \
    else SBK_GLA_LAUNCH(T, TO, 64);       \
  } while (0)
  if (in_dtype == SBK_BF16) {
    if (out_dtype == SBK_BF16) SBK_GLA_DISPATCH_D(__nv_bfloat16, __nv_bfloat16);
    else SBK_GLA_DISPATCH_D(__nv_bfloat16, float);
  } else {
    if (out_dtype == SBK_BF16) SBK_GLA_DISPATCH_D(float, __nv_bfloat16);
    else SBK_GLA_DISPATCH_D(float, float);
  }
#undef SBK_GLA_DISPATCH_D
#undef SBK_GLA_LAUNCH
#undef SBK_GLA_LAUNCH_F
  return check_launch("sbk_gla_step");
}
}  // namespace sbk

extern "C" int sbk_gla_step(const void* q, const void* k, const void* v, const void* g,
                            int in_dtype, float* state, int64_t num_slots,
                            const int64_t* slot_idx, int B, int H, int Hkv, int D, float scale,
                            void* out, int out_dtype, int fuse_flags, float gate_normalizer,
                            const void* norm_weight, float norm_eps, int32_t* status, void* stream) {
  return sbk::gla_step_impl(q, k, v, g, in_dtype, state, num_slots, slot_idx, B, H, Hkv, D, scale, out, out_dtype,
                            fuse_flags, gate_normalizer, norm_weight, norm_eps, status, stream, nullptr);
}

extern "C" int sbk_gla_step_gather(const void* q, const void* k, const void* v, const void* g,
                                   float* state, int64_t num_slots, const int64_t* slot_idx, int B, int H,
                                   int Hkv, int D, float scale, void* out, int64_t out_seq_stride,
                                   int fuse_flags, float gate_normalizer, const void* norm_weight,
                                   float norm_eps, int32_t* counter, void* const* peer_out,
                                   int32_t* const* peer_flag, int n_peer, int32_t flag_value,
                                   const int32_t* flag_base, int32_t* status, void* stream) {
  using namespace sbk;
  if (n_peer < 0 || n_peer > kPeerTableSize || (n_peer > 0 && (!peer_out || !peer_flag)) || !counter) {
    set_error("sbk_gla_step_gather: n_peer=%d outside [0,%d], null peer tables or null counter", n_peer,
              kPeerTableSize);
    return SBK_E_ARG;
  }
  if (B > 0 && out_seq_stride < (int64_t)H * D) {
    set_error("sbk_gla_step_gather: row stride %lld smaller than this rank's %d heads", (long long)out_seq_stride, H);
    return SBK_E_ARG;
  }
  GlaPeer pp = {};
  for (int p = 0; p < n_peer; ++p) {
    if (!peer_out[p] || !peer_flag[p] || (reinterpret_cast<uintptr_t>(peer_out[p]) & 1u) ||
        (reinterpret_cast<uintptr_t>(peer_flag[p]) & 3u)) {
      set_error("sbk_gla_step_gather: peer %d: null or misaligned buffer / flag address", p);
      return SBK_E_ALIGN;
    }
    pp.out[p] = peer_out[p];
    pp.flag[p] = peer_flag[p];
  }
  pp.n = n_peer; pp.value = flag_value; pp.base = flag_base; pp.counter = counter;
  pp.out_seq_stride = out_seq_stride;
  if (B == 0) return sbk_peer_signal(peer_flag, n_peer, flag_value, flag_base, stream);
  return gla_step_impl(q, k, v, g, SBK_BF16, state, num_slots, slot_idx, B, H, Hkv, D, scale, out, SBK_BF16,
                       fuse_flags, gate_normalizer, norm_weight, norm_eps, status, stream, &pp);
}
