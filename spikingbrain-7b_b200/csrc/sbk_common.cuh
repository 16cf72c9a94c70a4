// Shared device helpers for libsbk (sm_100a): PTX wrappers for mbarrier, bulk
// async copies, ldmatrix / movmatrix / mma, and the host-side error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sbk.h"

namespace sbk {

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);
int check_launch(const char* what);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Other ranks of a head-sharded group that one kernel stores to (8 GPUs behind one switch).
constexpr int kPeerTableSize = 7;
struct Int32PtrTable { int32_t* p[kPeerTableSize]; };

// -------------------------------------------------------------- device side
__device__ __forceinline__ void raise_status(int32_t* status, int bit) {
  if (status != nullptr) atomicOr(status, bit);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls and reports false; the caller
// records SBK_ST_WAIT_TIMEOUT and unwinds instead of spinning for ever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  uint32_t limit = (1u << 24)) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// generic-proxy accesses (any state space) before, async-proxy accesses after
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ---- bulk async copies (TMA engine, untiled form) ---------------------------
// global -> shared, completion counted in bytes on an mbarrier. Both addresses
// 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// shared -> global
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- warp-level matrix ops --------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// streaming 128-bit global accesses (the state / cache lines are touched once per step)
__device__ __forceinline__ float4 ld_stream_f4(const float4* p) {
  float4 v;
  asm volatile("ld.global.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream_f4(float4* p, const float4& v) {
  asm volatile("st.global.L1::no_allocate.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

// ---- optional element-wise work fused into the GLA kernels ---------------------------------
struct GlaFusion {
  int relu_qk;              // q <- relu(q), k <- relu(k)            (feature map of the model)
  int gate_logits;          // g <- logsigmoid(g) / gate_normalizer  (g arrives as gate logits)
  float gate_normalizer;
  const void* norm_weight;  // [D] in the input dtype: o <- rms_norm(o) * weight per head, or NULL
  float norm_eps;
};
bool make_gla_fusion(GlaFusion* fu, const char* who, int flags, float gate_normalizer,
                     const void* norm_weight, float norm_eps);

// The log-decay of a key row. With gate logits, logsigmoid is evaluated in fp32 and rounded to
// the input type before the division, which is what the reference's `F.logsigmoid(gk) / 16` on a
// bf16 tensor produces.
template <typename T>
__device__ __forceinline__ float gla_gate_logit(float x, float gate_normalizer) {
  float ls = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
  if (sizeof(T) == 2) ls = __bfloat162float(__float2bfloat16_rn(ls));
  float gq = ls / gate_normalizer;
  if (sizeof(T) == 2) gq = __bfloat162float(__float2bfloat16_rn(gq));
  return gq;
}
template <typename T>
__device__ __forceinline__ float gla_gate(float x, const GlaFusion& fu) {
  return fu.gate_logits ? gla_gate_logit<T>(x, fu.gate_normalizer) : x;
}

// first token a decode query at position seq_len-1 can still see
__device__ __host__ __forceinline__ int first_visible(int seq_len, int n_new, int window_left) {
  if (window_left < 0) return 0;
  int t0 = seq_len - n_new - window_left;
  return t0 > 0 ? t0 : 0;
}

// Window retirement of one sequence's block-table row (thread b of the retirement CTAs of the
// append kernels): entries of blocks wholly before the first visible token become -1 and their
// ids are listed in retired_out[b, :].
__device__ __forceinline__ void retire_rows(int b, int32_t* __restrict__ block_tables, int max_blocks,
                                            const int32_t* __restrict__ seq_lens,
                                            const int32_t* __restrict__ query_start_loc, int B,
                                            int window_left, int block_size,
                                            int32_t* __restrict__ retired_out, int max_retired,
                                            int32_t* status) {
  if (block_tables == nullptr || b >= B) return;
  const int L = seq_lens[b];
  int n_new = query_start_loc ? (query_start_loc[b + 1] - query_start_loc[b]) : 1;
  if (n_new < 1) n_new = 1;  // a row without a query this step keeps what its last query saw
  const int t0 = first_visible(L, n_new, window_left);
  int first_live = t0 / block_size;
  if (first_live > max_blocks) first_live = max_blocks;
  int32_t* row = block_tables + (int64_t)b * max_blocks;
  int32_t* rout = retired_out ? retired_out + (int64_t)b * max_retired : nullptr;
  int cnt = 0;
  // Blocks retired by earlier calls are already -1, so walk back from the window edge until
  // the first entry that is already retired.
  int j = first_live - 1;
  while (j >= 0 && row[j] >= 0) --j;
  for (int i = j + 1; i < first_live; ++i) {
    const int32_t id = row[i];
    row[i] = -1;
    if (rout) {
      if (cnt < max_retired) rout[cnt] = id;
      else raise_status(status, SBK_ST_RETIRE_OVERFLOW);
    }
    ++cnt;
  }
  if (rout)
    for (int i = cnt; i < max_retired; ++i) rout[i] = -1;
}

}  // namespace sbk
