// Rotary position embedding fused into the paged-KV append: one launch rotates the new tokens'
// query rows in place, rotates their key rows on the way into the cache (and, on request, in
// place too), copies the value rows, and retires the blocks that left the window. It stands in
// for the reference's rotary call followed by its cache write
// (vllm_hymeta/model_for_7B/modeling_gla_swa.py:79-93 and :215, then
// vllm_hymeta/attention/meta_attention.py:790-799; on the HF side
// hf_7B_model/window_attention.py:161-162 followed by Cache.update).
//
// The rotation is the NeoX (rotate-half) form: with h = rot_dim / 2 and i < h,
//     out[i]     = x[i]     * cos[i] - x[i + h] * sin[i]
//     out[i + h] = x[i + h] * cos[i] + x[i]     * sin[i]
// and every product and the final sum is rounded to the element type separately, which is what
// the reference's tensor expression (q * cos) + (rotate_half(q) * sin) yields on bf16 (or fp32)
// tensors. cos / sin come from a [max_position, rot_dim] table (cos half, then sin half).
#include "sbk_common.cuh"

namespace sbk {

// ---- 16-byte vectors of the element type ----
template <typename T>
struct RopeVec;

template <>
struct RopeVec<__nv_bfloat16> {
  static constexpr int kElems = 8;
  __device__ static void rotate(const uint4& lo, const uint4& hi, const uint4& c, const uint4& s,
                                uint4& olo, uint4& ohi) {
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(&lo);
    const __nv_bfloat16* y = reinterpret_cast<const __nv_bfloat16*>(&hi);
    const __nv_bfloat16* cc = reinterpret_cast<const __nv_bfloat16*>(&c);
    const __nv_bfloat16* ss = reinterpret_cast<const __nv_bfloat16*>(&s);
    __nv_bfloat16* ol = reinterpret_cast<__nv_bfloat16*>(&olo);
    __nv_bfloat16* oh = reinterpret_cast<__nv_bfloat16*>(&ohi);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float xf = __bfloat162float(x[i]), yf = __bfloat162float(y[i]);
      const float cf = __bfloat162float(cc[i]), sf = __bfloat162float(ss[i]);
      // a product of two bf16 values is exact in fp32, so each line rounds once, to bf16
      const float xc = __bfloat162float(__float2bfloat16_rn(xf * cf));
      const float ys = __bfloat162float(__float2bfloat16_rn(yf * sf));
      const float yc = __bfloat162float(__float2bfloat16_rn(yf * cf));
      const float xs = __bfloat162float(__float2bfloat16_rn(xf * sf));
      ol[i] = __float2bfloat16_rn(__fsub_rn(xc, ys));
      oh[i] = __float2bfloat16_rn(__fadd_rn(yc, xs));
    }
  }
};

template <>
struct RopeVec<float> {
  static constexpr int kElems = 4;
  __device__ static void rotate(const uint4& lo, const uint4& hi, const uint4& c, const uint4& s,
                                uint4& olo, uint4& ohi) {
    const float* x = reinterpret_cast<const float*>(&lo);
    const float* y = reinterpret_cast<const float*>(&hi);
    const float* cc = reinterpret_cast<const float*>(&c);
    const float* ss = reinterpret_cast<const float*>(&s);
    float* ol = reinterpret_cast<float*>(&olo);
    float* oh = reinterpret_cast<float*>(&ohi);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // no fused multiply-add: the reference rounds each product
      ol[i] = __fsub_rn(__fmul_rn(x[i], cc[i]), __fmul_rn(y[i], ss[i]));
      oh[i] = __fadd_rn(__fmul_rn(y[i], cc[i]), __fmul_rn(x[i], ss[i]));
    }
  }
};

struct RopeParams {
  uint8_t* query;            // [T, H, D] rotated in place, or NULL
  int H;
  int64_t q_token_stride;    // bytes
  uint8_t* key;              // [T, kvh, D]
  const uint8_t* value;
  int64_t kv_token_stride;   // bytes
  int key_in_place;
  uint8_t* k_cache;
  uint8_t* v_cache;
  const int64_t* slot_mapping;
  const int64_t* positions;
  const uint8_t* cos_sin;    // [max_position, rot_dim]
  int64_t max_position;
  int rot_dim;
  int T, kvh, D;
  int64_t num_slots;
  int block_size;
  int64_t cache_block_stride;
  int32_t* block_tables;
  int max_blocks;
  const int32_t* seq_lens;
  const int32_t* query_start_loc;
  int B, window_left;
  int32_t* retired_out;
  int max_retired;
  int32_t* status;
};

// One CTA of 128 threads per token; a thread's unit of work is a pair of 16-byte vectors (the
// two halves of a rotation) or one 16-byte vector of a plain copy. CTAs past the last token
// retire blocks, one thread per sequence.
template <typename T>
__global__ void __launch_bounds__(128) rope_kv_append_kernel(const RopeParams p) {
  constexpr int VE = RopeVec<T>::kElems;
  const int bid = blockIdx.x;
  if (bid >= p.T) {
    retire_rows((bid - p.T) * 128 + threadIdx.x, p.block_tables, p.max_blocks, p.seq_lens,
                p.query_start_loc, p.B, p.window_left, p.block_size, p.retired_out, p.max_retired,
                p.status);
    return;
  }
  const int64_t pos = p.positions[bid];
  if (pos < 0 || pos >= p.max_position) {
    if (threadIdx.x == 0) raise_status(p.status, SBK_ST_BAD_POSITION);
    return;  // nothing of this token is written
  }
  const int64_t slot = p.slot_mapping[bid];
  bool to_cache = slot >= 0;  // a padding token still has its query (and key) rotated
  if (slot >= p.num_slots) {
    if (threadIdx.x == 0) raise_status(p.status, SBK_ST_BAD_SLOT);
    to_cache = false;
  }
  const int half_v = p.rot_dim / 2 / VE;        // vector pairs per head
  const int head_v = p.D / VE;                  // vectors per head
  const int tail_v = head_v - 2 * half_v;       // vectors per head beyond rot_dim (passed through)
  const int n_kp = p.kvh * half_v, n_kt = p.kvh * tail_v, n_v = p.kvh * head_v;
  const int n_qp = p.query ? p.H * half_v : 0;
  const int total = n_kp + n_kt + n_v + n_qp;

  const uint4* cs = reinterpret_cast<const uint4*>(p.cos_sin + pos * p.rot_dim * (int64_t)sizeof(T));
  uint4* krow = reinterpret_cast<uint4*>(p.key + (int64_t)bid * p.kv_token_stride);
  const uint4* vrow = reinterpret_cast<const uint4*>(p.value + (int64_t)bid * p.kv_token_stride);
  uint4 *kdst = nullptr, *vdst = nullptr;
  if (to_cache) {
    const int64_t blk = slot / p.block_size;
    const int64_t off = blk * p.cache_block_stride + (slot - blk * p.block_size) * (int64_t)n_v * 16;
    kdst = reinterpret_cast<uint4*>(p.k_cache + off);
    vdst = reinterpret_cast<uint4*>(p.v_cache + off);
  }
  for (int item = threadIdx.x; item < total; item += 128) {
    if (item < n_kp) {
      const int head = item / half_v, j = item - head * half_v;
      const int ilo = head * head_v + j, ihi = ilo + half_v;
      uint4 olo, ohi;
      RopeVec<T>::rotate(krow[ilo], krow[ihi], cs[j], cs[half_v + j], olo, ohi);
      if (to_cache) {
        kdst[ilo] = olo;
        kdst[ihi] = ohi;
      }
      if (p.key_in_place) {
        krow[ilo] = olo;
        krow[ihi] = ohi;
      }
    } else if (item < n_kp + n_kt) {
      const int r = item - n_kp;
      const int head = r / tail_v, j = r - head * tail_v;
      const int idx = head * head_v + 2 * half_v + j;
      if (to_cache) kdst[idx] = krow[idx];
    } else if (item < n_kp + n_kt + n_v) {
      const int idx = item - n_kp - n_kt;
      if (to_cache) vdst[idx] = vrow[idx];
    } else {
      const int r = item - n_kp - n_kt - n_v;
      const int head = r / half_v, j = r - head * half_v;
      uint4* qrow = reinterpret_cast<uint4*>(p.query + (int64_t)bid * p.q_token_stride);
      const int ilo = head * head_v + j, ihi = ilo + half_v;
      uint4 olo, ohi;
      RopeVec<T>::rotate(qrow[ilo], qrow[ihi], cs[j], cs[half_v + j], olo, ohi);
      qrow[ilo] = olo;
      qrow[ihi] = ohi;
    }
  }
}

}  // namespace sbk

extern "C" int sbk_rope_kv_append(void* query, int H, int64_t q_token_stride_bytes, void* key,
                                  const void* value, int key_in_place, void* k_cache, void* v_cache,
                                  const int64_t* slot_mapping, const int64_t* positions,
                                  const void* cos_sin_cache, int rot_dim, int64_t max_position,
                                  int T, int kvh, int D, int dtype, int64_t kv_token_stride_bytes,
                                  int64_t num_blocks, int block_size,
                                  int64_t cache_block_stride_bytes, int32_t* block_tables,
                                  int max_blocks, const int32_t* seq_lens,
                                  const int32_t* query_start_loc, int B, int window_left,
                                  int32_t* retired_out, int max_retired, int32_t* status,
                                  void* stream) {
  using namespace sbk;
  if (T < 0 || B < 0 || kvh <= 0 || D <= 0 || block_size <= 0 || num_blocks < 0 || max_position < 0) {
    set_error("sbk_rope_kv_append: negative or zero dimension");
    return SBK_E_ARG;
  }
  if (dtype != SBK_BF16 && dtype != SBK_F32) {
    set_error("sbk_rope_kv_append: dtype=%d unsupported", dtype);
    return SBK_E_ARG;
  }
  const int es = dtype == SBK_BF16 ? 2 : 4;
  const int ve = 16 / es;
  if (rot_dim <= 0 || rot_dim > D || rot_dim % (2 * ve) != 0 || D % ve != 0) {
    set_error("sbk_rope_kv_append: rot_dim=%d must be in (0, D=%d] and a multiple of %d elements", rot_dim, D,
              2 * ve);
    return SBK_E_ARG;
  }
  if (query && H <= 0) {
    set_error("sbk_rope_kv_append: query given with H=%d", H);
    return SBK_E_ARG;
  }
  const int64_t row_bytes = (int64_t)kvh * D * es;
  if (T > 0) {
    if (!key || !value || !k_cache || !v_cache || !slot_mapping || !positions || !cos_sin_cache) {
      set_error("sbk_rope_kv_append: null pointer with T=%d", T);
      return SBK_E_ARG;
    }
    if (kv_token_stride_bytes % 16 || cache_block_stride_bytes % 16 || !aligned16(key) || !aligned16(value) ||
        !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(cos_sin_cache) ||
        (query && (!aligned16(query) || q_token_stride_bytes % 16))) {
      set_error("sbk_rope_kv_append: strides and base pointers must be multiples of 16 bytes");
      return SBK_E_ALIGN;
    }
    if (kv_token_stride_bytes < row_bytes || cache_block_stride_bytes < row_bytes * block_size ||
        (query && q_token_stride_bytes < (int64_t)H * D * es)) {
      set_error("sbk_rope_kv_append: stride smaller than the row it spans");
      return SBK_E_ARG;
    }
  }
  const bool retire = block_tables != nullptr && B > 0;
  if (retire && (!seq_lens || max_blocks <= 0 || (retired_out && max_retired <= 0))) {
    set_error("sbk_rope_kv_append: retirement needs seq_lens, max_blocks>0 and max_retired>0");
    return SBK_E_ARG;
  }
  const int grid = T + (retire ? (B + 127) / 128 : 0);
  if (grid == 0) return SBK_OK;
  RopeParams p;
  p.query = (uint8_t*)query;
  p.H = H;
  p.q_token_stride = q_token_stride_bytes;
  p.key = (uint8_t*)key;
  p.value = (const uint8_t*)value;
  p.kv_token_stride = kv_token_stride_bytes;
  p.key_in_place = key_in_place;
  p.k_cache = (uint8_t*)k_cache;
  p.v_cache = (uint8_t*)v_cache;
  p.slot_mapping = slot_mapping;
  p.positions = positions;
  p.cos_sin = (const uint8_t*)cos_sin_cache;
  p.max_position = max_position;
  p.rot_dim = rot_dim;
  p.T = T;
  p.kvh = kvh;
  p.D = D;
  p.num_slots = num_blocks * block_size;
  p.block_size = block_size;
  p.cache_block_stride = cache_block_stride_bytes;
  p.block_tables = retire ? block_tables : nullptr;
  p.max_blocks = max_blocks;
  p.seq_lens = seq_lens;
  p.query_start_loc = query_start_loc;
  p.B = B;
  p.window_left = window_left;
  p.retired_out = retired_out;
  p.max_retired = max_retired;
  p.status = status;
  if (dtype == SBK_BF16)
    rope_kv_append_kernel<__nv_bfloat16><<<grid, 128, 0, (cudaStream_t)stream>>>(p);
  else
    rope_kv_append_kernel<float><<<grid, 128, 0, (cudaStream_t)stream>>>(p);
  return check_launch("sbk_rope_kv_append");
}
