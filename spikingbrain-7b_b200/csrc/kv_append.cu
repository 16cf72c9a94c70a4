// Paged-KV append with sliding-window block retirement, and the block-table
// gather that materialises a window as dense tensors. Both are pure byte
// movers: results are bit-exact copies of their inputs whatever the element type.
#include "sbk_common.cuh"

namespace sbk {

// One CTA of 128 threads per token: threads 0-63 move the K row, 64-127 the V
// row, 16 bytes each per trip. CTAs past the last token retire blocks, one
// thread per sequence.
__global__ void __launch_bounds__(128)
kv_append_kernel(const uint8_t* __restrict__ key, const uint8_t* __restrict__ value,
                 uint8_t* __restrict__ k_cache, uint8_t* __restrict__ v_cache,
                 const int64_t* __restrict__ slot_mapping, int T, int row_bytes,
                 int64_t kv_token_stride, int64_t num_slots, int block_size,
                 int64_t cache_block_stride, int32_t* __restrict__ block_tables, int max_blocks,
                 const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ query_start_loc,
                 int B, int window_left, int32_t* __restrict__ retired_out, int max_retired,
                 int32_t* status) {
  const int bid = blockIdx.x;
  if (bid < T) {
    const int64_t slot = slot_mapping[bid];
    if (slot < 0) return;  // padding token
    if (slot >= num_slots) {
      if (threadIdx.x == 0) raise_status(status, SBK_ST_BAD_SLOT);
      return;
    }
    const int64_t blk = slot / block_size;
    const int64_t off = slot - blk * block_size;
    const bool is_v = threadIdx.x >= 64;
    const uint8_t* src = (is_v ? value : key) + (int64_t)bid * kv_token_stride;
    uint8_t* dst = (is_v ? v_cache : k_cache) + blk * cache_block_stride + off * row_bytes;
    for (int o = (threadIdx.x & 63) * 16; o < row_bytes; o += 64 * 16) {
      *reinterpret_cast<uint4*>(dst + o) = *reinterpret_cast<const uint4*>(src + o);
    }
    return;
  }
  // ---- retirement: blocks wholly before the first token still visible ----
  retire_rows((bid - T) * 128 + threadIdx.x, block_tables, max_blocks, seq_lens, query_start_loc, B,
              window_left, block_size, retired_out, max_retired, status);
}

// Dense gather of the visible window: out[b, h, i, :] = cache[token t0+i, head h].
// One thread moves 16 bytes; consecutive threads walk d, then tokens, then heads.
__global__ void __launch_bounds__(256)
kv_gather_kernel(const uint8_t* __restrict__ k_cache, const uint8_t* __restrict__ v_cache,
                 const int32_t* __restrict__ block_tables, int max_blocks,
                 const int32_t* __restrict__ seq_lens, int kvh, int head_bytes,
                 int64_t num_blocks, int block_size, int64_t cache_block_stride, int window_left,
                 uint8_t* __restrict__ k_out, uint8_t* __restrict__ v_out, int n_out,
                 int32_t* status) {
  const int b = blockIdx.y;
  const int L = seq_lens[b];
  const int t0 = first_visible(L, 1, window_left);
  const int n_vis = L - t0;
  const int vec_per_head = head_bytes / 16;
  const int64_t per_seq = (int64_t)kvh * n_out * vec_per_head;
  const int32_t* row = block_tables + (int64_t)b * max_blocks;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < per_seq;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int dv = (int)(idx % vec_per_head);
    const int64_t r = idx / vec_per_head;
    const int i = (int)(r % n_out);
    const int h = (int)(r / n_out);
    uint4 kx = make_uint4(0, 0, 0, 0), vx = kx;
    if (i < n_vis) {
      const int t = t0 + i;
      const int lb = t / block_size;
      const int32_t pb = lb < max_blocks ? row[lb] : -1;
      if (pb < 0 || pb >= num_blocks) {
        raise_status(status, SBK_ST_BAD_BLOCK);
      } else {
        const int64_t off = (int64_t)pb * cache_block_stride +
                            ((int64_t)(t - lb * block_size) * kvh + h) * head_bytes + dv * 16;
        kx = *reinterpret_cast<const uint4*>(k_cache + off);
        vx = *reinterpret_cast<const uint4*>(v_cache + off);
      }
    }
    const int64_t o = ((int64_t)b * per_seq + idx) * 16;
    *reinterpret_cast<uint4*>(k_out + o) = kx;
    *reinterpret_cast<uint4*>(v_out + o) = vx;
  }
}

}  // namespace sbk

extern "C" int sbk_kv_append(const void* key, const void* value, void* k_cache, void* v_cache,
                             const int64_t* slot_mapping, int T, int kvh, int D, int elem_bytes,
                             int64_t kv_token_stride_bytes, int64_t num_blocks, int block_size,
                             int64_t cache_block_stride_bytes, int32_t* block_tables,
                             int max_blocks, const int32_t* seq_lens,
                             const int32_t* query_start_loc, int B, int window_left,
                             int32_t* retired_out, int max_retired, int32_t* status,
                             void* stream) {
  using namespace sbk;
  if (T < 0 || B < 0 || kvh <= 0 || D <= 0 || elem_bytes <= 0 || block_size <= 0 || num_blocks < 0) {
    set_error("sbk_kv_append: negative or zero dimension");
    return SBK_E_ARG;
  }
  const int64_t row_bytes = (int64_t)kvh * D * elem_bytes;
  if (T > 0) {
    if (!key || !value || !k_cache || !v_cache || !slot_mapping) {
      set_error("sbk_kv_append: null pointer with T=%d", T);
      return SBK_E_ARG;
    }
    if (row_bytes % 16 || kv_token_stride_bytes % 16 || cache_block_stride_bytes % 16 ||
        !aligned16(key) || !aligned16(value) || !aligned16(k_cache) || !aligned16(v_cache)) {
      set_error("sbk_kv_append: rows, strides and base pointers must be multiples of 16 bytes");
      return SBK_E_ALIGN;
    }
    if (kv_token_stride_bytes < row_bytes || cache_block_stride_bytes < row_bytes * block_size) {
      set_error("sbk_kv_append: stride smaller than the row it spans");
      return SBK_E_ARG;
    }
  }
  const bool retire = block_tables != nullptr && B > 0;
  if (retire && (!seq_lens || max_blocks <= 0 || (retired_out && max_retired <= 0))) {
    set_error("sbk_kv_append: retirement needs seq_lens, max_blocks>0 and max_retired>0");
    return SBK_E_ARG;
  }
  const int grid = T + (retire ? (B + 127) / 128 : 0);
  if (grid == 0) return SBK_OK;
  kv_append_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)key, (const uint8_t*)value, (uint8_t*)k_cache, (uint8_t*)v_cache, slot_mapping,
      T, (int)row_bytes, kv_token_stride_bytes, num_blocks * block_size, block_size,
      cache_block_stride_bytes, retire ? block_tables : nullptr, max_blocks, seq_lens,
      query_start_loc, B, window_left, retired_out, max_retired, status);
  return check_launch("sbk_kv_append");
}

extern "C" int sbk_kv_gather(const void* k_cache, const void* v_cache, const int32_t* block_tables,
                             int max_blocks, const int32_t* seq_lens, int B, int kvh, int D,
                             int elem_bytes, int64_t num_blocks, int block_size,
                             int64_t cache_block_stride_bytes, int window_left, void* k_out,
                             void* v_out, int n_out, int32_t* status, void* stream) {
  using namespace sbk;
  if (B < 0 || n_out < 0 || kvh <= 0 || D <= 0 || elem_bytes <= 0 || block_size <= 0 ||
      max_blocks <= 0) {
    set_error("sbk_kv_gather: negative or zero dimension");
    return SBK_E_ARG;
  }
  if (B == 0 || n_out == 0) return SBK_OK;
  if (!k_cache || !v_cache || !block_tables || !seq_lens || !k_out || !v_out) {
    set_error("sbk_kv_gather: null pointer");
    return SBK_E_ARG;
  }
  const int64_t head_bytes = (int64_t)D * elem_bytes;
  if (head_bytes % 16 || cache_block_stride_bytes % 16 || !aligned16(k_cache) ||
      !aligned16(v_cache) || !aligned16(k_out) || !aligned16(v_out)) {
    set_error("sbk_kv_gather: head rows, strides and base pointers must be multiples of 16 bytes");
    return SBK_E_ALIGN;
  }
  if (B > 65535) {
    set_error("sbk_kv_gather: B=%d exceeds 65535", B);
    return SBK_E_ARG;
  }
  const int64_t per_seq = (int64_t)kvh * n_out * (head_bytes / 16);
  int gx = (int)((per_seq + 255) / 256);
  if (gx > 1024) gx = 1024;
  dim3 grid(gx, B);
  kv_gather_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)k_cache, (const uint8_t*)v_cache, block_tables, max_blocks, seq_lens, kvh,
      (int)head_bytes, num_blocks, block_size, cache_block_stride_bytes, window_left,
      (uint8_t*)k_out, (uint8_t*)v_out, n_out, status);
  return check_launch("sbk_kv_gather");
}
