// Host side of the tensor maps: encoding through the driver entry point and a small cache.
#include <mutex>

#include "sbk_tma.cuh"

namespace sbk {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

static bool encode_map(CUtensorMap* m, const MapKey& k, bool tile_copy) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t row_bytes = k.tok_stride ? (cuuint64_t)k.tok_stride : (cuuint64_t)k.kvh * 256;
  cuuint64_t dim[4], stride[3];
  cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
  dim[0] = 64; dim[3] = (cuuint64_t)k.num_blocks;
  stride[2] = (cuuint64_t)k.block_stride;
  if (tile_copy) {
    dim[1] = (cuuint64_t)k.block_size; dim[2] = 2 * k.kvh;
    stride[0] = row_bytes; stride[1] = 128;
    box[0] = 64; box[1] = 16; box[2] = (cuuint32_t)k.box_rows; box[3] = 1;
  } else {
    dim[1] = 2 * k.kvh; dim[2] = (cuuint64_t)k.block_size;
    stride[0] = 128; stride[1] = row_bytes;
    box[0] = 64; box[1] = 1; box[2] = 16; box[3] = 1;
  }
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(k.base), dim, stride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int g_copy_mode = -1;
int copy_mode() { return g_copy_mode; }

// A map holds nothing but the address and the dimensions, so a cached one stays valid as long
// as the geometry does. The cache is keyed by the geometry and the form (tile / row copies).
static bool cached_map(CUtensorMap* out, const MapKey& key, bool tile_copy) {
  constexpr int kSlots = 128;
  static MapKey keys[kSlots];
  static bool forms[kSlots];
  static CUtensorMap maps[kSlots];
  static int used = 0, next = 0;
  for (int i = 0; i < used; ++i)
    if (forms[i] == tile_copy && keys[i] == key) { *out = maps[i]; return true; }
  CUtensorMap m;
  if (!encode_map(&m, key, tile_copy)) return false;
  const int slot = used < kSlots ? used++ : (next++ % kSlots);
  keys[slot] = key; forms[slot] = tile_copy; maps[slot] = m;
  *out = m;
  return true;
}

bool get_maps(CUtensorMap* out, const MapKey* keys, int n, int* tile_copy) {
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (g_copy_mode < 0) {
    // Whether this driver takes the permuted strides is asked once, with a fixed geometry (one
    // block of 16 tokens x 4 kv heads, rows contiguous) at the first caller's base address: the
    // answer must not depend on what that caller happens to pass.
    CUtensorMap probe;
    g_copy_mode = encode_map(&probe, MapKey{keys[0].base, 4, 1, 16, 16 * 4 * 256, 8}, true) ? 1 : 0;
  }
  // Every map of one launch has the same form. A geometry the tile form cannot express (a token
  // stride or block stride the encoder rejects there) falls back to row copies for this call only.
  for (int form = g_copy_mode; form >= 0; --form) {
    bool ok = true;
    for (int i = 0; i < n && ok; ++i) ok = cached_map(&out[i], keys[i], form == 1);
    if (ok) { *tile_copy = form; return true; }
  }
  return false;
}

}  // namespace sbk
