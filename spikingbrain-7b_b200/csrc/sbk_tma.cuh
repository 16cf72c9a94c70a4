// TMA tensor maps over a paged K/V cache, shared by the decode and the prefill attention kernels.
#pragma once

#include <cuda.h>

#include "sbk_common.cuh"

namespace sbk {

// A cache [num_blocks][block][kvh][128] bf16 seen as 64-element (128-byte) rows. (A dense
// [T][kvh][128] tensor, possibly a strided view of a wider row, is the same thing with one block of T
// tokens and its own token stride; tokens past T read as zeros.)
//   tile copies: dims (64, token in block, 128-byte row of a token, block) -- the token stride
//                (kvh*256 B) comes BEFORE the row stride (128 B), so a box of (64, 16, box_rows, 1)
//                lands in shared memory as [row][token][128 B];
//   row copies : dims (64, 128-byte row, token in block, block), box (64, 1, 16, 1): the same
//                shared-memory picture built from one copy per 128-byte row.
// Both use the 128-byte swizzle (16-byte chunk index XOR token & 7 for tiles on 1 KiB boundaries).
struct MapKey {
  const void* base; int kvh; int64_t num_blocks; int block_size; int64_t block_stride;
  int box_rows;   // 128-byte rows per tile copy: 2*kvh (all kv heads), 2 (one kv head) or 1 (64 dims)
  int64_t tok_stride = 0;   // bytes between tokens; 0: kvh*256 (rows of a block contiguous)
  bool operator==(const MapKey& o) const {
    return base == o.base && kvh == o.kvh && num_blocks == o.num_blocks && block_size == o.block_size &&
           block_stride == o.block_stride && box_rows == o.box_rows && tok_stride == o.tok_stride;
  }
};

// Encoded maps for the `n` geometries of one launch, from a small process-wide cache, all in one
// form: *tile_copy = 1 for tile copies (the permuted-stride form, when the driver takes it --
// asked once per process with a fixed geometry -- and every key can be expressed in it), else 0
// for row copies. False when some key cannot be encoded in either form.
bool get_maps(CUtensorMap* out, const MapKey* keys, int n, int* tile_copy);
int copy_mode();   // -1 unknown, 1 tile copies, 0 row copies

// 4-D tensor copy global -> shared (TMA), completion in bytes on an mbarrier
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::
          "r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

}  // namespace sbk
