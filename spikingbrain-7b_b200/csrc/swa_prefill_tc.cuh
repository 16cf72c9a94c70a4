// Interface between the prefill entry point and its tcgen05 kernel.
#pragma once

#include "sbk_common.cuh"
#include "sbk_tma.cuh"

namespace sbk {
namespace prefill_tc {

struct Params {
  const __nv_bfloat16* q; int64_t q_tok_stride;
  const int32_t* block_tables; int max_blocks;
  const int32_t* query_start_loc; const int32_t* context_lens;
  int n_seqs; int tiles_per_seq; int H; int G; int64_t num_blocks; int block_size;
  int bq;              // query tokens per CTA: 128 / G (the 128 rows of a tile are bq queries x G heads)
  int window_left; float scale_log2;
  __nv_bfloat16* out; int64_t out_tok_stride;
  int32_t* status; int tile_copy;
  int n_meta_chunks;   // 16-token chunks of always-visible sink keys, streamed ahead of the window
  // dense mode: K/V are not in a paged cache but tensors [T, kvh, D] (the maps see them as one block of
  // T tokens); sequence s owns keys k_start_loc[s] .. k_start_loc[s+1]-1 and its last query sees its last key
  const int32_t* k_start_loc;   // NULL: paged mode
  int noncausal;                // dense mode only: every query sees every key of its sequence
};

// Tensor maps with ONE 128-byte row (64 dims of one kv head) per copy: box_rows == 1.
inline int queries_per_tile(int G) { return 128 / G; }
int launch(const Params& P, int kvh, const CUtensorMap& map_k, const CUtensorMap& map_v,
           const CUtensorMap& map_k2, const CUtensorMap& map_v2, cudaStream_t stream);

}  // namespace prefill_tc

// the same work with two query tiles per CTA taking turns (tiles_per_seq counts pairs of tiles)
namespace prefill_tc2 {
int launch(const prefill_tc::Params& P, int kvh, const CUtensorMap& map_k, const CUtensorMap& map_v,
           const CUtensorMap& map_k2, const CUtensorMap& map_v2, cudaStream_t stream);
}  // namespace prefill_tc2
}  // namespace sbk
