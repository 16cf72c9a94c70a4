// Interface between the GLA scan entry point and its tensor-core (tcgen05) kernel.
#pragma once

#include "sbk_common.cuh"

namespace sbk {
namespace gla_tc {

struct Params {
  const __nv_bfloat16* q; const __nv_bfloat16* k; const __nv_bfloat16* v; const __nv_bfloat16* g;
  const int32_t* query_start_loc;
  float* state; int64_t num_slots; const int64_t* slot_idx; const uint8_t* reset;
  int H; int Hkv; float scale;
  void* out; int out_f32;
  int32_t* status;
  GlaFusion fu;
  // [n_seqs * H]: first token of the run that this kernel did NOT process (the run's end when it
  // went all the way). A chunk whose decay is too strong for the factored form stops the chain; the
  // token-by-token kernel picks the run up from there.
  int32_t* resume;
  // Chunk-parallel use (n_sub > 1): a run is cut into n_sub pieces of sub_chunks 128-token chunks that
  // different CTAs own. The local pass (launch(..., local = true)) scans every piece but a run's last
  // without read-out, piece 0 from the run's incoming state and the others from zero, and leaves
  // the end states in `tiles` [n_seqs][n_sub-1][H][D*D] and the products of the decays in `decays`
  // [n_seqs][n_sub-1][H][D]; after the carry between them the full pass starts every piece from
  // its true incoming state. `bail` [n_seqs * H], zeroed by the caller: set by the local pass when a
  // piece met a chunk it does not take; the full pass then leaves the whole run to the other kernel.
  float* tiles; float* decays; int n_sub; int sub_chunks; int32_t* bail;
};

constexpr int kMinRun = 256;   // shortest longest-run for which the entry point takes this kernel
constexpr int kChunkTokens = 128;

int launch(const Params& P, int n_seqs, bool local, cudaStream_t stream);

}  // namespace gla_tc
}  // namespace sbk
