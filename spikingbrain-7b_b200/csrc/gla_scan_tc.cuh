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
};

constexpr int kMinRun = 256;   // shortest longest-run for which the entry point takes this kernel

int launch(const Params& P, int n_seqs, cudaStream_t stream);

}  // namespace gla_tc
}  // namespace sbk
