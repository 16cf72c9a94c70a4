/*
 * sbk.h -- C ABI of libsbk.so: the B200 (sm_100a) kernels behind the hybrid
 * decode-time cache path of SpikingBrain-7B (sliding-window paged KV + GLA
 * recurrent state).
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless the name ends in `_host`.
 *  - The library allocates nothing, keeps no pointer after a call returns and
 *    never synchronises; every launch is ordered on `stream` (a cudaStream_t
 *    passed as void*; NULL = the legacy default stream).
 *  - Return value: 0 on success, a negative SBK_E_* code when the host can see
 *    that the arguments are wrong (nothing is launched); sbk_last_error()
 *    then returns a thread-local description.
 *  - Device-side violations (a slot or block id outside the pool) never trap:
 *    the offending work item is skipped and a bit is OR-ed into `*status`
 *    (a device int32 the caller zeroes and reads when it wishes; may be NULL).
 *  - Element types are given as SBK_BF16 / SBK_F32 codes.
 *
 * Citations name the file of BICLab/SpikingBrain-7B whose call the entry point
 * stands in for.
 */
#ifndef SBK_H_
#define SBK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SBK_ABI_VERSION 5

/* element type codes */
#define SBK_BF16 0
#define SBK_F32 1

/* host-side error codes (return values) */
#define SBK_OK 0
#define SBK_E_ARG (-1)      /* bad shape / null pointer / unsupported combination */
#define SBK_E_ALIGN (-2)    /* a pointer or stride breaks the 16-byte rule */
#define SBK_E_WORKSPACE (-3) /* workspace too small */
#define SBK_E_LAUNCH (-4)   /* cudaGetLastError() after the launch was not cudaSuccess */

/* device-side status bits (OR-ed into *status) */
#define SBK_ST_BAD_SLOT 1      /* slot id >= num_blocks*block_size: token not written */
#define SBK_ST_BAD_BLOCK 2     /* block-table entry outside [0,num_blocks) inside the window */
#define SBK_ST_WAIT_TIMEOUT 4  /* a bounded in-kernel wait ran out; result of that CTA invalid */
#define SBK_ST_RETIRE_OVERFLOW 8 /* more blocks left the window than retired_out has columns */
#define SBK_ST_BAD_POSITION 16   /* a position outside the cos/sin table (token left untouched) */
#define SBK_ST_OUT_OF_BLOCKS 32  /* sbk_plan_step: the ring of free blocks cannot serve the step */
#define SBK_ST_TABLE_FULL 64     /* sbk_plan_step: a table row or slot_mapping is too short for the step */
#define SBK_ST_VALUE_RANGE 128   /* sbk_swa_prefill, two-tile tcgen05 kernel: a V value of magnitude 2^16 or more
                                    (or inf / NaN) met its fp16 second GEMM; SBK_PREFILL_TCGEN05 serves such a cache */

int sbk_abi_version(void);
const char* sbk_last_error(void);

/*
 * Paged-KV append with sliding-window block retirement.
 * Stands in for torch.ops._C_cache_ops.reshape_and_cache_flash as called at
 * vllm_hymeta/attention/meta_attention.py:790-799 (kv_cache_dtype "auto": a
 * plain copy), and for the block retirement the reference leaves to vLLM's
 * block manager behind the window-truncated block table of
 * meta_attention.py:479-485.
 *
 *  key,value     [T, kvh, D] rows of `elem_bytes`-wide elements; token stride
 *                `kv_token_stride_bytes` (>= kvh*D*elem_bytes)
 *  k_cache,v_cache  [num_blocks, block_size, kvh, D]; `cache_block_stride_bytes`
 *                between blocks, rows of one block contiguous
 *  slot_mapping  [T] int64 flat slot = block*block_size + offset; negative = skip
 *                (PAD_SLOT_ID, meta_attention.py:558)
 * Retirement (skipped when block_tables == NULL):
 *  block_tables  [B, max_blocks] int32, MUTATED: entries of logical blocks that
 *                lie wholly before the window are replaced by -1
 *  seq_lens      [B] int32 length of each sequence INCLUDING the appended tokens
 *  query_start_loc [B+1] int32 or NULL (NULL: one new token per sequence)
 *  window_left   keys visible to the left of a query (-1: unbounded, nothing retires).
 *                The first token still needed is max(0, seq_len - n_new - window_left).
 *  retired_out   [B, max_retired] int32: ids that left the window this call, in
 *                logical order, padded with -1 (may be NULL: only the table is edited)
 */
int sbk_kv_append(const void* key, const void* value, void* k_cache, void* v_cache,
                  const int64_t* slot_mapping, int T, int kvh, int D, int elem_bytes,
                  int64_t kv_token_stride_bytes, int64_t num_blocks, int block_size,
                  int64_t cache_block_stride_bytes,
                  int32_t* block_tables, int max_blocks, const int32_t* seq_lens,
                  const int32_t* query_start_loc, int B, int window_left,
                  int32_t* retired_out, int max_retired,
                  int32_t* status, void* stream);

/*
 * Gather the in-window tokens of every sequence through the block table into
 * dense head-first tensors [B, kvh, n_out, D] -- the tensors the reference's
 * Cache.update returns as `attn_state` (hf_7B_model/cache.py:94-108).
 * Row i of sequence b is token t0+i, t0 = max(0, seq_len-1-window_left);
 * rows past the visible length are zero-filled.
 */
int sbk_kv_gather(const void* k_cache, const void* v_cache, const int32_t* block_tables,
                  int max_blocks, const int32_t* seq_lens, int B, int kvh, int D,
                  int elem_bytes, int64_t num_blocks, int block_size,
                  int64_t cache_block_stride_bytes, int window_left,
                  void* k_out, void* v_out, int n_out,
                  int32_t* status, void* stream);

/*
 * Sliding-window paged-attention decode (one query token per sequence).
 * Stands in for flash_attn_cuda.fwd_kvcache as reached from
 * meta_attention.py:955-981 through fa_kernel_metatoken.py:84-105
 * (causal, window (window_left, -1), no alibi, no softcap, key2 == None).
 *
 *  q            [B, H, D] bf16, `q_seq_stride` elements between sequences
 *  k_cache,v_cache [num_blocks, block_size, kvh, D] bf16 (rows of a block contiguous)
 *  block_tables [B, max_blocks] int32; seq_lens [B] int32 (query is token seq_len-1)
 *  window_left  keys visible left of the query (-1 = all)
 *  out          [B, H, D] of `out_dtype` (SBK_BF16 or SBK_F32), `out_seq_stride` elements
 *  lse_out      [B, H] float natural-log-sum-exp of the scaled scores, or NULL
 *  workspace    at least sbk_swa_workspace_bytes(B,H,D,max_pieces) bytes, 16-byte aligned. It
 *               begins with the work-ticket counters and one completion counter per sequence
 *               (32 + 4*roundup(B,4) bytes): these must be ZERO before the first call with a
 *               given buffer and B, and every call that ends without SBK_ST_WAIT_TIMEOUT leaves
 *               them zero. A call in which a wait ran out leaves them where they stood and
 *               MARKS the workspace: every later call given it raises SBK_ST_WAIT_TIMEOUT again
 *               and computes nothing, so the fault cannot turn into silently wrong rows; zero
 *               those leading bytes (or the whole buffer) to use it again. Split-K partials
 *               follow. Calls that overlap on the GPU need separate workspaces.
 *  key2,value2  [num_meta, kvh, D] bf16 contiguous "meta" (sink) tokens that every query sees on top of
 *               its window -- the second attention pass over k2/v2 and the log-sum-exp merge of
 *               fa_kernel_metatoken.py:124-194, done here as extra leading tiles of the same
 *               softmax; num_meta a multiple of 16, 0 (with NULLs) for none
 *  split_chunks how a sequence is split over CTAs.  > 0: fixed pieces of that many 16-token
 *               chunks, handed to the CTAs through a ticket counter.  < 0: balanced mode -- the
 *               chunks of the whole batch are cut into one equal run per CTA, and -split_chunks
 *               is the shortest run allowed (with max_pieces == 1 this degrades to whole
 *               sequences).  0: fixed pieces of 32 chunks. The Python wrapper's default is -8.
 *               A balanced-mode launch is a cooperative launch (the CTAs that hold the pieces of a
 *               sequence cut into many pieces wait for one another to share its fold): the grid of
 *               two CTAs per SM must be resident at once, which the driver guarantees or refuses
 *               (SBK_E_LAUNCH); it can be captured into a CUDA graph like any launch.
 *  max_pieces   upper bound on the pieces of one sequence (sizes the workspace); >= 1
 *  item_cost    balanced mode only: what starting and finishing a sequence is charged, in chunks,
 *               when the runs are made equal in cost (< 0: the library's tuned value, 8)
 * Supported: D == 128, H % kvh == 0, H/kvh <= 8, kvh in {1,2,4}, block_size % 16 == 0.
 */
size_t sbk_swa_workspace_bytes(int B, int H, int D, int max_pieces);
/* How sbk_swa_decode moves a 16-token tile into shared memory on this driver: 1 = one tensor
 * copy per tile (kvh*4 KiB), 0 = one per 128-byte row (2 KiB), -1 = no call made yet.
 * Diagnostic only; no counterpart in the reference. */
int sbk_swa_copy_mode(void);
int sbk_swa_decode(const void* q, int64_t q_seq_stride, const void* k_cache, const void* v_cache,
                   const int32_t* block_tables, int max_blocks, const int32_t* seq_lens,
                   int B, int H, int kvh, int D, int64_t num_blocks, int block_size,
                   int64_t cache_block_stride_bytes, int window_left, float scale,
                   void* out, int out_dtype, int64_t out_seq_stride, float* lse_out,
                   void* workspace, size_t workspace_bytes, int split_chunks, int max_pieces,
                   int item_cost, const void* key2, const void* value2, int num_meta,
                   int32_t* status, void* stream);

/*
 * sbk_swa_decode for callers that cannot allocate device memory -- a server that gave all free
 * HBM to its KV pool at start-up, a loop that forbids allocator calls once running, a binding
 * with no tensor library behind it. No counterpart in the reference. The arguments of
 * sbk_swa_decode without `workspace`, `item_cost` (library value) and the sink tokens
 * key2/value2/num_meta (not served here: use sbk_swa_decode for layers that have them): the
 * scratch is a fixed array of sbk_swa_static_scratch_bytes() (16 MiB) inside the library,
 * resident on every GPU that loads the library until the process ends.
 *  - sbk_swa_workspace_bytes(B, H, D, max_pieces) must not exceed that size, else
 *    SBK_E_WORKSPACE is returned and nothing is launched (with one piece per sequence any B up
 *    to about four million fits; with 9 pieces and 28 heads B up to 128).
 *  - The first call on a device looks the array's device address up; make that call before
 *    starting a stream capture. The call itself performs no allocation of any kind.
 *  - All calls share the one array: two calls whose kernels can overlap on the GPU (different
 *    streams, no dependency) race on it. Calls on one stream are safe; the counters (and the
 *    mark a timed-out call leaves) are cleared on `stream` at the start of every call.
 *  - The per-device address table behind the first-call look-up is not locked: make the first
 *    call on a device from one thread.
 */
size_t sbk_swa_static_scratch_bytes(void);
int sbk_swa_decode_static(const void* q, int64_t q_seq_stride, const void* k_cache, const void* v_cache,
                          const int32_t* block_tables, int max_blocks, const int32_t* seq_lens,
                          int B, int H, int kvh, int D, int64_t num_blocks, int block_size,
                          int64_t cache_block_stride_bytes, int window_left, float scale,
                          void* out, int out_dtype, int64_t out_seq_stride, float* lse_out,
                          int split_chunks, int max_pieces, int32_t* status, void* stream);

/*
 * Head-sharded decode with the all-gather of the head outputs fused into the kernel.
 * The reference shards attention heads over tensor-parallel ranks and gathers the per-rank
 * head outputs with a collective before the output projection
 * (vllm_hymeta/model_for_7B/modeling_gla_swa.py:153-202, :228-231; gla_attention.py:126-145).
 * Here every rank owns a gathered buffer [tokens, H_total, D] bf16 that its peers can store to:
 * sbk_swa_decode_gather computes this rank's H heads exactly as sbk_swa_decode does, writes them
 * into its own buffer (`out` = the address of its head slice, `out_seq_stride` = H_total * D)
 * and stores each finished row into the same place of every peer's buffer (`peer_out[p]` = peer
 * p's address of this rank's slice) with plain 16-byte stores through NVLink. The last CTA
 * to finish then stores `flag_value` into `peer_flag[p]` (this rank's slot of peer p's flag
 * array) with release semantics -- unless a wait inside the kernel ran out, in which case the
 * flag stays and the peers' own wait reports the step. A rank sees the complete rows after
 * sbk_peer_wait on its own flag array.
 *  - flag values grow by one per step and are never reused; the caller alternates between two
 *    gathered buffers so that a peer one step ahead does not store into rows still being read.
 *  - `workspace`, `split_chunks`, `max_pieces`, `item_cost` as for sbk_swa_decode.
 *  - No collective library call, no multicast object, no copy through a tensor map: peers are
 *    reached by stores only.
 *
 * Peer memory: sbk_peer_alloc gives zeroed device memory of this process whose handle
 * (sbk_peer_export, sbk_peer_handle_bytes() bytes, any byte transport between the processes)
 * another process maps with sbk_peer_open; sbk_peer_close unmaps, sbk_peer_free releases.
 * sbk_peer_wait(flags, n, self, value, flag_base, advance, timeout_ms): one launch on `stream`
 * that returns once flags[p] >= value for every p != self, or after timeout_ms with
 * SBK_ST_WAIT_TIMEOUT raised in `status` (the context stays usable). sbk_peer_signal stores
 * `value` to n_peer flag addresses (a step in which this rank has no sequences).
 *  - `flag_base` (device int32, may be null) makes the calls replayable from a CUDA graph: the
 *    value stored / awaited is flag_value + *flag_base, read on the device, and sbk_peer_wait
 *    adds `advance` to *flag_base once it is through (timed out or not). With flag_value 1 and
 *    advance 1 on every rank each decode + wait pair is one step of a counter that lives on
 *    the device; a graph must hold an even number of such pairs, because the pairs alternate
 *    between the two gathered buffers and those addresses are fixed at capture.
 */
int sbk_swa_decode_gather(const void* q, int64_t q_seq_stride, const void* k_cache, const void* v_cache,
                          const int32_t* block_tables, int max_blocks, const int32_t* seq_lens,
                          int B, int H, int kvh, int D, int64_t num_blocks, int block_size,
                          int64_t cache_block_stride_bytes, int window_left, float scale,
                          void* out, int64_t out_seq_stride, void* workspace, size_t workspace_bytes,
                          int split_chunks, int max_pieces, int item_cost, const void* key2,
                          const void* value2, int num_meta, void* const* peer_out, int32_t* const* peer_flag, int n_peer,
                          int32_t flag_value, const int32_t* flag_base, int32_t* status, void* stream);
/* The GLA step of a head-sharded layer with the same delivery: arguments as sbk_gla_step (bf16 in
 * and out), `out` = this rank's head slice of its gathered buffer with `out_seq_stride` elements
 * between sequences, `counter` = one zeroed int32 on the device (left at zero by every call). */
int sbk_gla_step_gather(const void* q, const void* k, const void* v, const void* g,
                        float* state, int64_t num_slots, const int64_t* slot_idx, int B, int H,
                        int Hkv, int D, float scale, void* out, int64_t out_seq_stride,
                        int fuse_flags, float gate_normalizer, const void* norm_weight,
                        float norm_eps, int32_t* counter, void* const* peer_out,
                        int32_t* const* peer_flag, int n_peer, int32_t flag_value,
                        const int32_t* flag_base, int32_t* status, void* stream);
int sbk_peer_alloc(size_t bytes, void** ptr);
int sbk_peer_free(void* ptr);
int sbk_peer_handle_bytes(void);
int sbk_peer_export(const void* ptr, void* handle, int handle_bytes);
int sbk_peer_open(const void* handle, int handle_bytes, void** ptr);
int sbk_peer_close(void* ptr);
int sbk_peer_wait(const int32_t* flags, int n, int self, int32_t value, int32_t* flag_base,
                  int32_t advance, int timeout_ms, int32_t* status, void* stream);
int sbk_peer_signal(int32_t* const* peer_flag, int n_peer, int32_t value, const int32_t* flag_base,
                    void* stream);

/*
 * Rotary position embedding fused into the append: rotates the new tokens' query rows in place,
 * rotates their key rows on the way into the cache, copies the value rows and retires blocks,
 * all in one launch. Stands in for GLAswaRotaryEmbedding.forward
 * (vllm_hymeta/model_for_7B/modeling_gla_swa.py:79-93, called at :215) followed by the cache
 * write of MetaAttentionImpl.forward (vllm_hymeta/attention/meta_attention.py:790-799), and for
 * apply_rotary_pos_emb + Cache.update on the HF side (hf_7B_model/window_attention.py:161-175).
 * NeoX (rotate-half) form over the first rot_dim elements of every head; each product and the
 * sum are rounded to the element type separately, as the reference's tensor expression
 * (x * cos) + (rotate_half(x) * sin) rounds them.
 *
 *  query        [T, H, D], `q_token_stride_bytes` between tokens, rotated IN PLACE; NULL: skipped
 *  key          [T, kvh, D]; the rotated rows go to k_cache; with key_in_place != 0 they are also
 *               written back to `key` (the reference's prompt pass attends over that tensor)
 *  value        [T, kvh, D], copied to v_cache; key and value share kv_token_stride_bytes
 *  positions    [T] int64 position of every token; outside [0, max_position) raises
 *               SBK_ST_BAD_POSITION and the token is skipped
 *  cos_sin_cache [max_position, rot_dim] of `dtype`: cos of the rot_dim/2 frequencies, then sin
 *               (the layout of GLAswaRotaryEmbedding._compute_cos_sin_cache, :71-79)
 *  dtype        SBK_BF16 or SBK_F32: element type of query, key, value, the caches and the table
 *  slot_mapping entry -1: nothing is written to the cache for that token; its query (and key, with
 *               key_in_place) is still rotated
 *  remaining arguments: as in sbk_kv_append
 * rot_dim a multiple of 16 (bf16) or 8 (fp32) elements, rot_dim <= D.
 */
int sbk_rope_kv_append(void* query, int H, int64_t q_token_stride_bytes, void* key, const void* value,
                       int key_in_place, void* k_cache, void* v_cache, const int64_t* slot_mapping,
                       const int64_t* positions, const void* cos_sin_cache, int rot_dim,
                       int64_t max_position, int T, int kvh, int D, int dtype,
                       int64_t kv_token_stride_bytes, int64_t num_blocks, int block_size,
                       int64_t cache_block_stride_bytes, int32_t* block_tables, int max_blocks,
                       const int32_t* seq_lens, const int32_t* query_start_loc, int B,
                       int window_left, int32_t* retired_out, int max_retired, int32_t* status,
                       void* stream);

/*
 * Device-resident step planning and block allocation. State that stays on the GPU between steps:
 *    seq_lens [B] int32, block_tables [B, max_blocks] int32 (-1 = no block),
 *    ring [num_blocks] int32 (free block ids, FIFO), ctrl [4] uint64 (head, tail, lowest free
 *    count seen, steps planned).
 * sbk_plan_step does, in one launch, what the reference does on the host every step - the
 * per-sequence loop of MetaAttentionMetadataBuilder (vllm_hymeta/attention/meta_attention.py:
 * 435-494: context length, window-truncated block table, slot mapping) with the engine's block
 * manager behind it - and what MetaAttentionMetadata.advance_step (:338-409) does on the device
 * for multi-step decode. For every row b with n_new[b] > 0 (n_new NULL: one token per row):
 *   - blocks wholly before max(0, seq_lens[b] - window_left) are retired: pushed on the ring,
 *     their table entries set to -1 (retire != 0; window_left -1 retires nothing). retire == 2
 *     ("trim") also visits the rows WITHOUT new tokens and retires what their next token will not
 *     see: after a prompt chunk its look-back window (up to a chunk's worth of blocks beyond the
 *     window) is given back at once instead of at the row's next step;
 *   - missing table entries of the logical blocks the new tokens fall in are filled from the ring
 *     (retirement first, so blocks freed by this step can be reused by it);
 *   - slot_mapping [T] int64 and positions [T] int64 (or NULL) get one entry per new token,
 *     tokens of row b at query_start_loc[b] ...; entries past the last token: slot -1;
 *   - context_lens [B] (or NULL) = length before the step; query_start_loc [B+1] is written (it may
 *     be NULL only when n_new is NULL); seq_lens[b] += n_new[b].
 * ring == NULL (with ctrl NULL): no allocator; the tables are filled by someone else (the engine's
 * scheduler) and a missing entry raises SBK_ST_OUT_OF_BLOCKS: this is advance_step.
 * A step that cannot be served - ring too empty (SBK_ST_OUT_OF_BLOCKS), a row longer than its table
 * or more new tokens than T (SBK_ST_TABLE_FULL) - changes no state and fills slot_mapping with -1.
 * Pushes and pops are placed in row order, so the allocator is deterministic. One CTA; meant for
 * B up to a few thousand rows. T must equal the host's count of new tokens or exceed it (padding).
 *
 * sbk_pool_init: ring <- 0..num_blocks-1, counters reset; seq_lens <- 0 and block_tables <- -1
 * when given. sbk_release_rows: rows [n_rows] int32 name finished sequences; their live blocks go
 * back on the ring, their entries become -1 and their lengths 0. A row named more than once is
 * released once.
 */
int sbk_pool_init(int32_t* ring, uint64_t* ctrl, int num_blocks, int32_t* seq_lens,
                  int32_t* block_tables, int max_blocks, int B, void* stream);
int sbk_plan_step(const int32_t* n_new, int32_t* seq_lens, int32_t* block_tables, int max_blocks,
                  int B, int block_size, int window_left, int retire, int32_t* ring, uint64_t* ctrl,
                  int num_blocks, int64_t* slot_mapping, int64_t* positions, int32_t* context_lens,
                  int32_t* query_start_loc, int T, int32_t* status, void* stream);
int sbk_release_rows(const int32_t* rows, int n_rows, int32_t* seq_lens, int32_t* block_tables,
                     int max_blocks, int B, int block_size, int32_t* ring, uint64_t* ctrl,
                     int num_blocks, int32_t* status, void* stream);

/*
 * Fused GLA recurrent-state step, in place in the slot cache:
 *    S[slot] <- diag(exp(g)) . S[slot] + k^T v ;   o = (q*scale) . S[slot]
 * Stands in for my_fused_recurrent_gla
 * (vllm_hymeta/model_for_7B/my_fused_recurrent.py:138-153, kernel :9-80) and,
 * with slot_idx == NULL, for fused_recurrent_gla as called at
 * hf_7B_model/gla_attention.py:153 on a [B,H,D,D] state.
 *
 *  q            [B, H, D]; k,v,g [B, Hkv, D] with Hkv == H (heads already repeated,
 *               as the reference passes them) or Hkv a divisor of H (head h reads
 *               kv head h / (H/Hkv), the repeat_interleave order of repeat_kv)
 *  in_dtype     type of q,k,v,g: SBK_BF16 or SBK_F32; out_dtype likewise for out [B, H, D]
 *  state        [num_slots, H, D, D] float32 (k index before v index)
 *  slot_idx     [B] int64 (NULL: slot b for sequence b); -1: row untouched, out row not written
 *  D in {64, 128}
 *
 * The element-wise neighbours of the call in the reference layer can be folded in
 * (vllm_hymeta/model_for_7B/gla_attention.py:250-262 and :233; hf_7B_model/gla_attention.py:
 * 134-145, 170), so that q, k and the gate logits arrive straight from the projections:
 *  fuse_flags   SBK_GLA_RELU_QK: q <- relu(q), k <- relu(k) (the layer's feature map);
 *               SBK_GLA_GATE_LOGITS: g holds gate logits and the log-decay is
 *               logsigmoid(g) / gate_normalizer, each of the two steps rounded to in_dtype as
 *               the reference's tensor expression rounds them; 0: none
 *  norm_weight  [D] in in_dtype, or NULL: o <- o * rsqrt(mean_d(o^2) + norm_eps) * norm_weight per
 *               head (the layer's g_norm), computed on the fp32 read-out before the one rounding
 *               to out_dtype
 */
#define SBK_GLA_RELU_QK 1
#define SBK_GLA_GATE_LOGITS 2
int sbk_gla_step(const void* q, const void* k, const void* v, const void* g, int in_dtype,
                 float* state, int64_t num_slots, const int64_t* slot_idx,
                 int B, int H, int Hkv, int D, float scale,
                 void* out, int out_dtype, int fuse_flags, float gate_normalizer,
                 const void* norm_weight, float norm_eps, int32_t* status, void* stream);

/*
 * Sliding-window attention for runs of query tokens over the paged cache (prefill with block
 * tables, chunked prefill). Stands in for metatoken_flash_attn_varlen_func(..., causal=True,
 * window_size=(window_left, 0), block_tables=prefill_meta.block_tables) as called at
 * vllm_hymeta/attention/meta_attention.py:900-919 (-> flash-attn _flash_attn_varlen_forward,
 * fa_kernel_metatoken.py:235-253) with key2 == None. The K/V of the new tokens must already be in
 * the cache. Query i of sequence s sits at position context_lens[s] + i and sees keys
 * [position - window_left, position] (window_left -1: all keys up to itself).
 *
 *  q            [T, H, D] bf16 token-major, `q_tok_stride` elements between tokens; sequence s owns
 *               rows query_start_loc[s] .. query_start_loc[s+1]-1 (int32 [n_seqs+1])
 *  context_lens [n_seqs] int32 tokens of the sequence that were in the cache before this call
 *  max_query_len  longest run of this call (host value; sizes the grid)
 *  out          [T, H, D] bf16, `out_tok_stride` elements between tokens
 *  key2,value2,num_meta  sink tokens as in sbk_swa_decode (the k2/v2 pass of
 *               fa_kernel_metatoken.py:198-280), or NULL, NULL, 0
 *  kernel       SBK_PREFILL_AUTO: a tcgen05 kernel (tensor memory, 128-key tiles) when q and out
 *               are 16-byte aligned with token strides that are multiples of 8 elements -- two
 *               query tiles per CTA taking turns when max_query_len exceeds one tile's 128 / (H/kvh)
 *               queries, one tile per CTA otherwise -- else the mma.sync kernel;
 *               SBK_PREFILL_TCGEN05 (one tile) / SBK_PREFILL_TCGEN05_PAIR (two tiles) /
 *               SBK_PREFILL_MMA_SYNC force one (the tcgen05 ones return SBK_E_ALIGN when q / out
 *               do not meet their rule). All three compute the same function.
 * Supported: D == 128, H % kvh == 0, H/kvh <= 8, block_size % 16 == 0.
 */
#define SBK_PREFILL_AUTO 0
#define SBK_PREFILL_TCGEN05 1
#define SBK_PREFILL_MMA_SYNC 2
#define SBK_PREFILL_TCGEN05_PAIR 3
int sbk_swa_prefill(const void* q, int64_t q_tok_stride, const void* k_cache, const void* v_cache,
                    const int32_t* block_tables, int max_blocks, const int32_t* query_start_loc,
                    const int32_t* context_lens, int n_seqs, int max_query_len, int H, int kvh, int D,
                    int64_t num_blocks, int block_size, int64_t cache_block_stride_bytes,
                    int window_left, float scale, void* out, int64_t out_tok_stride,
                    const void* key2, const void* value2, int num_meta, int kernel,
                    int32_t* status, void* stream);

/*
 * The same attention over K/V that are NOT in a paged cache but passed as tensors: the prompt run
 * of MetaAttentionImpl.forward without block tables (vllm_hymeta/attention/meta_attention.py:833-884:
 * metatoken_flash_attn_varlen_func(q1=query, k1=key, v1=value, cu_seqlens_q, cu_seqlens_k, causal,
 * window_size)), which is also what the engine's memory-profiling run executes.
 *
 *  key, value   [n_kv_tokens, kvh, D] bf16, `kv_tok_stride` elements between tokens (>= kvh*D: they
 *               may be column slices of one projection output); 16-byte aligned
 *  k_start_loc  [n_seqs+1] int32: sequence s owns keys k_start_loc[s] .. k_start_loc[s+1]-1; its last
 *               query sees its last key (queries are aligned to the end of the keys, as flash-attn's
 *               causal mask does when a sequence has more keys than queries)
 *  causal       non-zero: as above. 0: every query sees every key of its sequence and the window is
 *               ignored (the pass of the sink tokens' own queries over key2/value2,
 *               fa_kernel_metatoken.py:262-276, which the reference runs with causal=False)
 *  q, out       as in sbk_swa_prefill, but 16-byte aligned with token strides multiples of 8 elements
 *               (tcgen05 kernel only)
 */
int sbk_swa_prefill_dense(const void* q, int64_t q_tok_stride, const void* key, const void* value,
                          int64_t kv_tok_stride, int64_t n_kv_tokens, const int32_t* query_start_loc,
                          const int32_t* k_start_loc, int n_seqs, int max_query_len, int H, int kvh, int D,
                          int window_left, int causal, float scale, void* out, int64_t out_tok_stride,
                          const void* key2, const void* value2, int num_meta, int32_t* status, void* stream);

/*
 * GLA scan over a run of tokens per sequence with state carry (prefill and chunked prefill):
 * for each sequence the state is read once, advanced token by token exactly as sbk_gla_step
 * would, and written back once. Stands in for the per-sequence loop of
 * GatedLinearAttention._prefill_and_mix_infer (vllm_hymeta/model_for_7B/gla_attention.py:179-211:
 * fused_chunk_gla with initial_state from the slot, then the copy back into the slot) and for
 * chunk_gla / fused_chunk_gla as called at hf_7B_model/gla_attention.py:155-157.
 *
 *  q            [T, H, D] token-major; k,v,g [T, Hkv, D]; tokens of sequence s are rows
 *               query_start_loc[s] .. query_start_loc[s+1]-1   (query_start_loc: [n_seqs+1] int32)
 *  state        [num_slots, H, D, D] float32; slot_idx [n_seqs] int64 (NULL: slot s; -1: skip)
 *  reset        [n_seqs] uint8 or NULL: non-zero = start this sequence from a zero state (a new
 *               prompt; the reference clears such slots in GLAswaModel._clear_prefill_cache,
 *               modeling_gla_swa.py:391-414) instead of reading the slot
 *  out          [T, H, D] of out_dtype
 *  fuse_flags, gate_normalizer, norm_weight, norm_eps   as in sbk_gla_step
 *  max_query_len, workspace, workspace_bytes
 *               the chunk-parallel form, which the reference reaches through chunk_gla /
 *               fused_chunk_gla spreading one sequence over the GPU: given the longest run of the
 *               call (host value) and sbk_gla_scan_workspace_bytes(n_seqs, max_query_len, H, D)
 *               bytes of 16-byte aligned scratch (contents irrelevant before, meaningless after),
 *               a call whose (sequence, head) chains would fill less than half of the GPU cuts
 *               every run into sub-chunks: a local scan of each from a zero state, a carry of the
 *               states from sub-chunk to sub-chunk, and the scan proper of every sub-chunk from its
 *               true incoming state -- three launches. The sum is the same in another association:
 *               state and outputs agree with the one-chain scan to fp32 rounding, not bit for
 *               bit. With bf16 tokens at D = 128, 16-byte aligned q/k/v/g/out and a longest run of
 *               at least 256 tokens the call takes the chunked form on the tensor cores instead
 *               (tcgen05, 128-token chunks, every fp32 operand as a bf16 head plus a bf16
 *               remainder; few long runs are cut into pieces as above): same agreement with the
 *               one-chain scan (1e-5 of the largest output). A chunk whose summed log-decay leaves
 *               the range of that form (|sum| > 80 on some key dim) ends it for that (sequence,
 *               head); the token-by-token kernel finishes the run from there in the same call.
 *               max_query_len only plans the cut: a run longer than stated is still scanned
 *               correctly (its last piece takes the rest). workspace NULL or max_query_len <= 0:
 *               one chain per (sequence, head), whose result does not depend on how the tokens
 *               were cut into calls. The size query returns 0 when the call needs no scratch.
 */
size_t sbk_gla_scan_workspace_bytes(int n_seqs, int max_query_len, int H, int D);
int sbk_gla_scan(const void* q, const void* k, const void* v, const void* g, int in_dtype,
                 const int32_t* query_start_loc, int n_seqs, float* state, int64_t num_slots,
                 const int64_t* slot_idx, const uint8_t* reset, int H, int Hkv, int D, float scale,
                 void* out, int out_dtype, int fuse_flags, float gate_normalizer,
                 const void* norm_weight, float norm_eps, int max_query_len, void* workspace,
                 size_t workspace_bytes, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SBK_H_ */
