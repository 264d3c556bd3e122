/*
 * b200attn — C ABI of the B200 (sm_100a) attention + paged KV-cache kernels.
 *
 * This library stands where tt-xla's vLLM plugin lowers its attention custom ops
 * through PJRT and TT-MLIR.  Every entry point replaces the device side of one
 * `torch.ops.tt.*` op (python_package/tt_torch/custom_ops.py) as it is called from
 * integrations/vllm_plugin/vllm_tt/attention_impls/attention.py; the citation
 * above each declaration names the reference interface it replaces.
 *
 * Conventions
 *   - All pointers are CUDA device pointers unless a parameter says "host".
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *     Every call is asynchronous on that stream.
 *   - Return value: 0 = launched; negative = argument rejected on the host, nothing
 *     was launched; positive = a cudaError_t from the launch.  Nothing throws,
 *     aborts or traps.  There is no CPU fallback: without a CUDA device every
 *     compute entry point returns B200ATTN_ERR_NO_DEVICE.
 *   - The library allocates no device memory; split-KV scratch is passed in by the
 *     caller (see b200attn_decode_workspace_bytes).
 *   - K/V cache layout is the plugin's: one K and one V tensor per layer, each
 *     [num_blocks, num_kv_heads, block_size, head_size] contiguous
 *     (attention.py:103-112).  Element (blk,h,off,d) sits at
 *     ((blk*num_kv_heads + h)*block_size + off)*head_size + d.
 *   - Head counts are the LOCAL (per tensor-parallel rank) counts.
 *   - Supported: bf16 data, head_size in {64,128}, block_size in {32,64},
 *     num_q_heads/num_kv_heads <= 16 for decode.  Anything else is rejected with
 *     B200ATTN_ERR_UNSUPPORTED.
 */
#ifndef B200ATTN_H_
#define B200ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200ATTN_VERSION 100

enum b200attn_status {
  B200ATTN_OK = 0,
  B200ATTN_ERR_NULL_POINTER = -1,
  B200ATTN_ERR_UNSUPPORTED = -2,   /* head_size / block_size / group size outside the supported set */
  B200ATTN_ERR_MISALIGNED = -3,    /* a pointer or stride breaks the 16-byte rule */
  B200ATTN_ERR_WORKSPACE = -4,     /* workspace missing or too small */
  B200ATTN_ERR_BAD_ARGUMENT = -5,  /* negative sizes, inconsistent head counts ... */
  B200ATTN_ERR_NO_DEVICE = -6,     /* no CUDA device / driver entry point unavailable */
  B200ATTN_ERR_TENSOR_MAP = -7,    /* cuTensorMapEncodeTiled refused the layout */
  B200ATTN_ERR_TOO_LARGE = -8      /* size beyond a documented maximum */
};

/* Device-side diagnostics word values (see b200attn_read_error_word). */
enum b200attn_device_error {
  B200ATTN_DEV_OK = 0,
  B200ATTN_DEV_WAIT_TIMEOUT = 1,   /* a bounded wait ran out; CTAs that start within the next second
                                      return without writing their output, later launches run
                                      normally; the word stays set until it is read */
  B200ATTN_DEV_BAD_INDEX = 2       /* a page id or slot was outside the cache */
};

/* Library version (B200ATTN_VERSION of the build). */
int b200attn_version(void);

/* Human-readable text for a status returned by any entry point. */
const char* b200attn_status_string(int status);

/* ------------------------------------------------------------------------------------------
 * KV-cache write, decode form.
 * Replaces: torch.ops.tt.paged_update_cache called once for K and once for V
 *           (custom_ops.py:962-1013; call site attention.py:468-484).
 * For every user u: pos = update_indices[u];
 *   cache[page_table[u, pos / block_size], :, pos % block_size, :] = new[u, :, :]
 * with Python floor-division / modulo and negative-index wrap-around on the page-table
 * column, exactly as the reference's CPU branch indexes (custom_ops.py:985-998).
 * k_new / v_new are token-major: element (u,h,d) at u*new_token_stride + h*head_size + d.
 * The caches are updated in place (the reference returns a clone and copies it back,
 * attention.py:513-515; the observable result is the same).
 * ------------------------------------------------------------------------------------------ */
int b200attn_paged_update_cache(void* k_cache, void* v_cache,
                                const void* k_new, const void* v_new,
                                int64_t new_token_stride,
                                const int32_t* update_indices,
                                const int32_t* page_table, int64_t page_table_stride,
                                int page_table_width,
                                int num_users, int num_kv_heads, int head_size,
                                int block_size, int64_t num_blocks, void* stream);

/* ------------------------------------------------------------------------------------------
 * KV-cache write, prefill / chunk form.
 * Replaces: torch.ops.tt.paged_fill_cache called once for K and once for V
 *           (custom_ops.py:1016-1104; call site attention.py:485-511).
 * User u's tokens_per_user tokens go to blocks fill_page_table[batch_idx[u], 0..),
 * token t at block column t / block_size, offset t % block_size.  batch_idx may be NULL
 * (= identity).  The reference's CPU branch serves one user per call
 * (custom_ops.py:1044); this entry point serves all users of the batch at once, which is
 * what the device op does.
 * k_new / v_new are token-major with user u's token t at row u*tokens_per_user + t.
 * ------------------------------------------------------------------------------------------ */
int b200attn_paged_fill_cache(void* k_cache, void* v_cache,
                              const void* k_new, const void* v_new,
                              int64_t new_token_stride,
                              const int32_t* fill_page_table, int64_t page_table_stride,
                              int page_table_width, const int32_t* batch_idx,
                              int num_users, int tokens_per_user,
                              int num_kv_heads, int head_size,
                              int block_size, int64_t num_blocks, void* stream);

/* ------------------------------------------------------------------------------------------
 * KV-cache write, slot-mapping form (what vLLM's own runners supply).
 * Replaces: write_to_kv_cache(key, value, kv_cache, slot_mapping, ...)
 *           (attention.py:671-716), re-targeted at the live cache layout above.
 * Token t goes to block slot_mapping[t] / block_size, offset slot_mapping[t] % block_size;
 * tokens with a negative slot are skipped (vLLM's padding convention).
 * ------------------------------------------------------------------------------------------ */
int b200attn_kv_scatter_slots(void* k_cache, void* v_cache,
                              const void* k_new, const void* v_new,
                              int64_t new_token_stride,
                              const int64_t* slot_mapping, int num_tokens,
                              int num_kv_heads, int head_size,
                              int block_size, int64_t num_blocks, void* stream);

/* ------------------------------------------------------------------------------------------
 * Step metadata built on the device (the producer on the left of every op above).
 * Replaces: the host loop + host-to-device copies of TTModelRunner._prepare_inputs that fill
 *           cache_position, page_table and fill_page_table
 *           (integrations/vllm_plugin/vllm_tt/model_runner.py:1722-1741, 1945-1993).
 * For row r < num_requests: cache_position = num_computed + num_scheduled - 1; page_table row =
 * block_table row; fill_page_table row = that row rolled left by num_computed / block_size,
 * first fill_page_table_width columns; slot_mapping[r, t] = block of position
 * num_computed + t times block_size plus its offset, -1 for t >= num_scheduled.  Rows beyond
 * num_requests, and rows with num_scheduled == 0, get cache_position -1 (resp. their true
 * position), an all-zero page table (the null block) and slots of -1.
 * ------------------------------------------------------------------------------------------ */
int b200attn_build_step_metadata(const int32_t* num_computed, const int32_t* num_scheduled,
                                 const int32_t* block_table, int64_t block_table_stride,
                                 int num_requests, int rows, int page_table_width,
                                 int fill_page_table_width, int tokens_per_row, int block_size,
                                 int32_t* cache_position, int32_t* page_table,
                                 int32_t* fill_page_table, int64_t* slot_mapping, void* stream);

/* ------------------------------------------------------------------------------------------
 * Rotary embedding fused with the slot-mapping KV-cache write (the caller on the left of the
 * cache write).
 * Replaces: TTRotaryEmbedding.forward(positions, query, key)
 *           (integrations/vllm_plugin/vllm_tt/layers/rotary_embedding.py:51-66, NeoX style via
 *           ApplyRotaryEmb.forward_static) followed by the KV-cache write above.
 * cos / sin are computed on the fly from positions and inv_freq in fp32 and rounded to bf16, and
 * every multiply / add of the rotation is rounded to bf16, as the reference layer computes them.
 * q and k ([num_tokens, heads*head_size] rows with the given strides) are rotated in place; the
 * rotated k and v go to slot_mapping[t] of the caches (negative slot: rotate only;
 * slot_mapping == NULL: no cache write at all).  The first rotary_dim elements of each head are
 * rotated (rotary_dim a multiple of 16, <= head_size); only is_neox_style = 1 is supported.
 * ------------------------------------------------------------------------------------------ */
int b200attn_rope_kv_scatter_slots(void* q, int64_t q_stride, void* k, int64_t k_stride,
                                   const void* v, int64_t v_stride, const int64_t* positions,
                                   const float* inv_freq, int rotary_dim, int is_neox_style,
                                   void* k_cache, void* v_cache, const int64_t* slot_mapping,
                                   int num_tokens, int num_q_heads, int num_kv_heads,
                                   int head_size, int block_size, int64_t num_blocks,
                                   void* stream);

/* ------------------------------------------------------------------------------------------
 * Paged GQA decode attention (one query token per user), split-KV with the merge of the
 * splits inside the same launch.
 * Replaces: torch.ops.tt.paged_scaled_dot_product_attention_decode with is_causal=True and
 *           cur_pos_tensor (custom_ops.py:1198-1331; call site attention.py:634-668).
 * out[u,h,:] = softmax_{j <= cur_pos[u]}(q[u,h,:] . K_u[j, h/G, :] * scale) . V_u[j, h/G, :]
 * where K_u/V_u are read through page_table[u, j / block_size].  Users with cur_pos < 0
 * (padding rows) get zeros.  q and out are [num_users, num_q_heads, head_size] with the
 * given row strides (elements).
 * num_splits: 0 = choose (b200attn_decode_auto_splits with max_context_len), at most 256; the
 * workspace must hold b200attn_decode_workspace_bytes(num_users, num_q_heads, head_size,
 * num_splits) bytes (it may be NULL when the split count in effect is 1).
 * Workspace contract: its first B200ATTN_DECODE_TICKET_BYTES bytes are arrival counters (one
 * per user and KV head; the split that arrives last merges the partials).  They must be ZERO
 * when the workspace is first used and every call leaves them zero, so zero the workspace once
 * after allocating it and again after a call that left a non-zero diagnostics word.  The rest
 * needs no initialisation.  Calls that share a workspace must not overlap on the GPU.  Batches
 * with more than B200ATTN_DECODE_TICKET_BYTES / 4 (user, KV head) pairs use a second, small
 * launch for the merge instead of the counters.
 * ------------------------------------------------------------------------------------------ */
int b200attn_paged_decode(void* out, int64_t out_row_stride,
                          const void* q, int64_t q_row_stride,
                          const void* k_cache, const void* v_cache,
                          const int32_t* page_table, int64_t page_table_stride,
                          int page_table_width, const int32_t* cur_pos,
                          int num_users, int num_q_heads, int num_kv_heads, int head_size,
                          int block_size, int64_t num_blocks, float scale,
                          int max_context_len, int num_splits,
                          void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * KV-cache element type.  The plugin maps the engine's kv_cache_dtype strings to torch dtypes
 * (attention.py:42-51: "fp8" / "fp8_e4m3" -> float8_e4m3fn) and its cache write clamps to the
 * finite range and casts (attention.py:692-700).  With B200ATTN_CACHE_FP8_E4M3 the three cache
 * writes below do the same per element -- round to nearest even, saturate at +-448, NaN stays
 * NaN, no scale factor -- into caches of one byte per element with the same
 * [num_blocks, num_kv_heads, block_size, head_size] layout; b200attn_paged_decode_ex reads them.
 * Prefill over an fp8 paged cache is not implemented (fresh-K/V prefill needs no cache). */
enum b200attn_cache_dtype {
  B200ATTN_CACHE_BF16 = 0,
  B200ATTN_CACHE_FP8_E4M3 = 1
};

int b200attn_paged_update_cache_ex(void* k_cache, void* v_cache,
                                   const void* k_new, const void* v_new,
                                   int64_t new_token_stride,
                                   const int32_t* update_indices,
                                   const int32_t* page_table, int64_t page_table_stride,
                                   int page_table_width,
                                   int num_users, int num_kv_heads, int head_size,
                                   int block_size, int64_t num_blocks, int cache_dtype,
                                   void* stream);
int b200attn_paged_fill_cache_ex(void* k_cache, void* v_cache,
                                 const void* k_new, const void* v_new,
                                 int64_t new_token_stride,
                                 const int32_t* fill_page_table, int64_t page_table_stride,
                                 int page_table_width, const int32_t* batch_idx,
                                 int num_users, int tokens_per_user,
                                 int num_kv_heads, int head_size, int block_size,
                                 int64_t num_blocks, int cache_dtype, void* stream);
int b200attn_kv_scatter_slots_ex(void* k_cache, void* v_cache,
                                 const void* k_new, const void* v_new,
                                 int64_t new_token_stride, const int64_t* slot_mapping,
                                 int num_tokens, int num_kv_heads, int head_size, int block_size,
                                 int64_t num_blocks, int cache_dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Paged GQA decode attention for callers that cannot allocate device memory.
 * No counterpart in the reference: this entry point exists for hosts of this library that
 * must not call cudaMalloc around it -- code running inside a region where allocation is
 * forbidden or would synchronise the device (a serving loop with a frozen memory pool, a
 * plugin loaded by a process that owns all device memory, a real-time path that may not take
 * the allocator lock).  It computes exactly what b200attn_paged_decode computes, with the same
 * arguments minus the workspace: the split-KV scratch lives in a fixed array inside the
 * library image, B200ATTN_STATIC_WORKSPACE_BYTES per GPU, which every GPU that loads the
 * library holds until the process exits.
 *   - num_splits = 0 picks the usual split count, lowered if needed until the scratch fits;
 *     an explicit num_splits whose scratch exceeds the array is rejected with
 *     B200ATTN_ERR_TOO_LARGE (nothing is launched).
 *   - The first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress with that device current).  Make that first call outside any
 *     stream capture.
 *   - The entry point calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - All calls on a device share the one array and it keeps the previous call's contents.
 *     The arrival counters at its start have to be zero when a call begins; the entry point
 *     clears the ones the call will use (a cudaMemsetAsync on the same stream, which allocates
 *     nothing) before it launches, the rest of the array needs no clearing (every slot that is
 *     read was written by the same call).  Two calls that overlap on the GPU -- different
 *     streams, or one stream from two threads without ordering -- race on it.  Serialise them.
 * ------------------------------------------------------------------------------------------ */
#define B200ATTN_DECODE_TICKET_BYTES 65536u
#define B200ATTN_STATIC_WORKSPACE_BYTES (16u << 20)
int b200attn_paged_decode_static(void* out, int64_t out_row_stride,
                                 const void* q, int64_t q_row_stride,
                                 const void* k_cache, const void* v_cache,
                                 const int32_t* page_table, int64_t page_table_stride,
                                 int page_table_width, const int32_t* cur_pos,
                                 int num_users, int num_q_heads, int num_kv_heads, int head_size,
                                 int block_size, int64_t num_blocks, float scale,
                                 int max_context_len, int num_splits, void* stream);

/* b200attn_paged_decode with the two optional features of the reference op's signature
 * (custom_ops.py:1198-1213: sliding_window_size, attention_sink):
 *   sliding_window > 0: user u attends only keys j with cur_pos[u] - sliding_window < j <=
 *                       cur_pos[u]; earlier pages are not read at all.
 *   sinks != NULL:      fp32 [num_q_heads]; head h's softmax gets one more column with logit
 *                       sinks[h] (in the scaled-score domain) that adds to the denominator only.
 * The reference's CPU branch ignores both arguments (custom_ops.py:1256-1312), so their parity
 * is checked against the published semantics, not against reference output.
 *   cache_dtype:        B200ATTN_CACHE_BF16, or B200ATTN_CACHE_FP8_E4M3 for caches written by the
 *                       *_ex cache writes below (head_size 128 only): K and V are then one byte
 *                       per element, unscaled, and are widened exactly inside the kernel; q, the
 *                       softmax weights and the output stay 16-bit with fp32 accumulation. */
int b200attn_paged_decode_ex(void* out, int64_t out_row_stride,
                             const void* q, int64_t q_row_stride,
                             const void* k_cache, const void* v_cache,
                             const int32_t* page_table, int64_t page_table_stride,
                             int page_table_width, const int32_t* cur_pos,
                             int num_users, int num_q_heads, int num_kv_heads, int head_size,
                             int block_size, int64_t num_blocks, float scale,
                             int sliding_window, const float* sinks, int cache_dtype,
                             int max_context_len, int num_splits,
                             void* workspace, size_t workspace_bytes, void* stream);

/* One decode step in one launch: b200attn_paged_decode_ex that first writes this step's K / V
 * rows into the caches.  Replaces the pair the plugin issues per layer and step,
 * tt.paged_update_cache for K and V followed by the paged decode op (attention.py:468-484,
 * 634-668).  k_new / v_new: [num_users, num_kv_heads, head_size] bf16 rows, new_token_stride
 * elements between users; user u's rows go to position cur_pos[u] with the addressing of
 * b200attn_paged_update_cache (update_indices = cur_pos), converted for an fp8 cache.  The CTA
 * that is about to stream the tile holding the new token writes it, fences, and then loads the
 * tile, so no second kernel and no extra pass over the cache.  wrap_negative_positions != 0 keeps
 * the reference's treatment of negative positions (torch floor division / negative column
 * index, custom_ops.py:985-998); 0 skips such rows (the slot_mapping convention: -1 = padding).
 * k_new == v_new == NULL makes it b200attn_paged_decode_ex. */
int b200attn_paged_decode_step(void* out, int64_t out_row_stride,
                               const void* q, int64_t q_row_stride,
                               void* k_cache, void* v_cache,
                               const void* k_new, const void* v_new, int64_t new_token_stride,
                               int wrap_negative_positions,
                               const int32_t* page_table, int64_t page_table_stride,
                               int page_table_width, const int32_t* cur_pos,
                               int num_users, int num_q_heads, int num_kv_heads, int head_size,
                               int block_size, int64_t num_blocks, float scale,
                               int sliding_window, const float* sinks, int cache_dtype,
                               int max_context_len, int num_splits,
                               void* workspace, size_t workspace_bytes, void* stream);

/* Split count the library would pick for a decode batch (host cost model fitted to B200
 * measurements; no device access beyond the SM count).  max_context_len <= 0 means "unknown": the page-table width bounds it. */
int b200attn_decode_auto_splits(int num_users, int num_kv_heads, int head_size,
                                int max_context_len);

/* Bytes of scratch b200attn_paged_decode needs for num_splits splits (0 when num_splits <= 1):
 * the ticket region, the fp32 partial outputs and their (max, sum) pairs. */
size_t b200attn_decode_workspace_bytes(int num_users, int num_q_heads, int head_size,
                                       int num_splits);

/* ------------------------------------------------------------------------------------------
 * Chunked prefill over an fp8 (e4m3) cache, step 1: widen the pages the batch reads.
 * Replaces: nothing of its own -- it is what lets b200attn_prefill (kv_is_paged = 1) stand in
 *           for torch.ops.tt.chunked_scaled_dot_product_attention (custom_ops.py:1334-1443) when
 *           the plugin's cache dtype is float8_e4m3fn (attention.py:42-51, 692-700).
 * For every sequence s and page slot i below ceil((q_start[s] + q_len[s]) / block_size), page
 * page_table[s, i] of both caches is copied, widened to bf16 (exact), into page s * width + i
 * of k_dst / v_dst, which must hold num_seqs * page_table_width pages of
 * [num_kv_heads, block_size, head_size] bf16 each.  Then call b200attn_prefill with k_dst /
 * v_dst as the caches, the identity page table (entry [s, i] = s * width + i) and
 * num_blocks = num_seqs * page_table_width.  Scratch and identity table are the caller's.
 * ------------------------------------------------------------------------------------------ */
int b200attn_dequant_pages_fp8(void* k_dst, void* v_dst, const void* k_cache, const void* v_cache,
                               const int32_t* page_table, int64_t page_table_stride,
                               int page_table_width, const int32_t* cu_q, const int32_t* q_start,
                               int num_seqs, int num_kv_heads, int head_size, int block_size,
                               int64_t num_blocks, void* stream);

/* ------------------------------------------------------------------------------------------
 * Causal varlen prefill / chunked-prefill attention on tcgen05 tensor cores.
 * Replaces: torch.ops.tt.scaled_dot_product_attention with is_causal=True, attn_mask=None
 *           (custom_ops.py:635-742; call site attention.py:575-598)            [kv_is_paged = 0]
 *      and: torch.ops.tt.chunked_scaled_dot_product_attention
 *           (custom_ops.py:1334-1443; call site attention.py:545-560)          [kv_is_paged = 1]
 * Sequence s owns query rows cu_q[s] .. cu_q[s+1]-1 of q/out (row strides in elements);
 * query row i of the sequence sits at absolute position q_start[s] + i and attends keys
 * 0 .. q_start[s] + i.  q_start may be NULL (= 0 for every sequence).  The reference passes
 * one chunk_start for the whole batch; per-sequence starts are a superset.
 *   kv_is_paged = 0: k_src / v_src are the fresh token-major K/V of the same tokens
 *                    (row t at t*kv_token_stride, head h at h*head_size); q_start must be
 *                    NULL or all zero; page_table is ignored.
 *   kv_is_paged = 1: k_src / v_src are the K and V caches; page_table[s, :] lists sequence
 *                    s's blocks in logical order (prefix + chunk already written).
 * cu_q_host mirrors cu_q on the host (the launch grid is sized from it).
 * The CTAs of a launch share out its work through a counter word inside the library (64 words
 * per device, handed to launches in turn and tagged per call, so launches on different streams
 * do not meet).  A launch captured into a CUDA graph keeps its word and tag: replay it as often
 * as needed, but never let two replays of the SAME captured launch run at the same time (two
 * streams replaying one graph), and read the diagnostics word (b200attn_read_error_word, which
 * also clears the counters) after a launch that reported a timeout before replaying it.
 * ------------------------------------------------------------------------------------------ */
int b200attn_prefill(void* out, int64_t out_row_stride,
                     const void* q, int64_t q_row_stride,
                     const void* k_src, const void* v_src, int kv_is_paged,
                     int64_t kv_token_stride,
                     const int32_t* page_table, int64_t page_table_stride, int page_table_width,
                     const int32_t* cu_q, const int32_t* cu_q_host,
                     const int32_t* q_start,
                     int num_seqs, int total_q, int num_q_heads, int num_kv_heads,
                     int head_size, int block_size, int64_t num_blocks, float scale,
                     void* stream);

/* b200attn_prefill with the reference op's optional sliding window
 * (custom_ops.py:635-646 `sliding_window_size`): query row at absolute position p attends
 * only keys j with p - sliding_window < j <= p (0 = full causal attention); KV tiles wholly
 * below a query tile's window are neither loaded nor multiplied.  The reference's CPU branch
 * ignores the argument (custom_ops.py:717-727), so this is checked against the published
 * semantics, not against reference output. */
int b200attn_prefill_ex(void* out, int64_t out_row_stride,
                        const void* q, int64_t q_row_stride,
                        const void* k_src, const void* v_src, int kv_is_paged,
                        int64_t kv_token_stride,
                        const int32_t* page_table, int64_t page_table_stride,
                        int page_table_width,
                        const int32_t* cu_q, const int32_t* cu_q_host,
                        const int32_t* q_start,
                        int num_seqs, int total_q, int num_q_heads, int num_kv_heads,
                        int head_size, int block_size, int64_t num_blocks, float scale,
                        int sliding_window, void* stream);

/* ------------------------------------------------------------------------------------------
 * Row-parallel linear layer with the tensor-parallel all-reduce fused into its epilogue.
 * Replaces: a row-sharded linear layer whose partial sums are all-reduced -- the reference marks
 * the weight sharded along its input dimension and leaves the all-reduce to the compiler
 * (vllm_tt/vllm_distributed_utils.py:356-363, partition_row_parallel_linear; it is the o_proj /
 * down_proj collective of the end-to-end model), vLLM's RowParallelLinear.forward runs a GEMM and
 * then tensor_model_parallel_all_reduce.  Here one launch per rank computes
 *     out[t, n] = sum over ranks r of sum_k x_r[t, k] * w_r[n, k]       (bf16 partials, fp32 sum)
 * for num_tokens <= 128: tcgen05 GEMM tiles (clusters split K) whose epilogue pushes the rank's
 * bf16-rounded partial sums into every peer's staging area as 8-byte units that carry their own
 * arrival flag (plain peer stores), waits (bounded) for the peers' units and adds all ranks'
 * partials in rank order, so all ranks return identical bits (bf16 partials, fp32 sum: what
 * vLLM's all-reduce of the GEMM outputs computes).
 *
 * Communicator: one device buffer per rank, b200attn_comm_bytes(world, max_tokens, max_n) bytes,
 * zero-initialised, mapped into every rank's process.  b200attn_comm_alloc / _export / _import /
 * _close / _free wrap cudaMalloc and the CUDA IPC handle calls so that a host without its own
 * CUDA runtime binding can set it up: each rank allocates, exports 64 handle bytes, exchanges
 * them over any channel, imports its peers' handles.  comm_bufs[r] is rank r's buffer as mapped
 * in the calling process (own buffer at [rank]); with world == 1 it may be NULL and the call is
 * a plain GEMM.
 *
 * reduce_mode: 1 = one shot (every rank sends its partial to every peer and adds all of them up),
 * 2 = two shots (each tile share has an owner rank that adds the partials and sends the result
 * back, so a rank's NVLink traffic does not grow with the number of ranks), 0 = one shot for two
 * ranks, two shots beyond.
 *
 * All ranks must issue the same sequence of calls with the same shapes on one stream each.  The
 * call is asynchronous and allocation-free.  A peer that does not arrive within peer_timeout_ns
 * (0 = 1 s) makes the kernel give up: the diagnostics word becomes 1, the communicator buffer of
 * this rank is marked out of step, the output of that call is unspecified, later calls through
 * the same communicator only run their local GEMM, and the communicator must be rebuilt
 * (collectively; a fresh buffer starts clean).  n_total, k_local and the strides must be multiples of 8;
 * n_total / 32 (or / 64) must not exceed the SM count (every CTA has to be resident). */
size_t b200attn_comm_bytes(int world, int max_tokens, int max_n);
/* The launch geometry b200attn_rowlinear_allreduce picks on the current device: token rows of
 * the MMA (32 / 64 / 128) and K splits (CTAs per cluster).  Staging units of one call are laid
 * out by these two numbers; exposed for tests and tools that fill or read the staging area. */
int b200attn_rowlinear_plan(int num_tokens, int n_total, int k_local, int* token_rows,
                            int* k_splits);
int b200attn_comm_alloc(size_t bytes, void** dev_ptr);
int b200attn_comm_free(void* dev_ptr);
int b200attn_comm_export(const void* dev_ptr, unsigned char* handle64);
int b200attn_comm_import(const unsigned char* handle64, void** peer_ptr);
int b200attn_comm_close(void* peer_ptr);
int b200attn_rowlinear_allreduce(void* out, int64_t out_row_stride,
                                 const void* x, int64_t x_row_stride,
                                 const void* w, int64_t w_row_stride,
                                 int num_tokens, int n_total, int k_local,
                                 int rank, int world, void* const* comm_bufs,
                                 int max_tokens, int max_n, int reduce_mode,
                                 uint64_t peer_timeout_ns, void* stream);

/* Copies the device diagnostics word of the current device to *out_host (synchronises the
 * stream) and clears it.  0 = no kernel reported a problem since the last read. */
int b200attn_read_error_word(int32_t* out_host, void* stream);

/* Queues an asynchronous copy of the diagnostics word to *out_pinned_host (page-locked host
 * memory the caller owns) on `stream`; nothing is cleared and nothing is waited for.  A serving
 * loop calls it once per step and looks at the value a later step finds there, so a kernel that
 * gave up on a wait is noticed within a step or two without a synchronisation of its own.
 * No counterpart in the reference (its runtime reports device errors through PJRT). */
int b200attn_peek_error_word_async(int32_t* out_pinned_host, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H_ */
