/*
 * echokv_b200 -- C ABI of the B200 (sm_100a) kernels for paged attention over a
 * per-layer mixed-precision (INT8 / INT4 / INT2) KV cache.
 *
 * Every entry point replaces one Python-level kernel launcher of the reference
 * plugin (paths below are relative to the reference project).  All device entry
 * points are asynchronous on `stream` (a cudaStream_t passed as void*), never
 * synchronise with the host, never allocate, and return 0 on success or a
 * negative ECHOKV_E_* code (the message is available from echokv_last_error()).
 * Pointers are plain device pointers; strides are in ELEMENTS of the pointed-to
 * type unless a name ends in _bytes.  Element types are given as ECHOKV_DT_*.
 *
 * Page byte layout (echokv_vllm/tiered_cache.py:13-25, :120-147), one page per
 * vLLM block of `block_size` tokens:
 *   [0, block_size)          header: [0] tier (0 never opened, else 2/4/8),
 *                            [1] bitmask of K groups sealed early,
 *                            [4:16] three int32 ids of extra pool chunks
 *   v_scale, v_min           fp16 [block_size, H, D / v_group] each
 *   k_scale, k_min           fp16 [block_size / k_group, H, D] each
 *   data                     mem_bits / 2 chunks of block_size*H*D/2 bytes;
 *                            token rows are [K codes of all heads | V codes of
 *                            all heads]; chunk j holds tokens [j*tpc, (j+1)*tpc),
 *                            tpc = 2*block_size/bits; chunk 0 is in the block's
 *                            own page, chunk j>0 is pool chunk id table[j-1]
 *                            (page = id / chunks_per_page, slot = id % ...).
 */
#ifndef ECHOKV_B200_H
#define ECHOKV_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ECHOKV_ABI_VERSION 1

enum {
  ECHOKV_OK = 0,
  ECHOKV_E_LAYOUT = -1,      /* layout rejected (same rules as TieredLayout.__post_init__) */
  ECHOKV_E_UNSUPPORTED = -2, /* shape / dtype the kernels are not built for */
  ECHOKV_E_ARGUMENT = -3,    /* null pointer, negative size, misaligned stride */
  ECHOKV_E_CUDA = -4         /* a CUDA runtime call failed */
};

enum { ECHOKV_DT_F32 = 0, ECHOKV_DT_F16 = 1, ECHOKV_DT_BF16 = 2 };

/* TieredLayout (echokv_vllm/tiered_cache.py:76-97). */
typedef struct echokv_layout {
  int32_t num_kv_heads;
  int32_t head_size;
  int32_t block_size;
  int32_t mem_bits; /* 2, 4, 6 or 8 */
  int32_t k_group;
  int32_t v_group;
} echokv_layout;

/* Derived byte offsets (TieredLayout.offsets / per_token_bytes, tiered_cache.py:99-147). */
typedef struct echokv_layout_info {
  int64_t o_v_scale, o_v_min, o_k_scale, o_k_min, o_data, page_bytes;
  int64_t chunk_bytes, per_token_bytes;
  int32_t chunks_per_page, k_groups_per_block, v_groups, reserved;
} echokv_layout_info;

/* A layer's slice of the paged pool: uint8 [num_blocks, >= page_bytes], row stride
 * `page_stride_bytes` (16-byte aligned; may exceed the page for layer-interleaved
 * pools) -- TieredKVCache.__init__ (tiered_cache.py:157-171). */
typedef struct echokv_pages {
  void* base;
  int64_t page_stride_bytes;
  int64_t num_blocks;
  int32_t max_tier; /* optional: upper bound of the tier of any block in this pool (2/4/8), 0 = unknown.
                       Informational only: no kernel depends on it (the decode kernel's shared-memory
                       stages have one size for every tier) */
  int32_t reserved;
} echokv_pages;

/* Residual buffer [slots + 1, k_group, H, D] in the model dtype
 * (backend.py:535-537) and the shared block -> slot map (write_plan.py:255-256). */
typedef struct echokv_residual {
  void* base;
  int32_t dtype;
  int32_t reserved;
  int64_t s_slot, s_pos, s_head;  /* element strides; the last dim is contiguous */
  const int64_t* block_res;       /* [num_blocks] residual slot of the block's open K group, -1 none */
  const int64_t* res_group;       /* [slots + 1] which K group a slot holds */
} echokv_residual;

int echokv_abi_version(void);
const char* echokv_last_error(void);

/* Host only. Validates like TieredLayout.__post_init__ and fills `out`. */
int echokv_layout_describe(const echokv_layout* layout, echokv_layout_info* out);

/* header[blocks[i]] = headers[i] (16 bytes each) -- TieredKVCache.write_headers
 * (tiered_cache.py:305-307). `blocks` int64 [n], `headers` uint8 [n,16], both on the device. */
int echokv_write_headers(const echokv_pages* pages, const int64_t* blocks, const uint8_t* headers,
                         int64_t n, void* stream);

/* dst[idx[i]] = val[i] -- SharedState.apply_res_map (write_plan.py:266-271). */
int echokv_scatter_i64(int64_t* dst, const int64_t* idx, const int64_t* val, int64_t n, void* stream);

/* Quantize-on-write of a step's token rows -- write_tokens / _write_tokens_kernel
 * (kernels/write.py:29-36, :171-229).  key/value [n_rows, H, D] of `kv_dtype`
 * (row stride s0, head stride s1, unit stride in D).  `tok` int64 [4, >= n_rows] with
 * row stride tok_s0: slot (-1 skip), residual slot or -1, sealed flag, K_ref ring row or -1.
 * `kref` float32 [W, H, D] or NULL. */
int echokv_write_tokens(const echokv_layout* layout, const echokv_pages* pages,
                        const void* key, int64_t k_s0, int64_t k_s1,
                        const void* value, int64_t v_s0, int64_t v_s1, int32_t kv_dtype,
                        const int64_t* tok, int64_t tok_s0, const echokv_residual* residual,
                        float* kref, int64_t kref_s0, int64_t kref_s1,
                        int64_t n_rows, void* stream);

/* Per-channel quantization of completed K groups -- finalize_k / _finalize_k_kernel
 * (kernels/write.py:39-50, :231-287).  `fin` int64 [>= n_launch, 3 + k_group]:
 * block, group, residual slot or -1, then the key row of each position or -1 (take it
 * from the residual).  Rows >= *fin_count are skipped (graph-captured full-grid launch). */
int echokv_finalize_k(const echokv_layout* layout, const echokv_pages* pages,
                      const void* key, int64_t k_s0, int64_t k_s1, int32_t kv_dtype,
                      const int64_t* fin, const int64_t* fin_count,
                      const echokv_residual* residual, int64_t n_launch, void* stream);

/* Seal an evicted residual slot: quantize its first `fill` keys against their own
 * stats into group `group` of `block` at `bits`, set header byte 1 to `sealed_mask`
 * -- TieredKVCache._seal (tiered_cache.py:379-394). */
int echokv_seal_group(const echokv_layout* layout, const echokv_pages* pages,
                      const echokv_residual* residual, int64_t slot, int64_t block, int32_t group,
                      int32_t fill, int32_t bits, int32_t sealed_mask, void* stream);

/* Host-side planner of a step's KV writes (no device work) -- WritePlanner (write_plan.py:77-240): the residual-slot
 * allocator, the K_ref ring cursor and `plan`, with the same decisions, slot numbering and output order, so its
 * plans are interchangeable with the Python planner's.  `slots` int64 [n_rows] (-1 = row not stored).  Outputs are
 * caller-allocated int64 arrays: tok [4, n_rows] (slot, residual slot, sealed, K_ref row), fin [n_rows, 3 + k_group],
 * evictions [n_rows, 4] (slot, block, group, fill), opened / touched / touched_fill / touched_count [n_rows],
 * map_block / map_value / grp_slot / grp_value [4 * n_rows + 8] (the ordered residual-map updates), counts [8] =
 * n_fin, n_evictions, n_opened, n_touched, n_map_block, n_map_group, step.  echokv_planner_get: 0 free slots,
 * 1 K_ref cursor, 2 K_ref fill, 3 step, 4 slots in all, 5 live slots. */
void* echokv_planner_create(int32_t block_size, int32_t k_group, int32_t residual_slots, int32_t kref_window);
void echokv_planner_destroy(void* planner);
int64_t echokv_planner_get(void* planner, int32_t what);
int64_t echokv_planner_sealed_mask(void* planner, int64_t block, int64_t otherwise);
int echokv_planner_plan(void* planner, const int64_t* slots, int64_t n_rows, int64_t* tok, int64_t* fin,
                        int64_t* evictions, int64_t* opened, int64_t* touched, int64_t* touched_fill,
                        int64_t* touched_count, int64_t* map_block, int64_t* map_value, int64_t* grp_slot,
                        int64_t* grp_value, int64_t* counts);

/* One layer's writes of a step in ONE launch: echokv_finalize_k (n_fin_launch CTAs masked by *fin_count),
 * echokv_write_tokens and echokv_gather_rows (the canary's query rows: stash_dst[i] = stash_src[stash_rows[i]],
 * skipped when stash_src is NULL or stash_n is 0) with the same arguments and the same stored bytes as the three
 * calls made in that order.  The reference launches them one after the other (tiered_cache.py:415-432,
 * backend.py:632-635); the group pass must come first there because a residual slot a completing group gives up
 * may be taken by a new group in the same step.  In the single launch the CTA of such a token row leaves the key
 * to the CTA of the completing group, which stores it after its own last read of the slot.  Steps of more than
 * 1,024 rows, and layouts or stash rows the single kernel does not take, run as the three launches. */
int echokv_write_step(const echokv_layout* layout, const echokv_pages* pages,
                      const void* key, int64_t k_s0, int64_t k_s1,
                      const void* value, int64_t v_s0, int64_t v_s1, int32_t kv_dtype,
                      const int64_t* tok, int64_t tok_s0, const echokv_residual* residual,
                      float* kref, int64_t kref_s0, int64_t kref_s1, int64_t n_rows,
                      const int64_t* fin, const int64_t* fin_count, int64_t n_fin_launch,
                      const void* stash_src, int64_t stash_src_row_stride_bytes, const int64_t* stash_rows,
                      int64_t stash_n, void* stash_dst, int64_t stash_row_bytes, void* stream);

/* Requantize full INT4/INT8 blocks to INT2 in place -- TieredKVCache._demote_lru
 * (tiered_cache.py:309-346).  `victims` int64 [n] on the device; `scratch` holds the blocks'
 * dequantized contents between the read and the rewrite (echokv_demote_scratch_bytes). */
int64_t echokv_demote_scratch_bytes(const echokv_layout* layout, int64_t n);
int echokv_demote_blocks(const echokv_layout* layout, const echokv_pages* pages,
                         const echokv_residual* residual, const int64_t* victims, int64_t n,
                         void* scratch, int64_t scratch_bytes, void* stream);

/* Dequantized K and V, float32 [n, H, D], of tokens (blk[i], off[i]) -- TieredKVCache.gather
 * (tiered_cache.py:451-478). Blocks never opened give zeros. */
int echokv_gather(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                  const int64_t* blk, const int64_t* off, int64_t n, float* k_out, float* v_out, void* stream);

/* Bytes of scratch echokv_decode needs: 256 bytes of work-queue state at the start (the counter
 * persistent CTAs claim work items from), then the split partials, acc float32
 * [S, Hq, num_splits, D] and (m, l) float32 [S, Hq, num_splits, 2] (kernels/decode.py:306-307
 * allocates the same two tensors per call), rounded up to 16 bytes.  echokv_decode zeroes the state
 * itself with a memset node on `stream`; echokv_decode_ex expects it zero (see there). */
int64_t echokv_decode_scratch_bytes(int64_t num_seqs, int32_t num_q_heads, int32_t head_size, int32_t num_splits);

/* Split-K paged decode attention + merge -- decode_attention / _decode_triton
 * (kernels/decode.py:44-92, :283-345).  Sequence i uses query row q_rows[i], block-table
 * row bt_rows[i], cache length lens[i] (0 = CUDA-graph padding: its output row is left
 * untouched) and writes out[q_rows[i]].  q_rows / bt_rows may be NULL (identity).
 * Split rule (decode.py:166-172): n_blocks = ceil(len / BS); bps = max(blocks_per_split,
 * ceil(n_blocks / num_splits)); split s covers blocks [s*bps, min((s+1)*bps, n_blocks)). */
int echokv_decode(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                  const void* query, int64_t q_s0, int64_t q_s1, int32_t q_dtype, const int64_t* q_rows,
                  const int32_t* block_table, int64_t bt_s0, const int64_t* bt_rows, const int64_t* lens,
                  void* scratch, int64_t scratch_bytes,
                  void* out, int64_t o_s0, int64_t o_s1, int32_t out_dtype,
                  float softmax_scale, int32_t num_splits, int32_t blocks_per_split,
                  int64_t num_seqs, int32_t num_q_heads, void* stream);

/* echokv_decode with the blocks per split also given at run time: when `blocks_per_split_dev` is not NULL
 * the kernels read one int32 from that device address and use max(blocks_per_split, that value) in the split
 * rule above.  A CUDA graph bakes the by-value arguments of a captured call; a host that replays such a
 * graph writes the value for the coming step into that word (on the same stream) and so keeps choosing the
 * split size per step.  The reference fixes BLOCKS_PER_SPLIT per process (kernels/decode.py:41); for a given
 * value the results are the same bits as echokv_decode's with blocks_per_split = max(both).
 * Unlike echokv_decode this call issues no memset: the first 256 bytes of `scratch` must be zero before the
 * first call that uses it, and every call leaves them zero (the merge kernel resets the counter), so the
 * split kernel follows the kernel before it on the stream directly and all three kernels of a layer's step
 * (write_step, split, merge) launch as programmatic dependents of one another. */
int echokv_decode_ex(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                     const void* query, int64_t q_s0, int64_t q_s1, int32_t q_dtype, const int64_t* q_rows,
                     const int32_t* block_table, int64_t bt_s0, const int64_t* bt_rows, const int64_t* lens,
                     void* scratch, int64_t scratch_bytes,
                     void* out, int64_t o_s0, int64_t o_s1, int32_t out_dtype,
                     float softmax_scale, int32_t num_splits, int32_t blocks_per_split,
                     const int32_t* blocks_per_split_dev, int64_t num_seqs, int32_t num_q_heads, void* stream);

/* How many work items (sequence, split) the split kernel works on at the same time on the current device for
 * this layout and number of query heads, or 0 when the shape takes the generic kernel (one CTA per item and KV
 * head).  A host that picks the split size per step sizes the splits so that the items fill this many slots
 * in whole waves.  No counterpart in the reference (Triton sizes its grid from the item count). */
int32_t echokv_decode_parallelism(const echokv_layout* layout, int32_t num_q_heads);

/* echokv_decode for callers that cannot allocate scratch (it has no counterpart in the reference,
 * which allocates its split buffers with torch on every call).  Meant for hosts that are not
 * allowed to allocate device memory where they call this: a plugin running inside another
 * framework's frozen memory pool, or a plain C host without a CUDA allocator of its own.  The
 * split partials go to a fixed 8 MiB array inside the library (each GPU that loads the library
 * holds those 8 MiB until the process exits), so the call is rejected with ECHOKV_E_UNSUPPORTED when
 * echokv_decode_scratch_bytes(num_seqs, num_q_heads, head_size, num_splits) exceeds
 * echokv_decode_static_scratch_bytes().  It calls no allocating routine.  The first call on a device
 * looks up the array's device address (with that device current); make that first call outside
 * any stream capture.  All calls on a device share the one array: it keeps the previous call's
 * partials (nothing in it needs to start at zero, every value the merge reads is written first by
 * the same call), and two calls whose kernels overlap on the GPU (different streams) race on it. */
int64_t echokv_decode_static_scratch_bytes(void);
int echokv_decode_static(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                         const void* query, int64_t q_s0, int64_t q_s1, int32_t q_dtype, const int64_t* q_rows,
                         const int32_t* block_table, int64_t bt_s0, const int64_t* bt_rows, const int64_t* lens,
                         void* out, int64_t o_s0, int64_t o_s1, int32_t out_dtype,
                         float softmax_scale, int32_t num_splits, int32_t blocks_per_split,
                         int64_t num_seqs, int32_t num_q_heads, void* stream);

/* Kernel selection of echokv_decode: 0 (default) picks the tensor-core kernel when the shape fits
 * (head_size 128, v_group 32, 1/2/4/8 KV heads, <= 8 query heads per KV head, block_size and k_group
 * multiples of 16) and the generic CUDA-core kernel otherwise; 1 always takes the generic kernel.  Returns the previous setting.
 * No counterpart in the reference (its Triton autotuner plays this role, kernels/decode.py:265-280). */
int echokv_set_decode_path(int path);

/* Timing hook: while set, every echokv_decode call that takes the tensor-core kernel records the CUDA
 * events `before` / `after` (cudaEvent_t) on its stream right around the split kernel (after the counter
 * memset, before the merge), so a benchmark can time that kernel alone with events on the launching
 * stream.  Pass two null pointers to clear.  Process-wide, not thread-safe, not for use during stream
 * capture.  No counterpart in the reference. */
int echokv_set_decode_events(void* before, void* after);

/* Dequantize whole contexts into dense [total_ctx, H, D] K and V of `out_dtype`
 * -- dequant_dense / _dequant_kernel (kernels/prefill.py:90-115, :329-369).
 * `work` int32 [n_work, 4]: request (block-table row), block index, dense row of the
 * block's first token, context length. */
int echokv_dequant_dense(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                         const int32_t* work, int64_t n_work, const int32_t* block_table, int64_t bt_s0,
                         void* k_out, void* v_out, int64_t out_s0, int64_t out_s1, int32_t out_dtype, void* stream);

/* Chunked-prefill attention over dense contexts: the attention step of the dense path of
 * prefill_attention (kernels/prefill.py:118-167; the reference calls a flash-attention library
 * there, :145-153; oracle :210-236).  k_dense / v_dense [total_ctx, H, D] are what
 * echokv_dequant_dense wrote, in the query's dtype (float16 or bfloat16).  `chunks` int32
 * [n_chunks, 4] (16-byte aligned): q_start, q_end, ctx, dense row of the context's first key.
 * Query i of a chunk of nq sees keys 0 .. ctx - nq + i.  query/out [T, Hq, D]; head_size 64 or 128.
 * `total_ctx` is the number of rows of k_dense / v_dense; every one of them must hold finite values
 * (key tiles are fetched whole, rows past a context's end are masked, not skipped).  0 = unknown:
 * the kernels then never touch a row outside the chunks' contexts. */
int echokv_prefill(const void* query, int64_t q_s0, int64_t q_s1, const void* k_dense, const void* v_dense,
                   int64_t kv_s0, int64_t kv_s1, int64_t total_ctx, int32_t dtype, const int32_t* chunks,
                   int64_t n_chunks, int32_t max_chunk_len, void* out, int64_t o_s0, int64_t o_s1, int32_t out_dtype,
                   float softmax_scale, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_size, void* stream);

/* dst row i = src row rows[i] for n rows of row_bytes bytes (rows 16-byte aligned, a multiple of 16
 * bytes long): the copy of the canary's query rows, torch.index_select(query, 0, canary_rows, out=stash)
 * in EchoKVAttentionImpl.forward (backend.py:632-634).  `rows` int64 [n] on the device. */
int echokv_gather_rows(const void* src, int64_t src_row_stride_bytes, const int64_t* rows, int64_t n, void* dst,
                       int64_t row_bytes, void* stream);

/* Kernel selection of echokv_prefill: 0 (default) takes the tcgen05 / TMEM kernel when the shape fits
 * (head size 128) and the mma.sync kernel otherwise; 1 always takes the mma.sync kernel; 2 takes the
 * tcgen05 kernel without the overlap of tensor work and softmax (two CTAs per SM); 3 takes the
 * overlapped tcgen05 kernel with the key / value tiles copied by its row threads instead of tensor-map
 * copies (what 0 does when total_ctx is unknown); 4 keeps 64-key tiles where 0 would take the
 * 128-key-tile kernel (chunks of more than 128 rows).  Returns the previous setting.  No counterpart in the
 * reference (it calls a flash-attention library there). */
int echokv_set_prefill_path(int path);

/* Every wait inside the kernels (on an mbarrier or a lock) gives up after a fixed number of polls and
 * raises a status word on the device instead of hanging; the output of that launch is then undefined.
 * Synchronizes the device and returns the words of the current device: bit 0 = a wait of the decode
 * kernel ran out, bit 1 = reserved (always 0), bit 2 = a wait of the prefill kernel ran out; negative on a CUDA error.  `clear` != 0 resets them.  No counterpart in
 * the reference. */
int echokv_kernel_status(int clear);

/* How long a wait inside the tensor-core decode kernel may last before it gives up (nanoseconds; <= 0 restores the
 * default of 2 s), and a test hook: with `idle_producer` != 0 the kernel's producer warps stage nothing, so every
 * consumer's first wait runs out, the kernel returns normally with no copy in flight, its output is undefined and
 * echokv_kernel_status reports bit 0.  Process-wide; meant for tests of the give-up path.  No counterpart in the
 * reference. */
int echokv_set_decode_wait_limit(int64_t limit_ns, int idle_producer);

/* Canary attention-KL estimator, batched over layers -- canary_kl (canary.py:59-89).
 * query [L, nq, Hq, D] of q_dtype, kref float32 [L, W, H, D] oldest key first (ring
 * already unrolled: row (ring_pos + i) % W when ring_fill == W).  Scores the last
 * floor(fill / k_group) * k_group keys at 2, 4 and 8 bits; out float32 [L, 3]. */
int echokv_canary_kl(const void* query, int32_t q_dtype, int64_t q_sl, int64_t q_sq, int64_t q_sh,
                     const float* kref, int64_t k_sl, int64_t k_sw, int64_t k_sh,
                     int32_t ring_pos, int32_t ring_fill, int32_t window,
                     int32_t num_layers, int32_t nq, int32_t num_q_heads, int32_t num_kv_heads,
                     int32_t head_size, int32_t k_group, float softmax_scale, float* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ECHOKV_B200_H */
