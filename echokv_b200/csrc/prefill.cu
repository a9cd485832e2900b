// Chunked-prefill attention over the tiered store.
#include "common.cuh"

using namespace echokv;

extern "C" {

int echokv_prefill(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                   const void* query, int64_t q_s0, int64_t q_s1, int32_t q_dtype, const int32_t* chunks,
                   int64_t n_chunks, int32_t max_chunk_len, const int32_t* block_table, int64_t bt_s0, void* out,
                   int64_t o_s0, int64_t o_s1, int32_t out_dtype, float softmax_scale, int32_t num_q_heads,
                   void* stream) {
  return set_error(ECHOKV_E_UNSUPPORTED, "prefill: not built yet");
}

int echokv_canary_kl(const void* query, int32_t q_dtype, int64_t q_sl, int64_t q_sq, int64_t q_sh, const float* kref,
                     int64_t k_sl, int64_t k_sw, int64_t k_sh, int32_t ring_pos, int32_t ring_fill, int32_t window,
                     int32_t num_layers, int32_t nq, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_size,
                     int32_t k_group, float softmax_scale, float* out, void* stream) {
  return set_error(ECHOKV_E_UNSUPPORTED, "canary_kl: not built yet");
}

}  // extern "C"
