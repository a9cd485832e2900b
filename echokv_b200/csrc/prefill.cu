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

}  // extern "C"
