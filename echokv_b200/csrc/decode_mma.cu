// Tensor-core split-K paged decode attention (selected by echokv_decode when the shape fits).
#include "decode_generic.cuh"

namespace echokv {

int launch_decode_mma(const LayoutDev& L, const ResidualDev& R, const uint8_t* pages, const DecodeArgs& A,
                      int64_t num_seqs, cudaStream_t st, bool* handled) {
  (void)L; (void)R; (void)pages; (void)A; (void)num_seqs; (void)st;
  *handled = false;
  return ECHOKV_OK;
}

}  // namespace echokv
