// C ABI of split-K paged decode attention: argument checks and kernel selection.
#include "decode_generic.cuh"

using namespace echokv;

namespace echokv {
int launch_decode_mma(const LayoutDev& L, const ResidualDev& R, const uint8_t* pages, const DecodeArgs& A,
                      int64_t num_seqs, int* counter, bool zero_counter, int* status, cudaStream_t st, bool* handled);
int decode_mma_teams(int H, int D, int VG, int KG, int BS, int gqa);
int decode_status_take(bool clear);
int prefill_status_take(bool clear);

// out[q_rows[seq], head] = splits merged in split order (kernels/decode.py:226-262).  One CTA per
// (sequence, query head): the log-sum-exp weights of the used splits are computed once into shared
// memory, then thread d sums channel d over the splits with the loads of a batch of splits in
// flight together.
constexpr int MERGE_MAX_SPLITS = 64;
__global__ void decode_merge_kernel(DecodeArgs A, int BS, int D) {
  __shared__ float wgt[MERGE_MAX_SPLITS], den[MERGE_MAX_SPLITS];
  __shared__ float red[2];
  const int seq = blockIdx.x, head = blockIdx.y;
  pdl_launch_dependents();
  pdl_wait();  // the split kernel has completed
  if (seq == 0 && head == 0 && threadIdx.x == 0) A.state[0] = 0;  // its item counter, for the next call
  const int64_t seq_len = A.lens[seq];
  if (seq_len == 0) return;  // CUDA-graph padding: leave the row alone
  const int n_blocks = (int)((seq_len + BS - 1) / BS);
  const int bps = max(bps_floor(A), (n_blocks + A.num_splits - 1) / A.num_splits);
  const int used = (n_blocks + bps - 1) / bps;
  const int64_t base = ((int64_t)seq * A.Hq + head) * A.num_splits;
  const int64_t o_row = A.q_rows ? A.q_rows[seq] : seq;
  if (used <= MERGE_MAX_SPLITS) {
    if (threadIdx.x < 32) {  // warp 0: maximum, weights and the denominator (summed in split order)
      float2 ml[MERGE_MAX_SPLITS / 32];
      float m = -INFINITY;
#pragma unroll
      for (int k = 0; k < MERGE_MAX_SPLITS / 32; ++k) {
        const int s = threadIdx.x + 32 * k;
        ml[k] = s < used ? *reinterpret_cast<const float2*>(A.ml + (base + s) * 2) : make_float2(-INFINITY, 0.f);
        m = fmaxf(m, ml[k].x);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
#pragma unroll
      for (int k = 0; k < MERGE_MAX_SPLITS / 32; ++k) {
        const int s = threadIdx.x + 32 * k;
        if (s < used) {
          const float w = exp2f(ml[k].x - m);
          wgt[s] = w;
          den[s] = ml[k].y * w;
        }
      }
      __syncwarp();
      if (threadIdx.x == 0) {
        float lt = 0.f;
        for (int s = 0; s < used; ++s) lt += den[s];
        red[0] = lt;
      }
    }
    // every thread has the loads of its channel in flight while warp 0 works out the weights
    constexpr int BATCH = 32;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      const float* src = A.acc + base * D + d;
      float x[BATCH];
#pragma unroll
      for (int k = 0; k < BATCH; ++k) x[k] = k < used ? src[(int64_t)k * D] : 0.f;
      __syncthreads();  // weights and denominator are ready (uniform: every thread of the CTA has a channel when D >= blockDim)
      float a = 0.f;
#pragma unroll
      for (int k = 0; k < BATCH; ++k) a += k < used ? x[k] * wgt[k] : 0.f;
      for (int s = BATCH; s < used; ++s) a += src[(int64_t)s * D] * wgt[s];
      st_dt(A.out, A.out_dt, o_row * A.o_s0 + (int64_t)head * A.o_s1 + d, a / red[0]);
    }
    return;
  }
  float mt = -INFINITY;
  for (int s = 0; s < used; ++s) mt = fmaxf(mt, A.ml[(base + s) * 2]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f, lt = 0.f;
    for (int s = 0; s < used; ++s) {
      const float w = exp2f(A.ml[(base + s) * 2] - mt);
      a += A.acc[(base + s) * D + d] * w;
      lt += A.ml[(base + s) * 2 + 1] * w;
    }
    st_dt(A.out, A.out_dt, o_row * A.o_s0 + (int64_t)head * A.o_s1 + d, a / lt);
  }
}

}  // namespace echokv

template <int GQ>
static int launch_generic_gq(const LayoutDev& L, const ResidualDev& R, const uint8_t* pages, const DecodeArgs& A,
                             dim3 grid, cudaStream_t st) {
  switch (L.D) {
    case 64: decode_generic_kernel<GQ, 2><<<grid, DG_WARPS * 32, 0, st>>>(L, R, pages, A); break;
    case 128: decode_generic_kernel<GQ, 4><<<grid, DG_WARPS * 32, 0, st>>>(L, R, pages, A); break;
    case 256:
      if constexpr (GQ <= 8) {
        decode_generic_kernel<GQ, 8><<<grid, DG_WARPS * 32, 0, st>>>(L, R, pages, A);
        break;
      } else {
        return set_error(ECHOKV_E_UNSUPPORTED, "decode: head_size 256 supports at most 8 query heads per KV head");
      }
    default: return set_error(ECHOKV_E_UNSUPPORTED, "decode: head_size %d is not one of 64/128/256", L.D);
  }
  return ECHOKV_OK;
}

extern "C" {

int64_t echokv_decode_scratch_bytes(int64_t num_seqs, int32_t num_q_heads, int32_t head_size, int32_t num_splits) {
  if (num_seqs <= 0 || num_q_heads <= 0 || head_size <= 0 || num_splits <= 0) return 0;
  // 256 bytes of work-queue state, then the split partials (accumulators + running max / sum)
  const int64_t partials = num_seqs * num_q_heads * (int64_t)num_splits * (head_size + 2) * (int64_t)sizeof(float);
  return (partials + 15) / 16 * 16 + 256;
}

static int decode_impl(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                       const void* query, int64_t q_s0, int64_t q_s1, int32_t q_dtype, const int64_t* q_rows,
                       const int32_t* block_table, int64_t bt_s0, const int64_t* bt_rows, const int64_t* lens,
                       void* scratch, int64_t scratch_bytes, void* out, int64_t o_s0, int64_t o_s1, int32_t out_dtype,
                       float softmax_scale, int32_t num_splits, int32_t blocks_per_split,
                       const int32_t* blocks_per_split_dev, bool zero_state, int64_t num_seqs, int32_t num_q_heads,
                       void* stream) {
  if (num_seqs <= 0) return ECHOKV_OK;
  LayoutDev L;
  ResidualDev R;
  int rc = make_layout(layout, pages, &L);
  if (rc) return rc;
  rc = make_residual(residual, &R);
  if (rc) return rc;
  if (!query || !block_table || !lens || !scratch || !out) return set_error(ECHOKV_E_ARGUMENT, "decode: null pointer");
  if (num_splits < 1 || blocks_per_split < 1) return set_error(ECHOKV_E_ARGUMENT, "decode: num_splits and blocks_per_split must be >= 1");
  if (num_q_heads % L.H) return set_error(ECHOKV_E_ARGUMENT, "decode: %d query heads not a multiple of %d KV heads", num_q_heads, L.H);
  if (q_dtype < 0 || q_dtype > 2 || out_dtype < 0 || out_dtype > 2) return set_error(ECHOKV_E_ARGUMENT, "decode: bad dtype");
  if (scratch_bytes < echokv_decode_scratch_bytes(num_seqs, num_q_heads, L.D, num_splits) ||
      (reinterpret_cast<uintptr_t>(scratch) & 15))
    return set_error(ECHOKV_E_ARGUMENT, "decode: scratch too small (%lld bytes) or misaligned", (long long)scratch_bytes);
  const int gqa = num_q_heads / L.H;
  if (gqa > 16) return set_error(ECHOKV_E_UNSUPPORTED, "decode: %d query heads per KV head (max 16)", gqa);

  DecodeArgs A;
  A.q = query; A.q_s0 = q_s0; A.q_s1 = q_s1; A.q_dt = q_dtype; A.q_rows = q_rows;
  A.bt = block_table; A.bt_s0 = bt_s0; A.bt_rows = bt_rows; A.lens = lens;
  // scratch = [256 bytes of work-queue state][split partials: accumulators, then running max / sum]
  A.state = reinterpret_cast<int*>(scratch);
  A.acc = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(scratch) + 256);
  A.ml = A.acc + num_seqs * num_q_heads * (int64_t)num_splits * L.D;
  A.out = out; A.o_s0 = o_s0; A.o_s1 = o_s1; A.out_dt = out_dtype;
  A.scale_log2e = softmax_scale * 1.4426950408889634f;
  A.num_splits = num_splits; A.bps_min = blocks_per_split; A.gqa = gqa; A.Hq = num_q_heads;
  A.bps_dev = blocks_per_split_dev;
  cudaStream_t st = (cudaStream_t)stream;
  const uint8_t* pg = (const uint8_t*)pages->base;

  bool handled = false;
  rc = launch_decode_mma(L, R, pg, A, num_seqs, A.state, zero_state, nullptr, st, &handled);
  if (rc) return rc;
  if (!handled) {
    dim3 grid((unsigned)num_seqs, (unsigned)L.H, (unsigned)num_splits);
    if (gqa == 1) rc = launch_generic_gq<1>(L, R, pg, A, grid, st);
    else if (gqa == 2) rc = launch_generic_gq<2>(L, R, pg, A, grid, st);
    else if (gqa <= 4) rc = launch_generic_gq<4>(L, R, pg, A, grid, st);
    else if (gqa <= 8) rc = launch_generic_gq<8>(L, R, pg, A, grid, st);
    else rc = launch_generic_gq<16>(L, R, pg, A, grid, st);
    if (rc) return rc;
    rc = check_launch("decode");
    if (rc) return rc;
  }
  dim3 mgrid((unsigned)num_seqs, (unsigned)num_q_heads);
  if (launch_pdl(decode_merge_kernel, mgrid, dim3(L.D < 128 ? L.D : 128), 0, st, A, L.BS, L.D) != cudaSuccess)
    return check_launch("decode merge");
  return check_launch("decode merge");
}

int echokv_decode_ex(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                     const void* query, int64_t q_s0, int64_t q_s1, int32_t q_dtype, const int64_t* q_rows,
                     const int32_t* block_table, int64_t bt_s0, const int64_t* bt_rows, const int64_t* lens,
                     void* scratch, int64_t scratch_bytes, void* out, int64_t o_s0, int64_t o_s1, int32_t out_dtype,
                     float softmax_scale, int32_t num_splits, int32_t blocks_per_split,
                     const int32_t* blocks_per_split_dev, int64_t num_seqs, int32_t num_q_heads, void* stream) {
  return decode_impl(layout, pages, residual, query, q_s0, q_s1, q_dtype, q_rows, block_table, bt_s0, bt_rows, lens, scratch,
                     scratch_bytes, out, o_s0, o_s1, out_dtype, softmax_scale, num_splits, blocks_per_split,
                     blocks_per_split_dev, false, num_seqs, num_q_heads, stream);
}

int echokv_decode(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                  const void* query, int64_t q_s0, int64_t q_s1, int32_t q_dtype, const int64_t* q_rows,
                  const int32_t* block_table, int64_t bt_s0, const int64_t* bt_rows, const int64_t* lens,
                  void* scratch, int64_t scratch_bytes, void* out, int64_t o_s0, int64_t o_s1, int32_t out_dtype,
                  float softmax_scale, int32_t num_splits, int32_t blocks_per_split, int64_t num_seqs,
                  int32_t num_q_heads, void* stream) {
  return decode_impl(layout, pages, residual, query, q_s0, q_s1, q_dtype, q_rows, block_table, bt_s0, bt_rows, lens, scratch,
                     scratch_bytes, out, o_s0, o_s1, out_dtype, softmax_scale, num_splits, blocks_per_split, nullptr, true,
                     num_seqs, num_q_heads, stream);
}

// Work items the tensor-core split kernel processes at the same time on the current device for this shape (its
// teams: one per group of H consumer warps), or 0 when the shape takes the generic kernel.
int32_t echokv_decode_parallelism(const echokv_layout* layout, int32_t num_q_heads) {
  if (!layout || layout->num_kv_heads <= 0 || num_q_heads <= 0 || num_q_heads % layout->num_kv_heads) return 0;
  return decode_mma_teams(layout->num_kv_heads, layout->head_size, layout->v_group, layout->k_group, layout->block_size,
                          num_q_heads / layout->num_kv_heads);
}


// ---- decode without any allocation by the caller ------------------------------------------------
// Some callers of echokv_decode cannot provide scratch memory: code that runs inside another
// framework's memory pool with allocation forbidden at that point (for example while that
// framework is capturing or replaying its own graphs, or in a plugin that is handed only the
// input and output buffers), or a C host that links this library but not a CUDA allocator.  For
// them the split partials live in a fixed array inside the library itself.
#define ECHOKV_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_static_decode_scratch[ECHOKV_STATIC_SCRATCH_BYTES];

int64_t echokv_decode_static_scratch_bytes(void) { return (int64_t)ECHOKV_STATIC_SCRATCH_BYTES; }

int echokv_decode_static(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                         const void* query, int64_t q_s0, int64_t q_s1, int32_t q_dtype, const int64_t* q_rows,
                         const int32_t* block_table, int64_t bt_s0, const int64_t* bt_rows, const int64_t* lens,
                         void* out, int64_t o_s0, int64_t o_s1, int32_t out_dtype, float softmax_scale,
                         int32_t num_splits, int32_t blocks_per_split, int64_t num_seqs, int32_t num_q_heads,
                         void* stream) {
  if (num_seqs <= 0) return ECHOKV_OK;
  if (!layout) return set_error(ECHOKV_E_ARGUMENT, "decode_static: layout is null");
  if (num_q_heads <= 0 || layout->head_size <= 0 || num_splits <= 0)
    return set_error(ECHOKV_E_ARGUMENT, "decode_static: num_q_heads, head_size and num_splits must be positive");
  const int64_t need = echokv_decode_scratch_bytes(num_seqs, num_q_heads, layout->head_size, num_splits);
  if (need > (int64_t)ECHOKV_STATIC_SCRATCH_BYTES)
    return set_error(ECHOKV_E_UNSUPPORTED,
                     "decode_static: %lld sequences x %d query heads x %d splits need %lld bytes of split partials, "
                     "the built-in scratch holds %lld; use echokv_decode with caller-provided scratch",
                     (long long)num_seqs, num_q_heads, num_splits, (long long)need,
                     (long long)ECHOKV_STATIC_SCRATCH_BYTES);
  // The array's name is only a host-side handle; its device address is looked up once per device,
  // with that device current.
  constexpr int MAX_DEVICES = 64;
  static void* device_ptr[MAX_DEVICES] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error(ECHOKV_E_CUDA, "decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= MAX_DEVICES) return set_error(ECHOKV_E_UNSUPPORTED, "decode_static: device index %d", dev);
  if (!device_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_decode_scratch);
    if (e != cudaSuccess || !p)
      return set_error(ECHOKV_E_CUDA, "decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    device_ptr[dev] = p;
  }
  return echokv_decode(layout, pages, residual, query, q_s0, q_s1, q_dtype, q_rows, block_table, bt_s0, bt_rows, lens,
                       device_ptr[dev], (int64_t)ECHOKV_STATIC_SCRATCH_BYTES, out, o_s0, o_s1, out_dtype, softmax_scale,
                       num_splits, blocks_per_split, num_seqs, num_q_heads, stream);
}

int echokv_kernel_status(int clear) {
  const int d = decode_status_take(clear != 0), p = prefill_status_take(clear != 0);
  if (d < 0 || p < 0) return set_error(ECHOKV_E_CUDA, "kernel_status: cannot read the status words"), -1;
  return (d == 1 ? 1 : 0) | (d == 2 ? 2 : 0) | (p ? 4 : 0);
}

}  // extern "C"
