// Canary attention-error estimator: for b in {2, 4, 8},
//   delta_b = mean over (query head, query) of KL( softmax(q . K~_b^T * s) || softmax(q . K_ref^T * s) )
// where K~_b is the storage round trip of the K_ref window at b bits in the cache's exact K
// format (per channel over consecutive groups of k_group tokens) -- echokv_vllm/canary.py:59-89,
// echokv_vllm/quant.py:82-96.  One CTA per layer; the whole problem of a layer lives in shared
// memory, so the estimator is one launch (the reference issues about a dozen small kernels).  The KV heads of a layer
// are independent until the final mean: a thread-block cluster of up to 8 CTAs per layer takes one head (or every
// eighth) each, and the cluster's first CTA adds the per-CTA sums in CTA order through distributed shared memory, so
// the result does not depend on timing.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace echokv {

constexpr int CK_THREADS = 256;
constexpr int CK_ROWS = 64;  // query rows (queries x query heads of one KV head) per pass

struct CanaryArgs {
  const void* q; int q_dt; int64_t q_sl, q_sq, q_sh;
  const float* kref; int64_t k_sl, k_sw, k_sh;
  int ring_pos, ring_fill, window;
  int nq, Hq, H, D, KG;
  float scale;
  float* out;
};

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < CK_THREADS / 32; ++i) t += red[i];
  return t;
}

__global__ void __launch_bounds__(CK_THREADS) canary_kl_kernel(CanaryArgs A) {
  extern __shared__ __align__(16) float sm[];
  cg::cluster_group cluster = cg::this_cluster();
  const int layer = blockIdx.y;
  const int crank = (int)cluster.block_rank(), csize = (int)cluster.num_blocks();
  const int D = A.D, KG = A.KG;
  const int w = (A.ring_fill / KG) * KG;       // whole groups only; the newest w keys
  const int gqa = A.Hq / A.H;
  const int rows_total = A.nq * gqa;
  float* kr = sm;                    // [w][D] K_ref window of this head
  float* kq = kr + w * D;            // [w][D] its round trip at the current tier
  float* qs = kq + w * D;            // [CK_ROWS][D] query rows (pre-scaled)
  float* lr = qs + CK_ROWS * D;      // [CK_ROWS][w] reference log-weights
  float* lq = lr + CK_ROWS * w;      // [CK_ROWS][w] quantized log-weights
  __shared__ float red[CK_THREADS / 32];
  __shared__ float cta_total[3];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float total[3] = {0.f, 0.f, 0.f};

  for (int h = crank; h < A.H; h += csize) {
    __syncthreads();
    for (int i = threadIdx.x; i < w * D; i += CK_THREADS) {
      const int t = i / D, d = i % D;
      const int v = A.ring_fill - w + t;  // index in the oldest-first view
      const int row = A.ring_fill < A.window ? v : (A.ring_pos + v) % A.window;
      kr[i] = A.kref[layer * A.k_sl + (int64_t)row * A.k_sw + h * A.k_sh + d];
    }
    for (int r0 = 0; r0 < rows_total; r0 += CK_ROWS) {
      const int nr = min(CK_ROWS, rows_total - r0);
      __syncthreads();
      for (int i = threadIdx.x; i < nr * D; i += CK_THREADS) {
        const int rr = r0 + i / D, d = i % D;
        const int qi = rr / gqa, g = rr % gqa;
        qs[i] = ld_dt(A.q, A.q_dt, layer * A.q_sl + (int64_t)qi * A.q_sq + (int64_t)(h * gqa + g) * A.q_sh + d);
      }
      for (int pass = 0; pass < 4; ++pass) {  // 0: reference, 1..3: tiers 2, 4, 8
        __syncthreads();
        const float* kk = kr;
        float* dst = lr;
        if (pass) {
          const int bits = 1 << pass;
          const float levels = (float)((1 << bits) - 1);
          for (int i = threadIdx.x; i < (w / KG) * D; i += CK_THREADS) {
            const int grp = i / D, d = i % D;
            float mn = INFINITY, mx = -INFINITY;
            for (int p = 0; p < KG; ++p) { const float x = kr[(grp * KG + p) * D + d]; mn = fminf(mn, x); mx = fmaxf(mx, x); }
            __half s16, m16;
            group_stats(mn, mx, levels, s16, m16);
            const float sc = __half2float(s16), m = __half2float(m16);
            for (int p = 0; p < KG; ++p) {
              const int e = (grp * KG + p) * D + d;
              kq[e] = __fadd_rn(__fmul_rn((float)quant_code(kr[e], m, sc, levels), sc), m);
            }
          }
          __syncthreads();
          kk = kq;
          dst = lq;
        }
        // scores: one (row, key) pair per thread and iteration
        for (int i = threadIdx.x; i < nr * w; i += CK_THREADS) {
          const int rr = i / w, t = i % w;
          const float4* a = reinterpret_cast<const float4*>(qs + rr * D);
          const float4* b = reinterpret_cast<const float4*>(kk + t * D);
          float acc = 0.f;
          for (int d4 = 0; d4 < D / 4; ++d4) {
            const float4 x = a[d4], y = b[d4];
            acc += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
          }
          dst[rr * w + t] = acc * A.scale;
        }
        __syncthreads();
        // log-softmax per row (one warp per row), and for tiers the row's KL
        float part = 0.f;
        for (int rr = warp; rr < nr; rr += CK_THREADS / 32) {
          float mx = -INFINITY;
          for (int t = lane; t < w; t += 32) mx = fmaxf(mx, dst[rr * w + t]);
#pragma unroll
          for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
          float se = 0.f;
          for (int t = lane; t < w; t += 32) se += expf(dst[rr * w + t] - mx);
#pragma unroll
          for (int o = 16; o; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
          const float lse = mx + logf(se);
          float kl = 0.f;
          for (int t = lane; t < w; t += 32) {
            const float v = dst[rr * w + t] - lse;
            dst[rr * w + t] = v;
            if (pass) kl += expf(v) * (v - lr[rr * w + t]);
          }
          part += kl;
        }
        if (pass) total[pass - 1] += block_sum(part, red);
      }
    }
  }
  if (threadIdx.x == 0) {
    for (int b = 0; b < 3; ++b) cta_total[b] = total[b];
  }
  cluster.sync();  // every CTA's sums are in its shared memory
  if (crank == 0 && threadIdx.x == 0) {
    const float inv = 1.f / (float)(A.Hq * A.nq);
    for (int b = 0; b < 3; ++b) {
      float t = 0.f;
      for (int r = 0; r < csize; ++r) t += cluster.map_shared_rank(cta_total, r)[b];  // in CTA order = head order
      A.out[layer * 3 + b] = fmaxf(t * inv, 0.f);
    }
  }
  cluster.sync();  // no CTA leaves (and gives up its shared memory) before the first one has read it
}

}  // namespace echokv

using namespace echokv;

extern "C" int echokv_canary_kl(const void* query, int32_t q_dtype, int64_t q_sl, int64_t q_sq, int64_t q_sh,
                                const float* kref, int64_t k_sl, int64_t k_sw, int64_t k_sh, int32_t ring_pos,
                                int32_t ring_fill, int32_t window, int32_t num_layers, int32_t nq, int32_t num_q_heads,
                                int32_t num_kv_heads, int32_t head_size, int32_t k_group, float softmax_scale,
                                float* out, void* stream) {
  if (num_layers <= 0) return ECHOKV_OK;
  if (!query || !kref || !out) return set_error(ECHOKV_E_ARGUMENT, "canary_kl: null pointer");
  if (q_dtype < 0 || q_dtype > 2) return set_error(ECHOKV_E_ARGUMENT, "canary_kl: bad dtype");
  if (nq <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads || head_size % 4 || k_group <= 0 || window <= 0 ||
      ring_fill > window || ring_pos < 0 || ring_pos >= window)
    return set_error(ECHOKV_E_ARGUMENT, "canary_kl: bad shape");
  const int w = (ring_fill / k_group) * k_group;
  if (w == 0) return set_error(ECHOKV_E_ARGUMENT, "canary_kl: K_ref has %d keys, fewer than k_group=%d", ring_fill, k_group);
  if ((reinterpret_cast<uintptr_t>(kref) & 3) != 0) return set_error(ECHOKV_E_ARGUMENT, "canary_kl: misaligned K_ref");
  const size_t smem = (size_t)(2 * w * head_size + CK_ROWS * head_size + 2 * CK_ROWS * w) * sizeof(float);
  if (smem > 48 * 1024) {  // per call: the attribute belongs to the current device
    cudaError_t e = cudaFuncSetAttribute(canary_kl_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(ECHOKV_E_UNSUPPORTED, "canary_kl: window %d x head %d needs %zu bytes of shared memory", w, head_size, smem);
  }
  CanaryArgs A;
  A.q = query; A.q_dt = q_dtype; A.q_sl = q_sl; A.q_sq = q_sq; A.q_sh = q_sh;
  A.kref = kref; A.k_sl = k_sl; A.k_sw = k_sw; A.k_sh = k_sh;
  A.ring_pos = ring_pos; A.ring_fill = ring_fill; A.window = window;
  A.nq = nq; A.Hq = num_q_heads; A.H = num_kv_heads; A.D = head_size; A.KG = k_group;
  A.scale = softmax_scale; A.out = out;
  const int csize = num_kv_heads < 8 ? num_kv_heads : 8;  // 8 = the portable cluster size
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)csize, (unsigned)num_layers);
  cfg.blockDim = dim3(CK_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, canary_kl_kernel, A) != cudaSuccess) return check_launch("canary_kl");
  return check_launch("canary_kl");
}
