// Chunked-prefill attention over dense (already dequantized) contexts.
//
// The reference's dense path dequantizes every context once into [total_ctx, H, D] in the model
// dtype and hands it to a variable-length flash-attention library call (kernels/prefill.py:118-167,
// call site :145-153).  This file is that attention step: queries of a chunk attend to the request's
// whole context, bottom-right causal (query i of nq sees keys <= ctx - nq + i).
//
// One CTA = one (chunk, KV head, tile of BM rows); a row is a (query token, query head of the
// group) pair, so the K/V tiles a CTA streams are shared by all query heads of the KV head.  Eight
// warps x 16 rows, two CTAs per SM.  K/V tiles of BN keys travel through a two-stage cp.async ring in shared memory
// (16-byte chunks XOR-swizzled by row so ldmatrix is conflict free); S = Q K^T and O += P V run on
// mma.sync m16n8k16 with fp32 accumulators; softmax is the usual running max / running sum in the
// exp2 domain.  Compute bound: 4 * Hq * D flop per (query, visible key).
#include "common.cuh"

using namespace echokv;

namespace {

constexpr int NWARP = 8;

struct PrefillArgs {
  const void *q, *k, *v;
  void* out;
  const int32_t* chunks;  // [n, 4]: q_start, q_end, ctx, dense_start
  int64_t q_s0, q_s1, kv_s0, kv_s1, o_s0, o_s1;
  int gqa, out_dtype;
  float scale_log2;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp16(uint32_t dst, const void* src, bool on) {
  int n = on ? 16 : 0;  // zero-fill past the end
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <typename T> struct Mma;
template <> struct Mma<__half> {
  __device__ static void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  __device__ static uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <> struct Mma<__nv_bfloat16> {
  __device__ static void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  __device__ static uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

__device__ __forceinline__ float ex2(float x) {  // 2^x, hardware approximation (2^-inf = 0)
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of 16-byte chunk `c` of row `r` in a swizzled [rows][D] tile of 2-byte elements.
template <int D>
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)(r * (D * 2) + ((c ^ (r & 7)) << 4));
}

// MT m-tiles of 16 rows per warp (a warp's K / V fragments feed MT x as many MMAs), BNK keys per tile,
// NST stages of K / V in flight; one CTA-wide barrier per tile.
template <typename T, int D, int MT, int BNK, int NST>
__global__ void __launch_bounds__(NWARP * 32, MT == 1 ? 2 : 1) prefill_dense_kernel(PrefillArgs A) {
  constexpr int BMR = NWARP * 16 * MT;  // rows per CTA
  constexpr int CH = D / 8;             // 16-byte chunks per row
  constexpr int KS = D / 16;            // k-steps of Q K^T
  constexpr int TILE_BYTES = BNK * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                           // [BMR][D]
  unsigned char* k_s = smem + BMR * D * 2;             // [NST][BNK][D]
  unsigned char* v_s = k_s + NST * TILE_BYTES;         // [NST][BNK][D]

  const int4 ck = reinterpret_cast<const int4*>(A.chunks)[blockIdx.z];
  const int q0 = ck.x, nq = ck.y - ck.x, ctx = ck.z;
  const int64_t dense0 = ck.w;
  const int gqa = A.gqa, h = blockIdx.y;
  const int rows = nq * gqa;
  const int row0 = blockIdx.x * BMR;
  if (row0 >= rows) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;

  // Keys this CTA can see: up to the causal limit of its last row.
  const int last_tok = min(nq - 1, (row0 + BMR - 1) / gqa);
  const int n_keys = min(ctx, ctx - nq + last_tok + 1);
  const int n_tiles = (n_keys + BNK - 1) / BNK;

  const T* qp = reinterpret_cast<const T*>(A.q);
  const T* kp = reinterpret_cast<const T*>(A.k) + dense0 * A.kv_s0 + (int64_t)h * A.kv_s1;
  const T* vp = reinterpret_cast<const T*>(A.v) + dense0 * A.kv_s0 + (int64_t)h * A.kv_s1;

  auto load_tile = [&](int tile, int stage) {
    const int key0 = tile * BNK;
    for (int i = tid; i < BNK * CH; i += NWARP * 32) {
      int r = i / CH, c = i % CH;
      bool on = key0 + r < n_keys;
      int64_t src = (int64_t)(on ? key0 + r : 0) * A.kv_s0 + c * 8;
      uint32_t off = stage * TILE_BYTES + swz<D>(r, c);
      cp16(smem_u32(k_s) + off, kp + src, on);
      cp16(smem_u32(v_s) + off, vp + src, on);
    }
  };

  // Q tile (rows past the end are zero) and the first NST - 1 K/V tiles.
  for (int i = tid; i < BMR * CH; i += NWARP * 32) {
    int r = i / CH, c = i % CH;
    int row = row0 + r;
    bool on = row < rows;
    int tok = on ? row / gqa : 0, hq = on ? h * gqa + row % gqa : 0;
    cp16(smem_u32(q_s) + swz<D>(r, c), qp + (int64_t)(q0 + tok) * A.q_s0 + (int64_t)hq * A.q_s1 + c * 8, on);
  }
#pragma unroll
  for (int st = 0; st < NST - 1; ++st) {
    if (st < n_tiles) load_tile(st, st);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  float o[MT][D / 8][4];
#pragma unroll
  for (int mi = 0; mi < MT; ++mi)
#pragma unroll
    for (int j = 0; j < D / 8; ++j) o[mi][j][0] = o[mi][j][1] = o[mi][j][2] = o[mi][j][3] = 0.f;
  float m_run[MT][2], l_run[MT][2];
  int lim[MT][2];  // causal limits of this thread's rows (g and g + 8 of each m-tile): last visible key
  const int wrow0 = row0 + warp * 16 * MT;
#pragma unroll
  for (int mi = 0; mi < MT; ++mi)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      m_run[mi][i] = -INFINITY; l_run[mi][i] = 0.f;
      int row = wrow0 + 16 * mi + g + 8 * i;
      lim[mi][i] = row < rows ? ctx - nq + row / gqa : -1;
    }
  const int warp_lim = ctx - nq + min(nq - 1, (wrow0 + 16 * MT - 1) / gqa);
  int min_lim = lim[0][0];
#pragma unroll
  for (int mi = 0; mi < MT; ++mi) min_lim = min(min_lim, min(lim[mi][0], lim[mi][1]));

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile % NST;
    // this thread's copies of the tile have landed; after the barrier everyone's have, and everyone is
    // done with the previous tile, whose stage the next load overwrites
    asm volatile("cp.async.wait_group %0;" ::"n"(NST - 2) : "memory");
    __syncthreads();
    if (tile + NST - 1 < n_tiles) load_tile(tile + NST - 1, (tile + NST - 1) % NST);
    asm volatile("cp.async.commit_group;" ::: "memory");

    const int key0 = tile * BNK;
    if (key0 > warp_lim) continue;
    const uint32_t kb = smem_u32(k_s) + stage * TILE_BYTES, vb = smem_u32(v_s) + stage * TILE_BYTES;
    float s[MT][BNK / 8][4];
#pragma unroll
    for (int mi = 0; mi < MT; ++mi)
#pragma unroll
      for (int j = 0; j < BNK / 8; ++j) s[mi][j][0] = s[mi][j][1] = s[mi][j][2] = s[mi][j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t a[MT][4];
#pragma unroll
      for (int mi = 0; mi < MT; ++mi)
        ldsm4(smem_u32(q_s) + swz<D>(warp * 16 * MT + 16 * mi + (lane & 15), 2 * ks + (lane >> 4)), a[mi]);
#pragma unroll
      for (int jp = 0; jp < BNK / 16; ++jp) {
        uint32_t b[4];
        ldsm4(kb + swz<D>(jp * 16 + (lane & 7) + 8 * (lane >> 4), 2 * ks + ((lane >> 3) & 1)), b);
#pragma unroll
        for (int mi = 0; mi < MT; ++mi) {
          Mma<T>::run(s[mi][2 * jp], a[mi], b[0], b[1]);
          Mma<T>::run(s[mi][2 * jp + 1], a[mi], b[2], b[3]);
        }
      }
    }
    // scale, mask, running max / sum per m-tile
    const bool edge = key0 + BNK - 1 > min_lim || key0 + BNK > n_keys;
    uint32_t p[MT][BNK / 16][4];
#pragma unroll
    for (int mi = 0; mi < MT; ++mi) {
      float mx[2] = {m_run[mi][0], m_run[mi][1]};
#pragma unroll
      for (int j = 0; j < BNK / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x = s[mi][j][e] * A.scale_log2;
          if (edge && key0 + 8 * j + 2 * t + (e & 1) > lim[mi][e >> 1]) x = -INFINITY;
          s[mi][j][e] = x;
          mx[e >> 1] = fmaxf(mx[e >> 1], x);
        }
      }
      float corr[2], sum[2] = {0.f, 0.f}, base[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        base[i] = mx[i] == -INFINITY ? 0.f : mx[i];  // a row with nothing visible yet
        corr[i] = ex2(m_run[mi][i] - base[i]);
        m_run[mi][i] = mx[i];
      }
#pragma unroll
      for (int j = 0; j < BNK / 8; ++j) {
        float e0 = ex2(s[mi][j][0] - base[0]), e1 = ex2(s[mi][j][1] - base[0]);
        float e2 = ex2(s[mi][j][2] - base[1]), e3 = ex2(s[mi][j][3] - base[1]);
        sum[0] += e0 + e1;
        sum[1] += e2 + e3;
        p[mi][j >> 1][(j & 1) * 2] = Mma<T>::pack(e0, e1);
        p[mi][j >> 1][(j & 1) * 2 + 1] = Mma<T>::pack(e2, e3);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) l_run[mi][i] = l_run[mi][i] * corr[i] + sum[i];
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        o[mi][j][0] *= corr[0]; o[mi][j][1] *= corr[0];
        o[mi][j][2] *= corr[1]; o[mi][j][3] *= corr[1];
      }
    }
#pragma unroll
    for (int kk = 0; kk < BNK / 16; ++kk) {
#pragma unroll
      for (int jp = 0; jp < D / 16; ++jp) {
        uint32_t b[4];
        ldsm4t(vb + swz<D>(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), 2 * jp + (lane >> 4)), b);
#pragma unroll
        for (int mi = 0; mi < MT; ++mi) {
          Mma<T>::run(o[mi][2 * jp], p[mi][kk], b[0], b[1]);
          Mma<T>::run(o[mi][2 * jp + 1], p[mi][kk], b[2], b[3]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // normalise and store
#pragma unroll
  for (int mi = 0; mi < MT; ++mi)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float l = l_run[mi][i];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      int row = wrow0 + 16 * mi + g + 8 * i;
      if (row >= rows) continue;
      float inv = l > 0.f ? 1.f / l : 0.f;
      int tok = row / gqa, hq = h * gqa + row % gqa;
      int64_t base_o = (int64_t)(q0 + tok) * A.o_s0 + (int64_t)hq * A.o_s1;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        float x0 = o[mi][j][2 * i] * inv, x1 = o[mi][j][2 * i + 1] * inv;
        int d = 8 * j + 2 * t;
        if (A.out_dtype == ECHOKV_DT_F32) {
          *reinterpret_cast<float2*>(reinterpret_cast<float*>(A.out) + base_o + d) = make_float2(x0, x1);
        } else if (A.out_dtype == ECHOKV_DT_F16) {
          *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(A.out) + base_o + d) = __floats2half2_rn(x0, x1);
        } else {
          *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(A.out) + base_o + d) =
              __floats2bfloat162_rn(x0, x1);
        }
      }
    }
}

template <typename T, int D, int MT, int BNK, int NST>
int launch_cfg(const PrefillArgs& A, int64_t n_chunks, int max_rows, int H, cudaStream_t st) {
  constexpr int BMR = NWARP * 16 * MT;
  constexpr int SMEM = BMR * D * 2 + 2 * NST * BNK * D * 2;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(prefill_dense_kernel<T, D, MT, BNK, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    configured[dev] = true;
  }
  dim3 grid((max_rows + BMR - 1) / BMR, H, (unsigned)n_chunks);
  prefill_dense_kernel<T, D, MT, BNK, NST><<<grid, NWARP * 32, SMEM, st>>>(A);
  return check_launch("prefill");
}

// Long chunks: 32 rows per warp (256 per CTA), 32-key tiles, three stages; short ones: 16 rows per warp.
template <typename T, int D>
int launch(const PrefillArgs& A, int64_t n_chunks, int max_rows, int H, cudaStream_t st) {
  if (max_rows > 128) return launch_cfg<T, D, 2, 32, 3>(A, n_chunks, max_rows, H, st);
  return launch_cfg<T, D, 1, 64, 2>(A, n_chunks, max_rows, H, st);
}

}  // namespace

namespace echokv {
int launch_prefill_umma(const void* q, int64_t q_s0, int64_t q_s1, const void* k, const void* v, int64_t kv_s0,
                        int64_t kv_s1, int64_t total_rows, int dtype, const int32_t* chunks, int64_t n_chunks, int max_rows,
                        void* out, int64_t o_s0, int64_t o_s1, int out_dtype, float scale_log2, int gqa, int H, int head_size,
                        cudaStream_t st, int mode, bool* handled);
}
// 0: pipelined tcgen05 kernel when the shape fits (tiles by tensor-map copies), 1: always the mma.sync kernel,
// 2: plain tcgen05 kernel, 3: pipelined tcgen05 kernel with the tiles copied by the row threads
static int g_prefill_path = 0;

extern "C" {

int echokv_set_prefill_path(int path) {
  const int old = g_prefill_path;
  g_prefill_path = path;
  return old;
}

int echokv_prefill(const void* query, int64_t q_s0, int64_t q_s1, const void* k_dense, const void* v_dense,
                   int64_t kv_s0, int64_t kv_s1, int64_t total_ctx, int32_t dtype, const int32_t* chunks,
                   int64_t n_chunks, int32_t max_chunk_len, void* out, int64_t o_s0, int64_t o_s1, int32_t out_dtype,
                   float softmax_scale, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_size, void* stream) {
  if (n_chunks == 0 || max_chunk_len <= 0) return ECHOKV_OK;
  if (!query || !k_dense || !v_dense || !chunks || !out) return set_error(ECHOKV_E_ARGUMENT, "prefill: null pointer");
  if (dtype != ECHOKV_DT_F16 && dtype != ECHOKV_DT_BF16)
    return set_error(ECHOKV_E_UNSUPPORTED, "prefill: query and dense K/V must be float16 or bfloat16");
  if (head_size != 64 && head_size != 128) return set_error(ECHOKV_E_UNSUPPORTED, "prefill: head_size must be 64 or 128");
  if (num_kv_heads <= 0 || num_q_heads % num_kv_heads) return set_error(ECHOKV_E_ARGUMENT, "prefill: bad head counts");
  if (n_chunks > 65535) return set_error(ECHOKV_E_ARGUMENT, "prefill: more than 65535 chunks in one launch");
  if ((q_s0 | q_s1 | kv_s0 | kv_s1) % 8 || (o_s0 | o_s1) % 2 || (reinterpret_cast<uintptr_t>(query) & 15) ||
      (reinterpret_cast<uintptr_t>(k_dense) & 15) || (reinterpret_cast<uintptr_t>(v_dense) & 15) ||
      (reinterpret_cast<uintptr_t>(chunks) & 15) || (reinterpret_cast<uintptr_t>(out) & 7))
    return set_error(ECHOKV_E_ARGUMENT, "prefill: rows must be 16-byte aligned");
  PrefillArgs A;
  A.q = query; A.k = k_dense; A.v = v_dense; A.out = out; A.chunks = chunks;
  A.q_s0 = q_s0; A.q_s1 = q_s1; A.kv_s0 = kv_s0; A.kv_s1 = kv_s1; A.o_s0 = o_s0; A.o_s1 = o_s1;
  A.gqa = num_q_heads / num_kv_heads;
  A.out_dtype = out_dtype;
  A.scale_log2 = softmax_scale * 1.4426950408889634f;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int max_rows = max_chunk_len * A.gqa;
  if (g_prefill_path != 1) {
    bool handled = false;
    const int rc = launch_prefill_umma(query, q_s0, q_s1, k_dense, v_dense, kv_s0, kv_s1, total_ctx, dtype, chunks, n_chunks,
                                       max_rows, out, o_s0, o_s1, out_dtype, A.scale_log2, A.gqa, num_kv_heads, head_size, st,
                                       g_prefill_path, &handled);
    if (rc || handled) return rc;
  }
  if (dtype == ECHOKV_DT_F16)
    return head_size == 128 ? launch<__half, 128>(A, n_chunks, max_rows, num_kv_heads, st)
                            : launch<__half, 64>(A, n_chunks, max_rows, num_kv_heads, st);
  return head_size == 128 ? launch<__nv_bfloat16, 128>(A, n_chunks, max_rows, num_kv_heads, st)
                          : launch<__nv_bfloat16, 64>(A, n_chunks, max_rows, num_kv_heads, st);
}

}  // extern "C"
