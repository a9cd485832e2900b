// Chunked-prefill attention over dense contexts on the 5th-generation tensor cores (tcgen05 + TMEM),
// head size 128.  Same contract as prefill_dense_kernel in prefill.cu: queries of a chunk attend to the
// request's whole context, bottom-right causal.
//
// One CTA = one (chunk, KV head, 128 rows); a row is a (query token, query head of the group) pair and
// owns one TMEM lane, and thread r of the CTA's 128 owns row r.  Per 64-key tile:
//   S  = Q K^T   one thread issues 8 tcgen05.mma (M 128, N 64, K 16 each): Q [128 x 128] and the K tile
//                [64 x 128] sit in shared memory as 128-byte-swizzled K-major panels of 64 channels;
//                the fp32 result lands in 64 TMEM columns;
//   softmax      thread r reads its row of S with tcgen05.ld, masks, exponentiates against a running
//                reference (moved only when a row outgrows it by more than 2^8, then the row of O in TMEM
//                is rescaled with tcgen05.ld / tcgen05.st) and writes P as a 16-bit K-major panel;
//   O += P V     4 tcgen05.mma (M 128, N 128, K 16): the V tile is used as it lies in memory
//                ([key][channel], an MN-major B operand), O accumulates in 128 TMEM columns.
// K / V tiles are double-buffered with cp.async; completion of the MMAs comes back through
// tcgen05.commit on an mbarrier.  Every wait is bounded; a wait that gives up ends the CTA's work, frees
// its TMEM and raises the status word.
#include <cuda.h>  // CUtensorMap and its enums; the encoder is looked up at run time, nothing links against the driver
#include "common.cuh"

using namespace echokv;

namespace echokv {
namespace umma {

constexpr int UM = 128;  // rows per CTA = TMEM lanes
constexpr int UN = 64;   // keys per tile
constexpr int UD = 128;  // head size
constexpr int TMEM_COLS = 256;  // S: columns [0, 64), O: columns [64, 192)
constexpr int O_COL = 64;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

#ifdef ECHOKV_PROFILE
// profile builds only: cycles that row thread 0 of every group spends per phase of the tile loop
__device__ unsigned long long g_pphase[8];
#define PF_T(x) const long long x = clock64()
#define PF_ADD(k, a, b) pf[k] += (b) - (a)
#else
#define PF_T(x)
#define PF_ADD(k, a, b)
#endif
constexpr float REF_SLACK = 8.f;  // log2 units a row may exceed the softmax reference before it moves

constexpr int Q_BYTES = UM * UD * 2;        // two panels of 128 rows x 128 bytes
constexpr int KV_BYTES = UN * UD * 2;       // two panels of 64 rows x 128 bytes
constexpr int P_BYTES = UM * UN * 2;        // one panel of 128 rows x 128 bytes
constexpr int SMEM_BYTES = Q_BYTES + 4 * KV_BYTES + P_BYTES + 1024;  // K, V double-buffered; slack for 1024-byte alignment

struct Args {
  const void *q, *k, *v;
  void* out;
  const int32_t* chunks;  // [n, 4]: q_start, q_end, ctx, dense_start
  int64_t q_s0, q_s1, kv_s0, kv_s1, o_s0, o_s1;
  int gqa, out_dtype, is_bf16;
  float scale_log2;
  int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// byte offset of 16-byte chunk c (0..7) of row r inside a 128-byte-swizzled panel (rows of 128 bytes)
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

__device__ __forceinline__ void cp16(uint32_t dst, const void* src, bool on) {
  const int n = on ? 16 : 0;  // zero-fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle: start address, leading / stride byte offsets (>> 4).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of this architecture
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// A operand in tensor memory (row i of A = lane i, two 16-bit elements of K per 32-bit column)
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t a = smem_u32(bar);
  for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(a), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                 "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
                 "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                 "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  tmem_ld32_nowait(taddr, r);
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// The registers of a tcgen05.ld may only be read after this.
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                 "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                 "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                 "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                 "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                 "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                 "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                 "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
               : "memory");
}
__device__ __forceinline__ void tmem_st32_raw(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
                 "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]),
                 "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
                 "r"(v[30]), "r"(v[31])
               : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack16(float lo, float hi, bool bf16) {
  uint32_t d;
  if (bf16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

__global__ void __launch_bounds__(UM, 2) prefill_umma_kernel(Args A) {
  extern __shared__ unsigned char dyn[];
  __shared__ __align__(8) uint64_t bar_s, bar_o;
  __shared__ uint32_t tmem_slot;
  const uint32_t base = (smem_u32(dyn) + 1023u) & ~1023u;  // swizzled panels want 1024-byte alignment
  const uint32_t q_s = base, k_s = q_s + Q_BYTES, v_s = k_s + 2 * KV_BYTES, p_s = v_s + 2 * KV_BYTES;

  const int4 ck = reinterpret_cast<const int4*>(A.chunks)[blockIdx.z];
  const int q0 = ck.x, nq = ck.y - ck.x, ctx = ck.z;
  const int64_t dense0 = ck.w;
  const int gqa = A.gqa, h = blockIdx.y;
  const int rows = nq * gqa;
  const int row0 = blockIdx.x * UM;
  if (row0 >= rows) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const bool bf16 = A.is_bf16 != 0;

  // this thread's row
  const int row = row0 + tid;
  const bool live = row < rows;
  const int tok = live ? row / gqa : 0, hq = live ? h * gqa + row % gqa : 0;
  const int lim = live ? ctx - nq + tok : -1;  // last visible key
  // keys this CTA can see: up to the causal limit of its last row
  const int last_tok = min(nq - 1, (row0 + UM - 1) / gqa);
  const int n_keys = min(ctx, ctx - nq + last_tok + 1);
  const int n_tiles = (n_keys + UN - 1) / UN;

  const uint16_t* qp = reinterpret_cast<const uint16_t*>(A.q) + (int64_t)(q0 + tok) * A.q_s0 + (int64_t)hq * A.q_s1;
  const uint16_t* kp = reinterpret_cast<const uint16_t*>(A.k) + dense0 * A.kv_s0 + (int64_t)h * A.kv_s1;
  const uint16_t* vp = reinterpret_cast<const uint16_t*>(A.v) + dense0 * A.kv_s0 + (int64_t)h * A.kv_s1;

  auto load_tile = [&](int tile, int stage) {
    const int key0 = tile * UN;
#pragma unroll
    for (int j = 0; j < (UN * 16) / UM; ++j) {
      const int idx = tid + UM * j, key = idx >> 4, c = idx & 15;
      const bool on = key0 + key < n_keys;
      const int64_t src = (int64_t)(on ? key0 + key : 0) * A.kv_s0 + c * 8;
      const uint32_t off = stage * KV_BYTES + (c >> 3) * (UN * 128) + swz(key, c & 7);
      cp16(k_s + off, kp + src, on);
      cp16(v_s + off, vp + src, on);
    }
  };

  // Q (this thread's row, zero past the end) and the first K / V tile
#pragma unroll
  for (int c = 0; c < 16; ++c) cp16(q_s + (c >> 3) * (UM * 128) + swz(tid, c & 7), qp + c * 8, live);
  load_tile(0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_s)));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_o)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;");
  const uint32_t tmem = tmem_slot;
  const uint32_t t_row = tmem + ((uint32_t)(warp * 32) << 16);  // this warp's quarter of the lanes

  // instruction descriptors (kind::f16): fp32 accumulator, 16-bit A / B, N, M; the P.V one takes B MN-major
  const uint32_t fmt = bf16 ? 1u : 0u;
  const uint32_t idesc_qk = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(UN >> 3) << 17) | ((uint32_t)(UM >> 4) << 24);
  const uint32_t idesc_pv = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(UD >> 3) << 17) | ((uint32_t)(UM >> 4) << 24);

  float m_ref = -INFINITY, l_run = 0.f;
  bool ok = true;
  for (int tile = 0; tile < n_tiles && ok; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < n_tiles) load_tile(tile + 1, stage ^ 1);  // its buffer was released by the wait on bar_o below
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // cp.async writes -> tensor-core reads
    __syncthreads();

    if (tid == 0) {  // S = Q K^T
      asm volatile("tcgen05.fence::after_thread_sync;");
#pragma unroll
      for (int k = 0; k < UD / 16; ++k) {
        const uint64_t a = make_desc(q_s + (k >> 2) * (UM * 128) + (k & 3) * 32, 16, 1024);
        const uint64_t b = make_desc(k_s + stage * KV_BYTES + (k >> 2) * (UN * 128) + (k & 3) * 32, 16, 1024);
        mma_f16(tmem, a, b, idesc_qk, k > 0);
      }
      mma_commit(&bar_s);
    }
    if (!bar_wait(&bar_s, tile & 1)) { ok = false; }
    ok = __syncthreads_and(ok);
    if (!ok) break;
    asm volatile("tcgen05.fence::after_thread_sync;");

    // this row's scores: both halves in flight, then one wait
    uint32_t raw[UN];
    tmem_ld32_nowait(t_row, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
    tmem_ld32_nowait(t_row + 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[32]));
    tmem_ld_wait();
    float s[UN];
#pragma unroll
    for (int j = 0; j < UN; ++j) s[j] = __uint_as_float(raw[j]);
    const int key0 = tile * UN;
    if (key0 + UN - 1 > lim) {  // the tile crosses this row's causal limit
#pragma unroll
      for (int j = 0; j < UN; ++j)
        if (key0 + j > lim) s[j] = -INFINITY;
    }
    // maximum in raw units (the scale is positive), four independent chains
    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < UN; ++j) m4[j & 3] = fmaxf(m4[j & 3], s[j]);
    const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * A.scale_log2;
    // the reference only moves when some row of the warp outgrows it by more than REF_SLACK
    if (__any_sync(0xffffffffu, mx > m_ref + REF_SLACK)) {
      const float m_new = fmaxf(m_ref, mx);
      const float corr = m_new == -INFINITY ? 1.f : ex2(m_ref - m_new);
      m_ref = m_new;
      l_run *= corr;
      if (tile > 0) {  // O holds earlier tiles: rescale this row of it
#pragma unroll
        for (int c0 = 0; c0 < UD; c0 += 32) {
          float o[32];
          tmem_ld32(t_row + O_COL + c0, o);
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] *= corr;
          tmem_st32(t_row + O_COL + c0, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
    }
    const float nref = m_ref == -INFINITY ? 0.f : -m_ref;
    float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < UN / 8; ++c) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p0 = ex2(fmaf(s[8 * c + 2 * e], A.scale_log2, nref)), p1 = ex2(fmaf(s[8 * c + 2 * e + 1], A.scale_log2, nref));
        sum4[e] += p0 + p1;
        w[e] = pack16(p0, p1, bf16);
      }
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(p_s + swz(tid, c)), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
    }
    const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
    l_run += sum;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P stores -> tensor-core reads
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();

    if (tid == 0) {  // O += P V
      asm volatile("tcgen05.fence::after_thread_sync;");
#pragma unroll
      for (int k = 0; k < UN / 16; ++k) {
        const uint64_t a = make_desc(p_s + k * 32, 16, 1024);
        // V as it lies in memory: rows = keys, 128 bytes = 64 channels per panel; 16 keys = two 8-key groups
        const uint64_t b = make_desc(v_s + stage * KV_BYTES + k * 2048, UN * 128, 1024);
        mma_f16(tmem + O_COL, a, b, idesc_pv, (tile > 0 || k > 0) ? 1u : 0u);
      }
      mma_commit(&bar_o);
    }
    // P, this stage of K / V and O are free again once the MMAs have completed
    if (!bar_wait(&bar_o, tile & 1)) { ok = false; }
    ok = __syncthreads_and(ok);
    asm volatile("tcgen05.fence::after_thread_sync;");
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  if (ok) {  // every lane takes part in the TMEM loads; rows past the end just do not store
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    const int64_t base_o = (int64_t)(q0 + tok) * A.o_s0 + (int64_t)hq * A.o_s1;
#pragma unroll
    for (int c0 = 0; c0 < UD; c0 += 32) {
      float o[32];
      tmem_ld32(t_row + O_COL + c0, o);
      if (live) {
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float x0 = o[j] * inv, x1 = o[j + 1] * inv;
          const int d = c0 + j;
          if (A.out_dtype == ECHOKV_DT_F32) {
            *reinterpret_cast<float2*>(reinterpret_cast<float*>(A.out) + base_o + d) = make_float2(x0, x1);
          } else {
            *reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(A.out) + base_o + d) = pack16(x0, x1, A.out_dtype == ECHOKV_DT_BF16);
          }
        }
      }
    }
  }
  if (!ok && tid == 0 && A.status) atomicExch(A.status, 1);
  asm volatile("tcgen05.fence::before_thread_sync;");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
}


// The same computation with the tensor work overlapped with the softmax and no CTA-wide barrier in the
// loop.  G groups of 128 rows (G = 2: all 512 TMEM columns) share the K / V tiles of a CTA; one extra warp
// only issues MMAs.  Per 64-key tile t:
//   row threads   wait for the scores of t (bar_s), take the softmax, wait until O += P V of t - 1 is done
//                 (bar_o), start the copies of tile t + 3 into the stage t - 1 used, write P, arrive on bar_p;
//                 at the top of the step they report that their copies of tile t + 1 have landed (bar_kv);
//   issuer        waits bar_kv of t + 1 and issues its scores into the other score buffer, waits bar_p and
//                 issues O += P V of t.
// So the scores of t + 1 and O += P V of t run on the tensor cores under the softmax of t and t + 1.
constexpr bool P_IN_TMEM = true;  // P of a tile overwrites the first 32 columns of its scores and is the A operand from there
constexpr int PIPE_STAGES = P_IN_TMEM ? 5 : 4;  // what fits beside Q for two groups (and P, when it is staged in shared memory)
constexpr int S1_COL = 192;
template <int G> constexpr int smem_pipe() { return G * (Q_BYTES + (P_IN_TMEM ? 0 : P_BYTES)) + 2 * PIPE_STAGES * KV_BYTES + 1024; }

__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

struct alignas(64) Maps {
  CUtensorMap k, v;  // dense K / V as (channel, head, row) tensors, boxes of 64 channels x 64 rows, 128-byte swizzle
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}

// TMA = true: one more warp streams the K / V tiles with tensor-map copies (a stage is free once the commit
// after the O += P V that read it has arrived on its bar_free); TMA = false: the row threads copy them.
template <int G, bool TMA>
__global__ void __launch_bounds__(UM * G + (TMA ? 64 : 32), 1) prefill_umma_pipe_kernel(Args A, const __grid_constant__ Maps M) {
  extern __shared__ unsigned char dyn[];
  __shared__ __align__(8) uint64_t bar_s[2], bar_o, bar_p, bar_kv[PIPE_STAGES], bar_free[PIPE_STAGES];
  __shared__ uint32_t tmem_slot;
  constexpr int NROW = UM * G;  // row threads
  const uint32_t base = (smem_u32(dyn) + 1023u) & ~1023u;
  const uint32_t q_s = base, k_s = q_s + G * Q_BYTES, v_s = k_s + PIPE_STAGES * KV_BYTES, p_s = v_s + PIPE_STAGES * KV_BYTES;

  const int4 ck = reinterpret_cast<const int4*>(A.chunks)[blockIdx.z];
  const int q0 = ck.x, nq = ck.y - ck.x, ctx = ck.z;
  const int64_t dense0 = ck.w;
  const int gqa = A.gqa, h = blockIdx.y;
  const int rows = nq * gqa;
  const int row0 = blockIdx.x * NROW;
  if (row0 >= rows) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const bool issuer_warp = tid >= NROW && tid < NROW + 32;
  const bool producer_warp = tid >= NROW + 32;
  const bool row_thread = tid < NROW;
  const int grp = !row_thread ? 0 : tid / UM, r128 = tid % UM;  // group of 128 rows, row inside it (= TMEM lane)
  const bool bf16 = A.is_bf16 != 0;
  const int row = row0 + tid;
  const bool live = row_thread && row < rows;
  const int tok = live ? row / gqa : 0, hq = live ? h * gqa + row % gqa : 0;
  const int lim = live ? ctx - nq + tok : -1;
  const int last_tok = min(nq - 1, (row0 + NROW - 1) / gqa);
  const int n_keys = min(ctx, ctx - nq + last_tok + 1);
  const int n_tiles = (n_keys + UN - 1) / UN;

  const uint16_t* qp = reinterpret_cast<const uint16_t*>(A.q) + (int64_t)(q0 + tok) * A.q_s0 + (int64_t)hq * A.q_s1;
  const uint16_t* kp = reinterpret_cast<const uint16_t*>(A.k) + dense0 * A.kv_s0 + (int64_t)h * A.kv_s1;
  const uint16_t* vp = reinterpret_cast<const uint16_t*>(A.v) + dense0 * A.kv_s0 + (int64_t)h * A.kv_s1;
  auto load_tile = [&](int tile) {  // row threads only
    const int key0 = tile * UN, stage = tile % PIPE_STAGES;
#pragma unroll
    for (int j = 0; j < (UN * 16) / NROW; ++j) {
      const int idx = tid + NROW * j, key = idx >> 4, c = idx & 15;
      const bool on = key0 + key < n_keys;
      const int64_t src = (int64_t)(on ? key0 + key : 0) * A.kv_s0 + c * 8;
      const uint32_t off = stage * KV_BYTES + (c >> 3) * (UN * 128) + swz(key, c & 7);
      cp16(k_s + off, kp + src, on);
      cp16(v_s + off, vp + src, on);
    }
  };
  if (row_thread) {
#pragma unroll
    for (int c = 0; c < 16; ++c) cp16(q_s + grp * Q_BYTES + (c >> 3) * (UM * 128) + swz(r128, c & 7), qp + c * 8, live);
    if constexpr (TMA) {  // Q is visible to the tensor cores after the barrier below
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    } else {
      // tiles 0 .. PIPE_STAGES - 2 in flight, one commit group each (empty groups keep the count regular)
#pragma unroll
      for (int t0 = 0; t0 < PIPE_STAGES - 1; ++t0) {
        if (t0 < n_tiles) load_tile(t0);
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
    }
  }
  if (tid == 0) {
    auto init = [](uint64_t* b, int n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(n)); };
    init(&bar_s[0], 1); init(&bar_s[1], 1); init(&bar_o, 1); init(&bar_p, NROW);
    for (int i = 0; i < PIPE_STAGES; ++i) { init(&bar_kv[i], TMA ? 1 : NROW); init(&bar_free[i], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS * G));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;");
  const uint32_t tmem = tmem_slot;
  const uint32_t fmt = bf16 ? 1u : 0u;
  const uint32_t idesc_qk = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(UN >> 3) << 17) | ((uint32_t)(UM >> 4) << 24);
  const uint32_t idesc_pv = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(UD >> 3) << 17) | ((uint32_t)(UM >> 4) << 24);
  bool ok = true;

  if (issuer_warp) {
    if (tid == NROW) {
      auto issue_qk = [&](int tile) {  // S[tile & 1] = Q K_tile^T for every group
        const int stage = tile % PIPE_STAGES;
        const uint32_t s_col = (tile & 1) ? S1_COL : 0;
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
          for (int k = 0; k < UD / 16; ++k) {
            const uint64_t a = make_desc(q_s + g * Q_BYTES + (k >> 2) * (UM * 128) + (k & 3) * 32, 16, 1024);
            const uint64_t b = make_desc(k_s + stage * KV_BYTES + (k >> 2) * (UN * 128) + (k & 3) * 32, 16, 1024);
            mma_f16(tmem + g * TMEM_COLS + s_col, a, b, idesc_qk, k > 0);
          }
        mma_commit(&bar_s[tile & 1]);
      };
      if (bar_wait(&bar_kv[0], 0)) {
        asm volatile("tcgen05.fence::after_thread_sync;");
        issue_qk(0);
      } else {
        ok = false;
      }
      for (int tile = 0; tile < n_tiles && ok; ++tile) {
        if (tile + 1 < n_tiles) {  // the next tile's scores: their buffer was last read before bar_p of tile - 1
          if (!bar_wait(&bar_kv[(tile + 1) % PIPE_STAGES], ((tile + 1) / PIPE_STAGES) & 1)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;");
          issue_qk(tile + 1);
        }
        if (!bar_wait(&bar_p, tile & 1)) { ok = false; break; }  // every row thread has written its P
        asm volatile("tcgen05.fence::after_thread_sync;");
        const int stage = tile % PIPE_STAGES;
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
          for (int k = 0; k < UN / 16; ++k) {
            const uint64_t b = make_desc(v_s + stage * KV_BYTES + k * 2048, UN * 128, 1024);
            if constexpr (P_IN_TMEM) {  // 16 keys = 8 columns of P
              mma_f16_ts(tmem + g * TMEM_COLS + O_COL, tmem + g * TMEM_COLS + ((tile & 1) ? S1_COL : 0) + k * 8, b, idesc_pv,
                         (tile > 0 || k > 0) ? 1u : 0u);
            } else {
              const uint64_t a = make_desc(p_s + g * P_BYTES + k * 32, 16, 1024);
              mma_f16(tmem + g * TMEM_COLS + O_COL, a, b, idesc_pv, (tile > 0 || k > 0) ? 1u : 0u);
            }
          }
        mma_commit(&bar_o);
        if constexpr (TMA) mma_commit(&bar_free[stage]);
      }
    }
  } else if (producer_warp) {
    if constexpr (TMA) {
      if (tid == NROW + 32) {
        auto load = [&](int tile) {
          const int stage = tile % PIPE_STAGES;
          const int z = (int)dense0 + tile * UN;
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&bar_kv[stage])), "r"(2 * KV_BYTES) : "memory");
#pragma unroll
          for (int p = 0; p < 2; ++p) {  // the two panels of 64 channels
            tma_load_3d(k_s + stage * KV_BYTES + p * (UN * 128), &M.k, 64 * p, h, z, &bar_kv[stage]);
            tma_load_3d(v_s + stage * KV_BYTES + p * (UN * 128), &M.v, 64 * p, h, z, &bar_kv[stage]);
          }
        };
        for (int tile = 0; tile < n_tiles && tile < PIPE_STAGES; ++tile) load(tile);
        for (int tile = PIPE_STAGES; tile < n_tiles; ++tile) {  // the stage of tile - PIPE_STAGES, once its O += P V is done
          if (!bar_wait(&bar_free[tile % PIPE_STAGES], ((tile / PIPE_STAGES) - 1) & 1)) { ok = false; break; }
          load(tile);
        }
      }
    }
  } else {
    const uint32_t t_row = tmem + ((uint32_t)((warp & 3) * 32) << 16) + grp * TMEM_COLS;  // this warp's lanes, this group's columns
    if constexpr (!TMA) {  // Q and tile 0 have landed
      asm volatile("cp.async.wait_group %0;" ::"n"(PIPE_STAGES - 2) : "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      bar_arrive(&bar_kv[0]);
    }
    float m_ref = -INFINITY, l_run = 0.f;
    for (int tile = 0; tile < n_tiles; ++tile) {
      if (!TMA && tile + 1 < n_tiles) {  // my copies of tile + 1 have landed (all but the newest copy group are complete)
        asm volatile("cp.async.wait_group %0;" ::"n"(PIPE_STAGES - 3) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        bar_arrive(&bar_kv[(tile + 1) % PIPE_STAGES]);
      }
      if (!__all_sync(0xffffffffu, bar_wait(&bar_s[tile & 1], (tile >> 1) & 1))) { ok = false; break; }  // the scores of this tile
      asm volatile("tcgen05.fence::after_thread_sync;");
      uint32_t raw[UN];
      const uint32_t s_col = (tile & 1) ? S1_COL : 0;
      tmem_ld32_nowait(t_row + s_col, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
      tmem_ld32_nowait(t_row + s_col + 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[32]));
      tmem_ld_wait();
      float s[UN];
#pragma unroll
      for (int j = 0; j < UN; ++j) s[j] = __uint_as_float(raw[j]);
      const int key0 = tile * UN;
      if (key0 + UN - 1 > lim) {
#pragma unroll
        for (int j = 0; j < UN; ++j)
          if (key0 + j > lim) s[j] = -INFINITY;
      }
      float m16[16];  // a tree: 16 independent chains of 3, then 4 levels
#pragma unroll
      for (int j = 0; j < 16; ++j) m16[j] = fmaxf(fmaxf(s[j], s[j + 16]), fmaxf(s[j + 32], s[j + 48]));
#pragma unroll
      for (int w = 8; w >= 1; w >>= 1)
#pragma unroll
        for (int j = 0; j < w; ++j) m16[j] = fmaxf(m16[j], m16[j + w]);
      const float mx = m16[0] * A.scale_log2;
      bool o_idle = tile == 0;  // O += P V of the previous tile is known to have completed
      if (__any_sync(0xffffffffu, mx > m_ref + REF_SLACK)) {
        const float m_new = fmaxf(m_ref, mx);
        const float corr = m_new == -INFINITY ? 1.f : ex2(m_ref - m_new);
        m_ref = m_new;
        l_run *= corr;
        if (tile > 0) {  // rescale this row of O, once the MMAs that accumulate into it are done
          if (!bar_wait(&bar_o, (tile - 1) & 1)) ok = false;
          ok = __all_sync(0xffffffffu, ok);  // the TMEM accesses below are warp-wide
          if (!ok) break;
          o_idle = true;
          asm volatile("tcgen05.fence::after_thread_sync;");
#pragma unroll
          for (int c0 = 0; c0 < UD; c0 += 32) {
            float o[32];
            tmem_ld32(t_row + O_COL + c0, o);
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= corr;
            tmem_st32(t_row + O_COL + c0, o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      const float nref = m_ref == -INFINITY ? 0.f : -m_ref;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t w[UN / 2];
#pragma unroll
      for (int c = 0; c < UN / 8; ++c) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = ex2(fmaf(s[8 * c + 2 * e], A.scale_log2, nref)), p1 = ex2(fmaf(s[8 * c + 2 * e + 1], A.scale_log2, nref));
          sum4[e] += p0 + p1;
          w[4 * c + e] = pack16(p0, p1, bf16);
        }
      }
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // The P buffer in shared memory and the stage tile - 1 used are free once the previous O += P V has
      // completed.  P in tensor memory needs no wait: it goes where this tile's scores were, and the scores of
      // tile + 1 that will overwrite it are issued after the O += P V that reads it.
      if constexpr (!(P_IN_TMEM && TMA)) {
        if (!o_idle && !bar_wait(&bar_o, (tile - 1) & 1)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if constexpr (!TMA) {
        if (tile + PIPE_STAGES - 1 < n_tiles) load_tile(tile + PIPE_STAGES - 1);  // into the stage tile - 1 used
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
      if constexpr (P_IN_TMEM) {
        tmem_st32_raw(t_row + s_col, w);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int c = 0; c < UN / 8; ++c)
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(p_s + grp * P_BYTES + swz(r128, c)), "r"(w[4 * c]), "r"(w[4 * c + 1]),
                       "r"(w[4 * c + 2]), "r"(w[4 * c + 3]) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      asm volatile("tcgen05.fence::before_thread_sync;");
      bar_arrive(&bar_p);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (ok && !bar_wait(&bar_o, (n_tiles - 1) & 1)) ok = false;
    ok = __all_sync(0xffffffffu, ok);
    asm volatile("tcgen05.fence::after_thread_sync;");
    if (ok) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const int64_t base_o = (int64_t)(q0 + tok) * A.o_s0 + (int64_t)hq * A.o_s1;
#pragma unroll
      for (int c0 = 0; c0 < UD; c0 += 32) {
        float o[32];
        tmem_ld32(t_row + O_COL + c0, o);
        if (live) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float x0 = o[j] * inv, x1 = o[j + 1] * inv;
            const int d = c0 + j;
            if (A.out_dtype == ECHOKV_DT_F32) {
              *reinterpret_cast<float2*>(reinterpret_cast<float*>(A.out) + base_o + d) = make_float2(x0, x1);
            } else {
              *reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(A.out) + base_o + d) = pack16(x0, x1, A.out_dtype == ECHOKV_DT_BF16);
            }
          }
        }
      }
    }
  }
  if (!ok && (tid & 31) == 0 && A.status) atomicExch(A.status, 1);
  asm volatile("tcgen05.fence::before_thread_sync;");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS * G));
}

// 128-key tiles, two groups of 128 rows that alternate.  Each group owns 256 TMEM columns: its scores S (128
// columns, fp32) and its O (128 columns).  P of a tile overwrites the first 64 columns of S and is the A operand
// of O += P V from there, so a group's next scores can only be issued after that MMA: while one group takes its
// softmax, the tensor cores run the other group's O += P V and next Q K^T.  K and V tiles travel in separate
// two-stage rings (a K stage is free as soon as both groups' scores of its tile are issued and done, long
// before the V stage of the same tile).  M 128 x N 128 score MMAs read 8 KB of shared memory per 64-cycle
// instruction, inside what shared memory delivers; the N 64 ones of the kernel above need 6 KB per 32 cycles.
constexpr int WN = 128;                    // keys per tile
constexpr int WKV_BYTES = WN * UD * 2;     // one K or V tile: two panels of 128 rows x 128 bytes
constexpr int W_STAGES = 2;
constexpr int W_SCOL = 0, W_OCOL = 128, W_GCOLS = 256;
constexpr int smem_wide() { return 2 * Q_BYTES + 2 * W_STAGES * WKV_BYTES + 1024; }

__device__ __forceinline__ void tmem_st16_raw(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
                 "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
               : "memory");
}

__device__ __forceinline__ void tmem_ld16_raw(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                 "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(2 * UM + 64, 1) prefill_umma_wide_kernel(Args A, const __grid_constant__ Maps M) {
  extern __shared__ unsigned char dyn[];
  __shared__ __align__(8) uint64_t bar_s[2], bar_p[2], bar_o[2], bar_k[W_STAGES], bar_v[W_STAGES], bar_kfree[W_STAGES],
      bar_vfree[W_STAGES];
  __shared__ uint32_t tmem_slot;
  constexpr int NROW = 2 * UM;
  const uint32_t base = (smem_u32(dyn) + 1023u) & ~1023u;
  const uint32_t q_s = base, k_s = q_s + 2 * Q_BYTES, v_s = k_s + W_STAGES * WKV_BYTES;

  const int4 ck = reinterpret_cast<const int4*>(A.chunks)[blockIdx.z];
  const int q0 = ck.x, nq = ck.y - ck.x, ctx = ck.z;
  const int dense0 = ck.w;
  const int gqa = A.gqa, h = blockIdx.y;
  const int rows = nq * gqa;
  const int row0 = blockIdx.x * NROW;
  if (row0 >= rows) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const bool row_thread = tid < NROW;
  const int grp = row_thread ? tid / UM : 0, r128 = tid % UM;
  const bool bf16 = A.is_bf16 != 0;
  const int row = row0 + tid;
  const bool live = row_thread && row < rows;
  const int tok = live ? row / gqa : 0, hq = live ? h * gqa + row % gqa : 0;
  const int lim = live ? ctx - nq + tok : -1;
  const int last_tok = min(nq - 1, (row0 + NROW - 1) / gqa);
  const int n_keys = min(ctx, ctx - nq + last_tok + 1);
  const int n_tiles = (n_keys + WN - 1) / WN;

  if (row_thread) {
    const uint16_t* qp = reinterpret_cast<const uint16_t*>(A.q) + (int64_t)(q0 + tok) * A.q_s0 + (int64_t)hq * A.q_s1;
#pragma unroll
    for (int c = 0; c < 16; ++c) cp16(q_s + grp * Q_BYTES + (c >> 3) * (UM * 128) + swz(r128, c & 7), qp + c * 8, live);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (tid == 0) {
    auto init = [](uint64_t* b, int n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(n)); };
    for (int g = 0; g < 2; ++g) { init(&bar_s[g], 1); init(&bar_p[g], UM); init(&bar_o[g], 1); }
    for (int i = 0; i < W_STAGES; ++i) { init(&bar_k[i], 1); init(&bar_v[i], 1); init(&bar_kfree[i], 1); init(&bar_vfree[i], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(2 * W_GCOLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;");
  const uint32_t tmem = tmem_slot;
  const uint32_t fmt = bf16 ? 1u : 0u;
  const uint32_t idesc_qk = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(WN >> 3) << 17) | ((uint32_t)(UM >> 4) << 24);
  const uint32_t idesc_pv = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(UD >> 3) << 17) | ((uint32_t)(UM >> 4) << 24);
  bool ok = true;

  if (tid == NROW) {  // the MMA issuer
    auto issue_qk = [&](int g, int tile) {  // S_g = Q_g K_tile^T
      const uint32_t kb = k_s + (tile % W_STAGES) * WKV_BYTES;
#pragma unroll
      for (int k = 0; k < UD / 16; ++k) {
        const uint64_t a = make_desc(q_s + g * Q_BYTES + (k >> 2) * (UM * 128) + (k & 3) * 32, 16, 1024);
        const uint64_t b = make_desc(kb + (k >> 2) * (WN * 128) + (k & 3) * 32, 16, 1024);
        mma_f16(tmem + g * W_GCOLS + W_SCOL, a, b, idesc_qk, k > 0);
      }
      mma_commit(&bar_s[g]);
    };
    if (bar_wait(&bar_k[0], 0)) {
      asm volatile("tcgen05.fence::after_thread_sync;");
      issue_qk(0, 0);
      issue_qk(1, 0);
      mma_commit(&bar_kfree[0]);
    } else {
      ok = false;
    }
    for (int tile = 0; tile < n_tiles && ok; ++tile) {
      const int stage = tile % W_STAGES, nstage = (tile + 1) % W_STAGES;
      const bool more = tile + 1 < n_tiles;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        if (!bar_wait(&bar_p[g], tile & 1)) { ok = false; break; }  // the group's P is in tensor memory
        if (g == 0 && !bar_wait(&bar_v[stage], (tile / W_STAGES) & 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;");
#pragma unroll
        for (int k = 0; k < WN / 16; ++k) {  // 16 keys = 8 columns of P; V as it lies in memory (MN-major B)
          const uint64_t b = make_desc(v_s + stage * WKV_BYTES + k * 2048, WN * 128, 1024);
          mma_f16_ts(tmem + g * W_GCOLS + W_OCOL, tmem + g * W_GCOLS + W_SCOL + k * 8, b, idesc_pv, (tile > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(&bar_o[g]);
        if (g == 1) mma_commit(&bar_vfree[stage]);
        if (more) {  // the group's next scores go over its P, after the MMA that reads it
          if (g == 0 && !bar_wait(&bar_k[nstage], ((tile + 1) / W_STAGES) & 1)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;");
          issue_qk(g, tile + 1);
          if (g == 1) mma_commit(&bar_kfree[nstage]);
        }
      }
    }
  } else if (tid == NROW + 32) {  // the tile producer
    auto load = [&](const CUtensorMap* map, uint32_t dst, uint64_t* bar, int tile) {
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(WKV_BYTES) : "memory");
      tma_load_3d(dst, map, 0, h, dense0 + tile * WN, bar);
      tma_load_3d(dst + WN * 128, map, 64, h, dense0 + tile * WN, bar);
    };
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int stage = tile % W_STAGES;
      const uint32_t par = ((tile / W_STAGES) - 1) & 1;
      if (tile >= W_STAGES && !bar_wait(&bar_kfree[stage], par)) { ok = false; break; }
      load(&M.k, k_s + stage * WKV_BYTES, &bar_k[stage], tile);
      if (tile >= W_STAGES && !bar_wait(&bar_vfree[stage], par)) { ok = false; break; }
      load(&M.v, v_s + stage * WKV_BYTES, &bar_v[stage], tile);
    }
  } else if (row_thread) {
    const uint32_t t_row = tmem + ((uint32_t)((warp & 3) * 32) << 16) + grp * W_GCOLS;  // this warp's lanes, this group's columns
    float m_ref = -INFINITY, l_run = 0.f;
#ifdef ECHOKV_PROFILE
    long long pf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#endif
    for (int tile = 0; tile < n_tiles; ++tile) {
      PF_T(c0);
      if (!__all_sync(0xffffffffu, bar_wait(&bar_s[grp], tile & 1))) { ok = false; break; }  // the scores of this tile
      asm volatile("tcgen05.fence::after_thread_sync;");
      PF_T(c1);
      uint32_t raw[WN];
#pragma unroll
      for (int c = 0; c < WN / 32; ++c) tmem_ld32_nowait(t_row + W_SCOL + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&raw[32 * c]));
      tmem_ld_wait();
      PF_T(c2);
      const int key0 = tile * WN;
      if (key0 + WN - 1 > lim) {  // bottom-right causal mask, and the keys past the context
#pragma unroll
        for (int j = 0; j < WN; ++j)
          if (key0 + j > lim) raw[j] = 0xff800000u;  // -inf
      }
      float m16[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float a = fmaxf(fmaxf(__uint_as_float(raw[j]), __uint_as_float(raw[j + 16])), fmaxf(__uint_as_float(raw[j + 32]), __uint_as_float(raw[j + 48])));
        const float b = fmaxf(fmaxf(__uint_as_float(raw[j + 64]), __uint_as_float(raw[j + 80])), fmaxf(__uint_as_float(raw[j + 96]), __uint_as_float(raw[j + 112])));
        m16[j] = fmaxf(a, b);
      }
#pragma unroll
      for (int w = 8; w >= 1; w >>= 1)
#pragma unroll
        for (int j = 0; j < w; ++j) m16[j] = fmaxf(m16[j], m16[j + w]);
      const float mx = m16[0] * A.scale_log2;
      // the reference only moves when some row of the warp outgrows it by more than REF_SLACK
      const bool moves = __any_sync(0xffffffffu, mx > m_ref + REF_SLACK);
      PF_T(c3);
      if (moves) {
        const float m_new = fmaxf(m_ref, mx);
        const float corr = m_new == -INFINITY ? 1.f : ex2(m_ref - m_new);
        m_ref = m_new;
        l_run *= corr;
        if (tile > 0) {  // rescale this row of O, once the MMAs that accumulate into it are done
          if (!__all_sync(0xffffffffu, bar_wait(&bar_o[grp], (tile - 1) & 1))) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;");
#pragma unroll 1
          for (int c0 = 0; c0 < UD; c0 += 16) {  // 16 columns at a time: the tile's scores stay in registers
            uint32_t o[16];
            tmem_ld16_raw(t_row + W_OCOL + c0, o);
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
            tmem_st16_raw(t_row + W_OCOL + c0, o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      const float nref = m_ref == -INFINITY ? 0.f : -m_ref;
      PF_T(c4);
      // two elements per instruction (packed fp32 FMA / ADD) for the scaling and the row sum
      const float2 sc2 = make_float2(A.scale_log2, A.scale_log2), nr2 = make_float2(nref, nref);
      float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int c = 0; c < WN / 32; ++c) {  // 32 keys -> 16 columns of P, over scores already in registers
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(raw[32 * c + 2 * e]), __uint_as_float(raw[32 * c + 2 * e + 1])), sc2, nr2);
          const float2 pp = make_float2(ex2(x.x), ex2(x.y));
          sum2[e & 3] = __fadd2_rn(sum2[e & 3], pp);
          w[e] = pack16(pp.x, pp.y, bf16);
        }
        tmem_st16_raw(t_row + W_SCOL + 16 * c, w);
      }
      const float2 s01 = __fadd2_rn(sum2[0], sum2[1]), s23 = __fadd2_rn(sum2[2], sum2[3]);
      l_run += (s01.x + s01.y) + (s23.x + s23.y);
      PF_T(c5);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;");
      bar_arrive(&bar_p[grp]);
      PF_T(c6);
      PF_ADD(0, c0, c1); PF_ADD(1, c1, c2); PF_ADD(2, c2, c3); PF_ADD(3, c3, c4); PF_ADD(4, c4, c5); PF_ADD(5, c5, c6);
#ifdef ECHOKV_PROFILE
      pf[7] += 1;
#endif
    }
#ifdef ECHOKV_PROFILE
    if (r128 == 0)
      for (int i = 0; i < 8; ++i) atomicAdd(&g_pphase[i], (unsigned long long)pf[i]);
#endif
    if (ok && !bar_wait(&bar_o[grp], (n_tiles - 1) & 1)) ok = false;
    ok = __all_sync(0xffffffffu, ok);
    asm volatile("tcgen05.fence::after_thread_sync;");
    if (ok) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const int64_t base_o = (int64_t)(q0 + tok) * A.o_s0 + (int64_t)hq * A.o_s1;
#pragma unroll
      for (int c0 = 0; c0 < UD; c0 += 32) {
        float o[32];
        tmem_ld32(t_row + W_OCOL + c0, o);
        if (live) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float x0 = o[j] * inv, x1 = o[j + 1] * inv;
            const int d = c0 + j;
            if (A.out_dtype == ECHOKV_DT_F32) {
              *reinterpret_cast<float2*>(reinterpret_cast<float*>(A.out) + base_o + d) = make_float2(x0, x1);
            } else {
              *reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(A.out) + base_o + d) = pack16(x0, x1, A.out_dtype == ECHOKV_DT_BF16);
            }
          }
        }
      }
    }
  }
  if (!ok && (tid & 31) == 0 && A.status) atomicExch(A.status, 1);
  asm volatile("tcgen05.fence::before_thread_sync;");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * W_GCOLS));
}

}  // namespace umma

// Launches the tcgen05 kernel when the shape fits (head size 128, 16-bit inputs); otherwise leaves
// `handled` false.
// Raised (1) by a kernel of this file whose bounded wait on an mbarrier ran out; its output is then undefined.
__device__ int g_prefill_status;

#ifdef ECHOKV_PROFILE
extern "C" int echokv_debug_prefill_phase(unsigned long long* dst, int clear) {
  const int rc = (int)cudaMemcpyFromSymbol(dst, umma::g_pphase, sizeof(unsigned long long) * 8);
  if (clear) {
    const unsigned long long z[8] = {};
    cudaMemcpyToSymbol(umma::g_pphase, z, sizeof(z));
  }
  return rc;
}
#endif

int prefill_status_take(bool clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_prefill_status, sizeof(int)) != cudaSuccess) return -1;  // synchronizes
  if (v && clear) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_prefill_status, &zero, sizeof(int));
  }
  return v;
}

namespace {

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled tensor_map_encoder() {
  static EncodeTiled fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiled>(p);
  }();
  return fn;
}

// (channel, head, row) view of a dense [rows, H, 128] tensor; boxes of 64 channels x 1 head x `box_rows` rows land
// as a 128-byte-swizzled panel.  Rows past `rows` read as zeros.
bool encode_kv_map(CUtensorMap* map, const void* base, int64_t rows, int H, int64_t s_row, int64_t s_head, bool bf16, int box_rows) {
  EncodeTiled enc = tensor_map_encoder();
  if (!enc) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)umma::UD, (cuuint64_t)H, (cuuint64_t)rows};
  const cuuint64_t strides[2] = {(cuuint64_t)s_head * 2, (cuuint64_t)s_row * 2};
  const cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
  const cuuint32_t elem[3] = {1, 1, 1};
  return enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims,
             strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// mode 0: pipelined; K / V tiles by tensor-map copies when `total_rows` is known and the strides allow it, and then
// 128-key tiles for chunks of more than 128 rows; mode 4: the same with 64-key tiles throughout; mode 2: the plain
// kernel; mode 3: pipelined, 64-key tiles copied by the row threads.
int launch_prefill_umma(const void* q, int64_t q_s0, int64_t q_s1, const void* k, const void* v, int64_t kv_s0,
                        int64_t kv_s1, int64_t total_rows, int dtype, const int32_t* chunks, int64_t n_chunks, int max_rows,
                        void* out, int64_t o_s0, int64_t o_s1, int out_dtype, float scale_log2, int gqa, int H, int head_size,
                        cudaStream_t st, int mode, bool* handled) {
  using namespace umma;
  *handled = false;
  if (head_size != UD || (dtype != ECHOKV_DT_F16 && dtype != ECHOKV_DT_BF16)) return ECHOKV_OK;
  Args A;
  A.q = q; A.k = k; A.v = v; A.out = out; A.chunks = chunks;
  A.q_s0 = q_s0; A.q_s1 = q_s1; A.kv_s0 = kv_s0; A.kv_s1 = kv_s1; A.o_s0 = o_s0; A.o_s1 = o_s1;
  A.gqa = gqa; A.out_dtype = out_dtype; A.is_bf16 = dtype == ECHOKV_DT_BF16; A.scale_log2 = scale_log2;
  static bool configured[64] = {};
  static int* status_word[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64) return ECHOKV_OK;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(prefill_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_umma_pipe_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pipe<1>()) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_umma_pipe_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pipe<2>()) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_umma_pipe_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pipe<1>()) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_umma_pipe_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pipe<2>()) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_umma_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_wide()) != cudaSuccess ||
        cudaGetSymbolAddress(reinterpret_cast<void**>(&status_word[dev]), g_prefill_status) != cudaSuccess)
      return check_launch("prefill (tcgen05 kernel)");
    configured[dev] = true;
  }
  A.status = status_word[dev];
  dim3 grid((max_rows + UM - 1) / UM, H, (unsigned)n_chunks);
  if (mode == 2) {
    prefill_umma_kernel<<<grid, UM, SMEM_BYTES, st>>>(A);
  } else {
    Maps M;
    memset(&M, 0, sizeof(M));
    // tensor-map copies: strides in multiples of 16 bytes, rows addressed by a 32-bit coordinate
    const bool two = max_rows > UM;  // two groups of 128 rows per CTA share the K / V tiles
    const bool wide = two && mode == 0;  // 128-key tiles
    const bool tma = (mode == 0 || mode == 4) && total_rows > 0 && total_rows < (1ll << 31) && (kv_s0 % 8) == 0 && (kv_s1 % 8) == 0 &&
                     encode_kv_map(&M.k, k, total_rows, H, kv_s0, kv_s1, A.is_bf16, wide ? WN : UN) &&
                     encode_kv_map(&M.v, v, total_rows, H, kv_s0, kv_s1, A.is_bf16, wide ? WN : UN);
    if (two) grid.x = (max_rows + 2 * UM - 1) / (2 * UM);
    if (wide && tma) prefill_umma_wide_kernel<<<grid, 2 * UM + 64, smem_wide(), st>>>(A, M);
    else if (wide) prefill_umma_pipe_kernel<2, false><<<grid, 2 * UM + 32, smem_pipe<2>(), st>>>(A, M);
    else if (two && tma) prefill_umma_pipe_kernel<2, true><<<grid, 2 * UM + 64, smem_pipe<2>(), st>>>(A, M);
    else if (two) prefill_umma_pipe_kernel<2, false><<<grid, 2 * UM + 32, smem_pipe<2>(), st>>>(A, M);
    else if (tma) prefill_umma_pipe_kernel<1, true><<<grid, UM + 64, smem_pipe<1>(), st>>>(A, M);
    else prefill_umma_pipe_kernel<1, false><<<grid, UM + 32, smem_pipe<1>(), st>>>(A, M);
  }
  const int rc = check_launch("prefill (tcgen05 kernel)");
  if (rc) return rc;
  *handled = true;
  return ECHOKV_OK;
}

}  // namespace echokv
