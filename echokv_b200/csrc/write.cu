// Quantize-on-write kernels: token rows (V per token, K to residual / sealed codes / K_ref ring)
// and per-channel K groups.  Numerics follow echokv_vllm/quant.py bit for bit: fp16-rounded stats
// first, IEEE fp32 divide, round-half-to-even, clamp after rounding.
#include "common.cuh"

#include <type_traits>

namespace echokv {

constexpr int WT_WARPS = 4;

__global__ void write_headers_kernel(uint8_t* pages, int64_t ps, const int64_t* blocks, const uint8_t* headers,
                                     int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint4 h = reinterpret_cast<const uint4*>(headers)[i];
  *reinterpret_cast<uint4*>(pages + blocks[i] * ps) = h;
}

// dst row i = src row rows[i], 16 bytes per thread.
__global__ void gather_rows_kernel(const uint4* __restrict__ src, int64_t src_stride16, const int64_t* __restrict__ rows,
                                   uint4* __restrict__ dst, int64_t n, int row16) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n * row16) return;
  const int64_t r = i / row16;
  const int c = (int)(i % row16);
  dst[i] = src[rows[r] * src_stride16 + c];
}

__global__ void scatter_i64_kernel(int64_t* dst, const int64_t* idx, const int64_t* val, int64_t n) {
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) dst[idx[i]] = val[i];
}

// ---- the quantizer, many values under one reciprocal ---------------------------------------------
// code = clamp(rne((x - mn) / scale), 0, levels) without a divide per value.  With y = RN(1 / scale) computed once,
// q0 = RN(d * y), r = RN(d - scale * q0) (exact: one FMA) and q1 = RN(q0 + r * y), q1 IS the correctly rounded
// quotient RN(d / scale) (Markstein's correction step; it needs y correctly rounded and the significand of the
// divisor not all ones, and every scale here is an fp16 value).  q0 is capped at 512 first so that infinities and
// overflowing quotients stay ordered through the correction (anything >= 255.5 clamps to `levels` anyway; NaN
// clamps to 0 as on the divide route).  Adding 1.5 * 2^23 to the clamped quotient rounds it to the nearest-even
// integer in the float's low mantissa bits (0 and levels are integers, so clamping before or after the rounding
// gives the same code).
constexpr float QMAGIC = 12582912.f;            // 1.5 * 2^23
constexpr uint32_t QMAGIC_BITS = 0x4B400000u;   // its bit pattern; QMAGIC + code has bit pattern QMAGIC_BITS + code

__device__ __forceinline__ uint32_t quant_u(float x, float mn, float scale, float rscale, float levels) {
  const float d = __fsub_rn(x, mn);
  const float q0 = fminf(__fmul_rn(d, rscale), 512.0f);
  const float r = __fmaf_rn(-scale, q0, d);
  const float q1 = __fmaf_rn(r, rscale, q0);
  const float t = fminf(fmaxf(q1, 0.0f), levels);
  return __float_as_uint(__fadd_rn(t, QMAGIC));
}

// 8 values of QMAGIC_BITS + code -> the 8 codes packed at BITS (element k at bit k * BITS): the shifted sum of
// the words minus the shifted sum of the constant, modulo 2^32.
template <int BITS>
__device__ __forceinline__ uint64_t pack_u8(const uint32_t (&u)[8]) {
  if constexpr (BITS == 8) {
    constexpr uint32_t C = QMAGIC_BITS * 0x01010101u;
    const uint32_t lo = u[0] + (u[1] << 8) + (u[2] << 16) + (u[3] << 24) - C;
    const uint32_t hi = u[4] + (u[5] << 8) + (u[6] << 16) + (u[7] << 24) - C;
    return (uint64_t)lo | ((uint64_t)hi << 32);
  } else if constexpr (BITS == 4) {
    constexpr uint32_t C = QMAGIC_BITS * 0x11111111u;
    return u[0] + (u[1] << 4) + (u[2] << 8) + (u[3] << 12) + (u[4] << 16) + (u[5] << 20) + (u[6] << 24) +
           (u[7] << 28) - C;
  } else {
    constexpr uint32_t C = QMAGIC_BITS * 0x5555u;
    return (u[0] + (u[1] << 2) + (u[2] << 4) + (u[3] << 6) + (u[4] << 8) + (u[5] << 10) + (u[6] << 12) +
            (u[7] << 14) - C) & 0xffffu;
  }
}

// Quantize 8 values to their codes packed at BITS.  PER_CH: value k has its own stats m[k], sc[k], rsc[k]
// (K: per channel); otherwise all 8 share m[0], sc[0], rsc[0] (V: one group).
template <int BITS, bool PER_CH>
__device__ __forceinline__ uint64_t quant_pack8(const float (&x)[8], const float* m, const float* sc, const float* rsc) {
  constexpr float levels = (float)((1 << BITS) - 1);
  uint32_t u[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) u[k] = quant_u(x[k], m[PER_CH ? k : 0], sc[PER_CH ? k : 0], rsc[PER_CH ? k : 0], levels);
  return pack_u8<BITS>(u);
}
template <int BITS, bool PER_CH>
__device__ __forceinline__ void quant_store8(uint8_t* dst, const float (&x)[8], const float* m, const float* sc,
                                             const float* rsc) {
  store_packed8(dst, quant_pack8<BITS, PER_CH>(x, m, sc, rsc), BITS);
}
template <bool PER_CH>
__device__ __forceinline__ void quant_store8(int bits, uint8_t* dst, const float (&x)[8], const float* m,
                                             const float* sc, const float* rsc) {
  if (bits == 4) quant_store8<4, PER_CH>(dst, x, m, sc, rsc);
  else if (bits == 8) quant_store8<8, PER_CH>(dst, x, m, sc, rsc);
  else quant_store8<2, PER_CH>(dst, x, m, sc, rsc);
}

// 8 consecutive 16-bit elements as loaded (one 16-byte word) -> float
template <typename T>
__device__ __forceinline__ void cvt8(const uint4& raw, float (&x)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if constexpr (sizeof(T) == 2 && !std::is_same<T, __half>::value) {
      x[2 * k] = __uint_as_float(w[k] << 16);
      x[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
      x[2 * k] = f.x;
      x[2 * k + 1] = f.y;
    }
  }
}

// Running minimum / maximum of 8 channels over many rows, kept packed in the rows' own 16-bit type (two channels
// per register, one instruction per pair and row); minima and maxima of values of that type are exact in it.
template <typename T>
struct MinMax8 {
  uint32_t mn[4], mx[4];
  __device__ __forceinline__ void init() {
    const uint32_t pinf = std::is_same<T, __half>::value ? 0x7C007C00u : 0x7F807F80u;
#pragma unroll
    for (int k = 0; k < 4; ++k) { mn[k] = pinf; mx[k] = pinf | 0x80008000u; }
  }
  __device__ __forceinline__ void update(const uint4& raw) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if constexpr (std::is_same<T, __half>::value) {
        const __half2 v = *reinterpret_cast<const __half2*>(&w[k]);
        __half2 a = __hmin2(*reinterpret_cast<__half2*>(&mn[k]), v), b = __hmax2(*reinterpret_cast<__half2*>(&mx[k]), v);
        mn[k] = *reinterpret_cast<uint32_t*>(&a);
        mx[k] = *reinterpret_cast<uint32_t*>(&b);
      } else {
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&w[k]);
        __nv_bfloat162 a = __hmin2(*reinterpret_cast<__nv_bfloat162*>(&mn[k]), v);
        __nv_bfloat162 b = __hmax2(*reinterpret_cast<__nv_bfloat162*>(&mx[k]), v);
        mn[k] = *reinterpret_cast<uint32_t*>(&a);
        mx[k] = *reinterpret_cast<uint32_t*>(&b);
      }
    }
  }
  __device__ __forceinline__ void finish(float (&lo)[8], float (&hi)[8]) const {
    cvt8<T>(make_uint4(mn[0], mn[1], mn[2], mn[3]), lo);
    cvt8<T>(make_uint4(mx[0], mx[1], mx[2], mx[3]), hi);
  }
};

// Division and remainder by a layout constant that is usually a power of two: `sh` is its log2, or -1.
struct Shifts { int D, VG, BS, KG; };
__device__ __forceinline__ int qdiv(int x, int d, int sh) { return sh >= 0 ? x >> sh : x / d; }
__device__ __forceinline__ int qmod(int x, int d, int sh) { return sh >= 0 ? x & (d - 1) : x % d; }
static int log2_or_neg(int v) {
  if (v <= 0 || (v & (v - 1))) return -1;
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}
static Shifts make_shifts(const LayoutDev& L) { return {log2_or_neg(L.D), log2_or_neg(L.VG), log2_or_neg(L.BS), log2_or_neg(L.KG)}; }

// Byte offsets (from the pool base) of consecutive token rows of one block stored at `bits`: the chunk of a row is
// looked up once per chunk, not once per row.
struct RowWalk {
  int64_t base, row_bytes;
  int r, tpc, j;
  int64_t blk;
  __device__ __forceinline__ int64_t chunk_base(const uint8_t* pages, const LayoutDev& L) const {
    int64_t page = blk, slot = 0;
    if (j > 0) {
      const int id = reinterpret_cast<const int32_t*>(pages + blk * L.PS + 4)[j - 1];
      page = id / L.KC;
      slot = id % L.KC;
    }
    return page * L.PS + L.o_data + slot * L.CB;
  }
  __device__ __forceinline__ void start(const uint8_t* pages, const LayoutDev& L, int sh_bs, int64_t block, int off,
                                        int bits) {
    blk = block;
    const int sh_bits = bits == 2 ? 1 : (bits == 4 ? 2 : 3);
    tpc = (2 * L.BS) >> sh_bits;
    j = qdiv(off, tpc, sh_bs >= 0 ? sh_bs + 1 - sh_bits : -1);
    r = off - j * tpc;
    row_bytes = (int64_t)(2 * L.H * L.D * bits) / 8;
    base = chunk_base(pages, L);
  }
  __device__ __forceinline__ int64_t offset() const { return base + (int64_t)r * row_bytes; }
  __device__ __forceinline__ void next(const uint8_t* pages, const LayoutDev& L) {
    if (++r == tpc) { r = 0; ++j; base = chunk_base(pages, L); }
  }
};

// Token rows (kernels/write.py:171-229 does one program per (row, head)).  MODE 2: one CTA of four warps per
// row (few rows, a decode step: the shortest dependent chain); MODE 1: one warp per row (many rows); in both a
// thread owns 8 channels at a time and the V group's min / max is reduced over its VG / 8 neighbouring lanes by
// shuffles (needs VG / 8 to be a power of two <= 32).  MODE 0: one warp per row, a lane per V group, for the
// other group sizes.  All produce the same bytes: min and max do not depend on the order of reduction.
// `res_raw`: the residual buffer has the rows' own 16-bit type and 16-byte aligned rows, so an open group's key
// goes there as loaded; `kref_vec`: 16-byte aligned K_ref rows.
template <typename T>
struct TokArgs {
  LayoutDev L;
  uint8_t* pages;
  const T* key; int64_t k_s0, k_s1;
  const T* value; int64_t v_s0, v_s1;
  const int64_t* tok; int64_t tok_s0;
  void* res; int res_dt; int64_t r_s0, r_s1, r_s2;
  float* kref; int64_t kref_s0, kref_s1;
  int64_t n_rows;
  bool vec_in, res_raw, kref_vec;
  Shifts sh;
};

// K side of 8 channels (piece `c` of the row) of one token: the key goes to the residual row of its open group,
// and / or is quantized under the stored statistics of a sealed group, and / or goes to the K_ref ring.
template <typename T>
__device__ __forceinline__ void key_chunk(const TokArgs<T>& A, int64_t row, int c, int off, int bits, int64_t rowoff,
                                          int64_t rslot, bool sealed, int64_t kidx) {
  const LayoutDev& L = A.L;
  const Shifts sh = A.sh;
  const int h = qdiv(c * 8, L.D, sh.D), d0 = qmod(c * 8, L.D, sh.D);
  const int grp = qdiv(off, L.KG, sh.KG), gpos = off - grp * L.KG;
  const int64_t src = row * A.k_s0 + h * A.k_s1 + d0;
  if (rslot >= 0 && A.res_raw) {
    const int64_t ro = rslot * A.r_s0 + (int64_t)gpos * A.r_s1 + h * A.r_s2 + d0;
    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(A.res) + ro) = *reinterpret_cast<const uint4*>(A.key + src);
    if (!sealed && kidx < 0) return;
  }
  float x[8];
  ld8<T>(A.key, src, A.vec_in, x);
  if (rslot >= 0 && !A.res_raw) {
    const int64_t ro = rslot * A.r_s0 + (int64_t)gpos * A.r_s1 + h * A.r_s2 + d0;
#pragma unroll
    for (int k = 0; k < 8; ++k) st_dt(A.res, A.res_dt, ro + k, x[k]);
  }
  if (sealed) {
    const float levels = (float)((1 << bits) - 1);
    const int64_t e = ((int64_t)grp * L.H + h) * L.D + d0;
    const int64_t slot = A.tok[row];
    const int64_t blk = sh.BS >= 0 ? slot >> sh.BS : slot / L.BS;
    const uint8_t* pg = A.pages + blk * L.PS;
    const __half* ks = reinterpret_cast<const __half*>(pg + L.o_ks) + e;
    const __half* km = reinterpret_cast<const __half*>(pg + L.o_km) + e;
    uint32_t q[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) q[k] = quant_code(x[k], __half2float(km[k]), __half2float(ks[k]), levels);
    store_packed8(A.pages + rowoff + h * ((L.D * bits) / 8) + (d0 * bits) / 8, pack8(q, bits), bits);
  }
  if (kidx >= 0) {
    float* dst = A.kref + kidx * A.kref_s0 + h * A.kref_s1 + d0;
    if (A.kref_vec) {
      reinterpret_cast<float4*>(dst)[0] = make_float4(x[0], x[1], x[2], x[3]);
      reinterpret_cast<float4*>(dst)[1] = make_float4(x[4], x[5], x[6], x[7]);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) dst[k] = x[k];
    }
  }
}

// One token row.  `row_in_cta`: row index this CTA / warp works on; `skip_residual`: the row's open-group key is
// stored by someone else (see write_step_kernel).
template <typename T, int MODE>
__device__ __forceinline__ void token_row(const TokArgs<T>& A, int64_t row, bool skip_residual) {
  const LayoutDev& L = A.L;
  uint8_t* __restrict__ pages = A.pages;
  const T* __restrict__ key = A.key;
  const T* __restrict__ value = A.value;
  const int64_t* __restrict__ tok = A.tok;
  const int64_t k_s0 = A.k_s0, k_s1 = A.k_s1, v_s0 = A.v_s0, v_s1 = A.v_s1, tok_s0 = A.tok_s0;
  void* res = A.res;
  const int res_dt = A.res_dt;
  const int64_t r_s0 = A.r_s0, r_s1 = A.r_s1, r_s2 = A.r_s2, kref_s0 = A.kref_s0, kref_s1 = A.kref_s1;
  float* __restrict__ kref = A.kref;
  const bool vec_in = A.vec_in, res_raw = A.res_raw, kref_vec = A.kref_vec;
  const Shifts sh = A.sh;
  const int lane = threadIdx.x & 31;
  const int64_t slot = tok[row];
  if (slot < 0) return;  // padding, or a token that is not stored
  const int64_t blk = sh.BS >= 0 ? slot >> sh.BS : slot / L.BS;
  const int off = (int)(slot - blk * L.BS);
  const int bits = block_bits(pages, L, blk);
  const float levels = (float)((1 << bits) - 1);
  RowWalk walk;
  walk.start(pages, L, sh.BS, blk, off, bits);
  const int64_t rowoff = walk.offset();
  const int side_bytes = (L.H * L.D * bits) / 8;
  const int head_bytes = (L.D * bits) / 8;
  uint8_t* page = pages + blk * L.PS;
  const int units = (L.H * L.D) / 8;  // 8-channel pieces of a row
  const int first = MODE == 2 ? threadIdx.x : lane, step = MODE == 2 ? WT_WARPS * 32 : 32;

  if constexpr (MODE != 0) {
    // V: per token, groups of VG along head_dim; VG / 8 neighbouring threads share a group.
    const int upg = L.VG / 8;
    for (int base = first - lane; base < units; base += step) {
      const int u = base + lane;
      const bool on = u < units;
      const int h = on ? qdiv(u * 8, L.D, sh.D) : 0, d0 = on ? qmod(u * 8, L.D, sh.D) : 0;
      float x[8];
      float mn = INFINITY, mx = -INFINITY;
      if (on) {
        ld8<T>(value, row * v_s0 + h * v_s1 + d0, vec_in, x);
#pragma unroll
        for (int k = 0; k < 8; ++k) { mn = fminf(mn, x[k]); mx = fmaxf(mx, x[k]); }
      }
      for (int o = 1; o < upg; o <<= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      }
      if (!on) continue;
      __half s16, m16;
      group_stats(mn, mx, levels, s16, m16);
      const float sc = __half2float(s16), m = __half2float(m16);
      if (qmod(d0, L.VG, sh.VG) == 0) {
        const int64_t e = ((int64_t)off * L.H + h) * L.NG + qdiv(d0, L.VG, sh.VG);
        reinterpret_cast<__half*>(page + L.o_vs)[e] = s16;
        reinterpret_cast<__half*>(page + L.o_vm)[e] = m16;
      }
      const float rsc = __frcp_rn(sc);
      quant_store8<false>(bits, pages + rowoff + side_bytes + h * head_bytes + (d0 * bits) / 8, x, &m, &sc, &rsc);
    }
  } else {
    // V: per token, groups of VG along head_dim; one lane per group.
    for (int gi = lane; gi < L.H * L.NG; gi += 32) {
      const int h = gi / L.NG, g = gi % L.NG;
      const int64_t src = row * v_s0 + h * v_s1 + (int64_t)g * L.VG;
      float mn = INFINITY, mx = -INFINITY;
      float x[8];
      for (int c = 0; c < L.VG; c += 8) {
        ld8<T>(value, src + c, vec_in, x);
#pragma unroll
        for (int k = 0; k < 8; ++k) { mn = fminf(mn, x[k]); mx = fmaxf(mx, x[k]); }
      }
      __half s16, m16;
      group_stats(mn, mx, levels, s16, m16);
      const float sc = __half2float(s16), m = __half2float(m16);
      const int64_t e = ((int64_t)off * L.H + h) * L.NG + g;
      reinterpret_cast<__half*>(page + L.o_vs)[e] = s16;
      reinterpret_cast<__half*>(page + L.o_vm)[e] = m16;
      uint8_t* dst = pages + rowoff + side_bytes + h * head_bytes + (g * L.VG * bits) / 8;
      const float rsc = __frcp_rn(sc);
      for (int c = 0; c < L.VG; c += 8) {
        ld8<T>(value, src + c, vec_in, x);
        quant_store8<false>(bits, dst + (c * bits) / 8, x, &m, &sc, &rsc);
      }
    }
  }

  // K: residual row (open group), codes under stored stats (sealed group), K_ref ring row.
  const int64_t rslot = skip_residual ? -1 : tok[tok_s0 + row];
  const bool sealed = tok[2 * tok_s0 + row] != 0;
  const int64_t kidx = kref ? tok[3 * tok_s0 + row] : -1;
  if (rslot < 0 && !sealed && kidx < 0) return;
  for (int c = first; c < units; c += step) key_chunk<T>(A, row, c, off, bits, rowoff, rslot, sealed, kidx);
}

// Many token rows, one thread per (row, KV head, group of 32 channels): the V group's 64 bytes are loaded once,
// its statistics computed once, and its codes leave as one 16-byte store at INT4 (two at INT8, eight bytes at
// INT2); then the K side of the same channels.  For 16-bit rows on 16-byte boundaries with v_group 32; stores the
// same bytes as token_row.
template <typename T>
__global__ void __launch_bounds__(128, 8) write_tokens_bulk_kernel(const TokArgs<T> A, int gpr, int sh_gpr, int sh_ng) {
  const LayoutDev& L = A.L;
  const int64_t gid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t row = sh_gpr >= 0 ? gid >> sh_gpr : gid / gpr;
  if (row >= A.n_rows) return;
  const int g = (int)(gid - row * gpr);
  const int64_t slot = A.tok[row];
  if (slot < 0) return;
  const int64_t blk = A.sh.BS >= 0 ? slot >> A.sh.BS : slot / L.BS;
  const int off = (int)(slot - blk * L.BS);
  const int bits = block_bits(A.pages, L, blk);
  RowWalk walk;
  walk.start(A.pages, L, A.sh.BS, blk, off, bits);
  const int h = qdiv(g, L.NG, sh_ng), gi = g - h * L.NG;
  const uint4* src = reinterpret_cast<const uint4*>(A.value + (row * A.v_s0 + h * A.v_s1 + gi * 32));
  const uint4 r0 = src[0], r1 = src[1], r2 = src[2], r3 = src[3];
  float x[4][8];
  cvt8<T>(r0, x[0]); cvt8<T>(r1, x[1]); cvt8<T>(r2, x[2]); cvt8<T>(r3, x[3]);
  float mn = INFINITY, mx = -INFINITY;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int k = 0; k < 8; k += 2) {
      mn = fminf(mn, fminf(x[c][k], x[c][k + 1]));
      mx = fmaxf(mx, fmaxf(x[c][k], x[c][k + 1]));
    }
  }
  const float levels = (float)((1 << bits) - 1);
  __half s16, m16;
  group_stats(mn, mx, levels, s16, m16);
  const float sc = __half2float(s16), m = __half2float(m16), rsc = __frcp_rn(sc);
  uint8_t* page = A.pages + blk * L.PS;
  const int64_t e = ((int64_t)off * L.H + h) * L.NG + gi;
  reinterpret_cast<__half*>(page + L.o_vs)[e] = s16;
  reinterpret_cast<__half*>(page + L.o_vm)[e] = m16;
  // V codes of the row start after the K codes of all heads; this group's are 4 * bits bytes
  uint8_t* dst = A.pages + walk.offset() + (L.H * L.D * bits) / 8 + h * ((L.D * bits) / 8) + gi * 4 * bits;
  if (bits == 4) {
    uint4 w;
    w.x = (uint32_t)quant_pack8<4, false>(x[0], &m, &sc, &rsc);
    w.y = (uint32_t)quant_pack8<4, false>(x[1], &m, &sc, &rsc);
    w.z = (uint32_t)quant_pack8<4, false>(x[2], &m, &sc, &rsc);
    w.w = (uint32_t)quant_pack8<4, false>(x[3], &m, &sc, &rsc);
    *reinterpret_cast<uint4*>(dst) = w;
  } else if (bits == 8) {
    const uint64_t a = quant_pack8<8, false>(x[0], &m, &sc, &rsc), b = quant_pack8<8, false>(x[1], &m, &sc, &rsc);
    const uint64_t c = quant_pack8<8, false>(x[2], &m, &sc, &rsc), d = quant_pack8<8, false>(x[3], &m, &sc, &rsc);
    reinterpret_cast<uint4*>(dst)[0] = make_uint4((uint32_t)a, (uint32_t)(a >> 32), (uint32_t)b, (uint32_t)(b >> 32));
    reinterpret_cast<uint4*>(dst)[1] = make_uint4((uint32_t)c, (uint32_t)(c >> 32), (uint32_t)d, (uint32_t)(d >> 32));
  } else {
    const uint32_t a = (uint32_t)quant_pack8<2, false>(x[0], &m, &sc, &rsc) |
                       ((uint32_t)quant_pack8<2, false>(x[1], &m, &sc, &rsc) << 16);
    const uint32_t b = (uint32_t)quant_pack8<2, false>(x[2], &m, &sc, &rsc) |
                       ((uint32_t)quant_pack8<2, false>(x[3], &m, &sc, &rsc) << 16);
    *reinterpret_cast<uint2*>(dst) = make_uint2(a, b);
  }
  // K side of the same 32 channels (few rows of a bulk write have any: open or sealed groups, the K_ref window)
  const int64_t rslot = A.tok[A.tok_s0 + row];
  const bool sealed = A.tok[2 * A.tok_s0 + row] != 0;
  const int64_t kidx = A.kref ? A.tok[3 * A.tok_s0 + row] : -1;
  if (rslot < 0 && !sealed && kidx < 0) return;
#pragma unroll 1
  for (int i = 0; i < 4; ++i) key_chunk<T>(A, row, (h * L.D + gi * 32) / 8 + i, off, bits, walk.offset(), rslot, sealed, kidx);
}

template <typename T, int MODE>
__global__ void __launch_bounds__(WT_WARPS * 32) write_tokens_kernel(const TokArgs<T> A) {
  const int64_t row = MODE == 2 ? (int64_t)blockIdx.x : blockIdx.x * (int64_t)WT_WARPS + (threadIdx.x >> 5);
  if (row >= A.n_rows) return;
  token_row<T, MODE>(A, row, false);
}

// One CTA per completed K group; each thread owns 8 channels of one head over the KG tokens
// (kernels/write.py:231-287).  SEAL: the group's first `fill` tokens come from residual slot
// `seal_slot` and header byte 1 is set (tiered_cache.py:379-394).  `raw16`: key rows and residual rows are
// 16-byte aligned rows of the same 16-bit type T, so both passes work on 16-byte words as loaded.
template <typename T>
struct FinArgs {
  LayoutDev L;
  uint8_t* pages;
  const T* key; int64_t k_s0, k_s1;
  const int64_t* fin; const int64_t* fin_count;
  const void* res; int res_dt; int64_t r_s0, r_s1, r_s2;
  bool vec_in, raw16;
  Shifts sh;
  int64_t seal_slot, seal_block;
  int seal_group, seal_fill, seal_bits, seal_mask;
};

// One K group: line `f` of the completed-group list, or (SEAL) the group the arguments name.
template <typename T, bool SEAL>
__device__ __forceinline__ void finalize_group(const FinArgs<T>& A, int64_t f) {
  const LayoutDev& L = A.L;
  uint8_t* __restrict__ pages = A.pages;
  const T* __restrict__ key = A.key;
  const int64_t k_s0 = A.k_s0, k_s1 = A.k_s1, r_s0 = A.r_s0, r_s1 = A.r_s1, r_s2 = A.r_s2;
  const void* res = A.res;
  const int res_dt = A.res_dt;
  const bool vec_in = A.vec_in, raw16 = A.raw16;
  const Shifts sh = A.sh;
  int64_t blk, rslot;
  int grp, ntok, bits;
  const int64_t* rows = nullptr;
  if constexpr (SEAL) {
    blk = A.seal_block; grp = A.seal_group; rslot = A.seal_slot; ntok = A.seal_fill; bits = A.seal_bits;
  } else {
    const int64_t* line = A.fin + f * (3 + L.KG);
    blk = line[0]; grp = (int)line[1]; rslot = line[2]; rows = line + 3; ntok = L.KG;
    bits = block_bits(pages, L, blk);
  }
  const float levels = (float)((1 << bits) - 1);
  const int head_bytes = (L.D * bits) / 8;
  uint8_t* page = pages + blk * L.PS;
  const int64_t rs = rslot < 0 ? 0 : rslot;

  for (int c = threadIdx.x; c < (L.H * L.D) / 8; c += blockDim.x) {
    const int h = qdiv(c * 8, L.D, sh.D), d0 = qmod(c * 8, L.D, sh.D);
    float mn[8], mx[8], x[8];
    auto load = [&](int p) {
      const int64_t r = SEAL ? -1 : rows[p];
      if (r >= 0) {
        ld8<T>(key, r * k_s0 + h * k_s1 + d0, vec_in, x);
      } else {
        const int64_t ro = rs * r_s0 + (int64_t)p * r_s1 + h * r_s2 + d0;
#pragma unroll
        for (int k = 0; k < 8; ++k) x[k] = ld_dt(res, res_dt, ro + k);
      }
    };
    // raw16 rows: key row indices and strides fit 32 bits (checked by the launcher), so a row's offset is one
    // 32 x 32 -> 64-bit multiply
    const T* kcol = key + (h * k_s1 + d0);
    const T* rcol = reinterpret_cast<const T*>(res) + (rs * r_s0 + h * r_s2 + d0);
    const int ks0 = (int)k_s0, rs1 = (int)r_s1;
    auto load_raw = [&](int p) -> uint4 {
      const int r = SEAL ? -1 : (int)rows[p];
      const T* src = r >= 0 ? kcol + (int64_t)r * ks0 : rcol + (int64_t)p * rs1;
      return *reinterpret_cast<const uint4*>(src);
    };
    if constexpr (sizeof(T) == 2) {
      if (raw16) {
        MinMax8<T> acc;
        acc.init();
#pragma unroll 4
        for (int p = 0; p < ntok; ++p) acc.update(load_raw(p));
        acc.finish(mn, mx);
      }
    }
    if (sizeof(T) != 2 || !raw16) {
#pragma unroll
      for (int k = 0; k < 8; ++k) { mn[k] = INFINITY; mx[k] = -INFINITY; }
      for (int p = 0; p < ntok; ++p) {
        load(p);
#pragma unroll
        for (int k = 0; k < 8; ++k) { mn[k] = fminf(mn[k], x[k]); mx[k] = fmaxf(mx[k], x[k]); }
      }
    }
    __align__(16) __half s16[8], m16[8];
    float sc[8], m[8], rsc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      group_stats(mn[k], mx[k], levels, s16[k], m16[k]);
      sc[k] = __half2float(s16[k]); m[k] = __half2float(m16[k]);
      rsc[k] = __frcp_rn(sc[k]);
    }
    const int64_t e = ((int64_t)grp * L.H + h) * L.D + d0;
    *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(page + L.o_ks) + e) = *reinterpret_cast<uint4*>(s16);
    *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(page + L.o_km) + e) = *reinterpret_cast<uint4*>(m16);
    RowWalk walk;
    walk.start(pages, L, sh.BS, blk, grp * L.KG, bits);
    const int col_bytes = h * head_bytes + (d0 * bits) / 8;
    bool done = false;
    if constexpr (sizeof(T) == 2) {
      if (raw16) {
        // the tier is fixed for the group: one loop per tier, the row's address advanced by additions
        auto codes = [&](auto BITS) {
          uint8_t* dst = pages + walk.offset() + col_bytes;
          for (int p = 0; p < ntok; ++p) {
            cvt8<T>(load_raw(p), x);
            store_packed8(dst, quant_pack8<decltype(BITS)::value, true>(x, m, sc, rsc), decltype(BITS)::value);
            if (p + 1 < ntok) {
              if (walk.r + 1 == walk.tpc) { walk.next(pages, L); dst = pages + walk.offset() + col_bytes; }
              else { ++walk.r; dst += walk.row_bytes; }
            }
          }
        };
        if (bits == 4) codes(std::integral_constant<int, 4>{});
        else if (bits == 8) codes(std::integral_constant<int, 8>{});
        else codes(std::integral_constant<int, 2>{});
        done = true;
      }
    }
    if (!done) {
      for (int p = 0; p < ntok; ++p) {
        load(p);
        quant_store8<true>(bits, pages + walk.offset() + col_bytes, x, m, sc, rsc);
        if (p + 1 < ntok) walk.next(pages, L);
      }
    }
  }
  if constexpr (SEAL) {
    if (threadIdx.x == 0) page[1] = (uint8_t)A.seal_mask;
  }
}

template <typename T, bool SEAL>
__global__ void __launch_bounds__(256, 4) finalize_k_kernel(const FinArgs<T> A) {
  if constexpr (!SEAL) {
    if ((int64_t)blockIdx.x >= *A.fin_count) return;
  }
  finalize_group<T, SEAL>(A, blockIdx.x);
}

// A step's writes of one layer in one launch: CTAs [0, n_rows) store the token rows, the next n_fin_launch CTAs
// quantize the completed K groups (masked by the device-side count), the rest copy `stash_n` rows of `stash_src`
// (the canary's query rows) to `stash_dst`.  Run one after the other, the group pass comes first because a
// residual slot a completing group gives up may be taken by a new group in the same step; here the two run at
// once, so the CTA of a token row whose slot a completing group still reads leaves that key alone, and the
// group's CTA stores it after its own last read of the slot.
struct StashArgs {
  const uint4* src; int64_t src_stride16;
  const int64_t* rows; int64_t n;
  uint4* dst; int row16;
};
constexpr int STEP_MAX_ROWS = 1024;

template <typename T>
__global__ void __launch_bounds__(WT_WARPS * 32)
write_step_kernel(const TokArgs<T> TA, const FinArgs<T> FA, int64_t n_fin_launch, const StashArgs SA) {
  __shared__ int take[STEP_MAX_ROWS];
  __shared__ int n_take;
  pdl_launch_dependents();
  pdl_wait();
  const LayoutDev& L = TA.L;
  const int64_t b = blockIdx.x;
  const int w = 3 + L.KG;
  if (b < TA.n_rows) {
    if (TA.tok[b] < 0) return;  // padding, or a token that is not stored
    const int64_t rslot = TA.tok[TA.tok_s0 + b];
    bool skip = false;
    if (rslot >= 0) {
      const int64_t n_fin = n_fin_launch > 0 ? min(*FA.fin_count, n_fin_launch) : 0;  // no list, no pointer
      int hit = 0;
      for (int64_t f = threadIdx.x; f < n_fin; f += blockDim.x) hit |= FA.fin[f * w + 2] == rslot;
      skip = __syncthreads_or(hit) != 0;
    }
    token_row<T, 2>(TA, b, skip);
    return;
  }
  if (b < TA.n_rows + n_fin_launch) {
    const int64_t f = b - TA.n_rows;
    if (f >= *FA.fin_count) return;
    const int64_t slot = FA.fin[f * w + 2];
    if (threadIdx.x == 0) n_take = 0;
    __syncthreads();
    if (slot >= 0) {
      for (int r = threadIdx.x; r < (int)TA.n_rows; r += blockDim.x)
        if (TA.tok[r] >= 0 && TA.tok[TA.tok_s0 + r] == slot) take[atomicAdd(&n_take, 1)] = r;
    }
    __syncthreads();
    finalize_group<T, false>(FA, f);
    // Keys of the group that takes the slot over: each thread stores the channels it has just read for the last time.
    const int units = (L.H * L.D) / 8;
    for (int i = 0; i < n_take; ++i) {
      const int64_t row = take[i];
      const int64_t tslot = TA.tok[row];
      const int off = (int)(tslot - (TA.sh.BS >= 0 ? tslot >> TA.sh.BS : tslot / L.BS) * L.BS);
      const int gpos = qmod(off, L.KG, TA.sh.KG);
      for (int c = threadIdx.x; c < units; c += blockDim.x) {
        const int h = qdiv(c * 8, L.D, TA.sh.D), d0 = qmod(c * 8, L.D, TA.sh.D);
        const int64_t src = row * TA.k_s0 + h * TA.k_s1 + d0;
        const int64_t ro = slot * TA.r_s0 + (int64_t)gpos * TA.r_s1 + h * TA.r_s2 + d0;
        if (TA.res_raw) {
          *reinterpret_cast<uint4*>(reinterpret_cast<T*>(TA.res) + ro) = *reinterpret_cast<const uint4*>(TA.key + src);
        } else {
          float x[8];
          ld8<T>(TA.key, src, TA.vec_in, x);
#pragma unroll
          for (int k = 0; k < 8; ++k) st_dt(TA.res, TA.res_dt, ro + k, x[k]);
        }
      }
    }
    return;
  }
  const int64_t i = (b - TA.n_rows - n_fin_launch) * blockDim.x + threadIdx.x;
  if (i >= SA.n * SA.row16) return;
  const int64_t r = i / SA.row16;
  SA.dst[i] = SA.src[SA.rows[r] * SA.src_stride16 + (i - r * SA.row16)];
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
static bool vec_ok(const void* a, int64_t s0, int64_t s1) {
  const int64_t unit = 16 / (int64_t)sizeof(T);  // elements per 16 bytes
  return aligned16(a) && s0 % unit == 0 && s1 % unit == 0;
}

template <typename T> constexpr int dtype_code() {
  return std::is_same<T, float>::value ? ECHOKV_DT_F32 : (std::is_same<T, __half>::value ? ECHOKV_DT_F16 : ECHOKV_DT_BF16);
}

// The residual buffer holds rows of the 16-bit type T, every one on a 16-byte boundary.
template <typename T>
static bool residual_raw(const ResidualDev& R) {
  return sizeof(T) == 2 && R.base && R.dtype == dtype_code<T>() && aligned16(R.base) && R.s_slot % 8 == 0 &&
         R.s_pos % 8 == 0 && R.s_head % 8 == 0;
}

static bool shuffle_ok(const LayoutDev& L) {  // the V group's min / max can be reduced over VG / 8 neighbouring lanes
  const int upg = L.VG / 8;
  return L.VG % 8 == 0 && upg <= 32 && (upg & (upg - 1)) == 0 && L.D % L.VG == 0;
}

template <typename T>
static TokArgs<T> tok_args(const LayoutDev& L, const echokv_pages* pages, const ResidualDev& R, const void* key,
                           int64_t k_s0, int64_t k_s1, const void* value, int64_t v_s0, int64_t v_s1,
                           const int64_t* tok, int64_t tok_s0, float* kref, int64_t kref_s0, int64_t kref_s1,
                           int64_t n_rows) {
  TokArgs<T> A;
  A.L = L; A.pages = (uint8_t*)pages->base;
  A.key = (const T*)key; A.k_s0 = k_s0; A.k_s1 = k_s1;
  A.value = (const T*)value; A.v_s0 = v_s0; A.v_s1 = v_s1;
  A.tok = tok; A.tok_s0 = tok_s0;
  A.res = const_cast<void*>(R.base); A.res_dt = R.dtype; A.r_s0 = R.s_slot; A.r_s1 = R.s_pos; A.r_s2 = R.s_head;
  A.kref = kref; A.kref_s0 = kref_s0; A.kref_s1 = kref_s1;
  A.n_rows = n_rows;
  A.vec_in = vec_ok<T>(key, k_s0, k_s1) && vec_ok<T>(value, v_s0, v_s1);
  A.res_raw = residual_raw<T>(R) && vec_ok<T>(key, k_s0, k_s1);
  A.kref_vec = kref && aligned16(kref) && kref_s0 % 4 == 0 && kref_s1 % 4 == 0;
  A.sh = make_shifts(L);
  return A;
}

template <typename T>
static FinArgs<T> fin_args(const LayoutDev& L, const echokv_pages* pages, const ResidualDev& R, const void* key,
                           int64_t k_s0, int64_t k_s1, const int64_t* fin, const int64_t* fin_count) {
  FinArgs<T> A;
  A.L = L; A.pages = (uint8_t*)pages->base;
  A.key = (const T*)key; A.k_s0 = k_s0; A.k_s1 = k_s1;
  A.fin = fin; A.fin_count = fin_count;
  A.res = R.base; A.res_dt = R.dtype; A.r_s0 = R.s_slot; A.r_s1 = R.s_pos; A.r_s2 = R.s_head;
  A.vec_in = key && vec_ok<T>(key, k_s0, k_s1);
  A.raw16 = A.vec_in && residual_raw<T>(R) && k_s0 < (1ll << 31) && R.s_pos < (1ll << 31);
  A.sh = make_shifts(L);
  A.seal_slot = 0; A.seal_block = 0; A.seal_group = 0; A.seal_fill = 0; A.seal_bits = 0; A.seal_mask = 0;
  return A;
}

}  // namespace echokv

using namespace echokv;

extern "C" {

int echokv_gather_rows(const void* src, int64_t src_row_stride_bytes, const int64_t* rows, int64_t n, void* dst,
                       int64_t row_bytes, void* stream) {
  if (n <= 0 || row_bytes <= 0) return ECHOKV_OK;
  if (!src || !rows || !dst) return set_error(ECHOKV_E_ARGUMENT, "gather_rows: null pointer");
  if (row_bytes % 16 || src_row_stride_bytes % 16 || !aligned16(src) || !aligned16(dst))
    return set_error(ECHOKV_E_ARGUMENT, "gather_rows: rows must be 16-byte aligned multiples of 16 bytes");
  const int row16 = (int)(row_bytes / 16);
  const int64_t total = n * row16;
  gather_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src, src_row_stride_bytes / 16, rows, (uint4*)dst, n, row16);
  return check_launch("gather_rows");
}

int echokv_write_headers(const echokv_pages* pages, const int64_t* blocks, const uint8_t* headers, int64_t n,
                         void* stream) {
  if (n <= 0) return ECHOKV_OK;
  if (!pages || !pages->base || !blocks || !headers) return set_error(ECHOKV_E_ARGUMENT, "write_headers: null pointer");
  if (!aligned16(headers) || !aligned16(pages->base) || pages->page_stride_bytes % 16)
    return set_error(ECHOKV_E_ARGUMENT, "write_headers: headers and pages must be 16-byte aligned");
  write_headers_kernel<<<(unsigned)((n + 127) / 128), 128, 0, (cudaStream_t)stream>>>(
      (uint8_t*)pages->base, pages->page_stride_bytes, blocks, headers, n);
  return check_launch("write_headers");
}

int echokv_scatter_i64(int64_t* dst, const int64_t* idx, const int64_t* val, int64_t n, void* stream) {
  if (n <= 0) return ECHOKV_OK;
  if (!dst || !idx || !val) return set_error(ECHOKV_E_ARGUMENT, "scatter_i64: null pointer");
  scatter_i64_kernel<<<(unsigned)((n + 127) / 128), 128, 0, (cudaStream_t)stream>>>(dst, idx, val, n);
  return check_launch("scatter_i64");
}

int echokv_write_tokens(const echokv_layout* layout, const echokv_pages* pages, const void* key, int64_t k_s0,
                        int64_t k_s1, const void* value, int64_t v_s0, int64_t v_s1, int32_t kv_dtype,
                        const int64_t* tok, int64_t tok_s0, const echokv_residual* residual, float* kref,
                        int64_t kref_s0, int64_t kref_s1, int64_t n_rows, void* stream) {
  if (n_rows <= 0) return ECHOKV_OK;
  LayoutDev L;
  ResidualDev R;
  int rc = make_layout(layout, pages, &L);
  if (rc) return rc;
  rc = make_residual(residual, &R);
  if (rc) return rc;
  if (!key || !value || !tok) return set_error(ECHOKV_E_ARGUMENT, "write_tokens: null pointer");
  // few rows (a decode step): spread each row over a CTA to shorten the dependent chain; many rows
  // (prefill chunks): one warp per row keeps more rows in flight per SM
  const int mode = !shuffle_ok(L) ? 0 : (n_rows <= STEP_MAX_ROWS ? 2 : 1);
  const unsigned grid = mode == 2 ? (unsigned)n_rows : (unsigned)((n_rows + WT_WARPS - 1) / WT_WARPS);
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH(T)                                                                                                   \
  {                                                                                                                 \
    TokArgs<T> A = tok_args<T>(L, pages, R, key, k_s0, k_s1, value, v_s0, v_s1, tok, tok_s0, kref, kref_s0,         \
                               kref_s1, n_rows);                                                                    \
    if (mode == 1 && sizeof(T) == 2 && A.vec_in && L.VG == 32 && L.D % 32 == 0) {                                   \
      const int gpr = L.H * L.NG;                                                                                   \
      const int64_t threads = n_rows * gpr;                                                                         \
      write_tokens_bulk_kernel<T><<<(unsigned)((threads + 127) / 128), 128, 0, st>>>(A, gpr, log2_or_neg(gpr),      \
                                                                                      log2_or_neg(L.NG));           \
    } else                                                                                                          \
    if (mode == 2) write_tokens_kernel<T, 2><<<grid, WT_WARPS * 32, 0, st>>>(A);                                    \
    else if (mode == 1) write_tokens_kernel<T, 1><<<grid, WT_WARPS * 32, 0, st>>>(A);                               \
    else write_tokens_kernel<T, 0><<<grid, WT_WARPS * 32, 0, st>>>(A);                                              \
  }
  switch (kv_dtype) {
    case ECHOKV_DT_F32: LAUNCH(float); break;
    case ECHOKV_DT_F16: LAUNCH(__half); break;
    case ECHOKV_DT_BF16: LAUNCH(__nv_bfloat16); break;
    default: return set_error(ECHOKV_E_ARGUMENT, "write_tokens: bad dtype %d", kv_dtype);
  }
#undef LAUNCH
  return check_launch("write_tokens");
}

int echokv_finalize_k(const echokv_layout* layout, const echokv_pages* pages, const void* key, int64_t k_s0,
                      int64_t k_s1, int32_t kv_dtype, const int64_t* fin, const int64_t* fin_count,
                      const echokv_residual* residual, int64_t n_launch, void* stream) {
  if (n_launch <= 0) return ECHOKV_OK;
  LayoutDev L;
  ResidualDev R;
  int rc = make_layout(layout, pages, &L);
  if (rc) return rc;
  rc = make_residual(residual, &R);
  if (rc) return rc;
  if (!key || !fin || !fin_count) return set_error(ECHOKV_E_ARGUMENT, "finalize_k: null pointer");
  const int threads = (L.H * L.D / 8) < 256 ? ((L.H * L.D / 8 + 31) / 32 * 32) : 256;
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH(T) \
  finalize_k_kernel<T, false><<<(unsigned)n_launch, threads, 0, st>>>(fin_args<T>(L, pages, R, key, k_s0, k_s1, fin, fin_count))
  switch (kv_dtype) {
    case ECHOKV_DT_F32: LAUNCH(float); break;
    case ECHOKV_DT_F16: LAUNCH(__half); break;
    case ECHOKV_DT_BF16: LAUNCH(__nv_bfloat16); break;
    default: return set_error(ECHOKV_E_ARGUMENT, "finalize_k: bad dtype %d", kv_dtype);
  }
#undef LAUNCH
  return check_launch("finalize_k");
}

int echokv_seal_group(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                      int64_t slot, int64_t block, int32_t group, int32_t fill, int32_t bits, int32_t sealed_mask,
                      void* stream) {
  if (fill <= 0) return ECHOKV_OK;
  LayoutDev L;
  ResidualDev R;
  int rc = make_layout(layout, pages, &L);
  if (rc) return rc;
  rc = make_residual(residual, &R);
  if (rc) return rc;
  if (!(bits == 2 || bits == 4 || bits == 8) || fill > L.KG || group < 0 || group >= L.KGPB || block < 0 ||
      block >= L.NB || slot < 0)
    return set_error(ECHOKV_E_ARGUMENT, "seal_group: bad slot/block/group/fill/bits");
  const int threads = (L.H * L.D / 8) < 256 ? ((L.H * L.D / 8 + 31) / 32 * 32) : 256;
  FinArgs<float> A = fin_args<float>(L, pages, R, nullptr, 0, 0, nullptr, nullptr);
  A.vec_in = false; A.raw16 = false;
  A.seal_slot = slot; A.seal_block = block; A.seal_group = group; A.seal_fill = fill; A.seal_bits = bits;
  A.seal_mask = sealed_mask;
  finalize_k_kernel<float, true><<<1, threads, 0, (cudaStream_t)stream>>>(A);
  return check_launch("seal_group");
}

int echokv_write_step(const echokv_layout* layout, const echokv_pages* pages, const void* key, int64_t k_s0,
                      int64_t k_s1, const void* value, int64_t v_s0, int64_t v_s1, int32_t kv_dtype,
                      const int64_t* tok, int64_t tok_s0, const echokv_residual* residual, float* kref,
                      int64_t kref_s0, int64_t kref_s1, int64_t n_rows, const int64_t* fin, const int64_t* fin_count,
                      int64_t n_fin_launch, const void* stash_src, int64_t stash_src_row_stride_bytes,
                      const int64_t* stash_rows, int64_t stash_n, void* stash_dst, int64_t stash_row_bytes,
                      void* stream) {
  LayoutDev L;
  ResidualDev R;
  int rc = make_layout(layout, pages, &L);
  if (rc) return rc;
  rc = make_residual(residual, &R);
  if (rc) return rc;
  if (n_fin_launch < 0) n_fin_launch = 0;
  if (stash_n < 0 || !stash_src) stash_n = 0;
  const bool stash_vec = stash_n == 0 || (stash_rows && stash_dst && stash_row_bytes > 0 && stash_row_bytes % 16 == 0 &&
                                          stash_src_row_stride_bytes % 16 == 0 && aligned16(stash_src) && aligned16(stash_dst));
  if (n_rows <= 0 || n_rows > STEP_MAX_ROWS || !shuffle_ok(L) || !stash_vec || (n_fin_launch > 0 && (!fin || !fin_count))) {
    // shapes the one-launch kernel does not take: the same work as three launches
    rc = echokv_finalize_k(layout, pages, key, k_s0, k_s1, kv_dtype, fin, fin_count, residual, n_fin_launch, stream);
    if (rc) return rc;
    rc = echokv_write_tokens(layout, pages, key, k_s0, k_s1, value, v_s0, v_s1, kv_dtype, tok, tok_s0, residual, kref,
                             kref_s0, kref_s1, n_rows, stream);
    if (rc) return rc;
    return echokv_gather_rows(stash_src, stash_src_row_stride_bytes, stash_rows, stash_n, stash_dst, stash_row_bytes, stream);
  }
  if (!key || !value || !tok) return set_error(ECHOKV_E_ARGUMENT, "write_step: null pointer");
  StashArgs SA;
  SA.src = (const uint4*)stash_src; SA.src_stride16 = stash_src_row_stride_bytes / 16; SA.rows = stash_rows;
  SA.n = stash_n; SA.dst = (uint4*)stash_dst; SA.row16 = (int)(stash_row_bytes / 16);
  const int64_t stash_ctas = (stash_n * SA.row16 + WT_WARPS * 32 - 1) / (WT_WARPS * 32);
  const unsigned grid = (unsigned)(n_rows + n_fin_launch + stash_ctas);
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH(T)                                                                                                  \
  launch_pdl(write_step_kernel<T>, dim3(grid), dim3(WT_WARPS * 32), 0, st,                                         \
             tok_args<T>(L, pages, R, key, k_s0, k_s1, value, v_s0, v_s1, tok, tok_s0, kref, kref_s0, kref_s1, n_rows), \
             fin_args<T>(L, pages, R, key, k_s0, k_s1, fin, fin_count), n_fin_launch, SA)
  switch (kv_dtype) {
    case ECHOKV_DT_F32: LAUNCH(float); break;
    case ECHOKV_DT_F16: LAUNCH(__half); break;
    case ECHOKV_DT_BF16: LAUNCH(__nv_bfloat16); break;
    default: return set_error(ECHOKV_E_ARGUMENT, "write_step: bad dtype %d", kv_dtype);
  }
#undef LAUNCH
  return check_launch("write_step");
}

}  // extern "C"
