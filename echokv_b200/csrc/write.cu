// Quantize-on-write kernels: token rows (V per token, K to residual / sealed codes / K_ref ring)
// and per-channel K groups.  Numerics follow echokv_vllm/quant.py bit for bit: fp16-rounded stats
// first, IEEE fp32 divide, round-half-to-even, clamp after rounding.
#include "common.cuh"

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

// Token rows (kernels/write.py:171-229 does one program per (row, head)).  WIDE: one CTA of four warps
// per row, a thread per 8 channels, the V group's min / max reduced over its VG / 8 neighbouring lanes
// by shuffles (needs VG / 8 to be a power of two <= 32); otherwise one warp per row, a lane per V group.
// Both produce the same bytes: min and max do not depend on the order of reduction.
template <typename T, bool WIDE>
__global__ void __launch_bounds__(WT_WARPS * 32)
write_tokens_kernel(LayoutDev L, uint8_t* __restrict__ pages, const T* __restrict__ key, int64_t k_s0, int64_t k_s1,
                    const T* __restrict__ value, int64_t v_s0, int64_t v_s1, const int64_t* __restrict__ tok,
                    int64_t tok_s0, void* res, int res_dt, int64_t r_s0, int64_t r_s1, int64_t r_s2,
                    float* __restrict__ kref, int64_t kref_s0, int64_t kref_s1, int64_t n_rows, bool vec_in) {
  const int lane = threadIdx.x & 31;
  const int64_t row = WIDE ? (int64_t)blockIdx.x : blockIdx.x * (int64_t)WT_WARPS + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int64_t slot = tok[row];
  if (slot < 0) return;  // padding, or a token that is not stored
  const int64_t blk = slot / L.BS;
  const int off = (int)(slot % L.BS);
  const int bits = block_bits(pages, L, blk);
  const float levels = (float)((1 << bits) - 1);
  const int64_t rowoff = row_offset(pages, L, blk, off, bits);
  const int side_bytes = (L.H * L.D * bits) / 8;
  const int head_bytes = (L.D * bits) / 8;
  uint8_t* page = pages + blk * L.PS;
  const int units = (L.H * L.D) / 8;  // 8-channel pieces of a row
  const int first = WIDE ? threadIdx.x : lane, step = WIDE ? WT_WARPS * 32 : 32;

  if constexpr (WIDE) {
    // V: per token, groups of VG along head_dim; VG / 8 neighbouring threads share a group.
    const int upg = L.VG / 8;
    for (int base = (threadIdx.x >> 5) * 32; base < units; base += step) {
      const int u = base + lane;
      const bool on = u < units;
      const int h = on ? (u * 8) / L.D : 0, d0 = on ? (u * 8) % L.D : 0;
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
      if (d0 % L.VG == 0) {
        const int64_t e = ((int64_t)off * L.H + h) * L.NG + d0 / L.VG;
        reinterpret_cast<__half*>(page + L.o_vs)[e] = s16;
        reinterpret_cast<__half*>(page + L.o_vm)[e] = m16;
      }
      const float rsc = __frcp_rn(sc);
      uint32_t q[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) q[k] = quant_code_r(x[k], m, sc, rsc, levels);
      store_packed8(pages + rowoff + side_bytes + h * head_bytes + (d0 * bits) / 8, pack8(q, bits), bits);
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
        uint32_t q[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) q[k] = quant_code_r(x[k], m, sc, rsc, levels);
        store_packed8(dst + (c * bits) / 8, pack8(q, bits), bits);
      }
    }
  }

  // K: residual row (open group), codes under stored stats (sealed group), K_ref ring row.
  const int64_t rslot = tok[tok_s0 + row];
  const bool sealed = tok[2 * tok_s0 + row] != 0;
  const int64_t kidx = kref ? tok[3 * tok_s0 + row] : -1;
  if (rslot < 0 && !sealed && kidx < 0) return;
  const int grp = off / L.KG;
  for (int c = first; c < units; c += step) {
    const int h = (c * 8) / L.D, d0 = (c * 8) % L.D;
    float x[8];
    ld8<T>(key, row * k_s0 + h * k_s1 + d0, vec_in, x);
    if (rslot >= 0) {
      const int64_t ro = rslot * r_s0 + (int64_t)(off % L.KG) * r_s1 + h * r_s2 + d0;
#pragma unroll
      for (int k = 0; k < 8; ++k) st_dt(res, res_dt, ro + k, x[k]);
    }
    if (sealed) {
      const int64_t e = ((int64_t)grp * L.H + h) * L.D + d0;
      const __half* ks = reinterpret_cast<const __half*>(page + L.o_ks) + e;
      const __half* km = reinterpret_cast<const __half*>(page + L.o_km) + e;
      uint32_t q[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) q[k] = quant_code(x[k], __half2float(km[k]), __half2float(ks[k]), levels);
      store_packed8(pages + rowoff + h * head_bytes + (d0 * bits) / 8, pack8(q, bits), bits);
    }
    if (kidx >= 0) {
      float* dst = kref + kidx * kref_s0 + h * kref_s1 + d0;
#pragma unroll
      for (int k = 0; k < 8; ++k) dst[k] = x[k];
    }
  }
}

// One CTA per completed K group; each thread owns 8 channels of one head over the KG tokens
// (kernels/write.py:231-287).  SEAL: the group's first `fill` tokens come from residual slot
// `seal_slot` and header byte 1 is set (tiered_cache.py:379-394).
template <typename T, bool SEAL>
__global__ void __launch_bounds__(256)
finalize_k_kernel(LayoutDev L, uint8_t* __restrict__ pages, const T* __restrict__ key, int64_t k_s0, int64_t k_s1,
                  const int64_t* __restrict__ fin, const int64_t* __restrict__ fin_count, const void* res, int res_dt,
                  int64_t r_s0, int64_t r_s1, int64_t r_s2, bool vec_in, int64_t seal_slot, int64_t seal_block,
                  int seal_group, int seal_fill, int seal_bits, int seal_mask) {
  int64_t blk, rslot;
  int grp, ntok, bits;
  const int64_t* rows = nullptr;
  if constexpr (SEAL) {
    blk = seal_block; grp = seal_group; rslot = seal_slot; ntok = seal_fill; bits = seal_bits;
  } else {
    const int64_t f = blockIdx.x;
    if (f >= *fin_count) return;
    const int64_t* line = fin + f * (3 + L.KG);
    blk = line[0]; grp = (int)line[1]; rslot = line[2]; rows = line + 3; ntok = L.KG;
    bits = block_bits(pages, L, blk);
  }
  const float levels = (float)((1 << bits) - 1);
  const int head_bytes = (L.D * bits) / 8;
  uint8_t* page = pages + blk * L.PS;
  const int64_t rs = rslot < 0 ? 0 : rslot;

  for (int c = threadIdx.x; c < (L.H * L.D) / 8; c += blockDim.x) {
    const int h = (c * 8) / L.D, d0 = (c * 8) % L.D;
    float mn[8], mx[8], x[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { mn[k] = INFINITY; mx[k] = -INFINITY; }
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
    for (int p = 0; p < ntok; ++p) {
      load(p);
#pragma unroll
      for (int k = 0; k < 8; ++k) { mn[k] = fminf(mn[k], x[k]); mx[k] = fmaxf(mx[k], x[k]); }
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
    for (int p = 0; p < ntok; ++p) {
      load(p);
      uint32_t q[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) q[k] = quant_code_r(x[k], m[k], sc[k], rsc[k], levels);
      const int64_t ro = row_offset(pages, L, blk, grp * L.KG + p, bits);
      store_packed8(pages + ro + h * head_bytes + (d0 * bits) / 8, pack8(q, bits), bits);
    }
  }
  if constexpr (SEAL) {
    if (threadIdx.x == 0) page[1] = (uint8_t)seal_mask;
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
static bool vec_ok(const void* a, int64_t s0, int64_t s1) {
  const int64_t q = 16 / (int64_t)sizeof(T) * (sizeof(T) == 4 ? 2 : 1);  // elements per 8-chunk alignment unit
  (void)q;
  const int64_t unit = 16 / (int64_t)sizeof(T);  // elements per 16 bytes
  return aligned16(a) && s0 % unit == 0 && s1 % unit == 0;
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
  const int upg = L.VG / 8;  // 8-channel pieces per V group
  // few rows (a decode step): spread each row over a CTA to shorten the dependent chain; many rows
  // (prefill chunks): one warp per row keeps more rows in flight per SM
  const bool wide = n_rows <= 1024 && L.VG % 8 == 0 && upg <= 32 && (upg & (upg - 1)) == 0 && L.D % L.VG == 0;
  const unsigned grid = wide ? (unsigned)n_rows : (unsigned)((n_rows + WT_WARPS - 1) / WT_WARPS);
  cudaStream_t st = (cudaStream_t)stream;
#define ARGS(T)                                                                                                \
      L, (uint8_t*)pages->base, (const T*)key, k_s0, k_s1, (const T*)value, v_s0, v_s1, tok, tok_s0,            \
      const_cast<void*>(R.base), R.dtype, R.s_slot, R.s_pos, R.s_head, kref, kref_s0, kref_s1, n_rows,          \
      vec_ok<T>(key, k_s0, k_s1) && vec_ok<T>(value, v_s0, v_s1)
#define LAUNCH(T)                                                                       \
  if (wide) write_tokens_kernel<T, true><<<grid, WT_WARPS * 32, 0, st>>>(ARGS(T));      \
  else write_tokens_kernel<T, false><<<grid, WT_WARPS * 32, 0, st>>>(ARGS(T))
  switch (kv_dtype) {
    case ECHOKV_DT_F32: LAUNCH(float); break;
    case ECHOKV_DT_F16: LAUNCH(__half); break;
    case ECHOKV_DT_BF16: LAUNCH(__nv_bfloat16); break;
    default: return set_error(ECHOKV_E_ARGUMENT, "write_tokens: bad dtype %d", kv_dtype);
  }
#undef LAUNCH
#undef ARGS
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
#define LAUNCH(T)                                                                                            \
  finalize_k_kernel<T, false><<<(unsigned)n_launch, threads, 0, st>>>(                                       \
      L, (uint8_t*)pages->base, (const T*)key, k_s0, k_s1, fin, fin_count, R.base, R.dtype, R.s_slot, R.s_pos, \
      R.s_head, vec_ok<T>(key, k_s0, k_s1), 0, 0, 0, 0, 0, 0)
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
  finalize_k_kernel<float, true><<<1, threads, 0, (cudaStream_t)stream>>>(
      L, (uint8_t*)pages->base, nullptr, 0, 0, nullptr, nullptr, R.base, R.dtype, R.s_slot, R.s_pos, R.s_head, false,
      slot, block, group, fill, bits, sealed_mask);
  return check_launch("seal_group");
}

}  // extern "C"
