// Read-side dequantization kernels: arbitrary token gather (the store's oracle read), dense
// dequantization of whole contexts for chunked prefill, and LRU demotion to INT2.
#include "common.cuh"

namespace echokv {

// Dequantize 8 channels [d0, d0+8) of head h of token (blk, off): K and V as float.
// Mirrors TieredKVCache.gather (echokv_vllm/tiered_cache.py:451-478) / load_kv_tile
// (kernels/common.py:50-109): K comes from the residual when the token's group is the
// block's open group.  `zero_unopened`: blocks with tier 0 give zeros (gather) instead of
// being read as INT2 (the attention kernels).
__device__ __forceinline__ void dequant8(const LayoutDev& L, const ResidualDev& R, const uint8_t* pages, int64_t blk,
                                         int off, int h, int d0, bool zero_unopened, float (&k)[8], float (&v)[8]) {
  const uint8_t* page = pages + blk * L.PS;
  int bits = page[0];
  if (bits == 0) {
    if (zero_unopened) {
#pragma unroll
      for (int i = 0; i < 8; ++i) k[i] = v[i] = 0.f;
      return;
    }
    bits = 2;
  }
  const int64_t ro = row_offset(pages, L, blk, off, bits);
  const int side_bytes = (L.H * L.D * bits) / 8;
  const int head_bytes = (L.D * bits) / 8;
  const uint8_t* krow = pages + ro + h * head_bytes;
  const uint8_t* vrow = krow + side_bytes;
  // V: per-token stats per group of VG channels
  const int g = d0 / L.VG;
  const int64_t ve = ((int64_t)off * L.H + h) * L.NG + g;
  const float vs = __half2float(reinterpret_cast<const __half*>(page + L.o_vs)[ve]);
  const float vm = __half2float(reinterpret_cast<const __half*>(page + L.o_vm)[ve]);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __fadd_rn(__fmul_rn((float)extract_code(vrow, d0 + i, bits), vs), vm);
  // K
  const int grp = off / L.KG;
  const int64_t slot = R.block_res[blk];
  if (slot >= 0 && R.res_group[slot] == grp) {
    const int64_t o = slot * R.s_slot + (int64_t)(off % L.KG) * R.s_pos + h * R.s_head + d0;
#pragma unroll
    for (int i = 0; i < 8; ++i) k[i] = ld_dt(R.base, R.dtype, o + i);
  } else {
    const int64_t ke = ((int64_t)grp * L.H + h) * L.D + d0;
    const __half* ks = reinterpret_cast<const __half*>(page + L.o_ks) + ke;
    const __half* km = reinterpret_cast<const __half*>(page + L.o_km) + ke;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      k[i] = __fadd_rn(__fmul_rn((float)extract_code(krow, d0 + i, bits), __half2float(ks[i])), __half2float(km[i]));
  }
}

__global__ void gather_kernel(LayoutDev L, ResidualDev R, const uint8_t* __restrict__ pages,
                              const int64_t* __restrict__ blk, const int64_t* __restrict__ off, int64_t n,
                              float* __restrict__ k_out, float* __restrict__ v_out) {
  const int cpt = (L.H * L.D) / 8;  // chunks per token
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= n * cpt) return;
  const int64_t i = idx / cpt;
  const int c = (int)(idx % cpt);
  const int h = (c * 8) / L.D, d0 = (c * 8) % L.D;
  float k[8], v[8];
  dequant8(L, R, pages, blk[i], (int)off[i], h, d0, true, k, v);
  float* ko = k_out + (i * L.H + h) * L.D + d0;
  float* vo = v_out + (i * L.H + h) * L.D + d0;
#pragma unroll
  for (int j = 0; j < 8; ++j) { ko[j] = k[j]; vo[j] = v[j]; }
}

// One CTA per work item (request, block index, dense row, ctx) -- kernels/prefill.py:329-369.
template <typename T>
__global__ void __launch_bounds__(256)
dequant_dense_kernel(LayoutDev L, ResidualDev R, const uint8_t* __restrict__ pages, const int32_t* __restrict__ work,
                     const int32_t* __restrict__ bt, int64_t bt_s0, T* __restrict__ k_out, T* __restrict__ v_out,
                     int64_t o_s0, int64_t o_s1) {
  const int32_t* w = work + blockIdx.x * 4;
  const int req = w[0], bi = w[1], ctx = w[3];
  const int64_t row0 = w[2];
  const int64_t blk = bt[(int64_t)req * bt_s0 + bi];
  const int nvalid = min(L.BS, ctx - bi * L.BS);
  const int cpt = (L.H * L.D) / 8;
  for (int idx = threadIdx.x; idx < nvalid * cpt; idx += blockDim.x) {
    const int t = idx / cpt, c = idx % cpt;
    const int h = (c * 8) / L.D, d0 = (c * 8) % L.D;
    float k[8], v[8];
    dequant8(L, R, pages, blk, t, h, d0, false, k, v);
    const int64_t o = (row0 + t) * o_s0 + h * o_s1 + d0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { Elem<T>::st(k_out, o + j, k[j]); Elem<T>::st(v_out, o + j, v[j]); }
  }
}

// The same for 16-bit outputs whose rows allow 16-byte stores and blocks of at most 64 tokens: one thread per
// (token, 8 channels) loads the 8 codes of each side as one word and the K stats as two 16-byte vectors, and
// stores 16 bytes of K and of V.  The arithmetic is dequant8's: code * scale + min in fp32, two roundings.
template <typename T> __device__ __forceinline__ uint32_t pack2_rn(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2_rn<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2_rn<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// 8 codes as floats.  A code c < 2^23 placed in the mantissa of 2^23 is the float 2^23 + c, and subtracting 2^23 is
// exact: two full-rate instructions per code instead of an integer-to-float conversion.
__device__ __forceinline__ float code_f32(uint32_t c) { return __uint_as_float(0x4B000000u | c) - 8388608.f; }
__device__ __forceinline__ void load_codes8(const uint8_t* p, int bits, float (&q)[8]) {
  if (bits == 8) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) { q[i] = code_f32((w.x >> (8 * i)) & 0xFFu); q[4 + i] = code_f32((w.y >> (8 * i)) & 0xFFu); }
  } else if (bits == 4) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = code_f32((w >> (4 * i)) & 0xFu);
  } else {
    const uint32_t w = *reinterpret_cast<const uint16_t*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = code_f32((w >> (2 * i)) & 0x3u);
  }
}

constexpr int DENSE_MAX_BS = 64;

template <typename T>
__global__ void __launch_bounds__(256)
dequant_dense_vec_kernel(LayoutDev L, ResidualDev R, const uint8_t* __restrict__ pages, const int32_t* __restrict__ work,
                         const int32_t* __restrict__ bt, int64_t bt_s0, T* __restrict__ k_out, T* __restrict__ v_out,
                         int64_t o_s0, int64_t o_s1) {
  __shared__ int64_t s_row[DENSE_MAX_BS];
  const int4 w = reinterpret_cast<const int4*>(work)[blockIdx.x];
  const int req = w.x, bi = w.y, ctx = w.w;
  const int64_t row0 = w.z;
  const int64_t blk = bt[(int64_t)req * bt_s0 + bi];
  const int nvalid = min(L.BS, ctx - bi * L.BS);
  const uint8_t* page = pages + blk * L.PS;
  int bits = page[0];
  if (bits == 0) bits = 2;  // an unopened block reads as INT2, like the attention kernels
  if ((int)threadIdx.x < nvalid) s_row[threadIdx.x] = row_offset(pages, L, blk, threadIdx.x, bits);
  const int64_t slot = R.block_res[blk];
  const int open_grp = slot >= 0 ? (int)R.res_group[slot] : -1;
  __syncthreads();
  const int cpt = (L.H * L.D) / 8, cph = L.D / 8;
  const int side_bytes = (L.H * L.D * bits) / 8;
  const __half* vs_p = reinterpret_cast<const __half*>(page + L.o_vs);
  const __half* vm_p = reinterpret_cast<const __half*>(page + L.o_vm);
  // (token, chunk) of this thread's items without a division per item: 256 items ahead is t_step tokens and
  // c_step chunks further
  const int t_step = 256 / cpt, c_step = 256 % cpt;
  int t = (int)threadIdx.x / cpt, c = (int)threadIdx.x % cpt;
  int h = c / cph, d0 = (c - h * cph) * 8;
#pragma unroll 4
  for (; t < nvalid; t += t_step) {
    const uint8_t* krow = pages + s_row[t] + (c * bits);  // 8 channels * bits / 8 bytes per chunk of 8
    float qk[8], qv[8];
    load_codes8(krow + side_bytes, bits, qv);
    const int64_t ve = ((int64_t)t * L.H + h) * L.NG + d0 / L.VG;
    const float vs = __half2float(vs_p[ve]), vm = __half2float(vm_p[ve]);
    const int grp = t / L.KG;
    float k[8];
    if (grp == open_grp) {
      const int64_t o = slot * R.s_slot + (int64_t)(t - grp * L.KG) * R.s_pos + h * R.s_head + d0;
#pragma unroll
      for (int i = 0; i < 8; ++i) k[i] = ld_dt(R.base, R.dtype, o + i);
    } else {
      load_codes8(krow, bits, qk);
      const int64_t ke = ((int64_t)grp * L.H + h) * L.D + d0;
      const uint4 s8 = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(page + L.o_ks) + ke);
      const uint4 m8 = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(page + L.o_km) + ke);
      const __half2* sh = reinterpret_cast<const __half2*>(&s8);
      const __half2* mh = reinterpret_cast<const __half2*>(&m8);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 sc = __half22float2(sh[i]), mn = __half22float2(mh[i]);
        k[2 * i] = __fadd_rn(__fmul_rn(qk[2 * i], sc.x), mn.x);
        k[2 * i + 1] = __fadd_rn(__fmul_rn(qk[2 * i + 1], sc.y), mn.y);
      }
    }
    uint4 ko, vo;
    uint32_t* kw = reinterpret_cast<uint32_t*>(&ko);
    uint32_t* vw = reinterpret_cast<uint32_t*>(&vo);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      kw[i] = pack2_rn<T>(k[2 * i], k[2 * i + 1]);
      vw[i] = pack2_rn<T>(__fadd_rn(__fmul_rn(qv[2 * i], vs), vm), __fadd_rn(__fmul_rn(qv[2 * i + 1], vs), vm));
    }
    const int64_t o = (row0 + t) * o_s0 + h * o_s1 + d0;
    *reinterpret_cast<uint4*>(k_out + o) = ko;
    *reinterpret_cast<uint4*>(v_out + o) = vo;
    if (c_step) {
      c += c_step;
      if (c >= cpt) { c -= cpt; ++t; }
      h = c / cph;
      d0 = (c - h * cph) * 8;
    }
  }
}

// Demotion, phase 2: requantize a block's dequantized contents (scratch: K then V, float
// [n, BS, H, D]) to INT2 into chunk 0 of its own page (tiered_cache.py:322-340).
__global__ void __launch_bounds__(256)
demote_requant_kernel(LayoutDev L, uint8_t* __restrict__ pages, const int64_t* __restrict__ victims, int64_t n,
                      const float* __restrict__ scratch) {
  const int64_t b = victims[blockIdx.x];
  const float* ksrc = scratch + (int64_t)blockIdx.x * L.BS * L.H * L.D;
  const float* vsrc = scratch + (n + blockIdx.x) * (int64_t)L.BS * L.H * L.D;
  uint8_t* page = pages + b * L.PS;
  const float levels = 3.f;
  const int bits = 2;
  const int side_bytes = (L.H * L.D * bits) / 8, head_bytes = (L.D * bits) / 8;
  const int64_t row_bytes = 2 * side_bytes;
  uint8_t* data = page + L.o_data;  // INT2: every token row lives in chunk 0 of the own page
  if (threadIdx.x == 0) page[0] = 2;
  // K: per channel over each group of KG tokens
  const int cph = (L.H * L.D) / 8;
  for (int idx = threadIdx.x; idx < L.KGPB * cph; idx += blockDim.x) {
    const int grp = idx / cph, c = idx % cph;
    const int h = (c * 8) / L.D, d0 = (c * 8) % L.D;
    float mn[8], mx[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { mn[k] = INFINITY; mx[k] = -INFINITY; }
    for (int p = 0; p < L.KG; ++p) {
      const float* x = ksrc + ((int64_t)(grp * L.KG + p) * L.H + h) * L.D + d0;
#pragma unroll
      for (int k = 0; k < 8; ++k) { mn[k] = fminf(mn[k], x[k]); mx[k] = fmaxf(mx[k], x[k]); }
    }
    __align__(16) __half s16[8], m16[8];
    float sc[8], m[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      group_stats(mn[k], mx[k], levels, s16[k], m16[k]);
      sc[k] = __half2float(s16[k]); m[k] = __half2float(m16[k]);
    }
    const int64_t e = ((int64_t)grp * L.H + h) * L.D + d0;
    *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(page + L.o_ks) + e) = *reinterpret_cast<uint4*>(s16);
    *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(page + L.o_km) + e) = *reinterpret_cast<uint4*>(m16);
    for (int p = 0; p < L.KG; ++p) {
      const int t = grp * L.KG + p;
      const float* x = ksrc + ((int64_t)t * L.H + h) * L.D + d0;
      uint32_t q[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) q[k] = quant_code(x[k], m[k], sc[k], levels);
      store_packed8(data + t * row_bytes + h * head_bytes + (d0 * bits) / 8, pack8(q, bits), bits);
    }
  }
  // V: per token, groups of VG channels
  for (int idx = threadIdx.x; idx < L.BS * L.H * L.NG; idx += blockDim.x) {
    const int t = idx / (L.H * L.NG), r = idx % (L.H * L.NG);
    const int h = r / L.NG, g = r % L.NG;
    const float* x = vsrc + ((int64_t)t * L.H + h) * L.D + g * L.VG;
    float mn = INFINITY, mx = -INFINITY;
    for (int c = 0; c < L.VG; ++c) { mn = fminf(mn, x[c]); mx = fmaxf(mx, x[c]); }
    __half s16, m16;
    group_stats(mn, mx, levels, s16, m16);
    const float sc = __half2float(s16), m = __half2float(m16);
    const int64_t e = ((int64_t)t * L.H + h) * L.NG + g;
    reinterpret_cast<__half*>(page + L.o_vs)[e] = s16;
    reinterpret_cast<__half*>(page + L.o_vm)[e] = m16;
    uint8_t* dst = data + t * row_bytes + side_bytes + h * head_bytes + (g * L.VG * bits) / 8;
    for (int c = 0; c < L.VG; c += 8) {
      uint32_t q[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) q[k] = quant_code(x[c + k], m, sc, levels);
      store_packed8(dst + (c * bits) / 8, pack8(q, bits), bits);
    }
  }
}

__global__ void demote_index_kernel(const int64_t* victims, int64_t n, int BS, int64_t* blk, int64_t* off) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n * BS) return;
  blk[i] = victims[i / BS];
  off[i] = i % BS;
}

}  // namespace echokv

using namespace echokv;

extern "C" {

int echokv_gather(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                  const int64_t* blk, const int64_t* off, int64_t n, float* k_out, float* v_out, void* stream) {
  if (n <= 0) return ECHOKV_OK;
  LayoutDev L;
  ResidualDev R;
  int rc = make_layout(layout, pages, &L);
  if (rc) return rc;
  rc = make_residual(residual, &R);
  if (rc) return rc;
  if (!blk || !off || !k_out || !v_out) return set_error(ECHOKV_E_ARGUMENT, "gather: null pointer");
  const int64_t total = n * (L.H * L.D / 8);
  gather_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      L, R, (const uint8_t*)pages->base, blk, off, n, k_out, v_out);
  return check_launch("gather");
}

int echokv_dequant_dense(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                         const int32_t* work, int64_t n_work, const int32_t* block_table, int64_t bt_s0, void* k_out,
                         void* v_out, int64_t out_s0, int64_t out_s1, int32_t out_dtype, void* stream) {
  if (n_work <= 0) return ECHOKV_OK;
  LayoutDev L;
  ResidualDev R;
  int rc = make_layout(layout, pages, &L);
  if (rc) return rc;
  rc = make_residual(residual, &R);
  if (rc) return rc;
  if (!work || !block_table || !k_out || !v_out) return set_error(ECHOKV_E_ARGUMENT, "dequant_dense: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH(T)                                                                                              \
  dequant_dense_kernel<T><<<(unsigned)n_work, 256, 0, st>>>(L, R, (const uint8_t*)pages->base, work, block_table, \
                                                           bt_s0, (T*)k_out, (T*)v_out, out_s0, out_s1)
  // 16-byte loads and stores need the stat arrays, the rows of the outputs and 8-channel chunks aligned
  const bool vec = out_dtype != ECHOKV_DT_F32 && L.BS <= DENSE_MAX_BS && L.D % 8 == 0 && L.VG % 8 == 0 &&
                   ((L.o_ks | L.o_km | L.PS | L.o_data | L.CB) % 16) == 0 && (out_s0 % 8) == 0 && (out_s1 % 8) == 0 &&
                   ((reinterpret_cast<uintptr_t>(k_out) | reinterpret_cast<uintptr_t>(v_out) |
                     reinterpret_cast<uintptr_t>(pages->base) | reinterpret_cast<uintptr_t>(work)) % 16) == 0;
#define LAUNCH_VEC(T)                                                                                              \
  dequant_dense_vec_kernel<T><<<(unsigned)n_work, 256, 0, st>>>(L, R, (const uint8_t*)pages->base, work, block_table, \
                                                               bt_s0, (T*)k_out, (T*)v_out, out_s0, out_s1)
  if (vec) {
    if (out_dtype == ECHOKV_DT_F16) LAUNCH_VEC(__half); else LAUNCH_VEC(__nv_bfloat16);
    return check_launch("dequant_dense");
  }
#undef LAUNCH_VEC
  switch (out_dtype) {
    case ECHOKV_DT_F32: LAUNCH(float); break;
    case ECHOKV_DT_F16: LAUNCH(__half); break;
    case ECHOKV_DT_BF16: LAUNCH(__nv_bfloat16); break;
    default: return set_error(ECHOKV_E_ARGUMENT, "dequant_dense: bad dtype %d", out_dtype);
  }
#undef LAUNCH
  return check_launch("dequant_dense");
}

int64_t echokv_demote_scratch_bytes(const echokv_layout* layout, int64_t n) {
  if (!layout || n <= 0) return 0;
  const int64_t tok = n * layout->block_size;
  // dequantized K and V (float) + the (blk, off) index of every token
  return tok * layout->num_kv_heads * layout->head_size * 2 * (int64_t)sizeof(float) + tok * 2 * (int64_t)sizeof(int64_t);
}

int echokv_demote_blocks(const echokv_layout* layout, const echokv_pages* pages, const echokv_residual* residual,
                         const int64_t* victims, int64_t n, void* scratch, int64_t scratch_bytes, void* stream) {
  if (n <= 0) return ECHOKV_OK;
  LayoutDev L;
  ResidualDev R;
  int rc = make_layout(layout, pages, &L);
  if (rc) return rc;
  rc = make_residual(residual, &R);
  if (rc) return rc;
  if (!victims || !scratch) return set_error(ECHOKV_E_ARGUMENT, "demote_blocks: null pointer");
  if (scratch_bytes < echokv_demote_scratch_bytes(layout, n) || (reinterpret_cast<uintptr_t>(scratch) & 15))
    return set_error(ECHOKV_E_ARGUMENT, "demote_blocks: scratch too small or misaligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t tok = n * L.BS;
  float* kf = (float*)scratch;
  float* vf = kf + tok * L.H * L.D;
  int64_t* bi = (int64_t*)(vf + tok * L.H * L.D);
  int64_t* oi = bi + tok;
  demote_index_kernel<<<(unsigned)((tok + 255) / 256), 256, 0, st>>>(victims, n, L.BS, bi, oi);
  const int64_t total = tok * (L.H * L.D / 8);
  gather_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(L, R, (const uint8_t*)pages->base, bi, oi, tok, kf, vf);
  demote_requant_kernel<<<(unsigned)n, 256, 0, st>>>(L, (uint8_t*)pages->base, victims, n, kf);
  return check_launch("demote_blocks");
}

}  // extern "C"
