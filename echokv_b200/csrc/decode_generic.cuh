// Generic split-K paged decode attention on CUDA cores: any tier mix, any head size that is a
// multiple of 32 up to 256, up to 16 query heads per KV head.  It is the correctness baseline and
// the path for shapes the tensor-core kernel is not instantiated for.
//
// One CTA of 4 warps per (sequence, KV head, split); warp w takes blocks b_start + w, + 4, ...
// Each 32-token tile runs in two phases: lanes own tokens for Q.K^T (full-row dot products, one
// warp max / sum per query head), then lanes own channels for P.V.  The 4 warps' partial
// (m, l, acc) are merged in warp order, and splits in split order, so a sequence's result is a
// function of its own length only (batch-invariant, as kernels/decode.py:66-73 requires).
#pragma once

#include "common.cuh"

namespace echokv {

constexpr int DG_WARPS = 4;

struct DecodeArgs {
  const void* q; int64_t q_s0, q_s1; int q_dt;
  const int64_t* q_rows;
  const int32_t* bt; int64_t bt_s0;
  const int64_t* bt_rows;
  const int64_t* lens;
  float* acc;   // [S, Hq, splits, D]
  float* ml;    // [S, Hq, splits, 2]  (m in the log2 domain, l)
  void* out; int64_t o_s0, o_s1; int out_dt;
  float scale_log2e;
  int num_splits, bps_min, gqa, Hq;
  const int32_t* bps_dev;  // optional: blocks per split chosen by the host for this step, read at run time
  int* state;              // work-queue state at the start of the scratch: [0] = the split kernel's item counter
};

// Lower bound of a split's size in blocks: the call's argument, raised by the run-time value when there is one.
__device__ __forceinline__ int bps_floor(const DecodeArgs& A) {
  return A.bps_dev ? max(A.bps_min, (int)__ldg(A.bps_dev)) : A.bps_min;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Split rule of kernels/decode.py:166-172.
__device__ __forceinline__ bool split_range(int64_t seq_len, int BS, int num_splits, int bps_min, int split,
                                            int& b_start, int& b_end) {
  const int n_blocks = (int)((seq_len + BS - 1) / BS);
  const int bps = max(bps_min, (n_blocks + num_splits - 1) / num_splits);
  b_start = split * bps;
  if (b_start >= n_blocks) return false;
  b_end = min(b_start + bps, n_blocks);
  return true;
}

template <int GQ, int CH>
__global__ void __launch_bounds__(DG_WARPS * 32)
decode_generic_kernel(LayoutDev L, ResidualDev R, const uint8_t* __restrict__ pages, DecodeArgs A) {
  constexpr int D = CH * 32;
  const int seq = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int64_t seq_len = A.lens[seq];
  int b_start, b_end;
  if (!split_range(seq_len, L.BS, A.num_splits, bps_floor(A), split, b_start, b_end)) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t q_row = A.q_rows ? A.q_rows[seq] : seq;
  const int64_t bt_row = A.bt_rows ? A.bt_rows[seq] : seq;

  constexpr int SMEM_A = GQ * D * 4 + DG_WARPS * GQ * 32 * 4 + DG_WARPS * 32 * 8;
  constexpr int SMEM_B = DG_WARPS * GQ * (D + 2) * 4;
  __shared__ __align__(16) unsigned char smem[SMEM_A > SMEM_B ? SMEM_A : SMEM_B];
  float* qs = reinterpret_cast<float*>(smem);                          // [GQ][D], pre-scaled
  float* ps = qs + GQ * D + warp * GQ * 32;                            // [GQ][32] this warp
  int64_t* rowoff = reinterpret_cast<int64_t*>(qs + GQ * D + DG_WARPS * GQ * 32) + warp * 32;

  for (int i = threadIdx.x; i < GQ * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    qs[i] = g < A.gqa ? ld_dt(A.q, A.q_dt, q_row * A.q_s0 + (int64_t)(h * A.gqa + g) * A.q_s1 + d) * A.scale_log2e
                      : 0.f;
  }
  __syncthreads();

  float m[GQ], l[GQ], acc[GQ][CH];
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) acc[g][c] = 0.f;
  }

  for (int bi = b_start + warp; bi < b_end; bi += DG_WARPS) {
    const int64_t blk = A.bt[bt_row * A.bt_s0 + bi];
    const uint8_t* page = pages + blk * L.PS;
    const int bits = block_bits(pages, L, blk);
    const int n_valid = (int)min((int64_t)L.BS, seq_len - (int64_t)bi * L.BS);
    const int64_t rslot = R.block_res[blk];
    const int rgrp = rslot >= 0 ? (int)R.res_group[rslot] : -1;
    const int side_bytes = (L.H * D * bits) / 8, head_bytes = (D * bits) / 8;
    const uint32_t cmask = (1u << bits) - 1u;

    for (int t0 = 0; t0 < n_valid; t0 += 32) {
      const int t = t0 + lane;
      const bool valid = t < n_valid;
      float s[GQ];
#pragma unroll
      for (int g = 0; g < GQ; ++g) s[g] = 0.f;
      if (valid) {
        const int64_t ro = row_offset(pages, L, blk, t, bits);
        rowoff[lane] = ro;
        const int grp = t / L.KG;
        const bool in_res = rslot >= 0 && grp == rgrp;
        const uint8_t* krow = pages + ro + h * head_bytes;
        const __half* ksp = reinterpret_cast<const __half*>(page + L.o_ks) + ((int64_t)grp * L.H + h) * D;
        const __half* kmp = reinterpret_cast<const __half*>(page + L.o_km) + ((int64_t)grp * L.H + h) * D;
        const int64_t reso = rslot * R.s_slot + (int64_t)(t % L.KG) * R.s_pos + h * R.s_head;
        for (int d0 = 0; d0 < D; d0 += 8) {
          float k[8];
          if (in_res) {
#pragma unroll
            for (int i = 0; i < 8; ++i) k[i] = ld_dt(R.base, R.dtype, reso + d0 + i);
          } else {
            uint64_t raw;
            if (bits == 8) raw = *reinterpret_cast<const uint64_t*>(krow + d0);
            else if (bits == 4) raw = *reinterpret_cast<const uint32_t*>(krow + d0 / 2);
            else raw = *reinterpret_cast<const uint16_t*>(krow + d0 / 4);
            const uint4 sraw = *reinterpret_cast<const uint4*>(ksp + d0);
            const uint4 mraw = *reinterpret_cast<const uint4*>(kmp + d0);
            const __half* sh = reinterpret_cast<const __half*>(&sraw);
            const __half* mh = reinterpret_cast<const __half*>(&mraw);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float c = (float)((uint32_t)(raw >> (i * bits)) & cmask);
              k[i] = __fadd_rn(__fmul_rn(c, __half2float(sh[i])), __half2float(mh[i]));
            }
          }
#pragma unroll
          for (int g = 0; g < GQ; ++g) {
            const float4 qa = *reinterpret_cast<const float4*>(qs + g * D + d0);
            const float4 qb = *reinterpret_cast<const float4*>(qs + g * D + d0 + 4);
            s[g] += qa.x * k[0] + qa.y * k[1] + qa.z * k[2] + qa.w * k[3] + qb.x * k[4] + qb.y * k[5] +
                    qb.z * k[6] + qb.w * k[7];
          }
        }
      }
#pragma unroll
      for (int g = 0; g < GQ; ++g) {
        const float sv = valid ? s[g] : -INFINITY;
        const float m_new = fmaxf(m[g], warp_max(sv));
        const float alpha = exp2f(m[g] - m_new);
        const float p = valid ? exp2f(sv - m_new) : 0.f;
        l[g] = l[g] * alpha + warp_sum(p);
#pragma unroll
        for (int c = 0; c < CH; ++c) acc[g][c] *= alpha;
        ps[g * 32 + lane] = p;
        m[g] = m_new;
      }
      __syncwarp();
      const int ntile = min(32, n_valid - t0);
      const int d0 = lane * CH;
      const int vg = d0 / L.VG;
      for (int tt = 0; tt < ntile; ++tt) {
        const uint8_t* vrow = pages + rowoff[tt] + side_bytes + h * head_bytes;
        const int64_t ve = ((int64_t)(t0 + tt) * L.H + h) * L.NG + vg;
        const float vs = __half2float(reinterpret_cast<const __half*>(page + L.o_vs)[ve]);
        const float vm = __half2float(reinterpret_cast<const __half*>(page + L.o_vm)[ve]);
        float v[CH];
#pragma unroll
        for (int c = 0; c < CH; ++c) v[c] = __fadd_rn(__fmul_rn((float)extract_code(vrow, d0 + c, bits), vs), vm);
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
          const float p = ps[g * 32 + tt];
#pragma unroll
          for (int c = 0; c < CH; ++c) acc[g][c] += p * v[c];
        }
      }
      __syncwarp();
    }
  }

  // Merge the warps' partials in warp order (reuses the shared memory).
  __syncthreads();
  float* cacc = reinterpret_cast<float*>(smem);              // [W][GQ][D]
  float* cml = cacc + DG_WARPS * GQ * D;                     // [W][GQ][2]
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
#pragma unroll
    for (int c = 0; c < CH; ++c) cacc[(warp * GQ + g) * D + lane * CH + c] = acc[g][c];
    if (lane == 0) { cml[(warp * GQ + g) * 2] = m[g]; cml[(warp * GQ + g) * 2 + 1] = l[g]; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < A.gqa * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    float mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < DG_WARPS; ++w) mt = fmaxf(mt, cml[(w * GQ + g) * 2]);
    float a = 0.f, lt = 0.f;
#pragma unroll
    for (int w = 0; w < DG_WARPS; ++w) {
      const float wgt = exp2f(cml[(w * GQ + g) * 2] - mt);
      a += cacc[(w * GQ + g) * D + d] * wgt;
      lt += cml[(w * GQ + g) * 2 + 1] * wgt;
    }
    const int64_t o = ((int64_t)seq * A.Hq + h * A.gqa + g) * A.num_splits + split;
    A.acc[o * D + d] = a;
    if (d == 0) { A.ml[o * 2] = mt; A.ml[o * 2 + 1] = lt; }
  }
}

}  // namespace echokv
