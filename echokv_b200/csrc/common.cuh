// Shared device/host helpers for the echokv_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/echokv_b200.h"

namespace echokv {

// Layout constants every kernel needs (TieredLayout, echokv_vllm/tiered_cache.py:76-147).
struct LayoutDev {
  int H, D, BS, KG, VG, KC;          // heads, head dim, block size, K group, V group, chunks per page
  int NG;                            // V groups per head (D / VG)
  int KGPB;                          // K groups per block
  int64_t o_vs, o_vm, o_ks, o_km, o_data, CB;  // byte offsets in a page; chunk bytes
  int64_t PS;                        // page stride in bytes
  int64_t NB;                        // number of blocks
};

struct ResidualDev {
  const void* base;
  int dtype;
  int64_t s_slot, s_pos, s_head;
  const int64_t* block_res;
  const int64_t* res_group;
};

int set_error(int code, const char* fmt, ...);
int describe(const echokv_layout* l, echokv_layout_info* out);
int make_layout(const echokv_layout* l, const echokv_pages* p, LayoutDev* out);
int make_residual(const echokv_residual* r, ResidualDev* out);
int check_launch(const char* what);

#ifdef __CUDACC__

// ---- programmatic dependent launch ---------------------------------------------------------
// A kernel launched with `launch_pdl` may be scheduled while the kernel before it on the stream still runs: its
// CTAs take their places as SMs free up and run whatever precedes `pdl_wait()`, which returns once the earlier
// kernel has completed and its writes are visible.  Every CTA calls `pdl_wait()` before it reads or writes
// anything another kernel touches (so completion of this kernel implies completion of the one before it), and
// `pdl_launch_dependents()` lets the next such kernel start being scheduled.  Launched the ordinary way, or after
// something that is not a kernel, both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- element access by runtime dtype ----------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  __device__ static float ld(const void* p, int64_t i) { return reinterpret_cast<const float*>(p)[i]; }
  __device__ static void st(void* p, int64_t i, float v) { reinterpret_cast<float*>(p)[i] = v; }
};
template <> struct Elem<__half> {
  __device__ static float ld(const void* p, int64_t i) { return __half2float(reinterpret_cast<const __half*>(p)[i]); }
  __device__ static void st(void* p, int64_t i, float v) { reinterpret_cast<__half*>(p)[i] = __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  __device__ static float ld(const void* p, int64_t i) {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  }
  __device__ static void st(void* p, int64_t i, float v) {
    reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  }
};

__device__ __forceinline__ float ld_dt(const void* p, int dt, int64_t i) {
  if (dt == ECHOKV_DT_F32) return Elem<float>::ld(p, i);
  if (dt == ECHOKV_DT_F16) return Elem<__half>::ld(p, i);
  return Elem<__nv_bfloat16>::ld(p, i);
}
__device__ __forceinline__ void st_dt(void* p, int dt, int64_t i, float v) {
  if (dt == ECHOKV_DT_F32) Elem<float>::st(p, i, v);
  else if (dt == ECHOKV_DT_F16) Elem<__half>::st(p, i, v);
  else Elem<__nv_bfloat16>::st(p, i, v);
}

// 8 consecutive elements -> float (16-byte loads for 16-bit types). `p + i` must be 16-byte aligned
// for the vector path; callers check alignment once per launch and pass `vec`.
template <typename T>
__device__ __forceinline__ void ld8(const void* p, int64_t i, bool vec, float (&out)[8]) {
  if constexpr (sizeof(T) == 2) {
    if (vec) {
      uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p) + i);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int k = 0; k < 8; ++k) out[k] = static_cast<float>(e[k]);
      return;
    }
  } else {
    if (vec) {
      const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
      float4 a = q[0], b = q[1];
      out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
      out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
      return;
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) out[k] = Elem<T>::ld(p, i + k);
}

// ---- the quantizer (echokv_vllm/quant.py:39-45, :63-75) ------------------------------------
// mn16 = fp16(min); scale16 = fp16(max((max - mn16) / levels, 2^-14)); IEEE divide, no FMA contraction.
__device__ __forceinline__ void group_stats(float mn, float mx, float levels, __half& scale16, __half& mn16) {
  mn16 = __float2half_rn(mn);
  float m = __half2float(mn16);
  float s = __fdiv_rn(__fsub_rn(mx, m), levels);
  s = fmaxf(s, 6.103515625e-05f);
  scale16 = __float2half_rn(s);
}

// code = clamp(rne((x - mn) / scale), 0, levels)
__device__ __forceinline__ uint32_t quant_code(float x, float mn, float scale, float levels) {
  float q = rintf(__fdiv_rn(__fsub_rn(x, mn), scale));
  q = fminf(fmaxf(q, 0.0f), levels);
  return static_cast<uint32_t>(q);
}

// Pack 8 codes at `bits` into the low bits*8 bits of a 64-bit word (element i at bit i*bits).
__device__ __forceinline__ uint64_t pack8(const uint32_t (&c)[8], int bits) {
  uint64_t w = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) w |= static_cast<uint64_t>(c[k]) << (k * bits);
  return w;
}

// Store the low `bits` bytes (= 8 codes at `bits` bits) of `w` at `dst`.
__device__ __forceinline__ void store_packed8(uint8_t* dst, uint64_t w, int bits) {
  if (bits == 8) {
    if ((reinterpret_cast<uintptr_t>(dst) & 7) == 0) { *reinterpret_cast<uint64_t*>(dst) = w; return; }
    *reinterpret_cast<uint32_t*>(dst) = static_cast<uint32_t>(w);
    *reinterpret_cast<uint32_t*>(dst + 4) = static_cast<uint32_t>(w >> 32);
  } else if (bits == 4) {
    *reinterpret_cast<uint32_t*>(dst) = static_cast<uint32_t>(w);
  } else {
    *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(w);
  }
}

// ---- addressing (echokv_vllm/tiered_cache.py:350-359, kernels/write.py:141-153) ---------------
// Tier of a block from header byte 0; a never-opened block (0) is addressed as INT2 so every
// access stays inside its own page (kernels/common.py:32-34).
__device__ __forceinline__ int block_bits(const uint8_t* pages, const LayoutDev& L, int64_t blk) {
  int b = pages[blk * L.PS];
  return b == 0 ? 2 : b;
}

// Byte offset (from the pool base) of token `off`'s K+V row in block `blk` stored at `bits`.
__device__ __forceinline__ int64_t row_offset(const uint8_t* pages, const LayoutDev& L, int64_t blk, int off,
                                              int bits) {
  int tpc = (2 * L.BS) / bits;
  int j = off / tpc;
  int64_t page = blk, slot = 0;
  if (j > 0) {
    int id = reinterpret_cast<const int32_t*>(pages + blk * L.PS + 4)[j - 1];
    page = id / L.KC;
    slot = id % L.KC;
  }
  int64_t row_bytes = (int64_t)(2 * L.H * L.D * bits) / 8;
  return page * L.PS + L.o_data + slot * L.CB + (int64_t)(off % tpc) * row_bytes;
}

__device__ __forceinline__ uint32_t extract_code(const uint8_t* side, int d, int bits) {
  int bit = d * bits;
  return (side[bit >> 3] >> (bit & 7)) & ((1u << bits) - 1u);
}

#endif  // __CUDACC__

}  // namespace echokv
