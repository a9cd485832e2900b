// Tensor-core split-K paged decode attention for sm_100a.
//
// Persistent CTAs (a few per SM) claim (sequence, split) work items from a global counter.  A CTA
// is one producer warp plus H consumer warps, one per KV head.  The producer resolves block table
// -> page header -> chunk ids -> residual map for up to 32 blocks at a time and streams 16-token
// tiles into a ring of shared-memory stages with bulk asynchronous copies (cp.async.bulk +
// mbarrier complete_tx): the [K codes | V codes] rows of two neighbouring tokens go to a slot padded
// by 16 bytes (the MMA's token rows are permuted -- even tokens first, then odd -- so that ldmatrix
// over 8 rows stays bank-conflict free), plus the tile's V stats and its K group's per-channel stats
// and a small header (tier, valid tokens, item start / end).  Consumers wait
// for a stage's `full` barrier, compute, and arrive on its `empty` barrier; nothing in the loop
// synchronises the whole CTA.  Per tile a consumer warp
//   * folds the K group's per-channel scale into the query (q' = q * k_scale, fp16) and adds the
//     constant q . k_min through extra MMA k-steps, so packed K codes feed the tensor cores as
//     plain integers:  S^T[t, g] = sum_d code[t, d] * q'[g, d] + sum_d k_min[d] * q[g, d];
//   * turns INT8 / INT4 codes into fp16 operands by masking them in place (a code byte or nibble
//     alone in a 16-bit lane is the subnormal code * 2^-24; the power of two is undone on the
//     fp32 scores / accumulators) and INT2 codes with magic-number tricks (1024 + c etc.) and an
//     exact subtract, straight from ldmatrix fragments (non-transposed for K, transposed for V so
//     that register pairs run along tokens);
//   * keeps an online softmax per query head over tokens (the M dimension) with warp shuffles,
//     transposes P with movmatrix and accumulates O^T[d, g] += V^T[d, t] * P[t, g]; V's per-token
//     scale is folded into P per V group (INT8/INT4) or into the codes (INT2), V's min and the
//     softmax denominator come from one more MMA against [v_min | ones].
// Accumulator registers map to channels in a tier-specific order (it follows how ldmatrix deals
// out packed codes); when consecutive blocks differ in tier the warp re-maps its accumulators
// through shared memory.  A split's tiles are accumulated in order by one warp and splits are
// merged in split order, so a sequence's result depends on its own length only, not on which CTA
// ran which item.  Every wait on a barrier is bounded; a wait that gives up ends the CTA's work
// and raises the status word.
#include <utility>

#include "decode_generic.cuh"

namespace echokv {
namespace mma {

#ifdef ECHOKV_PROFILE
__device__ long long g_prof[1024 * 8];
__device__ unsigned long long g_phase[8];
#define PROF_T(x) const long long x = clock64()
#define PROF_ADD(acc, a, b) acc += (b) - (a)
#define PROF_PHASE(k, a, b) if (h == 0 && lane == 0) atomicAdd(&g_phase[k], (unsigned long long)((b) - (a)))
#else
#define PROF_T(x)
#define PROF_ADD(acc, a, b)
#define PROF_PHASE(k, a, b)
#endif

constexpr int D = 128;          // head size of this kernel
constexpr int NG = 4;           // V groups per head (v_group 32)
constexpr int TILE = 16;        // tokens per tile
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // bounded spin on every mbarrier wait

struct StageInfo {
  int bits;      // tier of the tile's block (0 mapped to 2)
  int n_valid;   // valid tokens in the tile (1..16)
  int in_res;    // K of this tile comes from the residual buffer
  int pos0;      // position of the tile's first token inside its K group
  long long res_slot;
};

// What the producer tells the consumers about a staged tile (stored at `o_hdr` of the stage).
constexpr int F_RES = 1, F_FIRST = 2, F_LAST = 4;  // K from the residual buffer / first / last tile of a work item
struct alignas(16) StageHeader {
  int bits, n_valid, flags, pos0;   // n_valid: 1..16 tokens, 0 = skip (tier above the caller's bound), -1 = no more work
  long long res_slot;
  int seq, split;
};
// The producer's own notes for one tile of the unit it is working off: the header and every copy source.
struct alignas(16) TilePlan {
  StageHeader hdr;
  const unsigned char* stats[4];    // V scale, V min, K scale, K min of the tile (one run from stats[0] when contiguous)
  const unsigned char* row_src[TILE];
};
constexpr int UNIT = 32;         // tiles planned at a time (one per producer lane)
constexpr int MAX_NS = 8;        // stage ring slots at most
constexpr int HDR_BYTES = 256;   // 2 * MAX_NS mbarriers + the remap lock
static_assert(sizeof(StageHeader) == 32 && sizeof(TilePlan) % 16 == 0, "16-byte copies of headers");
static_assert(2 * MAX_NS * 8 + 4 <= HDR_BYTES, "barriers and lock must fit the header");

struct Params {
  LayoutDev L;
  ResidualDev R;
  const uint8_t* pages;
  DecodeArgs A;
  int H, NS, max_bits, num_seqs;
  int stage_bytes, o_vs, o_vm, o_ks, o_km, o_hdr;  // stage layout (bytes from the stage base)
  int* status;                             // device status word (0 ok), may be null
  int* counter;                            // next unclaimed work item (zero at launch)
  int q_vec16;                             // 16-bit queries whose rows can be read with 16-byte loads
  int debug;                               // experiments only: 1 skip the math, 2 skip the copies
};

// ---- PTX helpers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Returns false if the barrier did not flip within the iteration limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t a = smem_u32(bar);
  for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Compile-time loop: the index is an integral constant, so it can feed template arguments.
template <class F, int... I>
__device__ __forceinline__ void static_for_impl(F&& f, std::integer_sequence<int, I...>) {
  (f(std::integral_constant<int, I>{}), ...);
}
template <int N, class F>
__device__ __forceinline__ void static_for(F&& f) {
  static_for_impl(f, std::make_integer_sequence<int, N>{});
}

// Shared-memory loads take a base register plus a compile-time byte offset so the offset folds
// into the instruction instead of costing an integer add each.
template <int OFF>
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr), "n"(OFF));
}
template <int OFF>
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr), "n"(OFF));
}
__device__ __forceinline__ void ldsm_x2_t(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
template <int OFF>
__device__ __forceinline__ void lds128(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr), "n"(OFF));
}
template <int OFF>
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
  return v;
}
// The same loads for lanes where `on` holds; the other lanes get zeros and cost no shared-memory
// traffic (a quarter warp without an active lane issues no wavefront).
template <int OFF>
__device__ __forceinline__ void lds128_if(uint32_t (&r)[4], uint32_t addr, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %5, 0;\n\t"
      "mov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\tmov.u32 %2, 0;\n\tmov.u32 %3, 0;\n\t"
      "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%6];\n\t}"
      : "=&r"(r[0]), "=&r"(r[1]), "=&r"(r[2]), "=&r"(r[3]) : "r"(addr), "r"(on), "n"(OFF));
}
template <int OFF>
__device__ __forceinline__ uint2 lds64_if(uint32_t addr, uint32_t on) {
  uint2 v;
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %3, 0;\n\t"
      "mov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\t"
      "@p ld.shared.v2.u32 {%0,%1}, [%2+%4];\n\t}"
      : "=&r"(v.x), "=&r"(v.y) : "r"(addr), "r"(on), "n"(OFF));
  return v;
}
__device__ __forceinline__ uint32_t movm_t(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
template <uint32_t MASK, uint32_t MAGIC>
__device__ __forceinline__ uint32_t and_or(uint32_t w) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(w), "n"(MASK), "n"(MAGIC));  // (w & MASK) | MAGIC
  return d;
}
__device__ __forceinline__ uint32_t hsub2u(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t hmul2u(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr uint32_t H2_1024 = 0x64006400u, H2_256 = 0x5c005c00u, H2_64 = 0x54005400u, H2_16 = 0x4c004c00u;
constexpr uint32_t H2_ONE = 0x3c003c00u;

// ---- unpacking packed codes to fp16 pairs ------------------------------------------------------
// A 32-bit word of packed codes yields `PAIRS` half2 values; pair i holds the codes at the element
// positions documented per tier (the two halves are `STRIDE` elements apart).
//   INT8: 4 codes  -> pairs (0,1) (2,3)
//   INT4: 8 codes  -> pairs (0,4) (1,5) (2,6) (3,7)
//   INT2: 16 codes -> pairs (0,8) (1,9) ... (7,15)
template <int BITS> struct Unpack;
template <> struct Unpack<8> {
  static constexpr int PAIRS = 2;
  __device__ static void run(uint32_t w, uint32_t (&o)[2]) {
    o[0] = hsub2u(prmt(w, 0x64646464u, 0x4140u), H2_1024);
    o[1] = hsub2u(prmt(w, 0x64646464u, 0x4342u), H2_1024);
  }
  // word = [a.c0 a.c1 | b.c0 b.c1] (two tokens): pairs (a.c0,b.c0) (a.c1,b.c1)
  __device__ static void run_t(uint32_t w, uint32_t (&o)[2]) {
    o[0] = hsub2u(prmt(w, 0x64646464u, 0x4240u), H2_1024);
    o[1] = hsub2u(prmt(w, 0x64646464u, 0x4341u), H2_1024);
  }
};
template <> struct Unpack<4> {
  static constexpr int PAIRS = 4;
  __device__ static void run(uint32_t w, uint32_t (&o)[4]) {
    o[0] = hsub2u(and_or<0x000f000fu, H2_1024>(w), H2_1024);
    o[1] = hsub2u(and_or<0x00f000f0u, H2_64>(w), H2_64);
    const uint32_t v = w >> 8;
    o[2] = hsub2u(and_or<0x000f000fu, H2_1024>(v), H2_1024);
    o[3] = hsub2u(and_or<0x00f000f0u, H2_64>(v), H2_64);
  }
};
template <> struct Unpack<2> {
  static constexpr int PAIRS = 8;
  __device__ static void run(uint32_t w, uint32_t (&o)[8]) {
    o[0] = hsub2u(and_or<0x00030003u, H2_1024>(w), H2_1024);
    o[1] = hsub2u(and_or<0x000c000cu, H2_256>(w), H2_256);
    o[2] = hsub2u(and_or<0x00300030u, H2_64>(w), H2_64);
    o[3] = hsub2u(and_or<0x00c000c0u, H2_16>(w), H2_16);
    const uint32_t v = w >> 8;
    o[4] = hsub2u(and_or<0x00030003u, H2_1024>(v), H2_1024);
    o[5] = hsub2u(and_or<0x000c000cu, H2_256>(v), H2_256);
    o[6] = hsub2u(and_or<0x00300030u, H2_64>(v), H2_64);
    o[7] = hsub2u(and_or<0x00c000c0u, H2_16>(v), H2_16);
  }
};

// Offset-carrying variants for INT8 / INT4: the fp16 values are OFF + code (OFF = 1024 for codes
// that sit in mantissa bits 0..7, 64 for nibbles in bits 4..7) and the offsets are cancelled
// exactly by a twin MMA whose A operand is the constant -OFF (products are exact in the fp32
// accumulator), which is cheaper than one fp16 subtract per pair.
__device__ __forceinline__ void raw8(uint32_t w, uint32_t (&o)[2]) {
  o[0] = prmt(w, 0x64646464u, 0x4140u);
  o[1] = prmt(w, 0x64646464u, 0x4342u);
}
__device__ __forceinline__ void raw8_t(uint32_t w, uint32_t (&o)[2]) {
  o[0] = prmt(w, 0x64646464u, 0x4240u);
  o[1] = prmt(w, 0x64646464u, 0x4341u);
}
__device__ __forceinline__ void raw4(uint32_t w, uint32_t (&o)[4]) {  // o[0], o[2]: 1024 + c; o[1], o[3]: 64 + c
  o[0] = and_or<0x000f000fu, H2_1024>(w);
  o[1] = and_or<0x00f000f0u, H2_64>(w);
  const uint32_t v = w >> 8;
  o[2] = and_or<0x000f000fu, H2_1024>(v);
  o[3] = and_or<0x00f000f0u, H2_64>(v);
}

// Channel held by accumulator row (mt, r, half) for blocks of tier BITS.
template <int BITS>
__device__ __forceinline__ int acc_channel(int mt, int r, int half) {
  if constexpr (BITS == 8) return 16 * mt + 2 * r + half;
  else if constexpr (BITS == 4) return 32 * (mt >> 1) + 4 * r + 2 * (mt & 1) + half;
  else return 64 * (mt >> 2) + 8 * r + 2 * (mt & 3) + half;
}

// Shared-memory geometry of the query block: [H][8 query rows][D] fp16, rows padded by 64 bytes so
// that the 128-bit fragment loads of two neighbouring rows fall into different bank halves.
constexpr int QT_ROW = D * 2 + 64;   // tier copy: rows padded so 128-bit fragment loads of two rows hit different bank halves
constexpr int QN_ROW = D * 2 + 16;   // natural copy: rows padded for ldmatrix over the 8 query rows
__host__ __device__ constexpr int q_head_bytes(int rows) { return rows * (QT_ROW + QN_ROW); }
constexpr int REMAP_ROW = D + 4;                      // floats per query head in the canonical layout
constexpr int REMAP_BYTES = 8 * REMAP_ROW * 4;

struct WarpState {
  float acc[8][4];  // O^T tiles: [m-tile][c0..c3], channel order depends on `bits`
  float bl[4];      // [0],[1]: sum_t p * v_min for V group r (lanes r < NG); [2],[3]: sum_t p
  float m0, m1;     // running max (log2 domain) of query heads 2j and 2j+1
  int bits;         // tier whose channel order `acc` is in (0: none yet)
  int qbits;        // tier the warp's scaled query copy was built for (0: none yet)
};

// The PV accumulators of INT8 / INT4 blocks hold code units: rows fed by in-place subnormal codes
// are 2^-24 of the true value (2^-20 for the rows fed by upper nibbles: `half` 1 at INT4).
template <int BITS>
__device__ __forceinline__ float acc_unit(int half) {
  if constexpr (BITS == 8) return 16777216.f;
  else if constexpr (BITS == 4) return half ? 1048576.f : 16777216.f;
  else return 1.f;
}

template <int BITS>
__device__ __forceinline__ void store_canonical(const WarpState& w, float* buf, int r, int j) {
#pragma unroll
  for (int mt = 0; mt < 8; ++mt) {
    const int c0 = acc_channel<BITS>(mt, r, 0), c1 = acc_channel<BITS>(mt, r, 1);
    buf[(2 * j) * REMAP_ROW + c0] = w.acc[mt][0] * acc_unit<BITS>(0);
    buf[(2 * j + 1) * REMAP_ROW + c0] = w.acc[mt][1] * acc_unit<BITS>(0);
    buf[(2 * j) * REMAP_ROW + c1] = w.acc[mt][2] * acc_unit<BITS>(1);
    buf[(2 * j + 1) * REMAP_ROW + c1] = w.acc[mt][3] * acc_unit<BITS>(1);
  }
}
template <int BITS>
__device__ __forceinline__ void load_canonical(WarpState& w, const float* buf, int r, int j) {
#pragma unroll
  for (int mt = 0; mt < 8; ++mt) {
    const int c0 = acc_channel<BITS>(mt, r, 0), c1 = acc_channel<BITS>(mt, r, 1);
    w.acc[mt][0] = buf[(2 * j) * REMAP_ROW + c0] * (1.f / acc_unit<BITS>(0));
    w.acc[mt][1] = buf[(2 * j + 1) * REMAP_ROW + c0] * (1.f / acc_unit<BITS>(0));
    w.acc[mt][2] = buf[(2 * j) * REMAP_ROW + c1] * (1.f / acc_unit<BITS>(1));
    w.acc[mt][3] = buf[(2 * j + 1) * REMAP_ROW + c1] * (1.f / acc_unit<BITS>(1));
  }
}
__device__ __forceinline__ void store_any(const WarpState& w, float* buf, int r, int j) {
  if (w.bits == 8) store_canonical<8>(w, buf, r, j);
  else if (w.bits == 4) store_canonical<4>(w, buf, r, j);
  else store_canonical<2>(w, buf, r, j);
}

// Everything a consumer warp needs to address one staged tile.
struct TileView {
  uint32_t krow, vrow;  // this lane's ldmatrix row address for the K side / V side of the staged rows
  uint32_t vs, vm;      // this lane's V scale (tokens 2j.., all groups) / V min (group r) address
  uint32_t vs_row;      // V scales of token r (this head, all groups): 8 bytes; token r + 8 is 8 * tok further
  uint32_t vm_ld;       // ldmatrix row address into the V mins: token (lane & 15), this head's pair of heads
  uint32_t ks, km;      // this head's K scale / min of the tile's group: fp16 [D]
  uint32_t tok;         // bytes between consecutive tokens in the V stats
};

// Per-lane byte offsets that do not change from tile to tile (computed once per warp).
struct LaneConst {
  uint32_t k2, k4, k8, v2, v4, v8;  // per tier: offset of this lane's ldmatrix row on the K / V side
  uint32_t vs_off, vm_off, ksm_off, tok, vs_row, vm_ld;
};
__device__ __forceinline__ LaneConst lane_const(int H, int h, int lane) {
  LaneConst c;
  const int r = lane >> 2, j = lane & 3, mi = lane >> 3;
  // Token rows are staged in pairs (tokens 2p, 2p+1 back to back, as they lie in the page, then 16 bytes
  // of padding), and the MMA's token rows are permuted to match: row rho of the first eight is token
  // 2 * rho, row rho of the second eight is token 2 * rho + 1.  The eight rows one ldmatrix piece reads
  // are then 2 * row_bytes + 16 apart: conflict free.  row_bytes = 32 * H * bits.
  const uint32_t pr = lane & 7, odd = mi & 1, piece = (mi >> 1) * 16u;
  c.k2 = pr * (128u * H + 16u) + odd * (64u * H) + h * 32u + piece;    c.v2 = c.k2 + 32u * H;
  c.k4 = pr * (256u * H + 16u) + odd * (128u * H) + h * 64u + piece;   c.v4 = c.k4 + 64u * H;
  c.k8 = pr * (512u * H + 16u) + odd * (256u * H) + h * 128u + piece;  c.v8 = c.k8 + 128u * H;
  c.tok = (uint32_t)H * NG * 2;
  c.vs_off = (uint32_t)((4 * j) * H + h) * NG * 2;
  c.vm_off = c.vs_off + (uint32_t)(r < NG ? r : 0) * 2;
  c.vs_row = (uint32_t)(2 * r * H + h) * NG * 2;  // token 2r; token 2r + 1 (MMA row r + 8) is one token further
  c.vm_ld = (uint32_t)((2 * (lane & 7) + ((lane >> 3) & 1)) * H + (h & ~1)) * NG * 2;  // k-order: tokens 0,2,..,14 then 1,3,..,15
  c.ksm_off = (uint32_t)h * D * 2;
  return c;
}

// ---- Q.K^T for one tile: scores c[4] = S^T[token r / r+8][query head 2j / 2j+1] (log2 domain) -----
//
// INT8 / INT4 codes enter the tensor cores as fp16 SUBNORMALS: a code byte or nibble masked in
// place inside a zero 16-bit lane is the number code * 2^-24 (nibbles at bits 4..7: code * 2^-20),
// exactly, with no conversion instruction at all.  The 2^-4 of the upper nibbles is pre-applied to
// the odd channels of the tier's query copy, and the 2^24 is applied once to the fp32 scores.
// INT2 keeps the magic-number path (its four crumb positions would need four query scalings and
// its V path multiplies codes by scales in fp16, which subnormals cannot take).
constexpr float CODE_UNSCALE = 16777216.f;  // 2^24
constexpr float RESCALE_SLACK = 6.f;

__device__ __forceinline__ void sub4(uint32_t w, uint32_t (&o)[4]) {  // INT4 word -> 4 subnormal pairs
  o[0] = w & 0x000f000fu;
  o[1] = w & 0x00f000f0u;
  const uint32_t v = w >> 8;
  o[2] = v & 0x000f000fu;
  o[3] = v & 0x00f000f0u;
}
__device__ __forceinline__ void sub8(uint32_t w, uint32_t (&o)[2]) {  // INT8 word -> pairs (0,1) (2,3)
  o[0] = prmt(w, 0u, 0x4140u);
  o[1] = prmt(w, 0u, 0x4342u);
}
__device__ __forceinline__ void sub8_t(uint32_t w, uint32_t (&o)[2]) {  // [a.c0 a.c1 | b.c0 b.c1] -> (a.c0,b.c0) (a.c1,b.c1)
  o[0] = prmt(w, 0u, 0x4240u);
  o[1] = prmt(w, 0u, 0x4341u);
}

// Constant term of the scores, sum_d q[g, d] * k_min[d]: 8 MMA k-steps whose A fragments are the
// group's k_min row broadcast to all 16 token rows (ldmatrix with every row address equal) and
// whose B fragments are the natural-order query (ldmatrix over the 8 query rows).
__device__ __forceinline__ void km_term(uint32_t km, uint32_t qn_ld, int lane, float (&c2)[4]) {
  // One ldmatrix feeds two k-steps: its four 8x8 pieces are channels [0,8) [8,16) [16,24) [24,32) of
  // the 32-channel slice, each read with all eight row addresses equal (the row is the same for
  // every token), so the A fragment of a k-step is (piece, piece, next piece, next piece).
  const uint32_t km_ld = km + (lane >> 3) * 16u;
  static_for<4>([&](auto k2c) {
    constexpr int k2 = decltype(k2c)::value;
    uint32_t B[4], A[4];
    ldsm_x4<k2 * 64>(B, qn_ld);
    ldsm_x4<k2 * 64>(A, km_ld);
    mma16816(c2, A[0], A[0], A[1], A[1], B[0], B[1]);
    mma16816(c2, A[2], A[2], A[3], A[3], B[2], B[3]);
  });
}

// `real`: this lane's MMA column (query head lane / 4 of the group) exists; the other lanes' B
// fragments are zero, so they skip the loads of the query and the K scales.
template <int BITS>
__device__ __forceinline__ void qk_codes(const TileView& tv, uint32_t qt_lane, uint32_t qn_ld, int lane, uint32_t real,
                                         float (&c)[4]) {
  const int j = lane & 3;
  const uint32_t krow = tv.krow;
  float c2[4] = {0.f, 0.f, 0.f, 0.f};
  km_term(tv.km, qn_ld, lane, c2);
  if constexpr (BITS == 8) {
    const uint32_t qb = qt_lane + j * 8, sb = tv.ks + j * 8;  // this lane's 4 channels of every 16-channel piece
    static_for<4>([&](auto ic) {  // pieces 2i, 2i+1 (16 channels each)
      constexpr int i = decltype(ic)::value;
      uint32_t R[4];
      ldsm_x4<i * 32>(R, krow);
      static_for<2>([&](auto ec) {
        constexpr int e = decltype(ec)::value, p = 2 * i + e;
        const uint2 qw = lds64_if<32 * p>(qb, real), sw = lds64_if<32 * p>(sb, real);
        uint32_t a[2], b[2];
        sub8(R[2 * e], a);
        sub8(R[2 * e + 1], b);
        mma16816(c, a[0], b[0], a[1], b[1], hmul2u(qw.x, sw.x), hmul2u(qw.y, sw.y));
      });
    });
#pragma unroll
    for (int k = 0; k < 4; ++k) c[k] = fmaf(c[k], CODE_UNSCALE, c2[k]);
  } else if constexpr (BITS == 4) {
    const uint32_t qb = qt_lane + j * 16, sb = tv.ks + j * 16;  // this lane's 8 channels of every 32-channel piece
    static_for<2>([&](auto ic) {  // pieces 2i, 2i+1 (32 channels each)
      constexpr int i = decltype(ic)::value;
      uint32_t R[4];
      ldsm_x4<i * 32>(R, krow);
      static_for<2>([&](auto ec) {
        constexpr int e = decltype(ec)::value, p = 2 * i + e;
        uint32_t W[4], S[4], Z[4];
        lds128_if<64 * p>(W, qb, real);
        lds128_if<64 * p>(S, sb, real);
#pragma unroll
        for (int k = 0; k < 4; ++k) Z[k] = hmul2u(W[k], S[k]);
        uint32_t a[4], b[4];
        sub4(R[2 * e], a);
        sub4(R[2 * e + 1], b);
        mma16816(c, a[0], b[0], a[1], b[1], prmt(Z[0], Z[2], 0x5410u), prmt(Z[0], Z[2], 0x7632u));
        mma16816(c, a[2], b[2], a[3], b[3], prmt(Z[1], Z[3], 0x5410u), prmt(Z[1], Z[3], 0x7632u));
      });
    });
#pragma unroll
    for (int k = 0; k < 4; ++k) c[k] = fmaf(c[k], CODE_UNSCALE, c2[k]);
  } else {
    const uint32_t qb = qt_lane + j * 32, sb = tv.ks + j * 32;  // this lane's 16 channels of every 64-channel piece
    uint32_t R[4];
    ldsm_x4<0>(R, krow);  // pieces 0, 1 (64 channels each)
    static_for<2>([&](auto pc) {
      constexpr int p = decltype(pc)::value;
      uint32_t W[8], S[8], Z[8];
      {
        uint32_t t4[4];
        lds128_if<128 * p>(t4, qb, real);      W[0] = t4[0]; W[1] = t4[1]; W[2] = t4[2]; W[3] = t4[3];
        lds128_if<128 * p + 16>(t4, qb, real); W[4] = t4[0]; W[5] = t4[1]; W[6] = t4[2]; W[7] = t4[3];
        lds128_if<128 * p>(t4, sb, real);      S[0] = t4[0]; S[1] = t4[1]; S[2] = t4[2]; S[3] = t4[3];
        lds128_if<128 * p + 16>(t4, sb, real); S[4] = t4[0]; S[5] = t4[1]; S[6] = t4[2]; S[7] = t4[3];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) Z[k] = hmul2u(W[k], S[k]);
      uint32_t a[8], b[8];
      Unpack<2>::run(R[2 * p], a);
      Unpack<2>::run(R[2 * p + 1], b);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        mma16816(c, a[2 * k], b[2 * k], a[2 * k + 1], b[2 * k + 1], prmt(Z[k], Z[k + 4], 0x5410u), prmt(Z[k], Z[k + 4], 0x7632u));
    });
#pragma unroll
    for (int k = 0; k < 4; ++k) c[k] += c2[k];
  }
}

// K of the tile comes from the residual buffer (the block's open group): fp16(k) straight into the
// A fragments, unscaled query as B.  Lane (r, j) takes channels 16p + 4j + {0..3} of rows r, r + 8.
__device__ __forceinline__ uint32_t res_pair(const ResidualDev& R, int64_t e) {
  if (R.dtype == ECHOKV_DT_F16) return *reinterpret_cast<const uint32_t*>(reinterpret_cast<const __half*>(R.base) + e);
  float x, y;
  if (R.dtype == ECHOKV_DT_BF16) {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const __nv_bfloat16*>(R.base) + e);
    x = __uint_as_float(u << 16);
    y = __uint_as_float(u & 0xffff0000u);
  } else {
    const float2 f = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(R.base) + e);
    x = f.x; y = f.y;
  }
  return pack_h2(x, y);
}
__device__ __forceinline__ void qk_residual(const ResidualDev& R, const StageInfo& si, uint32_t qn_lane, int h, int lane,
                                            float (&c)[4]) {
  const int r = lane >> 2, j = lane & 3;
  const bool v0 = 2 * r < si.n_valid, v1 = 2 * r + 1 < si.n_valid;  // MMA rows r / r + 8 are tokens 2r / 2r + 1
  const int64_t e0 = si.res_slot * R.s_slot + (int64_t)(si.pos0 + 2 * r) * R.s_pos + h * R.s_head;
  const int64_t e1 = e0 + R.s_pos;
  const uint32_t qb = qn_lane + j * 8;
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const int ch = 16 * p + 4 * j;
    uint2 qw;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(qw.x), "=r"(qw.y) : "r"(qb + p * 32));
    const uint32_t a0 = v0 ? res_pair(R, e0 + ch) : 0u, a2 = v0 ? res_pair(R, e0 + ch + 2) : 0u;
    const uint32_t a1 = v1 ? res_pair(R, e1 + ch) : 0u, a3 = v1 ? res_pair(R, e1 + ch + 2) : 0u;
    mma16816(c, a0, a1, a2, a3, qw.x, qw.y);
  }
}

// ---- P.V for one tile --------------------------------------------------------------------------
// p_lo / p_hi: this lane's probabilities in score layout (token r / r + 8, query heads 2j, 2j + 1), fp16.
// The B fragments of the MMAs are their 8x8 transposes (tokens 2j,2j+1 / 2j+8,2j+9 of head lane / 4).
// INT8 / INT4: V's per-token scale of group G multiplies P before the transpose, where a lane needs the
// scales of just its own two tokens (8 bytes each, all groups), one fragment pair per group.
// INT2: the scale goes into the codes, which needs it per token pair (the order of the A fragments).
template <int BITS, int H>
__device__ __forceinline__ void pv_codes(const TileView& tv, int lane, uint32_t p_lo, uint32_t p_hi, uint32_t pb0,
                                         uint32_t pb1, WarpState& w) {
  const uint32_t vrow = tv.vrow;
  if constexpr (BITS != 2) {
    uint32_t b0[NG], b1[NG];
    {
      const uint2 s0 = lds64<0>(tv.vs_row), s1 = lds64<H * NG * 2>(tv.vs_row);
      b0[0] = movm_t(hmul2u(p_lo, prmt(s0.x, s0.x, 0x1010u))); b0[1] = movm_t(hmul2u(p_lo, prmt(s0.x, s0.x, 0x3232u)));
      b0[2] = movm_t(hmul2u(p_lo, prmt(s0.y, s0.y, 0x1010u))); b0[3] = movm_t(hmul2u(p_lo, prmt(s0.y, s0.y, 0x3232u)));
      b1[0] = movm_t(hmul2u(p_hi, prmt(s1.x, s1.x, 0x1010u))); b1[1] = movm_t(hmul2u(p_hi, prmt(s1.x, s1.x, 0x3232u)));
      b1[2] = movm_t(hmul2u(p_hi, prmt(s1.y, s1.y, 0x1010u))); b1[3] = movm_t(hmul2u(p_hi, prmt(s1.y, s1.y, 0x3232u)));
    }
    if constexpr (BITS == 8) {
      static_for<4>([&](auto ic) {  // pieces 2i, 2i+1 = the two halves of V group i
        constexpr int i = decltype(ic)::value;
        uint32_t Q[4];
        ldsm_x4_t<i * 32>(Q, vrow);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          uint32_t lo[2], hi[2];
          sub8_t(Q[2 * e], lo);
          sub8_t(Q[2 * e + 1], hi);
          mma16816(w.acc[2 * i + e], lo[0], lo[1], hi[0], hi[1], b0[i], b1[i]);
        }
      });
    } else {
      static_for<2>([&](auto ic) {  // pieces 2i, 2i+1 = V groups 2i, 2i+1
        constexpr int i = decltype(ic)::value;
        uint32_t Q[4];
        ldsm_x4_t<i * 32>(Q, vrow);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int G = 2 * i + e;
          uint32_t lo[4], hi[4];
          sub4(Q[2 * e], lo);
          sub4(Q[2 * e + 1], hi);
          mma16816(w.acc[2 * G], lo[0], lo[1], hi[0], hi[1], b0[G], b1[G]);
          mma16816(w.acc[2 * G + 1], lo[2], lo[3], hi[2], hi[3], b0[G], b1[G]);
        }
      });
    }
  } else {
    // The scale multiplies the codes (A fragments: rows = channels, register pairs = tokens 2j, 2j+1 /
    // 2j+8, 2j+9), and a lane's channels of piece q lie in V group 2q + (r >= 4).  The scales are read in
    // score layout (token r / r + 8, all groups: 8 bytes each) and transposed into that order with
    // movmatrix: input column pair j carries group 2q + (j >= 2), so output lane r gets group 2q + (r >= 4).
    uint32_t sl[2], sh[2];
    {
      const uint2 s0 = lds64<0>(tv.vs_row), s1 = lds64<H * NG * 2>(tv.vs_row);
      const uint32_t sel = (lane & 2) ? 0x3232u : 0x1010u;
      sl[0] = movm_t(prmt(s0.x, s0.x, sel)); sl[1] = movm_t(prmt(s0.y, s0.y, sel));
      sh[0] = movm_t(prmt(s1.x, s1.x, sel)); sh[1] = movm_t(prmt(s1.y, s1.y, sel));
    }
    uint32_t Q[4];
    ldsm_x4_t<0>(Q, vrow);  // pieces 0, 1 = V groups {0,1}, {2,3}; this lane's channels lie in group 2q + (r >= 4)
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t lo[8], hi[8];
      Unpack<2>::run(Q[2 * q], lo);
      Unpack<2>::run(Q[2 * q + 1], hi);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        mma16816(w.acc[4 * q + u], hmul2u(lo[2 * u], sl[q]), hmul2u(lo[2 * u + 1], sl[q]), hmul2u(hi[2 * u], sh[q]),
                 hmul2u(hi[2 * u + 1], sh[q]), pb0, pb1);
    }
  }
}

// Row of the [v_min | ones] MMA that carries the bias of V group G for KV head h: with two or more
// heads the v_min fragment is read with ldmatrix over pairs of heads (16-byte rows), so the odd head
// of a pair sits in rows 4..7.
template <int H>
__device__ __forceinline__ int bias_row(int G, int h) { return H >= 2 ? G + 4 * (h & 1) : G; }

// A warp's two query copies in shared memory (see QT_ROW / QN_ROW).
struct QView {
  unsigned char *qn, *qt;      // natural copy [rows][QN_ROW], tier-scaled copy [rows][QT_ROW]
  int rows;                    // gqa real rows + one zero row that every unused query column reads
  uint32_t qt_lane, qn_lane;   // shared address of this lane's query row (row lane / 4) in each copy
  uint32_t qn_ld;              // this lane's ldmatrix row address in the natural copy
};

template <int BITS, int H>
__device__ __forceinline__ void process_tile(const Params& P, const TileView& tv, const StageInfo& si, const QView& qv,
                                             int h, int lane, WarpState& w, float* remap, int* lock, bool& ok) {
  const int r = lane >> 2, j = lane & 3;
  if (w.qbits != BITS) {  // (re)build the tier's query copy: INT4 needs its odd channels scaled by 2^-4
    __syncwarp();
    for (int i = lane; i < qv.rows * (D / 2); i += 32) {
      const int n = i / (D / 2), wd = i % (D / 2);
      uint32_t v = *reinterpret_cast<const uint32_t*>(qv.qn + n * QN_ROW + wd * 4);
      if constexpr (BITS == 4) v = hmul2u(v, 0x2c003c00u);  // (1, 2^-4)
      *reinterpret_cast<uint32_t*>(qv.qt + n * QT_ROW + wd * 4) = v;
    }
    __syncwarp();
    w.qbits = BITS;
  }
  if (w.bits != BITS) {
    if (w.bits != 0) {  // re-map the accumulators to this tier's channel order (rare: tier changes)
      if (lane == 0) {
        uint32_t it = 0;
        while (atomicCAS(lock, 0, 1) != 0 && ++it < WAIT_LIMIT) {}
        if (it >= WAIT_LIMIT) ok = false;
      }
      __syncwarp();
      store_any(w, remap, r, j);
      __syncwarp();
      load_canonical<BITS>(w, remap, r, j);
      __syncwarp();
      if (lane == 0) atomicExch(lock, 0);
    }
    w.bits = BITS;
  }
  // scores
  PROF_T(f0);
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  if (si.in_res) qk_residual(P.R, si, qv.qn_lane, h, lane, c);
  else qk_codes<BITS>(tv, qv.qt_lane, qv.qn_ld, lane, (uint32_t)(r < P.A.gqa), c);
  PROF_T(f1);
  PROF_PHASE(0, f0, f1);
  if (si.n_valid < TILE) {  // a partial tile (the sequence's last): tokens past the end do not count
    if (2 * r >= si.n_valid) { c[0] = -INFINITY; c[1] = -INFINITY; }      // MMA row r is token 2r
    if (2 * r + 1 >= si.n_valid) { c[2] = -INFINITY; c[3] = -INFINITY; }  // MMA row r + 8 is token 2r + 1
  }
  // online softmax over tokens (rows); columns 2j, 2j+1 belong to this lane
  float t0 = fmaxf(c[0], c[2]), t1 = fmaxf(c[1], c[3]);
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, o));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, o));
  }
  // The reference point of the exponentials only moves when a tile's maximum exceeds it by more
  // than RESCALE_SLACK (in log2 units): until then p <= 2^RESCALE_SLACK, well inside fp16, and the
  // accumulators need no rescaling.  The result is the same softmax (the reference point cancels).
  const bool grew = (t0 > w.m0 + RESCALE_SLACK) || (t1 > w.m1 + RESCALE_SLACK);
  float n0 = w.m0, n1 = w.m1;
  if (__any_sync(0xffffffffu, grew)) {
    n0 = fmaxf(w.m0, t0); n1 = fmaxf(w.m1, t1);
    const float a0 = ex2(w.m0 - n0), a1 = ex2(w.m1 - n1);
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) { w.acc[mt][0] *= a0; w.acc[mt][1] *= a1; w.acc[mt][2] *= a0; w.acc[mt][3] *= a1; }
    w.bl[0] *= a0; w.bl[1] *= a1; w.bl[2] *= a0; w.bl[3] *= a1;
    w.m0 = n0; w.m1 = n1;
  }
  const uint32_t p_lo = pack_h2(ex2(c[0] - n0), ex2(c[1] - n1));   // token r
  const uint32_t p_hi = pack_h2(ex2(c[2] - n0), ex2(c[3] - n1));   // token r + 8
  const uint32_t pb0 = movm_t(p_lo), pb1 = movm_t(p_hi);
  PROF_T(f2);
  PROF_PHASE(1, f1, f2);
  // [v_min | ones] rows: the bias of every V group and the softmax denominator
  if constexpr (H >= 2) {
    uint32_t X[2];
    ldsm_x2_t(X, tv.vm_ld);  // rows: groups of this pair of heads (row bias_row(G, h) is ours), k: tokens
    mma16816(w.bl, X[0], H2_ONE, X[1], H2_ONE, pb0, pb1);
  } else {
    const uint32_t base = tv.vm, tok = tv.tok;  // lanes r >= NG read group 0 and mask it to zero
    uint32_t x0, x1, x2, x3;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(x0) : "r"(base));            // token 4j     (k slot 2j)
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(x1) : "r"(base + 2 * tok));  // token 4j + 2 (k slot 2j + 1)
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(x2) : "r"(base + tok));      // token 4j + 1 (k slot 2j + 8)
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(x3) : "r"(base + 3 * tok));  // token 4j + 3 (k slot 2j + 9)
    const uint32_t keep = r < NG ? 0xffffffffu : 0u;
    mma16816(w.bl, prmt(x0, x1, 0x5410u) & keep, H2_ONE, prmt(x2, x3, 0x5410u) & keep, H2_ONE, pb0, pb1);
  }
  PROF_T(f3);
  PROF_PHASE(2, f2, f3);
  pv_codes<BITS, H>(tv, lane, p_lo, p_hi, pb0, pb1, w);
  PROF_T(f4);
  PROF_PHASE(3, f3, f4);
}

// ---- the kernel ------------------------------------------------------------------------------
// Persistent CTAs claim work items (item = split * num_seqs + seq, so neighbouring CTAs work on
// different sequences and the short tail splits come last) from a global counter, which evens out
// the speed differences between SMs.  H consumer warps (one per KV head) + one producer warp.
//
// The producer warp runs ahead of the consumers.  It resolves block table -> page header -> chunk
// ids -> residual map for up to 32 blocks at a time, one block per lane (the dependent global
// loads of the next batch are in flight while the current one is worked off), plans up to 32 tiles
// in parallel (lane l writes tile l's header and copy sources to shared memory) and then feeds the
// stage ring tile by tile: wait until every consumer warp has released the stage, write the tile's
// header, and start the tile's copies as bulk asynchronous copies that report their bytes to the
// stage's `full` mbarrier -- lane p < 8 copies token rows 2p and 2p + 1 in one piece (to a slot padded
// by 16 bytes), lanes 16.. copy the V / K stats.  Consumers only wait for `full`,
// compute, and arrive on `empty`; the header tells them where a work item starts (load the query,
// reset the accumulators) and ends (write the split's partial result).  There is no CTA-wide barrier
// in the loop.
__device__ __forceinline__ bool item_range(const Params& P, int item, int& seq, int& split, int64_t& seq_len,
                                           int& b_start, int& b_end) {
  seq = item % P.num_seqs;
  split = item / P.num_seqs;
  seq_len = P.A.lens[seq];
  return split_range(seq_len, P.L.BS, P.A.num_splits, P.A.bps_min, split, b_start, b_end);
}

// Block metadata the descriptor warp prefetches for up to 32 blocks at a time (one block per lane).
struct BlockMeta {
  int blk, bits, c1, c2, c3, rgrp;
  long long rslot;
};
__device__ __forceinline__ BlockMeta load_meta(const Params& P, int64_t bt_row, int bi, int b_end) {
  BlockMeta m;
  m.blk = 0; m.bits = 0; m.c1 = m.c2 = m.c3 = 0; m.rgrp = -1; m.rslot = -1;
  if (bi < b_end) {
    m.blk = P.A.bt[bt_row * P.A.bt_s0 + bi];
    const uint4 hd = *reinterpret_cast<const uint4*>(P.pages + (int64_t)m.blk * P.L.PS);
    m.bits = hd.x & 0xff; m.c1 = (int)hd.y; m.c2 = (int)hd.z; m.c3 = (int)hd.w;
    m.rslot = P.R.block_res[m.blk];
    if (m.rslot >= 0) m.rgrp = (int)P.R.res_group[m.rslot];
  }
  return m;
}

template <int BITS, int H>
__device__ __forceinline__ void write_partial(const Params& P, const WarpState& w, int seq, int split, int h, int lane) {
  const int r = lane >> 2, j = lane & 3;
  const DecodeArgs& A = P.A;
  const int g0 = 2 * j, g1 = 2 * j + 1;
  const int64_t o0 = (((int64_t)seq * A.Hq + h * A.gqa + g0) * A.num_splits + split);
  const int64_t o1 = o0 + A.num_splits;
#pragma unroll
  for (int mt = 0; mt < 8; ++mt) {
    // V min contribution of the channels' group: held by lane (r = G, j)
    int G;
    if constexpr (BITS == 8) G = mt >> 1;
    else if constexpr (BITS == 4) G = mt >> 1;
    else G = 2 * (mt >> 2) + (r >= 4 ? 1 : 0);
    const float bias0 = __shfl_sync(0xffffffffu, w.bl[0], bias_row<H>(G, h) * 4 + j);
    const float bias1 = __shfl_sync(0xffffffffu, w.bl[1], bias_row<H>(G, h) * 4 + j);
    const int c0 = acc_channel<BITS>(mt, r, 0), c1 = acc_channel<BITS>(mt, r, 1);
    if (g0 < A.gqa) {
      A.acc[o0 * D + c0] = fmaf(w.acc[mt][0], acc_unit<BITS>(0), bias0);
      A.acc[o0 * D + c1] = fmaf(w.acc[mt][2], acc_unit<BITS>(1), bias0);
    }
    if (g1 < A.gqa) {
      A.acc[o1 * D + c0] = fmaf(w.acc[mt][1], acc_unit<BITS>(0), bias1);
      A.acc[o1 * D + c1] = fmaf(w.acc[mt][3], acc_unit<BITS>(1), bias1);
    }
  }
  if (r == 0) {
    if (g0 < A.gqa) { A.ml[o0 * 2] = w.m0; A.ml[o0 * 2 + 1] = w.bl[2]; }
    if (g1 < A.gqa) { A.ml[o1 * 2] = w.m1; A.ml[o1 * 2 + 1] = w.bl[3]; }
  }
}

template <int H>
__global__ void __launch_bounds__((H + 1) * 32, H == 8 ? 2 : (H == 4 ? 4 : (H == 2 ? 5 : 8))) decode_mma_kernel(const Params P) {
  extern __shared__ __align__(128) unsigned char smem[];
  const LayoutDev& L = P.L;
  const DecodeArgs& A = P.A;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int NS = P.NS;
  const int n_items = P.num_seqs * A.num_splits;

  // shared memory: [barriers | lock][tile plans][remap][q copies per head][stage ring]
  uint64_t* sfull = reinterpret_cast<uint64_t*>(smem);   // stage ring: header written, copies landed
  uint64_t* sempty = sfull + MAX_NS;                     // stage ring: every consumer warp is done with the stage
  int* lock = reinterpret_cast<int*>(sempty + MAX_NS);
  TilePlan* plan = reinterpret_cast<TilePlan*>(smem + HDR_BYTES);
  float* remap = reinterpret_cast<float*>(smem + HDR_BYTES + UNIT * sizeof(TilePlan));
  unsigned char* qs = reinterpret_cast<unsigned char*>(remap) + REMAP_BYTES;
  const int q_rows = A.gqa + 1;
  unsigned char* ring = qs + H * q_head_bytes(q_rows);

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_NS; ++s) { mbar_init(sfull + s, 1); mbar_init(sempty + s, H * 32); }
    *lock = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  {  // zero the ring once: rows of a partial tile that are never copied must read as finite numbers
    const int n16 = (NS * P.stage_bytes) / 16;
    uint4* z = reinterpret_cast<uint4*>(ring);
    for (int i = threadIdx.x; i < n16; i += (H + 1) * 32) z[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the bulk copies write the same bytes later
  }
  __syncthreads();

  bool ok = true, bad_tier = false;
  if (warp == H) {
    // ===================== producer warp =====================
    const int tpb = L.BS / TILE;                     // tiles per block
    const int U = tpb >= UNIT ? 1 : UNIT / tpb;      // blocks per unit
    const bool contig = L.BS == TILE && L.KG == TILE;  // a tile's four stats arrays form one run in the page
    const uint32_t ring_u = smem_u32(ring);
    const uint32_t stat_bytes = H * (2 * TILE * NG * 2 + 2 * D * 2);
    int st = 0, round = 0;                           // next stage to fill and how often it has been filled
    uint32_t st_u = ring_u;
    int issued = 0;
    int seq = 0, split = 0, b_start = 0, b_end = 0, base = 0;
    int64_t seq_len = 0, bt_row = 0;
    bool have = false;
    auto advance = [&]() {  // move to the next unit (claiming a new item when needed); false when there is no work left
      if (have && base + U < b_end) { base += U; return true; }
      for (;;) {
        int it = 0;
        if (lane == 0) it = atomicAdd(P.counter, 1);
        it = __shfl_sync(0xffffffffu, it, 0);
        if (it >= n_items) { have = false; return false; }
        if (item_range(P, it, seq, split, seq_len, b_start, b_end)) {
          base = b_start; bt_row = A.bt_rows ? A.bt_rows[seq] : seq; have = true;
          return true;
        }
      }
    };
#ifdef ECHOKV_PROFILE
    long long p_wait = 0, p_meta = 0, p_plan = 0;
    const long long p_begin = clock64();
#endif
    bool more = advance();
    BlockMeta nxt = more ? load_meta(P, bt_row, lane < U ? base + lane : b_end, b_end) : BlockMeta{};
    while (more && ok) {
      const BlockMeta cur = nxt;
      const int u_base = base, u_end = b_end, u_seq = seq, u_split = split;
      const bool u_first = base == b_start, u_last = base + U >= b_end;
      const int64_t u_len = seq_len;
      PROF_T(m0);
      more = advance();
      if (more) nxt = load_meta(P, bt_row, lane < U ? base + lane : b_end, b_end);
      PROF_T(m1);
      PROF_ADD(p_meta, m0, m1);
      const int nb = min(U, u_end - u_base);
      // tokens of the unit: all blocks are full except possibly the item's last one
      const int unit_tok = (int)min((int64_t)nb * L.BS, u_len - (int64_t)u_base * L.BS);
      const int unit_tiles = (unit_tok + TILE - 1) / TILE;
      {  // plan: lane l takes tile l of the unit (its block's metadata sits in lane kb)
        const int kb = tpb == 1 ? lane : lane / tpb, tb = lane - kb * tpb;
        const int src = kb < 32 ? kb : 31;
        const int kblk = __shfl_sync(0xffffffffu, cur.blk, src);
        int bits = __shfl_sync(0xffffffffu, cur.bits, src);
        const int c1 = __shfl_sync(0xffffffffu, cur.c1, src), c2 = __shfl_sync(0xffffffffu, cur.c2, src),
                  c3 = __shfl_sync(0xffffffffu, cur.c3, src);
        const long long ks_slot = __shfl_sync(0xffffffffu, cur.rslot, src);
        const int kgrp = __shfl_sync(0xffffffffu, cur.rgrp, src);
        if (lane < unit_tiles) {
          if (bits != 2 && bits != 4 && bits != 8) bits = 2;  // never opened: stay inside the page
          const bool too_wide = bits > P.max_bits;             // the caller's tier bound was wrong
          if (too_wide) { bits = P.max_bits; bad_tier = true; }  // such tiles are staged empty
          const int row_bytes = 32 * H * bits;
          const int tpc = (2 * L.BS) / bits;
          const int t0 = tb * TILE;
          const int blk_tok = min(L.BS, unit_tok - kb * L.BS);
          const int grp = t0 / L.KG;
          const bool in_res = ks_slot >= 0 && grp == kgrp;
          const unsigned char* page = P.pages + (int64_t)kblk * L.PS;
          TilePlan& d = plan[lane];
          int jc = t0 / tpc, in_chunk = t0 - jc * tpc;      // chunk of the tile's first token, position inside it
          const unsigned char* chunk = nullptr;
          for (int t = 0; t < TILE; ++t) {
            if (t == 0 || in_chunk == tpc) {
              if (t) { ++jc; in_chunk = 0; }
              int64_t pg = kblk, cs = 0;
              if (jc > 0) { const int id = jc == 1 ? c1 : (jc == 2 ? c2 : c3); pg = id / L.KC; cs = id - pg * L.KC; }
              chunk = P.pages + pg * L.PS + L.o_data + cs * L.CB;
            }
            d.row_src[t] = chunk + (int64_t)in_chunk * row_bytes;
            ++in_chunk;
          }
          d.hdr.bits = bits; d.hdr.n_valid = too_wide ? 0 : min(TILE, blk_tok - t0);
          d.hdr.flags = (in_res ? F_RES : 0) | (u_first && lane == 0 ? F_FIRST : 0) | (u_last && lane == unit_tiles - 1 ? F_LAST : 0);
          d.hdr.pos0 = t0 - grp * L.KG; d.hdr.res_slot = ks_slot; d.hdr.seq = u_seq; d.hdr.split = u_split;
          d.stats[0] = page + L.o_vs + (int64_t)t0 * H * NG * 2;
          d.stats[1] = page + L.o_vm + (int64_t)t0 * H * NG * 2;
          d.stats[2] = page + L.o_ks + (int64_t)grp * H * D * 2;
          d.stats[3] = page + L.o_km + (int64_t)grp * H * D * 2;
        }
        __syncwarp();
      }
      PROF_T(m2);
      PROF_ADD(p_plan, m1, m2);
      for (int ti = 0; ti < unit_tiles; ++ti) {
        const TilePlan& d = plan[ti];
        const int4 h0 = *reinterpret_cast<const int4*>(&d.hdr);   // bits, n_valid, flags, pos0
        const uint32_t row_bytes = 32u * H * h0.x;
#ifdef ECHOKV_PROFILE
        const bool copy = h0.y > 0 && (P.debug & 3) != 2;
#else
        const bool copy = h0.y > 0;
#endif
        PROF_T(w0);
        if (round > 0 && !mbar_wait(sempty + st, (round - 1) & 1)) { ok = false; break; }
        PROF_T(w1);
        PROF_ADD(p_wait, w0, w1);
        const uint32_t bar = smem_u32(sfull + st);
        if (lane == 0) {
          int4* hd = reinterpret_cast<int4*>(ring + (size_t)st * P.stage_bytes + P.o_hdr);
          hd[0] = h0;
          hd[1] = reinterpret_cast<const int4*>(&d.hdr)[1];
          if (copy) mbar_expect_tx(sfull + st, h0.y * row_bytes + stat_bytes);
          else mbar_arrive(sfull + st);
        }
        __syncwarp();
        if (copy) {
          // lane p < 8 copies tokens 2p and 2p + 1 in one piece (neighbours in their chunk: a chunk holds an even number of tokens)
          if (lane < 8) { if (2 * lane < h0.y) bulk_copy(st_u + lane * (2 * row_bytes + 16), d.row_src[2 * lane], (2 * lane + 1 < h0.y ? 2u : 1u) * row_bytes, bar); }
          else if (contig) { if (lane == 16) bulk_copy(st_u + P.o_vs, d.stats[0], stat_bytes, bar); }
          else if (lane >= 16 && lane < 20) {
            const int which = lane - 16;  // vs, vm, ks, km
            const int dst_off = which == 0 ? P.o_vs : which == 1 ? P.o_vm : which == 2 ? P.o_ks : P.o_km;
            bulk_copy(st_u + dst_off, d.stats[which], which < 2 ? H * TILE * NG * 2 : H * D * 2, bar);
          }
        }
        ++issued;
        if (++st == NS) { st = 0; st_u = ring_u; ++round; } else { st_u += P.stage_bytes; }
      }
      __syncwarp();  // every lane is done reading the plans before the next unit overwrites them
      ok = !__any_sync(0xffffffffu, !ok);
    }
    if (ok) {  // no more work: tell the consumers
      if (round == 0 || mbar_wait(sempty + st, (round - 1) & 1)) {
        if (lane == 0) {
          reinterpret_cast<int4*>(ring + (size_t)st * P.stage_bytes + P.o_hdr)[0] = make_int4(2, -1, 0, 0);
          mbar_arrive(sfull + st);
        }
      } else {
        ok = false;
      }
    }
#ifdef ECHOKV_PROFILE
    if (lane == 0 && blockIdx.x < 1024) {
      g_prof[blockIdx.x * 8 + 0] = clock64() - p_begin;
      g_prof[blockIdx.x * 8 + 1] = p_wait;
      g_prof[blockIdx.x * 8 + 2] = p_meta;
      g_prof[blockIdx.x * 8 + 7] = p_plan;
    }
#endif
    if (!ok) {
      // A wait gave up: copies already started may still be landing; give each stage its (bounded)
      // time before the CTA's shared memory goes away.
      for (int s = 0; s < NS; ++s) {
        const int uses = issued > s ? (issued - s + NS - 1) / NS : 0;
        if (uses > 0) mbar_wait(sfull + s, (uses - 1) & 1);
      }
    }
  } else {
    // ===================== consumers: warp h owns KV head h =====================
    const int h = warp;
    const int r = lane >> 2;
    QView qv;
    qv.rows = q_rows;
    qv.qn = qs + h * q_head_bytes(q_rows);
    qv.qt = qv.qn + q_rows * QN_ROW;
    {  // query columns >= gqa of the MMAs read the shared zero row
      const int my_row = r < A.gqa ? r : A.gqa, ld_row = (lane & 7) < A.gqa ? (lane & 7) : A.gqa;
      qv.qt_lane = smem_u32(qv.qt + my_row * QT_ROW);
      qv.qn_lane = smem_u32(qv.qn + my_row * QN_ROW);
      qv.qn_ld = smem_u32(qv.qn + ld_row * QN_ROW + (lane >> 3) * 16);
      for (int i = lane; i < D / 2; i += 32) *reinterpret_cast<uint32_t*>(qv.qn + A.gqa * QN_ROW + i * 4) = 0u;
    }
    LaneConst lc = lane_const(H, h, lane);
    // fold the stage offsets of the stats arrays in: [vs | vm | ks | km] follow the token rows
    lc.vs_off += P.o_vs; lc.vs_row += P.o_vs; lc.vm_off += P.o_vm; lc.vm_ld += P.o_vm; lc.ksm_off += P.o_ks;
    const uint32_t ring_u = smem_u32(ring);
    const uint32_t stage_bytes = P.stage_bytes;
    int c_st = 0, c_round = 0;                  // stage being consumed and how often it has been consumed
    uint32_t c_sb = ring_u;
#ifdef ECHOKV_PROFILE
    long long c_wait = 0, c_math = 0, c_item = 0;
    const long long c_begin = clock64();
#endif
    WarpState w;
    w.bits = 0; w.qbits = 0;
    int seq = 0;
    while (ok) {
      PROF_T(w0);
      if (!mbar_wait(sfull + c_st, c_round & 1)) { ok = false; break; }  // header written, copies landed
      PROF_T(w1);
      PROF_ADD(c_wait, w0, w1);
      StageInfo si;
      int flags, split;
      {
        uint32_t hd[4], ex[4];
        lds128<0>(hd, c_sb + P.o_hdr);
        lds128<16>(ex, c_sb + P.o_hdr);
        si.bits = (int)hd[0]; si.n_valid = (int)hd[1]; flags = (int)hd[2]; si.pos0 = (int)hd[3];
        si.in_res = flags & F_RES;
        si.res_slot = (long long)(((unsigned long long)ex[1] << 32) | ex[0]);
        if (flags & F_FIRST) seq = (int)ex[2];
        split = (int)ex[3];
      }
      if (si.n_valid < 0) break;  // no more work for this CTA
      if (flags & F_FIRST) {
        // this head's queries -> fp16, pre-multiplied by softmax_scale * log2(e); rows >= gqa are zero.
        // All global loads are issued before the first use so the item pays one memory latency.
        const int64_t q_row = A.q_rows ? A.q_rows[seq] : seq;
        __syncwarp();
        if (P.q_vec16) {  // 16-bit queries, 16-byte aligned rows: lane l loads 8 channels of rows l / 16, + 2, + 4, + 6
          const int c8 = (lane & 15) * 8;
          uint4 raw[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int n = (lane >> 4) + 2 * k;
            raw[k] = make_uint4(0, 0, 0, 0);
            if (n < A.gqa)
              raw[k] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(A.q) + q_row * A.q_s0 +
                                                       (int64_t)(h * A.gqa + n) * A.q_s1 + c8);
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int n = (lane >> 4) + 2 * k;
            const uint32_t* wds = reinterpret_cast<const uint32_t*>(&raw[k]);
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float x, y;
              if (A.q_dt == ECHOKV_DT_BF16) { x = __uint_as_float(wds[e] << 16); y = __uint_as_float(wds[e] & 0xffff0000u); }
              else { const __half2 hh = *reinterpret_cast<const __half2*>(&wds[e]); x = __low2float(hh); y = __high2float(hh); }
              o[e] = pack_h2(x * A.scale_log2e, y * A.scale_log2e);
            }
            if (n < A.gqa) *reinterpret_cast<uint4*>(qv.qn + n * QN_ROW + c8 * 2) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
          for (int i = lane; i < A.gqa * (D / 2); i += 32) {
            const int d2 = i % (D / 2), n = i / (D / 2);
            const int64_t e = q_row * A.q_s0 + (int64_t)(h * A.gqa + n) * A.q_s1 + 2 * d2;
            const float x = ld_dt(A.q, A.q_dt, e) * A.scale_log2e, y = ld_dt(A.q, A.q_dt, e + 1) * A.scale_log2e;
            *reinterpret_cast<uint32_t*>(qv.qn + n * QN_ROW + d2 * 4) = pack_h2(x, y);
          }
        }
        __syncwarp();
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) { w.acc[mt][0] = w.acc[mt][1] = w.acc[mt][2] = w.acc[mt][3] = 0.f; }
        w.bl[0] = w.bl[1] = w.bl[2] = w.bl[3] = 0.f;
        w.m0 = w.m1 = -INFINITY;
        w.bits = 0;
        w.qbits = 0;
      }
      PROF_T(w2);
      PROF_ADD(c_item, w1, w2);
      TileView tv;
      tv.krow = c_sb + (si.bits == 8 ? lc.k8 : (si.bits == 4 ? lc.k4 : lc.k2));
      tv.vrow = c_sb + (si.bits == 8 ? lc.v8 : (si.bits == 4 ? lc.v4 : lc.v2));
      tv.vs = c_sb + lc.vs_off; tv.vm = c_sb + lc.vm_off;
      tv.ks = c_sb + lc.ksm_off; tv.km = tv.ks + H * D * 2; tv.tok = H * NG * 2;
      tv.vs_row = c_sb + lc.vs_row; tv.vm_ld = c_sb + lc.vm_ld;
#ifdef ECHOKV_PROFILE
      if (si.n_valid > 0 && (P.debug & 3) != 1) {
#else
      if (si.n_valid > 0) {
#endif
        if (si.bits == 4) process_tile<4, H>(P, tv, si, qv, h, lane, w, remap, lock, ok);
        else if (si.bits == 8) process_tile<8, H>(P, tv, si, qv, h, lane, w, remap, lock, ok);
        else process_tile<2, H>(P, tv, si, qv, h, lane, w, remap, lock, ok);
      }
      __syncwarp();
      PROF_T(w3);
      PROF_ADD(c_math, w2, w3);
      mbar_arrive(sempty + c_st);  // every lane arrives (the barrier counts threads): no branch, no warp sync needed
      if (++c_st == NS) { c_st = 0; c_sb = ring_u; ++c_round; } else { c_sb += stage_bytes; }
      if (flags & F_LAST) {
        if (w.bits == 4) write_partial<4, H>(P, w, seq, split, h, lane);
        else if (w.bits == 8) write_partial<8, H>(P, w, seq, split, h, lane);
        else write_partial<2, H>(P, w, seq, split, h, lane);
        PROF_T(w4);
        PROF_ADD(c_item, w3, w4);
      }
    }
#ifdef ECHOKV_PROFILE
    if (lane == 0 && h == 0 && blockIdx.x < 1024) {
      g_prof[blockIdx.x * 8 + 3] = clock64() - c_begin;
      g_prof[blockIdx.x * 8 + 4] = c_wait;
      g_prof[blockIdx.x * 8 + 5] = c_math;
      g_prof[blockIdx.x * 8 + 6] = c_item;
    }
#endif
  }
  if ((!ok || bad_tier) && lane == 0 && P.status) atomicExch(P.status, bad_tier ? 2 : 1);
}

}  // namespace mma

static int g_decode_path = 0;  // 0: pick by shape, 1: always the generic kernel
static cudaEvent_t g_ev_before = nullptr, g_ev_after = nullptr;  // optional timing hook around the split kernel

// Raised by decode_mma_kernel: 1 = a bounded wait ran out, 2 = a block of a tier wider than the stages.
__device__ int g_decode_status;

int decode_status_take(bool clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)) != cudaSuccess) return -1;  // synchronizes
  if (v && clear) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int));
  }
  return v;
}

// Chooses the tensor-core kernel when the shape fits; otherwise leaves `handled` false.
int launch_decode_mma(const LayoutDev& L, const ResidualDev& R, const uint8_t* pages, const DecodeArgs& A,
                      int64_t num_seqs, int max_tier, int* counter, int* status, cudaStream_t st, bool* handled) {
  using namespace mma;
  *handled = false;
  if ((g_decode_path & 15) == 1) return ECHOKV_OK;
  const int H = L.H;
  if (L.D != D || L.VG != 32 || L.KG % TILE || L.BS % TILE || A.gqa > 8) return ECHOKV_OK;
  if (!(H == 1 || H == 2 || H == 4 || H == 8)) return ECHOKV_OK;
  if ((R.s_slot | R.s_pos | R.s_head) & 3) return ECHOKV_OK;                 // 8-byte residual loads
  if ((reinterpret_cast<uintptr_t>(R.base) & 15) != 0) return ECHOKV_OK;
  if (num_seqs * (int64_t)A.num_splits > (1 << 30)) return ECHOKV_OK;
  Params P;
  P.L = L; P.R = R; P.pages = pages; P.A = A; P.H = H; P.num_seqs = (int)num_seqs;
  // Any tier can appear as soon as the pool has spare chunks (an INT8 block borrows 3 of them), so
  // stages are sized for INT8 rows unless the caller bounds the tiers present in this pool.
  P.max_bits = L.KC >= 2 ? 8 : 2;
  if (max_tier == 2 || max_tier == 4 || max_tier == 8) P.max_bits = max_tier < P.max_bits ? max_tier : P.max_bits;
  const int row_stride = (2 * H * D * P.max_bits) / 8 + 16;
  P.o_vs = TILE * row_stride;
  P.o_vm = P.o_vs + TILE * H * NG * 2;
  P.o_ks = P.o_vm + TILE * H * NG * 2;
  P.o_km = P.o_ks + H * D * 2;
  P.o_hdr = P.o_km + H * D * 2;
  P.stage_bytes = (P.o_hdr + (int)sizeof(StageHeader) + 127) / 128 * 128;
  P.counter = counter;
  P.q_vec16 = (A.q_dt != ECHOKV_DT_F32) && (reinterpret_cast<uintptr_t>(A.q) % 16 == 0) && A.q_s0 % 8 == 0 && A.q_s1 % 8 == 0;
  P.debug = (g_decode_path >> 4) & 15;
  const int fixed = HDR_BYTES + UNIT * (int)sizeof(TilePlan) + REMAP_BYTES + H * q_head_bytes(A.gqa + 1);
  static int max_smem = -1, num_sms = 0;
  static int* status_word = nullptr;
  if (max_smem < 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&status_word), g_decode_status);
    if (e != cudaSuccess) { max_smem = -1; return set_error(ECHOKV_E_CUDA, "decode: cannot raise shared memory: %s", cudaGetErrorString(e)); }
  }
  P.status = status ? status : status_word;
  // CTAs per SM: bounded by warps (16 consumer warps per SM is the target) and shared memory
  // (each SM has ~228 KB, 1 KB of it reserved per CTA)
  int per_sm = 16 / H;
  if (per_sm < 2) per_sm = 2;
  if (per_sm > 8) per_sm = 8;
  int ns = 0;
  for (; per_sm >= 1; --per_sm) {
    const int budget = (max_smem + 1024) / per_sm - 1024;
    ns = (budget - fixed) / P.stage_bytes;
    if (ns > 6) ns = 6;
    if (ns >= 2) break;
  }
  if (per_sm < 1 || ns < 2) return ECHOKV_OK;
  if ((g_decode_path >> 8) & 15) {  // experiments only: forced CTAs per SM / stage count
    const int f_sm = (g_decode_path >> 8) & 15, f_ns = (g_decode_path >> 12) & 15;
    if (fixed + f_ns * P.stage_bytes <= (max_smem + 1024) / f_sm - 1024) { per_sm = f_sm; ns = f_ns; }
  }
  P.NS = ns;
  const int smem_bytes = fixed + ns * P.stage_bytes;
  int64_t grid = (int64_t)num_sms * per_sm;
  const int64_t n_items = num_seqs * (int64_t)A.num_splits;
  if (grid > n_items) grid = n_items;
  if (cudaMemsetAsync(counter, 0, sizeof(int), st) != cudaSuccess) return check_launch("decode (work counter)");
  if (g_ev_before) cudaEventRecord(g_ev_before, st);
  switch (H) {
    case 1: decode_mma_kernel<1><<<(unsigned)grid, 2 * 32, smem_bytes, st>>>(P); break;
    case 2: decode_mma_kernel<2><<<(unsigned)grid, 3 * 32, smem_bytes, st>>>(P); break;
    case 4: decode_mma_kernel<4><<<(unsigned)grid, 5 * 32, smem_bytes, st>>>(P); break;
    default: decode_mma_kernel<8><<<(unsigned)grid, 9 * 32, smem_bytes, st>>>(P); break;
  }
  if (g_ev_after) cudaEventRecord(g_ev_after, st);
  int rc = check_launch("decode (tensor-core kernel)");
  if (rc) return rc;
  *handled = true;
  return ECHOKV_OK;
}

}  // namespace echokv

#ifdef ECHOKV_PROFILE
extern "C" int echokv_debug_prof(long long* dst, int n) {
  return (int)cudaMemcpyFromSymbol(dst, echokv::mma::g_prof, sizeof(long long) * n);
}
extern "C" int echokv_debug_phase(unsigned long long* dst, int reset) {
  int rc = (int)cudaMemcpyFromSymbol(dst, echokv::mma::g_phase, sizeof(unsigned long long) * 8);
  if (reset) { unsigned long long z[8] = {}; cudaMemcpyToSymbol(echokv::mma::g_phase, z, sizeof(z)); }
  return rc;
}
#endif

extern "C" int echokv_set_decode_events(void* before, void* after) {
  echokv::g_ev_before = reinterpret_cast<cudaEvent_t>(before);
  echokv::g_ev_after = reinterpret_cast<cudaEvent_t>(after);
  return ECHOKV_OK;
}

extern "C" int echokv_set_decode_path(int path) {
  const int old = echokv::g_decode_path;
  echokv::g_decode_path = path;
  return old;
}
