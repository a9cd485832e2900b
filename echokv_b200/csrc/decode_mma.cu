// Tensor-core split-K paged decode attention for sm_100a.
//
// Persistent CTAs (a few per SM) claim (sequence, split) work items from a global counter.  A CTA
// is one producer warp plus H consumer warps, one per KV head.  The producer resolves block table
// -> page header -> chunk ids -> residual map for up to 32 blocks at a time and streams 16-token
// tiles into a ring of shared-memory stages with bulk asynchronous copies (cp.async.bulk +
// mbarrier complete_tx).  A stage has one size whatever the tier of the block: eight slots of two
// token rows of 128 * H bytes (the row of an INT4 token), padded by 16 bytes so that ldmatrix over
// eight slots stays bank-conflict free (the MMA's token rows are permuted to match: even tokens
// first, then odd), then the tile's V stats, its K group's per-channel stats and a small header.
// An INT4 or INT2 tile takes one stage; an INT8 tile takes two, its K codes and K stats in the
// first and its V codes and V stats in the second.  Two consecutive full INT4 / INT2 tiles of a work
// item are flagged as a pair and worked off together by the consumers (one wait, one header, one
// softmax update and two independent chains of tensor-core instructions).
//
// Per group of one or two tiles a consumer warp
//   * folds the K group's per-channel scale into its register copy of the query (q' = q * k_scale,
//     fp16) and adds the constant q . k_min through extra MMA k-steps, so packed K codes feed the
//     tensor cores as plain integers:  S^T[t, g] = sum_d code[t, d] * q'[g, d] + sum_d k_min[d] * q[g, d];
//   * turns codes into fp16 operands by masking them in place (a code alone in a 16-bit lane is
//     the subnormal code * 2^-24 times a power of two that depends on its bit position; the powers of
//     two are pre-applied to the query copy / undone on the fp32 scores and accumulators), straight
//     from ldmatrix fragments (non-transposed for K, transposed for V so that register pairs run
//     along tokens); the V codes of INT2 blocks, which are multiplied by their scales in fp16, use
//     magic numbers (1024 + c etc.) and an exact subtract instead;
//   * keeps an online softmax per query head over tokens (the M dimension) with warp shuffles,
//     transposes P with movmatrix and accumulates O^T[d, g] += V^T[d, t] * P[t, g]; V's per-token
//     scale is folded into P per V group (INT8 / INT4) or into the codes (INT2), V's min and the
//     softmax denominator come from one more MMA against [v_min | ones].
// Accumulator registers map to channels in a tier-specific order (it follows how ldmatrix deals
// out packed codes); when consecutive blocks differ in tier the warp re-maps its accumulators
// through shared memory.  A split's tiles are accumulated in order by one warp, tiles are paired by
// a rule that looks at the split alone, and splits are merged in split order, so a sequence's
// result depends on its own length only, not on which CTA ran which item.  Every wait on a barrier
// is bounded in time; a wait that gives up ends the CTA's work and raises the status word.
#include <utility>

#include "decode_generic.cuh"

namespace echokv {
namespace mma {

#ifdef ECHOKV_PROFILE
// Instrumented build only (-DECHOKV_PROFILE): cycles spent per phase by lane 0 of consumer warp 0 of every CTA.
__device__ unsigned long long g_phase[16];
__device__ unsigned long long g_cta[1024 * 4];  // per CTA: start ns, end ns, SM id, cycles
#define PROF_T(x) const long long x = clock64()
#define PROF_PHASE(k, a, b) if (ln.h == 0 && ln.lane == 0) atomicAdd(&g_phase[k], (unsigned long long)((b) - (a)))
#else
#define PROF_T(x)
#define PROF_PHASE(k, a, b)
#endif

constexpr int D = 128;          // head size of this kernel
constexpr int NG = 4;           // V groups per head (v_group 32)
constexpr int TILE = 16;        // tokens per tile
constexpr unsigned long long WAIT_NS = 2000000000ull;  // a wait gives up after this long (echokv_set_decode_wait_limit changes it)

// What the producer tells the consumers about a staged group (stored at `o_hdr` of its first stage).
constexpr int F_RES = 1, F_FIRST = 2, F_LAST = 4;  // K from the residual buffer / first / last group of a work item
constexpr int F_PAIR = 8;                          // the next stage holds a second full tile of the same tier
constexpr int RT_LOG_SHIFT = 8;                    // plan entries only: bits 8..11 = log2(token rows per run), 15 = not a power of two
constexpr int F_MASK = 0xff;                       // the flag bits a stage header carries
struct alignas(16) StageHeader {
  int bits, n_valid, flags, pos0;   // n_valid: 1..16 tokens, -1 = no more work
  long long res_slot;
  int seq, split;
};
// The producer's own notes for one tile of the unit it is working off: the header and every copy source.
struct alignas(16) TilePlan {
  StageHeader hdr;
  const unsigned char* stats[4];    // V scale, V min, K scale, K min of the tile (one run from stats[0] when contiguous)
  const unsigned char* run[4];      // the tile's token rows lie in up to four runs (one per chunk it touches) of `TILE >> run_shift` rows
};
constexpr int UNIT = 16;         // tiles planned at a time (one per producer lane)
constexpr int MAX_NS = 8;        // stage ring slots at most
constexpr int HDR_BYTES = 256;   // 2 * MAX_NS mbarriers
static_assert(sizeof(StageHeader) == 32 && sizeof(TilePlan) % 16 == 0, "16-byte copies of headers");
static_assert(2 * MAX_NS * 8 <= HDR_BYTES, "barriers must fit the header");

// Stage layout (bytes from the stage base), the same for every tier.
__host__ __device__ constexpr int slot_bytes(int H) { return 256 * H + 16; }            // two INT4-sized token rows + padding
__host__ __device__ constexpr int o_vs(int H) { return (TILE / 2) * slot_bytes(H); }    // V scales fp16 [16][H][NG]
__host__ __device__ constexpr int o_vm(int H) { return o_vs(H) + TILE * H * NG * 2; }   // V mins
__host__ __device__ constexpr int o_ks(int H) { return o_vm(H) + TILE * H * NG * 2; }   // K scales fp16 [H][D]
__host__ __device__ constexpr int o_km(int H) { return o_ks(H) + H * D * 2; }           // K mins
__host__ __device__ constexpr int o_hdr(int H) { return o_km(H) + H * D * 2; }          // StageHeader
__host__ __device__ constexpr int o_ones(int H) { return o_hdr(H) + 32; }               // eight fp16 ones (never overwritten)
__host__ __device__ constexpr int stage_bytes(int H) { return (o_ones(H) + 16 + 127) / 128 * 128; }

struct Params {
  LayoutDev L;
  ResidualDev R;
  const uint8_t* pages;
  DecodeArgs A;
  int NS, num_seqs;
  int team_bytes;                          // shared memory of one team of a CTA
  int* status;                             // device status word (0 ok), may be null
  int* counter;                            // next unclaimed work item (zero at launch)
  int q_vec16;                             // 16-bit queries whose rows can be read with 16-byte loads
  unsigned long long wait_ns;              // a wait on a barrier or the remap lock gives up after this long
  int idle_producer;                       // test hook: the producer warps stage nothing, so every consumer wait runs out
};

// ---- PTX helpers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// One poll of the barrier's phase (the hardware may park the thread for a short, system-defined time).
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Returns false if the barrier did not flip within `limit_ns`.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned long long limit_ns) {
  if (mbar_try(bar, parity)) return true;
#pragma unroll 1
  for (int it = 0; it < 4; ++it) {  // the phase is usually about to complete: a few polls before backing off
    if (mbar_try(bar, parity)) return true;
  }
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int it = 0; it < 256; ++it) {
      __nanosleep(40);  // leave the issue slots to the warps that have work
      if (mbar_try(bar, parity)) return true;
    }
    if (global_ns() - t0 > limit_ns) return false;
  }
}
// The pages are read once per launch: their lines are marked evict-first in L2, so that what is read again (queries,
// block tables, split partials) stays there.
__device__ __forceinline__ uint64_t stream_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
// Ask for `bytes` (a multiple of 16) at `src` (16-byte aligned) to be brought into L2.
__device__ __forceinline__ void l2_prefetch(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
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
// a * (b.lo, b.lo) and a * (b.hi, b.hi): written with the intrinsics so that the compiler can use the
// half-select of the multiply instruction instead of a separate byte permute.
__device__ __forceinline__ uint32_t hmul2_lo(uint32_t a, uint32_t b) {
  const __half2 x = *reinterpret_cast<const __half2*>(&a), y = *reinterpret_cast<const __half2*>(&b);
  const __half2 z = __hmul2(x, __low2half2(y));
  return *reinterpret_cast<const uint32_t*>(&z);
}
__device__ __forceinline__ uint32_t hmul2_hi(uint32_t a, uint32_t b) {
  const __half2 x = *reinterpret_cast<const __half2*>(&a), y = *reinterpret_cast<const __half2*>(&b);
  const __half2 z = __hmul2(x, __high2half2(y));
  return *reinterpret_cast<const uint32_t*>(&z);
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

// ---- packed codes as fp16 operands ----------------------------------------------------------------
// A code byte, nibble or crumb masked in place inside a zero 16-bit lane is the fp16 SUBNORMAL
// code * 2^(pos - 24), pos being the bit position of the code's lowest bit (every position below bit 10
// is linear: the lowest normal binade has the subnormal spacing), with no conversion instruction at
// all.  A 32-bit word of packed codes yields register pairs (lo 16 bits, hi 16 bits):
//   INT8: 4 codes  -> pairs (0,1) (2,3)                           all at pos 0
//   INT4: 8 codes  -> pairs (0,4) (1,5) (2,6) (3,7)               pos 0, 4, 0, 4
//   INT2: 16 codes -> pairs (0,8) (1,9) ... (7,15)                pos 0, 2, 4, 6, 0, 2, 4, 6
// The 2^-pos of each position is pre-applied to the matching channels of the query copy (K side) or
// undone on the accumulator rows (V side), the 2^24 once on the fp32 scores / accumulators.
constexpr float CODE_UNSCALE = 16777216.f;  // 2^24
constexpr float RESCALE_SLACK = 6.f;

__device__ __forceinline__ void sub4(uint32_t w, uint32_t (&o)[4]) {
  o[0] = w & 0x000f000fu;
  o[1] = w & 0x00f000f0u;
  const uint32_t v = w >> 8;
  o[2] = v & 0x000f000fu;
  o[3] = v & 0x00f000f0u;
}
__device__ __forceinline__ void sub8(uint32_t w, uint32_t (&o)[2]) {
  o[0] = prmt(w, 0u, 0x4140u);
  o[1] = prmt(w, 0u, 0x4342u);
}
__device__ __forceinline__ void sub8_t(uint32_t w, uint32_t (&o)[2]) {  // [a.c0 a.c1 | b.c0 b.c1] -> (a.c0,b.c0) (a.c1,b.c1)
  o[0] = prmt(w, 0u, 0x4240u);
  o[1] = prmt(w, 0u, 0x4341u);
}
__device__ __forceinline__ void sub2(uint32_t w, uint32_t (&o)[8]) {
  o[0] = w & 0x00030003u;
  o[1] = w & 0x000c000cu;
  o[2] = w & 0x00300030u;
  o[3] = w & 0x00c000c0u;
  const uint32_t v = w >> 8;
  o[4] = v & 0x00030003u;
  o[5] = v & 0x000c000cu;
  o[6] = v & 0x00300030u;
  o[7] = v & 0x00c000c0u;
}
// INT2 codes as exact small integers (the V side multiplies them by their scales in fp16).
__device__ __forceinline__ void magic2(uint32_t w, uint32_t (&o)[8]) {
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

// Channel held by accumulator row (mt, r, half) for blocks of tier BITS.
template <int BITS>
__device__ __forceinline__ int acc_channel(int mt, int r, int half) {
  if constexpr (BITS == 8) return 16 * mt + 2 * r + half;
  else if constexpr (BITS == 4) return 32 * (mt >> 1) + 4 * r + 2 * (mt & 1) + half;
  else return 64 * (mt >> 2) + 8 * r + 2 * (mt & 3) + half;
}
// The PV accumulators of INT8 / INT4 blocks hold code units: rows fed by in-place subnormal codes
// are 2^-24 of the true value (2^-20 for the rows fed by upper nibbles: `half` 1 at INT4).
template <int BITS>
__device__ __forceinline__ float acc_unit(int half) {
  if constexpr (BITS == 8) return 16777216.f;
  else if constexpr (BITS == 4) return half ? 1048576.f : 16777216.f;
  else return 1.f;
}

// Shared-memory copy of a team's queries: [H][gqa query rows][D] fp16 and one zero row that every absent query
// column of the MMAs reads, pre-multiplied by softmax_scale * log2(e), rows padded by 16 bytes so that ldmatrix
// over the query rows is conflict free.
constexpr int QN_ROW = D * 2 + 16;
__host__ __device__ constexpr int q_copy_bytes(int H, int gqa) { return (H * gqa + 1) * QN_ROW; }
constexpr int REMAP_ROW = D + 4;                      // floats per query head in the canonical layout
constexpr int REMAP_BYTES = 8 * REMAP_ROW * 4;
constexpr int CTA_SHARED_BYTES = REMAP_BYTES + 128;  // the remap buffer and its lock, shared by the CTA's teams

struct WarpState {
  float acc[8][4];  // O^T tiles: [m-tile][c0..c3], channel order depends on `bits`
  float bl[4];      // [0],[1]: sum_t p * v_min for V group r (lanes r < NG); [2],[3]: sum_t p
  float m0, m1;     // running max (log2 domain) of query heads 2j and 2j+1
  int bits;         // tier whose channel order `acc` is in (0: none yet)
};

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

// Per-lane facts that do not change from tile to tile.
struct Lane {
  int h, lane, r, j;
  uint32_t qn_lane;   // shared address of this lane's query row (row lane / 4, or the zero row) in the warp's query copy
  uint32_t qn_ld;     // this lane's ldmatrix row address in the query copy (rows: query heads)
  uint32_t vs_row;    // stage offset of the V scales of token 2r (this head, all groups): 8 bytes; token 2r + 1 is H * 8 further
  uint32_t vm_ld;     // stage offset of this lane's ldmatrix row of the [v_min | ones] operand
  uint32_t km_ld;     // stage offset of this lane's ldmatrix row of the broadcast k_min operand (tile by lane & 8)
  uint32_t vs_row8;   // INT8 stages (eight tokens in natural order): V scales of token r of the stage
  uint32_t vm_ld8;    // INT8 stages: this lane's ldmatrix row of the [v_min | ones] operand (stage by lane & 16)
};

// This lane's ldmatrix row offset inside a stage for the K side / V side of tier BITS: lane & 7 picks the slot
// (tokens 2p, 2p + 1), lane & 8 the odd token of the slot, lane >> 4 the second 16-byte piece of the row.
// INT8 tiles lie in two stages of eight token rows each (tokens 0..7 and 8..15 in their natural order: MMA row r is
// token r): there lane & 7 picks the token of the stage and lane & 8 the stage.
template <int BITS, int H>
__device__ __forceinline__ uint32_t code_row(const Lane& ln, bool v_side) {
  const uint32_t pr = ln.lane & 7, odd = (ln.lane >> 3) & 1, piece = (ln.lane >> 4) * 16u;
  if constexpr (BITS == 8)  // a stage holds eight whole token rows, one per slot; the caller picks the stage by lane & 8
    return pr * slot_bytes(H) + ln.h * 128u + piece + (v_side ? 128u * H : 0u);
  else if constexpr (BITS == 4)
    return pr * slot_bytes(H) + odd * (128u * H) + ln.h * 64u + piece + (v_side ? 64u * H : 0u);
  else
    return pr * slot_bytes(H) + odd * (64u * H) + ln.h * 32u + piece + (v_side ? 32u * H : 0u);
}

// ---- Q.K^T over the codes of NT tiles, with the k_min term riding along -----------------------------------
// Per piece of channels the lane loads its slice of the query once (natural channel order, shared memory), and
// per tile multiplies it by the K group's scales (q' = q * k_scale, fp16), pairs the products the way the tier's
// unpacking pairs the codes, and runs the MMA k-steps:  c += codes * q'  in code units (2^-24).
// The query slice is pre-divided by the 2^pos of the code position each channel sits at (INT4: upper nibbles,
// INT2: crumbs at bits 2, 4, 6).
//
// The constant term of the scores, sum_d q[g, d] * k_min[d], is the same for every token of a K group; one chain
// of 8 more k-steps gives it for two tiles at once: the A fragment's rows 0..7 are the first tile's k_min row
// (ldmatrix with all eight row addresses equal), rows 8..15 the second tile's; the B fragments are the natural
// query (ldmatrix over the 8 query rows).  c2[0], c2[1]: first tile, query heads 2j, 2j+1; c2[2], c2[3]: second.
// The chains (one or two per tile, and this one) are interleaved so that no MMA waits for the one before it.
template <int BITS, int H, int NT>
__device__ __forceinline__ void qk_scores(const Lane& ln, const uint32_t (&sbk)[NT], uint32_t sb_hi, float (&c)[NT][4], float (&c2)[4]) {
  uint32_t krow[NT], ks[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    krow[t] = (BITS == 8 && (ln.lane & 8) ? sb_hi : sbk[t]) + code_row<BITS, H>(ln, false);
    ks[t] = sbk[t] + o_ks(H) + ln.h * (D * 2);
  }
  const uint32_t km_ld = ((ln.lane & 8) ? sbk[NT - 1] : sbk[0]) + ln.km_ld;
  uint32_t Bn[4];
  auto km_step = [&](auto kc) {  // k-step `k` of the k_min chain
    constexpr int k = decltype(kc)::value;
    uint32_t Am[4];
    if constexpr ((k & 1) == 0) ldsm_x4<(k / 2) * 64>(Bn, ln.qn_ld);
    ldsm_x4<k * 32>(Am, km_ld);
    mma16816(c2, Am[0], Am[1], Am[2], Am[3], Bn[2 * (k & 1)], Bn[2 * (k & 1) + 1]);
  };
  if constexpr (BITS == 8) {
    const uint32_t qp = ln.qn_lane + ln.j * 8;  // this lane's 4 channels of every 16-channel piece
    static_for<4>([&](auto ic) {  // pieces 2i, 2i+1 (16 channels each)
      constexpr int i = decltype(ic)::value;
      uint32_t R[NT][4];
#pragma unroll
      for (int t = 0; t < NT; ++t) ldsm_x4<i * 32>(R[t], krow[t]);
      static_for<2>([&](auto ec) {
        constexpr int e = decltype(ec)::value, p = 2 * i + e;
        const uint2 q = lds64<32 * p>(qp);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const uint2 sc = lds64<32 * p>(ks[t] + ln.j * 8);
          uint32_t a[2], b[2];
          sub8(R[t][2 * e], a);
          sub8(R[t][2 * e + 1], b);
          mma16816(c[t], a[0], b[0], a[1], b[1], hmul2u(q.x, sc.x), hmul2u(q.y, sc.y));
        }
        km_step(std::integral_constant<int, p>{});
      });
    });
  } else if constexpr (BITS == 4) {
    const uint32_t qp = ln.qn_lane + ln.j * 16;  // this lane's 8 channels of every 32-channel piece
    static_for<2>([&](auto ic) {  // pieces 2i, 2i+1 (32 channels each)
      constexpr int i = decltype(ic)::value;
      uint32_t R[NT][4];
#pragma unroll
      for (int t = 0; t < NT; ++t) ldsm_x4<i * 32>(R[t], krow[t]);
      static_for<2>([&](auto ec) {
        constexpr int e = decltype(ec)::value, p = 2 * i + e;
        uint32_t Q[4];
        lds128<64 * p>(Q, qp);
#pragma unroll
        for (int k = 0; k < 4; ++k) Q[k] = hmul2u(Q[k], 0x2c003c00u);  // odd channels sit in upper nibbles (pos 4): 2^-4
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          uint32_t S[4], Z[4];
          lds128<64 * p>(S, ks[t] + ln.j * 16);
#pragma unroll
          for (int k = 0; k < 4; ++k) Z[k] = hmul2u(Q[k], S[k]);
          uint32_t a[4], b[4];
          sub4(R[t][2 * e], a);
          sub4(R[t][2 * e + 1], b);
          mma16816(c[t], a[0], b[0], a[1], b[1], prmt(Z[0], Z[2], 0x5410u), prmt(Z[0], Z[2], 0x7632u));  // channels 0,4 | 1,5
          if (t == 0) km_step(std::integral_constant<int, 2 * p>{});
          mma16816(c[t], a[2], b[2], a[3], b[3], prmt(Z[1], Z[3], 0x5410u), prmt(Z[1], Z[3], 0x7632u));  // channels 2,6 | 3,7
        }
        km_step(std::integral_constant<int, 2 * p + 1>{});
      });
    });
  } else {
    const uint32_t qp = ln.qn_lane + ln.j * 32;  // this lane's 16 channels of every 64-channel piece
    uint32_t R[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) ldsm_x4<0>(R[t], krow[t]);  // pieces 0, 1 (64 channels each)
    static_for<2>([&](auto pc) {
      constexpr int p = decltype(pc)::value;
      uint32_t Q[8];
      {
        uint32_t t4[4];
        lds128<128 * p>(t4, qp);
        Q[0] = t4[0]; Q[1] = hmul2u(t4[1], 0x24002c00u); Q[2] = t4[2]; Q[3] = hmul2u(t4[3], 0x24002c00u);
        lds128<128 * p + 16>(t4, qp);
        Q[4] = t4[0]; Q[5] = hmul2u(t4[1], 0x24002c00u); Q[6] = t4[2]; Q[7] = hmul2u(t4[3], 0x24002c00u);
#pragma unroll
        for (int k = 0; k < 8; k += 2) Q[k] = hmul2u(Q[k], 0x34003c00u);  // crumbs at pos 0, 2: 1, 2^-2; at pos 4, 6: 2^-4, 2^-6
      }
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        uint32_t S[8], Z[8];
        {
          uint32_t t4[4];
          lds128<128 * p>(t4, ks[t] + ln.j * 32);      S[0] = t4[0]; S[1] = t4[1]; S[2] = t4[2]; S[3] = t4[3];
          lds128<128 * p + 16>(t4, ks[t] + ln.j * 32); S[4] = t4[0]; S[5] = t4[1]; S[6] = t4[2]; S[7] = t4[3];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) Z[k] = hmul2u(Q[k], S[k]);
        uint32_t a[8], b[8];
        sub2(R[t][2 * p], a);
        sub2(R[t][2 * p + 1], b);
        static_for<4>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          mma16816(c[t], a[2 * k], b[2 * k], a[2 * k + 1], b[2 * k + 1], prmt(Z[k], Z[k + 4], 0x5410u), prmt(Z[k], Z[k + 4], 0x7632u));
          if (t == 0) km_step(std::integral_constant<int, 4 * p + k>{});
        });
      }
    });
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
__device__ __noinline__ float4 qk_residual(const ResidualDev R, long long res_slot, int pos0, int n_valid, uint32_t qn_lane,
                                           int h, int lane, int natural) {
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  const int r = lane >> 2, j = lane & 3;
  const int t0 = natural ? r : 2 * r, t1 = natural ? r + 8 : 2 * r + 1;  // tokens of MMA rows r / r + 8
  const bool v0 = t0 < n_valid, v1 = t1 < n_valid;
  const int64_t e0 = res_slot * R.s_slot + (int64_t)(pos0 + t0) * R.s_pos + h * R.s_head;
  const int64_t e1 = e0 + (int64_t)(t1 - t0) * R.s_pos;
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
  return make_float4(c[0], c[1], c[2], c[3]);
}

// ---- P.V for one tile --------------------------------------------------------------------------
// p_lo / p_hi: this lane's probabilities in score layout (token 2r / 2r + 1, query heads 2j, 2j + 1), fp16.
// The B fragments of the MMAs are their 8x8 transposes.  INT8 / INT4: V's per-token scale of group G
// multiplies P before the transpose, where a lane needs the scales of just its own two tokens (8 bytes
// each, all groups), one fragment pair per group.  INT2: the scale goes into the codes, which needs it
// per token pair (the order of the A fragments).
template <int BITS, int H>
// `sb`: the tile's stage (INT8: the stage of tokens 0..7), `sb_hi`: the stage of tokens 8..15 of an INT8 tile.
__device__ __forceinline__ void pv_codes(const Lane& ln, uint32_t sb, uint32_t sb_hi, uint32_t p_lo, uint32_t p_hi, WarpState& w) {
  const uint32_t vrow = (BITS == 8 && (ln.lane & 8) ? sb_hi : sb) + code_row<BITS, H>(ln, true);
  const uint32_t pb0 = movm_t(p_lo), pb1 = movm_t(p_hi);
  // [v_min | ones] rows: the bias of every V group and the softmax denominator
  if constexpr (H >= 2) {
    uint32_t X[4];
    // (v_min of k slots 0..7, ones, v_min of k slots 8..15, ones): rows = groups of this pair of heads
    if constexpr (BITS == 8) ldsm_x4_t<0>(X, ((ln.lane & 16) ? sb_hi : sb) + ln.vm_ld8);
    else ldsm_x4_t<0>(X, sb + ln.vm_ld);
    mma16816(w.bl, X[0], X[1], X[2], X[3], pb0, pb1);
  } else {
    // k slots 2j, 2j+1, 2j+8, 2j+9 are tokens 4j, 4j+2, 4j+1, 4j+3 (INT8: tokens 2j, 2j+1 of either stage)
    const uint32_t g2 = (ln.r < NG ? ln.r : 0) * 2, tok = NG * 2;
    const uint32_t base = sb + o_vm(H) + (uint32_t)((BITS == 8 ? 2 : 4) * ln.j) * tok + g2;
    const uint32_t base_hi = BITS == 8 ? sb_hi + o_vm(H) + (uint32_t)(2 * ln.j) * tok + g2 : base + tok;
    uint32_t x0, x1, x2, x3;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(x0) : "r"(base));                                   // k slot 2j
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(x1) : "r"(base + (BITS == 8 ? 1 : 2) * tok));       // k slot 2j + 1
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(x2) : "r"(base_hi));                                // k slot 2j + 8
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(x3) : "r"(base_hi + (BITS == 8 ? 1 : 2) * tok));    // k slot 2j + 9
    const uint32_t keep = ln.r < NG ? 0xffffffffu : 0u;
    mma16816(w.bl, prmt(x0, x1, 0x5410u) & keep, 0x3c003c00u, prmt(x2, x3, 0x5410u) & keep, 0x3c003c00u, pb0, pb1);
  }
  const uint32_t vs_row = sb + (BITS == 8 ? ln.vs_row8 : ln.vs_row);
  if constexpr (BITS != 2) {
    uint32_t b0[NG], b1[NG];
    {
      // V scales (all four groups, 8 bytes) of this lane's two tokens: MMA rows r and r + 8
      const uint2 s0 = lds64<0>(vs_row), s1 = BITS == 8 ? lds64<0>(sb_hi + ln.vs_row8) : lds64<H * NG * 2>(vs_row);
      b0[0] = movm_t(hmul2_lo(p_lo, s0.x)); b0[1] = movm_t(hmul2_hi(p_lo, s0.x));
      b0[2] = movm_t(hmul2_lo(p_lo, s0.y)); b0[3] = movm_t(hmul2_hi(p_lo, s0.y));
      b1[0] = movm_t(hmul2_lo(p_hi, s1.x)); b1[1] = movm_t(hmul2_hi(p_hi, s1.x));
      b1[2] = movm_t(hmul2_lo(p_hi, s1.y)); b1[3] = movm_t(hmul2_hi(p_hi, s1.y));
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
    // score layout (token 2r / 2r + 1, all groups: 8 bytes each) and transposed into that order with
    // movmatrix: input column pair j carries group 2q + (j >= 2), so output lane r gets group 2q + (r >= 4).
    uint32_t sl[2], sh[2];
    {
      const uint2 s0 = lds64<0>(vs_row), s1 = lds64<H * NG * 2>(vs_row);
      const uint32_t sel = (ln.lane & 2) ? 0x3232u : 0x1010u;
      sl[0] = movm_t(prmt(s0.x, s0.x, sel)); sl[1] = movm_t(prmt(s0.y, s0.y, sel));
      sh[0] = movm_t(prmt(s1.x, s1.x, sel)); sh[1] = movm_t(prmt(s1.y, s1.y, sel));
    }
    uint32_t Q[4];
    ldsm_x4_t<0>(Q, vrow);  // pieces 0, 1 = V groups {0,1}, {2,3}; this lane's channels lie in group 2q + (r >= 4)
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t lo[8], hi[8];
      magic2(Q[2 * q], lo);
      magic2(Q[2 * q + 1], hi);
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

// Bring the warp's state to tier BITS: the register copy of the query and the accumulators' channel order.
template <int BITS>
__device__ __forceinline__ void enter_tier(WarpState& w, const Lane& ln, float* remap, int* lock, unsigned long long limit_ns, bool& ok) {
  if (w.bits != BITS) {
    if (w.bits != 0) {  // re-map the accumulators to this tier's channel order (rare: tier changes inside a work item)
      if (ln.lane == 0) {
        const unsigned long long t0 = global_ns();
        while (atomicCAS(lock, 0, 1) != 0) {
          if (global_ns() - t0 > limit_ns) { ok = false; break; }
        }
      }
      __syncwarp();
      store_any(w, remap, ln.r, ln.j);
      __syncwarp();
      load_canonical<BITS>(w, remap, ln.r, ln.j);
      __syncwarp();
      if (ln.lane == 0) atomicExch(lock, 0);
    }
    w.bits = BITS;
  }
}

// One group: NT tiles (stage bases sbk[t] for the K side, sbv[t] for the V side; they differ at INT8 only).
// With NT == 2 both tiles are full and code-based.  With NT == 1 the tile may be partial (`n_valid` < 16) and its
// K may come from the residual buffer.
template <int BITS, int H, int NT>
__device__ __forceinline__ void process_group(const Params& P, const Lane& ln, const uint32_t (&sbk)[NT], const uint32_t (&sbv)[NT],
                                              int n_valid, bool in_res, long long res_slot, int pos0, WarpState& w,
                                              float* remap, int* lock, bool& ok) {
  PROF_T(f0);
  enter_tier<BITS>(w, ln, remap, lock, P.wait_ns, ok);
  float c[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t) c[t][0] = c[t][1] = c[t][2] = c[t][3] = 0.f;
  if (NT == 1 && in_res) {
    const float4 s4 = qk_residual(P.R, res_slot, pos0, n_valid, ln.qn_lane, ln.h, ln.lane, BITS == 8);
    c[0][0] = s4.x; c[0][1] = s4.y; c[0][2] = s4.z; c[0][3] = s4.w;
  } else {
    // scores in code units; the k_min chain rides along
    float c2[4] = {0.f, 0.f, 0.f, 0.f};
    qk_scores<BITS, H, NT>(ln, sbk, sbv[0], c, c2);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
#pragma unroll
      for (int k = 0; k < 4; ++k) c[t][k] = fmaf(c[t][k], CODE_UNSCALE, c2[2 * (NT == 1 ? 0 : t) + (k & 1)]);
    }
  }
  if (NT == 1 && n_valid < TILE) {  // a partial tile (the sequence's last): tokens past the end do not count
    const int t0 = BITS == 8 ? ln.r : 2 * ln.r, t1 = BITS == 8 ? ln.r + 8 : 2 * ln.r + 1;  // tokens of MMA rows r / r + 8
    if (t0 >= n_valid) { c[0][0] = -INFINITY; c[0][1] = -INFINITY; }
    if (t1 >= n_valid) { c[0][2] = -INFINITY; c[0][3] = -INFINITY; }
  }
  PROF_T(f1);
  PROF_PHASE(0, f0, f1);
  // online softmax over tokens (rows); columns 2j, 2j+1 belong to this lane
  float t0 = fmaxf(c[0][0], c[0][2]), t1 = fmaxf(c[0][1], c[0][3]);
  if (NT == 2) {
    t0 = fmaxf(t0, fmaxf(c[NT - 1][0], c[NT - 1][2]));
    t1 = fmaxf(t1, fmaxf(c[NT - 1][1], c[NT - 1][3]));
  }
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, o));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, o));
  }
  // The reference point of the exponentials only moves when a group's maximum exceeds it by more
  // than RESCALE_SLACK (in log2 units): until then p <= 2^RESCALE_SLACK, well inside fp16, and the
  // accumulators need no rescaling.  The result is the same softmax (the reference point cancels).
  const bool grew = (t0 > w.m0 + RESCALE_SLACK) || (t1 > w.m1 + RESCALE_SLACK);
  if (__any_sync(0xffffffffu, grew)) {
    const float n0 = fmaxf(w.m0, t0), n1 = fmaxf(w.m1, t1);
    const float a0 = ex2(w.m0 - n0), a1 = ex2(w.m1 - n1);
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) { w.acc[mt][0] *= a0; w.acc[mt][1] *= a1; w.acc[mt][2] *= a0; w.acc[mt][3] *= a1; }
    w.bl[0] *= a0; w.bl[1] *= a1; w.bl[2] *= a0; w.bl[3] *= a1;
    w.m0 = n0; w.m1 = n1;
  }
  uint32_t p_lo[NT], p_hi[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    p_lo[t] = pack_h2(ex2(c[t][0] - w.m0), ex2(c[t][1] - w.m1));   // token 2r
    p_hi[t] = pack_h2(ex2(c[t][2] - w.m0), ex2(c[t][3] - w.m1));   // token 2r + 1
  }
  PROF_T(f2);
  PROF_PHASE(1, f1, f2);
#pragma unroll
  for (int t = 0; t < NT; ++t) pv_codes<BITS, H>(ln, BITS == 8 ? sbk[t] : sbv[t], sbv[t], p_lo[t], p_hi[t], w);
  PROF_T(f3);
  PROF_PHASE(2, f2, f3);
  PROF_PHASE(3, 0, 1);  // groups
}

// ---- the kernel ------------------------------------------------------------------------------
__device__ __forceinline__ bool item_range(const Params& P, int bps_min, int item, int& seq, int& split,
                                           int64_t& seq_len, int& b_start, int& b_end) {
  seq = item % P.num_seqs;
  split = item / P.num_seqs;
  seq_len = P.A.lens[seq];
  return split_range(seq_len, P.L.BS, P.A.num_splits, bps_min, split, b_start, b_end);
}

// Block metadata the producer warp prefetches for up to 32 blocks at a time (one block per lane).
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

// The split's partial result: accumulators (in true units, V min contributions added) to acc[seq, head, split, :],
// running maximum and denominator to ml.  A lane's accumulator rows are neighbouring channels (INT4: 4 per V group,
// INT2: 8 per half of the head, INT8: 2 per 16-channel tile), so they leave as 16- or 8-byte stores that the
// eight lanes of a query head put side by side.
template <int BITS, int H>
__device__ __forceinline__ void write_partial(const Params& P, const WarpState& w, int seq, int split, int h, int lane) {
  const int r = lane >> 2, j = lane & 3;
  const DecodeArgs& A = P.A;
  const int g0 = 2 * j, g1 = 2 * j + 1;
  const int64_t o0 = (((int64_t)seq * A.Hq + h * A.gqa + g0) * A.num_splits + split);
  const int64_t o1 = o0 + A.num_splits;
  float* dst0 = A.acc + o0 * D;
  float* dst1 = A.acc + o1 * D;
  const bool on0 = g0 < A.gqa, on1 = g1 < A.gqa;
  // V min contribution of V group G: held by lane (r = bias_row(G), j)
  float bias0[NG], bias1[NG];
#pragma unroll
  for (int G = 0; G < NG; ++G) {
    bias0[G] = __shfl_sync(0xffffffffu, w.bl[0], bias_row<H>(G, h) * 4 + j);
    bias1[G] = __shfl_sync(0xffffffffu, w.bl[1], bias_row<H>(G, h) * 4 + j);
  }
  if constexpr (BITS == 4) {  // m-tiles 2G, 2G+1: channels 32G + 4r + {0,1} and {2,3}
#pragma unroll
    for (int G = 0; G < NG; ++G) {
      const float u0 = acc_unit<4>(0), u1 = acc_unit<4>(1);
      const int ch = 32 * G + 4 * r;
      if (on0) *reinterpret_cast<float4*>(dst0 + ch) = make_float4(
          fmaf(w.acc[2 * G][0], u0, bias0[G]), fmaf(w.acc[2 * G][2], u1, bias0[G]),
          fmaf(w.acc[2 * G + 1][0], u0, bias0[G]), fmaf(w.acc[2 * G + 1][2], u1, bias0[G]));
      if (on1) *reinterpret_cast<float4*>(dst1 + ch) = make_float4(
          fmaf(w.acc[2 * G][1], u0, bias1[G]), fmaf(w.acc[2 * G][3], u1, bias1[G]),
          fmaf(w.acc[2 * G + 1][1], u0, bias1[G]), fmaf(w.acc[2 * G + 1][3], u1, bias1[G]));
    }
  } else if constexpr (BITS == 2) {  // m-tiles 4q .. 4q+3: channels 64q + 8r + {0..7}, all in V group 2q + (r >= 4)
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const float b0 = r >= 4 ? bias0[2 * q + 1] : bias0[2 * q], b1 = r >= 4 ? bias1[2 * q + 1] : bias1[2 * q];
      const int ch = 64 * q + 8 * r;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int m = 4 * q + 2 * e;
        if (on0) *reinterpret_cast<float4*>(dst0 + ch + 4 * e) = make_float4(w.acc[m][0] + b0, w.acc[m][2] + b0, w.acc[m + 1][0] + b0, w.acc[m + 1][2] + b0);
        if (on1) *reinterpret_cast<float4*>(dst1 + ch + 4 * e) = make_float4(w.acc[m][1] + b1, w.acc[m][3] + b1, w.acc[m + 1][1] + b1, w.acc[m + 1][3] + b1);
      }
    }
  } else {  // m-tile mt: channels 16 mt + 2r + {0, 1}, V group mt / 2
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      const float u = acc_unit<8>(0);
      const int ch = 16 * mt + 2 * r;
      if (on0) *reinterpret_cast<float2*>(dst0 + ch) = make_float2(fmaf(w.acc[mt][0], u, bias0[mt >> 1]), fmaf(w.acc[mt][2], u, bias0[mt >> 1]));
      if (on1) *reinterpret_cast<float2*>(dst1 + ch) = make_float2(fmaf(w.acc[mt][1], u, bias1[mt >> 1]), fmaf(w.acc[mt][3], u, bias1[mt >> 1]));
    }
  }
  if (r == 0) {
    if (on0) *reinterpret_cast<float2*>(A.ml + o0 * 2) = make_float2(w.m0, w.bl[2]);
    if (on1) *reinterpret_cast<float2*>(A.ml + o1 * 2) = make_float2(w.m1, w.bl[3]);
  }
}
__device__ __forceinline__ int ring_next(int st, int NS) { return st + 1 == NS ? 0 : st + 1; }

// Teams per CTA: a CTA is V independent teams of H consumer warps + 1 producer warp, each with its own barriers,
// plans, query copy and stage ring in its slice of the CTA's shared memory.  One CTA per SM.  Registers are handed
// out per SM sub-partition (16,384 each): with 17 to 20 warps per SM (5 on a sub-partition) a thread gets 96, so
// V is chosen to use those 18 to 20 warps for every H.  The smaller V of each H is for shapes whose per-team shared
// memory (many query heads per KV head) does not fit V times.
template <int H> struct Teams {
  static constexpr int V = H == 8 ? 2 : (H == 4 ? 4 : (H == 2 ? 6 : 10));   // 18 / 20 / 18 / 20 warps
  static constexpr int V_SMALL = H == 8 ? 1 : (H == 4 ? 3 : (H == 2 ? 4 : 7));
};

template <int H, int V>
__global__ void __launch_bounds__((H + 1) * 32 * V, 1) decode_mma_kernel(const Params P) {
  extern __shared__ __align__(128) unsigned char smem_all[];
  pdl_launch_dependents();  // the merge may take its place behind this kernel; it waits for this kernel to complete
  constexpr int TEAM_THREADS = (H + 1) * 32;
  const LayoutDev& L = P.L;
  const DecodeArgs& A = P.A;
  const int team = threadIdx.x / TEAM_THREADS, tid = threadIdx.x - team * TEAM_THREADS;
  const int warp = tid >> 5, lane = tid & 31;
  const int NS = P.NS;
  const int n_items = P.num_seqs * A.num_splits;
  constexpr int SB = stage_bytes(H);
#ifdef ECHOKV_PROFILE
  const unsigned long long cta_t0 = global_ns();
  const long long cta_c0 = clock64();
#endif

  // shared memory of the CTA: [remap buffer | its lock] once (a warp needs it only when the tier changes inside a work
  // item), then per team: [barriers][tile plans][query copy per head][stage ring]
  float* remap = reinterpret_cast<float*>(smem_all);
  int* lock = reinterpret_cast<int*>(smem_all + REMAP_BYTES);
  unsigned char* smem = smem_all + CTA_SHARED_BYTES + (size_t)team * P.team_bytes;
  uint64_t* sfull = reinterpret_cast<uint64_t*>(smem);   // stage ring: header written, copies landed
  uint64_t* sempty = sfull + MAX_NS;                     // stage ring: every consumer warp is done with the stage
  TilePlan* plan = reinterpret_cast<TilePlan*>(smem + HDR_BYTES);
  unsigned char* qs = smem + HDR_BYTES + UNIT * sizeof(TilePlan);
  unsigned char* ring = qs + (q_copy_bytes(H, A.gqa) + 127) / 128 * 128;
  const uint32_t ring_u = smem_u32(ring), full_u = smem_u32(sfull), empty_u = smem_u32(sempty);

  if (tid == 0) {
    for (int s = 0; s < MAX_NS; ++s) { mbar_init(sfull + s, 1); mbar_init(sempty + s, H * 32); }
    if (team == 0) *lock = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  {  // zero the ring once: rows of a partial tile that are never copied must read as finite numbers
    const int n16 = (NS * SB) / 16;
    uint4* z = reinterpret_cast<uint4*>(ring);
    for (int i = tid; i < n16; i += TEAM_THREADS) z[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    if (tid < NS)  // the row of ones the [v_min | ones] operand reads: no copy ever lands on it
      *reinterpret_cast<uint4*>(ring + (size_t)tid * SB + o_ones(H)) = make_uint4(0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the bulk copies write the same bytes later
  }
  __syncthreads();
  // Barriers and ring are set up.  From here on the consumers read what the kernels before this one wrote (queries,
  // pages, split partials); the producer first resolves its first work item's metadata, which no kernel of the step
  // writes (lengths, block table, page headers and the residual map are set before the step's kernels start).
  if (warp != H) pdl_wait();

  bool ok = true;
  if (warp == H) {
    // ===================== producer warp =====================
    const int tpb = L.BS / TILE;                     // tiles per block
    const int U = tpb >= UNIT ? 1 : UNIT / tpb;      // blocks per unit
    const bool contig = L.BS == TILE && L.KG == TILE;  // a tile's four stats arrays form one run in the page
    const uint64_t policy = stream_policy();
    if (P.q_vec16 && A.q_s1 == D) {  // the batch's query rows into L2 now: a work item's first step is to read one
      const int elt = 2, teams = gridDim.x * V, me = blockIdx.x * V + team;
      for (int sq = me * 32 + lane; sq < P.num_seqs; sq += teams * 32) {
        const int64_t q_row = A.q_rows ? A.q_rows[sq] : sq;
        l2_prefetch(reinterpret_cast<const unsigned char*>(A.q) + q_row * A.q_s0 * elt, (uint32_t)(A.Hq * D * elt));
      }
    }
    int st = 0;                                      // next stage to fill
    uint32_t pph = 0xffffffffu;                      // per stage: parity of the `empty` phase to wait for (all ones: first use is free)
    uint32_t fills = 0;                              // stages filled so far
    int seq = 0, split = 0, b_start = 0, b_end = 0, base = 0;
    int64_t seq_len = 0, bt_row = 0;
    bool have = false;
    const int bps_min = bps_floor(A);
    // A team's first work item is its own index; the counter (which the merge kernel before this one may still be
    // resetting when this runs ahead of `pdl_wait`) hands out the items after the first round.
    const int n_teams = gridDim.x * V;
    bool first_claim = true;
    auto advance = [&]() {  // move to the next unit (claiming a new item when needed); false when there is no work left
      if (have && base + U < b_end) { base += U; return true; }
      for (;;) {
        int it = 0;
        if (first_claim) {
          it = blockIdx.x * V + team;
          first_claim = false;
        } else {
          if (lane == 0) it = atomicAdd(P.counter, 1);
          it = __shfl_sync(0xffffffffu, it, 0) + n_teams;
        }
        if (it >= n_items) { have = false; return false; }
        if (item_range(P, bps_min, it, seq, split, seq_len, b_start, b_end)) {
          base = b_start; bt_row = A.bt_rows ? A.bt_rows[seq] : seq; have = true;
          return true;
        }
      }
    };
    // Fill one stage: wait until the consumers have released it, write the header, start the copies.
    // `rows`: 1 = a whole INT4 / INT2 tile (token rows in pairs, all stats); 2 / 3 = the first / second half of an INT8
    // tile (eight whole token rows, their V stats; the K stats with the first half).
    auto fill = [&](const TilePlan& d, int flags_extra, int rows) -> bool {
      // Everything that does not need the stage to be free comes first (header values, each lane's one copy: where
      // from, where to, how long), so that the wait for the consumers' release is followed by the header store, the
      // byte count and the copies alone.
      const int4 h0 = *reinterpret_cast<const int4*>(&d.hdr);   // bits, n_valid, flags, pos0
      const int4 h1 = reinterpret_cast<const int4*>(&d.hdr)[1];
      const int nv = h0.y;
      const uint32_t side = 16u * H * h0.x;                     // bytes of one side (K or V) of a token row: H * D * bits / 8
      const uint32_t k_stats = 2u * H * D * 2, v_stats = 2u * TILE * H * NG * 2;
      const int rt_log = (h0.z >> RT_LOG_SHIFT) & 15;           // token rows per run (see TilePlan) = 1 << rt_log
      auto row_src = [&](int t) {
        if (rt_log != 15) return d.run[t >> rt_log] + (uint32_t)(t & ((1 << rt_log) - 1)) * 2u * side;
        const int rt = min((2 * L.BS) / h0.x, TILE);
        return d.run[t / rt] + (uint32_t)(t % rt) * 2u * side;
      };
      const int half0 = rows == 3 ? TILE / 2 : 0;               // first token of an INT8 half
      const int nh = rows == 1 ? nv : max(0, min(nv - half0, TILE / 2));  // token rows this stage receives
      const uint32_t tx = rows == 1 ? nv * 2 * side + k_stats + v_stats : nh * 2 * side + v_stats / 2 + (rows == 2 ? k_stats : 0u);
      uint32_t c_dst = 0, c_bytes = 0;
      const unsigned char* c_src = nullptr;
      if (rows == 1) {
        // lane p < 8 copies tokens 2p and 2p + 1 in one piece (neighbours in their chunk: a chunk holds an even number of tokens)
        if (lane < 8) {
          if (2 * lane < nv) { c_dst = lane * slot_bytes(H); c_src = row_src(2 * lane); c_bytes = (2 * lane + 1 < nv ? 4u : 2u) * side; }
        } else if (contig) {
          if (lane == 16) { c_dst = o_vs(H); c_src = d.stats[0]; c_bytes = v_stats + k_stats; }
        } else if (lane >= 16 && lane < 20) {
          const int which = lane - 16;  // vs, vm, ks, km
          c_dst = which == 0 ? o_vs(H) : which == 1 ? o_vm(H) : which == 2 ? o_ks(H) : o_km(H);
          c_src = d.stats[which];
          c_bytes = which < 2 ? v_stats / 2 : k_stats / 2;
        }
      } else {
        // lane t < 8 copies the whole row [K | V] of token half0 + t to slot t
        if (lane < nh) { c_dst = lane * slot_bytes(H); c_src = row_src(half0 + lane); c_bytes = 2u * side; }
        // the V stats of the half's eight tokens; with the first half the K group's stats
        if (lane == 16) { c_dst = o_vs(H); c_src = d.stats[0] + half0 * (H * NG * 2); c_bytes = v_stats / 4; }
        if (lane == 17) { c_dst = o_vm(H); c_src = d.stats[1] + half0 * (H * NG * 2); c_bytes = v_stats / 4; }
        if (rows == 2) {
          if (contig) { if (lane == 18) { c_dst = o_ks(H); c_src = d.stats[2]; c_bytes = k_stats; } }
          else if (lane == 18 || lane == 19) { c_dst = lane == 18 ? o_ks(H) : o_km(H); c_src = d.stats[lane - 16]; c_bytes = k_stats / 2; }
        }
      }
      if (!mbar_wait(empty_u + st * 8, (pph >> st) & 1, P.wait_ns)) return false;
      pph ^= 1u << st;
      const uint32_t bar = full_u + st * 8, st_u = ring_u + (uint32_t)st * SB;
      if (lane == 0) {
        int4* hd = reinterpret_cast<int4*>(ring + (size_t)st * SB + o_hdr(H));
        hd[0] = make_int4(h0.x, h0.y, (h0.z & F_MASK) | flags_extra, h0.w);
        hd[1] = h1;
        mbar_expect_tx(bar, tx);
      }
      __syncwarp();
      if (c_bytes) bulk_copy(st_u + c_dst, c_src, c_bytes, bar, policy);
      ++fills;
      st = ring_next(st, NS);
      return true;
    };
    // Two stages in one pass (the two tiles of a pair, or the two halves of an INT8 tile): lanes 0..15 prepare and
    // issue the first stage's copies, lanes 16..31 the second's (rows from sub-lanes 0..7, statistics from 8..11).
    auto fill2 = [&](const TilePlan& dA, int fxA, int rowsA, const TilePlan& dB, int fxB, int rowsB) -> bool {
      const int half = lane >> 4, sl = lane & 15;
      const TilePlan& d = half ? dB : dA;
      const int rows = half ? rowsB : rowsA, fx = half ? fxB : fxA;
      const int4 h0 = *reinterpret_cast<const int4*>(&d.hdr);
      const int4 h1 = reinterpret_cast<const int4*>(&d.hdr)[1];
      const int nv = h0.y;
      const uint32_t side = 16u * H * h0.x;
      const uint32_t k_stats = 2u * H * D * 2, v_stats = 2u * TILE * H * NG * 2;
      const int rt_log = (h0.z >> RT_LOG_SHIFT) & 15;           // token rows per run (see TilePlan) = 1 << rt_log
      auto row_src = [&](int t) {
        if (rt_log != 15) return d.run[t >> rt_log] + (uint32_t)(t & ((1 << rt_log) - 1)) * 2u * side;
        const int rt = min((2 * L.BS) / h0.x, TILE);
        return d.run[t / rt] + (uint32_t)(t % rt) * 2u * side;
      };
      const int half0 = rows == 3 ? TILE / 2 : 0;
      const int nh = rows == 1 ? nv : max(0, min(nv - half0, TILE / 2));
      const uint32_t tx = rows == 1 ? nv * 2 * side + k_stats + v_stats : nh * 2 * side + v_stats / 2 + (rows == 2 ? k_stats : 0u);
      uint32_t c_dst = 0, c_bytes = 0;
      const unsigned char* c_src = nullptr;
      if (rows == 1) {
        if (sl < 8) {
          if (2 * sl < nv) { c_dst = sl * slot_bytes(H); c_src = row_src(2 * sl); c_bytes = (2 * sl + 1 < nv ? 4u : 2u) * side; }
        } else if (contig) {
          if (sl == 8) { c_dst = o_vs(H); c_src = d.stats[0]; c_bytes = v_stats + k_stats; }
        } else if (sl < 12) {
          const int which = sl - 8;  // vs, vm, ks, km
          c_dst = which == 0 ? o_vs(H) : which == 1 ? o_vm(H) : which == 2 ? o_ks(H) : o_km(H);
          c_src = d.stats[which];
          c_bytes = which < 2 ? v_stats / 2 : k_stats / 2;
        }
      } else {
        if (sl < nh && sl < 8) { c_dst = sl * slot_bytes(H); c_src = row_src(half0 + sl); c_bytes = 2u * side; }
        if (sl == 8) { c_dst = o_vs(H); c_src = d.stats[0] + half0 * (H * NG * 2); c_bytes = v_stats / 4; }
        if (sl == 9) { c_dst = o_vm(H); c_src = d.stats[1] + half0 * (H * NG * 2); c_bytes = v_stats / 4; }
        if (rows == 2) {
          if (contig) { if (sl == 10) { c_dst = o_ks(H); c_src = d.stats[2]; c_bytes = k_stats; } }
          else if (sl == 10 || sl == 11) { c_dst = sl == 10 ? o_ks(H) : o_km(H); c_src = d.stats[sl - 8]; c_bytes = k_stats / 2; }
        }
      }
      const int stB = ring_next(st, NS);
      if (!mbar_wait(empty_u + st * 8, (pph >> st) & 1, P.wait_ns)) return false;
      if (!mbar_wait(empty_u + stB * 8, (pph >> stB) & 1, P.wait_ns)) return false;
      pph ^= (1u << st) | (1u << stB);
      const int my = half ? stB : st;
      const uint32_t bar = full_u + my * 8, st_u = ring_u + (uint32_t)my * SB;
      if (sl == 0) {
        int4* hd = reinterpret_cast<int4*>(ring + (size_t)my * SB + o_hdr(H));
        hd[0] = make_int4(h0.x, h0.y, (h0.z & F_MASK) | fx, h0.w);
        hd[1] = h1;
        mbar_expect_tx(bar, tx);
      }
      __syncwarp();
      if (c_bytes) bulk_copy(st_u + c_dst, c_src, c_bytes, bar, policy);
      fills += 2;
      st = ring_next(stB, NS);
      return true;
    };
    bool more = P.idle_producer ? false : advance();
    BlockMeta nxt = more ? load_meta(P, bt_row, lane < U ? base + lane : b_end, b_end) : BlockMeta{};
    pdl_wait();  // pages and the work counter are final from here on
    while (more && ok) {
      const BlockMeta cur = nxt;
      const int u_base = base, u_end = b_end, u_seq = seq, u_split = split;
      const bool u_first = base == b_start, u_last = base + U >= b_end;
      const int64_t u_len = seq_len;
      more = advance();
      if (more) nxt = load_meta(P, bt_row, lane < U ? base + lane : b_end, b_end);
      const int nb = min(U, u_end - u_base);
      // tokens of the unit: all blocks are full except possibly the item's last one
      const int unit_tok = (int)min((int64_t)nb * L.BS, u_len - (int64_t)u_base * L.BS);
      const int unit_tiles = (unit_tok + TILE - 1) / TILE;
      uint32_t pair_ok;  // bit l: tile l is full, code-based and INT4 or INT2 (it can be half of a pair)
      {  // plan: lane l takes tile l of the unit (its block's metadata sits in lane kb)
        const int kb = tpb == 1 ? lane : lane / tpb, tb = lane - kb * tpb;
        const int src = kb < 32 ? kb : 31;
        const int kblk = __shfl_sync(0xffffffffu, cur.blk, src);
        int bits = __shfl_sync(0xffffffffu, cur.bits, src);
        const int c1 = __shfl_sync(0xffffffffu, cur.c1, src), c2 = __shfl_sync(0xffffffffu, cur.c2, src),
                  c3 = __shfl_sync(0xffffffffu, cur.c3, src);
        const long long ks_slot = __shfl_sync(0xffffffffu, cur.rslot, src);
        const int kgrp = __shfl_sync(0xffffffffu, cur.rgrp, src);
        bool can_pair = false;
        if (lane < unit_tiles) {
          if (bits != 2 && bits != 4 && bits != 8) bits = 2;  // never opened: stay inside the page
          const int row_bytes = 32 * H * bits;
          const int tpc = (2 * L.BS) / bits;
          const int t0 = tb * TILE;
          const int blk_tok = min(L.BS, unit_tok - kb * L.BS);
          const int grp = t0 / L.KG;
          const bool in_res = ks_slot >= 0 && grp == kgrp;
          const unsigned char* page = P.pages + (int64_t)kblk * L.PS;
          TilePlan& d = plan[lane];
          const int rt = min(tpc, TILE);                    // token rows per run: the tile's part of one chunk
          for (int rr = 0; rr < TILE / rt; ++rr) {
            const int tok = t0 + rr * rt, jc = tok / tpc;     // chunk of the run's first token
            int64_t pg = kblk, cs = 0;
            if (jc > 0) { const int id = jc == 1 ? c1 : (jc == 2 ? c2 : c3); pg = id / L.KC; cs = id - pg * L.KC; }
            d.run[rr] = P.pages + pg * L.PS + L.o_data + cs * L.CB + (int64_t)(tok - jc * tpc) * row_bytes;
          }
          const int nv = min(TILE, blk_tok - t0);
          d.hdr.bits = bits; d.hdr.n_valid = nv;
          const int rt_log = (rt & (rt - 1)) == 0 ? 31 - __clz(rt) : 15;  // for the fills: a run's rows by shift and mask
          d.hdr.flags = (in_res ? F_RES : 0) | (u_first && lane == 0 ? F_FIRST : 0) |
                        (u_last && lane == unit_tiles - 1 ? F_LAST : 0) | (rt_log << RT_LOG_SHIFT);
          d.hdr.pos0 = t0 - grp * L.KG; d.hdr.res_slot = ks_slot; d.hdr.seq = u_seq; d.hdr.split = u_split;
          d.stats[0] = page + L.o_vs + (int64_t)t0 * H * NG * 2;
          d.stats[1] = page + L.o_vm + (int64_t)t0 * H * NG * 2;
          d.stats[2] = page + L.o_ks + (int64_t)grp * H * D * 2;
          d.stats[3] = page + L.o_km + (int64_t)grp * H * D * 2;
          can_pair = nv == TILE && !in_res && bits != 8;
        }
        pair_ok = __ballot_sync(0xffffffffu, can_pair);
        __syncwarp();
      }
      for (int ti = 0; ti < unit_tiles && ok; ++ti) {
        const TilePlan& d = plan[ti];
        const int bits = d.hdr.bits;
        if (bits == 8) {  // two stages: K side with the K stats, then V side with the V stats
          ok = fill2(d, 0, 2, d, 0, 3);
        } else if (ti + 1 < unit_tiles && ((pair_ok >> ti) & 3) == 3 && plan[ti + 1].hdr.bits == bits) {
          ok = fill2(d, F_PAIR | (plan[ti + 1].hdr.flags & F_LAST), 1, plan[ti + 1], 0, 1);
          ++ti;
        } else {
          ok = fill(d, 0, 1);
        }
      }
      __syncwarp();  // every lane is done reading the plans before the next unit overwrites them
      ok = !__any_sync(0xffffffffu, !ok);
    }
    if (ok && !P.idle_producer) {  // no more work: tell the consumers
      if (mbar_wait(empty_u + st * 8, (pph >> st) & 1, P.wait_ns)) {
        if (lane == 0) {
          reinterpret_cast<int4*>(ring + (size_t)st * SB + o_hdr(H))[0] = make_int4(2, -1, 0, 0);
          mbar_arrive(full_u + st * 8);
        }
      } else {
        ok = false;
      }
    }
    if (!ok) {
      // A wait gave up: copies already started may still be landing; give each stage its (bounded)
      // time before the CTA's shared memory goes away.
      for (int s = 0; s < NS; ++s) {
        const uint32_t uses = fills > (uint32_t)s ? (fills - s + NS - 1) / NS : 0;
        if (uses > 0) mbar_wait(full_u + s * 8, (uses - 1) & 1, P.wait_ns);
      }
    }
  } else {
    // ===================== consumers: warp h owns KV head h =====================
    Lane ln;
    ln.h = warp; ln.lane = lane; ln.r = lane >> 2; ln.j = lane & 3;
    unsigned char* qn = qs + ln.h * A.gqa * QN_ROW;
    {  // query columns >= gqa of the MMAs read the team's zero row (every warp writes the same zeros)
      unsigned char* zero = qs + H * A.gqa * QN_ROW;
      ln.qn_lane = smem_u32(ln.r < A.gqa ? qn + ln.r * QN_ROW : zero);
      ln.qn_ld = smem_u32(((lane & 7) < A.gqa ? qn + (lane & 7) * QN_ROW : zero) + (lane >> 3) * 16);
      for (int i = lane; i < D / 2; i += 32) *reinterpret_cast<uint32_t*>(zero + i * 4) = 0u;
      __syncwarp();
    }
    ln.vs_row = o_vs(H) + (uint32_t)(2 * ln.r * H + ln.h) * NG * 2;  // token 2r; token 2r + 1 (MMA row r + 8) is one token further
    // [v_min | ones] operand, read transposed: matrices 0 / 2 = v_min of the even / odd tokens (k order: tokens 0,2,..,14
    // then 1,3,..,15), 16-byte rows = the four groups of this pair of heads; matrices 1 / 3 = the row of ones
    ln.vm_ld = (lane & 8) ? (uint32_t)o_ones(H)
                          : (uint32_t)o_vm(H) + (uint32_t)((2 * (lane & 7) + (lane >> 4)) * H + (ln.h & ~1)) * NG * 2;
    // broadcast k_min operand: matrices 0 / 1 = channels [0, 8) of the k-step for the first / second tile, 2 / 3 = channels [8, 16)
    ln.km_ld = (uint32_t)o_km(H) + ln.h * (D * 2) + (lane >> 4) * 16u;
    ln.vs_row8 = o_vs(H) + (uint32_t)(ln.r * H + ln.h) * NG * 2;
    ln.vm_ld8 = (lane & 8) ? (uint32_t)o_ones(H) : (uint32_t)o_vm(H) + (uint32_t)((lane & 7) * H + (ln.h & ~1)) * NG * 2;
    int c_st = 0;                  // stage being consumed
    uint32_t cph = 0;              // per stage: parity of the `full` phase to wait for
    WarpState w;
    w.bits = 0;
    w.m0 = w.m1 = -INFINITY;
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) { w.acc[mt][0] = w.acc[mt][1] = w.acc[mt][2] = w.acc[mt][3] = 0.f; }
    w.bl[0] = w.bl[1] = w.bl[2] = w.bl[3] = 0.f;
    int seq = 0;
    // The header of the group at the head of the ring.
    int bits = 0, n_valid = -1, flags = 0, pos0 = 0, split = 0;
    long long res_slot = -1;
    // Wait for the stage at the head of the ring and read its header; false when a wait ran out.
    auto fetch = [&]() -> bool {
      if (!mbar_wait(full_u + c_st * 8, (cph >> c_st) & 1, P.wait_ns)) return false;  // header written, copies landed
      uint32_t hd[4], ex[4];
      const uint32_t ha = ring_u + (uint32_t)c_st * SB + o_hdr(H);
      lds128<0>(hd, ha);
      lds128<16>(ex, ha);
      bits = (int)hd[0]; n_valid = (int)hd[1]; flags = (int)hd[2]; pos0 = (int)hd[3];
      res_slot = (long long)(((unsigned long long)ex[1] << 32) | ex[0]);
      if (flags & F_FIRST) seq = (int)ex[2];
      split = (int)ex[3];
      return true;
    };
    // This head's queries of sequence `seq` -> fp16 in shared memory, pre-multiplied by softmax_scale * log2(e)
    // (rows >= gqa are zero).  All global loads are issued before the first use so the item pays one memory latency.
    auto load_queries = [&]() {
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
                                                     (int64_t)(ln.h * A.gqa + n) * A.q_s1 + c8);
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
          if (n < A.gqa) *reinterpret_cast<uint4*>(qn + n * QN_ROW + c8 * 2) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      } else {
        for (int i = lane; i < A.gqa * (D / 2); i += 32) {
          const int d2 = i % (D / 2), n = i / (D / 2);
          const int64_t e = q_row * A.q_s0 + (int64_t)(ln.h * A.gqa + n) * A.q_s1 + 2 * d2;
          const float x = ld_dt(A.q, A.q_dt, e) * A.scale_log2e, y = ld_dt(A.q, A.q_dt, e + 1) * A.scale_log2e;
          *reinterpret_cast<uint32_t*>(qn + n * QN_ROW + d2 * 4) = pack_h2(x, y);
        }
      }
      __syncwarp();
    };
    // The team's first work item is its own index (see the producer): its queries are loaded while the producer
    // resolves the item's blocks and the first copies are in flight.
    int preloaded = -1;
    {
      const int item0 = blockIdx.x * V + team;
      if (item0 < n_items) {
        seq = item0 % P.num_seqs;
        load_queries();
        preloaded = seq;
      }
    }
    // A work item starts: its queries (unless they are the ones loaded ahead) and a fresh state.
    auto begin_item = [&]() {
      if (seq != preloaded) load_queries();
      preloaded = -1;
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) { w.acc[mt][0] = w.acc[mt][1] = w.acc[mt][2] = w.acc[mt][3] = 0.f; }
      w.bl[0] = w.bl[1] = w.bl[2] = w.bl[3] = 0.f;
      w.m0 = w.m1 = -INFINITY;
      w.bits = 0;
    };
    // Kinds of groups; each kind is worked off in a loop of its own for as long as groups of that kind follow one
    // another (one tier per layer is the common case), so that the loop body holds a single code path.
    constexpr int K_END = 0, K_PAIR4 = 1, K_PAIR2 = 2, K_TILE8 = 3, K_SINGLE = 4;
    auto kind_of = [&]() -> int {
      if (n_valid < 0) return K_END;
      if (bits == 8) return K_TILE8;
      if (flags & F_PAIR) return bits == 4 ? K_PAIR4 : K_PAIR2;
      return K_SINGLE;
    };
    // Releases the group's stages, writes the split's partial result after its last group, moves to the next header.
    auto run = [&](auto kind_c, auto bits_c) {
      constexpr int KIND = decltype(kind_c)::value, BITS = decltype(bits_c)::value;
      constexpr bool TWO = KIND != K_SINGLE;
      do {
        PROF_T(r0);
        if (flags & F_FIRST) begin_item();
        const uint32_t sb0 = ring_u + (uint32_t)c_st * SB;
        const int st1 = ring_next(c_st, NS);
        const uint32_t sb1 = ring_u + (uint32_t)st1 * SB;
        if (TWO && !mbar_wait(full_u + st1 * 8, (cph >> st1) & 1, P.wait_ns)) { ok = false; break; }
        PROF_T(r1);
        PROF_PHASE(4, r0, r1);  // item start + wait for the second stage
        const bool last = (flags & F_LAST) != 0;
        const int cur_split = split;
        if constexpr (KIND == K_TILE8) {
          const uint32_t sk[1] = {sb0}, sv[1] = {sb1};
          process_group<8, H, 1>(P, ln, sk, sv, n_valid, (flags & F_RES) != 0, res_slot, pos0, w, remap, lock, ok);
        } else if constexpr (KIND == K_SINGLE) {
          const uint32_t s1[1] = {sb0};
          if (bits == 4) process_group<4, H, 1>(P, ln, s1, s1, n_valid, (flags & F_RES) != 0, res_slot, pos0, w, remap, lock, ok);
          else process_group<2, H, 1>(P, ln, s1, s1, n_valid, (flags & F_RES) != 0, res_slot, pos0, w, remap, lock, ok);
        } else {
          const uint32_t s2[2] = {sb0, sb1};
          process_group<BITS, H, 2>(P, ln, s2, s2, TILE, false, 0, 0, w, remap, lock, ok);
        }
        __syncwarp();
        mbar_arrive(empty_u + c_st * 8);  // every lane arrives (the barrier counts threads): no branch, no warp sync needed
        cph ^= 1u << c_st;
        c_st = st1;
        if (TWO) {
          mbar_arrive(empty_u + c_st * 8);
          cph ^= 1u << c_st;
          c_st = ring_next(c_st, NS);
        }
        if (last) {
          if constexpr (KIND == K_SINGLE) {
            if (w.bits == 4) write_partial<4, H>(P, w, seq, cur_split, ln.h, lane);
            else write_partial<2, H>(P, w, seq, cur_split, ln.h, lane);
          } else {
            write_partial<BITS, H>(P, w, seq, cur_split, ln.h, lane);
          }
        }
        PROF_T(r2);
        if (!fetch()) { ok = false; break; }
        PROF_T(r3);
        PROF_PHASE(5, r2, r3);  // wait for the next group's first stage
        PROF_PHASE(6, r1, r2);  // the group's math, release, partial result
      } while (kind_of() == KIND);
    };
    if (!fetch()) ok = false;
    while (ok) {
      const int kind = kind_of();
      if (kind == K_END) break;  // no more work for this CTA
      if (kind == K_PAIR4) run(std::integral_constant<int, K_PAIR4>{}, std::integral_constant<int, 4>{});
      else if (kind == K_PAIR2) run(std::integral_constant<int, K_PAIR2>{}, std::integral_constant<int, 2>{});
      else if (kind == K_TILE8) run(std::integral_constant<int, K_TILE8>{}, std::integral_constant<int, 8>{});
      else run(std::integral_constant<int, K_SINGLE>{}, std::integral_constant<int, 0>{});
    }
  }
  if (!ok && lane == 0 && P.status) atomicExch(P.status, 1);
#ifdef ECHOKV_PROFILE
  if (tid == 0 && blockIdx.x * V + team < 1024) {
    const int slot = blockIdx.x * V + team;
    unsigned int smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    g_cta[slot * 4 + 0] = cta_t0; g_cta[slot * 4 + 1] = global_ns();
    g_cta[slot * 4 + 2] = smid; g_cta[slot * 4 + 3] = (unsigned long long)(clock64() - cta_c0);
  }
#endif
}

}  // namespace mma

static int g_decode_path = 0;  // 0: pick by shape, 1: always the generic kernel
static unsigned long long g_wait_ns = mma::WAIT_NS;  // see echokv_set_decode_wait_limit
static int g_idle_producer = 0;
static cudaEvent_t g_ev_before = nullptr, g_ev_after = nullptr;  // optional timing hook around the split kernel

// Raised by decode_mma_kernel: 1 = a bounded wait ran out.
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

// What the launcher needs to know about a device, looked up once per device (with that device current).
struct DecodeDevice {
  bool ready = false;
  int max_smem = 0, num_sms = 0;
  int* status_word = nullptr;
};
template <int H>
static cudaError_t allow_smem(int bytes) {
  using namespace mma;
  cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<H, Teams<H>::V>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(decode_mma_kernel<H, Teams<H>::V_SMALL>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  return e;
}
template <int H>
static void launch_teams(bool small, unsigned grid, int smem_bytes, cudaStream_t st, const mma::Params& P) {
  using namespace mma;
  if (small) launch_pdl(decode_mma_kernel<H, Teams<H>::V_SMALL>, dim3(grid), dim3((H + 1) * 32 * Teams<H>::V_SMALL), smem_bytes, st, P);
  else launch_pdl(decode_mma_kernel<H, Teams<H>::V>, dim3(grid), dim3((H + 1) * 32 * Teams<H>::V), smem_bytes, st, P);
}
static int decode_device(DecodeDevice** out) {
  using namespace mma;
  constexpr int MAX_DEVICES = 64;
  static DecodeDevice table[MAX_DEVICES];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return set_error(ECHOKV_E_CUDA, "decode: cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
  DecodeDevice& d = table[dev];
  if (!d.ready) {
    e = cudaDeviceGetAttribute(&d.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = allow_smem<1>(d.max_smem);
    if (e == cudaSuccess) e = allow_smem<2>(d.max_smem);
    if (e == cudaSuccess) e = allow_smem<4>(d.max_smem);
    if (e == cudaSuccess) e = allow_smem<8>(d.max_smem);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status_word), g_decode_status);
    if (e != cudaSuccess) return set_error(ECHOKV_E_CUDA, "decode: device %d set-up: %s", dev, cudaGetErrorString(e));
    d.ready = true;
  }
  *out = &d;
  return ECHOKV_OK;
}

// Teams per CTA and ring stages per team for H KV heads with gqa query heads each: every team gets an equal slice
// of the SM's shared memory; false when not even the smaller team count leaves room for four stages (a group of
// two stages in work and one in flight at the least).
struct TeamShape { int V, ns, fixed; bool small; };
static bool team_shape(const DecodeDevice& dv, int H, int gqa, TeamShape* out) {
  using namespace mma;
  const int fixed = HDR_BYTES + UNIT * (int)sizeof(TilePlan) + (q_copy_bytes(H, gqa) + 127) / 128 * 128;
  const int sbytes = stage_bytes(H);
  const int room = dv.max_smem - CTA_SHARED_BYTES;
  int V = H == 8 ? Teams<8>::V : H == 4 ? Teams<4>::V : H == 2 ? Teams<2>::V : Teams<1>::V;
  bool small = false;
  int ns = ((room / V) / 128 * 128 - fixed) / sbytes;
  if (ns < 4) {
    small = true;
    V = H == 8 ? Teams<8>::V_SMALL : H == 4 ? Teams<4>::V_SMALL : H == 2 ? Teams<2>::V_SMALL : Teams<1>::V_SMALL;
    ns = ((room / V) / 128 * 128 - fixed) / sbytes;
  }
  if (ns > MAX_NS) ns = MAX_NS;
  if (ns < 4) return false;
  out->V = V; out->ns = ns; out->fixed = fixed; out->small = small;
  return true;
}

static bool mma_shape_ok(int H, int D_, int VG, int KG, int BS, int gqa) {
  using namespace mma;
  return D_ == D && VG == 32 && KG % TILE == 0 && BS % TILE == 0 && gqa <= 8 && (H == 1 || H == 2 || H == 4 || H == 8);
}

// Teams of the tensor-core kernel on the current device for this shape (0: the generic kernel takes it, or no device).
int decode_mma_teams(int H, int D_, int VG, int KG, int BS, int gqa) {
  if (g_decode_path == 1 || !mma_shape_ok(H, D_, VG, KG, BS, gqa)) return 0;
  DecodeDevice* dv = nullptr;
  if (decode_device(&dv)) return 0;
  TeamShape ts;
  if (!team_shape(*dv, H, gqa, &ts)) return 0;
  return dv->num_sms * ts.V;
}

// Chooses the tensor-core kernel when the shape fits; otherwise leaves `handled` false.
int launch_decode_mma(const LayoutDev& L, const ResidualDev& R, const uint8_t* pages, const DecodeArgs& A,
                      int64_t num_seqs, int* counter, bool zero_counter, int* status, cudaStream_t st, bool* handled) {
  using namespace mma;
  *handled = false;
  if (g_decode_path == 1) return ECHOKV_OK;
  const int H = L.H;
  if (!mma_shape_ok(H, L.D, L.VG, L.KG, L.BS, A.gqa)) return ECHOKV_OK;
  if ((R.s_slot | R.s_pos | R.s_head) & 3) return ECHOKV_OK;                 // 8-byte residual loads
  if ((reinterpret_cast<uintptr_t>(R.base) & 15) != 0) return ECHOKV_OK;
  if (num_seqs * (int64_t)A.num_splits > (1 << 30)) return ECHOKV_OK;
  DecodeDevice* dv = nullptr;
  int rc = decode_device(&dv);
  if (rc) return rc;
  Params P;
  P.L = L; P.R = R; P.pages = pages; P.A = A; P.num_seqs = (int)num_seqs;
  P.counter = counter;
  P.q_vec16 = (A.q_dt != ECHOKV_DT_F32) && (reinterpret_cast<uintptr_t>(A.q) % 16 == 0) && A.q_s0 % 8 == 0 && A.q_s1 % 8 == 0;
  P.status = status ? status : dv->status_word;
  P.wait_ns = g_wait_ns;
  P.idle_producer = g_idle_producer;
  TeamShape ts;
  if (!team_shape(*dv, H, A.gqa, &ts)) return ECHOKV_OK;
  const int V = ts.V, ns = ts.ns, fixed = ts.fixed, sbytes = stage_bytes(H);
  const bool small = ts.small;
  P.NS = ns;
  P.team_bytes = (fixed + ns * sbytes + 127) / 128 * 128;
  const int smem_bytes = CTA_SHARED_BYTES + P.team_bytes * V;
  const int64_t n_items = num_seqs * (int64_t)A.num_splits;
  int64_t grid = dv->num_sms;
  if (grid * V > n_items) grid = (n_items + V - 1) / V;
  // The merge kernel leaves the counter at zero for the next call; a caller that cannot promise a zeroed state
  // gets it zeroed here.
  if (zero_counter && cudaMemsetAsync(counter, 0, sizeof(int), st) != cudaSuccess) return check_launch("decode (work counter)");
  if (g_ev_before) cudaEventRecord(g_ev_before, st);
  switch (H) {
    case 1: launch_teams<1>(small, (unsigned)grid, smem_bytes, st, P); break;
    case 2: launch_teams<2>(small, (unsigned)grid, smem_bytes, st, P); break;
    case 4: launch_teams<4>(small, (unsigned)grid, smem_bytes, st, P); break;
    default: launch_teams<8>(small, (unsigned)grid, smem_bytes, st, P); break;
  }
  if (g_ev_after) cudaEventRecord(g_ev_after, st);
  rc = check_launch("decode (tensor-core kernel)");
  if (rc) return rc;
  *handled = true;
  return ECHOKV_OK;
}

}  // namespace echokv

#ifdef ECHOKV_PROFILE
extern "C" int echokv_debug_cta(unsigned long long* dst, int n) {
  return (int)cudaMemcpyFromSymbol(dst, echokv::mma::g_cta, sizeof(unsigned long long) * n);
}
extern "C" int echokv_debug_phase(unsigned long long* dst, int reset) {
  int rc = (int)cudaMemcpyFromSymbol(dst, echokv::mma::g_phase, sizeof(unsigned long long) * 16);
  if (reset) { unsigned long long z[16] = {}; cudaMemcpyToSymbol(echokv::mma::g_phase, z, sizeof(z)); }
  return rc;
}
#endif

extern "C" int echokv_set_decode_events(void* before, void* after) {
  echokv::g_ev_before = reinterpret_cast<cudaEvent_t>(before);
  echokv::g_ev_after = reinterpret_cast<cudaEvent_t>(after);
  return ECHOKV_OK;
}

extern "C" int echokv_set_decode_wait_limit(int64_t limit_ns, int idle_producer) {
  echokv::g_wait_ns = limit_ns > 0 ? (unsigned long long)limit_ns : echokv::mma::WAIT_NS;
  echokv::g_idle_producer = idle_producer != 0;
  return ECHOKV_OK;
}

extern "C" int echokv_set_decode_path(int path) {
  const int old = echokv::g_decode_path;
  echokv::g_decode_path = path;
  return old;
}
