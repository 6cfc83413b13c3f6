// Flash-attention forward for sm_100a on the 5th-generation tensor cores:
//   S = Q K^T and O += P V are tcgen05.mma instructions with accumulators in TMEM,
//   Q / K / V tiles arrive by TMA (128-byte swizzle) through an mbarrier ring,
//   the softmax runs thread-per-row on scores read once from TMEM into registers, and P goes
//   back to TMEM as 16-bit pairs to be the A operand of the second product (its own columns
//   with D = 64, over the score columns with D = 128).
// Same math and BlockMask walk as fa_fwd.cuh (see there for the reference citations); this
// kernel covers fp16 / bf16, D = Dv in {64, 128}, block sizes that are multiples of 128 and a
// positive scale.
//
// One CTA owns two 128-row query tiles of one (batch, head) and streams 128-row K/V tiles
// past both.  Warp roles (12 warps = 3 warpgroups):
//   warps 0-3  softmax warpgroup of query tile 0      warps 4-7  of query tile 1
//   warp 8     TMA producer (one lane)
//   warps 9-10 MMA issuers (one lane each); warp 9 also allocates / frees TMEM.  With D = 64 warp 9
//              issues the S products and warp 10 the PV products; with D = 128 warp 9 issues both
//              products of query tile 0 and warp 10 those of tile 1; warp 11 is idle
// Registers are moved from the third warpgroup to the two softmax warpgroups (setmaxnreg),
// which hold a whole 128-column score row per thread.
// The S columns of a tile are released as soon as its scores are in registers, so with D = 64
// S of step j+1 is computed while the softmax of step j runs; with D = 128 (P over the S
// columns) the products of a tile form the chain  PV(j), S(j+1), PV(j+1) ...
// The running maximum is only raised when it grew by more than 2^8 (the stale maximum is
// exact as long as it is used consistently), so rescaling O in TMEM is rare.
//
// Every mbarrier wait is bounded; on expiry the CTA raises FA_STATUS_WAIT_TIMEOUT in the
// status word, all roles leave their loops, TMEM is freed and the kernel returns.
//
// Compile-time parameters (macros): FA_DTYPE (0 fp16, 1 bf16), FA_D (64 or 128), FA_TC_DECODE
// (split-KV variant, see below).
#pragma once
#include "fa_sm100.cuh"

struct FaTcParams {
  FaParams p;
  FaTensorMap tq, tk, tv;  // 4-d maps (D, S, H, B), box 64 x 128 x 1 x 1, 128-byte swizzle
  FaTensorMap to;          // the output, like tq (unused by the decode variant, which writes partial results)
};

namespace fa_tc {

constexpr int DT = FA_DTYPE;
constexpr int D = FA_D;
constexpr int BM = 128, BN = 128;
constexpr int ATOMS = D / 64;            // 64-element (128-byte) column groups per row
constexpr int ATOM_BYTES = 128 * 128;    // 128 rows x 128 bytes
// Split-KV decode variant (FA_TC_DECODE, D = 64, at most 64 query rows): the CTA owns a contiguous
// share of the kv tiles the BlockMask lists and the two softmax warpgroups take alternate kv tiles
// of that share.  A warpgroup's 128-row tile holds the query rows twice, in rows 0-63 and again in
// rows 64-127, so that two threads work on one query row: the thread of TMEM lane r < 64 takes kv
// columns 0-63 of the tile, the thread of lane r + 64 columns 64-127.  Each thread runs its own
// online softmax over its half tiles (own running maximum and sum) and writes P for its columns
// only; the other 64 columns of its lane are zero, so the P.V product gives every lane the
// partial output of its own columns.  No thread sits on a padding row while there are at least
// 33 queries, and a thread's serial work per kv tile is half that of the forward.  At the end the
// four partial results of a row (running maximum, sum, O of two warpgroups x two halves) are
// merged through shared memory and the CTA writes one un-normalised partial result per row for
// the combine kernel.  More stages, since the kv stream is all there is.
#ifndef FA_TC_DECODE
#define FA_TC_DECODE 0
#endif
constexpr bool DECODE = FA_TC_DECODE != 0;
constexpr int NSTAGE = DECODE ? 5 : (D == 64 ? 3 : 2);
constexpr int Q_BYTES = 2 * ATOMS * ATOM_BYTES;
constexpr int KV_STAGE = ATOMS * ATOM_BYTES;
constexpr int MAXT = 256;                // kv tiles per row of the block grid (Skv <= 32768)
constexpr int NBARS = 1 + 4 * NSTAGE + 8;
constexpr int OFF_K = Q_BYTES;
constexpr int OFF_V = OFF_K + NSTAGE * KV_STAGE;
constexpr int OFF_BAR = OFF_V + NSTAGE * KV_STAGE;
constexpr int OFF_MISC = OFF_BAR + NBARS * 8;       // tmem base, abort flag, nsteps, pad
constexpr int OFF_SCHED = OFF_MISC + 16;            // short tile[MAXT]
constexpr int OFF_MODE = OFF_SCHED + MAXT * 2;      // uchar mode[MAXT][2]
constexpr int OFF_CLS = OFF_MODE + MAXT * 2;        // uchar cls[2][MAXT]
constexpr int OFF_WCNT = OFF_CLS + 2 * MAXT;        // int wcount[MAXT / 32]: listed tiles per warp of the schedule build
constexpr int SMEM_BYTES = OFF_WCNT + (MAXT / 32) * 4 + 1024;  // + slack for the 1024-byte alignment
constexpr int TMEM_COLS = 512;
constexpr int COL_S = 0, COL_O = 256;
// With D = 64 there is TMEM left for P next to S (columns 384..511): S of the next kv step can
// then be produced while the softmax of the current step is still writing P.  With D = 128 the
// 512 columns are taken by S and O, and P overwrites the S columns it was computed from.
constexpr bool SEP_P = D == 64;
constexpr int COL_P = 384;
// One pair of exponentials in FA_TC_POLY_EVERY goes to the FMA pipe (a cubic, see fa_ex2_poly2).
// Measured (B8 H8 S2048 D64): every fourth pair takes the forward without a score_mod from 0.118 to
// 0.114 ms, with the checkerboard mod from 0.133 to 0.129 and causal + ALiBi from 0.088 to 0.085;
// every eighth is about the same, every third and every second are slower again (the issue slots).
#ifndef FA_TC_POLY_EVERY
#define FA_TC_POLY_EVERY 4
#endif
constexpr int NT = 384;
// Register split (setmaxnreg): the kernel starts with 168 registers per thread (65536 / 384, rounded
// down to a multiple of 8).  The third warpgroup gives up 72 each (128 x 72 = 9216) and the two
// softmax warpgroups take 32 each (256 x 32 = 8192).  The increase must not ask for more than the
// decrease releases: setmaxnreg.inc blocks until the registers are there, without a time limit.
constexpr int REGS_SOFTMAX = 200, REGS_OTHER = 96;
static_assert(256 * (REGS_SOFTMAX - 168) <= 128 * (168 - REGS_OTHER), "setmaxnreg.inc would wait forever");
constexpr int WARP_PRODUCER = 8, WARP_MMA = 9, WARP_MMA_B = 10;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

static_assert(D == 64 || D == 128, "head dim 64 or 128");
static_assert(!DECODE || D == 64, "the decode variant is written for head dim 64");
static_assert(DT == FA_DT_F16 || DT == FA_DT_BF16, "16-bit inputs");

__device__ __forceinline__ fa_u32 bar_addr(fa_u32 sbase, int i) { return sbase + OFF_BAR + i * 8; }
constexpr int BAR_Q = 0;
constexpr int BAR_KFULL = 1, BAR_KEMPTY = 1 + NSTAGE, BAR_VFULL = 1 + 2 * NSTAGE, BAR_VEMPTY = 1 + 3 * NSTAGE;
constexpr int BAR_S = 1 + 4 * NSTAGE, BAR_P = BAR_S + 2, BAR_O = BAR_S + 4;
// With separate P columns the S columns of a tile are released as soon as the softmax warps
// hold the scores in registers, and S of the next step is produced during the softmax.
constexpr int BAR_SFREE2 = BAR_S + 6;

// Work on one 32-column chunk of a score row held in registers (columns C0 .. C0+31 of the kv
// tile that starts at key n0).  C0 is a template parameter and n0 a multiple of 128, so the low
// bits of every key index are compile-time constants inside the mods.
struct RowMax {
  float a, b, c, d;
};
__device__ __forceinline__ void max_chunk(const float (&v)[32], RowMax& mx) {
#pragma unroll
  for (int e = 0; e < 32; e += 8) {
    mx.a = fa_max3(mx.a, v[e], v[e + 1]);
    mx.b = fa_max3(mx.b, v[e + 2], v[e + 3]);
    mx.c = fa_max3(mx.c, v[e + 4], v[e + 5]);
    mx.d = fa_max3(mx.d, v[e + 6], v[e + 7]);
  }
}
// score_mod (and the rounding of the raw scores to the input type, when asked for) in place;
// the results are in log2 units.  An affine score_mod (A * score + B) costs one FMA: A and B
// absorb the scale and log2(e).
template <int C0>
__device__ __forceinline__ void mod_chunk(float (&v)[32], int n0, int qi, int gb, int gh, float scale, float sc2) {
#if FA_HAS_SCORE_MOD && defined(FA_SCORE_AFFINE) && defined(FA_SCORE_LINEAR_KV)
  // The multiplier does not read kv and the bias is linear in it (relative-position biases such as
  // ALiBi): both are taken once, at the first column of the chunk, and column e adds e times the
  // slope - two packed FMAs per pair instead of an integer subtraction, an int-to-float conversion
  // (which shares the SFU with the exponentials) and a multiplication per element.
  {
    const int kv0 = n0 | C0;
    const float mulsc = fa_score_mul(0.f, gb, gh, qi, kv0) * sc2;
    const float base = fa_score_add2(0.f, gb, gh, qi, kv0);
    const float dkv = fa_score_add2_dkv(0.f, gb, gh, qi, kv0);
    const fa_u64 m2 = fa_f2(mulsc, mulsc), b2 = fa_f2(base, base), d2 = fa_f2(dkv, dkv);
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
      float x0 = v[e], x1 = v[e + 1];
#if FA_ROUND_SCORES
      fa_round2<DT>(x0, x1);
#endif
      fa_f2_unpack(fa_fma2(fa_f2(x0, x1), m2, fa_fma2(fa_f2((float)e, (float)(e + 1)), d2, b2)), x0, x1);
      v[e] = x0;
      v[e + 1] = x1;
    }
    return;
  }
#endif
#pragma unroll
  for (int e = 0; e < 32; e += 2) {
    float x0 = v[e], x1 = v[e + 1];
    const int kv0 = n0 | (C0 + e);
    const int kv1 = n0 | (C0 + e + 1);
#if FA_ROUND_SCORES
    fa_round2<DT>(x0, x1);
#endif
#if FA_HAS_SCORE_MOD && defined(FA_SCORE_AFFINE)
    x0 = fmaf(x0, fa_score_mul(0.f, gb, gh, qi, kv0) * sc2, fa_score_add2(0.f, gb, gh, qi, kv0));
    x1 = fmaf(x1, fa_score_mul(0.f, gb, gh, qi, kv1) * sc2, fa_score_add2(0.f, gb, gh, qi, kv1));
#elif FA_HAS_SCORE_MOD
    x0 = fa_score_mod(x0 * scale, gb, gh, qi, kv0) * FA_LOG2E;
    x1 = fa_score_mod(x1 * scale, gb, gh, qi, kv1) * FA_LOG2E;
#else
    x0 *= sc2;
    x1 *= sc2;
#endif
    v[e] = x0;
    v[e + 1] = x1;
  }
}
// mask_mod (on tiles the BlockMask lists as partial) and the end of the sequence (ragged last
// tile): masked scores become -inf.  Only the few tiles that need it come here, so the code is
// kept small rather than fast: a rolled loop evaluates the mask of this thread's columns into
// one word per 32 columns, and the words are applied to the registers.  (A second copy of the whole step with the
// mask evaluated in line, per element and fully unrolled, made a masked step take 12-15k clocks
// against 3.5k for a plain one: the step no longer fitted the instruction cache.)
template <int NW>
__device__ __forceinline__ void mask_bits(fa_u32 (&w)[NW], bool use_mask, int kv0, int qi, int gb, int gh, int Skv,
                                          const unsigned* rowbits) {
  // the end of the sequence alone needs no loop: word c covers keys kv0 + 32 c .. + 31
#pragma unroll
  for (int c = 0; c < NW; ++c) {
    const int left = Skv - (kv0 + 32 * c);
    w[c] = left >= 32 ? 0xffffffffu : (left <= 0 ? 0u : ((1u << left) - 1u));
  }
#if FA_HAS_MASK_MOD
  if (use_mask && rowbits != nullptr) {
    // mask_mod was evaluated once for all positions (FaTables::mask_bits): this row's words of the tile
    if (NW == 4) {
      const uint4 m = *(const uint4*)(rowbits + (kv0 >> 5));
      w[0] &= m.x; w[1] &= m.y; w[NW > 2 ? 2 : 0] &= m.z; w[NW > 2 ? 3 : 0] &= m.w;
    } else {
      const uint2 m = *(const uint2*)(rowbits + (kv0 >> 5));
      w[0] &= m.x; w[1] &= m.y;
    }
  } else if (use_mask) {
    // one rolled loop, the NW words side by side (independent evaluations in every iteration)
    fa_u32 m[NW];
#pragma unroll
    for (int c = 0; c < NW; ++c) m[c] = 0u;
#pragma unroll 2
    for (int e = 0; e < 32; ++e) {
#pragma unroll
      for (int c = 0; c < NW; ++c) m[c] |= (fa_mask_mod(gb, gh, qi, kv0 + 32 * c + e) ? 1u : 0u) << e;
    }
#pragma unroll
    for (int c = 0; c < NW; ++c) w[c] &= m[c];
  }
#endif
}
__device__ __forceinline__ void mask_apply(float (&v)[32], fa_u32 bits) {
#pragma unroll
  for (int e = 0; e < 32; ++e) v[e] = ((bits >> e) & 1u) ? v[e] : FA_NEG_INF;
}

// Pass-2 work on one chunk: p = 2^(x * cmul - m), packed to 16 bits, and the row-sum chains.
__device__ __forceinline__ void pass2_chunk(const float (&v)[32], fa_u32 (&pk)[16], fa_u64 cmul, fa_u64 negm,
                                            fa_u64& sum_a, fa_u64& sum_b) {
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    float a0, a1;
    fa_f2_unpack(fa_fma2(fa_f2(v[2 * e], v[2 * e + 1]), cmul, negm), a0, a1);
    // one pair in FA_TC_POLY_EVERY takes its exponentials on the FMA pipe: the SFU (16 per clock
    // and SM) is what bounds this loop
    float p0, p1;
    if (FA_TC_POLY_EVERY > 0 && (e % (FA_TC_POLY_EVERY > 0 ? FA_TC_POLY_EVERY : 1)) == (FA_TC_POLY_EVERY - 1)) {
      fa_ex2_poly2(a0, a1, p0, p1);
    } else {
      p0 = fa_ex2(a0);
      p1 = fa_ex2(a1);
    }
    pk[e] = fa_pack2<DT>(p0, p1);
    const fa_u64 pf = fa_f2(p0, p1);
    if (e & 1) sum_b = fa_add2(sum_b, pf);
    else sum_a = fa_add2(sum_a, pf);
  }
}

// State of one softmax warpgroup thread that a kv step reads and updates.
struct SoftmaxCtx {
  const FaParams& p;
  fa_u32 sb, t_s, t_o, t_p;
  int i, warp, qi, gb, gh;
  int half;  // decode variant: which 64 kv columns of a tile this thread owns (0 in the forward)
  float sc2;
  volatile int* abort_flag;
  const short* sched_tile;
  float m_ref, l;
  fa_u32 cnt;
  const unsigned* rowbits;  // this query row of the mask bit matrix, or null
};

// One kv step of this warpgroup's tile.  The few tiles that need mask_mod or end beyond the
// sequence take one extra block after the scores are in registers.  VARIANT 2: one copy of the
// step, the block behind a run-time flag (head dim 64, where a second copy of the step costs more
// in the instruction cache than the branch: causal forward 100 against 108 us).  VARIANT 0 / 1: a
// copy without and a copy with the block (head dim 128, where the run-time flag made the common,
// unmasked steps 16 % slower).
template <int VARIANT>
__device__ __forceinline__ bool softmax_step(SoftmaxCtx& c, const int j, const int mode, const bool masked_rt) {
  const bool masked = VARIANT == 2 ? masked_rt : VARIANT == 1;
  const FaParams& p = c.p;
  const fa_u32 sb = c.sb, t_s = c.t_s, t_o = c.t_o, t_p = c.t_p;
  const int i = c.i, qi = c.qi, gb = c.gb, gh = c.gh;
  const float sc2 = c.sc2;
  volatile int* abort_flag = c.abort_flag;
  float& m_ref = c.m_ref;
  float& l = c.l;
  fa_u32& cnt = c.cnt;
  const short* sched_tile = c.sched_tile;
  // first key of this thread's columns (decode variant: the thread's 64-column half of the tile)
  const int n0 = (int)sched_tile[DECODE ? 2 * j + i : j] * BN + (DECODE ? c.half * 64 : 0);
  const fa_u32 t_sh = DECODE ? t_s + c.half * 64 : t_s;
  if (!fa_mbar_wait_warp(bar_addr(sb, BAR_S + i), cnt & 1u, abort_flag)) return false;
  fa_tc_fence_after();
  // ---- pass 1: the whole score row (128 fp32 values) comes into registers, chunk by chunk,
  // with the score_mod (when there is one), the mask and the row maximum of a chunk computed
  // while the next chunk is on its way.  Without a score_mod the raw scores are kept and the
  // scale is folded into the exponent of pass 2.  The S columns are free again as soon as the
  // last load has landed, long before the softmax of the step is done.
  float s0[32], s1[32], s2[32], s3[32];
  RowMax rm = {FA_NEG_INF, FA_NEG_INF, FA_NEG_INF, FA_NEG_INF};
  // (the host routes a non-positive scale, which would turn the maximum around, elsewhere)
  constexpr bool in_place = FA_HAS_SCORE_MOD || FA_ROUND_SCORES;
  const bool use_mask = FA_HAS_MASK_MOD && mode == 1;
#define FA_P1(V, C0)                                                          \
  if (in_place) mod_chunk<C0>(V, n0, qi, gb, gh, p.scale, sc2);                \
  max_chunk(V, rm);
  fa_tmem_ld32(t_sh, s0);
  fa_tmem_wait_ld();
  fa_tmem_ld32(t_sh + 32, s1);
  FA_P1(s0, 0)
  fa_tmem_wait_ld();
  if (DECODE) {
    // two chunks are the whole share of this thread
    fa_tc_fence_before();
    fa_mbar_arrive(bar_addr(sb, BAR_SFREE2 + i));
    FA_P1(s1, 32)
  } else {
    fa_tmem_ld32(t_s + 64, s2);
    FA_P1(s1, 32)
    fa_tmem_wait_ld();
    fa_tmem_ld32(t_s + 96, s3);
    FA_P1(s2, 64)
    fa_tmem_wait_ld();
    if (SEP_P) {
      fa_tc_fence_before();
      fa_mbar_arrive(bar_addr(sb, BAR_SFREE2 + i));
    }
    FA_P1(s3, 96)
  }
#undef FA_P1
  if (masked) {
    // (the row maximum taken on the way is of the unmasked scores: it is taken again)
    fa_u32 keep[DECODE ? 2 : 4];
    mask_bits(keep, use_mask, n0, qi, gb, gh, p.Skv, c.rowbits);
    mask_apply(s0, keep[0]);
    mask_apply(s1, keep[1]);
    rm = {FA_NEG_INF, FA_NEG_INF, FA_NEG_INF, FA_NEG_INF};
    max_chunk(s0, rm);
    max_chunk(s1, rm);
    if (!DECODE) {
      mask_apply(s2, keep[DECODE ? 0 : 2]);
      mask_apply(s3, keep[DECODE ? 1 : 3]);
      max_chunk(s2, rm);
      max_chunk(s3, rm);
    }
  }
  float mx = fmaxf(fmaxf(rm.a, rm.b), fmaxf(rm.c, rm.d));
  if (!in_place) mx *= sc2;
  // running maximum, raised lazily
  const float m_new = fmaxf(m_ref, mx);
  bool need = false;
  float corr = 1.f;
  if (m_ref == FA_NEG_INF) {
    m_ref = m_new;  // nothing accumulated yet for this row
  } else if (m_new - m_ref > RESCALE_THRESHOLD) {
    need = true;
    corr = fa_ex2(m_ref - m_new);
    m_ref = m_new;
    l *= corr;
  }
  const bool rescale = cnt > 0 && __any_sync(0xffffffffu, need);
  if (cnt > 0 && (SEP_P || rescale)) {
    // the previous PV product of this tile must be complete: it reads the P columns that
    // are about to be overwritten (separate P columns), and O is rescaled in place
    if (!fa_mbar_wait_warp(bar_addr(sb, BAR_O + i), (cnt - 1) & 1u, abort_flag)) return false;
    fa_tc_fence_after();
  }
  if (rescale) {
#pragma unroll 1
    for (int c = 0; c < D / 16; ++c) {
      float o[16];
      fa_tmem_ld16(t_o + c * 16, o);
      fa_tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 16; ++e) o[e] *= corr;
      fa_tmem_st16f(t_o + c * 16, o);
    }
  }
  // ---- pass 2: p = 2^(x * cmul - m) and the row sum; P goes to TMEM as 16-bit pairs (its own
  // columns with D = 64, over the first 64 score columns otherwise).
  // (Packed 16-bit exponentials - ex2.approx.f16x2, one SFU operation per pair - were measured
  // slower: 143 against 131 us, the conversions around them cost more than the SFU time they save.)
  const float m_use = (m_ref == FA_NEG_INF) ? 0.f : m_ref;
  const fa_u64 negm = fa_f2(-m_use, -m_use);
  const float cm = in_place ? 1.f : sc2;
  const fa_u64 cmul = fa_f2(cm, cm);
  fa_u64 sum_a = fa_f2(0.f, 0.f), sum_b = fa_f2(0.f, 0.f);
  {
    fa_u32 pk[16];
    const fa_u32 t_ph = DECODE ? t_p + c.half * 32 : t_p;  // (the other 32 columns of the lane stay zero)
    pass2_chunk(s0, pk, cmul, negm, sum_a, sum_b);
    fa_tmem_st16(t_ph, pk);
    pass2_chunk(s1, pk, cmul, negm, sum_a, sum_b);
    fa_tmem_st16(t_ph + 16, pk);
    if (!DECODE) {
      pass2_chunk(s2, pk, cmul, negm, sum_a, sum_b);
      fa_tmem_st16(t_p + 32, pk);
      pass2_chunk(s3, pk, cmul, negm, sum_a, sum_b);
      fa_tmem_st16(t_p + 48, pk);
    }
  }
  float sum;
  {
    float a0, a1;
    fa_f2_unpack(fa_add2(sum_a, sum_b), a0, a1);
    sum = a0 + a1;
  }
  l += sum;
  fa_tmem_wait_st();
  fa_tc_fence_before();
  fa_mbar_arrive(bar_addr(sb, BAR_P + i));
  ++cnt;
  return true;
}

}  // namespace fa_tc

extern "C" __global__ void __launch_bounds__(fa_tc::NT, 1) fa_fwd_tc_kernel(const __grid_constant__ FaTcParams P) {
  using namespace fa_tc;
  const FaParams& p = P.p;
  extern __shared__ unsigned char smem_raw[];
  // a launch that does not fit the shared-memory map below (a host library built for another
  // version of this file) is refused before anything is written
  if (fa_dynamic_smem_size() < (fa_u32)SMEM_BYTES || blockDim.x != NT) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicOr(p.status, FA_STATUS_BAD_LAUNCH);
    return;
  }
  const fa_u32 raw = fa_smem_u32(smem_raw);
  const fa_u32 sb = (raw + 1023u) & ~1023u;  // shared-window address of the aligned base
  unsigned char* sm = smem_raw + (sb - raw);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#if FA_TC_DECODE
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;  // grid: (kv shares, heads, batch)
  const int m0 = 0;
#else
  const int pair = gridDim.z - 1 - blockIdx.z;  // grid: (heads, batch, tile pairs), the last pair first
  const int h = blockIdx.x, b = blockIdx.y;
  const int m0 = pair * 2 * BM;
#endif
  const int hk = h / (p.Hq / p.Hkv);
  const int gb = b + p.b_off, gh = h + p.h_off;

  volatile int* misc = (volatile int*)(sm + OFF_MISC);  // [0] tmem base, [1] abort, [2] nsteps
  short* sched_tile = (short*)(sm + OFF_SCHED);
  unsigned char* sched_mode = sm + OFF_MODE;
  unsigned char* cls = sm + OFF_CLS;

  // The BlockMask table reads of this CTA go out first: the two counts and, speculatively, this
  // thread's entry of the two index lists, for both query tiles.  They are all issued before any is
  // used (one round trip to memory instead of a chain of four dependent ones) and they are in flight
  // while the barriers are set up and TMEM is allocated.
  constexpr int NI = DECODE ? 1 : 2;
  const int ntiles = min((p.Skv + BN - 1) / BN, MAXT);
  const bool tables = p.t.kv_num != nullptr;
  const int tpb = tables ? (p.t.nKV == 1 ? ntiles : p.t.KVB / BN) : 1;
  const int bi0 = tid / tpb, ti0 = tid - bi0 * tpb;
  long long rows[NI];
  int num[NI][2], blk[NI][2];
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int mi = m0 + i * BM;
    const int bm = p.t.mB == 1 ? 0 : b, hm = p.t.mH == 1 ? 0 : h;
    const int qblk = tables ? min(mi / p.t.QB, p.t.nQ - 1) : 0;
    rows[i] = ((long long)bm * p.t.mH + hm) * p.t.nQ + qblk;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const int* nump = which ? p.t.full_kv_num : p.t.kv_num;
      const int* idxp = which ? p.t.full_kv_idx : p.t.kv_idx;
      const bool have = tables && nump != nullptr && mi < p.Sq;
      num[i][which] = have ? nump[rows[i]] : 0;
      blk[i][which] = (have && bi0 < p.t.nKV) ? idxp[rows[i] * p.t.nKV + bi0] : 0;
    }
  }

  // ---- set-up: barriers, TMEM, kv schedule ---------------------------------------------
  if (tid == 0) {
    fa_mbar_init(bar_addr(sb, BAR_Q), 1);
    for (int s = 0; s < NSTAGE; ++s) {
      fa_mbar_init(bar_addr(sb, BAR_KFULL + s), 1);
      // with D = 128 each of the two issuing warps releases a stage once
      fa_mbar_init(bar_addr(sb, BAR_KEMPTY + s), SEP_P ? 1 : 2);
      fa_mbar_init(bar_addr(sb, BAR_VFULL + s), 1);
      fa_mbar_init(bar_addr(sb, BAR_VEMPTY + s), SEP_P ? 1 : 2);
    }
    for (int i = 0; i < 2; ++i) {
      fa_mbar_init(bar_addr(sb, BAR_S + i), 1);
      fa_mbar_init(bar_addr(sb, BAR_P + i), 128);
      fa_mbar_init(bar_addr(sb, BAR_O + i), 1);
      fa_mbar_init(bar_addr(sb, BAR_SFREE2 + i), 128);
    }
    fa_mbar_init_fence();
    misc[1] = 0;
    misc[2] = 0;
    // the query tiles do not depend on the kv schedule: their loads start now and run while the
    // schedule is being built
    fa_tma_prefetch_desc(&P.tq);
    // (decode variant: the query map's box is 64 rows and each warpgroup's tile gets the queries
    //  twice, in rows 0-63 and in rows 64-127; rows beyond Sq are out of range and read as zero)
    fa_mbar_expect_tx(bar_addr(sb, BAR_Q), Q_BYTES);
    for (int i = 0; i < 2; ++i)
      for (int a = 0; a < ATOMS; ++a) {
        if (DECODE) {
          fa_tma_load_4d(sb + (i * ATOMS + a) * ATOM_BYTES, &P.tq, bar_addr(sb, BAR_Q), a * 64, 0, h, b);
          fa_tma_load_4d(sb + (i * ATOMS + a) * ATOM_BYTES + 64 * 128, &P.tq, bar_addr(sb, BAR_Q), a * 64, 0, h, b);
        } else {
          fa_tma_load_4d(sb + (i * ATOMS + a) * ATOM_BYTES, &P.tq, bar_addr(sb, BAR_Q), a * 64, m0 + i * BM, h, b);
        }
      }
  }
  for (int i = tid; i < 2 * MAXT; i += NT) cls[i] = 0;
  if (warp == WARP_MMA) fa_tmem_alloc(sb + OFF_MISC, TMEM_COLS);
  __syncthreads();
  // class of every kv tile for both query tiles: 0 skip, 1 apply mask_mod, 2 full (from the table
  // entries read at the top of the kernel)
  {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int mi = m0 + i * BM;
      if (mi >= p.Sq) continue;
      if (!tables) {
        for (int t = tid; t < ntiles; t += NT) cls[i * MAXT + t] = FA_HAS_MASK_MOD ? 1 : 2;
        continue;
      }
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const int* idxp = which ? p.t.full_kv_idx : p.t.kv_idx;
        const int n = min(max(num[i][which], 0), p.t.nKV) * tpb;
        if (tid < n) {
          const int t = min(max(blk[i][which], 0), p.t.nKV - 1) * tpb + ti0;
          if (t < ntiles) cls[i * MAXT + t] = (unsigned char)(which ? 2 : 1);
        }
        for (int e = tid + NT; e < n; e += NT) {  // (more list entries than threads)
          const int bi = e / tpb, ti = e - bi * tpb;
          const int t = min(max(idxp[rows[i] * p.t.nKV + bi], 0), p.t.nKV - 1) * tpb + ti;
          if (t < ntiles) cls[i * MAXT + t] = (unsigned char)(which ? 2 : 1);
        }
      }
    }
  }
  __syncthreads();
  // The kv schedule: the listed tiles in ascending order, compacted by the first 256 threads (one
  // tile each) with a ballot per warp and a prefix over the eight warp counts.
  {
    int* wcount = (int*)(sm + OFF_WCNT);
    const bool mine = tid < MAXT;
    const unsigned char c0 = (mine && tid < ntiles) ? cls[tid] : 0;
    const unsigned char c1 = (!DECODE && mine && tid < ntiles) ? cls[MAXT + tid] : 0;
    const bool listed = (c0 | c1) != 0;
    const unsigned vote = __ballot_sync(0xffffffffu, listed);
    if (mine && lane == 0) wcount[warp] = __popc(vote);
    __syncthreads();
    if (mine) {
      int before = 0, total = 0;
      for (int w = 0; w < MAXT / 32; ++w) {
        const int n = wcount[w];
        before += w < warp ? n : 0;
        total += n;
      }
      const int pos = before + __popc(vote & ((1u << lane) - 1u));
#if FA_TC_DECODE
      // this CTA's share of the listed kv tiles; entry k of the share belongs to warpgroup k % 2
      const int per = (total + (int)gridDim.x - 1) / (int)gridDim.x;
      const int lo = split * per, hi = min(total, lo + per);
      if (listed && pos >= lo && pos < hi) {
        sched_tile[pos - lo] = (short)tid;
        sched_mode[pos - lo] = c0;
      }
      if (tid == 0) {
        const int k = max(hi - lo, 0);
        sched_mode[k] = 0;  // an odd share leaves the second warpgroup without a tile in the last step
        misc[2] = (k + 1) / 2;
        misc[3] = k;
      }
#else
      if (listed) {
        sched_tile[pos] = (short)tid;
        sched_mode[2 * pos] = c0;
        sched_mode[2 * pos + 1] = c1;
      }
      if (tid == 0) {
        misc[2] = total;
        misc[3] = total;
      }
#endif
    }
  }
  fa_tc_fence_before();
  __syncthreads();
  fa_tc_fence_after();
  const fa_u32 tmem = (fa_u32)misc[0];
  const int nsteps = misc[2];   // steps of the softmax / MMA loops
  const int nloads = misc[3];   // kv tiles the producer brings in (two per step in the decode variant)
  volatile int* abort_flag = misc + 1;

  if (warp >= 8) fa_setmaxnreg_dec<REGS_OTHER>();
  if (warp == WARP_PRODUCER) {
    // ================================ TMA producer =======================================
    if (lane == 0) {
      fa_tma_prefetch_desc(&P.tk);
      fa_tma_prefetch_desc(&P.tv);
      // a CTA without kv tiles still has to see its query loads land before it may exit
      bool ok = nloads > 0 || fa_mbar_wait(bar_addr(sb, BAR_Q), 0, abort_flag);
      for (int j = 0; j < nloads && ok; ++j) {
        const int s = j % NSTAGE;
        const fa_u32 ph = (fa_u32)((j / NSTAGE) & 1);
        const int n0 = (int)sched_tile[j] * BN;
        if (j >= NSTAGE) ok = fa_mbar_wait(bar_addr(sb, BAR_KEMPTY + s), ph ^ 1u, abort_flag);
        if (!ok) break;
        fa_mbar_expect_tx(bar_addr(sb, BAR_KFULL + s), KV_STAGE);
        for (int a = 0; a < ATOMS; ++a)
          fa_tma_load_4d(sb + OFF_K + s * KV_STAGE + a * ATOM_BYTES, &P.tk, bar_addr(sb, BAR_KFULL + s), a * 64, n0, hk, b);
        if (j >= NSTAGE) ok = fa_mbar_wait(bar_addr(sb, BAR_VEMPTY + s), ph ^ 1u, abort_flag);
        if (!ok) break;
        fa_mbar_expect_tx(bar_addr(sb, BAR_VFULL + s), KV_STAGE);
        for (int a = 0; a < ATOMS; ++a)
          fa_tma_load_4d(sb + OFF_V + s * KV_STAGE + a * ATOM_BYTES, &P.tv, bar_addr(sb, BAR_VFULL + s), a * 64, n0, hk, b);
      }
    }
  } else if (SEP_P && (warp == WARP_MMA || warp == WARP_MMA_B)) {
    // ============ two MMA issuers (D = 64): warp A issues the S products, warp B the PV products ====
    // With P in its own TMEM columns the two streams only meet through the softmax warps, so each
    // issuer waits on its own barriers and the waits of one overlap the issue of the other.
    if (lane == 0 && nsteps > 0) {
      constexpr fa_u32 HI = fa_desc_hi_sw128();
      if (warp == WARP_MMA) {
        constexpr fa_u32 IDESC_S = fa_idesc(DT, BM, BN, 0, 0);
        bool ok = fa_mbar_wait(bar_addr(sb, BAR_Q), 0, abort_flag);
        fa_u32 nsi[2] = {0, 0};
        for (int j = 0; j < nsteps && ok; ++j) {
          // the kv tile of (step, query tile): the same for both tiles in the forward, alternate
          // tiles of the CTA's share in the decode variant
          int s = j % NSTAGE;
          if (!DECODE) ok = fa_mbar_wait(bar_addr(sb, BAR_KFULL + s), (fa_u32)((j / NSTAGE) & 1), abort_flag);
          for (int i = 0; i < 2 && ok; ++i) {
            if (!sched_mode[2 * j + i]) continue;
            if (DECODE) {
              const int t = 2 * j + i;
              s = t % NSTAGE;
              ok = fa_mbar_wait(bar_addr(sb, BAR_KFULL + s), (fa_u32)((t / NSTAGE) & 1), abort_flag);
              if (!ok) break;
            }
            if (nsi[i] > 0) {
              ok = fa_mbar_wait(bar_addr(sb, BAR_SFREE2 + i), (nsi[i] - 1) & 1u, abort_flag);
              if (!ok) break;
            }
            fa_tc_fence_after();
            const fa_u32 loQ = fa_desc_lo(sb + i * ATOMS * ATOM_BYTES, 16), loK = fa_desc_lo(sb + OFF_K + s * KV_STAGE, 16);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const fa_u32 koff = ((kk / 4) * ATOM_BYTES + (kk % 4) * 32) >> 4;
              fa_mma_ss(tmem + COL_S + i * BN, fa_desc_make(loQ + koff, HI), fa_desc_make(loK + koff, HI), IDESC_S, kk > 0);
            }
            fa_mma_commit(bar_addr(sb, BAR_S + i));
            if (DECODE) fa_mma_commit(bar_addr(sb, BAR_KEMPTY + s));
            ++nsi[i];
          }
          if (!DECODE) fa_mma_commit(bar_addr(sb, BAR_KEMPTY + s));
        }
      } else {
        constexpr fa_u32 IDESC_O = fa_idesc(DT, BM, D, 0, 1);
        bool ok = true;
        fa_u32 cnt[2] = {0, 0};
        for (int j = 0; j < nsteps && ok; ++j) {
          int s = j % NSTAGE;
          if (!DECODE) ok = fa_mbar_wait(bar_addr(sb, BAR_VFULL + s), (fa_u32)((j / NSTAGE) & 1), abort_flag);
          for (int i = 0; i < 2 && ok; ++i) {
            if (!sched_mode[2 * j + i]) continue;
            if (DECODE) {
              const int t = 2 * j + i;
              s = t % NSTAGE;
              ok = fa_mbar_wait(bar_addr(sb, BAR_VFULL + s), (fa_u32)((t / NSTAGE) & 1), abort_flag);
              if (!ok) break;
            }
            ok = fa_mbar_wait(bar_addr(sb, BAR_P + i), cnt[i] & 1u, abort_flag);
            if (!ok) break;
            fa_tc_fence_after();
            const fa_u32 loV = fa_desc_lo(sb + OFF_V + s * KV_STAGE, ATOM_BYTES);
            const fa_u32 acc = cnt[i] > 0;
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk)
              fa_mma_ts(tmem + COL_O + i * D, tmem + COL_P + i * 64 + kk * 8, fa_desc_make(loV + kk * 128, HI), IDESC_O, acc | (kk > 0));
            fa_mma_commit(bar_addr(sb, BAR_O + i));
            if (DECODE) fa_mma_commit(bar_addr(sb, BAR_VEMPTY + s));
            ++cnt[i];
          }
          if (!DECODE) fa_mma_commit(bar_addr(sb, BAR_VEMPTY + s));
        }
      }
    }
  } else if (!SEP_P && (warp == WARP_MMA || warp == WARP_MMA_B)) {
    // ============ two MMA issuers (D = 128): warp A issues both products of query tile 0, warp B of tile 1 ====
    // P overwrites the S columns here, so the products of one tile form a chain  PV_i(j), S_i(j+1),
    // PV_i(j+1) ...; the chains of the two tiles only share the K / V stages.  Issuing the sixteen
    // instructions of a step's two products takes one thread about as long as the tensor core needs
    // to run them, so each chain gets its own issuing warp; a K / V stage is released by one
    // arrival from each.  The whole warp runs the loop and one elected lane issues: in uniform
    // control flow the operands of tcgen05.mma sit in uniform registers, which makes the
    // instructions cheaper to issue than from a single-lane branch (attention-sink forward,
    // B4 H16 S8192: 0.80 ms with one issuing lane, 0.70 with one per tile, 0.65 with elected lanes).
    {
      const bool leader = fa_elect_one();
      const fa_u32 tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
      const int nsteps_u = __shfl_sync(0xffffffffu, nsteps, 0);
      const int i = warp == WARP_MMA ? 0 : 1;
      constexpr fa_u32 IDESC_S = fa_idesc(DT, BM, BN, 0, 0);
      constexpr fa_u32 IDESC_O = fa_idesc(DT, BM, D, 0, 1);
      bool ok = nsteps_u == 0 || fa_mbar_wait_all(bar_addr(sb, BAR_Q), 0, abort_flag);
      fa_u32 cnt = 0;  // PV products of this tile issued so far
      // Descriptors: constant high word; the low word (start address and MN-chunk distance in
      // 16-byte units) is stepped with one add per k-step.
      constexpr fa_u32 HI = fa_desc_hi_sw128();
      // S_i = Q_i K^T for step j into TMEM columns COL_S + 128 i
      auto issue_s = [&](int j) {
        const int s = j % NSTAGE;
        const fa_u32 loQ = fa_desc_lo(sb + i * ATOMS * ATOM_BYTES, 16);
        const fa_u32 loK = fa_desc_lo(sb + OFF_K + s * KV_STAGE, 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const fa_u32 koff = ((kk / 4) * ATOM_BYTES + (kk % 4) * 32) >> 4;
          if (leader) fa_mma_ss(tmem_u + COL_S + i * BN, fa_desc_make(loQ + koff, HI), fa_desc_make(loK + koff, HI), IDESC_S, kk > 0);
        }
        if (leader) fa_mma_commit(bar_addr(sb, BAR_S + i));
      };
      // O_i += P_i V for step j (P_i: 16-bit, in the first 64 columns of S_i)
      auto issue_pv = [&](int j, bool first) {
        const int s = j % NSTAGE;
        const fa_u32 loV = fa_desc_lo(sb + OFF_V + s * KV_STAGE, ATOM_BYTES);
        const fa_u32 acc = !first;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          if (leader) fa_mma_ts(tmem_u + COL_O + i * D, tmem_u + COL_S + i * BN + kk * 8, fa_desc_make(loV + kk * 128, HI), IDESC_O, acc | (kk > 0));
        if (leader) fa_mma_commit(bar_addr(sb, BAR_O + i));
      };
      if (ok && nsteps_u > 0) {
        ok = fa_mbar_wait_all(bar_addr(sb, BAR_KFULL + 0), 0, abort_flag);
        if (ok) {
          fa_tc_fence_after();
          if (sched_mode[i]) issue_s(0);
          if (leader) fa_mma_commit(bar_addr(sb, BAR_KEMPTY + 0));  // (a commit with nothing outstanding arrives at once)
        }
      }
      for (int j = 0; j < nsteps_u && ok; ++j) {
        const int s = j % NSTAGE;
        const fa_u32 ph = (fa_u32)((j / NSTAGE) & 1);
        const bool more = j + 1 < nsteps_u;
        const int s1 = (j + 1) % NSTAGE;
        const fa_u32 ph1 = (fa_u32)(((j + 1) / NSTAGE) & 1);
        // Every step waits for its stage to be full before it releases it, with or without a
        // product of this tile: the load of a stage follows both releases of its previous use, so a
        // warp whose tile skips several steps cannot release a stage twice before the other warp
        // has released it once.
        ok = fa_mbar_wait_all(bar_addr(sb, BAR_VFULL + s), ph, abort_flag);
        if (!ok) break;
        if (sched_mode[2 * j + i]) {
          ok = fa_mbar_wait_all(bar_addr(sb, BAR_P + i), cnt & 1u, abort_flag);
          if (!ok) break;
          fa_tc_fence_after();
          issue_pv(j, cnt == 0);
          ++cnt;
        }
        if (leader) fa_mma_commit(bar_addr(sb, BAR_VEMPTY + s));
        if (more) {
          ok = fa_mbar_wait_all(bar_addr(sb, BAR_KFULL + s1), ph1, abort_flag);
          if (!ok) break;
          // S of the next step overwrites the columns P was read from: it follows the PV product
          if (sched_mode[2 * (j + 1) + i]) {
            fa_tc_fence_after();
            issue_s(j + 1);
          }
          if (leader) fa_mma_commit(bar_addr(sb, BAR_KEMPTY + s1));
        }
      }
    }
  } else if (warp < 8) {
    // ================================ softmax warpgroups ==================================
    fa_setmaxnreg_inc<REGS_SOFTMAX>();
    const int i = warp >> 2;                       // query tile of this warpgroup
    const int lane_base = (warp & 3) * 32;         // TMEM lanes this warp may touch
    const int r = lane_base + lane;                // row inside the tile
    const int qi = DECODE ? (r & 63) : m0 + i * BM + r;  // query index
    const int half = DECODE ? (r >> 6) : 0;               // decode variant: kv columns 64 * half .. + 63 of every tile
    // decode variant: warps whose 32 rows are all padding (fewer than 33 queries) only keep the barrier protocol going
    const bool warp_active = !DECODE || (lane_base & 63) < p.Sq;
    fa_u32 idle_cnt = 0;
    const fa_u32 t_s = tmem + ((fa_u32)lane_base << 16) + COL_S + i * BN;
    const fa_u32 t_o = tmem + ((fa_u32)lane_base << 16) + COL_O + i * D;
    const fa_u32 t_p = SEP_P ? tmem + ((fa_u32)lane_base << 16) + COL_P + i * 64 : t_s;
    bool ok = true;
    // (rows beyond Sq have no row in the bit matrix: their scores are never stored, the mask is evaluated)
    const unsigned* rowbits = (p.t.mask_bits != nullptr && qi < p.Sq)
        ? p.t.mask_bits + (((long long)(p.t.mask_B == 1 ? 0 : b) * p.t.mask_H + (p.t.mask_H == 1 ? 0 : h)) * p.t.mask_rows + qi) * p.t.mask_stride
        : nullptr;
    SoftmaxCtx c = {p, sb, t_s, t_o, t_p, i, warp, qi, gb, gh, half, p.scale * FA_LOG2E, abort_flag, sched_tile, FA_NEG_INF, 0.f, 0u, rowbits};
    if (DECODE) {
      // the P columns of the other half of this lane's kv columns are never written again
      fa_u32 z[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) z[e] = 0u;
      fa_tmem_st16(t_p + (1 - half) * 32, z);
      fa_tmem_st16(t_p + (1 - half) * 32 + 16, z);
      fa_tmem_wait_st();
    }
    for (int j = 0; j < nsteps && ok; ++j) {
      const int mode = sched_mode[2 * j + i];
      if (mode == 0) continue;
      if (!warp_active) {
        // in step with the working warps: S of this step is there, then both arrivals they also make
        ok = fa_mbar_wait_warp(bar_addr(sb, BAR_S + i), idle_cnt & 1u, abort_flag);
        // The PV product of the previous step must be complete before this warp arrives on the P
        // barrier again: otherwise its arrival would be counted into the previous phase, which the
        // working warps may not have reached yet, and that product would start on unwritten P.
        if (ok && idle_cnt > 0) ok = fa_mbar_wait_warp(bar_addr(sb, BAR_O + i), (idle_cnt - 1) & 1u, abort_flag);
        if (!ok) break;
        fa_tc_fence_after();
        fa_tc_fence_before();
        if (SEP_P) fa_mbar_arrive(bar_addr(sb, BAR_SFREE2 + i));
        fa_mbar_arrive(bar_addr(sb, BAR_P + i));
        ++idle_cnt;
        continue;
      }
      const bool masked = (FA_HAS_MASK_MOD && mode == 1) || (int)sched_tile[DECODE ? 2 * j + i : j] * BN + BN > p.Skv;
      if (D == 64) ok = softmax_step<2>(c, j, mode, masked);
      else ok = masked ? softmax_step<1>(c, j, mode, true) : softmax_step<0>(c, j, mode, false);
    }
    const float m_ref = c.m_ref, l = c.l;
    const fa_u32 cnt = warp_active ? c.cnt : idle_cnt;
    // ---- epilogue: O / l and the logsumexp of this thread's row ---------------------------
    if (ok && cnt > 0) ok = fa_mbar_wait_warp(bar_addr(sb, BAR_O + i), (cnt - 1) & 1u, abort_flag);
#if FA_TC_DECODE
    // The four partial results of a query row (two warpgroups x two column halves) are merged
    // inside the CTA: every thread puts its (O, maximum, sum) into shared memory, over the K / V
    // ring, which nothing reads or writes any more once both warpgroups have seen their last
    // product complete; then the 256 threads merge 64 rows x 64 columns and the CTA writes ONE
    // un-normalised partial result per row for the combine kernel.  All 256 softmax threads reach
    // both barriers, whatever happened before (every earlier wait is bounded).
    {
      constexpr int MP = D + 4;  // floats per scratch row: O[D], maximum, sum, pad (16-byte rows)
      float* scratch = (float*)(sm + OFF_K);
      static_assert(2 * 128 * MP * 4 <= 2 * NSTAGE * KV_STAGE, "merge scratch fits the K / V ring");
      asm volatile("bar.sync 2, 256;" ::: "memory");
      const bool good = ok && *abort_flag == 0;
      if (good && warp_active) {
        fa_tc_fence_after();
        float* row = scratch + (i * 128 + r) * MP;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float o[32];
          if (cnt > 0) {
            fa_tmem_ld32(t_o + c * 32, o);
            fa_tmem_wait_ld();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = 0.f;
          }
#pragma unroll
          for (int e = 0; e < 32; e += 4) *(float4*)(row + c * 32 + e) = make_float4(o[e], o[e + 1], o[e + 2], o[e + 3]);
        }
        *(float2*)(row + D) = make_float2(m_ref, m_ref != FA_NEG_INF ? l : 0.f);
      }
      asm volatile("bar.sync 2, 256;" ::: "memory");
      if (*abort_flag == 0) {
        const int mt = tid;                     // 0 .. 255
        const int mrow = mt >> 2, c0 = (mt & 3) * 16;  // query row, first of this thread's 16 columns
        if (mrow < p.Sq) {
          const float* src[4];
          float mm[4], mstar = FA_NEG_INF;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            src[k] = scratch + ((k >> 1) * 128 + (k & 1) * 64 + mrow) * MP;
            mm[k] = src[k][D];
            mstar = fmaxf(mstar, mm[k]);
          }
          float acc[16], lsum = 0.f;
#pragma unroll
          for (int e = 0; e < 16; ++e) acc[e] = 0.f;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float w = mm[k] == FA_NEG_INF ? 0.f : fa_ex2(mm[k] - mstar);
            lsum += w * src[k][D + 1];
#pragma unroll
            for (int e = 0; e < 16; e += 4) {
              const float4 v4 = *(const float4*)(src[k] + c0 + e);
              acc[e] += w * v4.x; acc[e + 1] += w * v4.y; acc[e + 2] += w * v4.z; acc[e + 3] += w * v4.w;
            }
          }
          const long long prow = (((long long)b * p.Hq + h) * p.num_splits + split) * p.Sq + mrow;
#pragma unroll
          for (int e = 0; e < 16; e += 4)
            *(float4*)(p.part_o + prow * D + c0 + e) = make_float4(acc[e], acc[e + 1], acc[e + 2], acc[e + 3]);
          if ((mt & 3) == 0) *(float2*)(p.part_ml + prow * 2) = make_float2(mstar, lsum);
        }
      }
    }
#else
    {
      // The output tile leaves through the shared memory of this warpgroup's query tile, which
      // nothing reads any more (every S product of the tile is complete): each thread converts its
      // row into the layout of the tile (128-byte rows, 16-byte chunk k of row r at k ^ (r & 7)) and
      // one tensor-map store per 64 columns writes whole lines and clips the rows beyond Sq.  (Each
      // thread storing its own row to global memory costs 32 different lines per instruction.)
      // All four warps of the warpgroup reach the barrier below, whatever happened before: every
      // earlier wait is bounded.
      // (a tile without kv steps: nothing has waited for the load of the query tile yet)
      if (ok && cnt == 0) ok = fa_mbar_wait_warp(bar_addr(sb, BAR_Q), 0, abort_flag);
      if (ok) {
        fa_tc_fence_after();
        // a row that never saw an unmasked key has no mass (its sum may hold the tiny values the
        // polynomial exponential returns for -inf): its output is 0
        const float inv = (l > 0.f && m_ref != FA_NEG_INF) ? 1.f / l : 0.f;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float o[32];
          if (cnt > 0) {
            fa_tmem_ld32(t_o + c * 32, o);
            fa_tmem_wait_ld();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = 0.f;
          }
          unsigned char* strow = sm + (i * ATOMS + (c >> 1)) * ATOM_BYTES + r * 128;
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 w;
            w.x = fa_pack2<DT>(o[e] * inv, o[e + 1] * inv);
            w.y = fa_pack2<DT>(o[e + 2] * inv, o[e + 3] * inv);
            w.z = fa_pack2<DT>(o[e + 4] * inv, o[e + 5] * inv);
            w.w = fa_pack2<DT>(o[e + 6] * inv, o[e + 7] * inv);
            *(uint4*)(strow + ((((c & 1) * 4 + (e >> 3)) ^ (r & 7)) * 16)) = w;
          }
        }
        if (p.lse != nullptr && qi < p.Sq)
          p.lse[((long long)b * p.Hq + h) * p.Sq + qi] = (l > 0.f && m_ref != FA_NEG_INF) ? (m_ref + fa_lg2(l)) * FA_LN2 : FA_NEG_INF;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("bar.sync %0, 128;" ::"r"(3 + i) : "memory");
      if ((warp & 3) == 0 && lane == 0 && *abort_flag == 0 && m0 + i * BM < p.Sq) {
        for (int a = 0; a < ATOMS; ++a) fa_tma_store_4d(&P.to, sb + (i * ATOMS + a) * ATOM_BYTES, a * 64, m0 + i * BM, h, b);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the tile must outlive the reads of the store
      }
    }
#endif
  }

  // ---- teardown ----------------------------------------------------------------------------
  fa_tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    fa_tc_fence_after();
    fa_tmem_dealloc(tmem, TMEM_COLS);
  }
  if (tid == 0 && *abort_flag != 0 && p.status != nullptr) atomicOr(p.status, FA_STATUS_WAIT_TIMEOUT);
}
