// Flash-attention backward for sm_100a on the 5th-generation tensor cores (fp16 / bf16,
// D = Dv = 64 or 128).  One kernel computes dK, dV and dQ in a single pass over the
// (kv tile, q tile) pairs the BlockMask lists: five tcgen05.mma products per pair and one
// exponential per score, where the two-scan reference kernel
// (flaxattention/kernel/attention.py:423-553) and fa_bwd.cuh need seven products and two
// exponentials.
//
// The unit of work (an item) is a 128-row kv tile of one (batch, kv head) together with the q tiles
// of the query heads that share it.  The kernel is persistent: one CTA per SM, every CTA works
// through items it takes from a counter in global memory, and TMEM and the barriers are set up
// once per CTA.  A pair is 128 kv rows x BQ query rows, BQ = 128 with D = 64 and 64 with
// D = 128 (the 512 TMEM columns hold two D-wide accumulators, dK and dV, next to the pair's
// score tiles only for the smaller q tile).  Everything is kept transposed so that dK and dV
// have kv rows (TMEM lanes) and P^T can be fed to the tensor core straight from TMEM:
//   1. S^T  = K Q^T                      (TMEM, 128 kv x BQ q, fp32)
//   2. dP^T = V dO^T                     (TMEM)
//      p = 2^(x - lse), ds = p (dp - delta) score_mod'      thread (kv row, BQ/2 q columns)
//      P^T -> TMEM (16 bit),  dS^T -> shared memory (16 bit, [kv][q], 128-byte swizzle)
//   3. dV += P^T dO                      (A from TMEM)
//   4. dK += dS^T Q                      (A = dS^T from smem, K-major)
//   5. D = 64:   dQ   = dS K             (A = the same dS^T tile read MN-major, B = K; 128 q x 64 d)
//      D = 128:  dQ^T = K^T dS^T         (A = K read MN-major, B = dS^T read MN-major; 128 d x 64 q)
// Either way the dQ tile of a pair is 128 TMEM lanes x 64 columns of fp32.  It leaves through a
// staging buffer and two bulk reduce-adds into an fp32 accumulation buffer (summation order
// over kv tiles is not fixed; a small kernel scales, un-permutes and converts it afterwards).
// dK and dV are written once per item.
//
// Warp roles (16 warps): 0-3 and 4-7 compute (first / second half of the q columns of the pair),
// 8-11 drain (dQ of every pair, dK / dV of every item), 12 producer (pair lists and TMA loads), 13 MMA issuer A (products 1-2, TMEM owner), 14 MMA issuer B
// (products 3-4), 15 MMA issuer C (product 5).
// S^T/dP^T of pair n+1 are issued as soon as the compute warps hold pair n in registers, so
// the tensor core runs ahead of the element-wise work.
//
// TMEM (512 columns)   D = 64:  S^T 0-127, dP^T 128-255, P^T 256-319, dV 320-383, dK 384-447, dQ 448-511
//                      D = 128: S^T 0-63, dP^T 64-127, P^T 128-159, dQ^T 192-255, dV 256-383, dK 384-511
// Every mbarrier wait is bounded (see fa_sm100.cuh).
//
// Compile-time parameters (macros): FA_DTYPE (0 fp16, 1 bf16), FA_D (64 or 128; Dv = D), FA_BWD_KV2
// (two K / V buffers and a three-stage ring, head dim 64 only).
#pragma once
#include "fa_sm100.cuh"

#ifndef FA_D
#define FA_D 64
#endif

struct FaBwdTcParams {
  FaParams p;
  FaTensorMap tq, tk, tv, tdo;  // 4-d maps (D, S, H, B), 128-byte swizzle; box 64 x 128 rows (k, v), 64 x BQ rows (q, do)
  FaTensorMap tdk, tdv;         // the outputs dK and dV, like tk and tv
  float* dq_acc;                // per (b, h, BQ-row q tile): two [128 lanes][32 columns] fp32 blocks, 16-byte chunks of a row permuted
  const float* nlse2;           // [B, Hq, ceil(Sq/128)*128]: -lse * log2(e); -inf for rows without mass / beyond Sq
  const float* ndelta;          // same shape: -rowsum(O * dO); 0 beyond Sq
  int* work_counter;            // zero at launch: items beyond the first of every CTA are handed out through it
};

namespace fa_btc {

constexpr int DT = FA_DTYPE;
constexpr int D = FA_D;
static_assert(D == 64 || D == 128, "head dim 64 or 128");
constexpr int BT = 128;                    // kv rows of a tile
constexpr int BQ = D == 64 ? 128 : 64;     // q rows of a pair
constexpr int CW = BQ / 2;                 // q columns of one compute thread
constexpr int DATOMS = D / 64;             // 64-element (128-byte) column groups of a K / V / Q / dO row
constexpr int ATOM_BYTES = 128 * 128;      // 128 rows x 128 bytes
constexpr int KV_BYTES = DATOMS * ATOM_BYTES;        // one K or V tile
constexpr int Q_ATOM_BYTES = BQ * 128;               // BQ rows x 128 bytes
constexpr int Q_BYTES = DATOMS * Q_ATOM_BYTES;       // one Q or dO tile (16 KB in both configurations)
constexpr int DS_ATOMS = BQ / 64;                    // dS^T: [128 kv][BQ q] as atoms of 64 q columns
// K / V buffers and Q / dO ring depth.  With D = 64 shared memory holds either one K / V buffer and a
// ring of four stages, or two K / V buffers and a ring of three (FA_BWD_KV2): with two, K and V of the
// next item are loaded while the current one is computed and nothing waits at the change of items,
// which pays when items are short (causal S=2048, 8.5 pairs per item on average: 150 against 158 us)
// and costs when they are long (dense S=2048, 16 pairs: 215 against 206 us - the fourth stage matters
// more than the bubble).  The host picks.  With D = 128 there is one buffer and three stages.
#ifndef FA_BWD_KV2
#define FA_BWD_KV2 0
#endif
constexpr int KVBUF = (D == 64 && FA_BWD_KV2) ? 2 : 1;
constexpr int NSTAGE = (D == 64 && KVBUF == 1) ? 4 : 3;
constexpr int MAXPL = D == 64 ? 1024 : 2048;  // (head, q tile) pairs of one item (two such lists fit in shared memory)
constexpr int MAXC = 256;                // 128-row q tiles per head (Sq <= 32768)
constexpr int NT = 512;
constexpr int WARP_PRODUCER = 12, WARP_MMA = 13, WARP_MMA_B = 14, WARP_MMA_C = 15;
// Register split (setmaxnreg): the kernel starts with 128 registers per thread (65536 / 512).  The
// eight warps that are not compute warps give up 32 each and the eight compute warps take 32 each;
// an increase that asked for more than the decrease releases would wait forever.  The compute warps
// need no more than 160 (their 16-column steps keep few values live); with 200 / 56 the producer,
// drain and issuing warps spilled, and the kernel was 4-5 % slower (dense backward 218 against 205 us,
// attention sink 934 against 895; 192 / 64, 176 / 80, 168 / 88, 152 / 104 and 144 / 112 all lie within
// 1 % of 160 / 96, 184 / 72 was as slow as 200 / 56).
constexpr int REGS_COMPUTE = 160, REGS_OTHER = 96;
static_assert(256 * (REGS_COMPUTE - 128) <= 256 * (128 - REGS_OTHER), "setmaxnreg.inc would wait forever");

// shared memory map (from a 1024-byte aligned base)
constexpr int OFF_K = 0;
constexpr int OFF_V = OFF_K + KVBUF * KV_BYTES;
constexpr int OFF_Q = OFF_V + KVBUF * KV_BYTES;             // NSTAGE tiles
constexpr int OFF_DO = OFF_Q + NSTAGE * Q_BYTES;            // NSTAGE tiles
constexpr int OFF_DS = OFF_DO + NSTAGE * Q_BYTES;           // dS^T
constexpr int OFF_DQ = OFF_DS + DS_ATOMS * ATOM_BYTES;      // fp32 staging 128 x 32 (half of the dQ tile at a time)
constexpr int DQ_HALF_BYTES = 128 * 32 * 4;
constexpr int OFF_ROW = OFF_DQ + DQ_HALF_BYTES;             // NSTAGE x (nlse2[BQ], ndelta[BQ]) floats
constexpr int OFF_BAR = OFF_ROW + NSTAGE * 2 * BQ * 4;
constexpr int NBARS = 2 + 3 * NSTAGE + 15;
constexpr int OFF_MISC = OFF_BAR + NBARS * 8;               // tmem base, abort, -, drain flag
constexpr int OFF_ITEM = OFF_MISC + 16;                     // int item[2][2]: item number, pairs (-1: no more work)
constexpr int OFF_PAIR = OFF_ITEM + 16;                     // int pair[2][MAXPL]: q tile | mode << 16 | g << 20
constexpr int OFF_CLS = OFF_PAIR + 2 * MAXPL * 4;           // uchar cls[MAXC] (scratch of the list builder)
constexpr int SMEM_BYTES = OFF_CLS + MAXC + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
constexpr int TMEM_COLS = 512;
constexpr int COL_S = 0, COL_DP = BQ, COL_P = 2 * BQ;
constexpr int COL_DQ = D == 64 ? 448 : 192;
constexpr int COL_DV = D == 64 ? 320 : 256;
constexpr int COL_DK = D == 64 ? 384 : 384;
static_assert(COL_P + BQ / 2 <= (D == 64 ? COL_DV : COL_DQ), "TMEM map");

constexpr int BAR_KV = 0;                   // [2] K and V of an item have landed in buffer kb
// A stage's Q tile (with the row scalars) and dO tile are released separately: dO is last read by
// product 3, Q by product 4, and the sooner a slot is free the further ahead the producer runs.
constexpr int BAR_QFULL = 2, BAR_QEMPTY = 2 + NSTAGE, BAR_DOEMPTY = 2 + 2 * NSTAGE;
constexpr int BAR_SFULL = 2 + 3 * NSTAGE;   // S^T and dP^T of a pair are in TMEM
constexpr int BAR_SFREE = BAR_SFULL + 1;    // compute warps hold them in registers (256 arrivals)
constexpr int BAR_PREADY = BAR_SFULL + 2;   // P^T in TMEM and dS^T in smem (256 arrivals)
constexpr int BAR_PFREE = BAR_SFULL + 3;    // products 3-5 of the pair are complete
constexpr int BAR_DQFULL = BAR_SFULL + 4;   // dQ of the pair is in TMEM
constexpr int BAR_DQFREE = BAR_SFULL + 5;   // drain warps hold it in registers (128 arrivals)
constexpr int BAR_FINAL = BAR_SFULL + 6;    // [2] products 3-5 of the last pair of the item in buffer kb are complete
constexpr int BAR_DKVFREE = BAR_SFULL + 8;  // the drain warps have read dK and dV of an item out of TMEM (128 arrivals)
constexpr int BAR_LISTFULL = BAR_SFULL + 9; // [2] the producer has published an item and its pair list
constexpr int BAR_LISTFREE = BAR_SFULL + 11;  // [2] the 15 consumers of a list are done with it
constexpr int BAR_KVFREE = BAR_SFULL + 13;  // [2] (two K / V buffers) the stores of dK / dV staged in buffer kb have read it
constexpr int LIST_CONSUMERS = 3 + 8 + 4;   // MMA issuers, compute warps, drain warps (one arrival each)

__device__ __forceinline__ fa_u32 bar_addr(fa_u32 sb, int i) { return sb + OFF_BAR + i * 8; }

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void bulk_reduce_add_f32(float* gdst, fa_u32 ssrc, fa_u32 bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gdst), "r"(ssrc), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// brings a tile into L2 ahead of the load that will need it
__device__ __forceinline__ void tma_prefetch_l2_4d(const FaTensorMap* map, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

// byte offset (in 16-byte units) of k-step kk of a K-major operand whose 64-element column groups
// are `atom_bytes` apart: 32 bytes per step inside a 128-byte row, four steps per group
__device__ __forceinline__ constexpr fa_u32 kstep_kmajor(int kk, int atom_bytes) {
  return (fa_u32)(((kk >> 2) * atom_bytes + (kk & 3) * 32) >> 4);
}

// Element-wise work of one thread on a W-column chunk: scores s and dp (fp32, raw) for kv row
// `kv` and q columns q0 .. q0+W-1 -> packed P^T and dS^T (16 bit).  q0 is a multiple of W (the
// compiler can see that from how the caller builds it), so the low bits of every q index are
// compile-time constants inside the mods while one copy of this code serves all chunks of a
// tile row.  nlse2 / ndelta point at the row scalars of column q0.
template <int W>
__device__ __forceinline__ void chunk(const float (&s)[W], const float (&dp)[W], const float* nlse2, const float* ndelta,
                                      fa_u32 (&pp)[W / 2], fa_u32 (&ds)[W / 2], int mode, int q0, int kv, int gb, int gh,
                                      float scale, float sc2) {
#if !FA_ROUND_SCORES && (!FA_HAS_SCORE_MOD || defined(FA_SCORE_AFFINE))
  // no score_mod, or an affine one: two elements per instruction (packed fp32) wherever the
  // hardware has the form; only the exponentials and the mask are per element
#if FA_HAS_SCORE_MOD && defined(FA_SCORE_LINEAR_Q)
  // the multiplier does not read q and the bias is linear in it (relative-position biases such as
  // ALiBi): both are taken once, at the first column of the chunk, and column e adds e times the slope
  const float lin_g = fa_score_mul(0.f, gb, gh, q0, kv);
  const fa_u64 lin_g2 = fa_f2(lin_g, lin_g), lin_gs2 = fa_f2(lin_g * sc2, lin_g * sc2);
  const float lin_base = fa_score_add2(0.f, gb, gh, q0, kv), lin_dq = fa_score_add2_dq(0.f, gb, gh, q0, kv);
  const fa_u64 lin_b2 = fa_f2(lin_base, lin_base), lin_d2 = fa_f2(lin_dq, lin_dq);
#endif
#pragma unroll
  for (int e = 0; e < W; e += 4) {
    const float4 nl = *(const float4*)(nlse2 + e);
    const float4 nd = *(const float4*)(ndelta + e);
#pragma unroll
    for (int u = 0; u < 4; u += 2) {
      const int qi0 = q0 | (e + u), qi1 = q0 | (e + u + 1);
      const fa_u64 nl2 = u == 0 ? fa_f2(nl.x, nl.y) : fa_f2(nl.z, nl.w);
      const fa_u64 nd2 = u == 0 ? fa_f2(nd.x, nd.y) : fa_f2(nd.z, nd.w);
      const fa_u64 s2 = fa_f2(s[e + u], s[e + u + 1]);
#if FA_HAS_SCORE_MOD && defined(FA_SCORE_LINEAR_Q)
      const fa_u64 g2 = lin_g2;
      const fa_u64 b2 = fa_add2(fa_fma2(fa_f2((float)(e + u), (float)(e + u + 1)), lin_d2, lin_b2), nl2);
      const fa_u64 x2 = fa_fma2(s2, lin_gs2, b2);
#elif FA_HAS_SCORE_MOD
      const fa_u64 g2 = fa_f2(fa_score_mul(0.f, gb, gh, qi0, kv), fa_score_mul(0.f, gb, gh, qi1, kv));
      const fa_u64 b2 = fa_add2(fa_f2(fa_score_add2(0.f, gb, gh, qi0, kv), fa_score_add2(0.f, gb, gh, qi1, kv)), nl2);
      const fa_u64 x2 = fa_fma2(s2, fa_mul2(g2, fa_f2(sc2, sc2)), b2);
#else
      const fa_u64 x2 = fa_fma2(s2, fa_f2(sc2, sc2), nl2);
#endif
      float x0, x1;
      fa_f2_unpack(x2, x0, x1);
      float p0 = fa_ex2(x0), p1 = fa_ex2(x1);
#if FA_HAS_MASK_MOD
      if (mode == 1) {
        p0 = fa_mask_mod(gb, gh, qi0, kv) ? p0 : 0.f;
        p1 = fa_mask_mod(gb, gh, qi1, kv) ? p1 : 0.f;
      }
#endif
      fa_u64 d2 = fa_mul2(fa_f2(p0, p1), fa_add2(fa_f2(dp[e + u], dp[e + u + 1]), nd2));
#if FA_HAS_SCORE_MOD
      d2 = fa_mul2(d2, g2);
#endif
      float d0, d1;
      fa_f2_unpack(d2, d0, d1);
      pp[(e + u) / 2] = fa_pack2<DT>(p0, p1);
      ds[(e + u) / 2] = fa_pack2<DT>(d0, d1);
    }
  }
#else
#pragma unroll
  for (int e = 0; e < W; e += 4) {
    const float4 nl = *(const float4*)(nlse2 + e);
    const float4 nd = *(const float4*)(ndelta + e);
    float pv[4], dv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int qi = q0 | (e + u);
      const float nlu = u == 0 ? nl.x : (u == 1 ? nl.y : (u == 2 ? nl.z : nl.w));
      const float ndu = u == 0 ? nd.x : (u == 1 ? nd.y : (u == 2 ? nd.z : nd.w));
      float x = s[e + u];
      float g = 1.f;
#if FA_ROUND_SCORES
      {
        float dummy = 0.f;
        fa_round2<DT>(x, dummy);
      }
#endif
#if FA_HAS_SCORE_MOD && defined(FA_SCORE_AFFINE)
      g = fa_score_mul(0.f, gb, gh, qi, kv);
      x = fmaf(x, g * sc2, fa_score_add2(0.f, gb, gh, qi, kv) + nlu);
#elif FA_HAS_SCORE_MOD
      g = fa_score_mod_grad(x * scale, gb, gh, qi, kv);
      x = fa_score_mod(x * scale, gb, gh, qi, kv) * FA_LOG2E + nlu;
#else
      x = fmaf(x, sc2, nlu);
#endif
      float pr = fa_ex2(x);
#if FA_HAS_MASK_MOD
      if (mode == 1) pr = fa_mask_mod(gb, gh, qi, kv) ? pr : 0.f;
#endif
      pv[u] = pr;
      dv[u] = pr * (dp[e + u] + ndu) * g;
    }
    pp[e / 2] = fa_pack2<DT>(pv[0], pv[1]);
    pp[e / 2 + 1] = fa_pack2<DT>(pv[2], pv[3]);
    ds[e / 2] = fa_pack2<DT>(dv[0], dv[1]);
    ds[e / 2 + 1] = fa_pack2<DT>(dv[2], dv[3]);
  }
#endif
}


// The (query head, q tile) pairs of one item, written to `pl` by one warp: per head of the group,
// the 128-row q tiles the BlockMask lists for the item's kv tile (class 1: apply mask_mod, 2: full)
// in ascending order, each as 128 / BQ pairs.  Without tables every tile is listed.  Returns the
// number of pairs (the same in every lane).  `cl` is MAXC bytes of scratch.
__device__ __forceinline__ int build_pair_list(const FaParams& p, int hk, int b, int kt, int G, int n_ctiles,
                                               unsigned char* cl, int* pl, int lane) {
  constexpr int PPT = 128 / BQ;
  const bool tables = p.t.kv_num != nullptr && p.t.q_num != nullptr;
  int w = 0;
  for (int g = 0; g < G; ++g) {
    if (!tables) {
      const int nq = (p.Sq + BQ - 1) / BQ;
      const int mode = FA_HAS_MASK_MOD ? 1 : 2;
      for (int e = lane; e < nq && w + e < MAXPL; e += 32) pl[w + e] = e | (mode << 16) | (g << 20);
      w += nq;
      continue;
    }
    const int h = hk * G + g;
    ((uint2*)cl)[lane] = make_uint2(0u, 0u);  // MAXC = 256 bytes
    __syncwarp();
    {
      // both counts are read before either index list (two round trips to memory, not four)
      const int bm = p.t.mB == 1 ? 0 : b, hm = p.t.mH == 1 ? 0 : h;
      const int kvblk = min(kt * BT / p.t.KVB, p.t.nKV - 1);
      const long long row = ((long long)bm * p.t.mH + hm) * p.t.nKV + kvblk;
      const int tpb = p.t.nQ == 1 ? n_ctiles : p.t.QB / 128;
      int num[2];
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const int* nump = which ? p.t.full_q_num : p.t.q_num;
        num[which] = nump != nullptr ? min(max(nump[row], 0), p.t.nQ) * tpb : 0;
      }
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const int* idxp = which ? p.t.full_q_idx : p.t.q_idx;
        for (int e = lane; e < num[which]; e += 32) {
          const int bi = e / tpb, ti = e - bi * tpb;
          const int t = min(max(idxp[row * p.t.nQ + bi], 0), p.t.nQ - 1) * tpb + ti;
          if (t < n_ctiles) cl[t] = (unsigned char)(which ? 2 : 1);
        }
        __syncwarp();
      }
    }
    for (int t0 = 0; t0 < n_ctiles; t0 += 32) {
      const int t = t0 + lane;
      const int c = t < n_ctiles ? (int)cl[t] : 0;
      int n_t = 0;
      if (c != 0)
        for (int v = 0; v < PPT; ++v) n_t += (t * PPT + v) * BQ < p.Sq ? 1 : 0;
      int inc = n_t;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += o;
      }
      for (int v = 0; v < n_t; ++v)
        if (w + inc - n_t + v < MAXPL) pl[w + inc - n_t + v] = (t * PPT + v) | (c << 16) | (g << 20);
      w += __shfl_sync(0xffffffffu, inc, 31);
    }
    __syncwarp();
  }
  return min(w, MAXPL);
}

}  // namespace fa_btc

extern "C" __global__ void __launch_bounds__(fa_btc::NT, 1) fa_bwd_tc_kernel(const __grid_constant__ FaBwdTcParams P) {
  using namespace fa_btc;
  const FaParams& p = P.p;
  extern __shared__ unsigned char smem_raw[];
  // a launch that does not fit the shared-memory map above (a host library built for another
  // version of this file) is refused before anything is written
  if (fa_dynamic_smem_size() < (fa_u32)SMEM_BYTES || blockDim.x != NT) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicOr(p.status, FA_STATUS_BAD_LAUNCH);
    return;
  }
  const fa_u32 raw = fa_smem_u32(smem_raw);
  const fa_u32 sb = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_raw + (sb - raw);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.Hq / p.Hkv;
  const int n_ctiles = min((p.Sq + 127) / 128, MAXC);  // 128-row q tiles (the grain of the BlockMask walk)
  const int sq_pad = ((p.Sq + 127) / 128) * 128;
  const int n_kvt = (p.Skv + BT - 1) / BT;
  const int n_items = p.Hkv * p.B * n_kvt;
  const int Gd = (int)gridDim.x, cta = (int)blockIdx.x;

  volatile int* misc = (volatile int*)(sm + OFF_MISC);  // [0] tmem base, [1] abort, [2] unused, [3] drain warps leave
  int* pairs = (int*)(sm + OFF_PAIR);                   // two lists of MAXPL pairs
  volatile int* item = (volatile int*)(sm + OFF_ITEM);  // per list: item number, pairs

  // An item is the 128-row kv tile of one (batch, kv head); items are numbered with the head
  // fastest and the kv tile slowest (under a causal mask the heaviest come first).  The kernel is
  // persistent: CTA c starts with item c and takes further items from a counter in global memory,
  // so TMEM, the barriers and the descriptors are set up once per CTA, the loads of an item run
  // under the tail of the one before, and the CTAs stay level whatever the mask does to the work
  // per item.  The producer warp builds the pair list of the next item (two lists in shared
  // memory) while the others work on the current one.

  // ---- set-up --------------------------------------------------------------------------------
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      fa_mbar_init(bar_addr(sb, BAR_KV + i), 1);
      fa_mbar_init(bar_addr(sb, BAR_FINAL + i), 2);  // products 3-4 and product 5 of an item's last pair
      fa_mbar_init(bar_addr(sb, BAR_KVFREE + i), 1);
    }
    for (int s = 0; s < NSTAGE; ++s) {
      fa_mbar_init(bar_addr(sb, BAR_QFULL + s), 1);
      fa_mbar_init(bar_addr(sb, BAR_QEMPTY + s), 2);  // one arrival from each MMA issuer
      fa_mbar_init(bar_addr(sb, BAR_DOEMPTY + s), 2);
    }
    fa_mbar_init(bar_addr(sb, BAR_SFULL), 1);
    fa_mbar_init(bar_addr(sb, BAR_SFREE), 256);
    fa_mbar_init(bar_addr(sb, BAR_PREADY), 256);
    fa_mbar_init(bar_addr(sb, BAR_PFREE), 2);  // one arrival from each of the issuers of products 3-4 and 5
    fa_mbar_init(bar_addr(sb, BAR_DQFULL), 1);
    fa_mbar_init(bar_addr(sb, BAR_DQFREE), 128);
    fa_mbar_init(bar_addr(sb, BAR_DKVFREE), 128);
    for (int i = 0; i < 2; ++i) {
      fa_mbar_init(bar_addr(sb, BAR_LISTFULL + i), 1);
      fa_mbar_init(bar_addr(sb, BAR_LISTFREE + i), LIST_CONSUMERS);
    }
    fa_mbar_init_fence();
    misc[1] = 0;
    misc[2] = 0;
    misc[3] = 0;
    fa_tma_prefetch_desc(&P.tk);
    fa_tma_prefetch_desc(&P.tv);
    fa_tma_prefetch_desc(&P.tq);
    fa_tma_prefetch_desc(&P.tdo);
  }
  if (warp == WARP_MMA) fa_tmem_alloc(sb + OFF_MISC, TMEM_COLS);
  fa_tc_fence_before();
  __syncthreads();
  fa_tc_fence_after();
  const fa_u32 tmem = (fa_u32)misc[0];
  volatile int* abort_flag = misc + 1;
  // a copy the compiler can see is the same in every lane (read through a broadcast)
  const fa_u32 tmem_u = __shfl_sync(0xffffffffu, tmem, 0);

  if (warp >= 8) fa_setmaxnreg_dec<REGS_OTHER>();

  // Barrier phases: the pair-indexed barriers count the pairs of the CTA across its items (gn);
  // BAR_KV, BAR_FINAL and BAR_DKVFREE count the items that have pairs (kvc) - an item without
  // pairs loads no K / V and only has zeros written; the list barriers count all items (itc).
  if (warp == WARP_PRODUCER) {
    // ================================ producer ================================================
    // The whole warp builds the lists; lane 0 issues the loads.
    bool ok = true;
    int gn = 0, kvc = 0;
    int idx = cta;
    for (int itc = 0; ok; ++itc) {
      const int lb = itc & 1;
      // the consumers of the list that was in this buffer two items ago must be done with it
      if (itc >= 2) ok = fa_mbar_wait_warp(bar_addr(sb, BAR_LISTFREE + lb), (fa_u32)(((itc >> 1) - 1) & 1), abort_flag);
      if (!ok) break;
      int* pl = pairs + lb * MAXPL;
      const int hk = idx % p.Hkv, b = (idx / p.Hkv) % p.B, kt = idx / (p.Hkv * p.B);
      int np = -1;
      if (idx < n_items) np = build_pair_list(p, hk, b, kt, G, n_ctiles, sm + OFF_CLS, pl, lane);
      if (lane == 0) {
        item[2 * lb] = idx;
        item[2 * lb + 1] = np;
      }
      __syncwarp();
      if (lane == 0) fa_mbar_arrive(bar_addr(sb, BAR_LISTFULL + lb));
      if (np < 0) break;
      int next = 0;
      if (lane == 0) {
        // the next item is asked for now: the answer is not needed before this item's loads are out
        next = Gd + atomicAdd(P.work_counter, 1);
        const int n0 = kt * BT;
        // The K / V buffers are free once the last products of the previous item are complete;
        // the Q / dO slots of the item's first pairs free up earlier, so those loads go first.
        const int kb = kvc % KVBUF, use = kvc / KVBUF;
        const int kvpos = (KVBUF == 2 || kvc == 0) ? 0 : min(NSTAGE, np) - 1;
        for (int n = 0; n < np && ok; ++n, ++gn) {
          if (n == kvpos) {
            if (use > 0) ok = fa_mbar_wait(bar_addr(sb, (KVBUF == 2 ? BAR_KVFREE : BAR_FINAL) + kb), (fa_u32)((use - 1) & 1), abort_flag);
            if (!ok) break;
            const fa_u32 full = bar_addr(sb, BAR_KV + kb);
            fa_mbar_expect_tx(full, 2 * KV_BYTES);
            for (int a = 0; a < DATOMS; ++a) {
              fa_tma_load_4d(sb + OFF_K + kb * KV_BYTES + a * ATOM_BYTES, &P.tk, full, a * 64, n0, hk, b);
              fa_tma_load_4d(sb + OFF_V + kb * KV_BYTES + a * ATOM_BYTES, &P.tv, full, a * 64, n0, hk, b);
            }
          }
          const int s = gn % NSTAGE;
          const fa_u32 ph = (fa_u32)((gn / NSTAGE) & 1);
          const int pr = pl[n];
          const int m0 = (pr & 0xffff) * BQ, h = hk * G + (pr >> 20);
          if (gn >= NSTAGE) ok = fa_mbar_wait(bar_addr(sb, BAR_DOEMPTY + s), ph ^ 1u, abort_flag);
          if (!ok) break;
          // Q and dO tiles plus the per-row scalars of the q tile (prepared by fa_bwd_prep_kernel);
          // one transaction count covers all the copies
          const long long rbase = ((long long)b * p.Hq + h) * sq_pad + m0;
          const fa_u32 full = bar_addr(sb, BAR_QFULL + s);
          fa_mbar_expect_tx(full, 2 * Q_BYTES + 2 * BQ * 4);
          for (int a = 0; a < DATOMS; ++a)
            fa_tma_load_4d(sb + OFF_DO + s * Q_BYTES + a * Q_ATOM_BYTES, &P.tdo, full, a * 64, m0, h, b);
          if (gn >= NSTAGE) ok = fa_mbar_wait(bar_addr(sb, BAR_QEMPTY + s), ph ^ 1u, abort_flag);
          if (!ok) break;
          for (int a = 0; a < DATOMS; ++a)
            fa_tma_load_4d(sb + OFF_Q + s * Q_BYTES + a * Q_ATOM_BYTES, &P.tq, full, a * 64, m0, h, b);
          fa_bulk_load(sb + OFF_ROW + s * 2 * BQ * 4, P.nlse2 + rbase, BQ * 4, full);
          fa_bulk_load(sb + OFF_ROW + s * 2 * BQ * 4 + BQ * 4, P.ndelta + rbase, BQ * 4, full);
        }
        // K and V of the next item are asked into L2 now; their loads can only start when this
        // item is complete, and then they find the tiles close by
        if (KVBUF == 1 && ok && next < n_items) {
          const int hk2 = next % p.Hkv, b2 = (next / p.Hkv) % p.B, n2 = (next / (p.Hkv * p.B)) * BT;
          for (int a = 0; a < DATOMS; ++a) {
            tma_prefetch_l2_4d(&P.tk, a * 64, n2, hk2, b2);
            tma_prefetch_l2_4d(&P.tv, a * 64, n2, hk2, b2);
          }
        }
      }
      if (np > 0) ++kvc;
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      gn = __shfl_sync(0xffffffffu, gn, 0);
      idx = __shfl_sync(0xffffffffu, next, 0);
    }
  } else if (warp == WARP_MMA) {
    // ================================ MMA issuer A: products 1-2 ===============================
    // (several issuing warps, so that the waits of one overlap the issue of the other; warp A also
    //  owns the TMEM allocation).  The whole warp runs the loop and one elected lane issues: with
    //  uniform control flow the descriptors live in uniform registers, which makes each
    //  tcgen05.mma cheaper to issue than from a single-lane branch, and the issue rate of this
    //  one thread is what bounds the tensor core here.
    const bool leader = fa_elect_one();
    constexpr fa_u32 IDESC_KK = fa_idesc(DT, 128, BQ, 0, 0);  // A, B K-major, N = BQ
    constexpr fa_u32 HI = fa_desc_hi_sw128();
    bool ok = true;
    int gn = 0, kvc = 0;
    for (int itc = 0; ok; ++itc) {
      const int lb = itc & 1;
      ok = fa_mbar_wait_all(bar_addr(sb, BAR_LISTFULL + lb), (fa_u32)((itc >> 1) & 1), abort_flag);
      if (!ok) break;
      const int np = __shfl_sync(0xffffffffu, item[2 * lb + 1], 0);
      if (leader) fa_mbar_arrive(bar_addr(sb, BAR_LISTFREE + lb));  // (the issuers need the count only)
      if (np < 0) break;
      if (np == 0) continue;
      const int kb = kvc % KVBUF;
      const fa_u32 loK_k = fa_desc_lo(sb + OFF_K + kb * KV_BYTES, 16), loV_k = fa_desc_lo(sb + OFF_V + kb * KV_BYTES, 16);
      ok = fa_mbar_wait_all(bar_addr(sb, BAR_KV + kb), (fa_u32)((kvc / KVBUF) & 1), abort_flag);
      for (int n = 0; n < np && ok; ++n, ++gn) {
        const int s = gn % NSTAGE;
        ok = fa_mbar_wait_all(bar_addr(sb, BAR_QFULL + s), (fa_u32)((gn / NSTAGE) & 1), abort_flag);
        if (ok && gn > 0) ok = fa_mbar_wait_all(bar_addr(sb, BAR_SFREE), (fa_u32)((gn - 1) & 1), abort_flag);
        if (!ok) break;
        fa_tc_fence_after();
        const fa_u32 loQ = fa_desc_lo(sb + OFF_Q + s * Q_BYTES, 16), loDO = fa_desc_lo(sb + OFF_DO + s * Q_BYTES, 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          if (leader)
            fa_mma_ss(tmem_u + COL_S, fa_desc_make(loK_k + kstep_kmajor(kk, ATOM_BYTES), HI),
                      fa_desc_make(loQ + kstep_kmajor(kk, Q_ATOM_BYTES), HI), IDESC_KK, kk > 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          if (leader)
            fa_mma_ss(tmem_u + COL_DP, fa_desc_make(loV_k + kstep_kmajor(kk, ATOM_BYTES), HI),
                      fa_desc_make(loDO + kstep_kmajor(kk, Q_ATOM_BYTES), HI), IDESC_KK, kk > 0);
        if (leader) {
          fa_mma_commit(bar_addr(sb, BAR_SFULL));
          fa_mma_commit(bar_addr(sb, BAR_QEMPTY + s));  // first of the two arrivals that free each tile of the stage
          fa_mma_commit(bar_addr(sb, BAR_DOEMPTY + s));
        }
      }
      ++kvc;
    }
  } else if (warp == WARP_MMA_B) {
    // ================================ MMA issuer B: products 3-4 ===============================
    const bool leader = fa_elect_one();
    constexpr fa_u32 IDESC_TN = fa_idesc(DT, 128, D, 0, 1);    // A K-major (TMEM or smem), B MN-major, N = D
    constexpr fa_u32 HI = fa_desc_hi_sw128();
    const fa_u32 loDS_k = fa_desc_lo(sb + OFF_DS, 16);
    bool ok = true;
    int gn = 0, kvc = 0;
    for (int itc = 0; ok; ++itc) {
      const int lb = itc & 1;
      ok = fa_mbar_wait_all(bar_addr(sb, BAR_LISTFULL + lb), (fa_u32)((itc >> 1) & 1), abort_flag);
      if (!ok) break;
      const int np = __shfl_sync(0xffffffffu, item[2 * lb + 1], 0);
      if (leader) fa_mbar_arrive(bar_addr(sb, BAR_LISTFREE + lb));
      if (np < 0) break;
      if (np == 0) continue;
      for (int n = 0; n < np && ok; ++n, ++gn) {
        const int s = gn % NSTAGE;
        ok = fa_mbar_wait_all(bar_addr(sb, BAR_PREADY), (fa_u32)(gn & 1), abort_flag);
        // the first products of an item overwrite dV and dK: the drain warps must have read the
        // previous item's out of TMEM
        if (ok && n == 0 && kvc > 0) ok = fa_mbar_wait_all(bar_addr(sb, BAR_DKVFREE), (fa_u32)((kvc - 1) & 1), abort_flag);
        if (!ok) break;
        fa_tc_fence_after();
        // B operands read MN-major: the D columns are 64-element groups Q_ATOM_BYTES apart, a
        // k-step is 16 q rows = 2048 bytes
        const fa_u32 loQ_mn = fa_desc_lo(sb + OFF_Q + s * Q_BYTES, Q_ATOM_BYTES);
        const fa_u32 loDO_mn = fa_desc_lo(sb + OFF_DO + s * Q_BYTES, Q_ATOM_BYTES);
        const fa_u32 acc = n > 0;  // the first pair of an item starts its dK and dV
        // 3. dV += P^T dO      (K = BQ q values; A from TMEM)
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk)
          if (leader) fa_mma_ts(tmem_u + COL_DV, tmem_u + COL_P + kk * 8, fa_desc_make(loDO_mn + kk * 128, HI), IDESC_TN, acc | (kk > 0));
        if (leader) fa_mma_commit(bar_addr(sb, BAR_DOEMPTY + s));  // second arrival: the dO tile is free
        // 4. dK += dS^T Q     (A = dS^T K-major: k-step kk is 32 bytes into atom kk / 4)
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk)
          if (leader)
            fa_mma_ss(tmem_u + COL_DK, fa_desc_make(loDS_k + kstep_kmajor(kk, ATOM_BYTES), HI),
                      fa_desc_make(loQ_mn + kk * 128, HI), IDESC_TN, acc | (kk > 0));
        if (leader) {
          fa_mma_commit(bar_addr(sb, BAR_QEMPTY + s));   // second arrival: the Q tile and row scalars are free
          fa_mma_commit(bar_addr(sb, BAR_PFREE));        // one of the two arrivals that free P^T and dS^T
          if (n + 1 == np) fa_mma_commit(bar_addr(sb, BAR_FINAL + kvc % KVBUF));
        }
      }
      ++kvc;
    }
  } else if (warp == WARP_MMA_C) {
    // ================================ MMA issuer C: product 5 ==================================
    // (a third issuing warp: what bounds the tensor core in this kernel is how fast one thread
    //  can issue, so the instructions of a pair are spread over three threads)
    const bool leader = fa_elect_one();
    constexpr fa_u32 IDESC_NN = fa_idesc(DT, 128, 64, 1, 1);    // A, B MN-major, M = 128, N = 64
    constexpr fa_u32 HI = fa_desc_hi_sw128();
    const fa_u32 loDS_mn = fa_desc_lo(sb + OFF_DS, ATOM_BYTES);
    bool ok = true;
    int gn = 0, kvc = 0;
    for (int itc = 0; ok; ++itc) {
      const int lb = itc & 1;
      ok = fa_mbar_wait_all(bar_addr(sb, BAR_LISTFULL + lb), (fa_u32)((itc >> 1) & 1), abort_flag);
      if (!ok) break;
      const int np = __shfl_sync(0xffffffffu, item[2 * lb + 1], 0);
      if (leader) fa_mbar_arrive(bar_addr(sb, BAR_LISTFREE + lb));
      if (np < 0) break;
      if (np == 0) continue;
      const int kb = kvc % KVBUF;
      const fa_u32 loK_mn = fa_desc_lo(sb + OFF_K + kb * KV_BYTES, ATOM_BYTES);
      ok = fa_mbar_wait_all(bar_addr(sb, BAR_KV + kb), (fa_u32)((kvc / KVBUF) & 1), abort_flag);
      for (int n = 0; n < np && ok; ++n, ++gn) {
        ok = fa_mbar_wait_all(bar_addr(sb, BAR_PREADY), (fa_u32)(gn & 1), abort_flag);
        // the drain warps must have emptied the dQ columns of the previous pair
        if (ok && gn > 0) ok = fa_mbar_wait_all(bar_addr(sb, BAR_DQFREE), (fa_u32)((gn - 1) & 1), abort_flag);
        if (!ok) break;
        fa_tc_fence_after();
        // 5. K = 128 kv rows, a k-step is 16 rows = 2048 bytes of either operand.
        //    D = 64:  dQ = dS K       A = dS^T read MN-major (M = 128 q: two 64-column atoms), B = K (N = 64 d)
        //    D = 128: dQ^T = K^T dS^T A = K read MN-major (M = 128 d: two atoms), B = dS^T (N = 64 q)
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)
          if (leader) {
            if (D == 64)
              fa_mma_ss(tmem_u + COL_DQ, fa_desc_make(loDS_mn + kk * 128, HI), fa_desc_make(loK_mn + kk * 128, HI), IDESC_NN, kk > 0);
            else
              fa_mma_ss(tmem_u + COL_DQ, fa_desc_make(loK_mn + kk * 128, HI), fa_desc_make(loDS_mn + kk * 128, HI), IDESC_NN, kk > 0);
          }
        if (leader) {
          fa_mma_commit(bar_addr(sb, BAR_PFREE));
          fa_mma_commit(bar_addr(sb, BAR_DQFULL));
          if (n + 1 == np) fa_mma_commit(bar_addr(sb, BAR_FINAL + kb));  // (this product is the last reader of K)
        }
      }
      ++kvc;
    }
  } else if (warp < 8) {
    // ================================ compute warps ============================================
    fa_setmaxnreg_inc<REGS_COMPUTE>();
    const int half = warp >> 2;               // q columns CW*half .. +CW-1 of the pair tile
    const int lane_base = (warp & 3) * 32;
    const int r = lane_base + lane;           // kv row of this thread inside the tile
    const fa_u32 t_row = tmem + ((fa_u32)lane_base << 16);
    const float sc2 = p.scale * FA_LOG2E;
    bool ok = true;
    int gn = 0;
    for (int itc = 0; ok; ++itc) {
      const int lb = itc & 1;
      ok = fa_mbar_wait_warp(bar_addr(sb, BAR_LISTFULL + lb), (fa_u32)((itc >> 1) & 1), abort_flag);
      if (!ok) break;
      const int idx = item[2 * lb], np = item[2 * lb + 1];
      if (np < 0) break;
      const int* pl = pairs + lb * MAXPL;
      const int hk = idx % p.Hkv, b = (idx / p.Hkv) % p.B, n0 = (idx / (p.Hkv * p.B)) * BT;
      const int gb = b + p.b_off;
      const int kv = n0 + r;
      const bool row_ok = kv < p.Skv;
      for (int n = 0; n < np && ok; ++n, ++gn) {
        const int s = gn % NSTAGE;
        const int pr = pl[n];
        const int m0 = (pr & 0xffff) * BQ, mode = (pr >> 16) & 0xf, gh = hk * G + (pr >> 20) + p.h_off;
        ok = fa_mbar_wait_warp(bar_addr(sb, BAR_SFULL), (fa_u32)(gn & 1), abort_flag);
        if (ok) ok = fa_mbar_wait_warp(bar_addr(sb, BAR_QFULL + s), (fa_u32)((gn / NSTAGE) & 1), abort_flag);
        if (!ok) break;
        fa_tc_fence_after();
        const float* rowp = (const float*)(sm + OFF_ROW + s * 2 * BQ * 4);
        fa_u32 pp[CW / 2], ds[CW / 2];
        // The CW columns of this thread come in steps of 16 (S^T and dP^T), the loads of a step in
        // flight while the previous one is computed: few values are live at a time, which leaves
        // the scheduler registers to overlap the latencies of independent elements (with all the
        // values loaded up front this loop ran at 28 clocks per element).
        {
          const fa_u32 tS = t_row + COL_S + half * CW, tD = t_row + COL_DP + half * CW;
          const int c0 = half * CW;  // first q column of this thread inside the tile
          float sA[16], dA[16], sB[16], dB[16];
          fa_u32 p8[8], d8[8];
          fa_tmem_ld16(tS, sA);
          fa_tmem_ld16(tD, dA);
          fa_tmem_wait_ld();
#define FA_STEP(SC, DC, SN, DN, C, LAST)                                                                   \
  if (!(LAST)) {                                                                                           \
    fa_tmem_ld16(tS + (C) + 16, SN);                                                                       \
    fa_tmem_ld16(tD + (C) + 16, DN);                                                                       \
  } else {                                                                                                 \
    /* every score of the pair is in registers: the S^T / dP^T columns may be overwritten */              \
    fa_tc_fence_before();                                                                                  \
    fa_mbar_arrive(bar_addr(sb, BAR_SFREE));                                                               \
  }                                                                                                        \
  if (row_ok) {                                                                                            \
    chunk<16>(SC, DC, rowp + c0 + (C), rowp + BQ + c0 + (C), p8, d8, mode, m0 + c0 + (C), kv, gb, gh, p.scale, sc2); \
  } else {                                                                                                 \
    _Pragma("unroll") for (int e = 0; e < 8; ++e) p8[e] = d8[e] = 0u;                                      \
  }                                                                                                        \
  _Pragma("unroll") for (int e = 0; e < 8; ++e) {                                                          \
    pp[(C) / 2 + e] = p8[e];                                                                               \
    ds[(C) / 2 + e] = d8[e];                                                                               \
  }                                                                                                        \
  if (!(LAST)) fa_tmem_wait_ld();
          if (CW == 64) {
            FA_STEP(sA, dA, sB, dB, 0, false)
            FA_STEP(sB, dB, sA, dA, 16, false)
            FA_STEP(sA, dA, sB, dB, 32 % CW, false)
            FA_STEP(sB, dB, sA, dA, 48 % CW, true)
          } else {
            FA_STEP(sA, dA, sB, dB, 0, false)
            FA_STEP(sB, dB, sA, dA, 16, true)
          }
#undef FA_STEP
        }
        // pin the packed results here: without this the compiler sinks part of the math below the
        // wait that follows, onto the critical path between two groups of products
#pragma unroll
        for (int e = 0; e < CW / 2; ++e) asm volatile("" : "+r"(pp[e]), "+r"(ds[e]));
        // products 3-5 of the previous pair must be done with P^T and dS^T
        if (gn > 0) {
          ok = fa_mbar_wait_warp(bar_addr(sb, BAR_PFREE), (fa_u32)((gn - 1) & 1), abort_flag);
          if (!ok) break;
          fa_tc_fence_after();
        }
#pragma unroll
        for (int i = 0; i < CW / 32; ++i)
          fa_tmem_st16(t_row + COL_P + half * (CW / 2) + 16 * i, *(const fa_u32(*)[16])(pp + 16 * i));
        {
          // dS^T row r: this thread's CW columns are CW / 8 sixteen-byte chunks; chunk ck of a 128-byte
          // atom row goes to position ck ^ (r & 7) (the 128-byte swizzle of the operand layout)
#pragma unroll
          for (int c = 0; c < CW / 8; ++c) {
            const int col = half * CW + 8 * c;
            unsigned char* dsrow = sm + OFF_DS + (col >> 6) * ATOM_BYTES + r * 128;
            uint4 w;
            w.x = ds[4 * c]; w.y = ds[4 * c + 1]; w.z = ds[4 * c + 2]; w.w = ds[4 * c + 3];
            *(uint4*)(dsrow + ((((col & 63) >> 3) ^ (r & 7)) * 16)) = w;
          }
        }
        fa_tmem_wait_st();
        fence_proxy_async();
        fa_tc_fence_before();
        fa_mbar_arrive(bar_addr(sb, BAR_PREADY));
      }
      if (!ok) break;
      // every lane has read its last list entry: the list may be overwritten
      __syncwarp();
      if (lane == 0) fa_mbar_arrive(bar_addr(sb, BAR_LISTFREE + lb));
    }
  } else if (warp < 12) {
    // ================================ drain warps: dQ of every pair, dK / dV of every item =======
    const int lane_base = (warp & 3) * 32;
    const int r = lane_base + lane;  // TMEM lane: q row of the pair (D = 64) or head-dim index (D = 128); kv row for dK / dV
    const fa_u32 t_lane = tmem + ((fa_u32)lane_base << 16);
    const fa_u32 t_dq = t_lane + COL_DQ;
    const int dtid = tid - 256;
    const int n_qtiles = sq_pad / BQ;
    bool ok = true;
    int gn = 0, kvc = 0;
    for (int itc = 0; ok; ++itc) {
      const int lb = itc & 1;
      // The four drain warps meet at named barriers, so they have to leave their loops together: a
      // warp whose wait failed says so in a flag only the drain warps write, joins the next named
      // barrier like the others, and all four read the flag behind that barrier.
      ok = fa_mbar_wait_warp(bar_addr(sb, BAR_LISTFULL + lb), (fa_u32)((itc >> 1) & 1), abort_flag);
      if (!ok) misc[3] = 1;
      named_bar_sync(1, 128);
      if (misc[3] != 0) {
        ok = false;
        break;
      }
      const int idx = item[2 * lb], np = item[2 * lb + 1];
      if (np < 0) break;  // (the same in all four warps)
      const int* pl = pairs + lb * MAXPL;
      const int hk = idx % p.Hkv, b = (idx / p.Hkv) % p.B, n0 = (idx / (p.Hkv * p.B)) * BT;
      for (int n = 0; n < np && ok; ++n, ++gn) {
        const int pr = pl[n];
        const int qt = pr & 0xffff, h = hk * G + (pr >> 20);
        ok = fa_mbar_wait_warp(bar_addr(sb, BAR_DQFULL), (fa_u32)(gn & 1), abort_flag);
        if (!ok) misc[3] = 1;  // (read by all four warps behind the first barrier of the pair)
        fa_tc_fence_after();
        // The 128 x 64 fp32 tile leaves in two halves of 32 columns through one 16 KB staging buffer:
        // each half is one contiguous 16 KB block of the accumulation buffer.  16-byte chunk k of
        // lane r goes to position k ^ (r & 7), which spreads the rows of a warp over the banks.
        float* gdst = P.dq_acc + (((long long)b * p.Hq + h) * n_qtiles + qt) * (128 * 64);
        unsigned char* strow = sm + OFF_DQ + r * 128;
        float a[32];
        if (ok) {
          fa_tmem_ld32(t_dq, a);
          fa_tmem_wait_ld();
        }
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          // the previous bulk reduce must have finished reading the staging buffer
          if (dtid == 0) bulk_wait_read0();
          named_bar_sync(1, 128);
          if (hf == 0 && misc[3] != 0) {
            ok = false;
            break;
          }
#pragma unroll
          for (int k = 0; k < 8; ++k)
            *(float4*)(strow + ((k ^ (r & 7)) * 16)) = make_float4(a[4 * k], a[4 * k + 1], a[4 * k + 2], a[4 * k + 3]);
          if (hf == 0) {
            fa_tmem_ld32(t_dq + 32, a);
            fa_tmem_wait_ld();
            fa_tc_fence_before();
            fa_mbar_arrive(bar_addr(sb, BAR_DQFREE));
          }
          fence_proxy_async();
          named_bar_sync(1, 128);
          if (dtid == 0) {
            bulk_reduce_add_f32(gdst + hf * (DQ_HALF_BYTES / 4), sb + OFF_DQ, DQ_HALF_BYTES);
            bulk_commit();
          }
        }
      }
      if (!ok) break;
      // ---- dK (scaled) and dV of the item.  A thread owns one kv row (TMEM lane); 64 columns at a
      // time are converted into the staging buffer in the layout of a K tile (128-byte rows, 16-byte
      // chunk k of row r at k ^ (r & 7)) and leave through one tensor-map store, which writes whole
      // lines and clips the rows beyond Skv.  (Each thread storing its own row straight to global
      // memory took several thousand cycles per item: 32 different lines per instruction.)
      // An item without pairs has zeros written.
      if (np > 0) {
        const int kb = kvc % KVBUF;
        ok = fa_mbar_wait_warp(bar_addr(sb, BAR_FINAL + kb), (fa_u32)((kvc / KVBUF) & 1), abort_flag);
        if (!ok) misc[3] = 1;
        named_bar_sync(1, 128);
        if (misc[3] != 0) {
          ok = false;
          break;
        }
        fa_tc_fence_after();
#pragma unroll 1
        for (int part = 0; part < 2 * DATOMS; ++part) {
          const int which = part / DATOMS, a = part - which * DATOMS;  // dK atoms first, then dV
          const float mul = which == 0 ? p.scale : 1.f;
          // two K / V buffers: the staging buffers are the item's own K and V tiles, which nothing reads
          // any more; one: the parts go through the dQ staging buffer one after the other
          const int st_off = KVBUF == 2 ? (which == 0 ? OFF_K : OFF_V) + kb * KV_BYTES + a * ATOM_BYTES : OFF_DQ;
          unsigned char* strow = sm + st_off + r * 128;
          if (KVBUF == 1) {
            // the previous bulk operation must have finished reading the staging buffer
            if (dtid == 0) bulk_wait_read0();
            named_bar_sync(1, 128);
          }
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float o[16];
            fa_tmem_ld16(t_lane + (which == 0 ? COL_DK : COL_DV) + a * 64 + c * 16, o);
            fa_tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; e += 8) {
              uint4 w;
              w.x = fa_pack2<DT>(o[e] * mul, o[e + 1] * mul);
              w.y = fa_pack2<DT>(o[e + 2] * mul, o[e + 3] * mul);
              w.z = fa_pack2<DT>(o[e + 4] * mul, o[e + 5] * mul);
              w.w = fa_pack2<DT>(o[e + 6] * mul, o[e + 7] * mul);
              *(uint4*)(strow + (((2 * c + (e >> 3)) ^ (r & 7)) * 16)) = w;
            }
          }
          if (part == 2 * DATOMS - 1) {
            // dK and dV are out of TMEM: the next item's first products may overwrite them
            fa_tc_fence_before();
            fa_mbar_arrive(bar_addr(sb, BAR_DKVFREE));
          }
          if (KVBUF == 1 || part == 2 * DATOMS - 1) {
            fence_proxy_async();
            named_bar_sync(1, 128);
          }
          if (dtid == 0) {
            if (KVBUF == 1) {
              fa_tma_store_4d(which == 0 ? &P.tdk : &P.tdv, sb + OFF_DQ, a * 64, n0, hk, b);
              bulk_commit();
            } else if (part == 2 * DATOMS - 1) {
              for (int a2 = 0; a2 < DATOMS; ++a2) {
                fa_tma_store_4d(&P.tdk, sb + OFF_K + kb * KV_BYTES + a2 * ATOM_BYTES, a2 * 64, n0, hk, b);
                fa_tma_store_4d(&P.tdv, sb + OFF_V + kb * KV_BYTES + a2 * ATOM_BYTES, a2 * 64, n0, hk, b);
              }
              bulk_commit();
              bulk_wait_read0();
              fa_mbar_arrive(bar_addr(sb, BAR_KVFREE + kb));
            }
          }
        }
      } else {
        // an item without pairs: zeros, straight from the registers (rare; a row per thread)
        const int kv = n0 + r;
        if (kv < p.Skv) {
#pragma unroll
          for (int which = 0; which < 2; ++which) {
            const FaTensor& dst = which == 0 ? p.dk : p.dv;
            char* og = (char*)dst.ptr + ((long long)b * dst.sb + (long long)hk * dst.sh + (long long)kv * dst.ss) * 2;
            for (int c = 0; c < D / 8; ++c) *(uint4*)(og + c * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
      if (np > 0) ++kvc;
      __syncwarp();
      if (lane == 0) fa_mbar_arrive(bar_addr(sb, BAR_LISTFREE + lb));
    }
    if (dtid == 0) bulk_wait0();
  }

  // ---- teardown ------------------------------------------------------------------------------
  fa_tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    fa_tc_fence_after();
    fa_tmem_dealloc(tmem, TMEM_COLS);
  }
  if (tid == 0 && *abort_flag != 0 && p.status != nullptr) atomicOr(p.status, FA_STATUS_WAIT_TIMEOUT);
}
