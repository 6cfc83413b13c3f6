// Flash-attention backward, general tile kernels (same coverage as fa_fwd.cuh).
// Replaces mha_backward_kernel of flaxattention/kernel/attention.py:372-553, which does a
// dK/dV scan (:423-478) and a dQ scan (:486-553) in one program over all tiles.  Here the
// two scans are two kernels, each walking only the blocks its BlockMask tables list:
//   fa_bwd_dkdv_kernel  one CTA per kv tile, q tiles from the q tables, transposed products
//                       (S^T = K Q^T) so that the dK / dV accumulators stay in registers;
//                       with GQA the CTA also loops over the query heads of its kv head;
//   fa_bwd_dq_kernel    one CTA per q tile, kv tiles from the kv tables.
// Math (natural units; lse and delta = rowsum(O * dO) are inputs):
//   s = (q.k) * scale, t = score_mod(s), p = exp(t - lse) (0 where masked),
//   dV = P^T dO, dP = dO V^T, dS = p * (dP - delta) * score_mod'(s),
//   dQ = scale * dS K, dK = scale * dS^T Q.
//
// Compile-time parameters (macros): FA_DTYPE, FA_D, FA_DV, FA_BQ, FA_BK, FA_WARPS.
// FA_BQ = 16 * FA_WARPS rows per q-tile CTA (dq kernel) and FA_BK = 16 * FA_WARPS rows per
// kv-tile CTA (dkdv kernel); the inner tile is FA_BK resp. FA_BQ wide.
#pragma once
#include "fa_common.cuh"

namespace fa_bwd {

constexpr int DT = FA_DTYPE;
constexpr int D = FA_D;
constexpr int DV = FA_DV;
constexpr int BQ = FA_BQ;
constexpr int BK = FA_BK;
constexpr int NWARPS = FA_WARPS;
constexpr int NT = NWARPS * 32;
constexpr int ES = DT == FA_DT_F32 ? 4 : 2;
constexpr bool F32 = DT == FA_DT_F32;
constexpr int PQ = FaTile<D, ES>::PITCH;
constexpr int PV = FaTile<DV, ES>::PITCH;
constexpr bool A_IN_REGS = !F32 && D <= 64;

static_assert(BQ == 16 * NWARPS && BK == 16 * NWARPS, "one m16 row tile per warp");

// probability and score_mod derivative of one score element
__device__ __forceinline__ void elem(float sraw, float scale, int gb, int gh, int qi, int kv, bool masked_tile,
                                     bool in_range, float lse2, float& p, float& g) {
  const float x = sraw * scale;
  float t = x;
#if FA_HAS_SCORE_MOD
  t = fa_score_mod(x, gb, gh, qi, kv);
  g = fa_score_mod_grad(x, gb, gh, qi, kv);
#else
  g = 1.f;
#endif
  bool keep = in_range;
#if FA_HAS_MASK_MOD
  if (masked_tile) keep = keep && fa_mask_mod(gb, gh, qi, kv);
#endif
  keep = keep && (lse2 != FA_NEG_INF);
  if (F32) p = keep ? exp2f(t * FA_LOG2E - lse2) : 0.f;
  else p = keep ? fa_ex2(t * FA_LOG2E - lse2) : 0.f;
  if (!keep) g = 0.f;
}

}  // namespace fa_bwd

// ======================================================================================
// dQ
// ======================================================================================
namespace fa_bwd {
constexpr int PPK = FaTile<BK, 4>::PITCH;  // fp32 staging tile [BQ][BK] (fp32 path)
constexpr int DQ_SMEM = BQ * PQ + BQ * PV + 2 * BK * PQ + 2 * BK * PV + (F32 ? BQ * PPK : 0);
}  // namespace fa_bwd

extern "C" __global__ void __launch_bounds__(fa_bwd::NT) fa_bwd_dq_kernel(const __grid_constant__ FaParams p) {
  using namespace fa_bwd;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int m0 = qt * BQ;
  if (m0 >= p.Sq) return;
  const int hk = h / (p.Hq / p.Hkv);
  const int gb = b + p.b_off, gh = h + p.h_off;

  unsigned char* Qs = smem;
  unsigned char* dOs = Qs + BQ * PQ;
  unsigned char* Ks = dOs + BQ * PV;
  unsigned char* Vs = Ks + 2 * BK * PQ;
  unsigned char* Ps = Vs + 2 * BK * PV;
  const fa_u32 sQ = fa_smem_u32(Qs), sdO = fa_smem_u32(dOs), sK = fa_smem_u32(Ks), sV = fa_smem_u32(Vs);

  const char* qg = (const char*)p.q.ptr + ((long long)b * p.q.sb + (long long)h * p.q.sh + (long long)m0 * p.q.ss) * ES;
  const char* dog = (const char*)p.dout.ptr + ((long long)b * p.dout.sb + (long long)h * p.dout.sh + (long long)m0 * p.dout.ss) * ES;
  const char* kg = (const char*)p.k.ptr + ((long long)b * p.k.sb + (long long)hk * p.k.sh) * ES;
  const char* vg = (const char*)p.v.ptr + ((long long)b * p.v.sb + (long long)hk * p.v.sh) * ES;

  fa_load_tile<D, ES, NT>(sQ, qg, p.q.ss * ES, BQ, p.Sq - m0, tid);
  fa_load_tile<DV, ES, NT>(sdO, dog, p.dout.ss * ES, BQ, p.Sq - m0, tid);
  fa_cp_commit();

  // per-row scalars of this thread's two rows
  const long long rowbase = ((long long)b * p.Hq + h) * p.Sq;
  const int r_lo = m0 + warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  float lse2[2], delta[2];
  lse2[0] = r_lo < p.Sq ? p.lse[rowbase + r_lo] * FA_LOG2E : FA_NEG_INF;
  lse2[1] = r_hi < p.Sq ? p.lse[rowbase + r_hi] * FA_LOG2E : FA_NEG_INF;
  delta[0] = r_lo < p.Sq ? p.delta[rowbase + r_lo] : 0.f;
  delta[1] = r_hi < p.Sq ? p.delta[rowbase + r_hi] : 0.f;

  FaWalk walk;
  {
    int qblk = 0;
    if (p.t.kv_num != nullptr) qblk = min(m0 / p.t.QB, p.t.nQ - 1);
    walk.init_kv<BK>(p.t, b, h, qblk, p.Skv);
  }
  int slot = 0;
  auto load_kv = [&](int stage, int n0) {
    fa_load_tile<D, ES, NT>(sK + stage * BK * PQ, kg + (long long)n0 * p.k.ss * ES, p.k.ss * ES, BK, p.Skv - n0, tid);
    fa_load_tile<DV, ES, NT>(sV + stage * BK * PV, vg + (long long)n0 * p.v.ss * ES, p.v.ss * ES, BK, p.Skv - n0, tid);
  };

  float dq[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) dq[j][0] = dq[j][1] = dq[j][2] = dq[j][3] = 0.f;

  int n0c = 0, n0n = 0;
  bool fullc = false, fulln = false;
  bool have = walk.next<BK>(slot, n0c, fullc);
  if (have) load_kv(0, n0c);
  fa_cp_commit();
  int stage = 0;

  fa_u32 qf[A_IN_REGS ? D / 16 : 1][4], dof[A_IN_REGS ? DV / 16 : 1][4];
  bool a_loaded = false;

  while (have) {
    const bool have_n = walk.next<BK>(slot, n0n, fulln);
    if (have_n) load_kv(stage ^ 1, n0n);
    fa_cp_commit();
    fa_cp_wait<1>();
    __syncthreads();

    float s[BK / 8][4], dp[BK / 8][4];
#pragma unroll
    for (int j = 0; j < BK / 8; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      dp[j][0] = dp[j][1] = dp[j][2] = dp[j][3] = 0.f;
    }
    const int ko = stage * BK * PQ, vo = stage * BK * PV;
    if constexpr (F32) {
      fa_simt_nt<D, BK>(s, Qs, PQ, warp * 16, Ks + ko, PQ, lane);
      fa_simt_nt<DV, BK>(dp, dOs, PV, warp * 16, Vs + vo, PV, lane);
    } else if constexpr (A_IN_REGS) {
      if (!a_loaded) {
        a_loaded = true;
        fa_load_a_frags<A_IN_REGS ? D : 16>(qf, sQ, PQ, warp * 16, lane);
        fa_load_a_frags<A_IN_REGS ? DV : 16>(dof, sdO, PV, warp * 16, lane);
      }
      fa_mma_nt<DT, A_IN_REGS ? D : 16, BK>(s, qf, sK + ko, PQ, lane);
      fa_mma_nt<DT, A_IN_REGS ? DV : 16, BK>(dp, dof, sV + vo, PV, lane);
    } else {
      fa_mma_nt_smemA<DT, D, BK>(s, sQ, PQ, warp * 16, sK + ko, PQ, lane);
      fa_mma_nt_smemA<DT, DV, BK>(dp, sdO, PV, warp * 16, sV + vo, PV, lane);
    }

    fa_round_acc<DT, BK / 8>(s);
    const bool ragged = n0c + BK > p.Skv;
#pragma unroll
    for (int j = 0; j < BK / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kv = n0c + j * 8 + (lane & 3) * 2 + (e & 1);
        const int hh = e >> 1;
        const int qi = hh ? r_hi : r_lo;
        float pr, g;
        elem(s[j][e], p.scale, gb, gh, qi, kv, !fullc, !ragged || kv < p.Skv, lse2[hh], pr, g);
        s[j][e] = pr * (dp[j][e] - delta[hh]) * g;  // dS
      }
    }
    if constexpr (F32) fa_simt_nn<BK, D>(dq, s, Ps, PPK, warp * 16, Ks + ko, PQ, lane);
    else fa_mma_nn<DT, BK, D>(dq, s, sK + ko, PQ, lane);

    __syncthreads();
    have = have_n;
    n0c = n0n;
    fullc = fulln;
    stage ^= 1;
  }

  fa_cp_wait<0>();
  __syncthreads();
  fa_store_acc<DT, D>(Qs, PQ, warp * 16, dq, p.scale, lane);
  __syncthreads();
  char* dqg = (char*)p.dq.ptr + ((long long)b * p.dq.sb + (long long)h * p.dq.sh + (long long)m0 * p.dq.ss) * ES;
  fa_store_tile<D, ES, NT>(dqg, p.dq.ss * ES, Qs, min(BQ, p.Sq - m0), tid);
}

// ======================================================================================
// dK, dV
// ======================================================================================
namespace fa_bwd {
constexpr int PPQ = FaTile<BQ, 4>::PITCH;  // fp32 staging tile [BK][BQ] (fp32 path)
constexpr int ROWS_BYTES = 2 * BQ * 4;     // lse2 and delta of one q tile
constexpr int DKDV_SMEM = BK * PQ + BK * PV + 2 * BQ * PQ + 2 * BQ * PV + 2 * ROWS_BYTES + (F32 ? BK * PPQ : 0);
}  // namespace fa_bwd

extern "C" __global__ void __launch_bounds__(fa_bwd::NT) fa_bwd_dkdv_kernel(const __grid_constant__ FaParams p) {
  using namespace fa_bwd;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kt = blockIdx.x;
  const int hk = blockIdx.y, b = blockIdx.z;
  const int n0 = kt * BK;
  if (n0 >= p.Skv) return;
  const int G = p.Hq / p.Hkv;
  const int gb = b + p.b_off;

  unsigned char* Ks = smem;
  unsigned char* Vs = Ks + BK * PQ;
  unsigned char* Qs = Vs + BK * PV;
  unsigned char* dOs = Qs + 2 * BQ * PQ;
  unsigned char* Rs = dOs + 2 * BQ * PV;  // [2 stages][lse2[BQ], delta[BQ]]
  unsigned char* Ps = Rs + 2 * ROWS_BYTES;
  const fa_u32 sK = fa_smem_u32(Ks), sV = fa_smem_u32(Vs), sQ = fa_smem_u32(Qs), sdO = fa_smem_u32(dOs),
               sR = fa_smem_u32(Rs);

  const char* kg = (const char*)p.k.ptr + ((long long)b * p.k.sb + (long long)hk * p.k.sh + (long long)n0 * p.k.ss) * ES;
  const char* vg = (const char*)p.v.ptr + ((long long)b * p.v.sb + (long long)hk * p.v.sh + (long long)n0 * p.v.ss) * ES;
  fa_load_tile<D, ES, NT>(sK, kg, p.k.ss * ES, BK, p.Skv - n0, tid);
  fa_load_tile<DV, ES, NT>(sV, vg, p.v.ss * ES, BK, p.Skv - n0, tid);
  fa_cp_commit();

  float dk[D / 8][4], dv[DV / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) dk[j][0] = dk[j][1] = dk[j][2] = dk[j][3] = 0.f;
#pragma unroll
  for (int j = 0; j < DV / 8; ++j) dv[j][0] = dv[j][1] = dv[j][2] = dv[j][3] = 0.f;

  fa_u32 kf[A_IN_REGS ? D / 16 : 1][4], vf[A_IN_REGS ? DV / 16 : 1][4];
  bool a_loaded = false;
  const int kv_lo = n0 + warp * 16 + (lane >> 2), kv_hi = kv_lo + 8;
  const bool kv_ok[2] = {kv_lo < p.Skv, kv_hi < p.Skv};

  for (int g = 0; g < G; ++g) {
    const int h = hk * G + g;
    const int gh = h + p.h_off;
    const char* qg = (const char*)p.q.ptr + ((long long)b * p.q.sb + (long long)h * p.q.sh) * ES;
    const char* dog = (const char*)p.dout.ptr + ((long long)b * p.dout.sb + (long long)h * p.dout.sh) * ES;
    const long long rowbase = ((long long)b * p.Hq + h) * p.Sq;

    FaWalk walk;
    {
      int kvblk = 0;
      if (p.t.kv_num != nullptr) kvblk = min(n0 / p.t.KVB, p.t.nKV - 1);
      walk.init_q<BQ>(p.t, b, h, kvblk, p.Sq);
    }
    int slot = 0;
    auto load_q = [&](int stage, int m0) {
      fa_load_tile<D, ES, NT>(sQ + stage * BQ * PQ, qg + (long long)m0 * p.q.ss * ES, p.q.ss * ES, BQ, p.Sq - m0, tid);
      fa_load_tile<DV, ES, NT>(sdO + stage * BQ * PV, dog + (long long)m0 * p.dout.ss * ES, p.dout.ss * ES, BQ, p.Sq - m0, tid);
      for (int i = tid; i < 2 * BQ; i += NT) {
        const int which = i / BQ, r = i - which * BQ;
        const bool ok = m0 + r < p.Sq;
        const float* src = (which ? p.delta : p.lse) + rowbase + (ok ? m0 + r : 0);
        fa_cp_async4(sR + stage * ROWS_BYTES + i * 4, src, ok ? 4 : 0);
      }
    };

    int m0c = 0, m0n = 0;
    bool fullc = false, fulln = false;
    bool have = walk.next<BQ>(slot, m0c, fullc);
    if (have) load_q(0, m0c);
    fa_cp_commit();
    int stage = 0;

    while (have) {
      const bool have_n = walk.next<BQ>(slot, m0n, fulln);
      if (have_n) load_q(stage ^ 1, m0n);
      fa_cp_commit();
      fa_cp_wait<1>();
      __syncthreads();

      float s[BQ / 8][4], dp[BQ / 8][4];
#pragma unroll
      for (int j = 0; j < BQ / 8; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        dp[j][0] = dp[j][1] = dp[j][2] = dp[j][3] = 0.f;
      }
      const int qo = stage * BQ * PQ, doo = stage * BQ * PV;
      // S^T = K Q^T, dP^T = V dO^T
      if constexpr (F32) {
        fa_simt_nt<D, BQ>(s, Ks, PQ, warp * 16, Qs + qo, PQ, lane);
        fa_simt_nt<DV, BQ>(dp, Vs, PV, warp * 16, dOs + doo, PV, lane);
      } else if constexpr (A_IN_REGS) {
        if (!a_loaded) {
          a_loaded = true;
          fa_load_a_frags<A_IN_REGS ? D : 16>(kf, sK, PQ, warp * 16, lane);
          fa_load_a_frags<A_IN_REGS ? DV : 16>(vf, sV, PV, warp * 16, lane);
        }
        fa_mma_nt<DT, A_IN_REGS ? D : 16, BQ>(s, kf, sQ + qo, PQ, lane);
        fa_mma_nt<DT, A_IN_REGS ? DV : 16, BQ>(dp, vf, sdO + doo, PV, lane);
      } else {
        fa_mma_nt_smemA<DT, D, BQ>(s, sK, PQ, warp * 16, sQ + qo, PQ, lane);
        fa_mma_nt_smemA<DT, DV, BQ>(dp, sV, PV, warp * 16, sdO + doo, PV, lane);
      }

      fa_round_acc<DT, BQ / 8>(s);
      const float* rl = (const float*)(Rs + stage * ROWS_BYTES);
      const bool ragged = m0c + BQ > p.Sq;
#pragma unroll
      for (int j = 0; j < BQ / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int c = j * 8 + (lane & 3) * 2 + (e & 1);
          const int qi = m0c + c;
          const int hh = e >> 1;
          const int kv = hh ? kv_hi : kv_lo;
          float pr, gg;
          elem(s[j][e], p.scale, gb, gh, qi, kv, !fullc, kv_ok[hh] && (!ragged || qi < p.Sq), rl[c] * FA_LOG2E, pr, gg);
          s[j][e] = pr;                                  // P^T
          dp[j][e] = pr * (dp[j][e] - rl[BQ + c]) * gg;  // dS^T
        }
      }
      if constexpr (F32) {
        fa_simt_nn<BQ, DV>(dv, s, Ps, PPQ, warp * 16, dOs + doo, PV, lane);
        fa_simt_nn<BQ, D>(dk, dp, Ps, PPQ, warp * 16, Qs + qo, PQ, lane);
      } else {
        fa_mma_nn<DT, BQ, DV>(dv, s, sdO + doo, PV, lane);
        fa_mma_nn<DT, BQ, D>(dk, dp, sQ + qo, PQ, lane);
      }

      __syncthreads();
      have = have_n;
      m0c = m0n;
      fullc = fulln;
      stage ^= 1;
    }
    fa_cp_wait<0>();
    __syncthreads();
  }

  // epilogue: dK (scaled) and dV through the Q / dO staging buffers
  fa_cp_wait<0>();
  __syncthreads();
  fa_store_acc<DT, D>(Qs, PQ, warp * 16, dk, p.scale, lane);
  fa_store_acc<DT, DV>(dOs, PV, warp * 16, dv, 1.f, lane);
  __syncthreads();
  char* dkg = (char*)p.dk.ptr + ((long long)b * p.dk.sb + (long long)hk * p.dk.sh + (long long)n0 * p.dk.ss) * ES;
  char* dvg = (char*)p.dv.ptr + ((long long)b * p.dv.sb + (long long)hk * p.dv.sh + (long long)n0 * p.dv.ss) * ES;
  fa_store_tile<D, ES, NT>(dkg, p.dk.ss * ES, Qs, min(BK, p.Skv - n0), tid);
  fa_store_tile<DV, ES, NT>(dvg, p.dv.ss * ES, dOs, min(BK, p.Skv - n0), tid);
}
