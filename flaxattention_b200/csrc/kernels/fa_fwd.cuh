// Flash-attention forward, general tile kernel (any head dim that is a multiple of 16,
// ragged lengths, GQA, fp16 / bf16 / fp32).  Replaces mha_forward_kernel of
// flaxattention/kernel/attention.py:34-149; unlike it, the kv loop walks the BlockMask
// tables (partial blocks with mask_mod, full blocks without) and a true running max is
// kept.  Semantics follow the dense path of flaxattention/core/attention.py:14-106:
//   s = (q.k) * scale -> score_mod(s, b, h, q, kv) -> -inf where mask_mod is false
//   lse = logsumexp(s), fully masked rows: lse = -inf and output 0.
//
// 16-bit inputs use mma.sync m16n8k16 with fp32 accumulation; fp32 inputs use plain FMA
// so that the result is accurate to fp32 rounding.
//
// Compile-time parameters (macros): FA_DTYPE, FA_D, FA_DV, FA_BM, FA_BN, FA_WARPS.
// The mod fragment (fa_score_mod, fa_mask_mod, FA_HAS_*) is placed before this file.
#pragma once
#include "fa_common.cuh"

namespace fa_fwd {

constexpr int DT = FA_DTYPE;
constexpr int D = FA_D;
constexpr int DV = FA_DV;
constexpr int BM = FA_BM;
constexpr int BN = FA_BN;
constexpr int NWARPS = FA_WARPS;
constexpr int NT = NWARPS * 32;
constexpr int WM = BM / (16 * NWARPS);  // m16 tiles per warp
constexpr int ES = DT == FA_DT_F32 ? 4 : 2;
constexpr int PQ = FaTile<D, ES>::PITCH;
constexpr int PV = FaTile<DV, ES>::PITCH;
constexpr int PP = FaTile<BN, 4>::PITCH;  // fp32 probability tile (fp32 path only)
constexpr int Q_BYTES = BM * PQ;
constexpr int K_BYTES = BN * PQ;
constexpr int V_BYTES = BN * PV;
constexpr int P_BYTES = DT == FA_DT_F32 ? BM * PP : 0;
constexpr int SMEM_BYTES = Q_BYTES + 2 * K_BYTES + 2 * V_BYTES + P_BYTES;

static_assert(BM % (16 * NWARPS) == 0, "BM must be a multiple of 16 * warps");
static_assert(D % 16 == 0 && DV % 16 == 0 && BN % 16 == 0, "tile dims must be multiples of 16");
static_assert(DV <= D, "value head dim must not exceed the qk head dim");

struct RowState {
  float m[WM][2];  // running max, log2 units
  float l[WM][2];  // running sum (per-thread partial)
};

// scale -> score_mod -> mask -> log2 units, online-softmax update of one kv tile
template <bool MASKED>
__device__ __forceinline__ void softmax_tile(float (&s)[WM][BN / 8][4], float (&o)[WM][DV / 8][4], RowState& st,
                                             const FaParams& p, int gb, int gh, int row_base, int n0, int lane) {
  const bool ragged = n0 + BN > p.Skv;
#pragma unroll
  for (int wm = 0; wm < WM; ++wm) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int qi = row_base + wm * 16 + hh * 8 + (lane >> 2);
      float mx = FA_NEG_INF;
#pragma unroll
      for (int nj = 0; nj < BN / 8; ++nj) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kv = n0 + nj * 8 + (lane & 3) * 2 + e;
          float x = s[wm][nj][hh * 2 + e] * p.scale;
#if FA_HAS_SCORE_MOD
          x = fa_score_mod(x, gb, gh, qi, kv);
#endif
          bool keep = true;
#if FA_HAS_MASK_MOD
          if (MASKED) keep = fa_mask_mod(gb, gh, qi, kv);
#endif
          if (ragged) keep = keep && (kv < p.Skv);
          x = keep ? x * FA_LOG2E : FA_NEG_INF;
          s[wm][nj][hh * 2 + e] = x;
          mx = fmaxf(mx, x);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_old = st.m[wm][hh];
      const float m_new = fmaxf(m_old, mx);
      const float m_use = (m_new == FA_NEG_INF) ? 0.f : m_new;
      float corr, sum = 0.f;
      if (DT == FA_DT_F32) corr = exp2f(m_old - m_use); else corr = fa_ex2(m_old - m_use);
      st.m[wm][hh] = m_new;
#pragma unroll
      for (int nj = 0; nj < BN / 8; ++nj) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float pv;
          if (DT == FA_DT_F32) pv = exp2f(s[wm][nj][hh * 2 + e] - m_use);
          else pv = fa_ex2(s[wm][nj][hh * 2 + e] - m_use);
          s[wm][nj][hh * 2 + e] = pv;
          sum += pv;
        }
      }
      st.l[wm][hh] = st.l[wm][hh] * corr + sum;
#pragma unroll
      for (int dj = 0; dj < DV / 8; ++dj) {
        o[wm][dj][hh * 2] *= corr;
        o[wm][dj][hh * 2 + 1] *= corr;
      }
    }
  }
}

}  // namespace fa_fwd

extern "C" __global__ void __launch_bounds__(fa_fwd::NT) fa_fwd_kernel(const __grid_constant__ FaParams p) {
  using namespace fa_fwd;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int m0 = qt * BM;
  if (m0 >= p.Sq) return;
  const int hk = h / (p.Hq / p.Hkv);
  const int gb = b + p.b_off, gh = h + p.h_off;
  const int row_base = m0 + warp * (16 * WM);

  const fa_u32 sQ = fa_smem_u32(smem);
  const fa_u32 sK = sQ + Q_BYTES;
  const fa_u32 sV = sK + 2 * K_BYTES;

  const char* qg = (const char*)p.q.ptr + ((long long)b * p.q.sb + (long long)h * p.q.sh + (long long)m0 * p.q.ss) * ES;
  const char* kg = (const char*)p.k.ptr + ((long long)b * p.k.sb + (long long)hk * p.k.sh) * ES;
  const char* vg = (const char*)p.v.ptr + ((long long)b * p.v.sb + (long long)hk * p.v.sh) * ES;

  fa_load_tile<D, ES, NT>(sQ, qg, p.q.ss * ES, BM, p.Sq - m0, tid);
  fa_cp_commit();

  FaWalk walk;
  {
    int qblk = 0;
    if (p.t.kv_num != nullptr) qblk = min(m0 / p.t.QB, p.t.nQ - 1);
    walk.init_kv<BN>(p.t, b, h, qblk, p.Skv);
  }
  int slot = 0;
  auto next_tile = [&](int& n0, bool& full) -> bool { return walk.next<BN>(slot, n0, full); };
  auto load_kv = [&](int stage, int n0) {
    fa_load_tile<D, ES, NT>(sK + stage * K_BYTES, kg + (long long)n0 * p.k.ss * ES, p.k.ss * ES, BN, p.Skv - n0, tid);
    fa_load_tile<DV, ES, NT>(sV + stage * V_BYTES, vg + (long long)n0 * p.v.ss * ES, p.v.ss * ES, BN, p.Skv - n0, tid);
  };

  float o[WM][DV / 8][4];
  RowState st;
#pragma unroll
  for (int wm = 0; wm < WM; ++wm) {
    st.m[wm][0] = st.m[wm][1] = FA_NEG_INF;
    st.l[wm][0] = st.l[wm][1] = 0.f;
#pragma unroll
    for (int dj = 0; dj < DV / 8; ++dj) o[wm][dj][0] = o[wm][dj][1] = o[wm][dj][2] = o[wm][dj][3] = 0.f;
  }

  int n0c = 0, n0n = 0;
  bool fullc = false, fulln = false;
  bool have = next_tile(n0c, fullc);
  if (have) load_kv(0, n0c);
  fa_cp_commit();
  int stage = 0;

#if FA_DTYPE != FA_DT_F32
  fa_u32 qf[WM][D / 16][4];
  bool q_loaded = false;
#endif

  while (have) {
    const bool have_n = next_tile(n0n, fulln);
    if (have_n) load_kv(stage ^ 1, n0n);
    fa_cp_commit();
    fa_cp_wait<1>();
    __syncthreads();

    const fa_u32 sKc = sK + stage * K_BYTES;
    const fa_u32 sVc = sV + stage * V_BYTES;
    float s[WM][BN / 8][4];
#pragma unroll
    for (int wm = 0; wm < WM; ++wm)
#pragma unroll
      for (int nj = 0; nj < BN / 8; ++nj) s[wm][nj][0] = s[wm][nj][1] = s[wm][nj][2] = s[wm][nj][3] = 0.f;

#if FA_DTYPE != FA_DT_F32
    if (!q_loaded) {
      q_loaded = true;
#pragma unroll
      for (int wm = 0; wm < WM; ++wm)
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int r = warp * (16 * WM) + wm * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
          const int c = kk * 16 + (lane >> 4) * 8;
          fa_ldsm_x4(sQ + r * PQ + c * 2, qf[wm][kk][0], qf[wm][kk][1], qf[wm][kk][2], qf[wm][kk][3]);
        }
    }
    // S = Q K^T
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int nj = 0; nj < BN / 16; ++nj) {
        fa_u32 r0, r1, r2, r3;
        const int r = nj * 16 + (lane >> 4) * 8 + (lane & 7);
        const int c = kk * 16 + ((lane >> 3) & 1) * 8;
        fa_ldsm_x4(sKc + r * PQ + c * 2, r0, r1, r2, r3);
#pragma unroll
        for (int wm = 0; wm < WM; ++wm) {
          fa_mma16816<DT>(s[wm][2 * nj], qf[wm][kk], r0, r1);
          fa_mma16816<DT>(s[wm][2 * nj + 1], qf[wm][kk], r2, r3);
        }
      }
    }
#else
    {
      // fp32: every thread computes the score elements of its accumulator-fragment slots
      const unsigned char* Qs = smem;
      const unsigned char* Kc = smem + Q_BYTES + stage * K_BYTES;
#pragma unroll
      for (int wm = 0; wm < WM; ++wm) {
        const int r0_ = warp * (16 * WM) + wm * 16 + (lane >> 2);
        for (int d4 = 0; d4 < D / 4; ++d4) {
          const float4 qa = *(const float4*)(Qs + r0_ * PQ + d4 * 16);
          const float4 qb = *(const float4*)(Qs + (r0_ + 8) * PQ + d4 * 16);
#pragma unroll
          for (int nj = 0; nj < BN / 8; ++nj) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int c = nj * 8 + (lane & 3) * 2 + e;
              const float4 kk4 = *(const float4*)(Kc + c * PQ + d4 * 16);
              s[wm][nj][e] = fmaf(qa.x, kk4.x, fmaf(qa.y, kk4.y, fmaf(qa.z, kk4.z, fmaf(qa.w, kk4.w, s[wm][nj][e]))));
              s[wm][nj][2 + e] = fmaf(qb.x, kk4.x, fmaf(qb.y, kk4.y, fmaf(qb.z, kk4.z, fmaf(qb.w, kk4.w, s[wm][nj][2 + e]))));
            }
          }
        }
      }
    }
#endif

#pragma unroll
    for (int wm = 0; wm < WM; ++wm) fa_round_acc<DT, BN / 8>(s[wm]);
    if (fullc) softmax_tile<false>(s, o, st, p, gb, gh, row_base, n0c, lane);
    else softmax_tile<true>(s, o, st, p, gb, gh, row_base, n0c, lane);

#if FA_DTYPE != FA_DT_F32
    // O += P V
#pragma unroll
    for (int kj = 0; kj < BN / 16; ++kj) {
      fa_u32 a[WM][4];
#pragma unroll
      for (int wm = 0; wm < WM; ++wm) {
        a[wm][0] = fa_pack2<DT>(s[wm][2 * kj][0], s[wm][2 * kj][1]);
        a[wm][1] = fa_pack2<DT>(s[wm][2 * kj][2], s[wm][2 * kj][3]);
        a[wm][2] = fa_pack2<DT>(s[wm][2 * kj + 1][0], s[wm][2 * kj + 1][1]);
        a[wm][3] = fa_pack2<DT>(s[wm][2 * kj + 1][2], s[wm][2 * kj + 1][3]);
      }
#pragma unroll
      for (int dj = 0; dj < DV / 16; ++dj) {
        fa_u32 r0, r1, r2, r3;
        const int r = kj * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
        const int c = dj * 16 + (lane >> 4) * 8;
        fa_ldsm_x4_t(sVc + r * PV + c * 2, r0, r1, r2, r3);
#pragma unroll
        for (int wm = 0; wm < WM; ++wm) {
          fa_mma16816<DT>(o[wm][2 * dj], a[wm], r0, r1);
          fa_mma16816<DT>(o[wm][2 * dj + 1], a[wm], r2, r3);
        }
      }
    }
#else
    {
      unsigned char* Ps = smem + Q_BYTES + 2 * K_BYTES + 2 * V_BYTES;
      const unsigned char* Vc = smem + Q_BYTES + 2 * K_BYTES + stage * V_BYTES;
#pragma unroll
      for (int wm = 0; wm < WM; ++wm) {
        const int r0_ = warp * (16 * WM) + wm * 16 + (lane >> 2);
#pragma unroll
        for (int nj = 0; nj < BN / 8; ++nj) {
          const int c = nj * 8 + (lane & 3) * 2;
          *(float2*)(Ps + r0_ * PP + c * 4) = make_float2(s[wm][nj][0], s[wm][nj][1]);
          *(float2*)(Ps + (r0_ + 8) * PP + c * 4) = make_float2(s[wm][nj][2], s[wm][nj][3]);
        }
      }
      __syncwarp();
#pragma unroll
      for (int wm = 0; wm < WM; ++wm) {
        const int r0_ = warp * (16 * WM) + wm * 16 + (lane >> 2);
        for (int k = 0; k < BN; ++k) {
          const float pa = *(const float*)(Ps + r0_ * PP + k * 4);
          const float pb = *(const float*)(Ps + (r0_ + 8) * PP + k * 4);
#pragma unroll
          for (int dj = 0; dj < DV / 8; ++dj) {
            const float2 vv = *(const float2*)(Vc + k * PV + (dj * 8 + (lane & 3) * 2) * 4);
            o[wm][dj][0] = fmaf(pa, vv.x, o[wm][dj][0]);
            o[wm][dj][1] = fmaf(pa, vv.y, o[wm][dj][1]);
            o[wm][dj][2] = fmaf(pb, vv.x, o[wm][dj][2]);
            o[wm][dj][3] = fmaf(pb, vv.y, o[wm][dj][3]);
          }
        }
      }
      __syncwarp();
    }
#endif

    __syncthreads();  // every warp is done with this stage before the next prefetch overwrites it
    have = have_n;
    n0c = n0n;
    fullc = fulln;
    stage ^= 1;
  }

  // ---- epilogue ----------------------------------------------------------------------
  fa_cp_wait<0>();
  __syncthreads();
  unsigned char* Os = smem;  // reuse the Q tile
#pragma unroll
  for (int wm = 0; wm < WM; ++wm) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      float l = st.l[wm][hh];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int rl = warp * (16 * WM) + wm * 16 + hh * 8 + (lane >> 2);
      const int qi = m0 + rl;
      if (p.lse != nullptr && (lane & 3) == 0 && qi < p.Sq) {
        float lse;
        if (DT == FA_DT_F32) lse = l > 0.f ? (st.m[wm][hh] + log2f(l)) * FA_LN2 : FA_NEG_INF;
        else lse = l > 0.f ? (st.m[wm][hh] + fa_lg2(l)) * FA_LN2 : FA_NEG_INF;
        p.lse[((long long)b * p.Hq + h) * p.Sq + qi] = lse;
      }
#pragma unroll
      for (int dj = 0; dj < DV / 8; ++dj) {
        const int c = dj * 8 + (lane & 3) * 2;
        const float x0 = o[wm][dj][hh * 2] * inv, x1 = o[wm][dj][hh * 2 + 1] * inv;
        if (DT == FA_DT_F32) *(float2*)(Os + rl * PV + c * 4) = make_float2(x0, x1);
        else *(fa_u32*)(Os + rl * PV + c * 2) = fa_pack2<DT>(x0, x1);
      }
    }
  }
  __syncthreads();
  {
    constexpr int CPR = DV * ES / 16;
    char* og = (char*)p.o.ptr + ((long long)b * p.o.sb + (long long)h * p.o.sh + (long long)m0 * p.o.ss) * ES;
    const int valid = min(BM, p.Sq - m0);
    for (int i = tid; i < valid * CPR; i += NT) {
      const int r = i / CPR, c = i - r * CPR;
      *(uint4*)(og + (long long)r * p.o.ss * ES + c * 16) = *(const uint4*)(Os + r * PV + c * 16);
    }
  }
}
