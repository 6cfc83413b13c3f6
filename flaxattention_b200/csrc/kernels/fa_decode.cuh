// Split-KV decode kernel for short query blocks (Sq <= 64): the key/value range of one
// (batch, head) is cut into `num_splits` contiguous runs of tiles, one CTA each, so that a
// single (b, h) with a long KV cache still fills the GPU.  The reference has no such path:
// for Sq < 16 it pads the query to 16 rows and runs its forward kernel with one program per
// (b, h) (flaxattention/core/attention.py:269-273, :310-311).
//
// CTA = 4 warps arranged as RG row groups x CG column groups (RG = BM/16, CG = 4/RG).  All
// warps share the K/V tiles, which stream through a cp.async ring in 128-bit pieces; warp
// (rg, cg) owns query rows 16*rg.. and the cg-th slice of each kv tile and keeps its own
// running (max, sum, O).  The CG partial results are merged through shared memory at the
// end; with more than one split the CTA writes un-normalised (O, max, sum) to the workspace
// and a second kernel combines the splits, with one split it writes O and LSE directly.
//
// With grouped-query attention the G query heads of a kv head can share one CTA
// (FA_PACK_HEADS): its G * Sq query rows form one tile, row r belonging to head r / Sq and
// query r % Sq, so K and V of the kv head are read once instead of G times.  The mods see the
// head and query index of each row; the BlockMask walk is the one of the group's first head,
// which is why the host packs only when the tables do not depend on the head.
//
// Compile-time parameters (macros): FA_DTYPE (fp16 / bf16), FA_D, FA_DV, FA_BM (16, 32, 64),
// FA_BN (kv tile), FA_STAGES, FA_PACK_HEADS.
#pragma once
#include "fa_common.cuh"

#ifndef FA_PACK_HEADS
#define FA_PACK_HEADS 0
#endif

namespace fa_dec {

constexpr bool PACK = FA_PACK_HEADS != 0;

constexpr int DT = FA_DTYPE;
constexpr int D = FA_D;
constexpr int DV = FA_DV;
constexpr int BM = FA_BM;
constexpr int BN = FA_BN;
constexpr int STAGES = FA_STAGES;
constexpr int NWARPS = 4;
constexpr int NT = NWARPS * 32;
constexpr int RG = BM / 16;
constexpr int CG = NWARPS / RG;
constexpr int WN = BN / CG;  // kv columns per warp and tile
constexpr int ES = 2;
constexpr int PQ = FaTile<D, ES>::PITCH;
constexpr int PV = FaTile<DV, ES>::PITCH;
constexpr int Q_BYTES = BM * PQ;
constexpr int K_BYTES = BN * PQ;
constexpr int V_BYTES = BN * PV;
constexpr int MRG_PITCH = DV + 4;  // floats per merged row: O[DV], m, l, pad
constexpr int MRG_BYTES = CG * BM * MRG_PITCH * 4;
constexpr int PIPE_BYTES = STAGES * (K_BYTES + V_BYTES);
constexpr int SMEM_BYTES = Q_BYTES + (PIPE_BYTES > MRG_BYTES ? PIPE_BYTES : MRG_BYTES);

static_assert(DT != FA_DT_F32, "the decode kernel takes 16-bit inputs");
static_assert(BM == 16 || BM == 32 || BM == 64, "BM must be 16, 32 or 64");
static_assert(WN % 16 == 0, "each warp needs at least 16 kv columns per tile");

}  // namespace fa_dec

extern "C" __global__ void __launch_bounds__(fa_dec::NT) fa_decode_kernel(const __grid_constant__ FaParams p) {
  using namespace fa_dec;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp % RG, cg = warp / RG;
  // grid: (splits, query heads, batch), or (splits, kv heads, batch) when the heads of a group are packed
  const int split = blockIdx.x, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int hk = PACK ? (int)blockIdx.y : (int)blockIdx.y / G;
  const int h0 = PACK ? hk * G : (int)blockIdx.y;  // first query head of this CTA
  const int R = PACK ? G * p.Sq : p.Sq;            // query rows of this CTA
  const int gb = b + p.b_off;

  const fa_u32 sQ = fa_smem_u32(smem);
  const fa_u32 sK = sQ + Q_BYTES;
  const fa_u32 sV = sK + STAGES * K_BYTES;

  const char* qg = (const char*)p.q.ptr + (long long)b * p.q.sb * ES;
  const char* kg = (const char*)p.k.ptr + ((long long)b * p.k.sb + (long long)hk * p.k.sh) * ES;
  const char* vg = (const char*)p.v.ptr + ((long long)b * p.v.sb + (long long)hk * p.v.sh) * ES;

  {
    // query tile: row r is query r % Sq of head h0 + r / Sq; rows from R on are zero-filled
    constexpr int CPR = D * ES / 16;
    for (int i = tid; i < BM * CPR; i += NT) {
      const int r = i / CPR, c = i - r * CPR;
      const bool ok = r < R;
      const int g = PACK ? r / p.Sq : 0, q = r - g * p.Sq;
      const char* src = qg + (ok ? ((long long)(h0 + g) * p.q.sh + (long long)q * p.q.ss) * ES + c * 16 : 0);
      fa_cp_async16(sQ + r * PQ + c * 16, src, ok ? 16 : 0);
    }
  }
  fa_cp_commit();

  FaWalk walk;
  walk.init_kv<BN>(p.t, b, h0, 0, p.Skv);
  // this split's run of tile slots
  const int per = (walk.total + p.num_splits - 1) / p.num_splits;
  int slot = min(split * per, walk.total);
  const int slot_end = min(slot + per, walk.total);
  auto next_tile = [&](int& n0, bool& full) -> bool {
    while (slot < slot_end) {
      n0 = walk.tile_start<BN>(slot, full);
      ++slot;
      if (n0 >= 0) return true;
    }
    return false;
  };
  // With one row group (Sq <= 16) every warp reads only its own WN keys of a tile: it then loads
  // just those rows itself and the warps run as independent pipelines, with no block-wide
  // barrier inside the kv loop.  With several row groups the tile is loaded cooperatively.
  constexpr bool PRIVATE = RG == 1;
  auto load_kv = [&](int stage, int n0) {
    if (PRIVATE) {
      const int first = n0 + cg * WN, vr = p.Skv - first;
      const long long koff = vr > 0 ? (long long)first * p.k.ss * ES : 0;
      const long long voff = vr > 0 ? (long long)first * p.v.ss * ES : 0;
      fa_load_tile<D, ES, 32>(sK + stage * K_BYTES + cg * WN * PQ, kg + koff, p.k.ss * ES, WN, vr, lane);
      fa_load_tile<DV, ES, 32>(sV + stage * V_BYTES + cg * WN * PV, vg + voff, p.v.ss * ES, WN, vr, lane);
    } else {
      fa_load_tile<D, ES, NT>(sK + stage * K_BYTES, kg + (long long)n0 * p.k.ss * ES, p.k.ss * ES, BN, p.Skv - n0, tid);
      fa_load_tile<DV, ES, NT>(sV + stage * V_BYTES, vg + (long long)n0 * p.v.ss * ES, p.v.ss * ES, BN, p.Skv - n0, tid);
    }
  };

  float o[DV / 8][4];
#pragma unroll
  for (int j = 0; j < DV / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {FA_NEG_INF, FA_NEG_INF}, l_run[2] = {0.f, 0.f};

  // prologue: fill STAGES-1 stages
  int n0s[STAGES];
  bool fulls[STAGES];
  bool haves[STAGES];
#pragma unroll
  for (int i = 0; i < STAGES; ++i) { n0s[i] = 0; fulls[i] = false; haves[i] = false; }
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    haves[i] = next_tile(n0s[i], fulls[i]);
    if (haves[i]) load_kv(i, n0s[i]);
    fa_cp_commit();
  }
  fa_u32 qf[D / 16][4];
  bool q_loaded = false;
  int cur = 0;  // ring position of the tile being computed

  while (haves[cur]) {
    // prefetch into the stage that was consumed last iteration
    const int pf = (cur + STAGES - 1) % STAGES;
    haves[pf] = next_tile(n0s[pf], fulls[pf]);
    if (haves[pf]) load_kv(pf, n0s[pf]);
    fa_cp_commit();
    fa_cp_wait<STAGES - 1>();
    if (PRIVATE && q_loaded) __syncwarp();
    else __syncthreads();  // (first iteration: the query tile was loaded by all threads)

    if (!q_loaded) {
      q_loaded = true;
      fa_load_a_frags<D>(qf, sQ, PQ, rg * 16, lane);
    }
    const int n0 = n0s[cur] + cg * WN;
    const bool full = fulls[cur];
    float s[WN / 8][4];
#pragma unroll
    for (int j = 0; j < WN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    fa_mma_nt<DT, D, WN>(s, qf, sK + cur * K_BYTES + cg * WN * PQ, PQ, lane);

    fa_round_acc<DT, WN / 8>(s);
    const bool ragged = n0 + WN > p.Skv;
    const float sc2 = p.scale * FA_LOG2E;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      // rows 8..15 of a row group hold no query when there are at most 8 (+ 16 rg) rows: nothing to do for them
      if (rg * 16 + hh * 8 >= R) {
#pragma unroll
        for (int j = 0; j < WN / 8; ++j) s[j][hh * 2] = s[j][hh * 2 + 1] = 0.f;
        continue;
      }
      const int row = rg * 16 + hh * 8 + (lane >> 2);
      const int g_row = PACK ? row / p.Sq : 0;
      const int qi = row - g_row * p.Sq;
      const int gh = h0 + g_row + p.h_off;
      float mx = FA_NEG_INF;
#pragma unroll
      for (int j = 0; j < WN / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kv = n0 + j * 8 + (lane & 3) * 2 + e;
          float x = s[j][hh * 2 + e];
#if FA_HAS_SCORE_MOD && defined(FA_SCORE_AFFINE)
          // affine score_mod: scale and log2(e) folded into one FMA
          x = fmaf(x, fa_score_mul(0.f, gb, gh, qi, kv) * sc2, fa_score_add2(0.f, gb, gh, qi, kv));
#elif FA_HAS_SCORE_MOD
          x = fa_score_mod(x * p.scale, gb, gh, qi, kv) * FA_LOG2E;
#else
          x *= sc2;
#endif
          bool keep = true;
#if FA_HAS_MASK_MOD
          if (!full) keep = fa_mask_mod(gb, gh, qi, kv);
#endif
          if (ragged) keep = keep && (kv < p.Skv);
          x = keep ? x : FA_NEG_INF;
          s[j][hh * 2 + e] = x;
          mx = fmaxf(mx, x);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hh], mx);
      const float m_use = (m_new == FA_NEG_INF) ? 0.f : m_new;
      const float corr = fa_ex2(m_run[hh] - m_use);
      m_run[hh] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < WN / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pv = fa_ex2(s[j][hh * 2 + e] - m_use);
          s[j][hh * 2 + e] = pv;
          sum += pv;
        }
      }
      l_run[hh] = l_run[hh] * corr + sum;
#pragma unroll
      for (int j = 0; j < DV / 8; ++j) {
        o[j][hh * 2] *= corr;
        o[j][hh * 2 + 1] *= corr;
      }
    }
    fa_mma_nn<DT, WN, DV>(o, s, sV + cur * V_BYTES + cg * WN * PV, PV, lane);

    if (PRIVATE) __syncwarp();
    else __syncthreads();
    cur = (cur + 1) % STAGES;
  }

  // ---- merge the CG column groups ------------------------------------------------------
  fa_cp_wait<0>();
  __syncthreads();
  float* mrg = (float*)(smem + Q_BYTES);
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    float l = l_run[hh];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int r = rg * 16 + hh * 8 + (lane >> 2);
    float* row = mrg + ((long long)cg * BM + r) * MRG_PITCH;
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) {
      const int c = j * 8 + (lane & 3) * 2;
      row[c] = o[j][hh * 2];
      row[c + 1] = o[j][hh * 2 + 1];
    }
    if ((lane & 3) == 0) {
      row[DV] = m_run[hh];
      row[DV + 1] = l;
    }
  }
  __syncthreads();
  const int rows = min(R, BM);
  for (int i = tid; i < rows * DV; i += NT) {
    const int r = i / DV, c = i - r * DV;
    const int g_row = PACK ? r / p.Sq : 0, qr = r - g_row * p.Sq, h = h0 + g_row;
    const long long bh = (long long)b * p.Hq + h;
    float mstar = FA_NEG_INF;
#pragma unroll
    for (int g = 0; g < CG; ++g) mstar = fmaxf(mstar, mrg[((long long)g * BM + r) * MRG_PITCH + DV]);
    float acc = 0.f, lstar = 0.f;
#pragma unroll
    for (int g = 0; g < CG; ++g) {
      const float* row = mrg + ((long long)g * BM + r) * MRG_PITCH;
      const float w = row[DV] == FA_NEG_INF ? 0.f : fa_ex2(row[DV] - mstar);
      acc += w * row[c];
      lstar += w * row[DV + 1];
    }
    if (p.num_splits > 1) {
      const long long prow = (bh * p.num_splits + split) * p.Sq + qr;
      p.part_o[prow * DV + c] = acc;
      if (c == 0) {
        p.part_ml[prow * 2] = mstar;
        p.part_ml[prow * 2 + 1] = lstar;
      }
    } else {
      const float inv = lstar > 0.f ? 1.f / lstar : 0.f;
      char* og = (char*)p.o.ptr + ((long long)b * p.o.sb + (long long)h * p.o.sh + (long long)qr * p.o.ss) * ES;
      const float val = acc * inv;
      if (DT == FA_DT_F16) {
        fa_u16 hv;
        asm("cvt.rn.f16.f32 %0, %1;" : "=h"(hv) : "f"(val));
        ((fa_u16*)og)[c] = hv;
      } else {
        fa_u16 hv;
        asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(hv) : "f"(val));
        ((fa_u16*)og)[c] = hv;
      }
      if (c == 0 && p.lse != nullptr)
        p.lse[bh * p.Sq + qr] = lstar > 0.f ? (mstar + fa_lg2(lstar)) * FA_LN2 : FA_NEG_INF;
    }
  }
}
