// Device helpers shared by the attention kernel templates (sm_100a).
// Self-contained on purpose: no standard or CUDA headers, so the run-time compiler
// needs no include path beyond this directory.
#pragma once
#include "fa_params.h"

typedef unsigned int fa_u32;
typedef unsigned long long fa_u64;
typedef unsigned short fa_u16;

#define FA_DT_F16 0
#define FA_DT_BF16 1
#define FA_DT_F32 2

#define FA_LOG2E 1.4426950408889634f
#define FA_LN2 0.6931471805599453f
#define FA_NEG_INF __int_as_float(0xff800000)

__device__ __forceinline__ fa_u32 fa_smem_u32(const void* p) {
  return (fa_u32)__cvta_generic_to_shared(p);
}

// exp2 on the SFU; flush-to-zero, -inf -> 0.
__device__ __forceinline__ float fa_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fa_lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- 16-bit packing ------------------------------------------------------------------
template <int DT>
__device__ __forceinline__ fa_u32 fa_pack2(float lo, float hi) {
  fa_u32 r;
  if (DT == FA_DT_F16) {
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}
template <int DT>
__device__ __forceinline__ float fa_to_float(fa_u16 v) {
  if (DT == FA_DT_F16) {
    float f;
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(v));
    return f;
  } else {
    return __uint_as_float(((fa_u32)v) << 16);
  }
}

// Rounds two fp32 scores to the input dtype and back.  The reference's dense path computes
// Q.K^T in the input dtype before casting to fp32 (flaxattention/core/attention.py:27);
// kernels built with FA_ROUND_SCORES reproduce that rounding, the others keep the fp32
// product the way the reference's fused kernel does (flaxattention/kernel/attention.py:82).
template <int DT>
__device__ __forceinline__ void fa_round2(float& a, float& b) {
  if (DT == FA_DT_F16) {
    fa_u32 r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    fa_u16 lo, hi;
    asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(r));
    asm("cvt.f32.f16 %0, %1;" : "=f"(a) : "h"(lo));
    asm("cvt.f32.f16 %0, %1;" : "=f"(b) : "h"(hi));
  } else if (DT == FA_DT_BF16) {
    fa_u32 r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    a = __uint_as_float(r << 16);
    b = __uint_as_float(r & 0xffff0000u);
  }
}
#ifndef FA_ROUND_SCORES
#define FA_ROUND_SCORES 0
#endif
// applies the rounding to a whole accumulator tile
template <int DT, int N>
__device__ __forceinline__ void fa_round_acc(float (&acc)[N][4]) {
#if FA_ROUND_SCORES
  if (DT != FA_DT_F32) {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      fa_round2<DT>(acc[j][0], acc[j][1]);
      fa_round2<DT>(acc[j][2], acc[j][3]);
    }
  }
#endif
}

// ---- cp.async ------------------------------------------------------------------------
// 16-byte global->shared copy; src_bytes = 0 zero-fills the destination.
__device__ __forceinline__ void fa_cp_async16(fa_u32 dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void fa_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void fa_cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- ldmatrix / mma.sync m16n8k16 ----------------------------------------------------
__device__ __forceinline__ void fa_ldsm_x4(fa_u32 addr, fa_u32& r0, fa_u32& r1, fa_u32& r2, fa_u32& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void fa_ldsm_x4_t(fa_u32 addr, fa_u32& r0, fa_u32& r1, fa_u32& r2, fa_u32& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
template <int DT>
__device__ __forceinline__ void fa_mma16816(float (&c)[4], const fa_u32 (&a)[4], fa_u32 b0, fa_u32 b1) {
  if (DT == FA_DT_F16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// ---- shared-memory tiles -------------------------------------------------------------
// A tile of ROWS x COLS elements is stored row-major with one 16-byte pad per row.  The
// row pitch is then 16 * odd bytes for every COLS that is a multiple of 16 (2-byte
// elements) or 8 (4-byte elements), which makes the eight 16-byte rows an ldmatrix phase
// reads fall into distinct bank groups.
template <int COLS, int ESIZE>
struct FaTile {
  static constexpr int PITCH = COLS * ESIZE + 16;  // bytes
};

// Cooperative copy of `rows` x COLS elements (global, row stride `ss` elements) into a
// padded tile.  Rows at or beyond `valid_rows` are zero-filled.  NT = threads taking part.
template <int COLS, int ESIZE, int NT>
__device__ __forceinline__ void fa_load_tile(fa_u32 smem, const char* gbase, long long row_stride_bytes,
                                             int rows, int valid_rows, int tid) {
  constexpr int CPR = COLS * ESIZE / 16;  // 16-byte chunks per row
  constexpr int PITCH = FaTile<COLS, ESIZE>::PITCH;
  const int total = rows * CPR;
  for (int i = tid; i < total; i += NT) {
    const int r = i / CPR, c = i - r * CPR;
    const bool ok = r < valid_rows;
    const char* src = gbase + (ok ? (long long)r * row_stride_bytes + c * 16 : 0);
    fa_cp_async16(smem + r * PITCH + c * 16, src, ok ? 16 : 0);
  }
}

// ---- BlockMask table access ----------------------------------------------------------
// Sequence of tiles one row of the block grid has to visit: first the partial blocks
// (mask_mod is applied), then the full blocks (mask_mod skipped).  A block of BS tokens is
// cut into tiles of T tokens; tiles that start at or beyond the sequence length S are
// dropped.  Used for the kv tiles of a q block (kv tables) and for the q tiles of a kv
// block (q tables).
struct FaWalk {
  const int* idx[2];
  int num[2];
  int ncols, BS, S, tpb;  // tpb = tiles per block
  int total;              // number of (block, tile) slots = (num[0]+num[1]) * tpb

  template <int T>
  __device__ __forceinline__ void init_dense(int S_) {
    S = S_;
    idx[0] = idx[1] = nullptr;
    num[0] = 1; num[1] = 0;
    ncols = 1; BS = 0x40000000;
    tpb = (S + T - 1) / T;
    total = tpb;
  }
  template <int T>
  __device__ __forceinline__ void init_rows(const int* num_p, const int* idx_p, const int* fnum_p, const int* fidx_p,
                                            long long row, int ncols_, int BS_, int S_) {
    S = S_; ncols = ncols_; BS = BS_;
    idx[0] = idx_p + row * ncols;
    num[0] = min(max(num_p[row], 0), ncols);
    if (fnum_p != nullptr) {
      idx[1] = fidx_p + row * ncols;
      num[1] = min(max(fnum_p[row], 0), ncols);
    } else {
      idx[1] = nullptr; num[1] = 0;
    }
    const int span = min(BS, S);
    tpb = (span + T - 1) / T;
    total = (num[0] + num[1]) * tpb;
  }
  // kv tiles for q block `qblk` of (b, h)
  template <int T>
  __device__ __forceinline__ void init_kv(const FaTables& t, int b, int h, int qblk, int Skv) {
    if (t.kv_num == nullptr) { init_dense<T>(Skv); return; }
    const int bm = t.mB == 1 ? 0 : b, hm = t.mH == 1 ? 0 : h;
    const long long row = ((long long)bm * t.mH + hm) * t.nQ + qblk;
    init_rows<T>(t.kv_num, t.kv_idx, t.full_kv_num, t.full_kv_idx, row, t.nKV, t.KVB, Skv);
  }
  // q tiles for kv block `kvblk` of (b, h)
  template <int T>
  __device__ __forceinline__ void init_q(const FaTables& t, int b, int h, int kvblk, int Sq) {
    if (t.kv_num == nullptr || t.q_num == nullptr) { init_dense<T>(Sq); return; }
    const int bm = t.mB == 1 ? 0 : b, hm = t.mH == 1 ? 0 : h;
    const long long row = ((long long)bm * t.mH + hm) * t.nKV + kvblk;
    init_rows<T>(t.q_num, t.q_idx, t.full_q_num, t.full_q_idx, row, t.nQ, t.QB, Sq);
  }
  // slot -> first token of the tile (or -1 when the tile lies beyond S); full = skip mask_mod
  template <int T>
  __device__ __forceinline__ int tile_start(int slot, bool& full) const {
    int bi = slot / tpb;
    const int ti = slot - bi * tpb;
    int which = 0;
    if (bi >= num[0]) { bi -= num[0]; which = 1; }
    full = which == 1;
    int blk = 0;
    if (idx[which] != nullptr) blk = min(max(idx[which][bi], 0), ncols - 1);
    const long long n0 = (long long)blk * BS + (long long)ti * T;
    return n0 < S ? (int)n0 : -1;
  }
  template <int T>
  __device__ __forceinline__ bool next(int& slot, int& start, bool& full) const {
    while (slot < total) {
      start = tile_start<T>(slot, full);
      ++slot;
      if (start >= 0) return true;
    }
    return false;
  }
};

// ---- warp-level tile products (one m16 row tile per warp) ----------------------------
// Accumulator layout is that of mma.sync m16n8k16: acc[nj][0..1] = row g, cols nj*8+2t+{0,1};
// acc[nj][2..3] = row g+8, same cols (g = lane/4, t = lane%4).

// A fragments of a 16 x KD row-major tile (rows row0.. of the padded smem tile)
template <int KD>
__device__ __forceinline__ void fa_load_a_frags(fa_u32 (&a)[KD / 16][4], fa_u32 sA, int pitch, int row0, int lane) {
#pragma unroll
  for (int kk = 0; kk < KD / 16; ++kk) {
    const int r = row0 + ((lane >> 3) & 1) * 8 + (lane & 7);
    const int c = kk * 16 + (lane >> 4) * 8;
    fa_ldsm_x4(sA + r * pitch + c * 2, a[kk][0], a[kk][1], a[kk][2], a[kk][3]);
  }
}
// acc[16 x NN] += A[16 x KD] * B^T, B stored [NN rows][KD cols] row-major ("NT")
template <int DT, int KD, int NN>
__device__ __forceinline__ void fa_mma_nt(float (&acc)[NN / 8][4], const fa_u32 (&a)[KD / 16][4], fa_u32 sB, int pitchB,
                                          int lane) {
#pragma unroll
  for (int kk = 0; kk < KD / 16; ++kk) {
#pragma unroll
    for (int nj = 0; nj < NN / 16; ++nj) {
      fa_u32 r0, r1, r2, r3;
      const int r = nj * 16 + (lane >> 4) * 8 + (lane & 7);
      const int c = kk * 16 + ((lane >> 3) & 1) * 8;
      fa_ldsm_x4(sB + r * pitchB + c * 2, r0, r1, r2, r3);
      fa_mma16816<DT>(acc[2 * nj], a[kk], r0, r1);
      fa_mma16816<DT>(acc[2 * nj + 1], a[kk], r2, r3);
    }
  }
}
// same, A fragments fetched from shared memory on the fly (keeps registers free)
template <int DT, int KD, int NN>
__device__ __forceinline__ void fa_mma_nt_smemA(float (&acc)[NN / 8][4], fa_u32 sA, int pitchA, int row0, fa_u32 sB,
                                                int pitchB, int lane) {
#pragma unroll
  for (int kk = 0; kk < KD / 16; ++kk) {
    fa_u32 a[4];
    {
      const int r = row0 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const int c = kk * 16 + (lane >> 4) * 8;
      fa_ldsm_x4(sA + r * pitchA + c * 2, a[0], a[1], a[2], a[3]);
    }
#pragma unroll
    for (int nj = 0; nj < NN / 16; ++nj) {
      fa_u32 r0, r1, r2, r3;
      const int r = nj * 16 + (lane >> 4) * 8 + (lane & 7);
      const int c = kk * 16 + ((lane >> 3) & 1) * 8;
      fa_ldsm_x4(sB + r * pitchB + c * 2, r0, r1, r2, r3);
      fa_mma16816<DT>(acc[2 * nj], a, r0, r1);
      fa_mma16816<DT>(acc[2 * nj + 1], a, r2, r3);
    }
  }
}
// out[16 x NN] += P[16 x KK] * B, P taken from an accumulator (rounded to DT), B stored
// [KK rows][NN cols] row-major ("NN")
template <int DT, int KK, int NN>
__device__ __forceinline__ void fa_mma_nn(float (&out)[NN / 8][4], const float (&pacc)[KK / 8][4], fa_u32 sB, int pitchB,
                                          int lane) {
#pragma unroll
  for (int kj = 0; kj < KK / 16; ++kj) {
    fa_u32 a[4];
    a[0] = fa_pack2<DT>(pacc[2 * kj][0], pacc[2 * kj][1]);
    a[1] = fa_pack2<DT>(pacc[2 * kj][2], pacc[2 * kj][3]);
    a[2] = fa_pack2<DT>(pacc[2 * kj + 1][0], pacc[2 * kj + 1][1]);
    a[3] = fa_pack2<DT>(pacc[2 * kj + 1][2], pacc[2 * kj + 1][3]);
#pragma unroll
    for (int dj = 0; dj < NN / 16; ++dj) {
      fa_u32 r0, r1, r2, r3;
      const int r = kj * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const int c = dj * 16 + (lane >> 4) * 8;
      fa_ldsm_x4_t(sB + r * pitchB + c * 2, r0, r1, r2, r3);
      fa_mma16816<DT>(out[2 * dj], a, r0, r1);
      fa_mma16816<DT>(out[2 * dj + 1], a, r2, r3);
    }
  }
}

// fp32 counterparts on plain FMA (exact fp32 products; used when the inputs are fp32)
template <int KD, int NN>
__device__ __forceinline__ void fa_simt_nt(float (&acc)[NN / 8][4], const unsigned char* A, int pitchA, int row0,
                                           const unsigned char* B, int pitchB, int lane) {
  const int r = row0 + (lane >> 2);
  for (int d4 = 0; d4 < KD / 4; ++d4) {
    const float4 qa = *(const float4*)(A + r * pitchA + d4 * 16);
    const float4 qb = *(const float4*)(A + (r + 8) * pitchA + d4 * 16);
#pragma unroll
    for (int nj = 0; nj < NN / 8; ++nj) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int c = nj * 8 + (lane & 3) * 2 + e;
        const float4 k4 = *(const float4*)(B + c * pitchB + d4 * 16);
        acc[nj][e] = fmaf(qa.x, k4.x, fmaf(qa.y, k4.y, fmaf(qa.z, k4.z, fmaf(qa.w, k4.w, acc[nj][e]))));
        acc[nj][2 + e] = fmaf(qb.x, k4.x, fmaf(qb.y, k4.y, fmaf(qb.z, k4.z, fmaf(qb.w, k4.w, acc[nj][2 + e]))));
      }
    }
  }
}
// P (accumulator) goes through a per-warp fp32 smem tile [16+][KK] with pitch pitchP
template <int KK, int NN>
__device__ __forceinline__ void fa_simt_nn(float (&out)[NN / 8][4], const float (&pacc)[KK / 8][4], unsigned char* P,
                                           int pitchP, int row0, const unsigned char* B, int pitchB, int lane) {
  const int r = row0 + (lane >> 2);
  __syncwarp();
#pragma unroll
  for (int nj = 0; nj < KK / 8; ++nj) {
    const int c = nj * 8 + (lane & 3) * 2;
    *(float2*)(P + r * pitchP + c * 4) = make_float2(pacc[nj][0], pacc[nj][1]);
    *(float2*)(P + (r + 8) * pitchP + c * 4) = make_float2(pacc[nj][2], pacc[nj][3]);
  }
  __syncwarp();
  for (int k = 0; k < KK; ++k) {
    const float pa = *(const float*)(P + r * pitchP + k * 4);
    const float pb = *(const float*)(P + (r + 8) * pitchP + k * 4);
#pragma unroll
    for (int dj = 0; dj < NN / 8; ++dj) {
      const float2 vv = *(const float2*)(B + k * pitchB + (dj * 8 + (lane & 3) * 2) * 4);
      out[dj][0] = fmaf(pa, vv.x, out[dj][0]);
      out[dj][1] = fmaf(pa, vv.y, out[dj][1]);
      out[dj][2] = fmaf(pb, vv.x, out[dj][2]);
      out[dj][3] = fmaf(pb, vv.y, out[dj][3]);
    }
  }
}

// 4-byte cp.async (used for per-row scalars such as lse / delta); src_bytes = 0 zero-fills
__device__ __forceinline__ void fa_cp_async4(fa_u32 dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// Store a 16-row accumulator tile (scaled) into a padded smem tile in the output dtype
template <int DT, int NN>
__device__ __forceinline__ void fa_store_acc(unsigned char* S, int pitch, int row0, const float (&acc)[NN / 8][4],
                                             float mul, int lane) {
  const int r = row0 + (lane >> 2);
#pragma unroll
  for (int dj = 0; dj < NN / 8; ++dj) {
    const int c = dj * 8 + (lane & 3) * 2;
    if (DT == FA_DT_F32) {
      *(float2*)(S + r * pitch + c * 4) = make_float2(acc[dj][0] * mul, acc[dj][1] * mul);
      *(float2*)(S + (r + 8) * pitch + c * 4) = make_float2(acc[dj][2] * mul, acc[dj][3] * mul);
    } else {
      *(fa_u32*)(S + r * pitch + c * 2) = fa_pack2<DT>(acc[dj][0] * mul, acc[dj][1] * mul);
      *(fa_u32*)(S + (r + 8) * pitch + c * 2) = fa_pack2<DT>(acc[dj][2] * mul, acc[dj][3] * mul);
    }
  }
}
// Cooperative copy of `valid_rows` rows of a padded smem tile to global memory
template <int COLS, int ESIZE, int NT>
__device__ __forceinline__ void fa_store_tile(char* gbase, long long row_stride_bytes, const unsigned char* S,
                                              int valid_rows, int tid) {
  constexpr int CPR = COLS * ESIZE / 16;
  constexpr int PITCH = FaTile<COLS, ESIZE>::PITCH;
  for (int i = tid; i < valid_rows * CPR; i += NT) {
    const int r = i / CPR, c = i - r * CPR;
    *(uint4*)(gbase + (long long)r * row_stride_bytes + c * 16) = *(const uint4*)(S + r * PITCH + c * 16);
  }
}
