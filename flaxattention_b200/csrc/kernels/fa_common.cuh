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
// Sequence of kv tiles one q tile has to visit: first the partial blocks (mask_mod is
// applied), then the full blocks (mask_mod skipped).  A block of KVB tokens is cut into
// tiles of BN tokens; tiles that start at or beyond Skv are dropped.
struct FaKvWalk {
  const int* idx[2];
  int num[2];
  int nKV, KVB, Skv, tpb;  // tpb = tiles per block
  int total;               // number of (block, tile) slots = (num[0]+num[1]) * tpb

  template <int BN>
  __device__ __forceinline__ void init(const FaTables& t, int b, int h, int qblk, int Skv_) {
    Skv = Skv_;
    if (t.kv_num == nullptr) {
      idx[0] = idx[1] = nullptr;
      num[0] = 1; num[1] = 0;
      nKV = 1; KVB = 0x40000000;
      tpb = (Skv + BN - 1) / BN;
    } else {
      const int bm = t.mB == 1 ? 0 : b, hm = t.mH == 1 ? 0 : h;
      const long long row = ((long long)bm * t.mH + hm) * t.nQ + qblk;
      nKV = t.nKV; KVB = t.KVB;
      idx[0] = t.kv_idx + row * nKV;
      num[0] = min(max(t.kv_num[row], 0), nKV);
      if (t.full_kv_num != nullptr) {
        idx[1] = t.full_kv_idx + row * nKV;
        num[1] = min(max(t.full_kv_num[row], 0), nKV);
      } else {
        idx[1] = nullptr; num[1] = 0;
      }
      const int span = min(KVB, Skv);
      tpb = (span + BN - 1) / BN;
    }
    total = (num[0] + num[1]) * tpb;
  }
  // slot -> first key of the tile (or -1 when the tile lies beyond Skv); full = skip mask_mod
  template <int BN>
  __device__ __forceinline__ int tile_start(int slot, bool& full) const {
    int bi = slot / tpb;
    const int ti = slot - bi * tpb;
    int which = 0;
    if (bi >= num[0]) { bi -= num[0]; which = 1; }
    full = which == 1;
    int blk = 0;
    if (idx[which] != nullptr) blk = min(max(idx[which][bi], 0), nKV - 1);
    const long long n0 = (long long)blk * KVB + (long long)ti * BN;
    return n0 < Skv ? (int)n0 : -1;
  }
};
