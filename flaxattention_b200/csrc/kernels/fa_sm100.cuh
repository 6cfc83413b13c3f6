// Blackwell (sm_100a) primitives used by the tcgen05 attention kernels: mbarriers with
// bounded waits, TMA tile loads, TMEM allocation / load / store, tcgen05.mma descriptors.
// Self-contained (no CUDA headers), like fa_common.cuh.
#pragma once
#include "fa_common.cuh"

// 128-byte opaque tensor map (same size and alignment as the driver's CUtensorMap)
struct __align__(64) FaTensorMap {
  unsigned long long v[16];
};

// status bits a kernel ORs into FaParams::status
#define FA_STATUS_WAIT_TIMEOUT 1
#define FA_STATUS_BAD_LAUNCH 2  // launched with less dynamic shared memory or another block size than the kernel is written for

// dynamic shared memory this CTA was launched with
__device__ __forceinline__ fa_u32 fa_dynamic_smem_size() {
  fa_u32 v;
  asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(v));
  return v;
}

// ---- mbarrier --------------------------------------------------------------------------
__device__ __forceinline__ void fa_mbar_init(fa_u32 bar, fa_u32 count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fa_mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fa_mbar_arrive(fa_u32 bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fa_mbar_expect_tx(fa_u32 bar, fa_u32 bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool fa_mbar_try(fa_u32 bar, fa_u32 parity) {
  fa_u32 ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ fa_u64 fa_globaltimer() {
  fa_u64 t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up after ~2 s, or as soon as another thread of the CTA has given up
// (*abort != 0).  Returns false on failure; the caller then leaves its loop and the kernel
// tears down normally (no trap, the context stays usable, the host sees the status word).
#ifndef FA_WAIT_LIMIT_NS
#define FA_WAIT_LIMIT_NS 2000000000ull
#endif
#ifndef FA_WAIT_SLEEP_NS
#define FA_WAIT_SLEEP_NS 40
#endif
#ifndef FA_WAIT_ISSUER_SLEEP
#define FA_WAIT_ISSUER_SLEEP 0
#endif
// SLEEP: back off between polls so that waiting warps leave the issue slots of their scheduler
// to the warps that have work (the MMA issuer polls without sleeping).
template <bool SLEEP>
__device__ __forceinline__ bool fa_mbar_wait_t(fa_u32 bar, fa_u32 parity, volatile int* abort_flag) {
  if (fa_mbar_try(bar, parity)) return true;
  fa_u64 t0 = 0;
  for (fa_u32 it = 0;; ++it) {
    if (fa_mbar_try(bar, parity)) return true;
    if (SLEEP) __nanosleep(FA_WAIT_SLEEP_NS);
    if ((it & 63u) == 63u) {  // the expensive checks only now and then
      if (*abort_flag != 0) return false;
      const fa_u64 t = fa_globaltimer();
      if (t0 == 0) t0 = t;
      if (t - t0 > FA_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool fa_mbar_wait(fa_u32 bar, fa_u32 parity, volatile int* abort_flag) {
  return fa_mbar_wait_t<FA_WAIT_ISSUER_SLEEP != 0>(bar, parity, abort_flag);
}
// warp-uniform variant: every lane waits, the warp agrees on the outcome (needed before
// warp-collective tcgen05 instructions)
__device__ __forceinline__ bool fa_mbar_wait_warp(fa_u32 bar, fa_u32 parity, volatile int* abort_flag) {
  const bool ok = fa_mbar_wait_t<true>(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, ok);
}

// every lane polls (no back-off) and the warp agrees on the outcome: for a warp whose control
// flow stays uniform while one elected lane issues the tcgen05.mma instructions (every lane,
// the elected one included, has then observed the barrier itself)
__device__ __forceinline__ bool fa_mbar_wait_all(fa_u32 bar, fa_u32 parity, volatile int* abort_flag) {
  const bool ok = fa_mbar_wait_t<false>(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, ok);
}
// true in exactly one lane of a converged warp
__device__ __forceinline__ bool fa_elect_one() {
  fa_u32 pred;
  asm volatile(
      "{\n\t.reg .pred P1;\n\t.reg .b32 r;\n\t"
      "elect.sync r|P1, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- TMA -------------------------------------------------------------------------------
// 4-d tile load (coordinates innermost first), completion counted in bytes on `bar`
__device__ __forceinline__ void fa_tma_load_4d(fa_u32 dst, const FaTensorMap* map, fa_u32 bar, int c0, int c1, int c2,
                                               int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 1-d bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16)
__device__ __forceinline__ void fa_bulk_load(fa_u32 dst, const void* src, fa_u32 bytes, fa_u32 bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// tile store shared -> global (bulk async-group completion; rows beyond the tensor are clipped)
__device__ __forceinline__ void fa_tma_store_4d(const FaTensorMap* map, fa_u32 src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void fa_tma_prefetch_desc(const FaTensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- TMEM ------------------------------------------------------------------------------
// warp-collective; writes the base address of `ncols` (power of two >= 32) columns to smem
__device__ __forceinline__ void fa_tmem_alloc(fa_u32 smem_dst, fa_u32 ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void fa_tmem_dealloc(fa_u32 taddr, fa_u32 ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fa_tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fa_tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fa_tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fa_tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// each lane reads 32 consecutive 32-bit columns of its own TMEM lane (warp w may only touch
// lanes 32*(w%4) .. +31; taddr = base | lane_base << 16 | column)
__device__ __forceinline__ void fa_tmem_ld32(fa_u32 taddr, float (&v)[32]) {
  fa_u32 r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void fa_tmem_st32(fa_u32 taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
        "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
        "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
        "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
// 16 packed words (32 sixteen-bit values) per lane
__device__ __forceinline__ void fa_tmem_st16(fa_u32 taddr, const fa_u32 (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}

// ---- tcgen05.mma -----------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, 16-bit elements.  Both canonical forms
// used here have 8-row groups 1024 bytes apart (SBO); LBO is the distance between
// 64-element chunks of the MN dimension for MN-major operands (unused for K-major).
__device__ __forceinline__ fa_u64 fa_smem_desc_sw128(fa_u32 saddr, fa_u32 lbo_bytes) {
  fa_u64 d = 0;
  d |= (fa_u64)((saddr & 0x3FFFFu) >> 4);
  d |= (fa_u64)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (fa_u64)((1024u >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version of sm_100
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}
// The same descriptor split in two words, so that an issue loop can step the start address
// with one 32-bit add: high word = stride / version / swizzle (constant), low word = start
// address and MN-chunk distance, both in 16-byte units.  Stepping by `bytes` adds bytes >> 4.
__device__ __forceinline__ constexpr fa_u32 fa_desc_hi_sw128() { return (1024u >> 4) | (1u << 14) | (2u << 29); }
__device__ __forceinline__ fa_u32 fa_desc_lo(fa_u32 saddr, fa_u32 lbo_bytes) {
  return ((saddr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ fa_u64 fa_desc_make(fa_u32 lo, fa_u32 hi) {
  fa_u64 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// instruction descriptor: fp32 accumulate, A and B of type DT (0 = f16, 1 = bf16)
__device__ __forceinline__ constexpr fa_u32 fa_idesc(int dt, int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | ((fa_u32)dt << 7) | ((fa_u32)dt << 10) | ((fa_u32)a_mn_major << 15) | ((fa_u32)b_mn_major << 16) |
         ((fa_u32)(N >> 3) << 17) | ((fa_u32)(M >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void fa_mma_ss(fa_u32 d_tmem, fa_u64 a_desc, fa_u64 b_desc, fa_u32 idesc, fa_u32 accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void fa_mma_ts(fa_u32 d_tmem, fa_u32 a_tmem, fa_u64 b_desc, fa_u32 idesc, fa_u32 accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on `bar` once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void fa_mma_commit(fa_u32 bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- packed fp32 pairs and other sm_100 ALU forms -----------------------------------------
__device__ __forceinline__ fa_u64 fa_f2(float lo, float hi) {
  fa_u64 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void fa_f2_unpack(fa_u64 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ fa_u64 fa_mul2(fa_u64 a, fa_u64 b) {
  fa_u64 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ fa_u64 fa_add2(fa_u64 a, fa_u64 b) {
  fa_u64 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ fa_u64 fa_fma2(fa_u64 a, fa_u64 b, fa_u64 c) {
  fa_u64 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// 2^x for a pair of values on the FMA pipe instead of the SFU: x = n + r with n = round(x) taken
// from the mantissa of x + 1.5 * 2^23, a cubic for 2^r on [-0.5, 0.5] (Chebyshev interpolant,
// relative error 1.0e-4, below half a unit of the 16-bit types the result is rounded to), and n
// added to the exponent field.  Inputs below -125 (masked scores are -inf) give 2^-125.
__device__ __forceinline__ void fa_ex2_poly2(float x0, float x1, float& p0, float& p1) {
  const fa_u64 x = fa_f2(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
  const fa_u64 t = fa_add2(x, fa_f2(12582912.f, 12582912.f));
  const fa_u64 n = fa_add2(t, fa_f2(-12582912.f, -12582912.f));
  const fa_u64 r = fa_fma2(n, fa_f2(-1.f, -1.f), x);
  fa_u64 q = fa_fma2(r, fa_f2(0.05583828315138817f, 0.05583828315138817f), fa_f2(0.2426394820213318f, 0.2426394820213318f));
  q = fa_fma2(q, r, fa_f2(0.6931367516517639f, 0.6931367516517639f));
  q = fa_fma2(q, r, fa_f2(0.9999245405197144f, 0.9999245405197144f));
  float t0, t1, q0, q1;
  fa_f2_unpack(t, t0, t1);
  fa_f2_unpack(q, q0, q1);
  p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
  p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}
// max of three; written as nested fmaxf so that the compiler may pick the three-input form
__device__ __forceinline__ float fa_max3(float a, float b, float c) { return fmaxf(fmaxf(a, b), c); }
// register re-allocation between warpgroups (all four warps of a warpgroup must execute it)
template <int N>
__device__ __forceinline__ void fa_setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void fa_setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
// 16 columns per lane
__device__ __forceinline__ void fa_tmem_ld16(fa_u32 taddr, float (&v)[16]) {
  fa_u32 r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void fa_tmem_st16f(fa_u32 taddr, const float (&v)[16]) {
  fa_u32 r[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(v[i]);
  fa_tmem_st16(taddr, r);
}

