// Block classification for create_block_mask.  Replaces the dense-mask route of
// flaxattention/core/blockmask.py:277-369 (create_mask -> reshape -> block sums): one CTA
// evaluates mask_mod on the QB x KVB positions of one block and writes its class
// (0 = no position kept, 1 = some, 2 = all) without materialising the [B,H,Q,KV] mask.
// Positions beyond Q_LEN / KV_LEN are evaluated like any other, because the reference
// classifies on the lengths rounded up to whole blocks (core/blockmask.py:440-444).
// The mod fragment (fa_mask_mod, FA_HAS_MASK_MOD) is placed before this file.
#pragma once
#include "fa_params.h"

extern "C" __global__ void __launch_bounds__(256) fa_blockmask_classify_kernel(const __grid_constant__ FaMaskParams p) {
  const int kvb = blockIdx.x, qb = blockIdx.y;
  const int bh = blockIdx.z;
  const int b = bh / p.H, h = bh - b * p.H;
  const long long total = (long long)p.QB * p.KVB;
  int cnt = 0;
#if FA_HAS_MASK_MOD
  const int gb = b + p.b_off, gh = h + p.h_off;
  const int q0 = qb * p.QB, k0 = kvb * p.KVB;
  for (long long i = threadIdx.x; i < total; i += 256) {
    const int qi = (int)(i / p.KVB);
    const int kj = (int)(i - (long long)qi * p.KVB);
    cnt += fa_mask_mod(gb, gh, q0 + qi, k0 + kj) ? 1 : 0;
  }
#else
  for (long long i = threadIdx.x; i < total; i += 256) cnt += 1;
#endif
  __shared__ long long s_cnt;
  if (threadIdx.x == 0) s_cnt = 0;
  __syncthreads();
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if ((threadIdx.x & 31) == 0) atomicAdd((unsigned long long*)&s_cnt, (unsigned long long)cnt);
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long c = s_cnt;
    p.cls[(((long long)b * p.H + h) * p.nQ + qb) * p.nKV + kvb] = (signed char)(c == 0 ? 0 : (c == total ? 2 : 1));
  }
}

// mask_mod of every (query, key) position as a bit matrix: one word (32 keys) per thread, bits of
// keys beyond KV_LEN and the padding words of a row are 0.  The attention kernels read a row's words
// on the tiles the BlockMask lists as partial instead of evaluating mask_mod 128 times per row
// there (the reference materialises the whole boolean mask for the same purpose,
// flaxattention/core/blockmask.py:277-322; this is 1 bit per position).
extern "C" __global__ void __launch_bounds__(256) fa_mask_bits_kernel(const __grid_constant__ FaMaskBitsParams p) {
  const long long w = (long long)blockIdx.x * 256 + threadIdx.x;  // word inside the row
  const int q = blockIdx.y;
  const int bh = blockIdx.z;
  if (w >= p.stride) return;
  const int b = bh / p.H, h = bh - b * p.H;
  unsigned m = 0;
#if FA_HAS_MASK_MOD
  const int gb = b + p.b_off, gh = h + p.h_off;
  const long long k0 = w * 32;
#pragma unroll 4
  for (int e = 0; e < 32; ++e) {
    const long long kv = k0 + e;
    if (kv < p.KV_LEN && fa_mask_mod(gb, gh, q, (int)kv)) m |= 1u << e;
  }
#else
  const long long left = (long long)p.KV_LEN - w * 32;
  m = left >= 32 ? 0xffffffffu : (left <= 0 ? 0u : ((1u << (int)left) - 1u));
#endif
  p.bits[(((long long)b * p.H + h) * p.Q_LEN + q) * p.stride + w] = m;
}
