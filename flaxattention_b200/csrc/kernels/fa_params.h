// Kernel parameter block shared by the host library and the run-time compiled kernels.
// Only built-in types: the same text is compiled by nvcc/g++ (host) and by NVRTC (device).
#pragma once

struct FaTensor {
  void* ptr;
  long long sb, sh, ss;  // element strides of batch, head, sequence; the head dim is contiguous
};

// BlockMask tables (layout of flaxattention/core/blockmask.py:72-119): all int32.
//   kv_num [mB,mH,nQ]   kv_idx [mB,mH,nQ,nKV]   full_* same shapes or null
//   q_num  [mB,mH,nKV]  q_idx  [mB,mH,nKV,nQ]   full_* same shapes or null
// kv_num == nullptr means "no tables": one block that spans the whole key range.
struct FaTables {
  const int* kv_num;
  const int* kv_idx;
  const int* full_kv_num;
  const int* full_kv_idx;
  const int* q_num;
  const int* q_idx;
  const int* full_q_num;
  const int* full_q_idx;
  int mB, mH;    // 1 = broadcast over batch / head
  int nQ, nKV;   // number of q / kv blocks
  int QB, KVB;   // block sizes in tokens
  // optional: mask_mod evaluated once for all positions.  Bit (kv % 32) of word
  // [((bb * mask_H + hb) * mask_rows + q) * mask_stride + kv / 32] is mask_mod(b, h, q, kv), with
  // bb = b (hb = h) or 0 where the matrix is broadcast over the batch (heads).
  // Null: the kernels evaluate mask_mod themselves on partial tiles.
  const unsigned* mask_bits;
  long long mask_stride;  // words per row (a multiple of 4: rows start on 16-byte boundaries)
  int mask_rows;          // rows per (batch, head) entry
  int mask_B, mask_H;     // entries of the matrix along batch / heads (1 = broadcast)
};

struct FaParams {
  FaTensor q, k, v, o;
  FaTensor dout, dq, dk, dv;
  float* lse;      // [B,Hq,Sq] natural-log logsumexp (forward: output or null; backward: input)
  float* delta;    // [B,Hq,Sq] backward scratch: rowsum(O * dO)
  float* part_o;   // decode scratch [B*Hq, splits, Sq, Dv] un-normalised partial outputs
  float* part_ml;  // decode scratch [B*Hq, splits, Sq, 2] running max (log2 units) and sum
  int* status;     // optional device status word; kernels OR error bits into it
  int B, Hq, Hkv, Sq, Skv, D, Dv;
  int b_off, h_off;  // global index of this shard's first batch / head (what the mods see)
  int num_splits;
  int n_q_tiles;
  float scale;
  FaTables t;
};

// Block classification grid -> ordered tables.
struct FaMaskParams {
  signed char* cls;  // [B,H,nQ,nKV]: 0 empty, 1 partial, 2 full
  int B, H, nQ, nKV, QB, KVB;
  int b_off, h_off;
};

struct FaMaskBitsParams {
  unsigned* bits;      // [B,H,Q_LEN,stride] words
  long long stride;    // words per row
  int B, H, Q_LEN, KV_LEN;
  int b_off, h_off;
};
