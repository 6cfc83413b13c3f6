/*
 * flaxattn.h - C ABI of the B200 (sm_100a) flash-attention library.
 *
 * The entry points are what a custom-call binding (jax.ffi handler, ctypes, cffi) needs
 * in place of the Pallas launches of the reference:
 *   fa_fwd          <- pl.pallas_call(mha_forward_kernel ...)     flaxattention/kernel/attention.py:243, :321
 *   fa_bwd          <- _preprocess_backward + pl.pallas_call(mha_backward_kernel ...)
 *                                                                  flaxattention/kernel/attention.py:348-366, :612-647
 *   fa_decode       <- the Sq<16 padded forward launch             flaxattention/core/attention.py:269-273, :310-311
 *   fa_block_mask   <- create_mask + _convert_mask_to_block_mask + _dense_to_ordered
 *                                                                  flaxattention/core/blockmask.py:277-369, :57-64
 *   fa_module_*     <- jax.jit tracing of score_mod / mask_mod and the Triton compile they trigger
 *                                                                  flaxattention/core/attention.py:220-230, :281-296
 *
 * Conventions
 *   - every function returns 0 on success, a negative FA_E* code otherwise; fa_last_error()
 *     gives the message of the calling thread's last failure;
 *   - the caller owns all device memory (inputs, outputs, workspaces); the library owns only
 *     compiled modules; launches are asynchronous on the given stream;
 *   - tensors are described by a base pointer and element strides for batch, head and
 *     sequence; the head dimension is contiguous.  [B,H,S,D] and [B,S,H,D] are both
 *     expressible, so no transposed copies are needed around a call;
 *   - there is no CPU implementation: without a CUDA device every compute entry point
 *     fails with FA_ECUDA.
 */
#ifndef FLAXATTN_H_
#define FLAXATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA_OK 0
#define FA_EINVAL (-1)    /* bad argument (shape, stride, alignment, null pointer) */
#define FA_ECOMPILE (-2)  /* run-time compilation of a kernel failed; see fa_last_error */
#define FA_ECUDA (-3)     /* a CUDA call failed */
#define FA_EUNSUPPORTED (-4)
#define FA_EWORKSPACE (-5) /* workspace too small */

/* Round Q.K^T to the input dtype before the scale, as the reference's dense path does
 * (flaxattention/core/attention.py:27).  Without it the fp32 product is kept, as in the
 * reference's fused kernel (flaxattention/kernel/attention.py:82).  No effect for FA_F32. */
#define FA_FLAG_ROUND_SCORES 1
/* Use the general (mma.sync) kernels even where a tcgen05 kernel covers the shape. */
#define FA_FLAG_GENERAL_KERNELS 16

enum fa_dtype { FA_F16 = 0, FA_BF16 = 1, FA_F32 = 2 };

/* kernel kinds, for fa_module_prepare */
enum fa_kind { FA_KIND_FWD = 0, FA_KIND_BWD = 1, FA_KIND_DECODE = 2, FA_KIND_BLOCKMASK = 3 };

typedef struct fa_module fa_module; /* a lowered (score_mod, mask_mod) pair and its compiled kernels */

typedef struct fa_tensor {
  void* ptr;        /* device pointer, 16-byte aligned */
  int64_t stride_b; /* element strides; all byte strides must be multiples of 16 */
  int64_t stride_h;
  int64_t stride_s;
} fa_tensor;

/* BlockMask tables, the layout of flaxattention/core/blockmask.py:72-119 (int32, device).
 * kv_num_blocks == NULL means "no block mask": every key block is visited and mask_mod,
 * if the module has one, is applied everywhere. */
typedef struct fa_block_tables {
  const int32_t* kv_num_blocks;      /* [mask_B, mask_H, num_q_blocks] */
  const int32_t* kv_indices;         /* [mask_B, mask_H, num_q_blocks, num_kv_blocks] */
  const int32_t* full_kv_num_blocks; /* same shapes, or NULL */
  const int32_t* full_kv_indices;
  const int32_t* q_num_blocks;       /* [mask_B, mask_H, num_kv_blocks]; needed by fa_bwd only */
  const int32_t* q_indices;          /* [mask_B, mask_H, num_kv_blocks, num_q_blocks] */
  const int32_t* full_q_num_blocks;
  const int32_t* full_q_indices;
  int32_t mask_B, mask_H;            /* 1 = broadcast over batch / heads */
  int32_t num_q_blocks, num_kv_blocks;
  int32_t q_block_size, kv_block_size;
  /* Optional bit matrix of mask_mod (fa_mask_bits): bit (kv % 32) of word
   * [((bb * mask_bits_H + hb) * mask_bits_rows + q) * mask_bits_stride + kv / 32], with bb / hb = 0
   * where the matrix is broadcast (mask_bits_B / mask_bits_H = 1: a mask that does not read b / h needs
   * one entry).  The kernels then read a row's words on partial tiles instead of evaluating mask_mod
   * there; results are the same.  NULL: mask_mod is evaluated in the kernels.  The matrix belongs to
   * the same mask_mod, offsets and captured buffers as the tables. */
  const uint32_t* mask_bits;
  int64_t mask_bits_stride; /* words per row, fa_mask_bits_row_words(KV_LEN) */
  int32_t mask_bits_rows;   /* rows per (batch, head) entry (Q_LEN) */
  int32_t mask_bits_B, mask_bits_H; /* 1 or B / Hq */
} fa_block_tables;

typedef struct fa_attn_params {
  int32_t dtype; /* enum fa_dtype of q, k, v, o (and dout, dq, dk, dv) */
  int32_t B, Hq, Hkv, Sq, Skv, D, Dv;
  float scale;
  int32_t b_offset, h_offset; /* global index of this shard's first batch / head: what the mods see */
  fa_tensor q, k, v, o;
  float* lse;                 /* [B,Hq,Sq] natural-log logsumexp; fwd/decode: output or NULL; bwd: input */
  fa_block_tables tables;
  int32_t flags;              /* FA_FLAG_* */
  int32_t* status;            /* optional word the GPU can address; kernels OR error bits into it (0 = clean):
                                 1 = a bounded barrier wait ran out, 2 = a launch configuration the kernel refused */
} fa_attn_params;

const char* fa_last_error(void);
int fa_version(void);

/* Directory holding the kernel templates (*.cuh).  Default: "kernels" beside the library. */
int fa_set_kernel_dir(const char* path);
/* Directory for compiled-kernel cache files.  Default: $FLAXATTN_CACHE_DIR, else ~/.cache/flaxattn_b200.
 * An empty string disables the on-disk cache. */
int fa_set_cache_dir(const char* path);

/* mod_source: CUDA text defining fa_score_mod, fa_score_mod_grad, fa_mask_mod and the macros
 * FA_HAS_SCORE_MOD / FA_HAS_MASK_MOD.  NULL or "" = identity score_mod and no mask. */
int fa_module_create(const char* mod_source, fa_module** out);
void fa_module_destroy(fa_module* m);
/* Device addresses of the buffers the mods of this module read (`fa_mod_buf[k]` in mod_source, at
 * most 8): the tensors a score_mod / mask_mod closes over and indexes with b, h, q, kv - the
 * reference's score_mod_other_buffers / mask_mod_other_buffers (flaxattention/core/attention.py:22-23,
 * :35-52), there jaxpr constants.  The addresses are copied into the kernel image, in stream order,
 * before every later launch of a kernel of the module; calls that use one module with different
 * buffer sets must not overlap, and such launches cannot be stream-captured. */
int fa_module_set_buffers(fa_module* m, const void* const* ptrs, int n);
/* Compiles (or fetches from the cache) the kernels of one kind for a dtype / head-dim pair.
 * Needs no GPU.  seq_hint selects the tile configuration the same way a later launch would. */
int fa_module_prepare(fa_module* m, int kind, int dtype, int D, int Dv, int Sq_hint, int Skv_hint);
/* Number of kernels compiled (not fetched from a cache) since the library was loaded. */
int fa_compile_count(void);

/* Self test of the bounded waits.  Every mbarrier wait of the tcgen05 kernels gives up after a time
 * limit, raises the CTA's abort flag and lets the kernel return with FA_STATUS bit 1 set in the
 * status word (the reference has no such path: its kernels are scheduled by XLA and cannot wait on
 * one another, flaxattention/kernel/attention.py:166-205).  This entry point launches one CTA of
 * two warps that wait, through the same helpers, on a barrier nobody arrives at, with the limit
 * shortened to `limit_ns` (1 us .. 100 ms).  On return (after the stream has been synchronised by
 * the caller) *status has bit 1 set, gave_up[0] = 64 threads whose wait reported failure,
 * gave_up[1] = 0, and *waited_ns is the time thread 0 spent waiting.  All three pointers are
 * device-accessible memory (device or mapped pinned host memory), zeroed by the caller. */
int fa_selftest_bounded_wait(unsigned long long limit_ns, int* status, int* gave_up, unsigned long long* waited_ns,
                             void* stream);

/* Per-kernel device times.  While enabled (process-wide switch), fa_fwd, fa_bwd and fa_decode
 * record a pair of CUDA events around every kernel they launch on the caller's stream; results
 * are unaffected.  fa_profile_read waits for the calling thread's most recent such call to finish
 * on the device and stores, in launch order, the kernel names and their durations in milliseconds
 * (at most max_kernels of them); it returns the number of kernels that call launched, or a
 * negative FA_E* code.  The names stay valid until their module is destroyed.  This is what takes
 * the place of the per-program timings a Pallas/Triton profile of the reference's launches gives
 * (flaxattention/kernel/attention.py:243, :321, :352, :612). */
int fa_profile_enable(int on);
int fa_profile_read(int max_kernels, float* ms, const char** names);

int fa_fwd(fa_module* m, const fa_attn_params* p, void* stream);

size_t fa_bwd_workspace_bytes(const fa_attn_params* p);
int fa_bwd(fa_module* m, const fa_attn_params* p, const fa_tensor* dout, const fa_tensor* dq,
           const fa_tensor* dk, const fa_tensor* dv, void* workspace, size_t workspace_bytes, void* stream);

/* Split-KV decode for Sq <= 64.  num_splits <= 0 lets the library choose; num_splits is the number of
 * partial results per row that the combine pass merges (one per CTA of a (batch, head)).
 * Grouped-query attention (Hq = G * Hkv, validated by the reference at
 * flaxattention/core/attention.py:258-265): when G * Sq <= 64 and the BlockMask tables do not
 * depend on the head (no tables, or mask_H == 1) the G query heads of a kv head are packed into
 * one tile, so K and V are read once per kv head; fa_decode_packs_heads tells whether a call
 * will do that (1) or run one CTA group per query head (0). */
int fa_decode_packs_heads(const fa_attn_params* p);
int fa_decode_num_splits(const fa_attn_params* p, int sm_count);
size_t fa_decode_workspace_bytes(const fa_attn_params* p, int num_splits);
int fa_decode(fa_module* m, const fa_attn_params* p, int num_splits, void* workspace, size_t workspace_bytes,
              void* stream);

/* fa_decode for callers that cannot allocate device memory.  (No counterpart in the reference.)
 *
 * Some hosts of this library may not call cudaMalloc around a decode step: a custom-call
 * handler that is handed only the buffers its framework planned, a serving loop whose memory
 * pool is fixed at start-up, code that runs while a stream is being captured.  For them the
 * split-KV scratch lives inside the library, in a device array of
 * fa_decode_static_capacity() bytes (16 MiB) that every GPU which loads the library keeps
 * until the process exits.  The caller passes only inputs and outputs; the call itself
 * allocates nothing and frees nothing.
 *
 * Same arguments and results as fa_decode (num_splits <= 0 lets the library choose).  A
 * problem whose scratch (fa_decode_workspace_bytes) exceeds the capacity is refused with
 * FA_EWORKSPACE and a message that names both sizes.
 *
 * First call on a device: the library looks up the device address of its scratch array
 * (with that device current) and, if this module's decode kernel has not run on the device
 * yet, compiles and loads it.  Make that first call before any stream capture begins.
 *
 * All calls share the one array.  The kernels overwrite every scratch word they later read,
 * so nothing has to be cleared between calls, but two fa_decode_static calls that can
 * overlap on the same GPU (different streams, no ordering) race on it: serialise them. */
size_t fa_decode_static_capacity(void);
int fa_decode_static(fa_module* m, const fa_attn_params* p, int num_splits, void* stream);

/* BlockMask construction.  Q_LEN / KV_LEN are the raw lengths; the block grid is
 * ceil(Q_LEN/q_block) x ceil(KV_LEN/kv_block).  Output tables have the shapes listed in
 * fa_block_tables with mask_B = B and mask_H = H.  full_* may be NULL (then blocks that are
 * entirely kept are listed with the partial ones).  workspace: B*H*nQ*nKV bytes. */
size_t fa_block_mask_workspace_bytes(int B, int H, int Q_LEN, int KV_LEN, int q_block, int kv_block);
int fa_block_mask(fa_module* m, int B, int H, int Q_LEN, int KV_LEN, int q_block, int kv_block,
                  int b_offset, int h_offset,
                  int32_t* kv_num_blocks, int32_t* kv_indices,
                  int32_t* full_kv_num_blocks, int32_t* full_kv_indices,
                  int32_t* q_num_blocks, int32_t* q_indices,
                  int32_t* full_q_num_blocks, int32_t* full_q_indices,
                  void* workspace, size_t workspace_bytes, void* stream);

/* mask_mod of every position as a bit matrix [B, H, Q_LEN, fa_mask_bits_row_words(KV_LEN)] (uint32,
 * device, 16-byte aligned) for fa_block_tables::mask_bits.  The reference materialises the boolean
 * mask itself (create_mask, flaxattention/core/blockmask.py:277-322); this is its 1-bit form and is
 * optional: it saves the kernels the evaluation of mask_mod on partial tiles. */
int64_t fa_mask_bits_row_words(int KV_LEN);
int fa_mask_bits(fa_module* m, int B, int H, int Q_LEN, int KV_LEN, int b_offset, int h_offset, uint32_t* bits,
                 void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLAXATTN_H_ */
