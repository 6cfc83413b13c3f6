// jax.ffi custom-call handlers over the C ABI of include/flaxattn.h: what a JAX build binds in
// place of the reference's four pl.pallas_call sites (flaxattention/kernel/attention.py:243, :321,
// :352, :612) and of its dense mask construction (flaxattention/core/blockmask.py:277-369).
//
//   g++ -O2 -std=c++17 -shared -fPIC ffi_shim.cc -I<repo>/include \
//       -I$(python -c "import jax.ffi; print(jax.ffi.include_dir())") \
//       -L<repo>/flaxattention_b200 -lflaxattn -o libflaxattn_ffi.so
//
// This file needs the XLA FFI headers (xla/ffi/api/ffi.h), which ship with jaxlib.  Machines
// without JAX (the image this library was developed on has neither JAX nor the headers) drive the
// same C ABI through ctypes (flaxattention_b200/_cabi.py) and do not build this file;
// flaxattention_b200/csrc/build.py builds it only when jax.ffi is importable.
//
// Conventions shared by the handlers
//   - q, k, v, o (and dout, dq, dk, dv) are row-major [B, H, S, D] buffers, or [B, S, H, D] when
//     the attribute `bshd` is non-zero (the reference moves axes around its kernel instead,
//     flaxattention/core/attention.py:243-246, :312); the library reads both through strides;
//   - `module` is an fa_module* created on the Python side from the lowered mods
//     (fa_module_create) and passed as a 64-bit attribute, static under jit like the reference's
//     score_mod / mask_mod arguments (flaxattention/kernel/attention.py:166-205);
//   - BlockMask tables are int32 operand buffers; a call without a BlockMask passes buffers of
//     zero elements and has_tables = 0;
//   - workspaces are extra result buffers the Python side sizes with fa_*_workspace_bytes, so XLA
//     owns every byte and the handlers allocate nothing;
//   - errors come back as ffi::Error::Internal with fa_last_error()'s text.
#include <cstdint>

#include "flaxattn.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

int dtype_of(ffi::DataType t) {
  switch (t) {
    case ffi::DataType::F16: return FA_F16;
    case ffi::DataType::BF16: return FA_BF16;
    case ffi::DataType::F32: return FA_F32;
    default: return -1;
  }
}

// [B,H,S,D] (bshd = 0) or [B,S,H,D] (bshd = 1) row-major buffer -> strided tensor descriptor
fa_tensor tensor_of(void* ptr, int64_t H, int64_t S, int64_t D, bool bshd) {
  if (bshd) return fa_tensor{ptr, S * H * D, D, H * D};
  return fa_tensor{ptr, H * S * D, S * D, D};
}

struct Tables {
  ffi::Buffer<ffi::S32> kv_num, kv_idx, full_kv_num, full_kv_idx, q_num, q_idx, full_q_num, full_q_idx;
};

// Fills the problem description common to forward, backward and decode.
ffi::Error fill(fa_attn_params& p, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, void* o, bool bshd, float scale,
                int32_t b_offset, int32_t h_offset, int32_t flags) {
  const auto dq = q.dimensions(), dk = k.dimensions(), dv = v.dimensions();
  if (dq.size() != 4 || dk.size() != 4 || dv.size() != 4) return ffi::Error::InvalidArgument("q, k, v must be 4-dimensional");
  p = fa_attn_params{};
  p.dtype = dtype_of(q.element_type());
  if (p.dtype < 0) return ffi::Error::InvalidArgument("q, k, v must be float16, bfloat16 or float32");
  const int hs = bshd ? 2 : 1, ss = bshd ? 1 : 2;
  p.B = (int32_t)dq[0]; p.Hq = (int32_t)dq[hs]; p.Sq = (int32_t)dq[ss]; p.D = (int32_t)dq[3];
  p.Hkv = (int32_t)dk[hs]; p.Skv = (int32_t)dk[ss]; p.Dv = (int32_t)dv[3];
  p.scale = scale; p.b_offset = b_offset; p.h_offset = h_offset; p.flags = flags;
  p.q = tensor_of(q.untyped_data(), p.Hq, p.Sq, p.D, bshd);
  p.k = tensor_of(k.untyped_data(), p.Hkv, p.Skv, p.D, bshd);
  p.v = tensor_of(v.untyped_data(), p.Hkv, p.Skv, p.Dv, bshd);
  p.o = tensor_of(o, p.Hq, p.Sq, p.Dv, bshd);
  return ffi::Error::Success();
}

void fill_tables(fa_attn_params& p, const Tables& t, int32_t q_block, int32_t kv_block) {
  const auto d = t.kv_idx.dimensions();  // [mask_B, mask_H, num_q_blocks, num_kv_blocks]
  fa_block_tables& bt = p.tables;
  bt.kv_num_blocks = t.kv_num.typed_data(); bt.kv_indices = t.kv_idx.typed_data();
  bt.full_kv_num_blocks = t.full_kv_num.element_count() ? t.full_kv_num.typed_data() : nullptr;
  bt.full_kv_indices = t.full_kv_idx.element_count() ? t.full_kv_idx.typed_data() : nullptr;
  bt.q_num_blocks = t.q_num.element_count() ? t.q_num.typed_data() : nullptr;
  bt.q_indices = t.q_idx.element_count() ? t.q_idx.typed_data() : nullptr;
  bt.full_q_num_blocks = t.full_q_num.element_count() ? t.full_q_num.typed_data() : nullptr;
  bt.full_q_indices = t.full_q_idx.element_count() ? t.full_q_idx.typed_data() : nullptr;
  bt.mask_B = (int32_t)d[0]; bt.mask_H = (int32_t)d[1];
  bt.num_q_blocks = (int32_t)d[2]; bt.num_kv_blocks = (int32_t)d[3];
  bt.q_block_size = q_block; bt.kv_block_size = kv_block;
}

ffi::Error check(int rc) { return rc == FA_OK ? ffi::Error::Success() : ffi::Error::Internal(fa_last_error()); }

// ---- forward: replaces pl.pallas_call(mha_forward_kernel) (kernel/attention.py:243, :321) -------
ffi::Error FwdImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v,
                   ffi::Buffer<ffi::S32> kv_num, ffi::Buffer<ffi::S32> kv_idx, ffi::Buffer<ffi::S32> full_kv_num,
                   ffi::Buffer<ffi::S32> full_kv_idx, ffi::Result<ffi::AnyBuffer> o, ffi::Result<ffi::Buffer<ffi::F32>> lse,
                   int64_t module, float scale, int32_t bshd, int32_t has_tables, int32_t q_block, int32_t kv_block,
                   int32_t b_offset, int32_t h_offset, int32_t flags) {
  fa_attn_params p;
  if (auto e = fill(p, q, k, v, o->untyped_data(), bshd != 0, scale, b_offset, h_offset, flags); e.failure()) return e;
  p.lse = lse->typed_data();
  if (has_tables) {
    Tables t{kv_num, kv_idx, full_kv_num, full_kv_idx, kv_num, kv_idx, kv_num, kv_idx};
    fill_tables(p, t, q_block, kv_block);
    p.tables.q_num_blocks = p.tables.full_q_num_blocks = nullptr;  // the forward walks the kv tables only
    p.tables.q_indices = p.tables.full_q_indices = nullptr;
  }
  return check(fa_fwd(reinterpret_cast<fa_module*>(module), &p, stream));
}

// ---- backward: replaces _preprocess_backward + pl.pallas_call(mha_backward_kernel) --------------
// (kernel/attention.py:348-366, :612-647); operands are the reference's residual tuple
// (q, k, v, out, lse) (:335) and dout, results are (dq, dk, dv) (:650) and the workspace
ffi::Error BwdImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer out,
                   ffi::Buffer<ffi::F32> lse, ffi::AnyBuffer dout, ffi::Buffer<ffi::S32> kv_num, ffi::Buffer<ffi::S32> kv_idx,
                   ffi::Buffer<ffi::S32> full_kv_num, ffi::Buffer<ffi::S32> full_kv_idx, ffi::Buffer<ffi::S32> q_num,
                   ffi::Buffer<ffi::S32> q_idx, ffi::Buffer<ffi::S32> full_q_num, ffi::Buffer<ffi::S32> full_q_idx,
                   ffi::Result<ffi::AnyBuffer> dq, ffi::Result<ffi::AnyBuffer> dk, ffi::Result<ffi::AnyBuffer> dv,
                   ffi::Result<ffi::Buffer<ffi::U8>> workspace, int64_t module, float scale, int32_t bshd, int32_t has_tables,
                   int32_t q_block, int32_t kv_block, int32_t b_offset, int32_t h_offset, int32_t flags) {
  fa_attn_params p;
  if (auto e = fill(p, q, k, v, out.untyped_data(), bshd != 0, scale, b_offset, h_offset, flags); e.failure()) return e;
  p.lse = const_cast<float*>(lse.typed_data());
  if (has_tables) fill_tables(p, Tables{kv_num, kv_idx, full_kv_num, full_kv_idx, q_num, q_idx, full_q_num, full_q_idx}, q_block, kv_block);
  const bool b = bshd != 0;
  const fa_tensor tdo = tensor_of(dout.untyped_data(), p.Hq, p.Sq, p.Dv, b);
  const fa_tensor tdq = tensor_of(dq->untyped_data(), p.Hq, p.Sq, p.D, b);
  const fa_tensor tdk = tensor_of(dk->untyped_data(), p.Hkv, p.Skv, p.D, b);
  const fa_tensor tdv = tensor_of(dv->untyped_data(), p.Hkv, p.Skv, p.Dv, b);
  return check(fa_bwd(reinterpret_cast<fa_module*>(module), &p, &tdo, &tdq, &tdk, &tdv, workspace->typed_data(),
                      workspace->element_count(), stream));
}

// ---- decode: replaces the padded-query forward launch for short queries -------------------------
// (core/attention.py:269-273, :310-311); num_splits is static (the Python side asks
// fa_decode_num_splits) so that the workspace result has a static shape
ffi::Error DecodeImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::Buffer<ffi::S32> kv_num,
                      ffi::Buffer<ffi::S32> kv_idx, ffi::Buffer<ffi::S32> full_kv_num, ffi::Buffer<ffi::S32> full_kv_idx,
                      ffi::Result<ffi::AnyBuffer> o, ffi::Result<ffi::Buffer<ffi::F32>> lse,
                      ffi::Result<ffi::Buffer<ffi::U8>> workspace, int64_t module, float scale, int32_t bshd,
                      int32_t has_tables, int32_t q_block, int32_t kv_block, int32_t b_offset, int32_t h_offset, int32_t flags,
                      int32_t num_splits) {
  fa_attn_params p;
  if (auto e = fill(p, q, k, v, o->untyped_data(), bshd != 0, scale, b_offset, h_offset, flags); e.failure()) return e;
  p.lse = lse->typed_data();
  if (has_tables) {
    Tables t{kv_num, kv_idx, full_kv_num, full_kv_idx, kv_num, kv_idx, kv_num, kv_idx};
    fill_tables(p, t, q_block, kv_block);
    p.tables.q_num_blocks = p.tables.full_q_num_blocks = nullptr;
    p.tables.q_indices = p.tables.full_q_indices = nullptr;
  }
  return check(fa_decode(reinterpret_cast<fa_module*>(module), &p, num_splits, workspace->typed_data(),
                         workspace->element_count(), stream));
}

// ---- BlockMask construction: replaces create_mask -> _convert_mask_to_block_mask -> ------------
// _dense_to_ordered (core/blockmask.py:277-369, :57-64); eight int32 tables out, one byte of
// workspace per block
ffi::Error BlockMaskImpl(cudaStream_t stream, ffi::Result<ffi::Buffer<ffi::S32>> kv_num, ffi::Result<ffi::Buffer<ffi::S32>> kv_idx,
                         ffi::Result<ffi::Buffer<ffi::S32>> full_kv_num, ffi::Result<ffi::Buffer<ffi::S32>> full_kv_idx,
                         ffi::Result<ffi::Buffer<ffi::S32>> q_num, ffi::Result<ffi::Buffer<ffi::S32>> q_idx,
                         ffi::Result<ffi::Buffer<ffi::S32>> full_q_num, ffi::Result<ffi::Buffer<ffi::S32>> full_q_idx,
                         ffi::Result<ffi::Buffer<ffi::U8>> workspace, int64_t module, int32_t B, int32_t H, int32_t q_len,
                         int32_t kv_len, int32_t q_block, int32_t kv_block, int32_t b_offset, int32_t h_offset) {
  return check(fa_block_mask(reinterpret_cast<fa_module*>(module), B, H, q_len, kv_len, q_block, kv_block, b_offset, h_offset,
                             kv_num->typed_data(), kv_idx->typed_data(), full_kv_num->typed_data(), full_kv_idx->typed_data(),
                             q_num->typed_data(), q_idx->typed_data(), full_q_num->typed_data(), full_q_idx->typed_data(),
                             workspace->typed_data(), workspace->element_count(), stream));
}

}  // namespace

#define FA_ATTRS_COMMON                                                                                      \
  .Attr<int64_t>("module").Attr<float>("scale").Attr<int32_t>("bshd").Attr<int32_t>("has_tables")            \
      .Attr<int32_t>("q_block").Attr<int32_t>("kv_block").Attr<int32_t>("b_offset").Attr<int32_t>("h_offset") \
      .Attr<int32_t>("flags")

XLA_FFI_DEFINE_HANDLER_SYMBOL(FaFwd, FwdImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>()
                                  .Ret<ffi::AnyBuffer>().Ret<ffi::Buffer<ffi::F32>>() FA_ATTRS_COMMON);

XLA_FFI_DEFINE_HANDLER_SYMBOL(FaBwd, BwdImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::F32>>().Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>()
                                  .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::Buffer<ffi::U8>>() FA_ATTRS_COMMON);

XLA_FFI_DEFINE_HANDLER_SYMBOL(FaDecode, DecodeImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>()
                                  .Ret<ffi::AnyBuffer>().Ret<ffi::Buffer<ffi::F32>>().Ret<ffi::Buffer<ffi::U8>>()
                                      FA_ATTRS_COMMON.Attr<int32_t>("num_splits"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(FaBlockMask, BlockMaskImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Ret<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::S32>>()
                                  .Ret<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::S32>>()
                                  .Ret<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::S32>>()
                                  .Ret<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::S32>>()
                                  .Ret<ffi::Buffer<ffi::U8>>()
                                  .Attr<int64_t>("module").Attr<int32_t>("B").Attr<int32_t>("H").Attr<int32_t>("q_len")
                                  .Attr<int32_t>("kv_len").Attr<int32_t>("q_block").Attr<int32_t>("kv_block")
                                  .Attr<int32_t>("b_offset").Attr<int32_t>("h_offset"));
