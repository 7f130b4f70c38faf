// XLA FFI custom-call handlers over the C ABI of include/dtb200_attn.h: what a JAX build of the reference binds
// with jax.ffi in place of `pl.pallas_call` (diffusers_tpu/kernels/splash.py:496-523).
//
//   DtbAttnFwd          attention(query, key, value, kv_len, scale)            splash.py:566-650
//   DtbAttnFwdResidual  residual_attention(...) folding into (o_acc, m, l)     splash.py:665-742
//   DtbAttnFinalize     o_acc / l -> bf16 after a ring                         splash.py:367-375
//
// Handlers only unpack buffers ([B, H, S, D] row-major, as XLA lays them out) and forward; they allocate nothing
// (the forward handler uses the allocation-free entry point, since an FFI handler is handed its operand and
// result buffers and no allocator).  This file compiles only where the XLA FFI headers are on the include path
// (`jax.ffi.include_dir()`); elsewhere it is an empty translation unit.  It is not part of libdtb200_attn.so:
// build it into the extension module that registers the targets, and link that against the library.
//
// NOT COMPILED OR RUN where this repository is developed (no JAX, no XLA headers there).
#if defined(__has_include)
#if __has_include("xla/ffi/api/ffi.h")
#define DTB_HAVE_XLA_FFI 1
#endif
#endif

#ifdef DTB_HAVE_XLA_FFI

#include <cstdint>

#include <cuda_runtime_api.h>

#include "../../include/dtb200_attn.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

// Fills the shape and the contiguous [B, H, S, D] strides of one call.
template <typename QBuf, typename KBuf>
bool fill_shapes(const QBuf& q, const KBuf& k, dtb_attn_params* p) {
  const auto qd = q.dimensions();
  const auto kd = k.dimensions();
  if (qd.size() != 4 || kd.size() != 4) return false;
  p->B = static_cast<int32_t>(qd[0]);
  p->Hq = static_cast<int32_t>(qd[1]);
  p->Sq = static_cast<int32_t>(qd[2]);
  p->D = static_cast<int32_t>(qd[3]);
  p->Hkv = static_cast<int32_t>(kd[1]);
  p->Skv = static_cast<int32_t>(kd[2]);
  p->q_stride_s = p->o_stride_s = p->D;
  p->k_stride_s = p->v_stride_s = p->D;
  p->q_stride_h = p->o_stride_h = static_cast<int64_t>(p->Sq) * p->D;
  p->k_stride_h = p->v_stride_h = static_cast<int64_t>(p->Skv) * p->D;
  p->q_stride_b = p->o_stride_b = p->q_stride_h * p->Hq;
  p->k_stride_b = p->v_stride_b = p->k_stride_h * p->Hkv;
  return true;
}

ffi::Error to_error(int rc) {
  if (rc == DTB_OK) return ffi::Error::Success();
  if (rc == DTB_ERR_SHAPE || rc == DTB_ERR_DTYPE || rc == DTB_ERR_UNSUPPORTED)
    return ffi::Error::InvalidArgument(dtb_status_string(rc));
  return ffi::Error::Internal(dtb_status_string(rc));
}

// kv_len: int32 [B] valid key counts (pass S for unpadded calls); mk: f32 [2, H] or a zero-sized buffer for the
// online softmax.
ffi::Error AttnFwdImpl(cudaStream_t stream, ffi::Buffer<ffi::BF16> q, ffi::Buffer<ffi::BF16> k, ffi::Buffer<ffi::BF16> v,
                       ffi::Buffer<ffi::S32> kv_len, ffi::Buffer<ffi::F32> mk, float scale,
                       ffi::ResultBuffer<ffi::BF16> o) {
  dtb_attn_params p = {};
  if (!fill_shapes(q, k, &p)) return ffi::Error::InvalidArgument("query and key must be [B, H, S, D]");
  p.q = q.untyped_data();
  p.k = k.untyped_data();
  p.v = v.untyped_data();
  p.o = o->untyped_data();
  p.kv_len = kv_len.typed_data();
  p.scale = scale;
  p.flags = DTB_FLAG_ZERO_PADDED_ROWS;
  if (mk.element_count() > 0) {
    p.mk = mk.typed_data();
    p.flags |= DTB_FLAG_BOUNDED_LOGITS;
  }
  p.num_splits = 0;
  return to_error(dtb_attn_fwd_static_scratch(&p, stream));
}

// o_acc, m, l are input-output aliased (declare the aliasing in ffi_call's input_output_aliases); init != 0 starts
// from the empty state.
ffi::Error AttnFwdResidualImpl(cudaStream_t stream, ffi::Buffer<ffi::BF16> q, ffi::Buffer<ffi::BF16> k,
                               ffi::Buffer<ffi::BF16> v, ffi::Buffer<ffi::S32> kv_len, ffi::Buffer<ffi::F32> mk,
                               ffi::Buffer<ffi::F32> o_acc_in, ffi::Buffer<ffi::F32> m_in, ffi::Buffer<ffi::F32> l_in,
                               float scale, int32_t kv_offset, int32_t q_offset, int32_t init,
                               ffi::ResultBuffer<ffi::F32> o_acc, ffi::ResultBuffer<ffi::F32> m,
                               ffi::ResultBuffer<ffi::F32> l) {
  (void)o_acc_in;
  (void)m_in;
  (void)l_in;
  dtb_attn_params p = {};
  if (!fill_shapes(q, k, &p)) return ffi::Error::InvalidArgument("query and key must be [B, H, S, D]");
  p.q = q.untyped_data();
  p.k = k.untyped_data();
  p.v = v.untyped_data();
  p.kv_len = kv_len.typed_data();
  p.scale = scale;
  if (mk.element_count() > 0) {
    p.mk = mk.typed_data();
    p.flags |= DTB_FLAG_BOUNDED_LOGITS;
  }
  p.num_splits = 1;
  dtb_attn_residual r = {o_acc->typed_data(), m->typed_data(), l->typed_data(), kv_offset, q_offset, init};
  return to_error(dtb_attn_fwd_residual(&p, &r, stream));
}

ffi::Error AttnFinalizeImpl(cudaStream_t stream, ffi::Buffer<ffi::F32> o_acc, ffi::Buffer<ffi::F32> m,
                            ffi::Buffer<ffi::F32> l, ffi::Buffer<ffi::S32> kv_len, int32_t q_offset,
                            ffi::ResultBuffer<ffi::BF16> o) {
  const auto d = o_acc.dimensions();
  if (d.size() != 4) return ffi::Error::InvalidArgument("o_acc must be [B, H, S, D]");
  dtb_attn_params p = {};
  p.o = o->untyped_data();
  p.B = static_cast<int32_t>(d[0]);
  p.Hq = p.Hkv = static_cast<int32_t>(d[1]);
  p.Sq = p.Skv = static_cast<int32_t>(d[2]);
  p.D = static_cast<int32_t>(d[3]);
  p.o_stride_s = p.D;
  p.o_stride_h = static_cast<int64_t>(p.Sq) * p.D;
  p.o_stride_b = p.o_stride_h * p.Hq;
  p.kv_len = kv_len.typed_data();
  p.flags = DTB_FLAG_ZERO_PADDED_ROWS;
  dtb_attn_residual r = {o_acc.typed_data(), m.typed_data(), l.typed_data(), 0, q_offset, 0};
  return to_error(dtb_attn_finalize(&p, &r, stream));
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(DtbAttnFwd, AttnFwdImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>()
                                  .Arg<ffi::Buffer<ffi::S32>>()
                                  .Arg<ffi::Buffer<ffi::F32>>()
                                  .Attr<float>("scale")
                                  .Ret<ffi::Buffer<ffi::BF16>>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(DtbAttnFwdResidual, AttnFwdResidualImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>()
                                  .Arg<ffi::Buffer<ffi::S32>>()
                                  .Arg<ffi::Buffer<ffi::F32>>()
                                  .Arg<ffi::Buffer<ffi::F32>>()
                                  .Arg<ffi::Buffer<ffi::F32>>()
                                  .Arg<ffi::Buffer<ffi::F32>>()
                                  .Attr<float>("scale")
                                  .Attr<int32_t>("kv_offset")
                                  .Attr<int32_t>("q_offset")
                                  .Attr<int32_t>("init")
                                  .Ret<ffi::Buffer<ffi::F32>>()
                                  .Ret<ffi::Buffer<ffi::F32>>()
                                  .Ret<ffi::Buffer<ffi::F32>>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(DtbAttnFinalize, AttnFinalizeImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::F32>>()
                                  .Arg<ffi::Buffer<ffi::F32>>()
                                  .Arg<ffi::Buffer<ffi::F32>>()
                                  .Arg<ffi::Buffer<ffi::S32>>()
                                  .Attr<int32_t>("q_offset")
                                  .Ret<ffi::Buffer<ffi::BF16>>());

#endif  // DTB_HAVE_XLA_FFI
