// XLA FFI custom-call handlers over the C ABI of libflexattn.so: what a JAX host registers so that the
// reference's three entry points stay jax.jit-able while the work runs in the sm_100a kernels.
//
// One handler per reference call site, each replacing one pl.pallas_call:
//   flexattn_fwd_ffi         flex_attention_kernel.py:173-187      (q, k, v[, doc_ids, slopes]) -> o, l, m
//   flexattn_preprocess_ffi  flex_attention_dq_bwd.py:697          (o, do) -> delta
//   flexattn_dq_ffi          flex_attention_dq_bwd.py:251-265      (q, k, v, do, l, m, delta, ...) -> dq
//   flexattn_dkv_ffi         flex_attention_dkv_kernel.py:158-172  (q, k, v, do, l, m, delta, ...) -> dk, dv
//   flexattn_mask_map_ffi    the block_mask_fn closures (masks.py) -> workspace holding the block-sparse map
//
// The CUDA stream comes from the FFI call frame; buffers are XLA's; score / mask kinds and their scalars are
// attributes, so they are compile-time constants of the jitted program exactly as the closures are in the
// reference.  The mask-map workspace is an extra RESULT of each handler (XLA allocates it; its size is
// flexattn_workspace_bytes, which the Python side asks for when it builds the call), so the library itself still
// allocates nothing.  `doc_ids` and `alibi_slopes` are always passed; a zero-sized buffer stands for "unused".
//
// This file needs the XLA FFI headers that ship inside jaxlib (jax.ffi.include_dir()).  flex_attention_tpu_b200/
// build.py compiles it into libflexattn_xla.so only when that directory can be found; the library proper never
// depends on it.
#include <cuda_runtime.h>

#include <string>

#include "../../include/flexattn.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

struct Mods {
  float sm_scale;
  int32_t score_kind;
  float softcap;
  int32_t mask_kind, window, stride, backend;
  int32_t user_score;  // handle of flexattn_user_score_create (same process, same library instance), else 0
};

ffi::Error status_to_error(int status, const char* where) {
  if (status == FLEXATTN_OK) return ffi::Error::Success();
  const std::string msg = std::string(where) + ": " + flexattn_status_string(status);
  switch (status) {
    case FLEXATTN_ERR_CUDA:
    case FLEXATTN_ERR_TIMEOUT:
      return ffi::Error::Internal(msg);
    default:
      return ffi::Error::InvalidArgument(msg);
  }
}

// Fills the shape / dtype / modifier fields from the q and k buffers ([B, H, S, D]) and the attributes.
ffi::Error describe(FlexAttnParams* p, const ffi::AnyBuffer& q, const ffi::AnyBuffer& k, const Mods& mods,
                    const ffi::AnyBuffer& doc_ids, const ffi::AnyBuffer& slopes) {
  const auto qd = q.dimensions(), kd = k.dimensions();
  if (qd.size() != 4 || kd.size() != 4) return ffi::Error::InvalidArgument("flexattn: q and k must be [B, H, S, D]");
  if (qd[0] != kd[0] || qd[1] != kd[1] || qd[3] != kd[3])
    return ffi::Error::InvalidArgument("flexattn: q and k disagree on batch, heads or head_dim");
  if (q.element_type() == ffi::DataType::BF16) p->dtype = FLEXATTN_BF16;
  else if (q.element_type() == ffi::DataType::F32) p->dtype = FLEXATTN_F32;
  else return ffi::Error::InvalidArgument("flexattn: dtype must be bfloat16 or float32");
  p->batch = static_cast<int32_t>(qd[0]);
  p->heads = static_cast<int32_t>(qd[1]);
  p->seq_q = static_cast<int32_t>(qd[2]);
  p->seq_k = static_cast<int32_t>(kd[2]);
  p->head_dim = static_cast<int32_t>(qd[3]);
  p->sm_scale = mods.sm_scale;
  p->score_kind = mods.score_kind;
  p->softcap = mods.softcap;
  p->mask_kind = mods.mask_kind;
  p->window = mods.window;
  p->stride = mods.stride;
  p->backend = mods.backend;
  p->user_score = mods.user_score;
  p->doc_ids = doc_ids.size_bytes() > 0 ? static_cast<const int32_t*>(doc_ids.untyped_data()) : nullptr;
  p->alibi_slopes = slopes.size_bytes() > 0 ? static_cast<const float*>(slopes.untyped_data()) : nullptr;
  return ffi::Error::Success();
}

// Binds the workspace result and builds the mask map into it, on the call's stream.
ffi::Error bind_and_build_map(cudaStream_t stream, FlexAttnParams* p, ffi::Result<ffi::AnyBuffer>& ws) {
  p->workspace = ws->untyped_data();
  p->workspace_bytes = ws->size_bytes();
  return status_to_error(flexattn_build_mask_map(stream, p), "flexattn_build_mask_map");
}

ffi::Error Fwd(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer doc_ids,
               ffi::AnyBuffer slopes, ffi::Result<ffi::AnyBuffer> o, ffi::Result<ffi::AnyBuffer> l,
               ffi::Result<ffi::AnyBuffer> m, ffi::Result<ffi::AnyBuffer> ws, float sm_scale, int32_t score_kind,
               float softcap, int32_t mask_kind, int32_t window, int32_t stride, int32_t backend, int32_t user_score) {
  FlexAttnParams p{};
  ffi::Error e = describe(&p, q, k, Mods{sm_scale, score_kind, softcap, mask_kind, window, stride, backend, user_score}, doc_ids, slopes);
  if (e.failure()) return e;
  p.q = q.untyped_data();
  p.k = k.untyped_data();
  p.v = v.untyped_data();
  p.o = o->untyped_data();
  p.l = static_cast<float*>(l->untyped_data());
  p.m = static_cast<float*>(m->untyped_data());
  e = bind_and_build_map(stream, &p, ws);
  if (e.failure()) return e;
  return status_to_error(flexattn_fwd(stream, &p), "flexattn_fwd");
}

ffi::Error Preprocess(cudaStream_t stream, ffi::AnyBuffer o, ffi::AnyBuffer d_o, ffi::Result<ffi::AnyBuffer> delta) {
  FlexAttnParams p{};
  ffi::AnyBuffer none = o;  // never read: kinds are NONE
  ffi::Error e = describe(&p, o, o, Mods{1.0f, FLEXATTN_SCORE_NONE, 0.f, FLEXATTN_MASK_NONE, 0, 0, FLEXATTN_BACKEND_AUTO, 0},
                          none, none);
  if (e.failure()) return e;
  p.doc_ids = nullptr;
  p.alibi_slopes = nullptr;
  p.o = o.untyped_data();
  p.d_o = d_o.untyped_data();
  p.delta = static_cast<float*>(delta->untyped_data());
  return status_to_error(flexattn_bwd_preprocess(stream, &p), "flexattn_bwd_preprocess");
}

ffi::Error Dq(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer d_o,
              ffi::AnyBuffer l, ffi::AnyBuffer m, ffi::AnyBuffer delta, ffi::AnyBuffer doc_ids, ffi::AnyBuffer slopes,
              ffi::Result<ffi::AnyBuffer> dq, ffi::Result<ffi::AnyBuffer> ws, float sm_scale, int32_t score_kind,
              float softcap, int32_t mask_kind, int32_t window, int32_t stride, int32_t backend, int32_t user_score) {
  FlexAttnParams p{};
  ffi::Error e = describe(&p, q, k, Mods{sm_scale, score_kind, softcap, mask_kind, window, stride, backend, user_score}, doc_ids, slopes);
  if (e.failure()) return e;
  p.q = q.untyped_data();
  p.k = k.untyped_data();
  p.v = v.untyped_data();
  p.d_o = d_o.untyped_data();
  p.l = static_cast<float*>(l.untyped_data());
  p.m = static_cast<float*>(m.untyped_data());
  p.delta = static_cast<float*>(delta.untyped_data());
  p.dq = dq->untyped_data();
  e = bind_and_build_map(stream, &p, ws);
  if (e.failure()) return e;
  return status_to_error(flexattn_bwd_dq(stream, &p), "flexattn_bwd_dq");
}

ffi::Error Dkv(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer d_o,
               ffi::AnyBuffer l, ffi::AnyBuffer m, ffi::AnyBuffer delta, ffi::AnyBuffer doc_ids, ffi::AnyBuffer slopes,
               ffi::Result<ffi::AnyBuffer> dk, ffi::Result<ffi::AnyBuffer> dv, ffi::Result<ffi::AnyBuffer> ws,
               float sm_scale, int32_t score_kind, float softcap, int32_t mask_kind, int32_t window, int32_t stride,
               int32_t backend, int32_t user_score) {
  FlexAttnParams p{};
  ffi::Error e = describe(&p, q, k, Mods{sm_scale, score_kind, softcap, mask_kind, window, stride, backend, user_score}, doc_ids, slopes);
  if (e.failure()) return e;
  p.q = q.untyped_data();
  p.k = k.untyped_data();
  p.v = v.untyped_data();
  p.d_o = d_o.untyped_data();
  p.l = static_cast<float*>(l.untyped_data());
  p.m = static_cast<float*>(m.untyped_data());
  p.delta = static_cast<float*>(delta.untyped_data());
  p.dk = dk->untyped_data();
  p.dv = dv->untyped_data();
  e = bind_and_build_map(stream, &p, ws);
  if (e.failure()) return e;
  return status_to_error(flexattn_bwd_dkv(stream, &p), "flexattn_bwd_dkv");
}

// Builds only the map (q and k give the shapes; their contents are not read).
ffi::Error MaskMap(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer doc_ids,
                   ffi::Result<ffi::AnyBuffer> ws, int32_t mask_kind, int32_t window, int32_t stride) {
  FlexAttnParams p{};
  ffi::Error e = describe(&p, q, k, Mods{1.0f, FLEXATTN_SCORE_NONE, 0.f, mask_kind, window, stride, FLEXATTN_BACKEND_AUTO, 0},
                          doc_ids, doc_ids);
  if (e.failure()) return e;
  p.alibi_slopes = nullptr;
  return bind_and_build_map(stream, &p, ws);
}

}  // namespace

#define FLEXATTN_MOD_ATTRS()                                                                                  \
  .Attr<float>("sm_scale").Attr<int32_t>("score_kind").Attr<float>("softcap").Attr<int32_t>("mask_kind")      \
      .Attr<int32_t>("window").Attr<int32_t>("stride").Attr<int32_t>("backend").Attr<int32_t>("user_score")

XLA_FFI_DEFINE_HANDLER_SYMBOL(flexattn_fwd_ffi, Fwd,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // q
                                  .Arg<ffi::AnyBuffer>()   // k
                                  .Arg<ffi::AnyBuffer>()   // v
                                  .Arg<ffi::AnyBuffer>()   // doc_ids (int32 [B, S]) or empty
                                  .Arg<ffi::AnyBuffer>()   // alibi_slopes (f32 [H]) or empty
                                  .Ret<ffi::AnyBuffer>()   // o
                                  .Ret<ffi::AnyBuffer>()   // l
                                  .Ret<ffi::AnyBuffer>()   // m
                                  .Ret<ffi::AnyBuffer>()   // workspace (uint8 [flexattn_workspace_bytes])
                                  FLEXATTN_MOD_ATTRS());

XLA_FFI_DEFINE_HANDLER_SYMBOL(flexattn_preprocess_ffi, Preprocess,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // o
                                  .Arg<ffi::AnyBuffer>()   // do
                                  .Ret<ffi::AnyBuffer>()); // delta

XLA_FFI_DEFINE_HANDLER_SYMBOL(flexattn_dq_ffi, Dq,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // q
                                  .Arg<ffi::AnyBuffer>()   // k
                                  .Arg<ffi::AnyBuffer>()   // v
                                  .Arg<ffi::AnyBuffer>()   // do
                                  .Arg<ffi::AnyBuffer>()   // l
                                  .Arg<ffi::AnyBuffer>()   // m
                                  .Arg<ffi::AnyBuffer>()   // delta
                                  .Arg<ffi::AnyBuffer>()   // doc_ids or empty
                                  .Arg<ffi::AnyBuffer>()   // alibi_slopes or empty
                                  .Ret<ffi::AnyBuffer>()   // dq
                                  .Ret<ffi::AnyBuffer>()   // workspace
                                  FLEXATTN_MOD_ATTRS());

XLA_FFI_DEFINE_HANDLER_SYMBOL(flexattn_dkv_ffi, Dkv,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // q
                                  .Arg<ffi::AnyBuffer>()   // k
                                  .Arg<ffi::AnyBuffer>()   // v
                                  .Arg<ffi::AnyBuffer>()   // do
                                  .Arg<ffi::AnyBuffer>()   // l
                                  .Arg<ffi::AnyBuffer>()   // m
                                  .Arg<ffi::AnyBuffer>()   // delta
                                  .Arg<ffi::AnyBuffer>()   // doc_ids or empty
                                  .Arg<ffi::AnyBuffer>()   // alibi_slopes or empty
                                  .Ret<ffi::AnyBuffer>()   // dk
                                  .Ret<ffi::AnyBuffer>()   // dv
                                  .Ret<ffi::AnyBuffer>()   // workspace
                                  FLEXATTN_MOD_ATTRS());

XLA_FFI_DEFINE_HANDLER_SYMBOL(flexattn_mask_map_ffi, MaskMap,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // q (shape only)
                                  .Arg<ffi::AnyBuffer>()   // k (shape only)
                                  .Arg<ffi::AnyBuffer>()   // doc_ids or empty
                                  .Ret<ffi::AnyBuffer>()   // workspace
                                  .Attr<int32_t>("mask_kind")
                                  .Attr<int32_t>("window")
                                  .Attr<int32_t>("stride"));
