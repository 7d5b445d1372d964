// jax.ffi / XLA custom-call adapters over the mxk C ABI (include/mxk.h).
//
// memorax is a JAX library: its Memoroid.scan_fn (memoroid.py:60-91) runs under jit / grad, so the way it
// reaches these kernels is an XLA custom call.  Each handler below adapts XLA's typed buffers and the
// platform stream to one C-ABI entry point; residuals and workspaces are declared as extra results so that
// XLA plans and owns them (the library allocates nothing).  Python side (one line per target):
//   jax.ffi.register_ffi_target("mxk_lru_fwd", jax.ffi.pycapsule(lib.MxkLruFwd), platform="CUDA")
// and the call sites wrap jax.ffi.ffi_call(...) in a jax.custom_vjp whose forward returns the residuals.
//
// The file compiles to nothing unless XLA's FFI header is on the include path (jaxlib ships it under
// jaxlib/include); the library build of this repository does not compile it.
#if defined(__has_include)
#if __has_include("xla/ffi/api/ffi.h")
#define MXK_HAVE_XLA_FFI 1
#endif
#endif

#ifdef MXK_HAVE_XLA_FFI
#include <cuda_runtime.h>

#include "mxk.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error ToError(int status) {
  return status == MXK_OK ? ffi::Error::Success() : ffi::Error::Internal(mxk_status_string(status));
}
template <typename B>
const float* F32(const B& b) { return reinterpret_cast<const float*>(b.untyped_data()); }
template <typename B>
float* F32Out(B& b) { return reinterpret_cast<float*>(b->untyped_data()); }

// ---- LRU / S5: complex (state, decay) scan with a time-invariant lambda (lru.py:86-95, s5.py:127-136) ----
ffi::Error LruFwd(cudaStream_t stream, ffi::Buffer<ffi::C64> lam, ffi::Buffer<ffi::C64> bu, ffi::Buffer<ffi::C64> h0,
                  ffi::Buffer<ffi::C64> a0, ffi::Buffer<ffi::U8> done, ffi::ResultBuffer<ffi::C64> h,
                  ffi::ResultBuffer<ffi::C64> a_last) {
  auto d = bu.dimensions();   // (B, T, D)
  return ToError(mxk_linrec_c64_fwd(F32(lam), 1, F32(bu), F32(h0), F32(a0), done.typed_data(), F32Out(h), F32Out(a_last),
                                    (int)d[0], (int)d[1], (int)d[2], stream));
}
// ga is (D,); `partials` is the (B, D) complex scratch XLA allocates as a third result.
ffi::Error LruBwd(cudaStream_t stream, ffi::Buffer<ffi::C64> lam, ffi::Buffer<ffi::C64> h, ffi::Buffer<ffi::C64> h0,
                  ffi::Buffer<ffi::U8> done, ffi::Buffer<ffi::C64> gh, ffi::Buffer<ffi::C64> gh_last,
                  ffi::ResultBuffer<ffi::C64> gb, ffi::ResultBuffer<ffi::C64> ga, ffi::ResultBuffer<ffi::C64> gh0,
                  ffi::ResultBuffer<ffi::C64> partials) {
  auto d = h.dimensions();
  return ToError(mxk_linrec_c64_bwd(F32(lam), 1, F32(h), F32(h0), done.typed_data(), F32(gh), F32(gh_last), F32Out(gb),
                                    F32Out(ga), F32Out(gh0), partials->untyped_data(), partials->size_bytes(),
                                    (int)d[0], (int)d[1], (int)d[2], /*conjugate=*/0, stream));
}
// The variant for hosts that cannot add the scratch result (frozen signatures): scratch inside the library.
ffi::Error LruBwdNoAlloc(cudaStream_t stream, ffi::Buffer<ffi::C64> lam, ffi::Buffer<ffi::C64> h, ffi::Buffer<ffi::C64> h0,
                         ffi::Buffer<ffi::U8> done, ffi::Buffer<ffi::C64> gh, ffi::Buffer<ffi::C64> gh_last,
                         ffi::ResultBuffer<ffi::C64> gb, ffi::ResultBuffer<ffi::C64> ga, ffi::ResultBuffer<ffi::C64> gh0) {
  auto d = h.dimensions();
  return ToError(mxk_linrec_c64_bwd_noalloc(F32(lam), F32(h), F32(h0), done.typed_data(), F32(gh), F32(gh_last), F32Out(gb),
                                            F32Out(ga), F32Out(gh0), (int)d[0], (int)d[1], (int)d[2], 0, stream));
}

// ---- real (state, decay) scan: Mamba elements, RTRL sensitivities (mamba.py:119-122, memoroid.py:114-141) ----
ffi::Error LinRecFwd(cudaStream_t stream, ffi::Buffer<ffi::F32> a, ffi::Buffer<ffi::F32> b, ffi::Buffer<ffi::F32> h0,
                     ffi::Buffer<ffi::F32> a0, ffi::Buffer<ffi::U8> done, ffi::ResultBuffer<ffi::F32> h,
                     ffi::ResultBuffer<ffi::F32> a_last) {
  auto d = b.dimensions();
  return ToError(mxk_linrec_f32_fwd(a.typed_data(), a.dimensions().size() == 1, b.typed_data(), h0.typed_data(),
                                    a0.typed_data(), done.typed_data(), h->typed_data(), a_last->typed_data(),
                                    (int)d[0], (int)d[1], (int)d[2], stream));
}
// RTRL sensitivities after the last step (memoroid.py:114-141 returns x[:, -1:]): nothing is stored per step.
ffi::Error LinRecLast(cudaStream_t stream, ffi::Buffer<ffi::F32> a, ffi::Buffer<ffi::F32> b, ffi::Buffer<ffi::F32> h0,
                      ffi::Buffer<ffi::U8> done, ffi::ResultBuffer<ffi::F32> h_last) {
  auto d = b.dimensions();
  return ToError(mxk_linrec_f32_last(a.typed_data(), a.dimensions().size() == 1, b.typed_data(), h0.typed_data(),
                                     done.typed_data(), h_last->typed_data(), (int)d[0], (int)d[1], (int)d[2], stream));
}
ffi::Error LruLast(cudaStream_t stream, ffi::Buffer<ffi::C64> lam, ffi::Buffer<ffi::C64> b, ffi::Buffer<ffi::C64> h0,
                   ffi::Buffer<ffi::U8> done, ffi::ResultBuffer<ffi::C64> h_last) {
  auto d = b.dimensions();
  return ToError(mxk_linrec_c64_last((const float*)lam.typed_data(), lam.dimensions().size() == 1,
                                     (const float*)b.typed_data(), (const float*)h0.typed_data(), done.typed_data(),
                                     (float*)h_last->typed_data(), (int)d[0], (int)d[1], (int)d[2], stream));
}
ffi::Error LinRecBwd(cudaStream_t stream, ffi::Buffer<ffi::F32> a, ffi::Buffer<ffi::F32> h, ffi::Buffer<ffi::F32> h0,
                     ffi::Buffer<ffi::U8> done, ffi::Buffer<ffi::F32> gh, ffi::Buffer<ffi::F32> gh_last,
                     ffi::ResultBuffer<ffi::F32> gb, ffi::ResultBuffer<ffi::F32> ga, ffi::ResultBuffer<ffi::F32> gh0) {
  auto d = h.dimensions();
  return ToError(mxk_linrec_f32_bwd(a.typed_data(), 0, h.typed_data(), h0.typed_data(), done.typed_data(), gh.typed_data(),
                                    gh_last.typed_data(), gb->typed_data(), ga->typed_data(), gh0->typed_data(), nullptr, 0,
                                    (int)d[0], (int)d[1], (int)d[2], stream));
}

// ---- Mamba's scan with the per-head decay un-expanded (mamba.py:109-122): a is (B,T,G); `partials` is the
//      group-gradient scratch (empty when a group is exactly 128 channels) ----
ffi::Error LinRecGroupedFwd(cudaStream_t stream, ffi::Buffer<ffi::F32> a, ffi::Buffer<ffi::F32> b, ffi::Buffer<ffi::F32> h0,
                            ffi::Buffer<ffi::F32> a0, ffi::Buffer<ffi::U8> done, ffi::ResultBuffer<ffi::F32> h,
                            ffi::ResultBuffer<ffi::F32> a_last) {
  auto d = b.dimensions();
  return ToError(mxk_linrec_f32_grouped_fwd(a.typed_data(), b.typed_data(), h0.typed_data(), a0.typed_data(), done.typed_data(),
                                            h->typed_data(), a_last->typed_data(), (int)d[0], (int)d[1], (int)d[2],
                                            (int)a.dimensions()[2], stream));
}
ffi::Error LinRecGroupedBwd(cudaStream_t stream, ffi::Buffer<ffi::F32> a, ffi::Buffer<ffi::F32> h, ffi::Buffer<ffi::F32> h0,
                            ffi::Buffer<ffi::U8> done, ffi::Buffer<ffi::F32> gh, ffi::Buffer<ffi::F32> gh_last,
                            ffi::ResultBuffer<ffi::F32> gb, ffi::ResultBuffer<ffi::F32> ga, ffi::ResultBuffer<ffi::F32> gh0,
                            ffi::ResultBuffer<ffi::F32> partials) {
  auto d = h.dimensions();
  return ToError(mxk_linrec_f32_grouped_bwd(a.typed_data(), h.typed_data(), h0.typed_data(), done.typed_data(), gh.typed_data(),
                                            gh_last.typed_data(), gb->typed_data(), ga->typed_data(), gh0->typed_data(),
                                            partials->untyped_data(), partials->size_bytes(), (int)d[0], (int)d[1], (int)d[2],
                                            (int)a.dimensions()[2], stream));
}

// ---- mLSTM scan + memory read-out (mlstm.py:163-218); `scratch` is the backward call's workspace result ----
ffi::Error MlstmFwd(cudaStream_t stream, ffi::Buffer<ffi::F32> q, ffi::Buffer<ffi::F32> k, ffi::Buffer<ffi::F32> v,
                    ffi::Buffer<ffi::F32> log_i, ffi::Buffer<ffi::F32> log_f, ffi::Buffer<ffi::F32> c0, ffi::Buffer<ffi::F32> n0,
                    ffi::Buffer<ffi::F32> m0, ffi::Buffer<ffi::F32> f0, ffi::Buffer<ffi::U8> done, ffi::ResultBuffer<ffi::F32> h,
                    ffi::ResultBuffer<ffi::F32> c_last, ffi::ResultBuffer<ffi::F32> n_last, ffi::ResultBuffer<ffi::F32> m_last,
                    ffi::ResultBuffer<ffi::F32> f_last, float eps) {
  auto d = q.dimensions();
  return ToError(mxk_mlstm_f32_fwd(q.typed_data(), k.typed_data(), v.typed_data(), log_i.typed_data(), log_f.typed_data(),
                                   c0.typed_data(), n0.typed_data(), m0.typed_data(), f0.typed_data(), done.typed_data(),
                                   h->typed_data(), c_last->typed_data(), n_last->typed_data(), m_last->typed_data(),
                                   f_last->typed_data(), (int)d[0], (int)d[1], (int)d[2], (int)d[3], eps, stream));
}
ffi::Error MlstmBwd(cudaStream_t stream, ffi::Buffer<ffi::F32> q, ffi::Buffer<ffi::F32> k, ffi::Buffer<ffi::F32> v,
                    ffi::Buffer<ffi::F32> log_i, ffi::Buffer<ffi::F32> log_f, ffi::Buffer<ffi::F32> c0, ffi::Buffer<ffi::F32> n0,
                    ffi::Buffer<ffi::F32> m0, ffi::Buffer<ffi::U8> done, ffi::Buffer<ffi::F32> dh, ffi::Buffer<ffi::F32> dc_last,
                    ffi::Buffer<ffi::F32> dn_last, ffi::Buffer<ffi::F32> dm_last, ffi::ResultBuffer<ffi::F32> dq,
                    ffi::ResultBuffer<ffi::F32> dk, ffi::ResultBuffer<ffi::F32> dv, ffi::ResultBuffer<ffi::F32> dlog_i,
                    ffi::ResultBuffer<ffi::F32> dlog_f, ffi::ResultBuffer<ffi::F32> dc0, ffi::ResultBuffer<ffi::F32> dn0,
                    ffi::ResultBuffer<ffi::F32> dm0, ffi::ResultBuffer<ffi::F32> scratch, float eps) {
  auto d = q.dimensions();
  return ToError(mxk_mlstm_f32_bwd(q.typed_data(), k.typed_data(), v.typed_data(), log_i.typed_data(), log_f.typed_data(),
                                   c0.typed_data(), n0.typed_data(), m0.typed_data(), done.typed_data(), dh.typed_data(),
                                   dc_last.typed_data(), dn_last.typed_data(), dm_last.typed_data(), dq->typed_data(),
                                   dk->typed_data(), dv->typed_data(), dlog_i->typed_data(), dlog_f->typed_data(),
                                   dc0->typed_data(), dn0->typed_data(), dm0->typed_data(), scratch->untyped_data(),
                                   scratch->size_bytes(), (int)d[0], (int)d[1], (int)d[2], (int)d[3], eps, stream));
}

// ---- the same on the tensor cores: bf16 q, k, v, h; `m_steps` and `states` are the residuals the backward call takes ----
ffi::Error MlstmTcFwd(cudaStream_t stream, ffi::Buffer<ffi::BF16> q, ffi::Buffer<ffi::BF16> k, ffi::Buffer<ffi::BF16> v,
                      ffi::Buffer<ffi::F32> log_i, ffi::Buffer<ffi::F32> log_f, ffi::Buffer<ffi::F32> c0, ffi::Buffer<ffi::F32> n0,
                      ffi::Buffer<ffi::F32> m0, ffi::Buffer<ffi::F32> f0, ffi::Buffer<ffi::U8> done, ffi::ResultBuffer<ffi::BF16> h,
                      ffi::ResultBuffer<ffi::F32> c_last, ffi::ResultBuffer<ffi::F32> n_last, ffi::ResultBuffer<ffi::F32> m_last,
                      ffi::ResultBuffer<ffi::F32> f_last, ffi::ResultBuffer<ffi::F32> m_steps, ffi::ResultBuffer<ffi::U8> states,
                      ffi::ResultBuffer<ffi::S32> status, float eps) {
  auto d = q.dimensions();
  cudaMemsetAsync(status->typed_data(), 0, sizeof(int), stream);
  return ToError(mxk_mlstm_bf16_fwd(q.untyped_data(), k.untyped_data(), v.untyped_data(), log_i.typed_data(), log_f.typed_data(),
                                    c0.typed_data(), n0.typed_data(), m0.typed_data(), f0.typed_data(), done.typed_data(),
                                    h->untyped_data(), c_last->typed_data(), n_last->typed_data(), m_last->typed_data(),
                                    f_last->typed_data(), m_steps->typed_data(), states->untyped_data(), status->typed_data(),
                                    (int)d[0], (int)d[1], (int)d[2], (int)d[3], eps, stream));
}
ffi::Error MlstmTcBwd(cudaStream_t stream, ffi::Buffer<ffi::BF16> q, ffi::Buffer<ffi::BF16> k, ffi::Buffer<ffi::BF16> v,
                      ffi::Buffer<ffi::F32> log_i, ffi::Buffer<ffi::F32> log_f, ffi::Buffer<ffi::F32> c0, ffi::Buffer<ffi::F32> n0,
                      ffi::Buffer<ffi::F32> m0, ffi::Buffer<ffi::U8> done, ffi::Buffer<ffi::BF16> dh, ffi::Buffer<ffi::F32> c_last,
                      ffi::Buffer<ffi::F32> n_last, ffi::Buffer<ffi::F32> m_steps, ffi::Buffer<ffi::U8> states,
                      ffi::Buffer<ffi::F32> dc_last, ffi::Buffer<ffi::F32> dn_last, ffi::Buffer<ffi::F32> dm_last,
                      ffi::ResultBuffer<ffi::BF16> dq, ffi::ResultBuffer<ffi::BF16> dk, ffi::ResultBuffer<ffi::BF16> dv,
                      ffi::ResultBuffer<ffi::F32> dlog_i, ffi::ResultBuffer<ffi::F32> dlog_f, ffi::ResultBuffer<ffi::F32> dc0,
                      ffi::ResultBuffer<ffi::F32> dn0, ffi::ResultBuffer<ffi::F32> dm0, ffi::ResultBuffer<ffi::S32> status, float eps) {
  auto d = q.dimensions();
  cudaMemsetAsync(status->typed_data(), 0, sizeof(int), stream);
  return ToError(mxk_mlstm_bf16_bwd(q.untyped_data(), k.untyped_data(), v.untyped_data(), log_i.typed_data(), log_f.typed_data(),
                                    c0.typed_data(), n0.typed_data(), m0.typed_data(), done.typed_data(), dh.untyped_data(),
                                    c_last.typed_data(), n_last.typed_data(), m_steps.typed_data(), states.untyped_data(),
                                    dc_last.typed_data(), dn_last.typed_data(), dm_last.typed_data(), dq->untyped_data(),
                                    dk->untyped_data(), dv->untyped_data(), dlog_i->typed_data(), dlog_f->typed_data(),
                                    dc0->typed_data(), dn0->typed_data(), dm0->typed_data(), status->typed_data(), (int)d[0],
                                    (int)d[1], (int)d[2], (int)d[3], eps, stream));
}

// ---- MinGRU log-space scan + read-out (min_gru.py:67-78) ----
ffi::Error MinGruFwd(cudaStream_t stream, ffi::Buffer<ffi::F32> ls, ffi::Buffer<ffi::F32> dec, ffi::Buffer<ffi::F32> x0,
                     ffi::Buffer<ffi::F32> a0, ffi::Buffer<ffi::U8> done, ffi::ResultBuffer<ffi::F32> x,
                     ffi::ResultBuffer<ffi::F32> y, ffi::ResultBuffer<ffi::F32> a_last) {
  auto d = ls.dimensions();
  return ToError(mxk_loglinrec_f32_fwd(ls.typed_data(), dec.typed_data(), x0.typed_data(), a0.typed_data(), done.typed_data(),
                                       x->typed_data(), y->typed_data(), a_last->typed_data(), (int)d[0], (int)d[1], (int)d[2],
                                       stream));
}
ffi::Error MinGruBwd(cudaStream_t stream, ffi::Buffer<ffi::F32> dec, ffi::Buffer<ffi::F32> x, ffi::Buffer<ffi::F32> x0,
                     ffi::Buffer<ffi::U8> done, ffi::Buffer<ffi::F32> gx, ffi::Buffer<ffi::F32> gy, ffi::Buffer<ffi::F32> gx_last,
                     ffi::ResultBuffer<ffi::F32> gls, ffi::ResultBuffer<ffi::F32> gd, ffi::ResultBuffer<ffi::F32> gx0) {
  auto d = x.dimensions();
  return ToError(mxk_loglinrec_f32_bwd(dec.typed_data(), x.typed_data(), x0.typed_data(), done.typed_data(), gx.typed_data(),
                                       gy.typed_data(), gx_last.typed_data(), gls->typed_data(), gd->typed_data(),
                                       gx0->typed_data(), (int)d[0], (int)d[1], (int)d[2], stream));
}

// ---- linear attention (linear_attention.py:62-109); `states` is the residual result of the forward call ----
ffi::Error LinAttnFwd(cudaStream_t stream, ffi::Buffer<ffi::BF16> q, ffi::Buffer<ffi::BF16> k, ffi::Buffer<ffi::BF16> v,
                      ffi::Buffer<ffi::F32> s0, ffi::Buffer<ffi::F32> z0, ffi::Buffer<ffi::U8> done,
                      ffi::ResultBuffer<ffi::BF16> o, ffi::ResultBuffer<ffi::F32> s_last, ffi::ResultBuffer<ffi::F32> z_last,
                      ffi::ResultBuffer<ffi::U8> states, ffi::ResultBuffer<ffi::S32> status, float eps) {
  auto d = q.dimensions();   // (B, T, H, d)
  cudaMemsetAsync(status->typed_data(), 0, sizeof(int), stream);
  return ToError(mxk_linattn_bf16_fwd(q.untyped_data(), k.untyped_data(), v.untyped_data(), s0.typed_data(), z0.typed_data(),
                                      done.typed_data(), o->untyped_data(), s_last->typed_data(), z_last->typed_data(),
                                      states->untyped_data(), status->typed_data(), (int)d[0], (int)d[1], (int)d[2], (int)d[3],
                                      eps, /*feature_map=*/1, stream));
}
ffi::Error LinAttnBwd(cudaStream_t stream, ffi::Buffer<ffi::BF16> q, ffi::Buffer<ffi::BF16> k, ffi::Buffer<ffi::BF16> v,
                      ffi::Buffer<ffi::BF16> d_o, ffi::Buffer<ffi::U8> states, ffi::Buffer<ffi::U8> done,
                      ffi::Buffer<ffi::F32> ds_last, ffi::Buffer<ffi::F32> dz_last, ffi::ResultBuffer<ffi::BF16> dq,
                      ffi::ResultBuffer<ffi::BF16> dk, ffi::ResultBuffer<ffi::BF16> dv, ffi::ResultBuffer<ffi::F32> ds0,
                      ffi::ResultBuffer<ffi::F32> dz0, ffi::ResultBuffer<ffi::S32> status, float eps) {
  auto d = q.dimensions();
  cudaMemsetAsync(status->typed_data(), 0, sizeof(int), stream);
  return ToError(mxk_linattn_bf16_bwd(q.untyped_data(), k.untyped_data(), v.untyped_data(), d_o.untyped_data(),
                                      states.untyped_data(), done.typed_data(), ds_last.typed_data(), dz_last.typed_data(),
                                      dq->untyped_data(), dk->untyped_data(), dv->untyped_data(), ds0->typed_data(),
                                      dz0->typed_data(), status->typed_data(), (int)d[0], (int)d[1], (int)d[2], (int)d[3], eps, 1,
                                      stream));
}

// ---- gated delta rule (new cell); `states` and `workspace` are residual results of the forward call ----
ffi::Error GDeltaFwd(cudaStream_t stream, ffi::Buffer<ffi::BF16> q, ffi::Buffer<ffi::BF16> k, ffi::Buffer<ffi::BF16> v,
                     ffi::Buffer<ffi::F32> alpha, ffi::Buffer<ffi::F32> beta, ffi::Buffer<ffi::F32> s0, ffi::Buffer<ffi::U8> done,
                     ffi::ResultBuffer<ffi::BF16> o, ffi::ResultBuffer<ffi::F32> s_last, ffi::ResultBuffer<ffi::U8> states,
                     ffi::ResultBuffer<ffi::U8> workspace, ffi::ResultBuffer<ffi::S32> status) {
  auto d = q.dimensions();
  cudaMemsetAsync(status->typed_data(), 0, sizeof(int), stream);
  return ToError(mxk_gdelta_bf16_fwd(q.untyped_data(), k.untyped_data(), v.untyped_data(), alpha.typed_data(), beta.typed_data(),
                                     s0.typed_data(), done.typed_data(), o->untyped_data(), s_last->typed_data(),
                                     states->untyped_data(), workspace->untyped_data(), workspace->size_bytes(),
                                     status->typed_data(), (int)d[0], (int)d[1], (int)d[2], (int)d[3], stream));
}
ffi::Error GDeltaBwd(cudaStream_t stream, ffi::Buffer<ffi::BF16> q, ffi::Buffer<ffi::BF16> k, ffi::Buffer<ffi::BF16> v,
                     ffi::Buffer<ffi::F32> alpha, ffi::Buffer<ffi::F32> beta, ffi::Buffer<ffi::BF16> d_o,
                     ffi::Buffer<ffi::U8> states, ffi::Buffer<ffi::U8> workspace, ffi::Buffer<ffi::U8> done,
                     ffi::Buffer<ffi::F32> ds_last, ffi::ResultBuffer<ffi::BF16> dq, ffi::ResultBuffer<ffi::BF16> dk,
                     ffi::ResultBuffer<ffi::BF16> dv, ffi::ResultBuffer<ffi::F32> dalpha, ffi::ResultBuffer<ffi::F32> dbeta,
                     ffi::ResultBuffer<ffi::F32> ds0, ffi::ResultBuffer<ffi::S32> status) {
  auto d = q.dimensions();
  cudaMemsetAsync(status->typed_data(), 0, sizeof(int), stream);
  return ToError(mxk_gdelta_bf16_bwd(q.untyped_data(), k.untyped_data(), v.untyped_data(), alpha.typed_data(), beta.typed_data(),
                                     d_o.untyped_data(), states.untyped_data(), workspace.untyped_data(), done.typed_data(),
                                     ds_last.typed_data(), dq->untyped_data(), dk->untyped_data(), dv->untyped_data(),
                                     dalpha->typed_data(), dbeta->typed_data(), ds0->typed_data(), status->typed_data(),
                                     (int)d[0], (int)d[1], (int)d[2], (int)d[3], stream));
}

}  // namespace

#define MXK_BIND_STREAM() ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>()
#define C64B ffi::Buffer<ffi::C64>
#define F32B ffi::Buffer<ffi::F32>
#define BF16B ffi::Buffer<ffi::BF16>
#define U8B ffi::Buffer<ffi::U8>
#define S32B ffi::Buffer<ffi::S32>

XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkLruFwd, LruFwd,
    MXK_BIND_STREAM().Arg<C64B>().Arg<C64B>().Arg<C64B>().Arg<C64B>().Arg<U8B>().Ret<C64B>().Ret<C64B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkLruBwd, LruBwd,
    MXK_BIND_STREAM().Arg<C64B>().Arg<C64B>().Arg<C64B>().Arg<U8B>().Arg<C64B>().Arg<C64B>()
        .Ret<C64B>().Ret<C64B>().Ret<C64B>().Ret<C64B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkLruBwdNoAlloc, LruBwdNoAlloc,
    MXK_BIND_STREAM().Arg<C64B>().Arg<C64B>().Arg<C64B>().Arg<U8B>().Arg<C64B>().Arg<C64B>()
        .Ret<C64B>().Ret<C64B>().Ret<C64B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkLinRecFwd, LinRecFwd,
    MXK_BIND_STREAM().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<U8B>().Ret<F32B>().Ret<F32B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkLinRecLast, LinRecLast,
    MXK_BIND_STREAM().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<U8B>().Ret<F32B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkLruLast, LruLast,
    MXK_BIND_STREAM().Arg<C64B>().Arg<C64B>().Arg<C64B>().Arg<U8B>().Ret<C64B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkLinRecBwd, LinRecBwd,
    MXK_BIND_STREAM().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<U8B>().Arg<F32B>().Arg<F32B>()
        .Ret<F32B>().Ret<F32B>().Ret<F32B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkLinRecGroupedFwd, LinRecGroupedFwd,
    MXK_BIND_STREAM().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<U8B>().Ret<F32B>().Ret<F32B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkLinRecGroupedBwd, LinRecGroupedBwd,
    MXK_BIND_STREAM().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<U8B>().Arg<F32B>().Arg<F32B>()
        .Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<F32B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkMlstmFwd, MlstmFwd,
    MXK_BIND_STREAM().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>()
        .Arg<F32B>().Arg<U8B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Attr<float>("eps"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkMlstmBwd, MlstmBwd,
    MXK_BIND_STREAM().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>()
        .Arg<U8B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<F32B>()
        .Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Attr<float>("eps"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkMlstmTcFwd, MlstmTcFwd,
    MXK_BIND_STREAM().Arg<BF16B>().Arg<BF16B>().Arg<BF16B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>()
        .Arg<F32B>().Arg<U8B>().Ret<BF16B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<U8B>().Ret<S32B>()
        .Attr<float>("eps"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkMlstmTcBwd, MlstmTcBwd,
    MXK_BIND_STREAM().Arg<BF16B>().Arg<BF16B>().Arg<BF16B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>()
        .Arg<U8B>().Arg<BF16B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<U8B>().Arg<F32B>().Arg<F32B>().Arg<F32B>()
        .Ret<BF16B>().Ret<BF16B>().Ret<BF16B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<S32B>()
        .Attr<float>("eps"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkMinGruFwd, MinGruFwd,
    MXK_BIND_STREAM().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<U8B>().Ret<F32B>().Ret<F32B>().Ret<F32B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkMinGruBwd, MinGruBwd,
    MXK_BIND_STREAM().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<U8B>().Arg<F32B>().Arg<F32B>().Arg<F32B>()
        .Ret<F32B>().Ret<F32B>().Ret<F32B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkLinAttnFwd, LinAttnFwd,
    MXK_BIND_STREAM().Arg<BF16B>().Arg<BF16B>().Arg<BF16B>().Arg<F32B>().Arg<F32B>().Arg<U8B>()
        .Ret<BF16B>().Ret<F32B>().Ret<F32B>().Ret<U8B>().Ret<S32B>().Attr<float>("eps"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkLinAttnBwd, LinAttnBwd,
    MXK_BIND_STREAM().Arg<BF16B>().Arg<BF16B>().Arg<BF16B>().Arg<BF16B>().Arg<U8B>().Arg<U8B>().Arg<F32B>().Arg<F32B>()
        .Ret<BF16B>().Ret<BF16B>().Ret<BF16B>().Ret<F32B>().Ret<F32B>().Ret<S32B>().Attr<float>("eps"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkGDeltaFwd, GDeltaFwd,
    MXK_BIND_STREAM().Arg<BF16B>().Arg<BF16B>().Arg<BF16B>().Arg<F32B>().Arg<F32B>().Arg<F32B>().Arg<U8B>()
        .Ret<BF16B>().Ret<F32B>().Ret<U8B>().Ret<U8B>().Ret<S32B>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(MxkGDeltaBwd, GDeltaBwd,
    MXK_BIND_STREAM().Arg<BF16B>().Arg<BF16B>().Arg<BF16B>().Arg<F32B>().Arg<F32B>().Arg<BF16B>().Arg<U8B>().Arg<U8B>()
        .Arg<U8B>().Arg<F32B>().Ret<BF16B>().Ret<BF16B>().Ret<BF16B>().Ret<F32B>().Ret<F32B>().Ret<F32B>().Ret<S32B>());

#endif  // MXK_HAVE_XLA_FFI
