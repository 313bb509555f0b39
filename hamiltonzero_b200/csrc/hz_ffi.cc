// XLA FFI handlers around the C ABI of libhz_b200.so (include/hz_b200.h).
//
// This translation unit is the "thin shim" between JAX and the CUDA operators: each handler
// unpacks xla::ffi buffers into plain pointers and a shape struct, asks XLA's scratch allocator
// for the workspace where an operator needs one, calls the C entry point on the stream XLA
// hands over, and maps a non-zero status to an ffi::Error. Handlers only enqueue work: no host
// synchronisation, no allocation of their own, no global state, so XLA may call them from any
// of its execution threads.
//
// It is built (hamiltonzero_b200/build.py: build_ffi) only where jaxlib's headers are found
// (jaxlib/include/xla/ffi/api/ffi.h); nothing else in the package depends on it. The Python
// side that registers the targets and defines the differentiation rules is
// hamiltonzero_b200/jax_ffi.py. Replaces the lowerings of the reference's four attention
// primitives (src/hamiltonzero/model/_pallas_attn/mhsea_tuned.py:166-174,232-240,
// mhsea_full_ad.py:32-185) and the XLA-compiled bodies of execute_wavefunction,
// vmc_energy_custom_lap_compiled and the reverse pass (compiled/execute.py:79-118,
// energy/compiled.py:17-31, compiled/model.py:179-310).
#include <cuda_runtime.h>

#include <cstdint>
#include <optional>
#include <string>

#include "../../include/hz_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

using F32 = ffi::Buffer<ffi::F32>;
using U8 = ffi::Buffer<ffi::U8>;
using RF32 = ffi::ResultBuffer<ffi::F32>;

ffi::Error status_to_error(int status, const char* where) {
  if (status == HZ_OK) return ffi::Error::Success();
  std::string msg = std::string(where) + ": " + hz_status_string(status);
  if (status == HZ_ERR_CUDA) msg += " (cudaError " + std::to_string(hz_last_cuda_error()) + ")";
  const ffi::ErrorCode code = (status == HZ_ERR_BAD_SHAPE || status == HZ_ERR_NULL_POINTER ||
                               status == HZ_ERR_UNSUPPORTED || status == HZ_ERR_MISALIGNED)
                                  ? ffi::ErrorCode::kInvalidArgument
                                  : ffi::ErrorCode::kInternal;
  return ffi::Error(code, msg);
}

// a buffer of zero elements stands for "absent" (JAX cannot pass a null operand)
template <typename B>
auto* data_or_null(B& b) { return b.element_count() == 0 ? nullptr : b.typed_data(); }

// [..., N, H, D]: every leading axis (the batch and any axes added by vmap) folds into B, as the
// batching rules of the reference's primitives do (mhsea_tuned.py:121-163,224-229)
bool attn_shape(const F32& q, int32_t mask_mode, hz_attn_shape* s) {
  const auto dims = q.dimensions();
  if (dims.size() < 3) return false;
  int64_t b = 1;
  for (size_t i = 0; i + 3 < dims.size(); ++i) b *= dims[i];
  if (b > INT32_MAX) return false;
  s->B = (int32_t)b;
  s->N = (int32_t)dims[dims.size() - 3];
  s->H = (int32_t)dims[dims.size() - 2];
  s->D = (int32_t)dims[dims.size() - 1];
  s->mask_mode = mask_mode;
  return true;
}

ffi::Error MhseaFwd(cudaStream_t stream, F32 q, F32 k, F32 e, F32 v, U8 mask, RF32 out, RF32 lse,
                    int32_t mask_mode) {
  hz_attn_shape s;
  if (!attn_shape(q, mask_mode, &s)) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "hz_mhsea_fwd: rank");
  return status_to_error(hz_mhsea_fwd(&s, q.typed_data(), k.typed_data(), data_or_null(e), v.typed_data(),
                                      data_or_null(mask), out->typed_data(), lse->typed_data(), stream),
                         "hz_mhsea_fwd");
}

ffi::Error MhseaJvp(cudaStream_t stream, F32 q, F32 k, F32 e, F32 v, U8 mask, F32 out, F32 lse, F32 qt,
                    F32 kt, F32 et, F32 vt, RF32 tangent, int32_t mask_mode) {
  hz_attn_shape s;
  if (!attn_shape(q, mask_mode, &s)) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "hz_mhsea_jvp: rank");
  return status_to_error(
      hz_mhsea_jvp(&s, q.typed_data(), k.typed_data(), data_or_null(e), v.typed_data(), data_or_null(mask),
                   out.typed_data(), lse.typed_data(), qt.typed_data(), kt.typed_data(), data_or_null(et),
                   vt.typed_data(), tangent->typed_data(), stream),
      "hz_mhsea_jvp");
}

ffi::Error MhseaBwd(cudaStream_t stream, F32 q, F32 k, F32 e, F32 v, U8 mask, F32 lse, F32 out, F32 dout,
                    RF32 dq, RF32 dk, RF32 de, RF32 dv, int32_t mask_mode) {
  hz_attn_shape s;
  if (!attn_shape(q, mask_mode, &s)) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "hz_mhsea_bwd: rank");
  float* de_ptr = de->element_count() == 0 ? nullptr : de->typed_data();
  return status_to_error(
      hz_mhsea_bwd(&s, q.typed_data(), k.typed_data(), data_or_null(e), v.typed_data(), data_or_null(mask),
                   lse.typed_data(), out.typed_data(), dout.typed_data(), dq->typed_data(), dk->typed_data(),
                   de_ptr, dv->typed_data(), stream),
      "hz_mhsea_bwd");
}

// The compiled wavefunction travels as twelve operands, in the order of hz_wavefunction.
struct WfArgs {
  F32 q_weight, leaf_V, leaf_U, leaf_h, merge_T, merge_V, merge_U, merge_h;
  U8 opcodes;
  F32 readout_V, readout_U, readout_h;
};

bool fill_wavefunction(const WfArgs& a, float merge_eps, hz_wavefunction* w) {
  const auto qw = a.q_weight.dimensions(), lv = a.leaf_V.dimensions(), lu = a.leaf_U.dimensions(),
             lh = a.leaf_h.dimensions(), mt = a.merge_T.dimensions(), mv = a.merge_V.dimensions(),
             rv = a.readout_V.dimensions();
  if (qw.size() != 2 || lv.size() != 2 || lu.size() != 2 || lh.size() != 2 || rv.size() != 2) return false;
  w->n_sites = (int32_t)lh[0];
  w->d_o = (int32_t)qw[1];
  w->d_m = (int32_t)lu[1];
  w->r_leaf = (int32_t)lv[1];
  w->r_ro = (int32_t)rv[1];
  w->d_r = mt.size() == 4 ? (int32_t)mt[1] : 32;
  w->r_merge = mv.size() == 2 ? (int32_t)mv[1] : 4;
  w->merge_eps = merge_eps;
  w->q_weight = a.q_weight.typed_data();
  w->leaf_V = a.leaf_V.typed_data();
  w->leaf_U = a.leaf_U.typed_data();
  w->leaf_h = a.leaf_h.typed_data();
  w->merge_T = a.merge_T.element_count() ? a.merge_T.typed_data() : nullptr;
  w->merge_V = a.merge_V.element_count() ? a.merge_V.typed_data() : nullptr;
  w->merge_U = a.merge_U.element_count() ? a.merge_U.typed_data() : nullptr;
  w->merge_h = a.merge_h.element_count() ? a.merge_h.typed_data() : nullptr;
  w->opcodes = a.opcodes.element_count() ? a.opcodes.typed_data() : nullptr;
  w->readout_V = a.readout_V.typed_data();
  w->readout_U = a.readout_U.typed_data();
  w->readout_h = a.readout_h.typed_data();
  return true;
}

// walkers: every axis of q before [N, 4]
int64_t walker_count(const F32& q) {
  const auto dims = q.dimensions();
  int64_t b = 1;
  for (size_t i = 0; i + 2 < dims.size(); ++i) b *= dims[i];
  return b;
}

// Scratch for `chunk` walkers per pass from XLA's allocator (256-byte aligned).
ffi::Error take_workspace(ffi::ScratchAllocator& scratch, long long bytes, void** out) {
  if (bytes < 0) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "wavefunction extents are not supported");
  std::optional<void*> p = scratch.Allocate((size_t)bytes, 256);
  if (!p.has_value()) return ffi::Error(ffi::ErrorCode::kResourceExhausted, "scratch allocation failed");
  *out = *p;
  return ffi::Error::Success();
}

ffi::Error LogPsi(cudaStream_t stream, ffi::ScratchAllocator scratch, F32 q, F32 q_weight, F32 leaf_V,
                  F32 leaf_U, F32 leaf_h, F32 merge_T, F32 merge_V, F32 merge_U, F32 merge_h, U8 opcodes,
                  F32 readout_V, F32 readout_U, F32 readout_h, RF32 log_abs, RF32 phase, float merge_eps,
                  int64_t chunk_size) {
  hz_wavefunction w{};
  if (!fill_wavefunction({q_weight, leaf_V, leaf_U, leaf_h, merge_T, merge_V, merge_U, merge_h, opcodes,
                          readout_V, readout_U, readout_h}, merge_eps, &w))
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "hz_logpsi: wavefunction ranks");
  const int64_t B = walker_count(q);
  const long long chunk = chunk_size > 0 && chunk_size < B ? chunk_size : (B > 0 ? B : 1);
  const long long bytes = hz_walker_workspace_bytes(&w, 0, chunk);
  void* ws = nullptr;
  if (ffi::Error err = take_workspace(scratch, bytes, &ws); err.failure()) return err;
  return status_to_error(hz_logpsi(&w, q.typed_data(), B, log_abs->typed_data(), phase->typed_data(), ws,
                                   bytes, stream),
                         "hz_logpsi");
}

ffi::Error LocalEnergy(cudaStream_t stream, ffi::ScratchAllocator scratch, F32 q, F32 q_weight, F32 leaf_V,
                       F32 leaf_U, F32 leaf_h, F32 merge_T, F32 merge_V, F32 merge_U, F32 merge_h,
                       U8 opcodes, F32 readout_V, F32 readout_U, F32 readout_h, F32 J_eff, F32 one_body_field,
                       RF32 energies, RF32 log_abs, RF32 phase, RF32 grad, float merge_eps,
                       float radial_const, int64_t chunk_size) {
  hz_wavefunction w{};
  if (!fill_wavefunction({q_weight, leaf_V, leaf_U, leaf_h, merge_T, merge_V, merge_U, merge_h, opcodes,
                          readout_V, readout_U, readout_h}, merge_eps, &w))
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "hz_local_energy: wavefunction ranks");
  hz_energy_frame f{J_eff.typed_data(), one_body_field.typed_data(), radial_const};
  const int64_t B = walker_count(q);
  const long long chunk = chunk_size > 0 && chunk_size < B ? chunk_size : (B > 0 ? B : 1);
  const long long bytes = hz_walker_workspace_bytes(&w, 1, chunk);
  void* ws = nullptr;
  if (ffi::Error err = take_workspace(scratch, bytes, &ws); err.failure()) return err;
  float* grad_ptr = grad->element_count() == 0 ? nullptr : grad->typed_data();
  return status_to_error(hz_local_energy(&w, &f, q.typed_data(), B, energies->typed_data(),
                                         log_abs->typed_data(), phase->typed_data(), grad_ptr, ws, bytes,
                                         stream),
                         "hz_local_energy");
}

ffi::Error LogPsiGrad(cudaStream_t stream, ffi::ScratchAllocator scratch, F32 q, F32 q_weight, F32 leaf_V,
                      F32 leaf_U, F32 leaf_h, F32 merge_T, F32 merge_V, F32 merge_U, F32 merge_h, U8 opcodes,
                      F32 readout_V, F32 readout_U, F32 readout_h, RF32 log_abs, RF32 phase, RF32 grad,
                      float merge_eps, int64_t chunk_size) {
  hz_wavefunction w{};
  if (!fill_wavefunction({q_weight, leaf_V, leaf_U, leaf_h, merge_T, merge_V, merge_U, merge_h, opcodes,
                          readout_V, readout_U, readout_h}, merge_eps, &w))
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "hz_logpsi_grad: wavefunction ranks");
  const int64_t B = walker_count(q);
  const long long chunk = chunk_size > 0 && chunk_size < B ? chunk_size : (B > 0 ? B : 1);
  const long long bytes = hz_walker_workspace_bytes(&w, 2, chunk);
  void* ws = nullptr;
  if (ffi::Error err = take_workspace(scratch, bytes, &ws); err.failure()) return err;
  return status_to_error(hz_logpsi_grad(&w, q.typed_data(), B, log_abs->typed_data(), phase->typed_data(),
                                        grad->typed_data(), ws, bytes, stream),
                         "hz_logpsi_grad");
}

// Reverse pass: the eleven parameter gradients and dq (factor sums are requested through the C ABI
// directly; as XLA results they would be seventeen more buffers).
ffi::Error LogPsiVjp(cudaStream_t stream, ffi::ScratchAllocator scratch, F32 q, F32 cot_log_abs, F32 cot_phase,
                     F32 q_weight, F32 leaf_V, F32 leaf_U, F32 leaf_h, F32 merge_T, F32 merge_V, F32 merge_U,
                     F32 merge_h, U8 opcodes, F32 readout_V, F32 readout_U, F32 readout_h, RF32 g_q_weight,
                     RF32 g_leaf_V, RF32 g_leaf_U, RF32 g_leaf_h, RF32 g_merge_T, RF32 g_merge_V,
                     RF32 g_merge_U, RF32 g_merge_h, RF32 g_readout_V, RF32 g_readout_U, RF32 g_readout_h,
                     RF32 dq, RF32 log_abs, RF32 phase, float merge_eps, int64_t chunk_size) {
  hz_wavefunction w{};
  if (!fill_wavefunction({q_weight, leaf_V, leaf_U, leaf_h, merge_T, merge_V, merge_U, merge_h, opcodes,
                          readout_V, readout_U, readout_h}, merge_eps, &w))
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "hz_logpsi_vjp: wavefunction ranks");
  hz_wavefunction_grads g{g_q_weight->typed_data(), g_leaf_V->typed_data(), g_leaf_U->typed_data(),
                          g_leaf_h->typed_data(), g_merge_T->typed_data(), g_merge_V->typed_data(),
                          g_merge_U->typed_data(), g_merge_h->typed_data(), g_readout_V->typed_data(),
                          g_readout_U->typed_data(), g_readout_h->typed_data()};
  const int64_t B = walker_count(q);
  const long long chunk = chunk_size > 0 && chunk_size < B ? chunk_size : (B > 0 ? B : 1);
  const long long bytes = hz_vjp_workspace_bytes(&w, chunk, 0);
  void* ws = nullptr;
  if (ffi::Error err = take_workspace(scratch, bytes, &ws); err.failure()) return err;
  return status_to_error(hz_logpsi_vjp(&w, q.typed_data(), B, cot_log_abs.typed_data(), cot_phase.typed_data(),
                                       &g, nullptr, dq->typed_data(), log_abs->typed_data(),
                                       phase->typed_data(), ws, bytes, stream),
                         "hz_logpsi_vjp");
}

// binder pieces shared by the walker handlers: q, then the twelve wavefunction operands
template <typename Binder>
auto wavefunction_args(Binder b) {
  return b.template Arg<F32>().template Arg<F32>().template Arg<F32>().template Arg<F32>()
      .template Arg<F32>().template Arg<F32>().template Arg<F32>().template Arg<F32>()
      .template Arg<U8>().template Arg<F32>().template Arg<F32>().template Arg<F32>();
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    hz_ffi_mhsea_fwd, MhseaFwd,
    ffi::Ffi::Bind()
        .Ctx<ffi::PlatformStream<cudaStream_t>>()
        .Arg<F32>().Arg<F32>().Arg<F32>().Arg<F32>().Arg<U8>()
        .Ret<F32>().Ret<F32>()
        .Attr<int32_t>("mask_mode"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    hz_ffi_mhsea_jvp, MhseaJvp,
    ffi::Ffi::Bind()
        .Ctx<ffi::PlatformStream<cudaStream_t>>()
        .Arg<F32>().Arg<F32>().Arg<F32>().Arg<F32>().Arg<U8>().Arg<F32>().Arg<F32>()
        .Arg<F32>().Arg<F32>().Arg<F32>().Arg<F32>()
        .Ret<F32>()
        .Attr<int32_t>("mask_mode"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    hz_ffi_mhsea_bwd, MhseaBwd,
    ffi::Ffi::Bind()
        .Ctx<ffi::PlatformStream<cudaStream_t>>()
        .Arg<F32>().Arg<F32>().Arg<F32>().Arg<F32>().Arg<U8>().Arg<F32>().Arg<F32>().Arg<F32>()
        .Ret<F32>().Ret<F32>().Ret<F32>().Ret<F32>()
        .Attr<int32_t>("mask_mode"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    hz_ffi_logpsi, LogPsi,
    wavefunction_args(ffi::Ffi::Bind()
                          .Ctx<ffi::PlatformStream<cudaStream_t>>()
                          .Ctx<ffi::ScratchAllocator>()
                          .Arg<F32>())
        .Ret<F32>().Ret<F32>()
        .Attr<float>("merge_eps")
        .Attr<int64_t>("chunk_size"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    hz_ffi_local_energy, LocalEnergy,
    wavefunction_args(ffi::Ffi::Bind()
                          .Ctx<ffi::PlatformStream<cudaStream_t>>()
                          .Ctx<ffi::ScratchAllocator>()
                          .Arg<F32>())
        .Arg<F32>().Arg<F32>()
        .Ret<F32>().Ret<F32>().Ret<F32>().Ret<F32>()
        .Attr<float>("merge_eps")
        .Attr<float>("radial_const")
        .Attr<int64_t>("chunk_size"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    hz_ffi_logpsi_grad, LogPsiGrad,
    wavefunction_args(ffi::Ffi::Bind()
                          .Ctx<ffi::PlatformStream<cudaStream_t>>()
                          .Ctx<ffi::ScratchAllocator>()
                          .Arg<F32>())
        .Ret<F32>().Ret<F32>().Ret<F32>()
        .Attr<float>("merge_eps")
        .Attr<int64_t>("chunk_size"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    hz_ffi_logpsi_vjp, LogPsiVjp,
    wavefunction_args(ffi::Ffi::Bind()
                          .Ctx<ffi::PlatformStream<cudaStream_t>>()
                          .Ctx<ffi::ScratchAllocator>()
                          .Arg<F32>().Arg<F32>().Arg<F32>())
        .Ret<F32>().Ret<F32>().Ret<F32>().Ret<F32>().Ret<F32>().Ret<F32>().Ret<F32>().Ret<F32>()
        .Ret<F32>().Ret<F32>().Ret<F32>()
        .Ret<F32>().Ret<F32>().Ret<F32>()
        .Attr<float>("merge_eps")
        .Attr<int64_t>("chunk_size"));
