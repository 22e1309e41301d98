// XLA FFI handlers over libb200tri's C ABI: what FoldJAX binds with
// jax.ffi.register_ffi_target / jax.ffi.ffi_call, the route its cuEquivariance ops take
// (src/foldjax/models/_cueq.py:14-17). Each handler unpacks XLA's typed buffers into the
// POD argument struct of one entry point of include/b200tri.h and forwards the stream; it
// allocates nothing (scratch arrives as an extra result buffer XLA planned) and never
// waits on the device, so it is safe on XLA's per-device execution threads and under
// lax.scan.
//
// Needs xla/ffi/api/ffi.h, which ships inside jaxlib (jax.ffi.include_dir()).
// foldjax_b200/build.py compiles this file into libb200tri_ffi.so only when that header is
// found; without it the C ABI and everything else in this repository builds and runs as is.
#include <cstdint>

#include "b200tri.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error status(int rc) {
  if (rc == B200TRI_OK) return ffi::Error::Success();
  const ffi::ErrorCode code = rc == B200TRI_ERR_UNSUPPORTED ? ffi::ErrorCode::kUnimplemented
                              : rc == B200TRI_ERR_WORKSPACE ? ffi::ErrorCode::kResourceExhausted
                              : rc == B200TRI_ERR_CUDA      ? ffi::ErrorCode::kInternal
                                                            : ffi::ErrorCode::kInvalidArgument;
  return ffi::Error(code, b200tri_last_error());
}

int32_t dtype_code(ffi::DataType t) { return t == ffi::DataType::F32 ? B200TRI_DTYPE_F32 : B200TRI_DTYPE_BF16; }

// tokens of a pair tensor [..., n, n, c]
int32_t tokens(const ffi::AnyBuffer& x) {
  const auto d = x.dimensions();
  return static_cast<int32_t>(d[d.size() - 2]);
}

b200tri_stream_t as_stream(cudaStream_t s) { return reinterpret_cast<b200tri_stream_t>(s); }

// ------------------------------------------------------------------ triangle multiplication
ffi::Error TriMul(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer mask, ffi::AnyBuffer ln_in_s,
                  ffi::AnyBuffer ln_in_b, ffi::AnyBuffer p_in, ffi::AnyBuffer g_in, ffi::AnyBuffer ln_out_s,
                  ffi::AnyBuffer ln_out_b, ffi::AnyBuffer p_out, ffi::AnyBuffer g_out,
                  ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> scratch, int32_t incoming,
                  int32_t add_residual, float eps) {
  b200tri_trimul_args a = {};
  a.n = tokens(x);
  a.incoming = incoming;
  a.eps = eps;
  a.dtype = dtype_code(x.element_type());
  a.x = x.untyped_data();
  a.mask = mask.element_count() ? static_cast<const float*>(mask.untyped_data()) : nullptr;
  a.norm_in_scale = ln_in_s.untyped_data();
  a.norm_in_bias = ln_in_b.untyped_data();
  a.p_in = p_in.untyped_data();
  a.g_in = g_in.untyped_data();
  a.norm_out_scale = ln_out_s.untyped_data();
  a.norm_out_bias = ln_out_b.untyped_data();
  a.p_out = p_out.untyped_data();
  a.g_out = g_out.untyped_data();
  a.residual = add_residual ? x.untyped_data() : nullptr;  // z + update; out may alias x
  a.out = out->untyped_data();
  a.workspace = scratch->untyped_data();
  a.workspace_bytes = scratch->size_bytes();
  return status(b200tri_trimul_forward(&a, as_stream(stream)));
}

// ------------------------------------------------------------------ triangle attention
ffi::Error TriAtt(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer mask, ffi::AnyBuffer ln_s, ffi::AnyBuffer ln_b,
                  ffi::AnyBuffer w_bias, ffi::AnyBuffer w_q, ffi::AnyBuffer w_k, ffi::AnyBuffer w_v, ffi::AnyBuffer w_g,
                  ffi::AnyBuffer w_o, ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> scratch,
                  int32_t starting, int32_t add_residual, int32_t heads, int32_t head_dim, float inf, float eps) {
  b200tri_triatt_args a = {};
  a.n = tokens(x);
  a.starting = starting;
  a.heads = heads;
  a.head_dim = head_dim;
  a.inf = inf;
  a.eps = eps;
  a.dtype = dtype_code(x.element_type());
  a.x = x.untyped_data();
  a.mask = mask.element_count() ? static_cast<const float*>(mask.untyped_data()) : nullptr;
  a.norm_scale = ln_s.untyped_data();
  a.norm_bias = ln_b.untyped_data();
  a.w_bias = w_bias.untyped_data();
  a.w_q = w_q.untyped_data();
  a.w_k = w_k.untyped_data();
  a.w_v = w_v.untyped_data();
  a.w_g = w_g.untyped_data();
  a.w_o = w_o.untyped_data();
  a.residual = add_residual ? x.untyped_data() : nullptr;
  a.out = out->untyped_data();
  a.workspace = scratch->untyped_data();
  a.workspace_bytes = scratch->size_bytes();
  return status(b200tri_triatt_forward(&a, as_stream(stream)));
}

// ------------------------------------------------------------------ attention core
// The operator FoldJAX's fused cores implement: q, k, v [B, I, H, J, D] already laid out as the
// kernel reads them by the caller-side jnp code (q, k [I, J, H*D]; vT [I, H*D, ld] fp16; bias
// [H, J, ld]; additive mask bias [I, K] fp32).
ffi::Error AttCore(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer vt, ffi::AnyBuffer bias,
                   ffi::AnyBuffer mask_bias, ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> scratch,
                   int32_t heads, int32_t head_dim) {
  b200tri_triatt_core_args a = {};
  const auto qd = q.dimensions(), kd = k.dimensions(), vd = vt.dimensions(), bd = bias.dimensions();
  a.n_i = static_cast<int32_t>(qd[0]);
  a.n_j = static_cast<int32_t>(qd[1]);
  a.n_k = static_cast<int32_t>(kd[1]);
  a.heads = heads;
  a.head_dim = head_dim;
  a.q = q.untyped_data();
  a.k = k.untyped_data();
  a.vt = vt.untyped_data();
  a.v_ld = vd[2];
  a.bias = bias.untyped_data();
  a.bias_ld = bd[2];
  a.bias_head_stride = bd[1] * bd[2];
  a.mask = static_cast<const float*>(mask_bias.untyped_data());
  a.ms_i = a.n_k;
  a.ms_k = 1;
  a.mask_additive = 1;
  a.o = out->untyped_data();
  a.workspace = scratch->untyped_data();
  a.workspace_bytes = scratch->size_bytes();
  return status(b200tri_triatt_core(&a, as_stream(stream)));
}

// ------------------------------------------------------------------ pair transition
ffi::Error PairTransition(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer ln_s, ffi::AnyBuffer ln_b,
                          ffi::AnyBuffer fc1, ffi::AnyBuffer fc2, ffi::AnyBuffer fc3, ffi::Result<ffi::AnyBuffer> out,
                          ffi::Result<ffi::AnyBuffer> scratch, int32_t add_residual, float eps) {
  b200tri_pair_transition_args a = {};
  const auto d = x.dimensions();
  a.channels = static_cast<int32_t>(d[d.size() - 1]);
  a.rows = static_cast<int64_t>(x.element_count()) / a.channels;
  a.hidden = static_cast<int32_t>(fc1.dimensions()[1]);
  a.eps = eps;
  a.x = x.untyped_data();
  a.norm_scale = ln_s.untyped_data();
  a.norm_bias = ln_b.untyped_data();
  a.fc1 = fc1.untyped_data();
  a.fc2 = fc2.untyped_data();
  a.fc3 = fc3.untyped_data();
  a.residual = add_residual ? x.untyped_data() : nullptr;
  a.out = out->untyped_data();
  a.workspace = scratch->untyped_data();
  a.workspace_bytes = scratch->size_bytes();
  return status(b200tri_pair_transition(&a, as_stream(stream)));
}

// ------------------------------------------------------------------ 2-D context parallelism
// Inside shard_map every device runs the handler on its own tile. The communicator is
// created once per device outside the traced program (b200tri_comm_init / _init_all) and its
// address travels as a 64-bit attribute.
ffi::Error TriMulCp(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer mask, ffi::AnyBuffer ln_in_s,
                    ffi::AnyBuffer ln_in_b, ffi::AnyBuffer p_in, ffi::AnyBuffer g_in, ffi::AnyBuffer ln_out_s,
                    ffi::AnyBuffer ln_out_b, ffi::AnyBuffer p_out, ffi::AnyBuffer g_out,
                    ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> scratch, int64_t comm, int32_t tokens_n,
                    int32_t incoming, int32_t add_residual, float eps) {
  b200tri_trimul_cp_args a = {};
  a.n = tokens_n;
  a.incoming = incoming;
  a.eps = eps;
  a.x = x.untyped_data();
  a.mask = mask.element_count() ? static_cast<const float*>(mask.untyped_data()) : nullptr;
  a.norm_in_scale = ln_in_s.untyped_data();
  a.norm_in_bias = ln_in_b.untyped_data();
  a.p_in = p_in.untyped_data();
  a.g_in = g_in.untyped_data();
  a.norm_out_scale = ln_out_s.untyped_data();
  a.norm_out_bias = ln_out_b.untyped_data();
  a.p_out = p_out.untyped_data();
  a.g_out = g_out.untyped_data();
  a.residual = add_residual ? x.untyped_data() : nullptr;
  a.out = out->untyped_data();
  a.workspace = scratch->untyped_data();
  a.workspace_bytes = scratch->size_bytes();
  return status(b200tri_trimul_cp(reinterpret_cast<b200tri_comm*>(comm), &a, as_stream(stream)));
}

ffi::Error TriAttCp(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer mask, ffi::AnyBuffer ln_s,
                    ffi::AnyBuffer ln_b, ffi::AnyBuffer w_bias, ffi::AnyBuffer w_q, ffi::AnyBuffer w_k, ffi::AnyBuffer w_v,
                    ffi::AnyBuffer w_g, ffi::AnyBuffer w_o, ffi::Result<ffi::AnyBuffer> out,
                    ffi::Result<ffi::AnyBuffer> scratch, int64_t comm, int32_t tokens_n, int32_t starting,
                    int32_t add_residual, int32_t heads, int32_t head_dim, float inf, float eps) {
  b200tri_triatt_cp_args a = {};
  a.n = tokens_n;
  a.starting = starting;
  a.heads = heads;
  a.head_dim = head_dim;
  a.inf = inf;
  a.eps = eps;
  a.x = x.untyped_data();
  a.mask = mask.element_count() ? static_cast<const float*>(mask.untyped_data()) : nullptr;
  a.norm_scale = ln_s.untyped_data();
  a.norm_bias = ln_b.untyped_data();
  a.w_bias = w_bias.untyped_data();
  a.w_q = w_q.untyped_data();
  a.w_k = w_k.untyped_data();
  a.w_v = w_v.untyped_data();
  a.w_g = w_g.untyped_data();
  a.w_o = w_o.untyped_data();
  a.residual = add_residual ? x.untyped_data() : nullptr;
  a.out = out->untyped_data();
  a.workspace = scratch->untyped_data();
  a.workspace_bytes = scratch->size_bytes();
  return status(b200tri_triatt_cp(reinterpret_cast<b200tri_comm*>(comm), &a, as_stream(stream)));
}

}  // namespace

#define B200_BUFFERS_10                                                                                \
  Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>() \
      .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()

XLA_FFI_DEFINE_HANDLER_SYMBOL(b200tri_trimul, TriMul,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .B200_BUFFERS_10.Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int32_t>("incoming")
                                  .Attr<int32_t>("add_residual")
                                  .Attr<float>("eps"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(b200tri_triatt, TriAtt,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .B200_BUFFERS_10.Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int32_t>("starting")
                                  .Attr<int32_t>("add_residual")
                                  .Attr<int32_t>("heads")
                                  .Attr<int32_t>("head_dim")
                                  .Attr<float>("inf")
                                  .Attr<float>("eps"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(b200tri_att_core, AttCore,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int32_t>("heads")
                                  .Attr<int32_t>("head_dim"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(b200tri_transition, PairTransition,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int32_t>("add_residual")
                                  .Attr<float>("eps"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(b200tri_trimul_cp_ffi, TriMulCp,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .B200_BUFFERS_10.Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int64_t>("comm")
                                  .Attr<int32_t>("tokens")
                                  .Attr<int32_t>("incoming")
                                  .Attr<int32_t>("add_residual")
                                  .Attr<float>("eps"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(b200tri_triatt_cp_ffi, TriAttCp,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .B200_BUFFERS_10.Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int64_t>("comm")
                                  .Attr<int32_t>("tokens")
                                  .Attr<int32_t>("starting")
                                  .Attr<int32_t>("add_residual")
                                  .Attr<int32_t>("heads")
                                  .Attr<int32_t>("head_dim")
                                  .Attr<float>("inf")
                                  .Attr<float>("eps"));
