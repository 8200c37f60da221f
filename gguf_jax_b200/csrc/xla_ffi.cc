// XLA FFI adapter: exposes ggq_dequant / ggq_gemv / ggq_gemm as XLA custom-call handlers so that
// JAX can call libggq_b200.so through jax.ffi.ffi_call (this replaces the cutejax.call launches
// of the reference, src/gguf_jax/cute/q4_k.py:93-101,314-320 and cute/q4_k_gemm.py:369-391).
//
// This file needs the XLA FFI headers that ship with jaxlib:
//     g++ -std=c++17 -fPIC -shared -I"$(python -c 'import jax.ffi; print(jax.ffi.include_dir())')" \
//         -I../../include -I/usr/local/cuda/include xla_ffi.cc -L.. -lggq_b200 -o ../libggq_xla_ffi.so
// gguf_jax_b200.build.build_xla_ffi() runs exactly that when `import jax.ffi` succeeds and does
// nothing otherwise.  On an image without jaxlib it is therefore not compiled; the handlers add
// no logic of their own (argument unpacking and status mapping only), everything they call is
// covered by the ctypes-driven tests.
//
// Python side (one registration per handler, then ffi_call under jit / shard_map):
//     jax.ffi.register_ffi_target("ggq_gemv", jax.ffi.pycapsule(lib.ggq_ffi_gemv), platform="CUDA")
//     y = jax.ffi.ffi_call("ggq_gemv", jax.ShapeDtypeStruct((M, N), jnp.bfloat16))(
//             w.data, x2d, workspace, qtype=np.int32(int(w.qtype)))
// `workspace` is a uint8 device array of ggq_workspace_bytes(...) bytes, zero-filled once and passed
// to every call (the kernels leave it zeroed); XLA owns it like any other operand.
#include <cuda_runtime_api.h>

#include <cstdint>

#include "ggq.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

// ggq_status -> ffi::Error: caller mistakes become InvalidArgument, the rest Internal.
ffi::Error to_error(int32_t rc) {
  switch (rc) {
    case GGQ_OK:
      return ffi::Error::Success();
    case GGQ_BAD_QTYPE:
    case GGQ_BAD_SHAPE:
    case GGQ_MISALIGNED:
    case GGQ_BAD_DTYPE:
    case GGQ_BAD_WORKSPACE:
    case GGQ_UNSUPPORTED:
    case GGQ_NO_TABLES:
      return ffi::Error::InvalidArgument(ggq_last_error());
    default:
      return ffi::Error::Internal(ggq_last_error());
  }
}

bool out_dtype_code(ffi::DataType t, int32_t* code) {
  if (t == ffi::F32) { *code = GGQ_F32; return true; }
  if (t == ffi::BF16) { *code = GGQ_BF16; return true; }
  if (t == ffi::F16) { *code = GGQ_F16; return true; }
  return false;
}

// blocks: u8[..., row_bytes]; out: f32|bf16|f16[..., n]; attribute qtype.
ffi::Error DequantImpl(cudaStream_t stream, ffi::AnyBuffer blocks, ffi::Result<ffi::AnyBuffer> out, int32_t qtype) {
  int32_t elems = 0, bytes = 0, dt = 0;
  if (int32_t rc = ggq_type_info(qtype, &elems, &bytes)) return to_error(rc);
  if (blocks.element_type() != ffi::U8) return ffi::Error::InvalidArgument("ggq_ffi_dequant: blocks must be uint8");
  if (!out_dtype_code(out->element_type(), &dt)) return ffi::Error::InvalidArgument("ggq_ffi_dequant: output must be f32, bf16 or f16");
  const int64_t n_blocks = static_cast<int64_t>(blocks.size_bytes()) / bytes;
  if (n_blocks * bytes != static_cast<int64_t>(blocks.size_bytes()) ||
      n_blocks * elems != static_cast<int64_t>(out->element_count()))
    return ffi::Error::InvalidArgument("ggq_ffi_dequant: byte count and output size do not describe the same blocks");
  return to_error(ggq_dequant(qtype, blocks.untyped_data(), n_blocks, out->untyped_data(), dt, stream));
}

// w: u8[N, row_bytes]; x: bf16[..., K]; ws: u8[workspace bytes]; y: [..., N]; attribute qtype.
template <bool kGemm>
ffi::Error MatmulImpl(cudaStream_t stream, ffi::AnyBuffer w, ffi::AnyBuffer x, ffi::AnyBuffer ws,
                      ffi::Result<ffi::AnyBuffer> y, int32_t qtype) {
  int32_t elems = 0, bytes = 0, dt = 0;
  if (int32_t rc = ggq_type_info(qtype, &elems, &bytes)) return to_error(rc);
  if (w.element_type() != ffi::U8 || w.dimensions().size() != 2)
    return ffi::Error::InvalidArgument("ggq_ffi_matmul: w must be uint8[N, row_bytes]");
  if (x.element_type() != ffi::BF16 || x.dimensions().size() < 1)
    return ffi::Error::InvalidArgument("ggq_ffi_matmul: x must be bfloat16[..., K]");
  if (!out_dtype_code(y->element_type(), &dt)) return ffi::Error::InvalidArgument("ggq_ffi_matmul: y must be f32, bf16 or f16");
  const int64_t N = w.dimensions()[0];
  const int64_t K = x.dimensions().back();
  if (K <= 0 || w.dimensions()[1] % bytes || w.dimensions()[1] / bytes * elems != K)
    return ffi::Error::InvalidArgument("ggq_ffi_matmul: contraction mismatch between x and w");
  const int64_t M = static_cast<int64_t>(x.element_count()) / K;
  if (static_cast<int64_t>(y->element_count()) != M * N)
    return ffi::Error::InvalidArgument("ggq_ffi_matmul: y must hold M * N elements");
  auto* fn = kGemm ? &ggq_gemm : &ggq_gemv;
  return to_error(fn(qtype, w.untyped_data(), N, K, x.untyped_data(), static_cast<int32_t>(M), y->untyped_data(), dt,
                     ws.untyped_data(), ws.size_bytes(), stream));
}

}  // namespace

// None of the launchers allocates, synchronises or reads back, so the handlers may be recorded
// into XLA command buffers (CUDA graphs).
XLA_FFI_DEFINE_HANDLER_SYMBOL(ggq_ffi_dequant, DequantImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int32_t>("qtype"),
                              {ffi::Traits::kCmdBufferCompatible});

XLA_FFI_DEFINE_HANDLER_SYMBOL(ggq_ffi_gemv, MatmulImpl<false>,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int32_t>("qtype"),
                              {ffi::Traits::kCmdBufferCompatible});

XLA_FFI_DEFINE_HANDLER_SYMBOL(ggq_ffi_gemm, MatmulImpl<true>,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int32_t>("qtype"),
                              {ffi::Traits::kCmdBufferCompatible});
