// XLA FFI handlers for the C ABI of include/qwix_b200.h: the glue through which
// `jax.ffi.ffi_call` reaches the kernels.  One handler per entry point that touches device
// memory; buffers become pointers, attributes become scalars, the stream comes from the
// platform, a non-zero status becomes an ffi::Error carrying qwx_status_string().
//
// This translation unit needs the XLA FFI headers that ship with jaxlib
// (`jaxlib/include/xla/ffi/api/ffi.h`).  Where they are absent it compiles to nothing, so the
// library builds the same with or without them; build it on a jax machine with
//   g++ -shared -fPIC -I$(python -c 'import jaxlib,os;print(os.path.join(os.path.dirname(jaxlib.__file__),"include"))')
//       -Iinclude qwix_b200/csrc/xla_ffi_shim.cc -Lqwix_b200 -lqwix_b200 -o libqwix_b200_ffi.so
// and register every `*_ffi` symbol with
//   jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(getattr(lib, name)), platform="CUDA").
//
// Buffers and scratch are XLA's: every workspace is a result buffer of the custom call, sized
// on the host with the matching qwx_*_workspace_bytes query.  The library never allocates.
#if defined(__has_include)
#if __has_include("xla/ffi/api/ffi.h")
#define QWX_HAVE_XLA_FFI 1
#endif
#endif

#ifdef QWX_HAVE_XLA_FFI

#include <cstdint>

#include "../../include/qwix_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;
using Buf = ffi::AnyBuffer;
using Out = ffi::Result<ffi::AnyBuffer>;
struct CUstream_st;
typedef CUstream_st* cudaStream_t;

namespace {

ffi::Error Status(int rc) {
  if (rc == QWX_OK) return ffi::Error::Success();
  const ffi::ErrorCode code =
      (rc == QWX_ERR_SHAPE || rc == QWX_ERR_ALIGN || rc == QWX_ERR_DTYPE || rc == QWX_ERR_NULL)
          ? ffi::ErrorCode::kInvalidArgument
          : (rc == QWX_ERR_UNSUPPORTED ? ffi::ErrorCode::kUnimplemented : ffi::ErrorCode::kInternal);
  return ffi::Error(code, qwx_status_string(rc));
}

qwx_stream_t S(cudaStream_t s) { return reinterpret_cast<qwx_stream_t>(s); }

int FloatCode(ffi::DataType t) {
  switch (t) {
    case ffi::DataType::F32: return QWX_F32;
    case ffi::DataType::BF16: return QWX_BF16;
    case ffi::DataType::F16: return QWX_F16;
    default: return -1;
  }
}

// The code dtype of a buffer of quantized values.  XLA:GPU is believed to keep S4 arrays packed
// two per byte, but that is a layout decision of the compiler: the byte size of the buffer
// decides between the packed (QWX_S4) and the byte-per-code (QWX_S4U) form, anything else is
// refused.
int CodeDtype(const ffi::AnyBuffer& q, int64_t elements, int* out) {
  switch (q.element_type()) {
    case ffi::DataType::S8: *out = QWX_S8; return QWX_OK;
    case ffi::DataType::F8E4M3FN: *out = QWX_E4M3; return QWX_OK;
    case ffi::DataType::S4:
      if ((int64_t)q.size_bytes() * 2 == elements) { *out = QWX_S4; return QWX_OK; }
      if ((int64_t)q.size_bytes() == elements) { *out = QWX_S4U; return QWX_OK; }
      return QWX_ERR_SHAPE;
    default: return QWX_ERR_DTYPE;
  }
}

void* OptionalData(const ffi::AnyBuffer& b) { return b.element_count() == 0 ? nullptr : b.untyped_data(); }

// ---- quantize / dequantize: operands are given as the collapsed [P, R, C] view --------------

ffi::Error QuantizeImpl(cudaStream_t stream, Buf x, Out q, Out scale, Out zero_point, Out workspace,
                        int64_t P, int64_t R, int64_t C, int64_t tp, int64_t tr, int64_t tc,
                        int32_t method, int32_t has_arg, double arg, int32_t rounding) {
  int qtype = 0;
  if (int rc = CodeDtype(*q, P * R * C, &qtype)) return Status(rc);
  return Status(qwx_quantize(x.untyped_data(), FloatCode(x.element_type()), P, R, C, tp, tr, tc, method,
                             has_arg, arg, qtype, rounding, q->untyped_data(), scale->untyped_data(),
                             OptionalData(*zero_point), workspace->untyped_data(),
                             workspace->size_bytes(), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_quantize_ffi, QuantizeImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Ret<Buf>().Ret<Buf>().Ret<Buf>().Ret<Buf>()
        .Attr<int64_t>("P").Attr<int64_t>("R").Attr<int64_t>("C").Attr<int64_t>("tp").Attr<int64_t>("tr")
        .Attr<int64_t>("tc").Attr<int32_t>("method").Attr<int32_t>("has_arg").Attr<double>("arg")
        .Attr<int32_t>("rounding"));

ffi::Error CalibrateImpl(cudaStream_t stream, Buf x, Out out_a, Out out_b, Out workspace, int64_t P,
                         int64_t R, int64_t C, int64_t tp, int64_t tr, int64_t tc, int32_t method,
                         int32_t has_arg, double arg) {
  return Status(qwx_calibrate(x.untyped_data(), FloatCode(x.element_type()), P, R, C, tp, tr, tc, method,
                              has_arg, arg, out_a->untyped_data(), OptionalData(*out_b),
                              workspace->untyped_data(), workspace->size_bytes(), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_calibrate_ffi, CalibrateImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Ret<Buf>().Ret<Buf>().Ret<Buf>()
        .Attr<int64_t>("P").Attr<int64_t>("R").Attr<int64_t>("C").Attr<int64_t>("tp").Attr<int64_t>("tr")
        .Attr<int64_t>("tc").Attr<int32_t>("method").Attr<int32_t>("has_arg").Attr<double>("arg"));

ffi::Error ScaleZeroPointImpl(cudaStream_t stream, Buf calib_a, Buf calib_b, Out scale, Out zero_point,
                              int32_t qtype) {
  return Status(qwx_compute_scale_zero_point(calib_a.untyped_data(), OptionalData(calib_b),
                                             FloatCode(calib_a.element_type()),
                                             (int64_t)calib_a.element_count(), qtype, scale->untyped_data(),
                                             OptionalData(*zero_point), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_compute_scale_zero_point_ffi, ScaleZeroPointImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Ret<Buf>().Ret<Buf>()
        .Attr<int32_t>("qtype"));

ffi::Error QuantizeWithScaleImpl(cudaStream_t stream, Buf x, Buf scale, Buf zero_point, Out q, int64_t P,
                                 int64_t R, int64_t C, int64_t tp, int64_t tr, int64_t tc,
                                 int32_t rounding) {
  int qtype = 0;
  if (int rc = CodeDtype(*q, P * R * C, &qtype)) return Status(rc);
  return Status(qwx_quantize_with_scale(x.untyped_data(), FloatCode(x.element_type()), P, R, C, tp, tr, tc,
                                        scale.untyped_data(), OptionalData(zero_point), qtype, rounding,
                                        q->untyped_data(), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_quantize_with_scale_ffi, QuantizeWithScaleImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Ret<Buf>()
        .Attr<int64_t>("P").Attr<int64_t>("R").Attr<int64_t>("C").Attr<int64_t>("tp").Attr<int64_t>("tr")
        .Attr<int64_t>("tc").Attr<int32_t>("rounding"));

ffi::Error DequantizeImpl(cudaStream_t stream, Buf q, Buf scale, Buf zero_point, Out out, int64_t P,
                          int64_t R, int64_t C, int64_t tp, int64_t tr, int64_t tc) {
  int qtype = 0;
  if (int rc = CodeDtype(q, P * R * C, &qtype)) return Status(rc);
  return Status(qwx_dequantize(q.untyped_data(), qtype, P, R, C, tp, tr, tc, scale.untyped_data(),
                               FloatCode(scale.element_type()), OptionalData(zero_point),
                               out->untyped_data(), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_dequantize_ffi, DequantizeImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Ret<Buf>()
        .Attr<int64_t>("P").Attr<int64_t>("R").Attr<int64_t>("C").Attr<int64_t>("tp").Attr<int64_t>("tr")
        .Attr<int64_t>("tc"));

// ---- contractions: a [M, K] codes, b [K, N] or [N, K] codes, scales [M(, T)] / [(T,) N] ------

int OutCode(ffi::DataType t) { return t == ffi::DataType::S32 ? QWX_S32 : FloatCode(t); }

ffi::Error GemmQ8Impl(cudaStream_t stream, Buf a, Buf b, Buf sa, Buf sb, Out out, Out workspace, Out err,
                      int32_t b_layout, int64_t k_tile, int32_t sa_tiled, int32_t sb_tiled,
                      int32_t epilogue) {
  const auto ad = a.dimensions();
  const auto od = out->dimensions();
  int code = 0;
  if (int rc = CodeDtype(a, (int64_t)a.element_count(), &code)) return Status(rc);
  const int scale_dtype = sa.element_count() ? FloatCode(sa.element_type()) : FloatCode(sb.element_type());
  return Status(qwx_gemm_q8_ws(a.untyped_data(), b.untyped_data(), code, b_layout, ad[0], od[1], ad[1], k_tile,
                               OptionalData(sa), sa_tiled, OptionalData(sb), sb_tiled, scale_dtype,
                               out->untyped_data(), OutCode(out->element_type()), epilogue,
                               OptionalData(*workspace), workspace->size_bytes(), /*workspace_is_zero=*/0,
                               static_cast<int32_t*>(err->untyped_data()), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_gemm_q8_ffi, GemmQ8Impl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Arg<Buf>()
        .Ret<Buf>().Ret<Buf>().Ret<Buf>().Attr<int32_t>("b_layout").Attr<int64_t>("k_tile")
        .Attr<int32_t>("sa_tiled").Attr<int32_t>("sb_tiled").Attr<int32_t>("epilogue"));

ffi::Error GemmQ8TiledImpl(cudaStream_t stream, Buf a, Buf b, Buf sa, Buf sb, Buf corr_row, Buf corr_col,
                           Out out, Out err, int32_t b_layout, int64_t k_tile, int32_t sa_tiled,
                           int32_t sb_tiled, int32_t epilogue) {
  const auto ad = a.dimensions();
  const auto od = out->dimensions();
  int code = 0;
  if (int rc = CodeDtype(a, (int64_t)a.element_count(), &code)) return Status(rc);
  const int scale_dtype = sa.element_count() ? FloatCode(sa.element_type()) : FloatCode(sb.element_type());
  return Status(qwx_gemm_q8_tiled(a.untyped_data(), b.untyped_data(), code, b_layout, ad[0], od[1], ad[1], k_tile,
                                  OptionalData(sa), sa_tiled, OptionalData(sb), sb_tiled, scale_dtype,
                                  static_cast<const int32_t*>(OptionalData(corr_row)),
                                  static_cast<const int32_t*>(OptionalData(corr_col)), out->untyped_data(),
                                  OutCode(out->element_type()), epilogue,
                                  static_cast<int32_t*>(err->untyped_data()), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_gemm_q8_tiled_ffi, GemmQ8TiledImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Arg<Buf>()
        .Arg<Buf>().Arg<Buf>().Ret<Buf>().Ret<Buf>().Attr<int32_t>("b_layout").Attr<int64_t>("k_tile")
        .Attr<int32_t>("sa_tiled").Attr<int32_t>("sb_tiled").Attr<int32_t>("epilogue"));

ffi::Error CodeSumsImpl(cudaStream_t stream, Buf codes, Out out, int32_t k_axis, int64_t k_tile,
                        int32_t t_major) {
  const auto d = codes.dimensions();
  return Status(qwx_code_sums(codes.untyped_data(), d[0], d[1], k_axis, k_tile, t_major,
                              static_cast<int32_t*>(out->untyped_data()), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_code_sums_ffi, CodeSumsImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Ret<Buf>().Attr<int32_t>("k_axis")
        .Attr<int64_t>("k_tile").Attr<int32_t>("t_major"));

// ---- MXFP8 block-scaled contraction --------------------------------------------------------------

ffi::Error MxPackScalesImpl(cudaStream_t stream, Buf scale, Out packed, int32_t operand, int64_t rows,
                            int64_t k, int32_t k_major) {
  return Status(qwx_mx_pack_scales(operand, scale.untyped_data(), FloatCode(scale.element_type()), rows, k,
                                   k_major, packed->untyped_data(), packed->size_bytes(), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_mx_pack_scales_ffi, MxPackScalesImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Ret<Buf>().Attr<int32_t>("operand")
        .Attr<int64_t>("rows").Attr<int64_t>("k").Attr<int32_t>("k_major"));

ffi::Error GemmMx8Impl(cudaStream_t stream, Buf a, Buf b, Buf sfa, Buf sfb, Out out, Out err,
                       int32_t b_layout) {
  const auto ad = a.dimensions();
  const auto od = out->dimensions();
  return Status(qwx_gemm_mx8(a.untyped_data(), b.untyped_data(), b_layout, ad[0], od[1], ad[1],
                             sfa.untyped_data(), sfb.untyped_data(), out->untyped_data(),
                             OutCode(out->element_type()), static_cast<int32_t*>(err->untyped_data()),
                             S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_gemm_mx8_ffi, GemmMx8Impl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Arg<Buf>()
        .Ret<Buf>().Ret<Buf>().Attr<int32_t>("b_layout"));

// ---- MXFP4 block-scaled contraction (codes two per byte, both operands K-major) -------------------

ffi::Error Mx4PackScalesImpl(cudaStream_t stream, Buf scale, Out packed, int32_t operand, int64_t rows,
                             int64_t k, int32_t k_major) {
  return Status(qwx_mx4_pack_scales(operand, scale.untyped_data(), FloatCode(scale.element_type()), rows, k,
                                    k_major, packed->untyped_data(), packed->size_bytes(), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_mx4_pack_scales_ffi, Mx4PackScalesImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Ret<Buf>().Attr<int32_t>("operand")
        .Attr<int64_t>("rows").Attr<int64_t>("k").Attr<int32_t>("k_major"));

ffi::Error Mx4PackCodesImpl(cudaStream_t stream, Buf codes, Out packed, int64_t rows, int64_t k,
                            int32_t k_major) {
  if ((int64_t)codes.size_bytes() != rows * k)   // one code per byte is what the packer reads
    return Status(QWX_ERR_SHAPE);
  return Status(qwx_mx4_pack_codes(codes.untyped_data(), rows, k, k_major, packed->untyped_data(), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_mx4_pack_codes_ffi, Mx4PackCodesImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Ret<Buf>().Attr<int64_t>("rows")
        .Attr<int64_t>("k").Attr<int32_t>("k_major"));

ffi::Error GemmMx4Impl(cudaStream_t stream, Buf a_packed, Buf b_packed, Buf sfa, Buf sfb, Out out, Out err,
                       int64_t k) {
  const auto od = out->dimensions();
  return Status(qwx_gemm_mx4(a_packed.untyped_data(), b_packed.untyped_data(), od[0], od[1], k,
                             sfa.untyped_data(), sfb.untyped_data(), out->untyped_data(),
                             OutCode(out->element_type()), static_cast<int32_t*>(err->untyped_data()),
                             S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_gemm_mx4_ffi, GemmMx4Impl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Arg<Buf>()
        .Ret<Buf>().Ret<Buf>().Attr<int64_t>("k"));

// ---- NVFP4 block-scaled contraction (codes packed by qwx_mx4_pack_codes) --------------------------

ffi::Error Nvfp4PackScalesImpl(cudaStream_t stream, Buf scale, Out packed, int32_t operand, int64_t rows,
                               int64_t k, int32_t k_major) {
  return Status(qwx_nvfp4_pack_scales(operand, scale.untyped_data(), FloatCode(scale.element_type()), rows, k,
                                      k_major, packed->untyped_data(), packed->size_bytes(), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_nvfp4_pack_scales_ffi, Nvfp4PackScalesImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Ret<Buf>().Attr<int32_t>("operand")
        .Attr<int64_t>("rows").Attr<int64_t>("k").Attr<int32_t>("k_major"));

ffi::Error GemmNvfp4Impl(cudaStream_t stream, Buf a_packed, Buf b_packed, Buf sfa, Buf sfb, Out out, Out err,
                         int64_t k) {
  const auto od = out->dimensions();
  return Status(qwx_gemm_nvfp4(a_packed.untyped_data(), b_packed.untyped_data(), od[0], od[1], k,
                               sfa.untyped_data(), sfb.untyped_data(), out->untyped_data(),
                               OutCode(out->element_type()), static_cast<int32_t*>(err->untyped_data()),
                               S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_gemm_nvfp4_ffi, GemmNvfp4Impl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Arg<Buf>()
        .Ret<Buf>().Ret<Buf>().Attr<int64_t>("k"));

ffi::Error QuantGemmQ8Impl(cudaStream_t stream, Buf a, Buf wq, Buf sw, Out out, Out workspace, Out err,
                           int32_t b_layout, int32_t rounding, int32_t epilogue) {
  const auto ad = a.dimensions();
  const auto od = out->dimensions();
  int code = 0;
  if (int rc = CodeDtype(wq, (int64_t)wq.element_count(), &code)) return Status(rc);
  return Status(qwx_quant_gemm_q8(a.untyped_data(), ad[0], ad[1], wq.untyped_data(), sw.untyped_data(), od[1],
                                  code, b_layout, rounding, out->untyped_data(), OutCode(out->element_type()),
                                  epilogue, workspace->untyped_data(), workspace->size_bytes(),
                                  static_cast<int32_t*>(err->untyped_data()), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_quant_gemm_q8_ffi, QuantGemmQ8Impl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Ret<Buf>()
        .Ret<Buf>().Ret<Buf>().Attr<int32_t>("b_layout").Attr<int32_t>("rounding").Attr<int32_t>("epilogue"));

ffi::Error PackW4Impl(cudaStream_t stream, Buf q, Out packed) {
  const auto d = q.dimensions();
  if ((int64_t)q.size_bytes() != d[0] * d[1])   // one code per byte is what the packer reads
    return Status(QWX_ERR_SHAPE);
  return Status(qwx_pack_w4(q.untyped_data(), d[0], d[1], packed->untyped_data(), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(qwx_pack_w4_ffi, PackW4Impl,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Ret<Buf>());

ffi::Error GemmA16W4Impl(cudaStream_t stream, Buf a, Buf w_packed, Buf scale, Out out, Out workspace,
                         int64_t K, int64_t k_tile) {
  const auto od = out->dimensions();
  return Status(qwx_gemm_a16w4(a.untyped_data(), w_packed.untyped_data(), scale.untyped_data(),
                               FloatCode(scale.element_type()), od[0], od[1], K, k_tile, out->untyped_data(),
                               FloatCode(out->element_type()), workspace->untyped_data(),
                               workspace->size_bytes(), /*workspace_is_zero=*/0, nullptr, S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_gemm_a16w4_ffi, GemmA16W4Impl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Ret<Buf>()
        .Ret<Buf>().Attr<int64_t>("K").Attr<int64_t>("k_tile"));

ffi::Error PackW4TilesImpl(cudaStream_t stream, Buf q, Out packed) {
  const auto d = q.dimensions();
  if ((int64_t)q.size_bytes() != d[0] * d[1])   // one code per byte is what the packer reads
    return Status(QWX_ERR_SHAPE);
  return Status(qwx_pack_w4_tiles(q.untyped_data(), d[0], d[1], packed->untyped_data(), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(qwx_pack_w4_tiles_ffi, PackW4TilesImpl,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Ret<Buf>());

ffi::Error GemmA16W4MmaImpl(cudaStream_t stream, Buf a, Buf w_tiles, Buf scale, Out out, Out workspace,
                            Out err, int64_t K, int64_t k_tile) {
  const auto od = out->dimensions();
  return Status(qwx_gemm_a16w4_mma(a.untyped_data(), w_tiles.untyped_data(), scale.untyped_data(),
                                   FloatCode(scale.element_type()), od[0], od[1], K, k_tile,
                                   out->untyped_data(), FloatCode(out->element_type()),
                                   workspace->untyped_data(), workspace->size_bytes(),
                                   /*workspace_is_zero=*/0, static_cast<int32_t*>(err->untyped_data()),
                                   S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_gemm_a16w4_mma_ffi, GemmA16W4MmaImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Ret<Buf>()
        .Ret<Buf>().Ret<Buf>().Attr<int64_t>("K").Attr<int64_t>("k_tile"));

// ---- Hadamard family ------------------------------------------------------------------------

ffi::Error HadamardRotateImpl(cudaStream_t stream, Buf x, Buf signs_in, Buf signs_out, Out out, int32_t axis,
                              int32_t block) {
  const auto d = x.dimensions();
  return Status(qwx_hadamard_rotate(x.untyped_data(), FloatCode(x.element_type()), d[0], d[1], axis, block,
                                    static_cast<const int8_t*>(OptionalData(signs_in)),
                                    static_cast<const int8_t*>(OptionalData(signs_out)), out->untyped_data(),
                                    S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_hadamard_rotate_ffi, HadamardRotateImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Ret<Buf>()
        .Attr<int32_t>("axis").Attr<int32_t>("block"));

ffi::Error HadamardQuantizeImpl(cudaStream_t stream, Buf x, Buf signs_in, Buf signs_out, Out q, Out scale,
                                int32_t block, int32_t rounding) {
  const auto d = x.dimensions();
  int qtype = 0;
  if (int rc = CodeDtype(*q, d[0] * d[1], &qtype)) return Status(rc);
  return Status(qwx_hadamard_quantize(x.untyped_data(), FloatCode(x.element_type()), d[0], d[1], block,
                                      static_cast<const int8_t*>(OptionalData(signs_in)),
                                      static_cast<const int8_t*>(OptionalData(signs_out)), qtype, rounding,
                                      q->untyped_data(), scale->untyped_data(), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_hadamard_quantize_ffi, HadamardQuantizeImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Ret<Buf>()
        .Ret<Buf>().Attr<int32_t>("block").Attr<int32_t>("rounding"));

ffi::Error HadamardGemmImpl(cudaStream_t stream, Buf a, Buf signs_in, Buf signs_out, Buf wq, Buf sw, Out out,
                            Out workspace, Out err, int32_t b_layout, int32_t rounding, int32_t epilogue) {
  const auto ad = a.dimensions();
  const auto od = out->dimensions();
  int code = 0;
  if (int rc = CodeDtype(wq, (int64_t)wq.element_count(), &code)) return Status(rc);
  return Status(qwx_hadamard_gemm(a.untyped_data(), ad[0], ad[1], static_cast<const int8_t*>(OptionalData(signs_in)),
                                  static_cast<const int8_t*>(OptionalData(signs_out)), wq.untyped_data(),
                                  sw.untyped_data(), od[1], code, b_layout, rounding, out->untyped_data(),
                                  OutCode(out->element_type()), epilogue, workspace->untyped_data(),
                                  workspace->size_bytes(), static_cast<int32_t*>(err->untyped_data()),
                                  S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_hadamard_gemm_ffi, HadamardGemmImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Arg<Buf>()
        .Arg<Buf>().Ret<Buf>().Ret<Buf>().Ret<Buf>().Attr<int32_t>("b_layout").Attr<int32_t>("rounding")
        .Attr<int32_t>("epilogue"));

// ---- decoder stages fused with the activation quantizer ---------------------------------------

ffi::Error AddRmsNormQuantizeImpl(cudaStream_t stream, Buf x, Buf delta, Buf weight, Out x_out, Out y_out,
                                  Out q, Out scale, double eps) {
  const auto d = x.dimensions();
  const int64_t width = d.back();
  return Status(qwx_add_rmsnorm_quantize(x.untyped_data(), OptionalData(delta), weight.untyped_data(), eps,
                                         (int64_t)x.element_count() / width, width, OptionalData(*x_out),
                                         OptionalData(*y_out), OptionalData(*q), OptionalData(*scale),
                                         S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_add_rmsnorm_quantize_ffi, AddRmsNormQuantizeImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Arg<Buf>().Arg<Buf>().Ret<Buf>()
        .Ret<Buf>().Ret<Buf>().Ret<Buf>().Attr<double>("eps"));

ffi::Error SiluMulQuantizeImpl(cudaStream_t stream, Buf gu, Out y_out, Out q, Out scale) {
  const auto d = gu.dimensions();
  const int64_t f = d.back() / 2;
  return Status(qwx_silu_mul_quantize(gu.untyped_data(), (int64_t)gu.element_count() / (2 * f), f,
                                      OptionalData(*y_out), OptionalData(*q), OptionalData(*scale), S(stream)));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(
    qwx_silu_mul_quantize_ffi, SiluMulQuantizeImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<Buf>().Ret<Buf>().Ret<Buf>().Ret<Buf>());

}  // namespace

#endif  // QWX_HAVE_XLA_FFI
