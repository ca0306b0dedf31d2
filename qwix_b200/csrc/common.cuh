// Shared device/host helpers for the qwix_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <type_traits>

#include "../../include/qwix_b200.h"

#define QWX_CHECK_LAUNCH()                                 \
  do {                                                     \
    cudaError_t e__ = cudaGetLastError();                  \
    if (e__ != cudaSuccess) return (int)QWX_ERR_LAUNCH;        \
  } while (0)

namespace qwx {

// ---- element types ---------------------------------------------------------------
// Every arithmetic step of the reference happens in the array dtype T; on the device a
// step is a float32 operation followed by round<T>() (round-to-nearest-even into T).

struct F32 { using storage = float; static constexpr int kBytes = 4; };
struct BF16 { using storage = __nv_bfloat16; static constexpr int kBytes = 2; };
struct F16 { using storage = __half; static constexpr int kBytes = 2; };

template <typename T> __device__ __forceinline__ float round_to(float v);
template <> __device__ __forceinline__ float round_to<F32>(float v) { return v; }
template <> __device__ __forceinline__ float round_to<BF16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
template <> __device__ __forceinline__ float round_to<F16>(float v) {
  return __half2float(__float2half_rn(v));
}

template <typename T> __device__ __forceinline__ float load1(const void* p, int64_t i);
template <> __device__ __forceinline__ float load1<F32>(const void* p, int64_t i) {
  return reinterpret_cast<const float*>(p)[i];
}
template <> __device__ __forceinline__ float load1<BF16>(const void* p, int64_t i) {
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
template <> __device__ __forceinline__ float load1<F16>(const void* p, int64_t i) {
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

template <typename T> __device__ __forceinline__ void store1(void* p, int64_t i, float v);
template <> __device__ __forceinline__ void store1<F32>(void* p, int64_t i, float v) {
  reinterpret_cast<float*>(p)[i] = v;
}
template <> __device__ __forceinline__ void store1<BF16>(void* p, int64_t i, float v) {
  reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ void store1<F16>(void* p, int64_t i, float v) {
  reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

// Eight consecutive elements starting at element index i (i % 8 == 0, base 16B aligned).
template <typename T> __device__ __forceinline__ void load8(const void* p, int64_t i, float (&v)[8]);
template <> __device__ __forceinline__ void load8<F32>(const void* p, int64_t i, float (&v)[8]) {
  const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  float4 a = q[0], b = q[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void unpack_bf16x8(const uint4& u, float (&v)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(w[j] << 16);
    v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
  }
}
template <> __device__ __forceinline__ void load8<BF16>(const void* p, int64_t i, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
  unpack_bf16x8(u, v);
}
template <> __device__ __forceinline__ void load8<F16>(const void* p, int64_t i, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p) + i);
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = __half22float2(h[j]);
    v[2 * j] = f.x; v[2 * j + 1] = f.y;
  }
}

template <typename T> __device__ __forceinline__ void store8(void* p, int64_t i, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<F32>(void* p, int64_t i, const float (&v)[8]) {
  float4* q = reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i);
  q[0] = make_float4(v[0], v[1], v[2], v[3]);
  q[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<BF16>(void* p, int64_t i, const float (&v)[8]) {
  uint4 u;
  uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    w[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = u;
}
template <> __device__ __forceinline__ void store8<F16>(void* p, int64_t i, const float (&v)[8]) {
  uint4 u;
  uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
    w[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p) + i) = u;
}

// ---- quantized code types ----------------------------------------------------------

struct S8 { static constexpr int kLo = -128, kHi = 127; static constexpr bool kFloat = false; };
struct S4 { static constexpr int kLo = -8, kHi = 7; static constexpr bool kFloat = false; };
struct E4M3 { static constexpr bool kFloat = true; };
// e4m3 codes under a power-of-two scale per 32 values (OCP microscaling, "mxfp8")
struct MX8 { static constexpr bool kFloat = true; };
// e2m1 codes (sign, two exponent bits, one significand bit: 0, 0.5, 1, 1.5, 2, 3, 4, 6), one
// per byte in the low nibble, under a power-of-two scale per 32 values ("mxfp4")
struct MX4 { static constexpr bool kFloat = true; };
// the same e2m1 codes under a scale per 16 values that is itself an e4m3 number ("nvfp4")
struct NV4 { static constexpr bool kFloat = true; };

// Symmetric bound B (codes cover [-B, B]) and asymmetric (qmin, qmax).
template <typename Q> __host__ __device__ constexpr float sym_bound();
template <> __host__ __device__ constexpr float sym_bound<S8>() { return 127.5f; }
template <> __host__ __device__ constexpr float sym_bound<S4>() { return 7.5f; }
template <> __host__ __device__ constexpr float sym_bound<E4M3>() { return 448.0f; }
template <> __host__ __device__ constexpr float sym_bound<MX8>() { return 448.0f; }
template <> __host__ __device__ constexpr float sym_bound<MX4>() { return 6.0f; }
template <> __host__ __device__ constexpr float sym_bound<NV4>() { return 6.0f; }

// Scaled float -> code, returned as the byte that is stored for 8-bit codes or the
// sign-extended value for int4.  Integers: round-half-even, saturate, NaN -> 0 (the
// float->int convert of XLA); e4m3: clip to +/-448 then round-to-nearest-even, NaN stays.
template <typename Q> __device__ __forceinline__ int to_code(float y) {
  if constexpr (std::is_same<Q, MX4>::value || std::is_same<Q, NV4>::value) {
    // e2m1 has neither NaN nor infinity: clip to +/-6, round to nearest even; a NaN becomes a
    // zero of the opposite sign (what ml_dtypes' cast does; the reference pins no value)
    if (y != y) return (__float_as_uint(y) >> 31) ? 0x0 : 0x8;
    y = fminf(fmaxf(y, -6.0f), 6.0f);
    return (int)__nv_cvt_float_to_fp4(y, __NV_E2M1, cudaRoundNearest);
  } else if constexpr (Q::kFloat) {
    if (y != y) return 0x7f;
    y = fminf(fmaxf(y, -448.0f), 448.0f);
    return (int)__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
  } else if constexpr (Q::kLo == -128) {
    int q;  // one instruction: round-half-even, saturate to [-128, 127], NaN -> 0
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(y));
    return (int)(signed char)q;
  } else {
    int q = __float2int_rn(y);  // saturates at int32 range, NaN -> 0
    return min(max(q, Q::kLo), Q::kHi);
  }
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

__device__ __forceinline__ float e2m1_to_float(uint8_t b) {
  const uint32_t m = b & 7u;
  // 0, 0.5, then (1 + significand / 2) * 2^(exponent - 1)
  const float mag = m < 2 ? 0.5f * (float)m : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
  return (b & 8u) ? -mag : mag;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}


// ---- programmatic dependent launch ---------------------------------------------------------
//
// The kernels of a decode step are short and run back to back on one stream, so a good part of
// each one's time is launch latency, set-up and the first loads.  A kernel launched with the
// programmatic-stream-serialization attribute may start while its predecessor is still
// running; it does whatever does not depend on the predecessor (barrier set-up, tensor-memory
// allocation, fetching WEIGHTS, which are static) and then executes griddepcontrol.wait, which
// returns once the predecessor has completed and its writes are visible.  Everything that
// reads activations or writes global memory comes after that wait.  Without the attribute both
// instructions do nothing.  qwx_set_programmatic_launch() turns the attribute on for the
// kernels that contain the wait.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

bool programmatic_launch_enabled();   // capi.cu

template <typename... P, typename... A>
inline cudaError_t launch_dependent(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t st, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = programmatic_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

// Function attributes (the dynamic shared-memory limit) are per device: a launch site keeps
// one of these and sets its attributes the first time it runs on each device.  The flags are
// idempotent; a benign race sets an attribute twice.
struct PerDeviceOnce {
  bool done[64] = {};
  // true when the caller still has to configure the current device
  bool first() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return true;
    return !done[d];
  }
  void mark() {
    int d = 0;
    if (cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < 64) done[d] = true;
  }
};

}  // namespace qwx
