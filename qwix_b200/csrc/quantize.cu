// HBM-bound quantizer kernels: calibrate, scale/zero-point, quantize, dequantize.
//
// Numerics follow qwix/_src/core/qarray.py:470-708 and numerics.py:139-196 step by step:
// every primitive is a float32 operation rounded to the array dtype (strict mode).  All
// loads and stores are 128-bit wide and coalesced; reductions use warp shuffles plus one
// shared-memory hop, and cross-CTA reductions use integer atomics on float bit patterns.
#include "common.cuh"

#include <mutex>

namespace qwx {
namespace {

constexpr int kThreads = 256;
constexpr float kTinyScale = 0x1p-63f;  // sqrt(finfo.tiny) for float32 / bfloat16

struct View {
  int64_t P, R, C, tp, tr, tc;
  int64_t GP, GR, GC;  // tile counts per axis
  __host__ __device__ int64_t groups() const { return GP * GR * GC; }
};

struct CalibArgs {
  int method;      // qwx_calibration
  int has_arg;
  float arg;       // already narrowed to float
};

enum class Out { kS8, kS4U, kS4P, kE4M3, kMX8, kMX4, kNV4 };
template <Out O> struct OutTraits;
template <> struct OutTraits<Out::kS8> { using Q = S8; };
template <> struct OutTraits<Out::kS4U> { using Q = S4; };
template <> struct OutTraits<Out::kS4P> { using Q = S4; };
template <> struct OutTraits<Out::kE4M3> { using Q = E4M3; };
template <> struct OutTraits<Out::kMX8> { using Q = MX8; };
template <> struct OutTraits<Out::kMX4> { using Q = MX4; };
template <> struct OutTraits<Out::kNV4> { using Q = NV4; };

// ---- scalar recipes -------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ float apply_arg(float v, const CalibArgs& c) {
  if (c.has_arg) v = round_to<T>(__fmul_rn(v, round_to<T>(c.arg)));
  return v;
}

template <typename T>
__device__ __forceinline__ float guard_scale(float s) {
  // scale < sqrt(tiny) -> 1 (qarray.py:553-554, 561-562); NaN compares false and stays.
  constexpr float thr = std::is_same<T, F16>::value ? 0.0078125f /*2^-7*/ : kTinyScale;
  return (s < thr) ? 1.0f : s;
}

template <typename T, typename Q>
__device__ __forceinline__ float symmetric_scale(float absmax) {
  float s = guard_scale<T>(round_to<T>(__fdiv_rn(absmax, sym_bound<Q>())));
  if constexpr (std::is_same<Q, MX8>::value || std::is_same<Q, MX4>::value) {
    // Microscaling: the scale becomes a power of two.  scale * 60/31 (e4m3) or 12/7 (e2m1) in
    // the input dtype (outlier-aware bias), rounded to bfloat16, significand dropped
    // (qarray.py:566-579).
    constexpr float c = std::is_same<Q, MX4>::value ? 12.0f / 7.0f : 60.0f / 31.0f;
    const float biased = round_to<T>(__fmul_rn(s, round_to<T>(c)));
    s = __uint_as_float(__float_as_uint(round_to<BF16>(biased)) & 0x7F800000u);
  } else if constexpr (std::is_same<Q, NV4>::value) {
    // the scale becomes an e4m3 number: clip to +/-448, round to nearest even (qarray.py:580-581)
    s = s != s ? s : e4m3_to_float((uint8_t)to_code<E4M3>(s));
  }
  return s;
}

template <typename T, typename Q>
__device__ __forceinline__ void asymmetric_scale(float lo, float hi, float& s, int& zp) {
  if constexpr (Q::kFloat) {
    s = 1.f; zp = 0;  // floating codes have no asymmetric form (numerics.py:64-92)
    return;
  } else {
  constexpr float qmin = (float)Q::kLo, qmax = (float)Q::kHi;
  float range = round_to<T>(__fsub_rn(hi, lo));
  s = guard_scale<T>(round_to<T>(__fdiv_rn(range, round_to<T>(qmax - qmin))));
  float z = round_to<T>(__fsub_rn(qmin, round_to<T>(__fdiv_rn(lo, s))));
  zp = to_code<Q>(z);
  }
}

// x / s as the reference computes it (true division).  For bfloat16 operands in strict mode
// the bf16 rounding of the quotient is obtained from x * rcp(s) instead: x and s carry 8-bit
// significands, so the exact quotient is never closer than 2^-17 (relative) to a bf16
// rounding boundary and never on one, while x * rcp_rn(s) is within 2^-22 of it -- both round
// to the same bf16 value.  Scales outside [2^-100, 2^100] take the division.
template <typename T>
struct Divider {
  float s, r;
  bool fast;
  __device__ __forceinline__ Divider(float scale, bool strict) : s(scale) {
    const float a = fabsf(scale);
    fast = std::is_same<T, BF16>::value && strict && a > 0x1p-100f && a < 0x1p100f;
    r = fast ? __frcp_rn(scale) : 0.f;
  }
  __device__ __forceinline__ float operator()(float x) const {
    return fast ? __fmul_rn(x, r) : __fdiv_rn(x, s);
  }
};

template <typename T, typename Q>
__device__ __forceinline__ int quantize_one(float x, const Divider<T>& div, float zp, bool has_zp,
                                            bool strict) {
  float y = div(x);
  if (strict) y = round_to<T>(y);
  if (has_zp) {
    y = __fadd_rn(y, zp);
    if (strict) y = round_to<T>(y);
  }
  return to_code<Q>(y);
}

template <Out O>
__device__ __forceinline__ void store_codes8(void* q, int64_t i, const int (&c)[8]) {
  if constexpr (O == Out::kS4P) {
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) w |= (uint32_t)(c[j] & 0xf) << (4 * j);
    reinterpret_cast<uint32_t*>(q)[i >> 3] = w;
  } else {
    uint2 w;
    w.x = (c[0] & 0xff) | ((c[1] & 0xff) << 8) | ((c[2] & 0xff) << 16) | ((uint32_t)(c[3] & 0xff) << 24);
    w.y = (c[4] & 0xff) | ((c[5] & 0xff) << 8) | ((c[6] & 0xff) << 16) | ((uint32_t)(c[7] & 0xff) << 24);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(q) + i) = w;
  }
}

template <Out O>
__device__ __forceinline__ void store_code1(void* q, int64_t i, int c) {
  if constexpr (O == Out::kS4P) {
    // Two neighbours share a byte; only used on the scalar fallback where one thread owns
    // both nibbles of a byte (caller guarantees i is even and passes the pair separately).
    uint8_t* b = reinterpret_cast<uint8_t*>(q) + (i >> 1);
    if (i & 1) *b = (uint8_t)((*b & 0x0f) | ((c & 0xf) << 4));
    else *b = (uint8_t)((*b & 0xf0) | (c & 0xf));
  } else {
    reinterpret_cast<int8_t*>(q)[i] = (int8_t)c;
  }
}

// ---- one-pass kernel for tiles that are row segments (tp = tr = 1) ------------------------
//
// G threads own one segment of `tc` contiguous elements: load it once into registers
// (up to kCache vectors per thread; longer segments are re-read and mostly hit L2),
// reduce, derive the scale, quantize from registers.  G threads per segment: 4, 8 or 16 lanes of
// a warp for segments of 32 / 64 / 128 values (microscaling blocks, small sub-channel tiles: a
// whole warp would leave 28 lanes idle), 32: one warp, 256: one CTA.

constexpr int kCache = 4;

template <typename T, Out O, int G>
__global__ void __launch_bounds__(kThreads)
quantize_rows_kernel(const void* __restrict__ x, int64_t segments, int64_t tc, CalibArgs cal,
                     int rounding, void* __restrict__ q, void* __restrict__ scale,
                     int8_t* __restrict__ zero_point) {
  using Q = typename OutTraits<O>::Q;
  constexpr int kSegs = kThreads / G;
  __shared__ float red[2][kThreads / 32];
  griddep_launch_dependents();
  griddep_wait();
  const int lane_in_group = threadIdx.x % G;
  const int64_t seg = (int64_t)blockIdx.x * kSegs + threadIdx.x / G;
  const bool live = seg < segments;
  const int64_t base = seg * tc;
  const int64_t nvec = tc >> 3;
  const bool strict = rounding == QWX_STRICT;

  uint4 cache[kCache];
  uint32_t amax_bits = 0;
  float lo = 0.f, hi = 0.f, sumsq = 0.f;

  // bfloat16 absmax on packed pairs: |x| and max are exact in bf16, NaN propagates.
  __nv_bfloat162 amax2 = __floats2bfloat162_rn(0.f, 0.f);
  auto accumulate_packed = [&](const uint4& u) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      amax2 = __hmax2_nan(amax2, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[j])));
  };
  auto accumulate = [&](const float (&v)[8]) {
    if (cal.method == QWX_ABSMAX) {
#pragma unroll
      for (int j = 0; j < 8; ++j) amax_bits = max(amax_bits, __float_as_uint(v[j]) & 0x7fffffffu);
    } else if (cal.method == QWX_MINMAX) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { lo = fminf(lo, v[j]); hi = fmaxf(hi, v[j]); }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) sumsq += round_to<T>(__fmul_rn(v[j], v[j]));
    }
  };

  if (live) {
#pragma unroll
    for (int it = 0; it < kCache; ++it) {
      int64_t vi = lane_in_group + (int64_t)it * G;
      if (vi < nvec) {
        float v[8];
        if constexpr (T::kBytes == 2) {
          cache[it] = *reinterpret_cast<const uint4*>(
              reinterpret_cast<const uint16_t*>(x) + base + vi * 8);
          if constexpr (std::is_same<T, BF16>::value) {
            if (cal.method == QWX_ABSMAX) { accumulate_packed(cache[it]); continue; }
            unpack_bf16x8(cache[it], v);
          } else {
            load8<T>(x, base + vi * 8, v);
          }
        } else {
          load8<T>(x, base + vi * 8, v);
        }
        accumulate(v);
      }
    }
    for (int64_t vi = lane_in_group + (int64_t)kCache * G; vi < nvec; vi += G) {
      float v[8];
      load8<T>(x, base + vi * 8, v);
      accumulate(v);
    }
  }

  // Reduce across the G threads of the segment.
  float r0, r1;
  if (cal.method == QWX_ABSMAX) {
    const float2 packed = __bfloat1622float2(amax2);
    amax_bits = max(amax_bits, max(__float_as_uint(packed.x), __float_as_uint(packed.y)));
    r0 = __uint_as_float(amax_bits); r1 = 0.f;
  }
  else if (cal.method == QWX_MINMAX) { r0 = fabsf(lo); r1 = hi; }
  else { r0 = sumsq; r1 = 0.f; }
  if (cal.method == QWX_RMS) {
    r0 = warp_sum(r0);
  } else {
    // max over non-negative floats == max over their bit patterns (NaN sorts last).
    uint32_t b0 = __float_as_uint(r0), b1 = __float_as_uint(r1);
#pragma unroll
    for (int o = (G < 32 ? G : 32) / 2; o > 0; o >>= 1) {
      b0 = max(b0, __shfl_xor_sync(0xffffffffu, b0, o));
      b1 = max(b1, __shfl_xor_sync(0xffffffffu, b1, o));
    }
    r0 = __uint_as_float(b0); r1 = __uint_as_float(b1);
  }
  if constexpr (G > 32) {
    const int w = threadIdx.x / 32;
    if ((threadIdx.x & 31) == 0) { red[0][w] = r0; red[1][w] = r1; }
    __syncthreads();
    float a0 = red[0][0], a1 = red[1][0];
#pragma unroll
    for (int i = 1; i < kThreads / 32; ++i) {
      if (cal.method == QWX_RMS) a0 += red[0][i];
      else {
        a0 = __uint_as_float(max(__float_as_uint(a0), __float_as_uint(red[0][i])));
        a1 = __uint_as_float(max(__float_as_uint(a1), __float_as_uint(red[1][i])));
      }
    }
    r0 = a0; r1 = a1;
  }
  if (!live) return;

  float s, zpf = 0.f;
  bool has_zp = false;
  if (cal.method == QWX_MINMAX) {
    float mn = apply_arg<T>(-r0, cal), mx = apply_arg<T>(r1, cal);
    int zp;
    asymmetric_scale<T, Q>(mn, mx, s, zp);
    zpf = (float)zp; has_zp = true;
    if (lane_in_group == 0 && zero_point) zero_point[seg] = (int8_t)zp;
  } else {
    float a = r0;
    if (cal.method == QWX_RMS) {
      float mean = round_to<T>(__fdiv_rn(r0, (float)tc));
      a = round_to<T>(__fsqrt_rn(mean));
      a = round_to<T>(__fmul_rn(a, round_to<T>(cal.arg)));
    } else {
      a = apply_arg<T>(a, cal);
    }
    s = symmetric_scale<T, Q>(a);
  }
  if (lane_in_group == 0) store1<T>(scale, seg, s);

  const Divider<T> div(s, strict);
  // bf16 -> int8, strict rounding, symmetric: x * rcp(s) -> round to bf16 -> round-half-even
  // with saturation, two values per conversion/pack instruction where the ISA allows.
  auto emit_packed = [&](const uint4& u, int64_t vi) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    int c[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float y0 = __fmul_rn(__uint_as_float(w[j] << 16), div.r);
      const float y1 = __fmul_rn(__uint_as_float(w[j] & 0xffff0000u), div.r);
      const __nv_bfloat162 b = __floats2bfloat162_rn(y0, y1);
      const uint32_t bw = *reinterpret_cast<const uint32_t*>(&b);
      c[2 * j] = to_code<S8>(__uint_as_float(bw << 16));
      c[2 * j + 1] = to_code<S8>(__uint_as_float(bw & 0xffff0000u));
    }
    uint2 o;
    o.x = __byte_perm(__byte_perm(c[0], c[1], 0x0040), __byte_perm(c[2], c[3], 0x0040), 0x5410);
    o.y = __byte_perm(__byte_perm(c[4], c[5], 0x0040), __byte_perm(c[6], c[7], 0x0040), 0x5410);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(q) + base + vi * 8) = o;
  };
  const bool packed_path = std::is_same<T, BF16>::value && O == Out::kS8 && div.fast && !has_zp;
  auto emit = [&](const float (&v)[8], int64_t vi) {
    int c[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) c[j] = quantize_one<T, Q>(v[j], div, zpf, has_zp, strict);
    store_codes8<O>(q, base + vi * 8, c);
  };
#pragma unroll
  for (int it = 0; it < kCache; ++it) {
    int64_t vi = lane_in_group + (int64_t)it * G;
    if (vi < nvec) {
      float v[8];
      if constexpr (std::is_same<T, BF16>::value) {
        if (packed_path) { emit_packed(cache[it], vi); continue; }
        unpack_bf16x8(cache[it], v);
      } else {
        load8<T>(x, base + vi * 8, v);
      }
      emit(v, vi);
    }
  }
  for (int64_t vi = lane_in_group + (int64_t)kCache * G; vi < nvec; vi += G) {
    float v[8];
    load8<T>(x, base + vi * 8, v);
    emit(v, vi);
  }
}

// ---- microscaling blocks: 32 consecutive values -> e4m3 codes + one power-of-two scale ------
//
// Four lanes per block, one 16-byte vector of input each (a warp reads 512 contiguous values),
// absmax over the block with two shuffles, the scale by the outlier-aware rule, and -- the
// scale being a power of two -- x / scale as an exact multiplication by its reciprocal.  Two
// values per fp8 conversion instruction.
template <typename T, typename Q = MX8>
__global__ void __launch_bounds__(kThreads)
quantize_mx8_blocks_kernel(const void* __restrict__ x, int64_t nvec, void* __restrict__ q,
                           void* __restrict__ scale, int strict) {
  // lanes per block: four 16-byte vectors of a 32-wide block, two of a 16-wide one (nvfp4)
  constexpr int kLanes = std::is_same<Q, NV4>::value ? 2 : 4;
  griddep_launch_dependents();
  griddep_wait();
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const bool live = i < nvec;                 // whole groups: nvec is a multiple of kLanes
  float v[8];
  if (live) {
    load8<T>(x, i * 8, v);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
  }
  uint32_t bits = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) bits = max(bits, __float_as_uint(v[j]) & 0x7fffffffu);   // NaN sorts last
  bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, 1));
  if constexpr (kLanes == 4) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, 2));
  if (!live) return;
  const float s = symmetric_scale<T, Q>(__uint_as_float(bits));
  if ((threadIdx.x & (kLanes - 1)) == 0) store1<T>(scale, i / kLanes, s);
  if constexpr (std::is_same<Q, NV4>::value) {
    // the scale is an e4m3 number, not a power of two: the reference's true division
    const Divider<T> div(s, strict != 0);
    uint32_t w4[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float y = div(v[j]);
      if (strict) y = round_to<T>(y);
      w4[j >> 2] |= (uint32_t)to_code<NV4>(y) << (8 * (j & 3));
    }
    *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(q) + i * 8) = make_uint2(w4[0], w4[1]);
    return;
  }
  const float inv = __fdiv_rn(1.0f, s);       // exact: s is a power of two (or NaN, which propagates)
  if constexpr (std::is_same<Q, MX4>::value) {
    // e2m1 codes, one per byte
    uint32_t w4[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j)
      w4[j >> 2] |= (uint32_t)to_code<MX4>(round_to<T>(__fmul_rn(v[j], inv))) << (8 * (j & 3));
    *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(q) + i * 8) = make_uint2(w4[0], w4[1]);
    return;
  }
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      // the quotient in the input dtype (exact unless it underflows), NaN -> 0x7f, clip to +/-448
      const float y0 = round_to<T>(__fmul_rn(v[4 * h + 2 * j], inv));
      const float y1 = round_to<T>(__fmul_rn(v[4 * h + 2 * j + 1], inv));
      const __nv_fp8x2_storage_t p2 = __nv_cvt_float2_to_fp8x2(make_float2(y0, y1), __NV_SATFINITE, __NV_E4M3);
      packed |= (uint32_t)p2 << (16 * j);
    }
    w[h] = packed;
  }
  *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(q) + i * 8) = make_uint2(w[0], w[1]);
}

// ---- the per-token hot path: bf16 rows -> int8, absmax, strict rounding ---------------------
//
// Persistent CTAs walk the rows with a stride of gridDim.x and keep the next row in flight
// through a shared-memory ring while one is reduced and quantized.  The arithmetic is arranged to work on packed bf16
// pairs: |x| and max on packed bf16, the division as three packed bf16 FMAs that give the
// correctly rounded bf16 quotient, one conversion per value and a saturating pack.  Rows whose
// absmax is not finite (inf / NaN inputs) or whose scale leaves the fast range take the general
// per-element recipe.

// kRowVec: 16-byte vectors per thread; rows up to 256 * kRowVec * 8 elements (4: 8192, 8: 16384)
// Two rows per CTA in the shared-memory ring (one in use, one in flight) and six CTAs per SM:
// the row loop is a dependent chain (wait for the row, reduce across the CTA, barrier, divide,
// convert, store), so warps hide it better than a deeper ring does.  [4096, 8192] / [16384,
// 8192] bf16: 25.3 / 83.9 us with four rows x three CTAs, 24.9 / 76.3 with three x four,
// 23.1 / 74.7 with two x six, 26.2 / 88.6 with two x seven (36 registers: spills).
constexpr int kRowDepth = 2;
constexpr int kRowCtas = 6;

template <int kRowVec>
__global__ void __launch_bounds__(kThreads, kRowVec == 4 ? kRowCtas : kRowCtas / 2)
quantize_rows_bf16_s8_kernel(const uint4* __restrict__ x, int64_t segments, int nvec,
                             uint2* __restrict__ q, __nv_bfloat16* __restrict__ scale) {
  extern __shared__ uint4 ring[];   // [kRowDepth][nvec]; thread t only touches vectors t + 256 i
  __shared__ uint32_t red[2][kThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint4 cur[kRowVec];
  griddep_launch_dependents();
  griddep_wait();

  // Rows reach shared memory through 16-byte cp.async copies that every thread issues for its
  // own vectors, kRowDepth - 1 rows ahead: the bytes in flight per SM do not depend on registers.
  int64_t fetch_row = blockIdx.x;
  int fetch_stage = 0;
  auto fetch = [&]() {
    if (fetch_row < segments) {
#pragma unroll
      for (int it = 0; it < kRowVec; ++it) {
        const int vi = tid + it * kThreads;
        if (vi < nvec) {
          const uint32_t dst = (uint32_t)__cvta_generic_to_shared(ring + fetch_stage * nvec + vi);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst),
                       "l"(x + fetch_row * nvec + vi) : "memory");
        }
      }
      fetch_row += gridDim.x;
    }
    if (++fetch_stage == kRowDepth) fetch_stage = 0;
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  for (int d = 0; d < kRowDepth - 1; ++d) fetch();

  int stage = 0;
  int64_t row = blockIdx.x;
  for (int iter = 0; row < segments; ++iter) {
    const int64_t next = row + gridDim.x;
    asm volatile("cp.async.wait_group %0;" ::"n"(kRowDepth - 2) : "memory");
#pragma unroll
    for (int it = 0; it < kRowVec; ++it) {
      const int vi = tid + it * kThreads;
      if (vi < nvec) cur[it] = ring[stage * nvec + vi];
    }
    if (++stage == kRowDepth) stage = 0;
    fetch();   // refills the stage consumed one iteration ago

    // absmax of the row
    __nv_bfloat162 m2 = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
    for (int it = 0; it < kRowVec; ++it) {
      if (tid + it * kThreads < nvec) {
        const uint32_t w[4] = {cur[it].x, cur[it].y, cur[it].z, cur[it].w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          m2 = __hmax2_nan(m2, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[j])));
      }
    }
    const float2 mf = __bfloat1622float2(m2);
    uint32_t bits = max(__float_as_uint(mf.x), __float_as_uint(mf.y));  // NaN sorts last
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
    uint32_t* slot = red[iter & 1];
    if (lane == 0) slot[warp] = bits;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) bits = max(bits, slot[i]);
    const float absmax = __uint_as_float(bits);

    const float s = symmetric_scale<BF16, S8>(absmax);
    if (tid == 0) scale[row] = __float2bfloat16_rn(s);
    const Divider<BF16> div(s, true);
    const bool fast = div.fast && bits < 0x7f800000u;  // finite absmax, scale in the fast range
    const __nv_bfloat16 sb = __float2bfloat16_rn(s);
    const __nv_bfloat16 rb = __float2bfloat16_rn(__frcp_rn(s));  // RN_bf16(1 / s), no double rounding
    const __nv_bfloat162 r2 = __halves2bfloat162(rb, rb);
    const __nv_bfloat162 ns2 = __hneg2(__halves2bfloat162(sb, sb));

#pragma unroll
    for (int it = 0; it < kRowVec; ++it) {
      const int vi = tid + it * kThreads;
      if (vi >= nvec) continue;
      const uint32_t w[4] = {cur[it].x, cur[it].y, cur[it].z, cur[it].w};
      uint2 o;
      if (fast) {
        // Correctly rounded bf16 quotients from three packed bf16 FMAs (Markstein's division):
        // q0 = x * r, rem = x - q0 * s (one rounding), z = q0 + rem * r, with r = RN(1 / s).
        // Checked exhaustively for all 128 x 128 pairs of bf16 significands.  Then
        // round-half-even to int32 and a saturating pack of four codes per word.
        uint32_t packed[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          int c[4];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(&w[2 * half + j]);
            const __nv_bfloat162 q0 = __hmul2(xv, r2);
            const __nv_bfloat162 rem = __hfma2(q0, ns2, xv);
            const __nv_bfloat162 z = __hfma2(rem, r2, q0);
            const uint32_t zw = *reinterpret_cast<const uint32_t*>(&z);
            asm("{ .reg .b16 lo, hi;\n\t mov.b32 {lo, hi}, %2;\n\t"
                " cvt.rni.s32.bf16 %0, lo;\n\t cvt.rni.s32.bf16 %1, hi; }"
                : "=r"(c[2 * j]), "=r"(c[2 * j + 1]) : "r"(zw));
          }
          uint32_t hi16;
          asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi16) : "r"(c[3]), "r"(c[2]), "r"(0u));
          asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(packed[half]) : "r"(c[1]), "r"(c[0]), "r"(hi16));
        }
        o.x = packed[0];
        o.y = packed[1];
      } else {
        uint32_t code[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          code[2 * j] = (uint32_t)quantize_one<BF16, S8>(__uint_as_float(w[j] << 16), div, 0.f,
                                                        false, true);
          code[2 * j + 1] = (uint32_t)quantize_one<BF16, S8>(
              __uint_as_float(w[j] & 0xffff0000u), div, 0.f, false, true);
        }
        o.x = __byte_perm(__byte_perm(code[0], code[1], 0x0040), __byte_perm(code[2], code[3], 0x0040), 0x5410);
        o.y = __byte_perm(__byte_perm(code[4], code[5], 0x0040), __byte_perm(code[6], code[7], 0x0040), 0x5410);
      }
      q[row * nvec + vi] = o;
    }
    row = next;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---- general tiled view: statistics by atomics, then an elementwise pass --------------------
//
// A CTA covers kChunkRows rows x 256 columns inside one row tile.  Each lane owns eight
// adjacent columns and walks down the rows, so global loads are 128-bit and coalesced.
// Column groups inside the CTA reduce through shared-memory atomics, then one global atomic
// per (CTA, column group).  Statistics are kept as int32 bit patterns of non-negative
// floats: slot 0 = absmax, -min or sum of squares, slot 1 = max.

constexpr int kChunkRows = 128;
constexpr int kChunkCols = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads)
calibrate_tiles_kernel(const void* __restrict__ x, View vw, int method, int vec_ok,
                       int* __restrict__ stats) {
  __shared__ int sh[2][kChunkCols + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t chunks_per_tile = (vw.tr + kChunkRows - 1) / kChunkRows;
  const int64_t row_tile = blockIdx.y / chunks_per_tile;
  const int64_t chunk = blockIdx.y % chunks_per_tile;
  const int64_t r_begin = row_tile * vw.tr + chunk * kChunkRows;
  const int64_t r_end = min(r_begin + kChunkRows, (row_tile + 1) * vw.tr);
  const int64_t p = blockIdx.z;
  const int64_t c0 = (int64_t)blockIdx.x * kChunkCols;
  const int64_t col = c0 + lane * 8;

  for (int i = threadIdx.x; i < 2 * (kChunkCols + 1); i += kThreads) (&sh[0][0])[i] = 0;
  __syncthreads();

  uint32_t a[8];
  float lo[8], hi[8], sq[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { a[j] = 0; lo[j] = 0.f; hi[j] = 0.f; sq[j] = 0.f; }

  if (col < vw.C) {
    for (int64_t r = r_begin + warp; r < r_end; r += kThreads / 32) {
      const int64_t off = (p * vw.R + r) * vw.C + col;
      float v[8];
      if (vec_ok) {
        load8<T>(x, off, v);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (col + j < vw.C) ? load1<T>(x, off + j) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (method == QWX_ABSMAX) a[j] = max(a[j], __float_as_uint(v[j]) & 0x7fffffffu);
        else if (method == QWX_MINMAX) { lo[j] = fminf(lo[j], v[j]); hi[j] = fmaxf(hi[j], v[j]); }
        else sq[j] += round_to<T>(__fmul_rn(v[j], v[j]));
      }
    }
    const int64_t first_group = c0 / vw.tc;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (col + j >= vw.C) break;
      const int slot = (int)((col + j) / vw.tc - first_group);
      if (method == QWX_ABSMAX) atomicMax(&sh[0][slot], (int)a[j]);
      else if (method == QWX_MINMAX) {
        atomicMax(&sh[0][slot], __float_as_int(fabsf(lo[j])));
        atomicMax(&sh[1][slot], __float_as_int(hi[j]));
      } else atomicAdd(reinterpret_cast<float*>(&sh[0][slot]), sq[j]);
    }
  }
  __syncthreads();
  const int64_t first_group = c0 / vw.tc;
  const int64_t last_col = min(c0 + kChunkCols, vw.C) - 1;
  const int nslots = (int)(last_col / vw.tc - first_group) + 1;
  for (int s = threadIdx.x; s < nslots; s += kThreads) {
    const int64_t g = ((p / vw.tp) * vw.GR + row_tile) * vw.GC + first_group + s;
    if (method == QWX_RMS) atomicAdd(reinterpret_cast<float*>(&stats[2 * g]), __int_as_float(sh[0][s]));
    else {
      atomicMax(&stats[2 * g], sh[0][s]);
      if (method == QWX_MINMAX) atomicMax(&stats[2 * g + 1], sh[1][s]);
    }
  }
}

// stats -> calibration values in the array dtype (what qarray.calibrate returns).
template <typename T>
__global__ void finish_calibration_kernel(const int* __restrict__ stats, int64_t groups,
                                          int64_t tile_elems, CalibArgs cal,
                                          void* __restrict__ out_a, void* __restrict__ out_b) {
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  float r0 = __int_as_float(stats[2 * g]), r1 = __int_as_float(stats[2 * g + 1]);
  if (cal.method == QWX_MINMAX) {
    store1<T>(out_a, g, apply_arg<T>(-r0, cal));
    store1<T>(out_b, g, apply_arg<T>(r1, cal));
  } else if (cal.method == QWX_RMS) {
    float mean = round_to<T>(__fdiv_rn(r0, (float)tile_elems));
    float a = round_to<T>(__fsqrt_rn(mean));
    store1<T>(out_a, g, round_to<T>(__fmul_rn(a, round_to<T>(cal.arg))));
  } else {
    store1<T>(out_a, g, apply_arg<T>(r0, cal));
  }
}

template <typename T, typename Q>
__global__ void scale_zero_point_kernel(const void* __restrict__ ca, const void* __restrict__ cb,
                                        int64_t n, void* __restrict__ scale,
                                        int8_t* __restrict__ zero_point) {
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n) return;
  if (cb == nullptr) {
    store1<T>(scale, g, symmetric_scale<T, Q>(load1<T>(ca, g)));
  } else {
    float s; int zp;
    asymmetric_scale<T, Q>(load1<T>(ca, g), load1<T>(cb, g), s, zp);
    store1<T>(scale, g, s);
    zero_point[g] = (int8_t)zp;
  }
}

// Elementwise quantize with generic broadcast of scale / zero point over the tiles.
template <typename T, Out O>
__global__ void __launch_bounds__(kThreads)
apply_scale_kernel(const void* __restrict__ x, View vw, const void* __restrict__ scale,
                   const int8_t* __restrict__ zero_point, int rounding, int vec_ok,
                   void* __restrict__ q) {
  using Q = typename OutTraits<O>::Q;
  const int64_t vec_per_row = (vw.C + 7) >> 3;
  const int64_t total = vw.P * vw.R * vec_per_row;
  const bool strict = rounding == QWX_STRICT;
  const bool has_zp = zero_point != nullptr;
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * kThreads) {
    const int64_t row = t / vec_per_row;          // p * R + r
    const int64_t col = (t - row * vec_per_row) << 3;
    const int64_t p = row / vw.R, r = row - p * vw.R;
    const int64_t gbase = ((p / vw.tp) * vw.GR + r / vw.tr) * vw.GC;
    const int64_t off = row * vw.C + col;
    float v[8];
    int c[8];
    if (vec_ok) {
      load8<T>(x, off, v);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (col + j < vw.C) ? load1<T>(x, off + j) : 0.f;
    }
    const int64_t g0 = gbase + col / vw.tc;
    const int64_t g7 = gbase + min(col + 7, vw.C - 1) / vw.tc;
    if (g0 == g7) {
      const Divider<T> div(load1<T>(scale, g0), strict);
      const float z = has_zp ? (float)zero_point[g0] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = quantize_one<T, Q>(v[j], div, z, has_zp, strict);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int64_t g = gbase + min(col + j, vw.C - 1) / vw.tc;
        const Divider<T> div(load1<T>(scale, g), false);  // one use: plain division
        const float z = has_zp ? (float)zero_point[g] : 0.f;
        c[j] = quantize_one<T, Q>(v[j], div, z, has_zp, strict);
      }
    }
    if (vec_ok) {
      store_codes8<O>(q, off, c);
    } else {
      if constexpr (O == Out::kS4P) {
        // C is even for packed int4 (checked on the host): pairs never straddle rows.
        for (int j = 0; j < 8 && col + j < vw.C; j += 2)
          reinterpret_cast<uint8_t*>(q)[(off + j) >> 1] = (uint8_t)((c[j] & 0xf) | ((c[j + 1] & 0xf) << 4));
      } else {
        for (int j = 0; j < 8 && col + j < vw.C; ++j) store_code1<O>(q, off + j, c[j]);
      }
    }
  }
}

// (q - zero_point) * scale in the scale dtype S, generic broadcast (qarray.py:692-708).
template <typename S, Out O>
__global__ void __launch_bounds__(kThreads)
dequantize_kernel(const void* __restrict__ q, View vw, const void* __restrict__ scale,
                  const int8_t* __restrict__ zero_point, int vec_ok, void* __restrict__ out) {
  const int64_t vec_per_row = (vw.C + 7) >> 3;
  const int64_t total = vw.P * vw.R * vec_per_row;
  const bool has_zp = zero_point != nullptr;
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * kThreads) {
    const int64_t row = t / vec_per_row;
    const int64_t col = (t - row * vec_per_row) << 3;
    const int64_t p = row / vw.R, r = row - p * vw.R;
    const int64_t gbase = ((p / vw.tp) * vw.GR + r / vw.tr) * vw.GC;
    const int64_t off = row * vw.C + col;
    float code[8], v[8];
    const int nvalid = (int)min((int64_t)8, vw.C - col);
    if constexpr (O == Out::kS4P) {
      uint32_t w = 0;
      if (vec_ok) w = reinterpret_cast<const uint32_t*>(q)[off >> 3];
      else for (int j = 0; j < nvalid; j += 2)
        w |= (uint32_t)reinterpret_cast<const uint8_t*>(q)[(off + j) >> 1] << (4 * j);
#pragma unroll
      for (int j = 0; j < 8; ++j) code[j] = (float)(((int)(w << (28 - 4 * j))) >> 28);
    } else {
      uint8_t b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (vec_ok) *reinterpret_cast<uint2*>(b) =
          *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(q) + off);
      else for (int j = 0; j < nvalid; ++j) b[j] = reinterpret_cast<const uint8_t*>(q)[off + j];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        code[j] = (O == Out::kE4M3 || O == Out::kMX8) ? e4m3_to_float(b[j])
                  : ((O == Out::kMX4 || O == Out::kNV4) ? e2m1_to_float(b[j]) : (float)(int8_t)b[j]);
    }
    // scale group of each of the eight columns: one division, then a running remainder
    int64_t g = gbase + col / vw.tc;
    int64_t left = vw.tc - (col - (col / vw.tc) * vw.tc);   // columns left in this group
    float sc = load1<S>(scale, g);
    float zp = has_zp ? (float)zero_point[g] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float cv = round_to<S>(code[j]);
      if (has_zp) cv = round_to<S>(__fsub_rn(cv, zp));
      v[j] = round_to<S>(__fmul_rn(cv, sc));
      if (--left == 0 && col + j + 1 < vw.C) {
        ++g;
        left = vw.tc;
        sc = load1<S>(scale, g);
        if (has_zp) zp = (float)zero_point[g];
      }
    }
    if (vec_ok) store8<S>(out, off, v);
    else for (int j = 0; j < nvalid; ++j) store1<S>(out, off + j, v[j]);
  }
}

// [rows, cols] bytes -> [cols, rows] bytes through a padded shared tile.
__global__ void __launch_bounds__(kThreads)
transpose_bytes_kernel(const uint8_t* __restrict__ src, int64_t rows, int64_t cols,
                       uint8_t* __restrict__ dst) {
  __shared__ uint8_t tile[64][64 + 4];
  const int64_t r0 = (int64_t)blockIdx.y * 64, c0 = (int64_t)blockIdx.x * 64;
  for (int i = threadIdx.x; i < 64 * 64; i += kThreads) {
    const int r = i / 64, c = i % 64;
    if (r0 + r < rows && c0 + c < cols) tile[r][c] = src[(r0 + r) * cols + c0 + c];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 64; i += kThreads) {
    const int c = i / 64, r = i % 64;
    if (r0 + r < rows && c0 + c < cols) dst[(c0 + c) * rows + r0 + r] = tile[r][c];
  }
}

// ---- host-side dispatch ----------------------------------------------------------------------

int make_view(int64_t P, int64_t R, int64_t C, int64_t tp, int64_t tr, int64_t tc, View* v) {
  if (P <= 0 || R <= 0 || C <= 0 || tp <= 0 || tr <= 0 || tc <= 0) return QWX_ERR_SHAPE;
  if (P % tp || R % tr || C % tc) return QWX_ERR_SHAPE;
  *v = View{P, R, C, tp, tr, tc, P / tp, R / tr, C / tc};
  return QWX_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int grid_for(int64_t items) {
  int64_t blocks = (items + kThreads - 1) / kThreads;
  const int64_t cap = 148 * 16;  // a few waves of resident CTAs per SM
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <typename Fn>
int dispatch_float(int dtype, Fn&& fn) {
  switch (dtype) {
    case QWX_F32: return fn(F32{});
    case QWX_BF16: return fn(BF16{});
    case QWX_F16: return fn(F16{});
    default: return (int)QWX_ERR_DTYPE;
  }
}

template <typename Fn>
int dispatch_out(int qtype, Fn&& fn) {
  switch (qtype) {
    case QWX_S8: return fn(std::integral_constant<Out, Out::kS8>{});
    case QWX_S4U: return fn(std::integral_constant<Out, Out::kS4U>{});
    case QWX_S4: return fn(std::integral_constant<Out, Out::kS4P>{});
    case QWX_E4M3: return fn(std::integral_constant<Out, Out::kE4M3>{});
    case QWX_MXFP8: return fn(std::integral_constant<Out, Out::kMX8>{});
    case QWX_MXFP4: return fn(std::integral_constant<Out, Out::kMX4>{});
    case QWX_NVFP4: return fn(std::integral_constant<Out, Out::kNV4>{});
    default: return (int)QWX_ERR_DTYPE;
  }
}

// Tiles that are contiguous row segments of whole 16-byte vectors are quantized in one pass
// over x with no scratch memory at all.
bool row_segment_view(const void* x, const void* q, int64_t tp, int64_t tr, int64_t tc) {
  return tp == 1 && tr == 1 && tc % 8 == 0 && aligned16(x) && aligned16(q);
}

int check_method(int method, int has_arg, int qtype) {
  if (method != QWX_ABSMAX && method != QWX_MINMAX && method != QWX_RMS) return QWX_ERR_UNSUPPORTED;
  if (method == QWX_RMS && !has_arg) return QWX_ERR_SHAPE;
  if (method == QWX_MINMAX && (qtype == QWX_E4M3 || qtype == QWX_MXFP8 || qtype == QWX_MXFP4 || qtype == QWX_NVFP4)) return QWX_ERR_DTYPE;  // numerics.py:64-92
  return QWX_OK;
}

int run_calibrate_tiles(const void* x, int x_dtype, const View& vw, const CalibArgs& cal,
                        void* out_a, void* out_b, void* ws, size_t ws_bytes, cudaStream_t st) {
  const size_t need = (size_t)vw.groups() * 2 * sizeof(int);
  if (ws == nullptr || ws_bytes < need) return QWX_ERR_WORKSPACE;
  // every refusal comes before the first thing put on the stream
  const int64_t chunks = (vw.tr + kChunkRows - 1) / kChunkRows;
  const int64_t gy = vw.GR * chunks;
  if (gy > 65535 || vw.P > 65535) return QWX_ERR_UNSUPPORTED;
  if (cudaMemsetAsync(ws, 0, need, st) != cudaSuccess) return QWX_ERR_LAUNCH;
  dim3 grid((unsigned)((vw.C + kChunkCols - 1) / kChunkCols), (unsigned)gy, (unsigned)vw.P);
  const int vec_ok = (vw.C % 8 == 0) && aligned16(x);
  return dispatch_float(x_dtype, [&](auto t) {
    using T = decltype(t);
    calibrate_tiles_kernel<T><<<grid, kThreads, 0, st>>>(x, vw, cal.method, vec_ok, (int*)ws);
    QWX_CHECK_LAUNCH();
    finish_calibration_kernel<T><<<(unsigned)((vw.groups() + 255) / 256), 256, 0, st>>>(
        (const int*)ws, vw.groups(), vw.tp * vw.tr * vw.tc, cal, out_a, out_b);
    QWX_CHECK_LAUNCH();
    return (int)QWX_OK;
  });
}

int run_apply(const void* x, int x_dtype, const View& vw, const void* scale, const void* zp,
              int qtype, int rounding, void* q, cudaStream_t st) {
  if (qtype == QWX_S4 && (vw.C & 1)) return QWX_ERR_SHAPE;
  const int vec_ok = (vw.C % 8 == 0) && aligned16(x) && aligned16(q);
  const int64_t vecs = vw.P * vw.R * ((vw.C + 7) / 8);
  return dispatch_float(x_dtype, [&](auto t) {
    using T = decltype(t);
    return dispatch_out(qtype, [&](auto o) {
      apply_scale_kernel<T, decltype(o)::value><<<grid_for(vecs), kThreads, 0, st>>>(
          x, vw, scale, (const int8_t*)zp, rounding, vec_ok, q);
      QWX_CHECK_LAUNCH();
      return (int)QWX_OK;
    });
  });
}

}  // namespace
}  // namespace qwx

using namespace qwx;

extern "C" {

size_t qwx_quantize_workspace_bytes(int64_t P, int64_t R, int64_t C, int64_t tp, int64_t tr,
                                    int64_t tc) {
  View vw;
  if (make_view(P, R, C, tp, tr, tc, &vw) != QWX_OK) return 0;
  // statistics (two int32 per tile) + calibration values for the fused entry point.
  return (size_t)vw.groups() * (2 * sizeof(int) + 2 * sizeof(float)) + 256;
}

int qwx_calibrate(const void* x, int x_dtype, int64_t P, int64_t R, int64_t C, int64_t tp,
                  int64_t tr, int64_t tc, int method, int has_arg, double arg, void* out_a,
                  void* out_b, void* workspace, size_t workspace_bytes, qwx_stream_t stream) {
  if (!x || !out_a) return QWX_ERR_NULL;
  View vw;
  int rc = make_view(P, R, C, tp, tr, tc, &vw);
  if (rc) return rc;
  rc = check_method(method, has_arg, QWX_S8);
  if (rc) return rc;
  if (method == QWX_MINMAX && !out_b) return QWX_ERR_NULL;
  CalibArgs cal{method, has_arg, (float)arg};
  return run_calibrate_tiles(x, x_dtype, vw, cal, out_a, out_b, workspace, workspace_bytes,
                             (cudaStream_t)stream);
}

int qwx_compute_scale_zero_point(const void* calib_a, const void* calib_b, int dtype, int64_t n,
                                 int qtype, void* scale, void* zero_point, qwx_stream_t stream) {
  if (!calib_a || !scale) return QWX_ERR_NULL;
  if (calib_b && !zero_point) return QWX_ERR_NULL;
  if (calib_b && (qtype == QWX_E4M3 || qtype == QWX_MXFP8 || qtype == QWX_MXFP4 || qtype == QWX_NVFP4)) return QWX_ERR_DTYPE;
  if (n <= 0) return QWX_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  return dispatch_float(dtype, [&](auto t) {
    using T = decltype(t);
    switch (qtype) {
      case QWX_S8:
        scale_zero_point_kernel<T, S8><<<blocks, 256, 0, st>>>(calib_a, calib_b, n, scale, (int8_t*)zero_point);
        break;
      case QWX_S4: case QWX_S4U:
        scale_zero_point_kernel<T, S4><<<blocks, 256, 0, st>>>(calib_a, calib_b, n, scale, (int8_t*)zero_point);
        break;
      case QWX_E4M3:
        scale_zero_point_kernel<T, E4M3><<<blocks, 256, 0, st>>>(calib_a, calib_b, n, scale, (int8_t*)zero_point);
        break;
      case QWX_MXFP8:
        scale_zero_point_kernel<T, MX8><<<blocks, 256, 0, st>>>(calib_a, calib_b, n, scale, (int8_t*)zero_point);
        break;
      case QWX_MXFP4:
        scale_zero_point_kernel<T, MX4><<<blocks, 256, 0, st>>>(calib_a, calib_b, n, scale, (int8_t*)zero_point);
        break;
      case QWX_NVFP4:
        scale_zero_point_kernel<T, NV4><<<blocks, 256, 0, st>>>(calib_a, calib_b, n, scale, (int8_t*)zero_point);
        break;
      default: return (int)QWX_ERR_DTYPE;
    }
    QWX_CHECK_LAUNCH();
    return (int)QWX_OK;
  });
}

int qwx_quantize_with_scale(const void* x, int x_dtype, int64_t P, int64_t R, int64_t C,
                            int64_t tp, int64_t tr, int64_t tc, const void* scale,
                            const void* zero_point, int qtype, int rounding, void* q,
                            qwx_stream_t stream) {
  if (!x || !scale || !q) return QWX_ERR_NULL;
  if (zero_point && (qtype == QWX_E4M3 || qtype == QWX_MXFP8 || qtype == QWX_MXFP4 || qtype == QWX_NVFP4)) return QWX_ERR_DTYPE;
  View vw;
  int rc = make_view(P, R, C, tp, tr, tc, &vw);
  if (rc) return rc;
  return run_apply(x, x_dtype, vw, scale, zero_point, qtype, rounding, q, (cudaStream_t)stream);
}

int qwx_quantize(const void* x, int x_dtype, int64_t P, int64_t R, int64_t C, int64_t tp,
                 int64_t tr, int64_t tc, int method, int has_arg, double arg, int qtype,
                 int rounding, void* q, void* scale, void* zero_point, void* workspace,
                 size_t workspace_bytes, qwx_stream_t stream) {
  if (!x || !q || !scale) return QWX_ERR_NULL;
  View vw;
  int rc = make_view(P, R, C, tp, tr, tc, &vw);
  if (rc) return rc;
  rc = check_method(method, has_arg, qtype);
  if (rc) return rc;
  if (method == QWX_MINMAX && !zero_point) return QWX_ERR_NULL;
  if (qtype == QWX_S4 && (C & 1)) return QWX_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  CalibArgs cal{method, has_arg, (float)arg};

  // One pass when every tile is a contiguous row segment of whole 16-byte vectors.
  if (row_segment_view(x, q, tp, tr, tc)) {
    const int64_t segments = P * R * (C / tc);
    if (x_dtype == QWX_BF16 && qtype == QWX_S8 && method == QWX_ABSMAX && !has_arg &&
        rounding == QWX_STRICT && tc > 32 * 8 * kCache && tc <= kThreads * 8 * 8) {
      const bool wide = tc > kThreads * 4 * 8;   // rows of 8193..16384 values: 8 vectors per thread
      const int64_t cap = 148 * (wide ? kRowCtas / 2 : kRowCtas);
      const unsigned grid = (unsigned)(segments < cap ? segments : cap);
      const size_t ring_bytes = (size_t)kRowDepth * (tc / 8) * 16;
      static PerDeviceOnce configured;
      if (configured.first()) {
        if (cudaFuncSetAttribute(quantize_rows_bf16_s8_kernel<4>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kRowDepth * kThreads * 4 * 16) != cudaSuccess ||
            cudaFuncSetAttribute(quantize_rows_bf16_s8_kernel<8>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kRowDepth * kThreads * 8 * 16) != cudaSuccess)
          return (int)QWX_ERR_LAUNCH;
        configured.mark();
      }
      const cudaError_t e =
          wide ? launch_dependent(quantize_rows_bf16_s8_kernel<8>, dim3(grid), dim3(kThreads), ring_bytes,
                                  st, (const uint4*)x, segments, (int)(tc / 8), (uint2*)q,
                                  (__nv_bfloat16*)scale)
               : launch_dependent(quantize_rows_bf16_s8_kernel<4>, dim3(grid), dim3(kThreads), ring_bytes,
                                  st, (const uint4*)x, segments, (int)(tc / 8), (uint2*)q,
                                  (__nv_bfloat16*)scale);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return (int)QWX_ERR_LAUNCH;
      }
      return (int)QWX_OK;
    }
    if (qtype == QWX_NVFP4 && tc == 16 && method == QWX_ABSMAX && !has_arg &&
        (x_dtype == QWX_BF16 || x_dtype == QWX_F32)) {
      const int64_t nvec = segments * 2;
      const unsigned blocks = (unsigned)((nvec + kThreads - 1) / kThreads);
      const int strict = rounding == QWX_STRICT ? 1 : 0;
      const cudaError_t e =
          x_dtype == QWX_BF16
              ? launch_dependent(quantize_mx8_blocks_kernel<BF16, NV4>, dim3(blocks), dim3(kThreads), 0, st, x, nvec, q, scale, strict)
              : launch_dependent(quantize_mx8_blocks_kernel<F32, NV4>, dim3(blocks), dim3(kThreads), 0, st, x, nvec, q, scale, strict);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return (int)QWX_ERR_LAUNCH;
      }
      return (int)QWX_OK;
    }
    if (qtype == QWX_MXFP4 && tc == 32 && method == QWX_ABSMAX && !has_arg &&
        (x_dtype == QWX_BF16 || x_dtype == QWX_F32)) {
      const int64_t nvec = segments * 4;
      const unsigned blocks = (unsigned)((nvec + kThreads - 1) / kThreads);
      const cudaError_t e =
          x_dtype == QWX_BF16
              ? launch_dependent(quantize_mx8_blocks_kernel<BF16, MX4>, dim3(blocks), dim3(kThreads), 0, st, x, nvec, q, scale, 1)
              : launch_dependent(quantize_mx8_blocks_kernel<F32, MX4>, dim3(blocks), dim3(kThreads), 0, st, x, nvec, q, scale, 1);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return (int)QWX_ERR_LAUNCH;
      }
      return (int)QWX_OK;
    }
    if (qtype == QWX_MXFP8 && tc == 32 && method == QWX_ABSMAX && !has_arg &&
        (x_dtype == QWX_BF16 || x_dtype == QWX_F32)) {
      const int64_t nvec = segments * 4;
      const unsigned blocks = (unsigned)((nvec + kThreads - 1) / kThreads);
      const cudaError_t e =
          x_dtype == QWX_BF16
              ? launch_dependent(quantize_mx8_blocks_kernel<BF16>, dim3(blocks), dim3(kThreads), 0, st, x, nvec, q, scale, 1)
              : launch_dependent(quantize_mx8_blocks_kernel<F32>, dim3(blocks), dim3(kThreads), 0, st, x, nvec, q, scale, 1);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return (int)QWX_ERR_LAUNCH;
      }
      return (int)QWX_OK;
    }
    return dispatch_float(x_dtype, [&](auto t) {
      using T = decltype(t);
      return dispatch_out(qtype, [&](auto o) {
        constexpr Out O = decltype(o)::value;
        cudaError_t e;
        auto small = [&](auto g) {
          constexpr int G = decltype(g)::value;
          const int64_t blocks = (segments + kThreads / G - 1) / (kThreads / G);
          return launch_dependent(quantize_rows_kernel<T, O, G>, dim3((unsigned)blocks), dim3(kThreads), 0, st,
                                  x, segments, tc, cal, rounding, q, scale, (int8_t*)zero_point);
        };
        // one 16-byte vector per lane where the segment is shorter than a warp's worth (the sum
        // of squares keeps the whole-warp order)
        if (tc <= 32 && method != QWX_RMS) {
          e = small(std::integral_constant<int, 4>{});
        } else if (tc <= 64 && method != QWX_RMS) {
          e = small(std::integral_constant<int, 8>{});
        } else if (tc <= 128 && method != QWX_RMS) {
          e = small(std::integral_constant<int, 16>{});
        } else if (tc <= 32 * 8 * kCache) {
          e = small(std::integral_constant<int, 32>{});
        } else {
          e = launch_dependent(quantize_rows_kernel<T, O, 256>, dim3((unsigned)segments), dim3(kThreads), 0,
                               st, x, segments, tc, cal, rounding, q, scale, (int8_t*)zero_point);
        }
        if (e != cudaSuccess) {
          (void)cudaGetLastError();
          return (int)QWX_ERR_LAUNCH;
        }
        return (int)QWX_OK;
      });
    });
  }

  // General view: statistics -> calibration -> scale -> elementwise pass.
  const size_t stats_bytes = (size_t)vw.groups() * 2 * sizeof(int);
  const size_t need = stats_bytes + (size_t)vw.groups() * 2 * sizeof(float);
  if (!workspace || workspace_bytes < need) return QWX_ERR_WORKSPACE;
  char* ws = (char*)workspace;
  void* calib_a = ws + stats_bytes;
  void* calib_b = ws + stats_bytes + (size_t)vw.groups() * sizeof(float);
  rc = run_calibrate_tiles(x, x_dtype, vw, cal, calib_a, calib_b, ws, stats_bytes, st);
  if (rc) return rc;
  rc = qwx_compute_scale_zero_point(calib_a, method == QWX_MINMAX ? calib_b : nullptr, x_dtype,
                                    vw.groups(), qtype, scale, zero_point, stream);
  if (rc) return rc;
  return run_apply(x, x_dtype, vw, scale, method == QWX_MINMAX ? zero_point : nullptr, qtype,
                   rounding, q, st);
}

// ---- quantize without any allocation by anyone --------------------------------------------
//
// Some callers cannot obtain device scratch at the moment they need to quantize: a custom-call
// handler that runs inside a framework whose buffers were all planned before the step began
// has nobody to ask for a workspace, and a serving loop that has finished warm-up must not
// call cudaMalloc, because that call synchronises the whole device and can fail under memory
// pressure.  For them the statistics scratch of the tiled quantizer lives in the library
// image: a fixed array in device global memory that every GPU loading the library keeps
// until the process exits.

constexpr size_t kBuiltinScratchBytes = 1u << 20;  // 1 MiB: views of up to 65,520 tiles
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

namespace {

// Device address of g_builtin_scratch on the current device.  In host code the array's name
// is only a handle; the address a kernel can use comes from cudaGetSymbolAddress, asked once
// per device while that device is current, and remembered.
int builtin_scratch_address(void** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void* address[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return QWX_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(mu);
  if (address[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_builtin_scratch) != cudaSuccess || p == nullptr)
      return QWX_ERR_LAUNCH;
    address[dev] = p;
  }
  *out = address[dev];
  return QWX_OK;
}

}  // namespace

size_t qwx_quantize_builtin_scratch_bytes(void) { return kBuiltinScratchBytes; }

int qwx_quantize_noalloc(const void* x, int x_dtype, int64_t P, int64_t R, int64_t C, int64_t tp,
                         int64_t tr, int64_t tc, int method, int has_arg, double arg, int qtype,
                         int rounding, void* q, void* scale, void* zero_point,
                         qwx_stream_t stream) {
  View vw;
  int rc = make_view(P, R, C, tp, tr, tc, &vw);
  if (rc) return rc;
  // Refuse, before touching anything, a view whose statistics do not fit the built-in array.
  // Row-segment views take the one-pass kernels, which use no scratch: they are never refused,
  // whatever their tile count.
  if (!row_segment_view(x, q, tp, tr, tc) &&
      qwx_quantize_workspace_bytes(P, R, C, tp, tr, tc) > kBuiltinScratchBytes)
    return QWX_ERR_WORKSPACE;
  void* scratch = nullptr;
  rc = builtin_scratch_address(&scratch);
  if (rc) return rc;
  // qwx_quantize clears the statistics it accumulates into (an asynchronous memset on
  // `stream`) and neither it nor the kernels behind it allocate.
  return qwx_quantize(x, x_dtype, P, R, C, tp, tr, tc, method, has_arg, arg, qtype, rounding, q,
                      scale, zero_point, scratch, kBuiltinScratchBytes, stream);
}

int qwx_dequantize(const void* q, int qtype, int64_t P, int64_t R, int64_t C, int64_t tp,
                   int64_t tr, int64_t tc, const void* scale, int scale_dtype,
                   const void* zero_point, void* out, qwx_stream_t stream) {
  if (!q || !scale || !out) return QWX_ERR_NULL;
  View vw;
  int rc = make_view(P, R, C, tp, tr, tc, &vw);
  if (rc) return rc;
  if (qtype == QWX_S4 && (C & 1)) return QWX_ERR_SHAPE;
  const int vec_ok = (C % 8 == 0) && aligned16(out) &&
                     ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
  const int64_t vecs = P * R * ((C + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
  return dispatch_float(scale_dtype, [&](auto s) {
    using S = decltype(s);
    return dispatch_out(qtype, [&](auto o) {
      dequantize_kernel<S, decltype(o)::value><<<grid_for(vecs), kThreads, 0, st>>>(
          q, vw, scale, (const int8_t*)zero_point, vec_ok, out);
      QWX_CHECK_LAUNCH();
      return (int)QWX_OK;
    });
  });
}

int qwx_transpose_codes(const void* src, int64_t rows, int64_t cols, void* dst,
                        qwx_stream_t stream) {
  if (!src || !dst) return QWX_ERR_NULL;
  if (rows <= 0 || cols <= 0) return QWX_ERR_SHAPE;
  dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64));
  if (grid.y > 65535) return QWX_ERR_UNSUPPORTED;
  transpose_bytes_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)src, rows, cols, (uint8_t*)dst);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

}  // extern "C"
