// Blockwise Walsh-Hadamard rotation fused with quantization: the device side of
// qwix/contrib/hadamard_rot.py:99-117 (x . H per block of the contraction axis for the
// activation, H . w / d for the weight) and of the activation half of
// qwix/contrib/kernels/fused_hadamard_quantized_matmul.py:150-170 (sign flip, rotate, sign
// flip, absmax-quantize).  H is the Sylvester matrix with +/-1 entries, so x . H is a fast
// Walsh-Hadamard transform in natural order: log2(d) butterfly stages, done here in float32 on
// values held in registers (three stages inside a thread's 8 values, the rest by warp shuffles
// between the 16 lanes that share a 128-value block).
#include "common.cuh"

namespace qwx {
namespace {

constexpr int kHThreads = 256;
constexpr int kHVec = 4;      // 16-byte vectors per thread: rows up to 256 * 4 * 8 = 8192 values
constexpr int kBlock = 128;   // Hadamard block (2^7)

__device__ __forceinline__ void fwht8(float (&v)[8]) {
#pragma unroll
  for (int s = 1; s < 8; s <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if ((i & s) == 0) {
        const float a = v[i], b = v[i | s];
        v[i] = a + b;
        v[i | s] = a - b;
      }
    }
  }
}

// Stages over the four lane bits that index the 16 vectors of a 128-value block.
__device__ __forceinline__ void fwht_lanes(float (&v)[8], int lane) {
#pragma unroll
  for (int m = 1; m < 16; m <<= 1) {
    const bool upper = (lane & m) != 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = upper ? other - v[i] : v[i] + other;
    }
  }
}

__device__ __forceinline__ void apply_signs8(float (&v)[8], const int8_t* s, int64_t at) {
  const int2 w = *reinterpret_cast<const int2*>(s + at);
  const int words[2] = {w.x, w.y};
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if ((int8_t)(words[i >> 2] >> (8 * (i & 3))) < 0) v[i] = -v[i];
}

// One CTA per row (persistent, stride gridDim.x): load the row, rotate every 128-value block,
// round to bf16 (the rotated activation of the reference is a bf16 array), row absmax, scale,
// quantize.  Q = S8 or E4M3.
template <typename Q>
__global__ void __launch_bounds__(kHThreads, 2)
hadamard_quantize_rows_kernel(const uint4* __restrict__ x, int64_t rows, int nvec,
                              const int8_t* __restrict__ signs_in,
                              const int8_t* __restrict__ signs_out, int rounding,
                              uint2* __restrict__ q, __nv_bfloat16* __restrict__ scale) {
  __shared__ uint32_t red[2][kHThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool strict = rounding == QWX_STRICT;
  uint4 rot[kHVec];  // the rotated row, as packed bf16

  int iter = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, ++iter) {
    uint32_t bits = 0;
#pragma unroll
    for (int it = 0; it < kHVec; ++it) {
      const int vi = tid + it * kHThreads;
      // Whole warps run or skip together: nvec is a multiple of 16 and a block never
      // straddles a half-warp, but the shuffles need all 32 lanes, so inactive lanes
      // rotate zeros.
      float v[8];
      if (vi < nvec) unpack_bf16x8(x[row * nvec + vi], v);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
      }
      if (signs_in && vi < nvec) apply_signs8(v, signs_in, (int64_t)vi * 8);
      fwht8(v);
      fwht_lanes(v, lane);
      if (signs_out && vi < nvec) apply_signs8(v, signs_out, (int64_t)vi * 8);
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
        bits = max(bits, max((w[j] << 16) & 0x7fffffffu, w[j] & 0x7fff0000u));
      }
      rot[it] = make_uint4(w[0], w[1], w[2], w[3]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
    uint32_t* slot = red[iter & 1];
    if (lane == 0) slot[warp] = bits;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kHThreads / 32; ++i) bits = max(bits, slot[i]);
    const float absmax = __uint_as_float(bits);

    // scale = absmax / bound in bf16 with the tiny-scale guard (qarray.py:557-562)
    float s = round_to<BF16>(__fdiv_rn(absmax, sym_bound<Q>()));
    if (s < 0x1p-63f) s = 1.0f;
    if (tid == 0) scale[row] = __float2bfloat16_rn(s);

#pragma unroll
    for (int it = 0; it < kHVec; ++it) {
      const int vi = tid + it * kHThreads;
      if (vi >= nvec) continue;
      float v[8];
      unpack_bf16x8(rot[it], v);
      int c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float y = __fdiv_rn(v[j], s);
        if (strict) y = round_to<BF16>(y);
        c[j] = to_code<Q>(y);
      }
      uint2 o;
      o.x = (c[0] & 0xff) | ((c[1] & 0xff) << 8) | ((c[2] & 0xff) << 16) | ((uint32_t)(c[3] & 0xff) << 24);
      o.y = (c[4] & 0xff) | ((c[5] & 0xff) << 8) | ((c[6] & 0xff) << 16) | ((uint32_t)(c[7] & 0xff) << 24);
      q[row * nvec + vi] = o;
    }
  }
}

// ---- one thread per 128-value block ----------------------------------------------------------
//
// The kernel above spends most of its issue slots on the four shuffle stages.  When a row is
// 1..32 blocks long (a power of two), a warp takes 32 consecutive blocks instead, one per lane:
// all seven butterfly stages run on registers, and the row absmax is a shuffle reduction over the
// lanes that share a row.  Blocks reach the lanes through a per-warp cp.async ring in shared
// memory; chunk j of block b sits at slot j ^ (b & 15) so that the 16-byte reads of eight
// neighbouring lanes fall in different banks.
constexpr int kBWarps = 4;
constexpr int kBThreads = kBWarps * 32;
constexpr int kBDepth = 3;
constexpr int kBStageVec = 32 * 16;   // 16-byte vectors per stage: 32 blocks of 256 bytes
constexpr size_t kBSmemBytes = (size_t)kBWarps * kBDepth * kBStageVec * 16;

__device__ __forceinline__ void fwht128(float (&v)[kBlock]) {
#pragma unroll
  for (int s = 1; s < kBlock; s <<= 1) {
#pragma unroll
    for (int i = 0; i < kBlock; ++i) {
      if ((i & s) == 0) {
        const float a = v[i], b = v[i | s];
        v[i] = a + b;
        v[i | s] = a - b;
      }
    }
  }
}

template <typename Q>
__global__ void __launch_bounds__(kBThreads, 2)
hadamard_quantize_blocks_kernel(const uint4* __restrict__ x, int64_t rows, int nblk_log2,
                                uint4* __restrict__ q, __nv_bfloat16* __restrict__ scale) {
  extern __shared__ uint4 bring[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint4* ring = bring + (size_t)warp * kBDepth * kBStageVec;
  const int64_t total_blocks = rows << nblk_log2;
  const int64_t groups = (total_blocks + 31) >> 5;
  const int64_t gstride = (int64_t)gridDim.x * kBWarps;
  const int64_t first = (int64_t)warp * gridDim.x + blockIdx.x;

  int64_t fetch_g = first;
  int fetch_stage = 0;
  auto fetch = [&]() {
    if (fetch_g < groups) {
      const uint4* src = x + fetch_g * kBStageVec;
      const int64_t left = (total_blocks - fetch_g * 32) * 16;
      const int valid = (int)(left < kBStageVec ? left : kBStageVec);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int c = i * 32 + lane;
        if (c < valid) {
          const int b = c >> 4, j = c & 15;
          const uint32_t dst = (uint32_t)__cvta_generic_to_shared(
              ring + fetch_stage * kBStageVec + b * 16 + (j ^ (b & 15)));
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + c) : "memory");
        }
      }
      fetch_g += gstride;
    }
    if (++fetch_stage == kBDepth) fetch_stage = 0;
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  for (int d = 0; d < kBDepth - 1; ++d) fetch();

  int stage = 0;
  for (int64_t g = first; g < groups; g += gstride) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kBDepth - 2) : "memory");
    __syncwarp();
    const int64_t blk = g * 32 + lane;
    const bool active = blk < total_blocks;
    float v[kBlock];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      uint4 u = make_uint4(0u, 0u, 0u, 0u);
      if (active) u = ring[stage * kBStageVec + lane * 16 + (j ^ (lane & 15))];
      float t[8];
      unpack_bf16x8(u, t);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[j * 8 + i] = t[i];
    }
    __syncwarp();   // every lane has read the stage before it is refilled
    if (++stage == kBDepth) stage = 0;
    fetch();

    fwht128(v);

    // The rotated activation is a bf16 array in the reference: round, then row absmax.
    uint32_t w[kBlock / 2];
    __nv_bfloat162 m2 = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < kBlock / 2; ++k) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
      w[k] = *reinterpret_cast<const uint32_t*>(&h);
      m2 = __hmax2_nan(m2, __habs2(h));
    }
    const float2 mf = __bfloat1622float2(m2);
    uint32_t bits = max(__float_as_uint(mf.x), __float_as_uint(mf.y));  // NaN sorts last
    for (int o = (1 << nblk_log2) >> 1; o > 0; o >>= 1)
      bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
    const float absmax = __uint_as_float(bits);

    float s = round_to<BF16>(__fdiv_rn(absmax, sym_bound<Q>()));
    if (s < 0x1p-63f) s = 1.0f;
    if (active && (lane & ((1 << nblk_log2) - 1)) == 0) scale[blk >> nblk_log2] = __float2bfloat16_rn(s);

    const float as = fabsf(s);
    const bool fast = as > 0x1p-100f && as < 0x1p100f && bits < 0x7f800000u;
    uint32_t code[kBlock / 4];
    if (fast) {
      // Correctly rounded bf16 quotients from three packed bf16 FMAs (Markstein's division):
      // q0 = x * r, rem = x - q0 * s (one rounding), z = q0 + rem * r, with r = RN_bf16(1 / s).
      const __nv_bfloat16 sb = __float2bfloat16_rn(s);
      const __nv_bfloat16 rb = __float2bfloat16_rn(__frcp_rn(s));
      const __nv_bfloat162 r2 = __halves2bfloat162(rb, rb);
      const __nv_bfloat162 ns2 = __hneg2(__halves2bfloat162(sb, sb));
#pragma unroll
      for (int k = 0; k < kBlock / 4; ++k) {
        uint32_t zw[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(&w[2 * k + h]);
          const __nv_bfloat162 q0 = __hmul2(xv, r2);
          const __nv_bfloat162 rem = __hfma2(q0, ns2, xv);
          const __nv_bfloat162 z = __hfma2(rem, r2, q0);
          zw[h] = *reinterpret_cast<const uint32_t*>(&z);
        }
        if constexpr (Q::kFloat) {
          // clip to +/-448 and round to nearest even: the saturating e4m3 convert
          uint16_t lo, hi;
          asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo)
              : "f"(__uint_as_float(zw[0] & 0xffff0000u)), "f"(__uint_as_float(zw[0] << 16)));
          asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi)
              : "f"(__uint_as_float(zw[1] & 0xffff0000u)), "f"(__uint_as_float(zw[1] << 16)));
          code[k] = (uint32_t)lo | ((uint32_t)hi << 16);
        } else {
          int c[4];
          asm("{ .reg .b16 lo, hi;\n\t mov.b32 {lo, hi}, %2;\n\t"
              " cvt.rni.s32.bf16 %0, lo;\n\t cvt.rni.s32.bf16 %1, hi; }"
              : "=r"(c[0]), "=r"(c[1]) : "r"(zw[0]));
          asm("{ .reg .b16 lo, hi;\n\t mov.b32 {lo, hi}, %2;\n\t"
              " cvt.rni.s32.bf16 %0, lo;\n\t cvt.rni.s32.bf16 %1, hi; }"
              : "=r"(c[2]), "=r"(c[3]) : "r"(zw[1]));
          uint32_t hi16;
          asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi16) : "r"(c[3]), "r"(c[2]), "r"(0u));
          asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(code[k]) : "r"(c[1]), "r"(c[0]), "r"(hi16));
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < kBlock / 4; ++k) {
        uint32_t word = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t pair = w[2 * k + (e >> 1)];
          const float xv = __uint_as_float((e & 1) ? (pair & 0xffff0000u) : (pair << 16));
          const float y = round_to<BF16>(__fdiv_rn(xv, s));
          word |= (uint32_t)(to_code<Q>(y) & 0xff) << (8 * e);
        }
        code[k] = word;
      }
    }
    if (active) {
      uint4* dst = q + blk * 8;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        dst[k] = make_uint4(code[4 * k], code[4 * k + 1], code[4 * k + 2], code[4 * k + 3]);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Rotation only, blocks along the contiguous axis: out = x . H per 128 columns (bf16).
__global__ void __launch_bounds__(kHThreads)
hadamard_rotate_cols_kernel(const uint4* __restrict__ x, int64_t total_vec,
                            const int8_t* __restrict__ signs_in,
                            const int8_t* __restrict__ signs_out, int vec_per_row,
                            uint4* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t start = (int64_t)blockIdx.x * kHThreads + threadIdx.x;
  // total_vec is a multiple of 16 and blocks are 16 consecutive vectors: keep warps whole.
  for (int64_t base = (int64_t)blockIdx.x * kHThreads; base < total_vec;
       base += (int64_t)gridDim.x * kHThreads) {
    const int64_t vi = base + threadIdx.x;
    float v[8];
    if (vi < total_vec) unpack_bf16x8(x[vi], v);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    const int64_t col = (vi % vec_per_row) * 8;
    if (signs_in && vi < total_vec) apply_signs8(v, signs_in, col);
    fwht8(v);
    fwht_lanes(v, lane);
    if (signs_out && vi < total_vec) apply_signs8(v, signs_out, col);
    if (vi < total_vec) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
      out[vi] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  (void)start;
}

// Rotation only, blocks along the row axis of a [K, N] weight: out = H . w_block / 128.  One
// thread owns one column of one block (128 values in registers); neighbouring threads own
// neighbouring columns, so every load and store is coalesced.
__global__ void __launch_bounds__(128)
hadamard_rotate_rows_kernel(const __nv_bfloat16* __restrict__ w, int64_t K, int64_t N,
                            const int8_t* __restrict__ signs_in,
                            const int8_t* __restrict__ signs_out, __nv_bfloat16* __restrict__ out) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t k0 = (int64_t)blockIdx.y * kBlock;
  if (n >= N) return;
  float v[kBlock];
#pragma unroll
  for (int i = 0; i < kBlock; ++i) {
    v[i] = __bfloat162float(w[(k0 + i) * N + n]);
    if (signs_in && signs_in[k0 + i] < 0) v[i] = -v[i];
  }
#pragma unroll
  for (int s = 1; s < kBlock; s <<= 1) {
#pragma unroll
    for (int i = 0; i < kBlock; ++i) {
      if ((i & s) == 0) {
        const float a = v[i], b = v[i | s];
        v[i] = a + b;
        v[i | s] = a - b;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kBlock; ++i) {
    // the reference rounds the product to bf16, then divides by the block size (exact)
    float r = round_to<BF16>(v[i]);
    if (signs_out && signs_out[k0 + i] < 0) r = -r;
    out[(k0 + i) * N + n] = __float2bfloat16_rn(r * (1.0f / kBlock));
  }
}

}  // namespace
}  // namespace qwx

using namespace qwx;

extern "C" {

int qwx_hadamard_quantize(const void* x, int x_dtype, int64_t rows, int64_t K, int block,
                          const int8_t* signs_in, const int8_t* signs_out, int qtype,
                          int rounding, void* q, void* scale, qwx_stream_t stream) {
  if (!x || !q || !scale) return QWX_ERR_NULL;
  if (x_dtype != QWX_BF16) return QWX_ERR_DTYPE;
  if (block != kBlock) return QWX_ERR_UNSUPPORTED;
  if (rows <= 0 || K <= 0 || K % kBlock) return QWX_ERR_SHAPE;
  if (K > (int64_t)kHThreads * kHVec * 8) return QWX_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7)) return QWX_ERR_ALIGN;
  if ((signs_in && (reinterpret_cast<uintptr_t>(signs_in) & 7)) ||
      (signs_out && (reinterpret_cast<uintptr_t>(signs_out) & 7)))
    return QWX_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t nblk = K / kBlock;
  if (!signs_in && !signs_out && rounding == QWX_STRICT && nblk <= 32 && (nblk & (nblk - 1)) == 0 &&
      (reinterpret_cast<uintptr_t>(q) & 15) == 0 && (qtype == QWX_E4M3 || qtype == QWX_S8)) {
    int log2 = 0;
    while ((1 << log2) < nblk) ++log2;
    const int64_t groups = (rows * nblk + 31) / 32;
    int64_t ctas = (groups + kBWarps - 1) / kBWarps;
    if (ctas > 148 * 2) ctas = 148 * 2;
    static PerDeviceOnce configured;
    if (configured.first()) {
      if (cudaFuncSetAttribute(hadamard_quantize_blocks_kernel<E4M3>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBSmemBytes) != cudaSuccess ||
          cudaFuncSetAttribute(hadamard_quantize_blocks_kernel<S8>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBSmemBytes) != cudaSuccess)
        return QWX_ERR_LAUNCH;
      configured.mark();
    }
    if (qtype == QWX_E4M3)
      hadamard_quantize_blocks_kernel<E4M3><<<(unsigned)ctas, kBThreads, kBSmemBytes, st>>>(
          (const uint4*)x, rows, log2, (uint4*)q, (__nv_bfloat16*)scale);
    else
      hadamard_quantize_blocks_kernel<S8><<<(unsigned)ctas, kBThreads, kBSmemBytes, st>>>(
          (const uint4*)x, rows, log2, (uint4*)q, (__nv_bfloat16*)scale);
    QWX_CHECK_LAUNCH();
    return QWX_OK;
  }
  const int64_t cap = 148 * 4;
  const unsigned grid = (unsigned)(rows < cap ? rows : cap);
  if (qtype == QWX_E4M3)
    hadamard_quantize_rows_kernel<E4M3><<<grid, kHThreads, 0, st>>>(
        (const uint4*)x, rows, (int)(K / 8), signs_in, signs_out, rounding, (uint2*)q,
        (__nv_bfloat16*)scale);
  else if (qtype == QWX_S8)
    hadamard_quantize_rows_kernel<S8><<<grid, kHThreads, 0, st>>>(
        (const uint4*)x, rows, (int)(K / 8), signs_in, signs_out, rounding, (uint2*)q,
        (__nv_bfloat16*)scale);
  else
    return QWX_ERR_DTYPE;
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

int qwx_hadamard_rotate(const void* x, int x_dtype, int64_t R, int64_t C, int axis, int block,
                        const int8_t* signs_in, const int8_t* signs_out, void* out,
                        qwx_stream_t stream) {
  if (!x || !out) return QWX_ERR_NULL;
  if (x_dtype != QWX_BF16) return QWX_ERR_DTYPE;
  if (block != kBlock) return QWX_ERR_UNSUPPORTED;
  if (R <= 0 || C <= 0) return QWX_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (axis == 1) {
    if (C % kBlock) return QWX_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return QWX_ERR_ALIGN;
    const int64_t total = R * (C / 8);
    int64_t blocks = (total + kHThreads - 1) / kHThreads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    hadamard_rotate_cols_kernel<<<(unsigned)blocks, kHThreads, 0, st>>>(
        (const uint4*)x, total, signs_in, signs_out, (int)(C / 8), (uint4*)out);
  } else if (axis == 0) {
    if (R % kBlock) return QWX_ERR_SHAPE;
    if (R / kBlock > 65535) return QWX_ERR_UNSUPPORTED;
    dim3 grid((unsigned)((C + 127) / 128), (unsigned)(R / kBlock));
    hadamard_rotate_rows_kernel<<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, R, C, signs_in,
                                                      signs_out, (__nv_bfloat16*)out);
  } else {
    return QWX_ERR_SHAPE;
  }
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

size_t qwx_hadamard_gemm_workspace_bytes(int64_t M, int64_t K) {
  if (M <= 0 || K <= 0) return 0;
  return (size_t)(M * K) + (size_t)((M * 2 + 255) / 256 * 256);
}

int qwx_hadamard_gemm(const void* a, int64_t M, int64_t K, const int8_t* signs_in,
                      const int8_t* signs_out, const void* wq, const void* sw, int64_t N,
                      int code_dtype, int b_layout, int rounding, void* out, int out_dtype,
                      int epilogue, void* workspace, size_t workspace_bytes, int32_t* error_flag,
                      qwx_stream_t stream) {
  if (!workspace) return QWX_ERR_NULL;
  if (workspace_bytes < qwx_hadamard_gemm_workspace_bytes(M, K)) return QWX_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return QWX_ERR_ALIGN;
  void* sa = workspace;                                     // [M] bf16 row scales
  void* aq = (char*)workspace + (M * 2 + 255) / 256 * 256;  // [M, K] codes
  int rc = qwx_hadamard_quantize(a, QWX_BF16, M, K, kBlock, signs_in, signs_out, code_dtype,
                                 rounding, aq, sa, stream);
  if (rc) return rc;
  return qwx_gemm_q8(aq, wq, code_dtype, b_layout, M, N, K, 0, sa, 0, sw, 0, QWX_BF16, out,
                     out_dtype, epilogue, error_flag, stream);
}

}  // extern "C"
