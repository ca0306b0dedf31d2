// int8 x int8 GEMM for decode-shaped problems: at most 32 rows of activations against a weight
// held [N, K] (K contiguous),
//
//   out[m, n] = (sum_k a[m, k] * w[n, k]) * sa[m] * sb[n]       (dot_general.py:220, :255-258)
//
// The weight is streamed exactly once and nothing else matters: a CTA-wide tcgen05 pipeline
// pays about 12 us of set-up, first-load latency, accumulator hand-over and split-K reduction
// before and after a few microseconds of streaming (the single-CTA kernel of gemm_q8.cu sits
// at 16-22 us for 16-58 MB of weights).  Here every warp owns a contiguous run of
// (16 channels x 256 K) chunks (stream-K at warp granularity, like the int4 weight-only
// kernel), loads its weight bytes with 128-bit loads straight into the A
// fragments of mma.sync.m16n8k32.s8 (channels are the MMA's M, tokens its N), and takes the
// B fragments with one 128-bit shared-memory load per 8 tokens from the activation codes the
// CTA keeps resident.  The K order inside a chunk is permuted consistently for both operands
// (a lane's 16 contiguous bytes feed two MMAs), which a dot product does not notice.
//
// K is cut into `split` slices so that the activation slice fits shared memory; partial sums
// of a strip that is spread over several warps meet as exact int32 atomics in a zeroed
// workspace, and the warp that contributes last scales, converts and clears.
#include "common.cuh"

namespace qwx {
namespace {

constexpr int kSStrip = 16;
constexpr int kSChunkK = 256;     // K per work item: four 64-byte pieces of each of 16 weight rows
constexpr int kSWarps = 12;
constexpr int kSThreads = kSWarps * 32;
constexpr int kSPrefetch = 2;      // chunks (4 KB each) in flight per warp
constexpr size_t kSActCap = 200 * 1024;

struct SkinnyParams {
  const int8_t* a;        // [M, K]
  const int8_t* w;        // [N, K]
  const void* sa;         // [M] or null
  const void* sb;         // [N] or null
  int scale_dtype;
  int M;
  int64_t N, K;
  int split, ks, pitch;
  void* out;
  int out_dtype;
  int epilogue;
  int32_t* ws;            // [M, N], zero on entry, left zero
  int* counters;          // [N / 16], zero on entry, left zero
};

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float load_scale_s(const void* p, int dtype, int64_t i) {
  if (dtype == QWX_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == QWX_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ float round_out_s(float v, int out_dtype) {
  if (out_dtype == QWX_BF16) return round_to<BF16>(v);
  if (out_dtype == QWX_F16) return round_to<F16>(v);
  return v;
}

template <int NT>   // token tiles of 8
__global__ void __launch_bounds__(kSThreads, 1) gemm_q8_skinny_kernel(const SkinnyParams p) {
  extern __shared__ __align__(16) uint8_t act[];
  constexpr int MPAD = NT * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int slice = blockIdx.x % p.split;
  const int cta_in_slice = blockIdx.x / p.split;
  const int ctas_per_slice = gridDim.x / p.split;

  // ---- activation codes of this K slice: tokens x ks bytes, rows `pitch` bytes apart ----
  const int vec_per_row = p.ks / 16;
  for (int idx = threadIdx.x; idx < MPAD * vec_per_row; idx += kSThreads) {
    const int token = idx / vec_per_row, cv = idx - token * vec_per_row;
    uint8_t* dst = act + (size_t)token * p.pitch + cv * 16;
    if (token < p.M) {
      const int8_t* src = p.a + (int64_t)token * p.K + (int64_t)slice * p.ks + cv * 16;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                       (uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");

  // ---- this warp's contiguous range of chunks, strip-major inside the slice ----
  const int cps = p.ks / kSChunkK;
  const int chunks_per_strip = (int)(p.K / kSChunkK);
  const int total = (int)(p.N / kSStrip) * cps;
  const int nwarps = ctas_per_slice * kSWarps;
  const int wg = cta_in_slice * kSWarps + warp;
  const int c_begin = (int)((int64_t)total * wg / nwarps);
  const int c_end = (int)((int64_t)total * (wg + 1) / nwarps);

  // weight rows g and g + 8 of the strip: 16 bytes at k = 16 t + 64 j of the chunk, j = 0..3
  // (the four loads of a row are adjacent 64-byte pieces: 256 contiguous bytes per row visit)
  uint4 wlo[kSPrefetch][4], whi[kSPrefetch][4];
  int f_c = c_begin;
  int f_strip = c_begin / cps;
  int f_kc = c_begin - f_strip * cps;
  const int8_t* f_w = p.w + ((int64_t)f_strip * kSStrip + g) * p.K + (int64_t)slice * p.ks +
                      (int64_t)f_kc * kSChunkK + t * 16;
  const int64_t hi_off = 8 * p.K;
  auto fetch = [&](uint4 (&lo)[4], uint4 (&hi)[4]) {
    if (f_c < c_end) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo[j] = __ldg(reinterpret_cast<const uint4*>(f_w + 64 * j));
        hi[j] = __ldg(reinterpret_cast<const uint4*>(f_w + hi_off + 64 * j));
      }
      ++f_c;
      f_w += kSChunkK;
      if (++f_kc == cps) {
        f_kc = 0;
        ++f_strip;
        f_w += (int64_t)kSStrip * p.K - p.ks;
      }
    }
  };
#pragma unroll
  for (int u = 0; u < kSPrefetch; ++u) fetch(wlo[u], whi[u]);

  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // B fragments: token g of each tile, 16 bytes at k = 16 t of the chunk
  const uint8_t* act_lane = act + (size_t)g * p.pitch + t * 16;

  int acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0;

  int strip = c_begin / cps;
  int kc = c_begin - strip * cps;
  int contributed = 0;
  const bool reference = p.epilogue == QWX_EPI_REFERENCE;

  for (int base = c_begin; base < c_end; base += kSPrefetch) {
#pragma unroll
    for (int u = 0; u < kSPrefetch; ++u) {
      const int c = base + u;
      if (c >= c_end) break;
      const uint8_t* ab = act_lane + kc * kSChunkK;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 lo = wlo[u][j], hi = whi[u][j];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const uint4 b = *reinterpret_cast<const uint4*>(ab + (size_t)(n * 8) * p.pitch + 64 * j);
          mma_s8(acc[n], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
          mma_s8(acc[n], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
        }
      }
      fetch(wlo[u], whi[u]);   // chunk c + kSPrefetch, into the registers just consumed
      ++contributed;

      if (kc == cps - 1 || c == c_end - 1) {
        // ---- this warp is done with the strip ----
        const bool whole = contributed == chunks_per_strip;
        const int64_t ch = (int64_t)strip * kSStrip + g;
        bool fin = whole;
        if (!whole) {
#pragma unroll
          for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int tok = n * 8 + 2 * t + (j & 1);
              if (tok < p.M) atomicAdd(p.ws + (int64_t)tok * p.N + ch + (j >> 1) * 8, acc[n][j]);
            }
          __threadfence();
          __syncwarp();
          int last = 0;
          if (lane == 0) {
            const int old = atomicAdd(p.counters + strip, contributed);
            last = old + contributed == chunks_per_strip;
            if (last) p.counters[strip] = 0;
          }
          fin = __shfl_sync(0xffffffffu, last, 0) != 0;
          if (fin) {
            __threadfence();
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int tok = n * 8 + 2 * t + (j & 1);
                acc[n][j] = tok < p.M ? __ldcg(p.ws + (int64_t)tok * p.N + ch + (j >> 1) * 8) : 0;
              }
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int tok = n * 8 + 2 * t + (j & 1);
                if (tok < p.M) p.ws[(int64_t)tok * p.N + ch + (j >> 1) * 8] = 0;
              }
          }
        }
        if (fin) {
          const float sb_lo = p.sb ? load_scale_s(p.sb, p.scale_dtype, ch) : 1.0f;
          const float sb_hi = p.sb ? load_scale_s(p.sb, p.scale_dtype, ch + 8) : 1.0f;
#pragma unroll
          for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int tok = n * 8 + 2 * t + (j & 1);
              if (tok >= p.M) continue;
              const int64_t at = (int64_t)tok * p.N + ch + (j >> 1) * 8;
              if (p.out_dtype == QWX_S32) {
                reinterpret_cast<int32_t*>(p.out)[at] = acc[n][j];
                continue;
              }
              const float sa = p.sa ? load_scale_s(p.sa, p.scale_dtype, tok) : 1.0f;
              const float sb = (j >> 1) ? sb_hi : sb_lo;
              float v = (float)acc[n][j];
              if (reference) {
                v = round_out_s(v, p.out_dtype);
                v = round_out_s(__fmul_rn(v, sa), p.out_dtype);
                v = round_out_s(__fmul_rn(v, sb), p.out_dtype);
              } else {
                v = __fmul_rn(__fmul_rn(v, sa), sb);
              }
              if (p.out_dtype == QWX_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(v);
              else if (p.out_dtype == QWX_F16) reinterpret_cast<__half*>(p.out)[at] = __float2half_rn(v);
              else reinterpret_cast<float*>(p.out)[at] = v;
            }
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0;
        contributed = 0;
      }
      if (++kc == cps) { kc = 0; ++strip; }
    }
  }
}

int sm_count_s() {
  static int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return v;
  }();
  return n;
}

// Fewest K slices (a divisor of K / 64) whose activation slice fits shared memory.
int skinny_split(int mpad, int64_t K) {
  const int64_t blocks = K / kSChunkK;
  for (int64_t d = 1; d <= blocks; ++d) {
    if (blocks % d) continue;
    if ((size_t)mpad * ((size_t)(K / d) + 64) <= kSActCap) return (int)d;
  }
  return 0;
}

}  // namespace
}  // namespace qwx

using namespace qwx;

extern "C" {

size_t qwx_gemm_q8_skinny_workspace_bytes(int64_t M, int64_t N) {
  if (M <= 0 || N <= 0) return 0;
  return (size_t)(M * N * 4 + ((N + kSStrip - 1) / kSStrip) * 4);
}

int qwx_gemm_q8_skinny(const void* a, const void* w, int64_t M, int64_t N, int64_t K,
                       const void* sa, const void* sb, int scale_dtype, void* out, int out_dtype,
                       int epilogue, void* workspace, size_t workspace_bytes,
                       int workspace_is_zero, qwx_stream_t stream) {
  if (!a || !w || !out || !workspace) return QWX_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (M > 32 || K % kSChunkK || N % kSStrip) return QWX_ERR_UNSUPPORTED;
  if (out_dtype == QWX_S32) {
    if (sa || sb) return QWX_ERR_DTYPE;
  } else if (out_dtype != QWX_BF16 && out_dtype != QWX_F32 && out_dtype != QWX_F16) {
    return QWX_ERR_DTYPE;
  }
  if ((sa || sb) && scale_dtype != QWX_F32 && scale_dtype != QWX_BF16 && scale_dtype != QWX_F16)
    return QWX_ERR_DTYPE;
  if (epilogue != QWX_EPI_F32 && epilogue != QWX_EPI_REFERENCE) return QWX_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (reinterpret_cast<uintptr_t>(workspace) & 15))
    return QWX_ERR_ALIGN;
  if ((N / kSStrip) * (K / kSChunkK) > INT32_MAX / 2) return QWX_ERR_UNSUPPORTED;
  const size_t need = qwx_gemm_q8_skinny_workspace_bytes(M, N);
  if (workspace_bytes < need) return QWX_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (!workspace_is_zero && cudaMemsetAsync(workspace, 0, need, st) != cudaSuccess)
    return QWX_ERR_LAUNCH;

  static PerDeviceOnce configured;
  if (configured.first()) {
    const int cap = (int)kSActCap + 1024;
    if (cudaFuncSetAttribute(gemm_q8_skinny_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_q8_skinny_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_q8_skinny_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  const int sms = sm_count_s();
  if (sms <= 0) return QWX_ERR_NO_DEVICE;
  const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  const int split = skinny_split(nt * 8, K);
  if (split <= 0 || split > sms) return QWX_ERR_UNSUPPORTED;
  SkinnyParams p;
  p.a = (const int8_t*)a; p.w = (const int8_t*)w;
  p.sa = sa; p.sb = sb; p.scale_dtype = scale_dtype;
  p.M = (int)M; p.N = N; p.K = K;
  p.split = split; p.ks = (int)(K / split);
  // rows 64 bytes (mod 128) apart: the 16-byte reads of a quarter warp (two tokens x four K
  // offsets) then fall in different banks
  p.pitch = p.ks + (p.ks % 128 == 0 ? 64 : 0);
  p.out = out; p.out_dtype = out_dtype; p.epilogue = epilogue;
  p.ws = (int32_t*)workspace;
  p.counters = (int*)((char*)workspace + M * N * 4);
  const int grid = (sms / split) * split;
  const size_t smem = (size_t)nt * 8 * p.pitch;
  if (nt == 1) gemm_q8_skinny_kernel<1><<<grid, kSThreads, smem, st>>>(p);
  else if (nt == 2) gemm_q8_skinny_kernel<2><<<grid, kSThreads, smem, st>>>(p);
  else gemm_q8_skinny_kernel<4><<<grid, kSThreads, smem, st>>>(p);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

}  // extern "C"
