// Weight-only int4 GEMM for decode-shaped problems (few tokens, huge weight): the device
// side of dot_general._slow_dot_general (dot_general.py:264-275) for a bf16 activation and an
// int4 sub-channel-quantized weight,
//
//   out[m, n] = sum_k a[m, k] * W~[k, n],   W~[k, n] = q[k, n] * s[k / tile, n]
//
// without ever writing W~ to global memory.  The kernel is HBM-bound on the packed weight:
// K*N/2 bytes are streamed exactly once, every warp reading its own contiguous run.
//
// Design.  With 1..64 tokens the arithmetic is small; what decides the time is how little
// happens per weight byte besides the load.  A CTA-wide tcgen05 pipeline (operand tiles in
// shared memory, one MMA-issuing thread, mbarrier hand-overs per 8 KB of weights) was measured
// at 80-90 us for 8192 x 28672 whatever the payload: each hand-over costs about 200 cycles of
// a single thread and a 128 x 128 unit needs several.  Here nothing is handed over: every warp
// owns a contiguous range of (16-channel strip, 64-wide K chunk) work items (stream-K at warp
// granularity), loads its packed codes straight into registers (128-bit loads, eight in
// flight per lane), converts them in registers into the A fragments of warp-level
// mma.sync.m16n8k16 (channels are the MMA's M, tokens its N), and takes the B fragments with
// ldmatrix from the activation slice that the CTA keeps resident in shared memory.  The weight
// layout is made for this by qwx_pack_w4: a lane's 16 bytes hold exactly its fragment values
// for four consecutive K tiles, so a warp's load is one contiguous 512-byte line.
//
// The tensor cores multiply the activation with the integer codes themselves (exact in bf16);
// every 128 K the float32 partial sums are multiplied by the channel's scale and added to the
// running sums.  With float32 scales this is the reference's arithmetic up to the order of the
// float32 sums (its dequantized weight q * s is exact in float32); with bf16 scales the
// reference rounds q * s to bf16 first, which this kernel does not reproduce -- it is closer to
// the unquantized product, within the stated output tolerance.
//
// K is cut into `split` slices so that the activation slice (tokens x K / split, bf16) fits
// shared memory; CTA c works on slice c % split.  A strip whose chunks are spread over several
// warps (always the case when split > 1) is summed with float atomics in a caller-provided
// zeroed workspace; the warp that contributes last converts it and clears the workspace.
#include "common.cuh"
#include <algorithm>

namespace qwx {
namespace {

constexpr int kStrip = 16;          // channels per work item: the M of mma.m16n8k16
constexpr int kChunkK = 128;        // K per work item: eight K16 tiles, 2 x 16 bytes per lane, one scale
constexpr int kScaleK = 128;        // partial sums are scaled every 128 K
// Warps per CTA: 32 for up to 8 tokens (few registers per thread, and twice the warps hide the
// latency of the dependent MMAs of a chunk), 16 beyond.
__host__ __device__ constexpr int w4_warps(int nt) { return nt == 1 ? 32 : 16; }
constexpr size_t kSmemCap = 226 * 1024;
// Chunks (1 KB each) a warp keeps in flight in its private cp.async ring: loaded HBM latency is
// a few microseconds, so an SM needs on the order of 100 KB in flight to stream at its share
// of the bandwidth.  More tokens leave less room beside the activation slice.
__host__ __device__ constexpr int w4_depth(int nt) { return nt == 1 ? 4 : (nt == 2 ? 6 : 4); }
__host__ __device__ constexpr size_t w4_ring_bytes(int nt) { return (size_t)w4_warps(nt) * w4_depth(nt) * 1024; }

struct W4Params {
  const uint4* wp;        // packed chunks, [N / 16][K / 128][2][32 lanes] x 16 bytes
  const void* scale;      // [K / tile, N], f32 or bf16
  int scale_dtype;
  const __nv_bfloat16* a; // [M, K]
  int M;
  int64_t N, K;
  int tile;               // scale tile along K (multiple of 128)
  int split;              // K slices
  int ks;                 // K per slice
  int pitch;              // bytes between token rows of the shared activation slice
  void* out;
  int out_dtype;
  float* ws;              // [M, N] partial sums, zero on entry, left zero
  int* counters;          // [N / 16], zero on entry, left zero
};

template <int OFF>
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4 + %5];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr), "n"(OFF));
}
template <int OFF>
__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, uint32_t (&r)[2]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2 + %3];"
               : "=r"(r[0]), "=r"(r[1]) : "r"(addr), "n"(OFF));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Eight offset-binary nibbles (value + 8) of one lane and one K16 tile -> the four A-fragment
// registers.  Nibble j sits under nibble j + 4 of the same register: 0x4300 | u is the bf16
// number 128 + u, and subtracting 136 gives the signed code exactly.
__device__ __forceinline__ void unpack_fragment(uint32_t w, uint32_t (&a)[4]) {
  const __nv_bfloat162 bias = __floats2bfloat162_rn(136.f, 136.f);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t v = ((w >> (4 * j)) & 0x000f000fu) | 0x43004300u;
    __nv_bfloat162 h = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), bias);
    a[j] = *reinterpret_cast<uint32_t*>(&h);
  }
}

__device__ __forceinline__ float load_scale_w4(const void* p, int dtype, int64_t i) {
  if (dtype == QWX_F32) return __ldg(reinterpret_cast<const float*>(p) + i);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

template <int NT>   // token tiles of 8: the activation is padded to NT * 8 rows
__global__ void __launch_bounds__(w4_warps(NT) * 32, 1) gemm_w4_kernel(const W4Params p) {
  constexpr int kW4Warps = w4_warps(NT);
  constexpr int kW4Threads = kW4Warps * 32;
  extern __shared__ __align__(16) uint8_t act[];
  constexpr int MPAD = NT * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int slice = blockIdx.x % p.split;
  const int cta_in_slice = blockIdx.x / p.split;
  const int ctas_per_slice = gridDim.x / p.split;

  // ---- the CTA's activation slice: tokens x ks, rows `pitch` bytes apart (16 bytes of padding
  // keep the eight rows of an ldmatrix in different banks); rows beyond M are zero ----
  const int vec_per_row = p.ks / 8;
  for (int idx = threadIdx.x; idx < MPAD * vec_per_row; idx += kW4Threads) {
    const int token = idx / vec_per_row, cv = idx - token * vec_per_row;
    uint8_t* dst = act + (size_t)token * p.pitch + cv * 16;
    if (token < p.M) {
      const __nv_bfloat16* src = p.a + (int64_t)token * p.K + (int64_t)slice * p.ks + cv * 8;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                       (uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");

  // ---- this warp's contiguous range of chunks, strip-major inside the slice ----
  const int cps = p.ks / kChunkK;                       // chunks per strip in one slice
  const int chunks_per_strip = (int)(p.K / kChunkK);    // ... in all slices
  const int total = (int)(p.N / kStrip) * cps;          // the host checks that this fits
  const int nwarps = ctas_per_slice * kW4Warps;
  const int wg = cta_in_slice * kW4Warps + warp;
  const int c_begin = (int)((int64_t)total * wg / nwarps);
  const int c_end = (int)((int64_t)total * (wg + 1) / nwarps);

  // Fetch cursor: two 16-byte loads per chunk and lane, plus the scales of this lane's two
  // channels for the chunk's K tile.  The loads land in registers that are first read
  // kPrefetch chunks later.
  constexpr int D = w4_depth(NT);
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(act) + (uint32_t)(MPAD * p.pitch) +
                        (uint32_t)(warp * D * 1024 + lane * 16);   // this lane's 16 bytes of stage 0, half 0
  float slo[D], shi[D];
  int f_c = c_begin;
  int f_strip = c_begin / cps;
  int f_kc = c_begin - f_strip * cps;
  const uint4* f_w = p.wp + (((int64_t)f_strip * chunks_per_strip + slice * cps + f_kc) * 64 + lane);
  // scale cursor: element index of channel g of the strip in the scale row of the chunk's K tile
  const int blocks_per_scale = p.tile / kChunkK;
  int f_left = blocks_per_scale - (slice * cps + f_kc) % blocks_per_scale;   // chunks left in the row
  int64_t f_s = (int64_t)((slice * cps + f_kc) / blocks_per_scale) * p.N + f_strip * kStrip + g;
  auto fetch = [&](int stage, float& lo, float& hi) {
    if (f_c < c_end) {
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring + stage * 1024), "l"(f_w) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring + stage * 1024 + 512), "l"(f_w + 32) : "memory");
      lo = load_scale_w4(p.scale, p.scale_dtype, f_s);
      hi = load_scale_w4(p.scale, p.scale_dtype, f_s + 8);
      ++f_c;
      f_w += 64;
      if (--f_left == 0) { f_left = blocks_per_scale; f_s += p.N; }
      if (++f_kc == cps) {
        f_kc = 0;
        ++f_strip;
        f_w += (int64_t)(chunks_per_strip - cps) * 64;
        f_left = blocks_per_scale - (slice * cps) % blocks_per_scale;
        f_s = (int64_t)((slice * cps) / blocks_per_scale) * p.N + f_strip * kStrip + g;
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // the activation slice is the oldest commit group: waiting until at most D groups pend
  // completes it
#pragma unroll
  for (int u = 0; u < D; ++u) fetch(u, slo[u], shi[u]);
  asm volatile("cp.async.wait_group %0;" ::"n"(D) : "memory");
  __syncthreads();

  // per-lane byte offset of its ldmatrix row: matrices 0..3 = (tokens 0-7, k 0-7), (tokens 0-7,
  // k 8-15), (tokens 8-15, k 0-7), (tokens 8-15, k 8-15)
  const int lm = lane >> 3, lr = lane & 7;
  const uint32_t act_lane = (uint32_t)__cvta_generic_to_shared(act) +
                            (uint32_t)(((lm >> 1) * 8 + lr) * p.pitch + (lm & 1) * 16);

  float acc[NT][4], run[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[n][j] = run[n][j] = 0.f;

  int strip = c_begin / cps;
  int kc = c_begin - strip * cps;
  int contributed = 0;

  for (int base = c_begin; base < c_end; base += D) {
#pragma unroll
    for (int u = 0; u < D; ++u) {
      const int c = base + u;
      if (c >= c_end) break;
      const float s_lo = slo[u], s_hi = shi[u];
      asm volatile("cp.async.wait_group %0;" ::"n"(D - 1) : "memory");
      uint4 wq[2];
      asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(wq[0].x), "=r"(wq[0].y), "=r"(wq[0].z), "=r"(wq[0].w) : "r"(ring + u * 1024) : "memory");
      asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(wq[1].x), "=r"(wq[1].y), "=r"(wq[1].z), "=r"(wq[1].w) : "r"(ring + u * 1024 + 512) : "memory");
      fetch(u, slo[u], shi[u]);   // chunk c + D, into the ring stage just read
      const uint32_t kaddr = act_lane + (uint32_t)(kc * kChunkK) * 2u;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4& q4 = wq[i >> 2];
        const uint32_t word = (i & 3) == 0 ? q4.x : ((i & 3) == 1 ? q4.y : ((i & 3) == 2 ? q4.z : q4.w));
        uint32_t a[4];
        unpack_fragment(word, a);
        if constexpr (NT == 1) {
          uint32_t b[2];
          if (i == 0) ldmatrix_x2<0>(kaddr, b);
          else if (i == 1) ldmatrix_x2<32>(kaddr, b);
          else if (i == 2) ldmatrix_x2<64>(kaddr, b);
          else if (i == 3) ldmatrix_x2<96>(kaddr, b);
          else if (i == 4) ldmatrix_x2<128>(kaddr, b);
          else if (i == 5) ldmatrix_x2<160>(kaddr, b);
          else if (i == 6) ldmatrix_x2<192>(kaddr, b);
          else ldmatrix_x2<224>(kaddr, b);
          mma_bf16(acc[0], a, b[0], b[1]);
        } else {
#pragma unroll
          for (int pr = 0; pr < NT / 2; ++pr) {
            uint32_t b[4];
            const uint32_t ka = kaddr + (uint32_t)(pr * 16 * p.pitch);
            if (i == 0) ldmatrix_x4<0>(ka, b);
            else if (i == 1) ldmatrix_x4<32>(ka, b);
            else if (i == 2) ldmatrix_x4<64>(ka, b);
            else if (i == 3) ldmatrix_x4<96>(ka, b);
            else if (i == 4) ldmatrix_x4<128>(ka, b);
            else if (i == 5) ldmatrix_x4<160>(ka, b);
            else if (i == 6) ldmatrix_x4<192>(ka, b);
            else ldmatrix_x4<224>(ka, b);
            mma_bf16(acc[2 * pr], a, b[0], b[1]);
            mma_bf16(acc[2 * pr + 1], a, b[2], b[3]);
          }
        }
      }
      ++contributed;

      // the chunk is one scale block: scale its partial sums into the running sums
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        run[n][0] = __fmaf_rn(acc[n][0], s_lo, run[n][0]);
        run[n][1] = __fmaf_rn(acc[n][1], s_lo, run[n][1]);
        run[n][2] = __fmaf_rn(acc[n][2], s_hi, run[n][2]);
        run[n][3] = __fmaf_rn(acc[n][3], s_hi, run[n][3]);
        acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      }
      const bool range_end = c == c_end - 1;
      if (kc == cps - 1 || range_end) {
        // ---- this warp is done with the strip ----
        const bool whole = contributed == chunks_per_strip;
        const int64_t ch = (int64_t)strip * kStrip + g;
        bool fin = whole;
        if (!whole) {
#pragma unroll
          for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int tok = n * 8 + 2 * t + (j & 1);
              if (tok < p.M) atomicAdd(p.ws + (int64_t)tok * p.N + ch + (j >> 1) * 8, run[n][j]);
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
            // whoever completes the strip converts it and leaves the workspace zero
            __threadfence();
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int tok = n * 8 + 2 * t + (j & 1);
                float* w = p.ws + (int64_t)tok * p.N + ch + (j >> 1) * 8;
                run[n][j] = tok < p.M ? __ldcg(w) : 0.f;
              }
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int tok = n * 8 + 2 * t + (j & 1);
                if (tok < p.M) p.ws[(int64_t)tok * p.N + ch + (j >> 1) * 8] = 0.f;
              }
          }
        }
        if (fin) {
#pragma unroll
          for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int tok = n * 8 + 2 * t + (j & 1);
              if (tok >= p.M) continue;
              const int64_t at = (int64_t)tok * p.N + ch + (j >> 1) * 8;
              if (p.out_dtype == QWX_BF16)
                reinterpret_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(run[n][j]);
              else
                reinterpret_cast<float*>(p.out)[at] = run[n][j];
            }
        }
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int j = 0; j < 4; ++j) run[n][j] = 0.f;
        contributed = 0;
      }
      if (++kc == cps) { kc = 0; ++strip; }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Logical codes q[K, N] (one sign-extended int4 per byte) -> fragment-ordered chunks.  A chunk
// is two 512-byte halves; word i (0..3) of lane (g, t) in half h covers K tile 4 h + i of the
// chunk; its nibble j holds channel strip * 16 + g + 8 * (j & 1) at
// k = 2 t + 8 * ((j >> 1) & 1) + (j >> 2) of the tile.
__global__ void pack_w4_kernel(const int8_t* __restrict__ q, int64_t K, int64_t N,
                               uint32_t* __restrict__ out, int64_t total_words) {
  const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= total_words) return;
  const int i = (int)(w & 3);
  const int lane = (int)((w >> 2) & 31);
  const int half = (int)((w >> 7) & 1);
  const int64_t chunk = w >> 8;                 // strip * (K / 128) + kc
  const int64_t cpsa = K / kChunkK;
  const int64_t strip = chunk / cpsa, kc = chunk % cpsa;
  const int g = lane >> 2, t = lane & 3;
  uint32_t word = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int64_t ch = strip * kStrip + g + 8 * (j & 1);
    const int64_t k = kc * kChunkK + (half * 4 + i) * 16 + 2 * t + 8 * ((j >> 1) & 1) + (j >> 2);
    const int v = (ch < N && k < K) ? (int)q[k * N + ch] : 0;
    word |= (uint32_t)((v + 8) & 0xf) << (4 * j);
  }
  out[w] = word;
}

int sm_count_w4() {
  static int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return v;
  }();
  return n;
}

// Fewest K slices (a divisor of K / 128) whose activation slice fits shared memory.
int w4_split(int mpad, int64_t K, size_t cap) {
  const int64_t blocks = K / kScaleK;
  for (int64_t d = 1; d <= blocks; ++d) {
    if (blocks % d) continue;
    if ((size_t)mpad * ((size_t)(K / d) * 2 + 16) <= cap) return (int)d;
  }
  return 0;
}

constexpr int kMaxTokensPerLaunch = 32;

}  // namespace
}  // namespace qwx

using namespace qwx;

extern "C" {

size_t qwx_w4_packed_bytes(int64_t K, int64_t N) {
  if (K <= 0 || N <= 0 || K % kScaleK) return 0;
  const int64_t strips = (N + kStrip - 1) / kStrip;
  return (size_t)(strips * (K / kChunkK) * 1024);
}

int qwx_pack_w4(const void* q, int64_t K, int64_t N, void* packed, qwx_stream_t stream) {
  if (!q || !packed) return QWX_ERR_NULL;
  if (K <= 0 || N <= 0 || K % kScaleK) return QWX_ERR_SHAPE;
  const int64_t strips = (N + kStrip - 1) / kStrip;
  const int64_t words = strips * (K / kChunkK) * 256;
  pack_w4_kernel<<<(unsigned)((words + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const int8_t*)q, K, N, (uint32_t*)packed, words);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

size_t qwx_gemm_a16w4_workspace_bytes(int64_t M, int64_t N) {
  if (M <= 0 || N <= 0) return 0;
  const int64_t strips = (N + kStrip - 1) / kStrip;
  return (size_t)(M * N * 4 + strips * 4);
}

int qwx_gemm_a16w4(const void* a, const void* w_packed, const void* scale, int scale_dtype,
                   int64_t M, int64_t N, int64_t K, int64_t k_tile, void* out, int out_dtype,
                   void* workspace, size_t workspace_bytes, int workspace_is_zero,
                   int32_t* error_flag, qwx_stream_t stream) {
  (void)error_flag;   // no device-side waits in this kernel
  if (!a || !w_packed || !scale || !out || !workspace) return QWX_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (M > 128) return QWX_ERR_UNSUPPORTED;            // larger batches: call per 128 rows
  if (K % kScaleK || N % kStrip) return QWX_ERR_UNSUPPORTED;
  if (k_tile <= 0 || K % k_tile || k_tile % kScaleK) return QWX_ERR_UNSUPPORTED;
  if (scale_dtype != QWX_F32 && scale_dtype != QWX_BF16) return QWX_ERR_DTYPE;
  if (out_dtype != QWX_BF16 && out_dtype != QWX_F32) return QWX_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w_packed) & 15) ||
      (reinterpret_cast<uintptr_t>(scale) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 15))
    return QWX_ERR_ALIGN;
  if (workspace_bytes < qwx_gemm_a16w4_workspace_bytes(M, N)) return QWX_ERR_WORKSPACE;
  if ((N / kStrip) * (K / kChunkK) > INT32_MAX / 2) return QWX_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  if (!workspace_is_zero &&
      cudaMemsetAsync(workspace, 0, qwx_gemm_a16w4_workspace_bytes(M, N), st) != cudaSuccess)
    return QWX_ERR_LAUNCH;

  static PerDeviceOnce configured;
  if (configured.first()) {
    const int cap = (int)kSmemCap;
    if (cudaFuncSetAttribute(gemm_w4_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_w4_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_w4_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  const int sms = sm_count_w4();
  if (sms <= 0) return QWX_ERR_NO_DEVICE;
  const int out_elem = out_dtype == QWX_BF16 ? 2 : 4;

  // The warp-level MMA holds up to 32 tokens: more tokens stream the weight once per 32.
  for (int64_t m0 = 0; m0 < M; m0 += kMaxTokensPerLaunch) {
    const int rows = (int)(M - m0 < kMaxTokensPerLaunch ? M - m0 : kMaxTokensPerLaunch);
    const int nt = rows <= 8 ? 1 : (rows <= 16 ? 2 : 4);
    const int split = w4_split(nt * 8, K, kSmemCap - w4_ring_bytes(nt));
    if (split <= 0 || split > sms) return QWX_ERR_UNSUPPORTED;
    W4Params p;
    p.wp = (const uint4*)w_packed;
    p.scale = scale; p.scale_dtype = scale_dtype;
    p.a = (const __nv_bfloat16*)a + m0 * K;
    p.M = rows; p.N = N; p.K = K; p.tile = (int)k_tile;
    p.split = split;
    p.ks = (int)(K / split);
    p.pitch = p.ks * 2 + 16;
    p.out = (char*)out + m0 * N * out_elem; p.out_dtype = out_dtype;
    p.ws = (float*)workspace + m0 * N;
    p.counters = (int*)((char*)workspace + M * N * 4);
    const int grid = (sms / split) * split;
    const size_t smem = (size_t)nt * 8 * p.pitch + w4_ring_bytes(nt);
    if (nt == 1) gemm_w4_kernel<1><<<grid, w4_warps(1) * 32, smem, st>>>(p);
    else if (nt == 2) gemm_w4_kernel<2><<<grid, w4_warps(2) * 32, smem, st>>>(p);
    else gemm_w4_kernel<4><<<grid, w4_warps(4) * 32, smem, st>>>(p);
    QWX_CHECK_LAUNCH();
  }
  return QWX_OK;
}

}  // extern "C"
