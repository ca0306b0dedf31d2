// Element-wise stages of a decoder layer fused with the per-token int8 quantization that
// feeds the next quantized projection.  The quantization half is qarray.quantize with
// per-token absmax scales (qwix/_src/core/qarray.py:638-644, the activation side of
// qwix/_src/providers/boxed_param.py:416-455); the element-wise halves are model code that
// lives outside qwix (RMSNorm, SwiGLU, rotary embedding of a Llama-style decoder) and are
// fused here only because every one of them is a full HBM pass over the activations:
//
//   add_rmsnorm      x' = bf16(x + delta);  y = bf16( (f32(x') * rsqrt(mean(x'^2) + eps)) * f32(w) )
//   silu_mul         y = bf16( bf16(silu(g)) * u ),  silu(g) = g / (1 + exp(-g)) in float32
//                    (fast exp and division: differs from libm in about 1 value in 10^4)
//   rope_cache       q, k rotated (x1 cos - x2 sin | x2 cos + x1 sin, float32, separate
//                    roundings), q written token-major, k and v written into the KV cache
//
// each followed, when asked, by scale = bf16(absmax(y) / 127.5) (1 if below 2^-63),
// code = sat_int8(round_half_even(bf16(y / scale))) per row -- the strict recipe of
// quantize.cu.  Every rounding of the unfused PyTorch composition is kept, so results differ
// from it only through the order of the float32 sum of squares.
#include <mutex>

#include "common.cuh"

namespace qwx {
namespace {

constexpr int kDThreads = 256;
constexpr int kDVec = 4;   // 16-byte vectors per thread for register-resident rows (d <= 8192)

__device__ __forceinline__ float block_sum(float v, float* red, int tid) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((tid & 31) == 0) red[tid >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kDThreads / 32; ++i) t += red[i];
  __syncthreads();
  return t;
}

__device__ __forceinline__ uint32_t block_max_bits(uint32_t v, uint32_t* red, int tid) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((tid & 31) == 0) red[tid >> 5] = v;
  __syncthreads();
  uint32_t t = 0;
#pragma unroll
  for (int i = 0; i < kDThreads / 32; ++i) t = max(t, red[i]);
  __syncthreads();
  return t;
}

// |a|, |b| of a packed bf16 pair as comparable bit patterns (NaN sorts last)
__device__ __forceinline__ uint32_t abs_bits2(uint32_t w) {
  return max((w << 16) & 0x7fffffffu, w & 0x7fff0000u);
}

struct RowQuantizer {
  float s;
  bool fast;
  __nv_bfloat162 r2, ns2;
  __device__ __forceinline__ explicit RowQuantizer(uint32_t absmax_bits) {
    const float absmax = __uint_as_float(absmax_bits);
    s = round_to<BF16>(__fdiv_rn(absmax, 127.5f));
    if (s < 0x1p-63f) s = 1.0f;
    const float as = fabsf(s);
    fast = as > 0x1p-100f && as < 0x1p100f && absmax_bits < 0x7f800000u;
    const __nv_bfloat16 sb = __float2bfloat16_rn(s);
    const __nv_bfloat16 rb = __float2bfloat16_rn(__frcp_rn(s));
    r2 = __halves2bfloat162(rb, rb);
    ns2 = __hneg2(__halves2bfloat162(sb, sb));
  }
  // eight bf16 values (four packed words) -> eight int8 codes
  __device__ __forceinline__ uint2 codes(const uint32_t (&w)[4]) const {
    uint32_t packed[2];
    if (fast) {
      // Correctly rounded bf16 quotients from three packed bf16 FMAs (Markstein's division,
      // checked exhaustively over bf16 significands), then round-half-even and saturate.
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
    } else {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t word = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t pair = w[2 * half + (e >> 1)];
          const float xv = __uint_as_float((e & 1) ? (pair & 0xffff0000u) : (pair << 16));
          const float y = round_to<BF16>(__fdiv_rn(xv, s));
          word |= (uint32_t)(to_code<S8>(y) & 0xff) << (8 * e);
        }
        packed[half] = word;
      }
    }
    return make_uint2(packed[0], packed[1]);
  }
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// One CTA per row, rows of up to kDThreads * kDVec * 8 values held in registers.
__global__ void __launch_bounds__(kDThreads)
add_rmsnorm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ delta,
                   const uint4* __restrict__ weight, float eps, int64_t rows, int nvec,
                   uint4* __restrict__ x_out, uint4* __restrict__ y_out, uint2* __restrict__ q,
                   __nv_bfloat16* __restrict__ scale) {
  __shared__ float red_f[kDThreads / 32];
  __shared__ uint32_t red_u[kDThreads / 32];
  const int tid = threadIdx.x;
  const float inv_d = 1.0f / (float)(nvec * 8);
  griddep_launch_dependents();
  griddep_wait();
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    uint4 cur[kDVec];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < kDVec; ++it) {
      const int vi = tid + it * kDThreads;
      if (vi >= nvec) continue;
      uint4 u = x[row * nvec + vi];
      if (delta) {
        // the residual stream is a bf16 tensor: x' = bf16(x + delta)
        const uint4 dl = delta[row * nvec + vi];
        float a[8], b[8];
        unpack_bf16x8(u, a);
        unpack_bf16x8(dl, b);
        u = make_uint4(pack_bf16(a[0] + b[0], a[1] + b[1]), pack_bf16(a[2] + b[2], a[3] + b[3]),
                       pack_bf16(a[4] + b[4], a[5] + b[5]), pack_bf16(a[6] + b[6], a[7] + b[7]));
        if (x_out) x_out[row * nvec + vi] = u;
      }
      cur[it] = u;
      float v[8];
      unpack_bf16x8(u, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = __fmaf_rn(v[j], v[j], ss);
    }
    ss = block_sum(ss, red_f, tid);
    const float rs = rsqrtf(__fadd_rn(__fmul_rn(ss, inv_d), eps));

    uint32_t bits = 0;
#pragma unroll
    for (int it = 0; it < kDVec; ++it) {
      const int vi = tid + it * kDThreads;
      if (vi >= nvec) continue;
      float v[8], w[8];
      unpack_bf16x8(cur[it], v);
      unpack_bf16x8(__ldg(weight + vi), w);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[j] = pack_bf16(__fmul_rn(__fmul_rn(v[2 * j], rs), w[2 * j]),
                         __fmul_rn(__fmul_rn(v[2 * j + 1], rs), w[2 * j + 1]));
        bits = max(bits, abs_bits2(o[j]));
      }
      cur[it] = make_uint4(o[0], o[1], o[2], o[3]);
      if (y_out) y_out[row * nvec + vi] = cur[it];
    }
    if (q == nullptr) continue;
    bits = block_max_bits(bits, red_u, tid);
    const RowQuantizer rq(bits);
    if (tid == 0) scale[row] = __float2bfloat16_rn(rq.s);
#pragma unroll
    for (int it = 0; it < kDVec; ++it) {
      const int vi = tid + it * kDThreads;
      if (vi >= nvec) continue;
      const uint32_t w[4] = {cur[it].x, cur[it].y, cur[it].z, cur[it].w};
      q[row * nvec + vi] = rq.codes(w);
    }
  }
}

// ---- the same stage fused with the all-reduce of a row-parallel projection ---------------------
//
// Under tensor parallelism the `delta` of add_rmsnorm is the sum over ranks of the partial
// outputs of a row-parallel GEMM.  Every rank leaves its partial (bf16) in a buffer that the
// other ranks have mapped (symmetric memory over NVLink); this kernel reads all of them with
// plain peer loads, adds them in rank order in float32, rounds the sum to bf16 (the value an
// all-reduce would have delivered) and goes on as add_rmsnorm does: no separate collective, no
// reduced tensor written and read back.
//
// Hand-shake, per CTA and bounded: CTA b of every rank raises flag [b][rank] in every peer's
// flag array to its own launch count (release, system scope) and waits until the flags of its
// peers reach that count.  A rank's CTA b runs only after that rank's GEMM has finished (stream
// order), so a raised flag means "my partial is complete".  Callers alternate two partial
// buffers: a buffer is rewritten only after a later hand-shake that every reader has passed.
constexpr int kMaxPeers = 8;
constexpr long long kPeerWaitCycles = 4000000000ll;

struct PeerArgs {
  const uint4* partial[kMaxPeers];   // every rank's partial buffer, as mapped here
  int* flags[kMaxPeers];             // every rank's flag array [ctas][world]
  int* launches;                     // this rank: [ctas] launch counts
  int world, rank;
  int32_t* error_flag;
  long long wait_cycles;             // budget of the hand-shake, SM clocks
};

__global__ void __launch_bounds__(kDThreads)
add_rmsnorm_peer_kernel(const uint4* __restrict__ x, const PeerArgs pa,
                        const uint4* __restrict__ weight, float eps, int64_t rows, int nvec,
                        uint4* __restrict__ x_out, uint4* __restrict__ y_out, uint2* __restrict__ q,
                        __nv_bfloat16* __restrict__ scale) {
  __shared__ float red_f[kDThreads / 32];
  __shared__ uint32_t red_u[kDThreads / 32];
  __shared__ int s_count, s_ok;
  const int tid = threadIdx.x;
  griddep_launch_dependents();
  griddep_wait();       // this rank's GEMM has finished: its partial is complete
  if (tid == 0) {
    s_count = ++pa.launches[blockIdx.x];
    s_ok = 1;
  }
  __syncthreads();
  const int count = s_count;
  if (tid < pa.world && tid != pa.rank) {
    __threadfence_system();
    int* theirs = pa.flags[tid] + (size_t)blockIdx.x * pa.world + pa.rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(count) : "memory");
    const int* mine = pa.flags[pa.rank] + (size_t)blockIdx.x * pa.world + tid;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (v >= count) break;
      if ((it & 255u) == 0 && clock64() - t0 > pa.wait_cycles) {
        s_ok = 0;
        if (pa.error_flag) atomicExch(pa.error_flag, QWX_ERR_DEVICE_WAIT);
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;   // a peer never arrived: reported, nothing is read

  const float inv_d = 1.0f / (float)(nvec * 8);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    uint4 cur[kDVec];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < kDVec; ++it) {
      const int vi = tid + it * kDThreads;
      if (vi >= nvec) continue;
      // sum of the ranks' partials in rank order, float32, rounded once to bf16; all ranks'
      // loads are issued before the first sum (a peer load takes microseconds)
      uint4 got[kMaxPeers];
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < pa.world) got[r] = __ldcg(pa.partial[r] + row * nvec + vi);
      float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < pa.world) {
          float b[8];
          unpack_bf16x8(got[r], b);
#pragma unroll
          for (int j = 0; j < 8; ++j) d[j] = __fadd_rn(d[j], b[j]);
        }
      }
      float a[8];
      unpack_bf16x8(x[row * nvec + vi], a);
#pragma unroll
      for (int j = 0; j < 8; ++j) d[j] = round_to<BF16>(d[j]);
      const uint4 u = make_uint4(pack_bf16(a[0] + d[0], a[1] + d[1]), pack_bf16(a[2] + d[2], a[3] + d[3]),
                                 pack_bf16(a[4] + d[4], a[5] + d[5]), pack_bf16(a[6] + d[6], a[7] + d[7]));
      x_out[row * nvec + vi] = u;
      cur[it] = u;
      float v[8];
      unpack_bf16x8(u, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = __fmaf_rn(v[j], v[j], ss);
    }
    ss = block_sum(ss, red_f, tid);
    const float rs = rsqrtf(__fadd_rn(__fmul_rn(ss, inv_d), eps));

    uint32_t bits = 0;
#pragma unroll
    for (int it = 0; it < kDVec; ++it) {
      const int vi = tid + it * kDThreads;
      if (vi >= nvec) continue;
      float v[8], w[8];
      unpack_bf16x8(cur[it], v);
      unpack_bf16x8(__ldg(weight + vi), w);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[j] = pack_bf16(__fmul_rn(__fmul_rn(v[2 * j], rs), w[2 * j]),
                         __fmul_rn(__fmul_rn(v[2 * j + 1], rs), w[2 * j + 1]));
        bits = max(bits, abs_bits2(o[j]));
      }
      cur[it] = make_uint4(o[0], o[1], o[2], o[3]);
      if (y_out) y_out[row * nvec + vi] = cur[it];
    }
    if (q == nullptr) continue;
    bits = block_max_bits(bits, red_u, tid);
    const RowQuantizer rq(bits);
    if (tid == 0) scale[row] = __float2bfloat16_rn(rq.s);
#pragma unroll
    for (int it = 0; it < kDVec; ++it) {
      const int vi = tid + it * kDThreads;
      if (vi >= nvec) continue;
      const uint32_t w[4] = {cur[it].x, cur[it].y, cur[it].z, cur[it].w};
      q[row * nvec + vi] = rq.codes(w);
    }
  }
}

// ---- all-reduce of the partials in place, for many rows -------------------------------------
//
// The kernel above lets every rank read every partial: (world - 1) x the tensor crosses NVLink
// into each GPU, which is the right trade for the 256 KB of a decode step but not for a prefill
// chunk of 64 MB.  Here rank r sums only its share of the rows (reading world - 1 remote
// slices), rounds once to bf16 and writes the sums back into the same rows of EVERY rank's
// buffer (plain peer stores): (world - 1) / world of the tensor in and the same out, both
// directions of the links busy at once, and afterwards each rank holds the reduced tensor in
// its own memory for an ordinary local consumer.  In place is safe: a thread reads all ranks'
// copies of a vector before it overwrites them, and no other rank touches those rows.
//
// Two hand-shakes, both bounded: per CTA before the first read (every rank's GEMM has
// finished, as above), and per rank at the end -- the CTA that finishes last tells every peer
// "my sums are in your buffer" and does not leave before all peers have said the same, so the
// end of the kernel on a rank means its buffer is complete.
struct PeerReduceArgs {
  uint4* partial[kMaxPeers];   // every rank's buffer, as mapped here
  int* flags[kMaxPeers];       // every rank's flags: [ctas][world] ready marks, then [world] done marks
  int* launches;               // this rank: [ctas] launch counts, a finished-CTA counter, a call count
  int world, rank, max_ctas;
  int32_t* error_flag;
  long long wait_cycles;
};

__device__ __forceinline__ bool wait_flag(const int* flag, int count, long long budget) {
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= count) return true;
    if ((it & 255u) == 0 && clock64() - t0 > budget) return false;
  }
}

__global__ void __launch_bounds__(kDThreads)
peer_allreduce_kernel(const PeerReduceArgs pa, int64_t rows, int nvec) {
  __shared__ int s_count, s_ok, s_last;
  const int tid = threadIdx.x;
  griddep_launch_dependents();
  griddep_wait();       // this rank's GEMM has finished: its partial is complete
  if (tid == 0) {
    s_count = ++pa.launches[blockIdx.x];
    s_ok = 1;
  }
  __syncthreads();
  const int count = s_count;
  if (tid < pa.world && tid != pa.rank) {
    __threadfence_system();
    int* theirs = pa.flags[tid] + (size_t)blockIdx.x * pa.world + pa.rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(count) : "memory");
    if (!wait_flag(pa.flags[pa.rank] + (size_t)blockIdx.x * pa.world + tid, count, pa.wait_cycles)) {
      s_ok = 0;
      if (pa.error_flag) atomicExch(pa.error_flag, QWX_ERR_DEVICE_WAIT);
    }
  }
  __syncthreads();
  if (s_ok) {
    const int64_t row0 = rows * pa.rank / pa.world, row1 = rows * (pa.rank + 1) / pa.world;
    const int64_t vec0 = row0 * nvec, vec1 = row1 * nvec;
    // two vectors per thread and step, all ranks' loads issued before the first sum: a peer
    // load takes microseconds, so the bytes in flight decide the rate
    const int64_t stride = (int64_t)gridDim.x * kDThreads;
    for (int64_t v = vec0 + (int64_t)blockIdx.x * kDThreads + tid; v < vec1; v += 2 * stride) {
      const int64_t v2 = v + stride;
      const bool two = v2 < vec1;
      uint4 got[2][kMaxPeers];
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < pa.world) {
          got[0][r] = __ldcg(pa.partial[r] + v);
          if (two) got[1][r] = __ldcg(pa.partial[r] + v2);
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (h == 1 && !two) break;
        float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r) {          // rank order, float32, one rounding
          if (r < pa.world) {
            float b[8];
            unpack_bf16x8(got[h][r], b);
#pragma unroll
            for (int j = 0; j < 8; ++j) d[j] = __fadd_rn(d[j], b[j]);
          }
        }
        const uint4 u = make_uint4(pack_bf16(d[0], d[1]), pack_bf16(d[2], d[3]), pack_bf16(d[4], d[5]),
                                   pack_bf16(d[6], d[7]));
        const int64_t at = h ? v2 : v;
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
          if (r < pa.world) pa.partial[r][at] = u;
      }
    }
  }
  // the rank's last CTA exchanges "done" marks with the peers
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    int* finished = pa.launches + pa.max_ctas;
    s_last = atomicAdd(finished, 1) == (int)gridDim.x - 1;
    if (s_last) *finished = 0;
  }
  __syncthreads();
  if (!s_last) return;
  // the done marks carry the number of this call (every rank makes the same sequence of calls)
  if (tid == 0) s_count = ++pa.launches[pa.max_ctas + 1];
  __syncthreads();
  const int call = s_count;
  if (tid < pa.world && tid != pa.rank) {
    __threadfence_system();
    int* done_there = pa.flags[tid] + (size_t)pa.max_ctas * pa.world + pa.rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(done_there), "r"(call) : "memory");
    if (!wait_flag(pa.flags[pa.rank] + (size_t)pa.max_ctas * pa.world + tid, call, pa.wait_cycles)) {
      if (pa.error_flag) atomicExch(pa.error_flag, QWX_ERR_DEVICE_WAIT);
    }
  }
}

// One CTA per row of [gate | up]; the product row is staged in shared memory (f * 2 bytes)
// between the absmax pass and the quantizing pass.
__global__ void __launch_bounds__(kDThreads)
silu_mul_kernel(const uint4* __restrict__ gu, int64_t rows, int fvec, uint4* __restrict__ y_out,
                uint2* __restrict__ q, __nv_bfloat16* __restrict__ scale) {
  extern __shared__ uint4 yrow[];
  __shared__ uint32_t red_u[kDThreads / 32];
  const int tid = threadIdx.x;
  griddep_launch_dependents();
  griddep_wait();
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* g = gu + row * 2 * fvec;
    const uint4* u = g + fvec;
    uint32_t bits = 0;
    for (int vi = tid; vi < fvec; vi += kDThreads) {
      float a[8], b[8];
      unpack_bf16x8(g[vi], a);
      unpack_bf16x8(u[vi], b);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // exp and the quotient with the fast float32 forms (2 ulp each): the bf16 rounding
        // that follows hides them except in about one value in 10^4
        float s0 = __fdividef(a[2 * j], 1.0f + __expf(-a[2 * j]));
        float s1 = __fdividef(a[2 * j + 1], 1.0f + __expf(-a[2 * j + 1]));
        s0 = round_to<BF16>(s0);     // F.silu returns a bf16 tensor
        s1 = round_to<BF16>(s1);
        o[j] = pack_bf16(__fmul_rn(s0, b[2 * j]), __fmul_rn(s1, b[2 * j + 1]));
        bits = max(bits, abs_bits2(o[j]));
      }
      const uint4 out = make_uint4(o[0], o[1], o[2], o[3]);
      if (y_out) y_out[row * fvec + vi] = out;
      if (q) yrow[vi] = out;
    }
    if (q == nullptr) continue;
    bits = block_max_bits(bits, red_u, tid);   // also orders the shared-memory row
    const RowQuantizer rq(bits);
    if (tid == 0) scale[row] = __float2bfloat16_rn(rq.s);
    for (int vi = tid; vi < fvec; vi += kDThreads) {
      const uint4 v = yrow[vi];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      q[row * fvec + vi] = rq.codes(w);
    }
    __syncthreads();   // the row buffer is reused by the next row
  }
}

// One thread per (batch, token, head, 8 of the head's first-half values): rotates q and k
// heads, copies v heads.  qkv: [B, T, (hq + 2 hkv) * hd]; q_out: [B, T, hq, hd];
// cache_k / cache_v: [B, hkv, S, hd] views given by their batch and head strides (elements).
__global__ void rope_cache_kernel(const __nv_bfloat16* __restrict__ qkv, int64_t B, int64_t T,
                                  int hq, int hkv, int hd, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, int64_t pos,
                                  const int64_t* __restrict__ pos_dev,
                                  __nv_bfloat16* __restrict__ q_out,
                                  __nv_bfloat16* __restrict__ cache_k,
                                  __nv_bfloat16* __restrict__ cache_v, int64_t cache_bs,
                                  int64_t cache_hs) {
  const int half = hd / 2, per_head = half / 8;
  const int heads = hq + 2 * hkv;
  const int64_t total = B * T * heads * per_head;
  griddep_launch_dependents();
  griddep_wait();
  const int64_t p0 = pos_dev ? *pos_dev : pos;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % per_head);
    const int h = (int)((i / per_head) % heads);
    const int64_t t = (i / ((int64_t)per_head * heads)) % T;
    const int64_t b = i / ((int64_t)per_head * heads * T);
    const __nv_bfloat16* src = qkv + ((b * T + t) * heads + h) * hd + c * 8;
    const uint4 u1 = *reinterpret_cast<const uint4*>(src);
    const uint4 u2 = *reinterpret_cast<const uint4*>(src + half);
    __nv_bfloat16* dst;
    if (h < hq) dst = q_out + ((b * T + t) * hq + h) * hd + c * 8;
    else if (h < hq + hkv) dst = cache_k + b * cache_bs + (h - hq) * cache_hs + (p0 + t) * hd + c * 8;
    else dst = cache_v + b * cache_bs + (h - hq - hkv) * cache_hs + (p0 + t) * hd + c * 8;
    if (h >= hq + hkv) {
      *reinterpret_cast<uint4*>(dst) = u1;
      *reinterpret_cast<uint4*>(dst + half) = u2;
      continue;
    }
    float x1[8], x2[8];
    unpack_bf16x8(u1, x1);
    unpack_bf16x8(u2, x2);
    const float* cs = cos_t + (p0 + t) * half + c * 8;
    const float* sn = sin_t + (p0 + t) * half + c * 8;
    uint32_t o1[4], o2[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float r1[2], r2[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float cv = cs[2 * j + e], sv = sn[2 * j + e];
        r1[e] = __fsub_rn(__fmul_rn(x1[2 * j + e], cv), __fmul_rn(x2[2 * j + e], sv));
        r2[e] = __fadd_rn(__fmul_rn(x2[2 * j + e], cv), __fmul_rn(x1[2 * j + e], sv));
      }
      o1[j] = pack_bf16(r1[0], r1[1]);
      o2[j] = pack_bf16(r2[0], r2[1]);
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    *reinterpret_cast<uint4*>(dst + half) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
  }
}

// ---- greedy sampling: argmax of every row of the logits --------------------------------------
//
// grid = (segments, rows): a CTA reduces one segment of one row to (largest value, its lowest
// index), leaves the pair in the workspace and counts itself; the CTA that counts last for a
// row merges the row's pairs, writes the result and clears the counter.  Values are compared
// through their order-preserving integer image, ties go to the lower index (what a whole-row
// argmax returns), a positive NaN sorts above everything.
constexpr int kArgThreads = 256;

__device__ __forceinline__ uint32_t orderable(uint32_t f32_bits) {
  return (f32_bits & 0x80000000u) ? ~f32_bits : (f32_bits | 0x80000000u);
}
__device__ __forceinline__ float from_orderable(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ void take_better(uint32_t& k, int& i, uint32_t k2, int i2) {
  if (k2 > k || (k2 == k && i2 < i)) { k = k2; i = i2; }
}

__global__ void __launch_bounds__(kArgThreads)
argmax_rows_kernel(const __nv_bfloat16* __restrict__ x, int64_t cols, int seg_cols,
                   int64_t index_offset, float* __restrict__ best_value,
                   int64_t* __restrict__ best_index, uint2* __restrict__ partial,
                   int* __restrict__ counters) {
  __shared__ uint32_t sk[kArgThreads / 32];
  __shared__ int si[kArgThreads / 32];
  __shared__ int s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seg = blockIdx.x, segs = gridDim.x;
  const int64_t row = blockIdx.y;
  griddep_launch_dependents();
  griddep_wait();
  const int64_t c0 = (int64_t)seg * seg_cols;
  const int64_t c1 = c0 + seg_cols < cols ? c0 + seg_cols : cols;
  const __nv_bfloat16* src = x + row * cols;
  uint32_t k = 0;          // below every real value's image
  int idx = 0x7fffffff;
  // 16-byte loads where the row pitch allows them (cols % 8 == 0 keeps every row aligned)
  if ((cols & 7) == 0 && (c0 & 7) == 0) {
    const int64_t v0 = c0 >> 3, v1 = c1 >> 3;
    const uint4* v = reinterpret_cast<const uint4*>(src);
    for (int64_t vi = v0 + tid; vi < v1; vi += kArgThreads) {
      const uint4 u = v[vi];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t klo = orderable(w[j] << 16), khi = orderable(w[j] & 0xffff0000u);
        const int base = (int)(vi * 8 + 2 * j);
        if (klo > k) { k = klo; idx = base; }
        if (khi > k) { k = khi; idx = base + 1; }
      }
    }
    for (int64_t c = (v1 << 3) + tid; c < c1; c += kArgThreads) {
      const uint32_t kk = orderable(__float_as_uint(__bfloat162float(src[c])));
      if (kk > k) { k = kk; idx = (int)c; }
    }
  } else {
    for (int64_t c = c0 + tid; c < c1; c += kArgThreads) {
      const uint32_t kk = orderable(__float_as_uint(__bfloat162float(src[c])));
      if (kk > k) { k = kk; idx = (int)c; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    take_better(k, idx, __shfl_xor_sync(0xffffffffu, k, o), __shfl_xor_sync(0xffffffffu, idx, o));
  if (lane == 0) { sk[warp] = k; si[warp] = idx; }
  __syncthreads();
  if (tid == 0) {
    for (int i = 1; i < kArgThreads / 32; ++i) take_better(k, idx, sk[i], si[i]);
    partial[row * segs + seg] = make_uint2(k, (uint32_t)idx);
    __threadfence();
    const int old = atomicAdd(counters + row, 1);
    s_last = old == segs - 1;
    if (s_last) counters[row] = 0;
  }
  __syncthreads();
  if (!s_last || warp != 0) return;
  __threadfence();
  k = 0;
  idx = 0x7fffffff;
  for (int s = lane; s < segs; s += 32) {
    const uint2 p = __ldcg(partial + row * segs + s);
    take_better(k, idx, p.x, (int)p.y);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    take_better(k, idx, __shfl_xor_sync(0xffffffffu, k, o), __shfl_xor_sync(0xffffffffu, idx, o));
  if (lane == 0) {
    if (best_value) best_value[row] = from_orderable(k);
    best_index[row] = (int64_t)idx + index_offset;
  }
}

}  // namespace
}  // namespace qwx

using namespace qwx;

extern "C" {

static int argmax_segments(int64_t rows, int64_t cols) {
  // enough CTAs to cover the SMs about twice, at least 2048 values each
  int64_t s = (2 * 148 + rows - 1) / rows;
  const int64_t most = (cols + 2047) / 2048;
  if (s > most) s = most;
  if (s > 64) s = 64;
  return (int)(s < 1 ? 1 : s);
}

size_t qwx_argmax_rows_workspace_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return (size_t)rows * 4 + 256 + (size_t)rows * argmax_segments(rows, cols) * 8;
}

int qwx_argmax_rows(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t index_offset,
                    float* best_value, int64_t* best_index, void* workspace,
                    size_t workspace_bytes, qwx_stream_t stream) {
  if (!x || !best_index || !workspace) return QWX_ERR_NULL;
  if (rows <= 0 || cols <= 0 || rows > 65535 || cols > 0x7fffffff) return QWX_ERR_SHAPE;
  if (x_dtype != QWX_BF16) return QWX_ERR_DTYPE;
  if (workspace_bytes < qwx_argmax_rows_workspace_bytes(rows, cols)) return QWX_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 15))
    return QWX_ERR_ALIGN;
  const int segs = argmax_segments(rows, cols);
  int64_t seg_cols = (cols + segs - 1) / segs;
  seg_cols = (seg_cols + 7) & ~(int64_t)7;
  int* counters = (int*)workspace;
  uint2* partial = (uint2*)((char*)workspace + (((size_t)rows * 4 + 255) & ~(size_t)255));
  if (launch_dependent(argmax_rows_kernel, dim3((unsigned)segs, (unsigned)rows), dim3(kArgThreads), 0,
                       (cudaStream_t)stream, (const __nv_bfloat16*)x, cols, (int)seg_cols,
                       index_offset, best_value, best_index, partial, counters) != cudaSuccess) {
    (void)cudaGetLastError();
    return QWX_ERR_LAUNCH;
  }
  return QWX_OK;
}

int qwx_add_rmsnorm_quantize(const void* x, const void* delta, const void* weight, double eps,
                             int64_t rows, int64_t d, void* x_out, void* y_out, void* q,
                             void* scale, qwx_stream_t stream) {
  if (!x || !weight || (!y_out && !q) || (q && !scale) || (delta && !x_out)) return QWX_ERR_NULL;
  if (rows <= 0 || d <= 0 || d % 8) return QWX_ERR_SHAPE;
  if (d > (int64_t)kDThreads * kDVec * 8) return QWX_ERR_UNSUPPORTED;
  const uintptr_t all = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) |
                        reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(x_out) |
                        reinterpret_cast<uintptr_t>(y_out);
  if ((all & 15) || (reinterpret_cast<uintptr_t>(q) & 7)) return QWX_ERR_ALIGN;
  const int64_t cap = 148 * 8;
  const unsigned grid = (unsigned)(rows < cap ? rows : cap);
  if (launch_dependent(add_rmsnorm_kernel, dim3(grid), dim3(kDThreads), 0, (cudaStream_t)stream,
                       (const uint4*)x, (const uint4*)delta, (const uint4*)weight, (float)eps, rows,
                       (int)(d / 8), (uint4*)x_out, (uint4*)y_out, (uint2*)q,
                       (__nv_bfloat16*)scale) != cudaSuccess) {
    (void)cudaGetLastError();
    return QWX_ERR_LAUNCH;
  }
  return QWX_OK;
}

// CTAs of the hand-shaking kernel that can be resident at once on the current device.  The
// hand-shake pairs CTA b of every rank, so every launched CTA must be running while it waits:
// the grid never exceeds this number (ranks on identical GPUs compute the same value).
static int peer_resident_ctas() {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int cached[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int per_sm = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, add_rmsnorm_peer_kernel, kDThreads, 0) !=
            cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return 0;
    cached[dev] = per_sm * sms;
  }
  return cached[dev];
}

int qwx_add_rmsnorm_quantize_peer(const void* x, const void* const* partials, void* const* flags,
                                  int world, int rank, int* launches, int max_ctas,
                                  const void* weight, double eps, int64_t rows, int64_t d,
                                  void* x_out, void* y_out, void* q, void* scale,
                                  int32_t* error_flag, int64_t wait_cycles, qwx_stream_t stream) {
  if (!x || !partials || !flags || !launches || !weight || !x_out || (!y_out && !q) || (q && !scale))
    return QWX_ERR_NULL;
  if (world < 2 || world > kMaxPeers || rank < 0 || rank >= world || max_ctas <= 0) return QWX_ERR_SHAPE;
  if (rows <= 0 || d <= 0 || d % 8) return QWX_ERR_SHAPE;
  if (d > (int64_t)kDThreads * kDVec * 8) return QWX_ERR_UNSUPPORTED;
  PeerArgs pa;
  uintptr_t all = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) |
                  reinterpret_cast<uintptr_t>(x_out) | reinterpret_cast<uintptr_t>(y_out);
  for (int r = 0; r < world; ++r) {
    if (!partials[r] || !flags[r]) return QWX_ERR_NULL;
    pa.partial[r] = (const uint4*)partials[r];
    pa.flags[r] = (int*)flags[r];
    all |= reinterpret_cast<uintptr_t>(partials[r]);
  }
  if ((all & 15) || (reinterpret_cast<uintptr_t>(q) & 7)) return QWX_ERR_ALIGN;
  pa.launches = launches;
  pa.world = world; pa.rank = rank;
  pa.error_flag = error_flag;
  pa.wait_cycles = wait_cycles > 0 ? wait_cycles : kPeerWaitCycles;
  // Every rank must launch the same number of CTAs (the hand-shake is per CTA), all of them
  // resident: rows, the caller's flag capacity and the device's occupancy bound the grid.
  const int resident = peer_resident_ctas();
  if (resident <= 0) return QWX_ERR_NO_DEVICE;
  int64_t cap = max_ctas < resident ? max_ctas : resident;
  const unsigned grid = (unsigned)(rows < cap ? rows : cap);
  if (launch_dependent(add_rmsnorm_peer_kernel, dim3(grid), dim3(kDThreads), 0, (cudaStream_t)stream,
                       (const uint4*)x, pa, (const uint4*)weight, (float)eps, rows, (int)(d / 8),
                       (uint4*)x_out, (uint4*)y_out, (uint2*)q, (__nv_bfloat16*)scale) != cudaSuccess) {
    (void)cudaGetLastError();
    return QWX_ERR_LAUNCH;
  }
  return QWX_OK;
}

static int peer_reduce_resident_ctas() {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int cached[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int per_sm = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, peer_allreduce_kernel, kDThreads, 0) !=
            cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return 0;
    cached[dev] = per_sm * sms;
  }
  return cached[dev];
}

int qwx_peer_allreduce(void* const* partials, void* const* flags, int world, int rank,
                       int* launches, int max_ctas, int64_t rows, int64_t d, int32_t* error_flag,
                       int64_t wait_cycles, qwx_stream_t stream) {
  if (!partials || !flags || !launches) return QWX_ERR_NULL;
  if (world < 2 || world > kMaxPeers || rank < 0 || rank >= world || max_ctas <= 0) return QWX_ERR_SHAPE;
  if (rows <= 0 || d <= 0 || d % 8) return QWX_ERR_SHAPE;
  PeerReduceArgs pa;
  for (int r = 0; r < world; ++r) {
    if (!partials[r] || !flags[r]) return QWX_ERR_NULL;
    if (reinterpret_cast<uintptr_t>(partials[r]) & 15) return QWX_ERR_ALIGN;
    pa.partial[r] = (uint4*)partials[r];
    pa.flags[r] = (int*)flags[r];
  }
  pa.launches = launches;
  pa.world = world; pa.rank = rank; pa.max_ctas = max_ctas;
  pa.error_flag = error_flag;
  pa.wait_cycles = wait_cycles > 0 ? wait_cycles : kPeerWaitCycles;
  // Every rank launches the same number of CTAs, all resident (the first hand-shake is per
  // CTA): a function of the row count only, bounded by the flag capacity and the occupancy.
  const int resident = peer_reduce_resident_ctas();
  if (resident <= 0) return QWX_ERR_NO_DEVICE;
  const int64_t vecs_per_rank = (rows / world + 1) * (d / 8);
  int64_t want = (vecs_per_rank + kDThreads - 1) / kDThreads;
  const int64_t cap = max_ctas < resident ? max_ctas : resident;
  const unsigned grid = (unsigned)(want < cap ? (want < 1 ? 1 : want) : cap);
  if (launch_dependent(peer_allreduce_kernel, dim3(grid), dim3(kDThreads), 0, (cudaStream_t)stream, pa,
                       rows, (int)(d / 8)) != cudaSuccess) {
    (void)cudaGetLastError();
    return QWX_ERR_LAUNCH;
  }
  return QWX_OK;
}

int qwx_silu_mul_quantize(const void* gu, int64_t rows, int64_t f, void* y_out, void* q,
                          void* scale, qwx_stream_t stream) {
  if (!gu || (!y_out && !q) || (q && !scale)) return QWX_ERR_NULL;
  if (rows <= 0 || f <= 0 || f % 8) return QWX_ERR_SHAPE;
  const size_t smem = q ? (size_t)f * 2 : 0;
  if (smem > 200 * 1024) return QWX_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(gu) & 15) || (reinterpret_cast<uintptr_t>(y_out) & 15) ||
      (reinterpret_cast<uintptr_t>(q) & 7))
    return QWX_ERR_ALIGN;
  static PerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(silu_mul_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             200 * 1024) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  const int64_t cap = 148 * 8;   // [8192, 2 x 14336]: 156.5 us with four CTAs per SM, 145.0 with six, 142.4 with eight
  const unsigned grid = (unsigned)(rows < cap ? rows : cap);
  if (launch_dependent(silu_mul_kernel, dim3(grid), dim3(kDThreads), smem, (cudaStream_t)stream,
                       (const uint4*)gu, rows, (int)(f / 8), (uint4*)y_out, (uint2*)q,
                       (__nv_bfloat16*)scale) != cudaSuccess) {
    (void)cudaGetLastError();
    return QWX_ERR_LAUNCH;
  }
  return QWX_OK;
}

int qwx_rope_cache(const void* qkv, int64_t B, int64_t T, int hq, int hkv, int hd, const float* cos_t,
                   const float* sin_t, int64_t pos, const int64_t* pos_dev, void* q_out,
                   void* cache_k, void* cache_v, int64_t cache_batch_stride,
                   int64_t cache_head_stride, qwx_stream_t stream) {
  if (!qkv || !cos_t || !sin_t || !q_out || !cache_k || !cache_v) return QWX_ERR_NULL;
  if (B <= 0 || T <= 0 || hq <= 0 || hkv <= 0 || hd <= 0 || hd % 16) return QWX_ERR_SHAPE;
  if (cache_batch_stride % 8 || cache_head_stride % 8) return QWX_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
       reinterpret_cast<uintptr_t>(cache_k) | reinterpret_cast<uintptr_t>(cache_v)) & 15)
    return QWX_ERR_ALIGN;
  const int64_t total = B * T * (hq + 2 * hkv) * (hd / 16);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (launch_dependent(rope_cache_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream,
                       (const __nv_bfloat16*)qkv, B, T, hq, hkv, hd, cos_t, sin_t, pos, pos_dev,
                       (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache_k, (__nv_bfloat16*)cache_v,
                       cache_batch_stride, cache_head_stride) != cudaSuccess) {
    (void)cudaGetLastError();
    return QWX_ERR_LAUNCH;
  }
  return QWX_OK;
}

}  // extern "C"
