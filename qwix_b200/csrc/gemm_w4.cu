// Weight-only int4 GEMM for decode-shaped problems (few tokens, huge weight): the device
// side of dot_general._slow_dot_general (dot_general.py:264-275) for a bf16 activation and an
// int4 sub-channel-quantized weight,
//
//   out[m, n] = sum_k a[m, k] * W~[k, n],   W~[k, n] = q[k, n] * s[k / tile, n]
//
// without ever writing W~ to global memory.  The kernel is HBM-bound on the packed weight:
// K*N/2 bytes are streamed exactly once, every warp reading its own contiguous run.
//
// Design.  With 1..32 tokens the arithmetic is small; what decides the time is how little
// happens per weight byte besides the load.  A CTA-wide tcgen05 pipeline (operand tiles in
// shared memory, one MMA-issuing thread, mbarrier hand-overs per 8 KB of weights) was measured
// at 80-90 us for 8192 x 28672 whatever the payload: each hand-over costs about 200 cycles of
// a single thread and a 128 x 128 unit needs several.  Here nothing is handed over: every warp
// owns a contiguous range of work items (1, 2 or 4 strips of 16 channels x one 128-wide K
// chunk; stream-K at warp granularity), brings the items' packed codes and scales into a
// private cp.async ring, converts the codes in registers into the A fragments of warp-level
// mma.sync.m16n8k16 (channels are the MMA's M, tokens its N), and takes the B fragments with
// ldmatrix from the activation slice that the CTA keeps resident in shared memory (one set of
// B fragments serves all strips of an item).  The weight layout is made for this by
// qwx_pack_w4: a lane's 16 bytes hold exactly its fragment values for four consecutive K
// tiles, so a warp's load is one contiguous 512-byte line.
//
// The tensor cores multiply the activation with 136 + code (one logic operation per pair of
// codes makes that bf16 number; exact); per 128 K the constant is taken out again with
// 136 x (sum of the chunk's activations) -- from the same MMAs against an operand of ones, once
// per CTA -- and the float32 partial sums are multiplied by the channel's scale and added to
// the running sums.  With float32 scales this is the reference's arithmetic up to the order of
// the float32 sums (its dequantized weight q * s is exact in float32) and the cancellation of
// the constant (about 2^-19 of a chunk's sum); with bf16 scales the reference rounds q * s to
// bf16 first, which this kernel does not reproduce -- it is closer to the unquantized product,
// within the stated output tolerance.
//
// K is cut into `split` slices so that the activation slice (tokens x K / split, bf16) fits
// shared memory; CTAs with blockIdx.x = s work on slice s.  A strip whose chunks are spread
// over several warps (always the case when split > 1) is summed with float atomics in a
// caller-provided zeroed workspace; the warp that contributes last converts it and clears the
// workspace.
#include "common.cuh"
#include <algorithm>

namespace qwx {
namespace {

constexpr int kStrip = 16;          // channels per strip: the M of mma.m16n8k16
constexpr int kChunkK = 128;        // K per work item: eight K16 tiles, 2 x 16 bytes per lane and strip, one scale
constexpr int kScaleK = 128;        // partial sums are scaled every 128 K
// Warps per CTA: 32 for up to 8 tokens (few registers per thread, and twice the warps hide the
// latency of the dependent MMAs of a chunk), 16 beyond.
__host__ __device__ constexpr int w4_warps(int nt, int sp) { return nt == 1 && sp < 4 ? 32 : 16; }
constexpr size_t kSmemCap = 226 * 1024;
// Work items (1 KB per strip) a warp keeps in flight in its private cp.async ring: loaded HBM
// latency is a few microseconds, so an SM needs on the order of 100 KB in flight to stream at
// its share of the bandwidth.  More tokens leave less room beside the activation slice.
__host__ __device__ constexpr int w4_depth(int nt, int sp) {
  return sp == 4 ? 2 : (nt == 1 ? 4 : (nt == 2 ? 6 : 4)) / sp;
}
// a ring stage: one work item's codes (1 KB per strip) and scales (a 64-byte slot per strip)
__host__ __device__ constexpr int w4_stage_bytes(int sp) { return sp * (1024 + 64); }
__host__ __device__ constexpr size_t w4_ring_bytes(int nt, int sp) {
  return (size_t)w4_warps(nt, sp) * w4_depth(nt, sp) * w4_stage_bytes(sp);
}

struct W4Params {
  const uint4* wp;        // packed chunks, [N / 16][K / 128][2][32 lanes] x 16 bytes
  const void* scale;      // [K / tile, N], f32 or bf16
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
  // x / d as umulhi(x, mul) + x * one: mul = ceil(2^32 / d), one = 0 (d > 1); mul = 0, one = 1 (d = 1)
  uint32_t cps_mul, cps_one;   // d = chunks per strip in a slice
  uint32_t bps_mul, bps_one;   // d = tile / 128
  int items_q, items_r;        // work items of a slice / its warps: quotient and remainder
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
// The first K16 tile of a chunk: the accumulator starts from zero, no registers to clear.
__device__ __forceinline__ void mma_bf16_first(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%10, %10, %10, %10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// Eight offset-binary nibbles (code + 8) of one lane and one K16 tile -> the four A-fragment
// registers.  Nibble j sits under nibble j + 4 of the same register: 0x4300 | u is the bf16
// number 128 + u = 136 + code, one logic operation per pair of codes.  The constant 136 is
// taken out again after the contraction: 136 * (sum of the chunk's activations) per token.
constexpr float kCodeBias = 136.f;
__device__ __forceinline__ void unpack_fragment(uint32_t w, uint32_t (&a)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) a[j] = ((w >> (4 * j)) & 0x000f000fu) | 0x43004300u;
}

template <int NT> struct BFrag { uint32_t r[NT == 1 ? 2 : 2 * NT]; };

// B fragments (activation) of K16 tile I of the chunk at `kaddr`: NT = 1 -> tokens 0-7
// (registers k 0-7, k 8-15); else per 16 tokens registers (tokens 0-7: k 0-7, k 8-15),
// (tokens 8-15: k 0-7, k 8-15).
template <int I, int NT>
__device__ __forceinline__ void load_b(uint32_t kaddr, int pitch, BFrag<NT>& b) {
  if constexpr (NT == 1) {
    uint32_t r[2];
    ldmatrix_x2<I * 32>(kaddr, r);
    b.r[0] = r[0]; b.r[1] = r[1];
  } else {
#pragma unroll
    for (int pr = 0; pr < NT / 2; ++pr) {
      uint32_t r[4];
      ldmatrix_x4<I * 32>(kaddr + (uint32_t)(pr * 16 * pitch), r);
      b.r[4 * pr] = r[0]; b.r[4 * pr + 1] = r[1]; b.r[4 * pr + 2] = r[2]; b.r[4 * pr + 3] = r[3];
    }
  }
}

// One K16 tile of a work item: SP strips against the same B fragments.
template <int I, int NT, int SP>
__device__ __forceinline__ void tile_step(uint32_t kaddr, int pitch, const uint4 (&wq)[SP][2],
                                          float (&acc)[SP][NT][4]) {
  BFrag<NT> b;
  load_b<I, NT>(kaddr, pitch, b);
#pragma unroll
  for (int s = 0; s < SP; ++s) {
    const uint4& q4 = wq[s][I >> 2];
    const uint32_t word = (I & 3) == 0 ? q4.x : ((I & 3) == 1 ? q4.y : ((I & 3) == 2 ? q4.z : q4.w));
    uint32_t a[4];
    unpack_fragment(word, a);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      if constexpr (I == 0) mma_bf16_first(acc[s][n], a, b.r[2 * n], b.r[2 * n + 1]);
      else mma_bf16(acc[s][n], a, b.r[2 * n], b.r[2 * n + 1]);
    }
  }
}

// A warp is done with its chunks of a strip pair.  If they were all of the strips' K it writes
// the output; otherwise it adds its running sums to the workspace, and whoever completes the
// strips converts them and leaves the workspace zero.  The running sums are cleared.
template <int NT, int SP>
__device__ __forceinline__ void w4_finish(const W4Params& p, float (&run)[SP][NT][4], int sp,
                                       int contributed, int chunks_per_strip, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const bool whole = contributed == chunks_per_strip;
  bool fin = whole;
  if (!whole) {
#pragma unroll
    for (int s = 0; s < SP; ++s) {
      const int64_t ch = (int64_t)(sp * SP + s) * kStrip + g;
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int tok = n * 8 + 2 * t + (j & 1);
          if (tok < p.M) atomicAdd(p.ws + (int64_t)tok * p.N + ch + (j >> 1) * 8, run[s][n][j]);
        }
    }
    __threadfence();
    __syncwarp();
    int last = 0;
    if (lane == 0) {
      const int old = atomicAdd(p.counters + sp, contributed);
      last = old + contributed == chunks_per_strip;
      if (last) p.counters[sp] = 0;
    }
    fin = __shfl_sync(0xffffffffu, last, 0) != 0;
    if (fin) {
      __threadfence();
#pragma unroll
      for (int s = 0; s < SP; ++s) {
        const int64_t ch = (int64_t)(sp * SP + s) * kStrip + g;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int tok = n * 8 + 2 * t + (j & 1);
            float* w = p.ws + (int64_t)tok * p.N + ch + (j >> 1) * 8;
            run[s][n][j] = tok < p.M ? __ldcg(w) : 0.f;
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
  }
  if (fin) {
#pragma unroll
    for (int s = 0; s < SP; ++s) {
      const int64_t ch = (int64_t)(sp * SP + s) * kStrip + g;
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int tok = n * 8 + 2 * t + (j & 1);
          if (tok >= p.M) continue;
          const int64_t at = (int64_t)tok * p.N + ch + (j >> 1) * 8;
          if (p.out_dtype == QWX_BF16)
            reinterpret_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(run[s][n][j]);
          else
            reinterpret_cast<float*>(p.out)[at] = run[s][n][j];
        }
    }
  }
#pragma unroll
  for (int s = 0; s < SP; ++s)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) run[s][n][j] = 0.f;
}

// NT token tiles of 8 (the activation is padded to NT * 8 rows); SP strips of 16 channels per
// work item (2 where N / 16 is even: the B fragments and the loop's bookkeeping serve both);
// F32S: float32 scales (else bf16).
//
// A warp's ring stage holds one work item: SP x 1 KB of packed codes and, behind them, the 16
// scales of each strip (a 64-byte slot per strip), all brought by cp.async so that one
// wait_group covers an item.  Where an item lies (strip pair, chunk, addresses) is computed
// from its linear index with a multiply-high division: no cursor state, no branches.
template <int NT, int SP, bool F32S>
__global__ void __launch_bounds__(w4_warps(NT, SP) * 32, 1) gemm_w4_kernel(const W4Params p) {
  constexpr int kW4Warps = w4_warps(NT, SP);
  constexpr int kW4Threads = kW4Warps * 32;
  constexpr int D = w4_depth(NT, SP);
  constexpr int kStage = w4_stage_bytes(SP);
  extern __shared__ __align__(16) uint8_t act[];
  constexpr int MPAD = NT * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int slice = blockIdx.x;           // neighbouring CTAs take the K slices of the same strips
  const int cta_in_slice = blockIdx.y;

  // ---- the CTA's activation slice: tokens x ks, rows `pitch` bytes apart (16 bytes of padding
  // keep the eight rows of an ldmatrix in different banks); rows beyond M are zero ----
  {
    const int vec_per_row = p.ks / 8;
    const uint32_t act_s = (uint32_t)__cvta_generic_to_shared(act);
    const uint4* a_slice = reinterpret_cast<const uint4*>(p.a + (int64_t)slice * p.ks);
    const int row_vec = (int)(p.K / 8);                        // 16-byte vectors per activation row
    // (token, vector) of this thread's element, advanced by kW4Threads elements per step
    const int d_tok = kW4Threads / vec_per_row, d_cv = kW4Threads - d_tok * vec_per_row;
    int token = (int)threadIdx.x / vec_per_row, cv = (int)threadIdx.x - token * vec_per_row;
    while (token < MPAD) {
      const uint32_t dst = act_s + (uint32_t)(token * p.pitch + cv * 16);
      if (token < p.M)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(a_slice + (int64_t)token * row_vec + cv) : "memory");
      else
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
      token += d_tok; cv += d_cv;
      if (cv >= vec_per_row) { cv -= vec_per_row; ++token; }
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");

  // ---- this warp's contiguous range of work items, strip-major inside the slice: the items
  // of a slice are dealt evenly to its warps (the first items_r warps take one more) ----
  const int cps = p.ks / kChunkK;                       // chunks per strip in one slice
  const int chunks_per_strip = (int)(p.K / kChunkK);    // ... in all slices
  const int wg = cta_in_slice * kW4Warps + warp;
  const int c_begin = wg * p.items_q + min(wg, p.items_r);
  const int c_end = c_begin + p.items_q + (wg < p.items_r ? 1 : 0);

  // shared memory: activation slice | 136 * chunk sums [cps][MPAD] float | per-warp rings
  float* csum = reinterpret_cast<float*>(act + (size_t)MPAD * p.pitch);
  const uint32_t ring_warp = (uint32_t)__cvta_generic_to_shared(act) + (uint32_t)(MPAD * p.pitch) +
                             (uint32_t)(cps * MPAD * 4) + (uint32_t)(warp * D * kStage);
  const uint32_t ring = ring_warp + lane * 16;   // this lane's 16 bytes of stage 0, strip 0, half 0

  // Per-lane constants of the fetch.  Codes: offsets in 16-byte units from wp.  Scales: one
  // 4-byte cp.async per lane -- float32: lane = strip * 16 + channel; bf16: lane = strip * 8 +
  // channel pair.
  const uint32_t w_lane = (uint32_t)(slice * cps) * 64u + lane;
  const uint32_t w_pair = (uint32_t)(SP * chunks_per_strip) * 64u;   // from one strip pair to the next
  const uint32_t strip_o = (uint32_t)chunks_per_strip * 64u;
  constexpr int kScCopy = SP == 4 ? 8 : 4;                          // bytes per lane
  constexpr int kScElems = kScCopy / (F32S ? 4 : 2);                 // channels per lane
  constexpr int kScLanes = kStrip / kScElems;                        // lanes per strip
  const bool sc_active = lane < kScLanes * SP;
  const int sc_strip = lane / kScLanes;
  const int sc_elem = (lane % kScLanes) * kScElems;                  // first channel of the lane's bytes
  const int sc_src = sc_strip * kStrip + sc_elem;
  const uint32_t sc_dst = ring_warp + SP * 1024 + sc_strip * 64 + sc_elem * (F32S ? 4 : 2);
  const int row0 = slice * cps;                                          // first 128-K block of the slice
  auto fetch = [&](int cf, int stage) {
    if (cf < c_end) {
      const uint32_t sp_f = __umulhi((uint32_t)cf, p.cps_mul) + (uint32_t)cf * p.cps_one;
      const uint32_t kc_f = (uint32_t)cf - sp_f * (uint32_t)cps;
      const uint32_t off = sp_f * w_pair + kc_f * 64u + w_lane;
#pragma unroll
      for (int s = 0; s < SP; ++s) {
        const uint4* src = p.wp + (off + s * strip_o);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring + stage * kStage + s * 1024), "l"(src) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring + stage * kStage + s * 1024 + 512), "l"(src + 32) : "memory");
      }
      if (sc_active) {
        const uint32_t blk = (uint32_t)row0 + kc_f;
        const uint32_t row = __umulhi(blk, p.bps_mul) + blk * p.bps_one;
        const uint32_t e = row * (uint32_t)p.N + sp_f * (SP * kStrip) + sc_src;
        const char* src = reinterpret_cast<const char*>(p.scale) + (size_t)e * (F32S ? 4 : 2);
        asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(sc_dst + stage * kStage), "l"(src), "n"(kScCopy) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // the activation slice is the oldest commit group: waiting until at most D groups pend
  // completes it
#pragma unroll
  for (int u = 0; u < D; ++u) fetch(c_begin + u, u);
  asm volatile("cp.async.wait_group %0;" ::"n"(D) : "memory");
  __syncthreads();

  // per-lane byte offset of its ldmatrix row: matrices 0..3 = (tokens 0-7, k 0-7), (tokens 0-7,
  // k 8-15), (tokens 8-15, k 0-7), (tokens 8-15, k 8-15)
  const int lm = lane >> 3, lr = lane & 7;
  const uint32_t act_lane = (uint32_t)__cvta_generic_to_shared(act) +
                            (uint32_t)(((lm >> 1) * 8 + lr) * p.pitch + (lm & 1) * 16);

  // ---- 136 * (sum of each token's activations over each 128-K chunk of the slice): the same
  // MMAs with an A operand of ones; every row of the result holds the sums ----
  {
    const uint32_t ones[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};
    constexpr int kPerChunk = NT == 1 ? 1 : NT / 2;
    for (int e = warp; e < cps * kPerChunk; e += kW4Warps) {
      const int ck = e / kPerChunk, pr = e - ck * kPerChunk;
      const uint32_t ka = act_lane + (uint32_t)(ck * kChunkK) * 2u + (uint32_t)(pr * 16 * p.pitch);
      float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if constexpr (NT == 1) {
          uint32_t b[2];
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];"
                       : "=r"(b[0]), "=r"(b[1]) : "r"(ka + i * 32));
          mma_bf16(d0, ones, b[0], b[1]);
        } else {
          uint32_t b[4];
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                       : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(ka + i * 32));
          mma_bf16(d0, ones, b[0], b[1]);
          mma_bf16(d1, ones, b[2], b[3]);
        }
      }
      if (g == 0) {
        float* row = csum + ck * MPAD + pr * 16 + 2 * t;
        *reinterpret_cast<float2*>(row) = make_float2(kCodeBias * d0[0], kCodeBias * d0[1]);
        if constexpr (NT > 1)
          *reinterpret_cast<float2*>(row + 8) = make_float2(kCodeBias * d1[0], kCodeBias * d1[1]);
      }
    }
  }
  __syncthreads();

  float acc[SP][NT][4], run[SP][NT][4];
#pragma unroll
  for (int s = 0; s < SP; ++s)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) run[s][n][j] = 0.f;
  const int sp_begin = (int)(__umulhi((uint32_t)c_begin, p.cps_mul) + (uint32_t)c_begin * p.cps_one);
  int sp = sp_begin;
  int kc = c_begin - sp * cps;
  const int kc_begin = kc;
  // this lane's scales in a stage: channels g and g + 8 of each strip
  const uint32_t sc_lane = ring_warp + SP * 1024 + (F32S ? g * 4 : g * 2);

  for (int base = c_begin; base < c_end; base += D) {
#pragma unroll
    for (int u = 0; u < D; ++u) {
      const int c = base + u;
      if (c >= c_end) break;
      asm volatile("cp.async.wait_group %0;" ::"n"(D - 1) : "memory");
      uint4 wq[SP][2];
#pragma unroll
      for (int s = 0; s < SP; ++s)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(wq[s][hf].x), "=r"(wq[s][hf].y), "=r"(wq[s][hf].z), "=r"(wq[s][hf].w)
                       : "r"(ring + u * kStage + s * 1024 + hf * 512) : "memory");
      float s_lo[SP], s_hi[SP];
#pragma unroll
      for (int s = 0; s < SP; ++s) {
        if constexpr (F32S) {
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s_lo[s]) : "r"(sc_lane + u * kStage + s * 64) : "memory");
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s_hi[s]) : "r"(sc_lane + u * kStage + s * 64 + 32) : "memory");
        } else {
          uint32_t lo, hi;
          asm volatile("ld.shared.u16 %0, [%1];" : "=r"(lo) : "r"(sc_lane + u * kStage + s * 64) : "memory");
          asm volatile("ld.shared.u16 %0, [%1];" : "=r"(hi) : "r"(sc_lane + u * kStage + s * 64 + 16) : "memory");
          s_lo[s] = __uint_as_float(lo << 16);
          s_hi[s] = __uint_as_float(hi << 16);
        }
      }
      fetch(c + D, u);   // into the ring stage just read
      const uint32_t kaddr = act_lane + (uint32_t)(kc * kChunkK) * 2u;
      tile_step<0, NT, SP>(kaddr, p.pitch, wq, acc);
      tile_step<1, NT, SP>(kaddr, p.pitch, wq, acc);
      tile_step<2, NT, SP>(kaddr, p.pitch, wq, acc);
      tile_step<3, NT, SP>(kaddr, p.pitch, wq, acc);
      tile_step<4, NT, SP>(kaddr, p.pitch, wq, acc);
      tile_step<5, NT, SP>(kaddr, p.pitch, wq, acc);
      tile_step<6, NT, SP>(kaddr, p.pitch, wq, acc);
      tile_step<7, NT, SP>(kaddr, p.pitch, wq, acc);

      // the chunk is one scale block: take the code bias out of its partial sums and scale
      // them into the running sums
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const float2 cs = *reinterpret_cast<const float2*>(csum + kc * MPAD + n * 8 + 2 * t);
#pragma unroll
        for (int s = 0; s < SP; ++s) {
          run[s][n][0] = __fmaf_rn(acc[s][n][0] - cs.x, s_lo[s], run[s][n][0]);
          run[s][n][1] = __fmaf_rn(acc[s][n][1] - cs.y, s_lo[s], run[s][n][1]);
          run[s][n][2] = __fmaf_rn(acc[s][n][2] - cs.x, s_hi[s], run[s][n][2]);
          run[s][n][3] = __fmaf_rn(acc[s][n][3] - cs.y, s_hi[s], run[s][n][3]);
        }
      }
      if (kc == cps - 1 || c == c_end - 1) {
        // ---- this warp is done with the strips of the item ----
        const int contributed = kc + 1 - (sp == sp_begin ? kc_begin : 0);
        w4_finish<NT, SP>(p, run, sp, contributed, chunks_per_strip, lane);
      }
      if (++kc == cps) { kc = 0; ++sp; }
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

// Fewest K slices (a divisor of K / 128) whose activation slice, with its table of chunk sums
// (one float per token and 128 K), fits shared memory.
int w4_split(int mpad, int64_t K, size_t cap) {
  const int64_t blocks = K / kScaleK;
  for (int64_t d = 1; d <= blocks; ++d) {
    if (blocks % d) continue;
    const size_t ks = (size_t)(K / d);
    if ((size_t)mpad * (ks * 2 + 16) + (ks / kChunkK) * mpad * 4 <= cap) return (int)d;
  }
  return 0;
}

template <int NT, int SP>
bool w4_configure() {
  return cudaFuncSetAttribute(gemm_w4_kernel<NT, SP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)kSmemCap) == cudaSuccess &&
         cudaFuncSetAttribute(gemm_w4_kernel<NT, SP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)kSmemCap) == cudaSuccess;
}

template <int NT, int SP>
void w4_launch(const W4Params& p, bool f32_scales, dim3 grid, size_t smem, cudaStream_t st) {
  if (f32_scales) gemm_w4_kernel<NT, SP, true><<<grid, w4_warps(NT, SP) * 32, smem, st>>>(p);
  else gemm_w4_kernel<NT, SP, false><<<grid, w4_warps(NT, SP) * 32, smem, st>>>(p);
}

// x / d for x * d < 2^32 as umulhi(x, mul) + x * one
void w4_divisor(uint32_t d, uint32_t* mul, uint32_t* one) {
  if (d <= 1) { *mul = 0; *one = 1; return; }
  *mul = (uint32_t)(((1ull << 32) + d - 1) / d);
  *one = 0;
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
  // 32-bit cursors in the kernel: the packed weight in 16-byte units and the scale elements
  if ((N / kStrip) * (K / kChunkK) > (1 << 24) || (K / k_tile) * N > INT32_MAX / 2)
    return QWX_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  if (!workspace_is_zero &&
      cudaMemsetAsync(workspace, 0, qwx_gemm_a16w4_workspace_bytes(M, N), st) != cudaSuccess)
    return QWX_ERR_LAUNCH;

  static PerDeviceOnce configured;
  if (configured.first()) {
    if (!w4_configure<1, 1>() || !w4_configure<2, 1>() || !w4_configure<4, 1>() ||
        !w4_configure<1, 2>() || !w4_configure<2, 2>() || !w4_configure<4, 2>() ||
        !w4_configure<1, 4>())
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
    // strips per work item: 4 for up to 8 tokens where the strips divide so, else 2, else 1
    const int sp = nt == 1 && (N / kStrip) % 4 == 0 ? 4 : ((N / kStrip) % 2 == 0 ? 2 : 1);
    const int split = w4_split(nt * 8, K, kSmemCap - w4_ring_bytes(nt, sp));
    if (split <= 0 || split > sms) return QWX_ERR_UNSUPPORTED;
    W4Params p;
    p.wp = (const uint4*)w_packed;
    p.scale = scale;
    p.a = (const __nv_bfloat16*)a + m0 * K;
    p.M = rows; p.N = N; p.K = K; p.tile = (int)k_tile;
    p.split = split;
    p.ks = (int)(K / split);
    p.pitch = p.ks * 2 + 16;
    p.out = (char*)out + m0 * N * out_elem; p.out_dtype = out_dtype;
    p.ws = (float*)workspace + m0 * N;
    p.counters = (int*)((char*)workspace + M * N * 4);
    const int ctas_per_slice = sms / split;
    const dim3 grid((unsigned)split, (unsigned)ctas_per_slice);
    {
      const int64_t items = (N / (kStrip * sp)) * (int64_t)(p.ks / kChunkK);
      const int64_t warps = (int64_t)ctas_per_slice * w4_warps(nt, sp);
      p.items_q = (int)(items / warps);
      p.items_r = (int)(items % warps);
    }
    const size_t smem = (size_t)nt * 8 * p.pitch + (size_t)(p.ks / kChunkK) * nt * 8 * 4 + w4_ring_bytes(nt, sp);
    w4_divisor((uint32_t)(p.ks / kChunkK), &p.cps_mul, &p.cps_one);
    w4_divisor((uint32_t)(k_tile / kChunkK), &p.bps_mul, &p.bps_one);
    // the multiply-high divisions are exact while dividend * divisor < 2^32
    if ((N / (kStrip * sp)) * (int64_t)(p.ks / kChunkK) * (p.ks / kChunkK) >= (1ll << 32) ||
        (K / kChunkK) * (k_tile / kChunkK) >= (1ll << 32))
      return QWX_ERR_UNSUPPORTED;
    const bool f32s = scale_dtype == QWX_F32;
    if (sp == 4) {
      w4_launch<1, 4>(p, f32s, grid, smem, st);
    } else if (sp == 2) {
      if (nt == 1) w4_launch<1, 2>(p, f32s, grid, smem, st);
      else if (nt == 2) w4_launch<2, 2>(p, f32s, grid, smem, st);
      else w4_launch<4, 2>(p, f32s, grid, smem, st);
    } else {
      if (nt == 1) w4_launch<1, 1>(p, f32s, grid, smem, st);
      else if (nt == 2) w4_launch<2, 1>(p, f32s, grid, smem, st);
      else w4_launch<4, 1>(p, f32s, grid, smem, st);
    }
    QWX_CHECK_LAUNCH();
  }
  return QWX_OK;
}

}  // extern "C"
