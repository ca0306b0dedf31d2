// Weight-only int4 GEMM on the tcgen05 tensor cores, for 33 tokens and more:
//
//   out[m, n] = sum_k a[m, k] * W~[k, n],   W~[k, n] = bf16( q[k, n] * s[k / tile, n] )
//
// the device side of dot_general._slow_dot_general (qwix/_src/core/dot_general.py:264-275: the
// weight is dequantized, qarray.py:692-708, then contracted in floating point) for a bf16
// activation and an int4 sub-channel-quantized weight, without W~ ever reaching global memory.
// With bfloat16 scales W~ is exactly the reference's dequantized weight; with float32 scales the
// reference keeps q * s in float32 and this kernel rounds it once to bfloat16 (2^-9 relative
// per weight, inside the stated output tolerance; the warp-level kernel in gemm_w4.cu, which
// serves up to 32 tokens, keeps float32 there).
//
// The operands are swapped on the tensor core, as in the int8 decode kernel: 128 output
// channels are the M of a tcgen05.mma (kind::f16, bf16 x bf16 -> float32), the tokens its N
// (32, 64 or 128).  A stage of the shared-memory ring holds 128 K of 128 channels as bfloat16
// (32 KB, two 128-byte-swizzled halves of 64 K) and the same K of the tokens (TMA).  The
// weight half is written by converter warps: a thread reads 16 bytes of packed codes (32
// consecutive K of one channel) at a time, turns every 32-bit word into four
// bf16 pairs with one logic operation per pair -- (w >> 4i) & 0x000F000F | 0x43004300 is the
// pair (128 + u, 128 + u') of offset-binary nibbles, the nibbles being stored in that order by
// qwx_pack_w4_tiles -- subtracts 136, multiplies by the channel's scale and stores 16 bytes
// into the swizzled tile.  Accumulation runs over all of K in tensor memory, so the epilogue
// runs once per tile, not once per scale tile.
//
// Work is cut stream-K style over (channel tile, K stage) units, every CTA taking an equal
// contiguous run; a tile shared by several CTAs is summed with float32 red.global.add in a
// zeroed scratch slot and finished by whoever adds last (the order of those additions is not
// fixed: the last bits of such tiles can differ from run to run).
//
// Roles (480 threads): warp 0 TMA producer of the token halves, warp 1 MMA issuer and
// tensor-memory owner, warps 2-5 epilogue, warps 6-13 converters, warp 14 loader of the packed
// codes and scales (bulk copies into a ring of eight 8.5 KB slots: 64 KB in flight per SM is
// what the latency of HBM asks for; with the converters loading their own 16 bytes one unit
// ahead the kernel ran at 0.9 TB/s whatever the token count).  Every wait is bounded.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qwix_b200.h"
#include "common.cuh"
#include "sm100.cuh"

namespace qwx {
namespace {

using namespace sm100;

constexpr int WT = 128;          // channels per tile: the MMA's M
constexpr int WK = 128;          // K per stage: one scale tile at most, two swizzle rows of 64 bf16
constexpr int WUK = 16;          // K per tcgen05.mma for 16-bit operands
constexpr int kWmThreads = 480;
constexpr int kWmConvWarp0 = 6;
constexpr int kWmConvWarps = 8;
constexpr int kWmGroups = 2;      // converter groups, each takes every other unit
constexpr int kWmGroupWarps = kWmConvWarps / kWmGroups;
constexpr int kWmLoadWarp = 14;
constexpr int kWmPacked = 8;     // packed units in flight per SM: 64 KB, what HBM latency asks for
constexpr int kWmSlotBytes = 8192 + 512;    // a unit's codes and its 128 scales
constexpr int kWmMaxGrid = 256;  // scratch slots: one per CTA
constexpr int kWmUnitBytes = WT * WK / 2;   // 8 KB of packed codes per (tile, stage)

template <int NT>
struct WmCfg {
  static constexpr int kStages = NT <= 64 ? 3 : 2;
  static constexpr int kWBytes = WT * WK * 2;
  static constexpr int kABytes = NT * WK * 2;
  static constexpr int kStageBytes = kWBytes + kABytes;
  static constexpr int kTmemCols = 2 * NT;
};

struct WmControl {
  uint64_t full[3];
  uint64_t empty[3];
  uint64_t pfull[kWmPacked];
  uint64_t pempty[kWmPacked];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t epi_bar;
  uint32_t tmem_base;
  int abort;
  int last;
};

template <int NT>
constexpr size_t wm_smem_bytes() {
  return 1024 + (size_t)WmCfg<NT>::kStages * WmCfg<NT>::kStageBytes + (size_t)kWmPacked * kWmSlotBytes +
         sizeof(WmControl);
}

struct WmParams {
  int M;
  int64_t N, K;
  const uint4* wp;        // [N / 128][K / 128][4 quarters of 32 K][128 channels][16 B]
  const void* scale;      // [K / tile, N], f32 or bf16
  int scale_dtype;
  int tile;               // scale tile along K (multiple of 128)
  void* out;
  int out_dtype;
  int32_t* error_flag;
  int kstages;            // stages of 128 K per tile
  long long units;        // tiles * kstages
  float* ws;              // [grid][NT][128] partial sums, zero on entry, left zero
  int* counters;          // [grid], zero on entry, left zero
};

__device__ __forceinline__ int wm_cta_of_unit(long long u, long long G, long long U) {
  return (int)(((u + 1) * G - 1) / U);
}

// Eight codes of one 32-bit word -> eight scaled bf16 values (K order), see the file comment.
template <bool F32SCALE>
__device__ __forceinline__ uint4 wm_convert(uint32_t w, float s, __nv_bfloat162 s2) {
  const __nv_bfloat162 off = __floats2bfloat162_rn(136.0f, 136.0f);
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t t = ((w >> (4 * i)) & 0x000F000Fu) | 0x43004300u;
    __nv_bfloat162 h = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&t), off);   // exact
    if (F32SCALE) {
      const float2 f = __bfloat1622float2(h);
      h = __floats2bfloat162_rn(__fmul_rn(f.x, s), __fmul_rn(f.y, s));
    } else {
      h = __hmul2(h, s2);
    }
    o[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

template <int NT>
__global__ void __launch_bounds__(kWmThreads, 1)
gemm_w4_mma_kernel(const __grid_constant__ CUtensorMap tma_a, const WmParams p) {
  using Cfg = WmCfg<NT>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
  uint8_t* packed_ptr = ring_ptr + (size_t)Cfg::kStages * Cfg::kStageBytes;
  const uint32_t packed_ring = ring + Cfg::kStages * Cfg::kStageBytes;
  WmControl* ctl = reinterpret_cast<WmControl*>(packed_ptr + (size_t)kWmPacked * kWmSlotBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort = &ctl->abort;
  const long long G = gridDim.x, U = p.units;
  const long long u_begin = (long long)blockIdx.x * U / G;
  const long long u_end = (long long)(blockIdx.x + 1) * U / G;
  const int S = p.kstages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1 + kWmGroupWarps);   // the TMA bytes and one group of converter warps
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int s = 0; s < kWmPacked; ++s) {
      mbar_init(smem_u32(&ctl->pfull[s]), 1);
      mbar_init(smem_u32(&ctl->pempty[s]), kWmGroupWarps);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->acc_full[a]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[a]), 4);
    }
    mbar_init(smem_u32(&ctl->epi_bar), 4);
    ctl->abort = 0;
    ctl->last = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_a);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), Cfg::kTmemCols);
    tmem_relinquish();
  }
  griddep_launch_dependents();
  griddep_wait();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer: the token halves ----------------
    int stage = 0;
    uint32_t phase = 0;
    long issued = 0;
    bool ok = true;
    for (long long u = u_begin; u < u_end && ok; ++u) {
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort);
        if (ok) {
          const int ks = (int)(u % S);
          const uint32_t bar = smem_u32(&ctl->full[stage]);
          const uint32_t sact = ring + stage * Cfg::kStageBytes + Cfg::kWBytes;
          mbar_expect_tx(bar, Cfg::kABytes);
          tma_load_2d(sact, &tma_a, ks * WK, 0, bar);
          tma_load_2d(sact + NT * 128, &tma_a, ks * WK + 64, 0, bar);
          ++issued;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
    }
    if (lane == 0 && *abort) {
      // Let copies that are still in flight land before the CTA gives up its shared memory.
      // (full[] also counts the converter warps, which may have given up: bounded polls.)
      long pending = issued < Cfg::kStages ? issued : Cfg::kStages;
      int s = stage;
      uint32_t ph = phase;
      for (long i = 0; i < pending; ++i) {
        if (--s < 0) { s = Cfg::kStages - 1; ph ^= 1u; }
        for (int it = 0; it < 100000; ++it)
          if (mbar_try_wait(smem_u32(&ctl->full[s]), ph)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc = make_idesc(1, 1, 1, 0, 0, WT, NT);   // f32 += bf16 x bf16, both K-major
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (long long u = u_begin; u < u_end && ok; ++u) {
      const int ks = (int)(u % S);
      const bool seg_first = (u == u_begin) || ks == 0;
      const bool seg_last = (u == u_end - 1) || ks == S - 1;
      if (lane == 0) {
        if (seg_first) {
          ok = mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort);
          tc_fence_after();
        }
        if (ok) ok = mbar_wait(smem_u32(&ctl->full[stage]), phase, abort);
        if (ok) {
          tc_fence_after();
          const uint32_t sw = ring + stage * Cfg::kStageBytes;
          const uint32_t sact = sw + Cfg::kWBytes;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int kk = 0; kk < 64 / WUK; ++kk) {
              // K-major operands: 8-row groups 1024 B apart, 32 B (16 bf16) steps inside the swizzled row
              const uint64_t da = make_smem_desc(sw + j * (WT * 128) + kk * 32, 16, 1024);
              const uint64_t db = make_smem_desc(sact + j * (NT * 128) + kk * 32, 16, 1024);
              mma_ss<MmaKind::kF16>(tmem_base + acc * NT, da, db, idesc,
                                    !(seg_first && j == 0 && kk == 0));
            }
          }
          mma_commit(smem_u32(&ctl->empty[stage]));
          if (seg_last) mma_commit(smem_u32(&ctl->acc_full[acc]));
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
      if (seg_last && ++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  } else if (warp == kWmLoadWarp) {
    // ---------------- loader: packed codes and scales of the units, eight units ahead ----------
    const int esz = p.scale_dtype == QWX_F32 ? 4 : 2;
    int slot = 0;
    uint32_t phase = 0;
    long issued = 0;
    bool ok = true;
    for (long long u = u_begin; u < u_end && ok; ++u) {
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&ctl->pempty[slot]), phase ^ 1u, abort);
        if (ok) {
          const int tile = (int)(u / S), ks = (int)(u % S);
          const uint32_t bar = smem_u32(&ctl->pfull[slot]);
          const uint32_t dst = packed_ring + slot * kWmSlotBytes;
          const int64_t n0 = (int64_t)tile * WT;
          const int valid = (int)(p.N - n0 < WT ? p.N - n0 : WT);
          const uint32_t sbytes = (uint32_t)(valid * esz);      // a multiple of 16: N is one of 8
          mbar_expect_tx(bar, kWmUnitBytes + sbytes);
          bulk_load(dst, p.wp + ((size_t)tile * S + ks) * (kWmUnitBytes / 16), kWmUnitBytes, bar);
          bulk_load(dst + kWmUnitBytes,
                    reinterpret_cast<const uint8_t*>(p.scale) +
                        ((size_t)((int64_t)ks * WK / p.tile) * p.N + n0) * esz,
                    sbytes, bar);
          ++issued;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (++slot == kWmPacked) { slot = 0; phase ^= 1u; }
    }
    if (lane == 0 && *abort) {
      // Let copies that are still in flight land before the CTA gives up its shared memory.
      long pending = issued < kWmPacked ? issued : kWmPacked;
      int s2 = slot;
      uint32_t ph = phase;
      for (long i = 0; i < pending; ++i) {
        if (--s2 < 0) { s2 = kWmPacked - 1; ph ^= 1u; }
        for (int it = 0; it < 100000; ++it)
          if (mbar_try_wait(smem_u32(&ctl->pfull[s2]), ph)) break;
      }
    }
  } else if (warp >= kWmConvWarp0) {
    // ---------------- converters: packed int4 -> scaled bf16 in the swizzled weight half -------
    // Two groups of four warps take alternate units: a unit's chain (wait for the packed slot,
    // wait for the operand stage, convert, fence, arrive) is mostly barrier latency, and the two
    // chains overlap.
    const int group = (warp - kWmConvWarp0) / kWmGroupWarps;
    const int gt = threadIdx.x - (kWmConvWarp0 + group * kWmGroupWarps) * 32;      // 0..127
    const bool f32scale = p.scale_dtype == QWX_F32;
    bool ok = true;
    // a thread's four 16-byte pieces of a unit: quarter gt / 32 of the 128 K (one per warp), rows
    // gt % 32 + 32 h.  Eight neighbouring lanes then write eight different rows of one 16-byte
    // column, which the 128-byte swizzle spreads over all banks (rows x quarters per warp gave
    // 2-way conflicts on every store: 54 % of the shared-memory wavefronts).
    const int row0 = gt & 31, quarter = gt >> 5;
    for (long long u = u_begin + group; u < u_end && ok; u += kWmGroups) {
      const long long i = u - u_begin;
      const int tile = (int)(u / S);
      const int slot = (int)(i % kWmPacked), stage = (int)(i % Cfg::kStages);
      const uint32_t pphase = (uint32_t)((i / kWmPacked) & 1), phase = (uint32_t)((i / Cfg::kStages) & 1);
      if (!mbar_try_wait(smem_u32(&ctl->pfull[slot]), pphase)) {
        if (lane == 0) ok = mbar_wait(smem_u32(&ctl->pfull[slot]), pphase, abort);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      const uint8_t* src = packed_ptr + (size_t)slot * kWmSlotBytes;
      uint4 c[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) c[h] = reinterpret_cast<const uint4*>(src)[quarter * 128 + row0 + 32 * h];
      const int valid = (int)(p.N - (int64_t)tile * WT < WT ? p.N - (int64_t)tile * WT : WT);
      float t[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const int row = row0 + 32 * h;
        t[h] = 0.0f;
        if (row < valid)
          t[h] = f32scale ? reinterpret_cast<const float*>(src + kWmUnitBytes)[row]
                          : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src + kWmUnitBytes)[row]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->pempty[slot]));      // the slot's bytes are in registers

      if (!mbar_try_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u)) {
        if (lane == 0) ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      uint8_t* sw = ring_ptr + (size_t)stage * Cfg::kStageBytes + (quarter >> 1) * (WT * 128);
      const int chunk0 = (quarter & 1) * 4;
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const int row = row0 + 32 * h;
        const float s = t[h];
        const __nv_bfloat162 s2 = __float2bfloat162_rn(s);
        const uint32_t words[4] = {c[h].x, c[h].y, c[h].z, c[h].w};
        uint8_t* rowp = sw + row * 128;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const uint4 v = f32scale ? wm_convert<true>(words[w], s, s2) : wm_convert<false>(words[w], s, s2);
          *reinterpret_cast<uint4*>(rowp + (((chunk0 + w) ^ (row & 7)) << 4)) = v;
        }
      }
      fence_proxy_async();      // the tensor core reads these bytes through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->full[stage]));
    }
  } else {
    // ---------------- epilogue (warps 2-5) ----------------
    const int q = warp & 3;                     // tensor-memory lane quarter this warp may read
    const int nl = q * 32 + lane;               // channel inside the tile
    int acc = 0;
    uint32_t acc_phase = 0, epi_phase = 0;
    bool ok = true;

    auto emit = [&](int m, int64_t n, float v) {
      const int64_t o = (int64_t)m * p.N + n;
      if (p.out_dtype == QWX_F32) reinterpret_cast<float*>(p.out)[o] = v;
      else reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
    };
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      bool good = true;
      if (lane == 0) {
        mbar_arrive(smem_u32(&ctl->epi_bar));
        good = mbar_wait(smem_u32(&ctl->epi_bar), epi_phase, abort);
      }
      epi_phase ^= 1u;
      return __shfl_sync(0xffffffffu, good, 0);
    };

    long long u = u_begin;
    while (u < u_end && ok) {
      const int tile = (int)(u / S);
      const long long t_begin = (long long)tile * S, t_end = t_begin + S;
      const long long seg_end = t_end < u_end ? t_end : u_end;
      const int c_first = wm_cta_of_unit(t_begin, G, U);
      const int nseg = wm_cta_of_unit(t_end - 1, G, U) - c_first + 1;
      const int64_t n = (int64_t)tile * WT + nl;
      const bool n_ok = n < p.N;
      float* slot = p.ws + (size_t)c_first * (NT * WT) + nl;

      if (lane == 0) ok = mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < NT / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * NT + c * 32, r);
        tmem_ld_wait();
        if (!n_ok) continue;
        if (nseg == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c * 32 + j < p.M) emit(c * 32 + j, n, __uint_as_float(r[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c * 32 + j < p.M) atomicAdd(slot + (c * 32 + j) * WT, __uint_as_float(r[j]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }

      if (nseg > 1) {
        // publish this segment's share; the CTA that adds last finishes the tile
        __threadfence();
        ok = epi_sync();
        if (!ok) break;
        if (warp == 2 && lane == 0) {
          const int old = atomicAdd(p.counters + c_first, 1);
          ctl->last = (old == nseg - 1);
          if (old == nseg - 1) p.counters[c_first] = 0;
        }
        ok = epi_sync();
        if (!ok) break;
        if (ctl->last) {
          __threadfence();
          if (n_ok) {
#pragma unroll 1
            for (int c = 0; c * 32 < p.M; ++c) {
              float v[32];
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] = c * 32 + j < p.M ? __ldcg(slot + (c * 32 + j) * WT) : 0.0f;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (c * 32 + j < p.M) __stcg(slot + (c * 32 + j) * WT, 0.0f);
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (c * 32 + j < p.M) emit(c * 32 + j, n, v[j]);
            }
          }
        }
      }
      u = seg_end;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && ctl->abort && p.error_flag) atomicExch(p.error_flag, QWX_ERR_DEVICE_WAIT);
}

// Logical codes q[K, N] (one sign-extended code per byte) -> [N / 128][K / 128][4][128][16 B]:
// per 128 channels x 128 K, four quarters of 32 K, each holding 16 bytes (four 32-bit words of
// eight offset-binary nibbles) per channel; nibble i of a word holds K offset 2i for i < 4 and
// 2(i - 4) + 1 for i >= 4.  Channels past N hold zeros.
__global__ void pack_w4_tiles_kernel(const int8_t* __restrict__ q, int64_t K, int64_t N,
                                     uint32_t* __restrict__ out, int64_t words) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= words) return;
  const int word = (int)(i % 4) + 4 * (int)((i / (4 * WT)) % 4);    // word of the channel's 16
  const int row = (int)((i / 4) % WT);
  const int64_t unit = i / (16 * WT);
  const int64_t S = K / WK;
  const int64_t tile = unit / S, ks = unit % S;
  const int64_t n = tile * WT + row;
  const int64_t k0 = ks * WK + word * 8;
  uint32_t w = 0;
#pragma unroll
  for (int nib = 0; nib < 8; ++nib) {
    const int kofs = nib < 4 ? 2 * nib : 2 * (nib - 4) + 1;
    const int code = n < N ? (int)q[(k0 + kofs) * N + n] : 0;
    w |= (uint32_t)((code + 8) & 0xF) << (4 * nib);
  }
  out[i] = w;
}

int sm_count_wm() {
  static int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return v;
  }();
  return n;
}

template <int NT>
int launch_wm(const CUtensorMap& ta, const WmParams& p, int grid, cudaStream_t st) {
  auto kern = gemm_w4_mma_kernel<NT>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)wm_smem_bytes<NT>()) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  if (launch_dependent(kern, dim3(grid), dim3(kWmThreads), wm_smem_bytes<NT>(), st, ta, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return QWX_ERR_LAUNCH;
  }
  return QWX_OK;
}

}  // namespace
}  // namespace qwx

using namespace qwx;

extern "C" size_t qwx_w4_tiles_packed_bytes(int64_t K, int64_t N) {
  if (K <= 0 || N <= 0 || K % WK) return 0;
  return (size_t)((N + WT - 1) / WT) * (size_t)(K / WK) * kWmUnitBytes;
}

extern "C" int qwx_pack_w4_tiles(const void* q, int64_t K, int64_t N, void* packed, qwx_stream_t stream) {
  if (!q || !packed) return QWX_ERR_NULL;
  if (K <= 0 || N <= 0 || K % WK) return QWX_ERR_SHAPE;
  const int64_t words = (int64_t)(qwx_w4_tiles_packed_bytes(K, N) / 4);
  pack_w4_tiles_kernel<<<(unsigned)((words + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const int8_t*)q, K, N, (uint32_t*)packed, words);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

extern "C" size_t qwx_gemm_a16w4_mma_workspace_bytes(int64_t M, int64_t N) {
  if (M <= 0 || M > 128 || N <= 0) return 0;
  const int nt = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  return (size_t)kWmMaxGrid * nt * WT * sizeof(float) + (size_t)kWmMaxGrid * sizeof(int);
}

extern "C" int qwx_gemm_a16w4_mma(const void* a, const void* w_tiles, const void* scale, int scale_dtype,
                                  int64_t M, int64_t N, int64_t K, int64_t k_tile, void* out,
                                  int out_dtype, void* workspace, size_t workspace_bytes,
                                  int workspace_is_zero, int32_t* error_flag, qwx_stream_t stream) {
  if (!a || !w_tiles || !scale || !out || !workspace) return QWX_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (M > 128) return QWX_ERR_UNSUPPORTED;            // larger batches: call per 128 rows
  if (K % WK || N % 8) return QWX_ERR_UNSUPPORTED;     // whole stages; 16-byte runs of scales
  if (k_tile <= 0 || K % k_tile || k_tile % WK) return QWX_ERR_UNSUPPORTED;
  if (scale_dtype != QWX_F32 && scale_dtype != QWX_BF16) return QWX_ERR_DTYPE;
  if (out_dtype != QWX_BF16 && out_dtype != QWX_F32) return QWX_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w_tiles) & 15) ||
      (reinterpret_cast<uintptr_t>(workspace) & 15) || (reinterpret_cast<uintptr_t>(scale) & 15))
    return QWX_ERR_ALIGN;
  const size_t need = qwx_gemm_a16w4_mma_workspace_bytes(M, N);
  if (workspace_bytes < need) return QWX_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (!workspace_is_zero && cudaMemsetAsync(workspace, 0, need, st) != cudaSuccess) return QWX_ERR_LAUNCH;

  const int nt = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  CUtensorMap ta;
  if (!get_encode_tiled()) return QWX_ERR_NO_DEVICE;
  if (!encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, (uint64_t)M, (uint64_t)K, (uint32_t)nt, 64))
    return QWX_ERR_LAUNCH;
  const int sms = sm_count_wm();
  if (sms <= 0) return QWX_ERR_NO_DEVICE;
  WmParams p;
  p.M = (int)M; p.N = N; p.K = K;
  p.wp = reinterpret_cast<const uint4*>(w_tiles);
  p.scale = scale; p.scale_dtype = scale_dtype; p.tile = (int)k_tile;
  p.out = out; p.out_dtype = out_dtype; p.error_flag = error_flag;
  p.kstages = (int)(K / WK);
  const int64_t tiles = (N + WT - 1) / WT;
  p.units = tiles * p.kstages;
  if (tiles > INT32_MAX / 4) return QWX_ERR_SHAPE;
  int grid = sms < kWmMaxGrid ? sms : kWmMaxGrid;
  if ((long long)grid > p.units) grid = (int)p.units;
  p.ws = reinterpret_cast<float*>(workspace);
  p.counters = reinterpret_cast<int*>((char*)workspace + (size_t)kWmMaxGrid * nt * WT * sizeof(float));
  if (nt == 32) return launch_wm<32>(ta, p, grid, st);
  if (nt == 64) return launch_wm<64>(ta, p, grid, st);
  return launch_wm<128>(ta, p, grid, st);
}
