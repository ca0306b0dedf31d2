// Quantized GEMM with scales that change along K and zero-point corrections, on CTA pairs
// (tcgen05 cta_group::2), sm_100a.  Same contract as the single-CTA form in gemm_q8_tiled.cu:
//
//   out[m, n] = sum_t ( acc_t[m, n] - corr_row[m, t] * corr_col[t, n] ) * sa[m, t] * sb[t, n]
//   acc_t[m, n] = sum_{k in K tile t} a[m, k] * b[k, n]
//
// (qwix/_src/core/dot_general.py:187-203 tiled contraction, :228-253 zero-point terms, :255-259
// scale and sum over tiles, :278-399 the loop form.)  Two CTAs on the two SMs of a TPC compute
// one 256 x 256 output tile: each holds 128 rows of A and 128 columns of B per K block (32 KB
// instead of the 32 KB a 128 x 128 tile needs for a quarter of the products), and 128
// accumulator rows x 256 columns in tensor memory, twice: the tensor cores fill one
// accumulator with K tile t+1 while the epilogue warps drain K tile t from the other.
//
// The epilogue is the pace-setter when the K tile is short, so it is written for issue slots:
//   * eight epilogue warps per CTA, two per tensor-memory lane quarter, 128 columns each; a
//     thread owns one output row and keeps 128 running float32 sums in registers (the
//     register file is re-split with setmaxnreg: 232 per epilogue thread, 40 per control thread);
//   * the variant is a template parameter, not a run-time branch in the inner loop;
//   * int32 -> float32 through the exact magic-number add where |acc| < 2^22 is guaranteed;
//   * the three float operations per value (subtract the magic, times sa, multiply-add with
//     sb) are the packed two-lane forms (add/mul/fma .f32x2), rounding as the scalar forms do;
//   * scales of a K tile are staged per warp in shared memory by the lanes that prefetched
//     them one K tile ahead, and read back four at a time.
//
// Per CTA: warp 0 TMA producer, warp 1 MMA issuer (even CTA only), warp 2 owns the pair's
// tensor-memory allocation, warps 4-11 epilogue.  Barriers as in gemm_q8_pair.cu, acc_full once
// per K tile.  Every wait is bounded; both CTAs always reach the closing cluster barrier.

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

constexpr int QM = 128;        // rows per CTA (256 per pair)
constexpr int QN = 256;        // columns per pair
constexpr int QNH = 128;       // columns of B held by one CTA; also the columns one epilogue warp drains
constexpr int QK = 128;        // one 128-byte swizzle row of 8-bit codes
constexpr int QUMMA_K = 32;
constexpr int kQStages = 6;
constexpr int kQABytes = QM * QK;
constexpr int kQBBytes = QNH * QK;
constexpr int kQStageBytes = kQABytes + kQBBytes;
constexpr int kQThreads = 384;       // one control warpgroup + two epilogue warpgroups
constexpr int kQEpiWarp0 = 4;
constexpr int kQEpiWarps = 8;
constexpr int kQRegsControl = 40;
constexpr int kQRegsEpilogue = 232;

// Epilogue variants (template parameter).
constexpr int kModeFast = 0;       // int8, |acc| < 2^22, no zero points: magic-number conversion
constexpr int kModeCvt = 1;        // cvt (int8) or float accumulators, no zero points
constexpr int kModeCorr = 2;       // int8 with the rank-1 zero-point term, cvt
constexpr int kModeRef = 3;        // the reference's rounding after every step
constexpr int kModeRefCorr = 4;

struct ControlQ {
  uint64_t full[kQStages];
  uint64_t empty[kQStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort;
  alignas(16) float sb[kQEpiWarps][2][QNH];    // per epilogue warp, double-buffered per K tile
  alignas(16) int32_t zc[kQEpiWarps][2][QNH];
};

constexpr size_t kQSmemBytes = 1024 + (size_t)kQStages * kQStageBytes + sizeof(ControlQ);
static_assert(kQSmemBytes <= 227 * 1024, "shared memory of the pair-tiled kernel");

struct TiledPairParams {
  int64_t M, N, K;
  int kb_per_tile;          // K blocks of 128 per scale tile
  int T;                    // number of K tiles
  const void* sa;           // [M, T] if sa_tiled else [M]; may be null
  const void* sb;           // [T, N] if sb_tiled else [N]; may be null
  int sa_tiled, sb_tiled;
  int scale_dtype;
  const int32_t* corr_row;  // [M, T] or null
  const int32_t* corr_col;  // [T, N] or null
  void* out;
  int out_dtype;
  int32_t* error_flag;
  int tiles_m, tiles_n;     // 256 x 256 tiles
};

__device__ __forceinline__ float load_scale_q(const void* p, int dtype, int64_t i) {
  if (dtype == QWX_F32) return __ldg(reinterpret_cast<const float*>(p) + i);
  if (dtype == QWX_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ float round_out_q(float v, int out_dtype) {
  if (out_dtype == QWX_BF16) return round_to<BF16>(v);
  if (out_dtype == QWX_F16) return round_to<F16>(v);
  return v;
}

template <int REGS>
__device__ __forceinline__ void regs_release() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}
template <int REGS>
__device__ __forceinline__ void regs_claim() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}

// One 32-column chunk of one K tile folded into the running sums v[0..16) (float2 each).
template <MmaKind KIND, int MODE>
__device__ __forceinline__ void fold_chunk(const uint32_t (&r)[32], const float* __restrict__ sbv,
                                           const int32_t* __restrict__ zcv, float sa, int32_t zr,
                                           int out_dtype, float2* v) {
  const float4* s4 = reinterpret_cast<const float4*>(sbv);
  const int4* z4 = reinterpret_cast<const int4*>(zcv);
  const float2 sa2 = make_float2(sa, sa);
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const float4 s = s4[g];
    int32_t x[4] = {(int32_t)r[4 * g], (int32_t)r[4 * g + 1], (int32_t)r[4 * g + 2],
                    (int32_t)r[4 * g + 3]};
    if (MODE == kModeCorr || MODE == kModeRefCorr) {
      const int4 z = z4[g];
      x[0] -= zr * z.x; x[1] -= zr * z.y; x[2] -= zr * z.z; x[3] -= zr * z.w;
    }
    float2 f0, f1;
    if (KIND != MmaKind::kI8) {
      f0 = make_float2(__uint_as_float(r[4 * g]), __uint_as_float(r[4 * g + 1]));
      f1 = make_float2(__uint_as_float(r[4 * g + 2]), __uint_as_float(r[4 * g + 3]));
    } else if (MODE == kModeFast) {
      const float2 magic = make_float2(-12582912.0f, -12582912.0f);
      f0 = __fadd2_rn(make_float2(__int_as_float(0x4B400000 + x[0]), __int_as_float(0x4B400000 + x[1])), magic);
      f1 = __fadd2_rn(make_float2(__int_as_float(0x4B400000 + x[2]), __int_as_float(0x4B400000 + x[3])), magic);
    } else {
      f0 = make_float2((float)x[0], (float)x[1]);
      f1 = make_float2((float)x[2], (float)x[3]);
    }
    if (MODE == kModeRef || MODE == kModeRefCorr) {
      float f[4] = {f0.x, f0.y, f1.x, f1.y};
      const float sv[4] = {s.x, s.y, s.z, s.w};
      float* vs = reinterpret_cast<float*>(v + 2 * g);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f[i] = round_out_q(f[i], out_dtype);
        f[i] = round_out_q(__fmul_rn(f[i], sa), out_dtype);
        f[i] = round_out_q(__fmul_rn(f[i], sv[i]), out_dtype);
        vs[i] = __fadd_rn(vs[i], f[i]);
      }
    } else {
      v[2 * g] = __ffma2_rn(__fmul2_rn(f0, sa2), make_float2(s.x, s.y), v[2 * g]);
      v[2 * g + 1] = __ffma2_rn(__fmul2_rn(f1, sa2), make_float2(s.z, s.w), v[2 * g + 1]);
    }
  }
}

template <MmaKind KIND, int BLAYOUT, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kQThreads, 1)
gemm_q8_tiled_pair_kernel(const __grid_constant__ CUtensorMap tma_a,
                          const __grid_constant__ CUtensorMap tma_b, const TiledPairParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  ControlQ* ctl = reinterpret_cast<ControlQ*>(smem_raw + (tiles - smem_u32(smem_raw)) +
                                              (size_t)kQStages * kQStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: issues the MMAs
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = p.T * p.kb_per_tile;
  volatile int* abort = &ctl->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->acc_full[a]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[a]), 2 * kQEpiWarps);
    }
    ctl->abort = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
  }
  if (warp == 2) {
    tmem_alloc_pair(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // the peer's barriers are initialised before anything arrives there
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp < kQEpiWarp0) {
    regs_release<kQRegsControl>();
    if (warp == 0) {
      // ---------------- TMA producer: this CTA's halves of A and B ----------------
      int stage = 0;
      uint32_t phase = 0;
      long issued = 0;
      bool ok = true;
      const uint32_t full0 = map_to_cta(smem_u32(&ctl->full[0]), 0);   // the even CTA's barriers
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile % p.tiles_m) * (2 * QM) + (int)rank * QM;
        const int n0 = (tile / p.tiles_m) * QN + (int)rank * QNH;
        for (int kb = 0; kb < kblocks && ok; ++kb) {
          if (lane == 0) {
            ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort);
            if (ok) {
              const uint32_t sa = tiles + stage * kQStageBytes;
              const uint32_t sb = sa + kQABytes;
              if (rank == 0) mbar_expect_tx(smem_u32(&ctl->full[stage]), 2 * kQStageBytes);
              const uint32_t bar = full0 + stage * 8;
              tma_load_2d_pair(sa, &tma_a, kb * QK, m0, bar);
              if (BLAYOUT == QWX_B_NK) tma_load_2d_pair(sb, &tma_b, kb * QK, n0, bar);
              else tma_load_2d_pair(sb, &tma_b, n0, kb * QK, bar);
              ++issued;
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (++stage == kQStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (lane == 0 && *abort && rank == 0) {
        // Let copies that are still in flight land before the CTA gives up its shared memory.
        long pending = issued < kQStages ? issued : kQStages;
        int s = stage;
        uint32_t ph = phase;
        for (long i = 0; i < pending; ++i) {
          if (--s < 0) { s = kQStages - 1; ph ^= 1u; }
          for (int it = 0; it < 100000; ++it)
            if (mbar_try_wait(smem_u32(&ctl->full[s]), ph)) break;
        }
      }
    } else if (warp == 1 && rank == 0) {
      // ---------------- MMA issuer (even CTA): one accumulator per (output tile, K tile) -------
      constexpr uint32_t idesc =
          KIND == MmaKind::kI8
              ? make_idesc(2, 1, 1, 0, BLAYOUT == QWX_B_KN ? 1 : 0, 2 * QM, QN)
              : make_idesc(1, 0, 0, 0, BLAYOUT == QWX_B_KN ? 1 : 0, 2 * QM, QN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t empty_peer = map_to_cta(smem_u32(&ctl->empty[0]), 1);
      const uint32_t acc_full_peer = map_to_cta(smem_u32(&ctl->acc_full[0]), 1);
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        for (int t = 0; t < p.T && ok; ++t) {
          if (lane == 0) {
            ok = mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort);
            tc_fence_after();
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          for (int kb = 0; kb < p.kb_per_tile && ok; ++kb) {
            if (lane == 0) {
              ok = mbar_wait(smem_u32(&ctl->full[stage]), phase, abort);
              if (ok) {
                tc_fence_after();
                const uint32_t sa = tiles + stage * kQStageBytes;
                const uint32_t sb = sa + kQABytes;
#pragma unroll
                for (int kk = 0; kk < QK / QUMMA_K; ++kk) {
                  const uint64_t da = make_smem_desc(sa + kk * QUMMA_K, 16, 1024);
                  const uint64_t db = BLAYOUT == QWX_B_NK
                                          ? make_smem_desc(sb + kk * QUMMA_K, 16, 1024)
                                          : make_smem_desc(sb + kk * QUMMA_K * 128, QK * 128, 1024);
                  mma_ss_pair<KIND>(tmem_base + acc * QN, da, db, idesc, kb != 0 || kk != 0);
                }
                mma_commit_pair(smem_u32(&ctl->empty[stage]));
                mma_commit_pair(empty_peer + stage * 8);
                if (kb == p.kb_per_tile - 1) {
                  mma_commit_pair(smem_u32(&ctl->acc_full[acc]));
                  mma_commit_pair(acc_full_peer + acc * 8);
                }
              }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (++stage == kQStages) { stage = 0; phase ^= 1u; }
          }
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
      }
    }
  } else {
    // ---------------- epilogue: drain one accumulator per K tile, keep running sums -----------
    regs_claim<kQRegsEpilogue>();
    const int ew = warp - kQEpiWarp0;         // epilogue warp 0..7
    const int q = warp & 3;                   // tensor-memory lane quarter of this warp
    const int ch = ew >> 2;                   // which 128 columns of the tile
    constexpr bool kCorr = MODE == kModeCorr || MODE == kModeRefCorr;
    const uint32_t acc_empty0 = map_to_cta(smem_u32(&ctl->acc_empty[0]), 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;

    // Scales and correction factors of one (output tile, K tile): four consecutive columns
    // per lane for the warp's shared copy, one row value per lane.
    struct Prefetch {
      float sb[4];
      int32_t zc[4];
      float sa;
      int32_t zr;
    };
    auto fetch = [&](int tile, int t) {
      Prefetch f;
      const int m0 = (tile % p.tiles_m) * (2 * QM) + (int)rank * QM;
      const int n0 = (tile / p.tiles_m) * QN + ch * QNH;
      const int64_t m = (int64_t)m0 + q * 32 + lane;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int64_t n = (int64_t)n0 + lane * 4 + i;
        const bool in = n < p.N;
        f.sb[i] = (p.sb && in) ? load_scale_q(p.sb, p.scale_dtype, (p.sb_tiled ? (int64_t)t * p.N : 0) + n)
                               : 1.0f;
        f.zc[i] = (kCorr && in) ? __ldg(p.corr_col + (int64_t)t * p.N + n) : 0;
      }
      const bool rin = m < p.M;
      f.sa = (p.sa && rin) ? load_scale_q(p.sa, p.scale_dtype, p.sa_tiled ? m * p.T + t : m) : 1.0f;
      f.zr = (kCorr && rin) ? __ldg(p.corr_row + m * p.T + t) : 0;
      return f;
    };

    int tile = pair, t = 0, it = 0;
    bool have = tile < num_tiles;
    Prefetch pf;
    if (have) pf = fetch(tile, t);
    float2 v[QNH / 2];

    while (have && ok) {
      const int buf = it & 1;
      *reinterpret_cast<float4*>(&ctl->sb[ew][buf][lane * 4]) =
          make_float4(pf.sb[0], pf.sb[1], pf.sb[2], pf.sb[3]);
      if (kCorr)
        *reinterpret_cast<int4*>(&ctl->zc[ew][buf][lane * 4]) =
            make_int4(pf.zc[0], pf.zc[1], pf.zc[2], pf.zc[3]);
      const float sa = pf.sa;
      const int32_t zr = pf.zr;
      __syncwarp();
      int ntile = tile, nt = t + 1;
      if (nt == p.T) { nt = 0; ntile += num_pairs; }
      const bool nhave = ntile < num_tiles;
      if (nhave) pf = fetch(ntile, nt);   // in flight while this K tile is drained

      if (lane == 0) ok = mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();

      if (t == 0) {
#pragma unroll
        for (int j = 0; j < QNH / 2; ++j) v[j] = make_float2(0.0f, 0.0f);
      }
      const float* sbv = ctl->sb[ew][buf];
      const int32_t* zcv = ctl->zc[ew][buf];
#pragma unroll
      for (int c = 0; c < QNH / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * QN + ch * QNH + c * 32, r);
        tmem_ld_wait();
        fold_chunk<KIND, MODE>(r, sbv + c * 32, zcv + c * 32, sa, zr, p.out_dtype, v + c * 16);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty0 + acc * 8);

      if (t == p.T - 1) {
        const int m0 = (tile % p.tiles_m) * (2 * QM) + (int)rank * QM;
        const int n0 = (tile / p.tiles_m) * QN + ch * QNH;
        const int64_t m = (int64_t)m0 + q * 32 + lane;
        if (m < p.M) {
#pragma unroll
          for (int c = 0; c < QNH / 32; ++c) {
            const int64_t ncol = (int64_t)n0 + c * 32;
            if (ncol >= p.N) break;
            const float* vc = reinterpret_cast<const float*>(v + c * 16);
            if (p.out_dtype == QWX_F32) {
              float* o = reinterpret_cast<float*>(p.out) + m * p.N + ncol;
              if (ncol + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  *reinterpret_cast<float4*>(o + j) = make_float4(vc[j], vc[j + 1], vc[j + 2], vc[j + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (ncol + j < p.N) o[j] = vc[j];
              }
            } else {
              uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + m * p.N + ncol;
              uint32_t w[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (p.out_dtype == QWX_BF16) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(vc[2 * j], vc[2 * j + 1]);
                  w[j] = *reinterpret_cast<uint32_t*>(&h);
                } else {
                  __half2 h = __floats2half2_rn(vc[2 * j], vc[2 * j + 1]);
                  w[j] = *reinterpret_cast<uint32_t*>(&h);
                }
              }
              if (ncol + 32 <= p.N && (p.N & 7) == 0) {
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                  *reinterpret_cast<uint4*>(o + 2 * j) = make_uint4(w[j], w[j + 1], w[j + 2], w[j + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (ncol + j < p.N) o[j] = (uint16_t)(w[j >> 1] >> ((j & 1) * 16));
              }
            }
          }
        }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      tile = ntile;
      t = nt;
      have = nhave;
      ++it;
    }
  }

  // Neither CTA may leave (or free tensor memory) while the other can still read its
  // accumulators or arrive on its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
  if (threadIdx.x == 0 && ctl->abort && p.error_flag) atomicExch(p.error_flag, QWX_ERR_DEVICE_WAIT);
}

template <MmaKind KIND, int BLAYOUT, int MODE>
int launch_tiled_pair(const CUtensorMap& ta, const CUtensorMap& tb, const TiledPairParams& p,
                      int grid, cudaStream_t st) {
  auto kern = gemm_q8_tiled_pair_kernel<KIND, BLAYOUT, MODE>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kQSmemBytes) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  kern<<<grid, kQThreads, kQSmemBytes, st>>>(ta, tb, p);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

template <MmaKind KIND, int MODE>
int launch_tiled_pair_layout(int b_layout, const CUtensorMap& ta, const CUtensorMap& tb,
                             const TiledPairParams& p, int grid, cudaStream_t st) {
  return b_layout == QWX_B_NK ? launch_tiled_pair<KIND, QWX_B_NK, MODE>(ta, tb, p, grid, st)
                              : launch_tiled_pair<KIND, QWX_B_KN, MODE>(ta, tb, p, grid, st);
}

}  // namespace

// Launches the CTA-pair form; the caller has validated the arguments (see qwx_gemm_q8_tiled).
int gemm_q8_tiled_pair_launch(const void* a, const void* b, int code_dtype, int b_layout,
                              int64_t M, int64_t N, int64_t K, int64_t k_tile, const void* sa,
                              int sa_tiled, const void* sb, int sb_tiled, int scale_dtype,
                              const int32_t* corr_row, const int32_t* corr_col, void* out,
                              int out_dtype, int epilogue, int32_t* error_flag, int sms,
                              cudaStream_t st) {
  CUtensorMap ta, tb;
  if (!get_encode_tiled()) return QWX_ERR_NO_DEVICE;
  if (!encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)M, (uint64_t)K, QM, QK))
    return QWX_ERR_LAUNCH;
  const bool ok_b = b_layout == QWX_B_NK
                        ? encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)N, (uint64_t)K, QNH, QK)
                        : encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)K, (uint64_t)N, QK, QNH);
  if (!ok_b) return QWX_ERR_LAUNCH;

  TiledPairParams p;
  p.M = M; p.N = N; p.K = K;
  p.T = (int)(K / k_tile);
  p.kb_per_tile = (int)((k_tile + QK - 1) / QK);
  p.sa = sa; p.sb = sb;
  p.sa_tiled = sa_tiled && p.T > 1; p.sb_tiled = sb_tiled && p.T > 1;
  p.scale_dtype = scale_dtype;
  p.corr_row = corr_row; p.corr_col = corr_col;
  p.out = out; p.out_dtype = out_dtype;
  p.error_flag = error_flag;
  p.tiles_m = (int)((M + 2 * QM - 1) / (2 * QM));
  p.tiles_n = (int)((N + QN - 1) / QN);
  const int64_t num_tiles = (int64_t)p.tiles_m * p.tiles_n;
  if (num_tiles > INT32_MAX / 2) return QWX_ERR_SHAPE;
  const int64_t pairs = num_tiles < sms / 2 ? num_tiles : sms / 2;
  const int grid = (int)(2 * pairs);
  const bool reference = epilogue == QWX_EPI_REFERENCE;
  const bool corr = corr_row != nullptr;
  if (code_dtype == QWX_S8) {
    // int8 products over at most 256 codes stay within [-2^22, 2^22]: the magic-number
    // conversion is exact there.  A zero-point term can leave that range, so it keeps cvt.
    const bool fast = k_tile <= 256 && !corr && !reference;
    if (fast) return launch_tiled_pair_layout<MmaKind::kI8, kModeFast>(b_layout, ta, tb, p, grid, st);
    if (reference)
      return corr ? launch_tiled_pair_layout<MmaKind::kI8, kModeRefCorr>(b_layout, ta, tb, p, grid, st)
                  : launch_tiled_pair_layout<MmaKind::kI8, kModeRef>(b_layout, ta, tb, p, grid, st);
    return corr ? launch_tiled_pair_layout<MmaKind::kI8, kModeCorr>(b_layout, ta, tb, p, grid, st)
                : launch_tiled_pair_layout<MmaKind::kI8, kModeCvt>(b_layout, ta, tb, p, grid, st);
  }
  return reference ? launch_tiled_pair_layout<MmaKind::kF8F6F4, kModeRef>(b_layout, ta, tb, p, grid, st)
                   : launch_tiled_pair_layout<MmaKind::kF8F6F4, kModeCvt>(b_layout, ta, tb, p, grid, st);
}

}  // namespace qwx
