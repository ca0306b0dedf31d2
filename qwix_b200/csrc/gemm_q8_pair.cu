// Quantized GEMM on CTA pairs (tcgen05 cta_group::2), sm_100a: the same product and epilogue as
// the single-CTA kernel,
//
//   out[m, n] = (sum_k a[m, k] * b[k, n]) * sa[m] * sb[n]      (dot_general.py:220, :255-258)
//
// for problems with at least two 128-row tiles.  Two CTAs of a cluster, on the two SMs of a
// TPC, compute one 256 x 256 output tile: each keeps 128 rows of A and 128 columns of B in its
// shared memory and 128 accumulator rows in its tensor memory, and the even CTA issues one
// M = 256 MMA for both.  What this buys is traffic: a CTA fetches 32 KB per 128-wide K block
// instead of 48 KB, and the single-CTA kernel is held back by the L2 -> shared-memory rate
// (148 SMs x 48 KB per 512 cycles), not by the tensor pipe.
//
// Per CTA: warp 0 TMA producer (its own halves; every load counts on the even CTA's `full`
// barrier), warp 1 MMA issuer (even CTA only), warp 2 owns the pair's tensor-memory
// allocation, warps 4-7 epilogue of the CTA's 128 rows.  Barriers:
//   full[s]      even CTA: 1 arrival (its producer, with the byte count of both CTAs' loads)
//   empty[s]     each CTA: commit of the MMAs that read stage s (the even CTA commits to both)
//   acc_full[a]  each CTA: commit of a tile's last MMA (the even CTA commits to both)
//   acc_empty[a] even CTA: the eight epilogue warps of the pair
// Every mbarrier wait is bounded; both CTAs always reach the closing cluster barrier.

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

constexpr int PM = 128;        // rows per CTA (256 per pair)
constexpr int PN = 256;        // columns per pair
constexpr int PNH = 128;       // columns of B held by one CTA
constexpr int PK = 128;        // bytes == elements for 8-bit codes: one 128-byte swizzle row
constexpr int PUMMA_K = 32;
constexpr int kPStages = 3;       // a stage holds two 128-wide K blocks: one barrier round trip per 256 K
constexpr int kPABytes = PM * PK;
constexpr int kPBBytes = PNH * PK;
constexpr int kPStageBytes = 2 * (kPABytes + kPBBytes);   // per CTA: [A k0][A k1][B k0][B k1]
constexpr int kPThreads = 256;
constexpr int kPEpiWarp0 = 4;

struct ControlP {
  uint64_t full[kPStages];
  uint64_t empty[kPStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort;
  float sb[4][2][PN];  // per epilogue warp, per accumulator
};

constexpr size_t kPSmemBytes = 1024 + (size_t)kPStages * kPStageBytes + sizeof(ControlP);

struct PairParams {
  int64_t M, N, K;
  const void* sa;
  const void* sb;
  int scale_dtype;
  void* out;
  int out_dtype;
  int epilogue;
  int32_t* error_flag;
  int tiles_m, tiles_n;    // 256 x 256 tiles
};

__device__ __forceinline__ float load_scale_p(const void* p, int dtype, int64_t i) {
  if (dtype == QWX_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == QWX_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ float round_out_p(float v, int out_dtype) {
  if (out_dtype == QWX_BF16) return round_to<BF16>(v);
  if (out_dtype == QWX_F16) return round_to<F16>(v);
  return v;
}

template <MmaKind KIND, int BLAYOUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPThreads, 1)
gemm_q8_pair_kernel(const __grid_constant__ CUtensorMap tma_a,
                    const __grid_constant__ CUtensorMap tma_b, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  ControlP* ctl = reinterpret_cast<ControlP*>(smem_raw + (tiles - smem_u32(smem_raw)) +
                                              (size_t)kPStages * kPStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: issues the MMAs
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int kblocks = (int)((p.K + 2 * PK - 1) / (2 * PK));   // stages of 256 K; a ragged tail reads zeros
  const int num_tiles = p.tiles_m * p.tiles_n;
  volatile int* abort = &ctl->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->acc_full[a]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[a]), 8);
    }
    ctl->abort = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
  }
  if (warp == 2) {
    // both CTAs of the pair issue the allocation, from the same warp and to the same offset
    tmem_alloc_pair(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // the peer's barriers are initialised before anything arrives there
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's halves of A and B ----------------
    int stage = 0;
    uint32_t phase = 0;
    long issued = 0;
    bool ok = true;
    const uint32_t full0 = map_to_cta(smem_u32(&ctl->full[0]), 0);   // the even CTA's barriers
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int m0 = (tile % p.tiles_m) * (2 * PM) + (int)rank * PM;
      const int n0 = (tile / p.tiles_m) * PN + (int)rank * PNH;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort);
          if (ok) {
            const uint32_t sa = tiles + stage * kPStageBytes;
            const uint32_t sb = sa + 2 * kPABytes;
            if (rank == 0) mbar_expect_tx(smem_u32(&ctl->full[stage]), 2 * kPStageBytes);
            const uint32_t bar = full0 + stage * 8;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int k0 = (2 * kb + h) * PK;
              tma_load_2d_pair(sa + h * kPABytes, &tma_a, k0, m0, bar);
              if (BLAYOUT == QWX_B_NK) tma_load_2d_pair(sb + h * kPBBytes, &tma_b, k0, n0, bar);
              else tma_load_2d_pair(sb + h * kPBBytes, &tma_b, n0, k0, bar);
            }
            ++issued;
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == kPStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (lane == 0 && *abort && rank == 0) {
      // Let copies that are still in flight land before the CTA gives up its shared memory.
      long pending = issued < kPStages ? issued : kPStages;
      int s = stage;
      uint32_t ph = phase;
      for (long i = 0; i < pending; ++i) {
        if (--s < 0) { s = kPStages - 1; ph ^= 1u; }
        for (int it = 0; it < 100000; ++it)
          if (mbar_try_wait(smem_u32(&ctl->full[s]), ph)) break;
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ---------------- MMA issuer (even CTA): M = 256 over the pair ----------------
    constexpr uint32_t idesc =
        KIND == MmaKind::kI8
            ? make_idesc(2, 1, 1, 0, BLAYOUT == QWX_B_KN ? 1 : 0, 2 * PM, PN)
            : make_idesc(1, 0, 0, 0, BLAYOUT == QWX_B_KN ? 1 : 0, 2 * PM, PN);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const uint32_t empty_peer = map_to_cta(smem_u32(&ctl->empty[0]), 1);
    const uint32_t acc_full_peer = map_to_cta(smem_u32(&ctl->acc_full[0]), 1);
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort);
        tc_fence_after();
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&ctl->full[stage]), phase, abort);
          if (ok) {
            tc_fence_after();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t sa = tiles + stage * kPStageBytes + h * kPABytes;
              const uint32_t sb = tiles + stage * kPStageBytes + 2 * kPABytes + h * kPBBytes;
#pragma unroll
              for (int kk = 0; kk < PK / PUMMA_K; ++kk) {
                const uint64_t da = make_smem_desc(sa + kk * PUMMA_K, 16, 1024);
                const uint64_t db = BLAYOUT == QWX_B_NK
                                        ? make_smem_desc(sb + kk * PUMMA_K, 16, 1024)
                                        : make_smem_desc(sb + kk * PUMMA_K * 128, PK * 128, 1024);
                mma_ss_pair<KIND>(tmem_base + acc * PN, da, db, idesc, kb != 0 || h != 0 || kk != 0);
              }
            }
            mma_commit_pair(smem_u32(&ctl->empty[stage]));
            mma_commit_pair(empty_peer + stage * 8);
            if (kb == kblocks - 1) {
              mma_commit_pair(smem_u32(&ctl->acc_full[acc]));
              mma_commit_pair(acc_full_peer + acc * 8);
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == kPStages) { stage = 0; phase ^= 1u; }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  } else if (warp >= kPEpiWarp0) {
    // ---------------- epilogue of this CTA's 128 rows ----------------
    const int q = warp - kPEpiWarp0;           // tensor-memory lane quarter of this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool reference = p.epilogue == QWX_EPI_REFERENCE;
    const uint32_t acc_empty0 = map_to_cta(smem_u32(&ctl->acc_empty[0]), 0);
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int m0 = (tile % p.tiles_m) * (2 * PM) + (int)rank * PM;
      const int n0 = (tile / p.tiles_m) * PN;
      for (int j = lane; j < PN; j += 32) {
        const int64_t n = (int64_t)n0 + j;
        ctl->sb[q][acc][j] = (p.sb && n < p.N) ? load_scale_p(p.sb, p.scale_dtype, n) : 1.0f;
      }
      __syncwarp();
      const int64_t m = (int64_t)m0 + q * 32 + lane;
      const float sa = (p.sa && m < p.M) ? load_scale_p(p.sa, p.scale_dtype, m) : 1.0f;

      if (lane == 0) ok = mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();

#pragma unroll 1
      for (int c = 0; c < PN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * PN + c * 32, r);
        tmem_ld_wait();
        const int64_t ncol = (int64_t)n0 + c * 32;
        if (m >= p.M || ncol >= p.N) continue;
        const float* sbv = &ctl->sb[q][acc][c * 32];
        if (p.out_dtype == QWX_S32) {
          int32_t* o = reinterpret_cast<int32_t*>(p.out) + m * p.N + ncol;
          if (ncol + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<uint4*>(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
          } else {
            for (int j = 0; j < 32 && ncol + j < p.N; ++j) o[j] = (int32_t)r[j];
          }
          continue;
        }
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float a = KIND == MmaKind::kI8 ? (float)(int32_t)r[j] : __uint_as_float(r[j]);
          if (reference) {
            a = round_out_p(a, p.out_dtype);
            a = round_out_p(__fmul_rn(a, sa), p.out_dtype);
            a = round_out_p(__fmul_rn(a, sbv[j]), p.out_dtype);
          } else {
            a = __fmul_rn(__fmul_rn(a, sa), sbv[j]);
          }
          v[j] = a;
        }
        if (p.out_dtype == QWX_F32) {
          float* o = reinterpret_cast<float*>(p.out) + m * p.N + ncol;
          if (ncol + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
            for (int j = 0; j < 32 && ncol + j < p.N; ++j) o[j] = v[j];
          }
        } else {
          uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + m * p.N + ncol;
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (p.out_dtype == QWX_BF16) {
              __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
              w[j] = *reinterpret_cast<uint32_t*>(&h);
            } else {
              __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
              w[j] = *reinterpret_cast<uint32_t*>(&h);
            }
          }
          if (ncol + 32 <= p.N && (p.N & 7) == 0) {
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              *reinterpret_cast<uint4*>(o + 2 * j) = make_uint4(w[j], w[j + 1], w[j + 2], w[j + 3]);
          } else {
            for (int j = 0; j < 32 && ncol + j < p.N; ++j)
              o[j] = (uint16_t)(w[j >> 1] >> ((j & 1) * 16));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty0 + acc * 8);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
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

template <MmaKind KIND, int BLAYOUT>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const PairParams& p, int grid,
                cudaStream_t st) {
  auto kern = gemm_q8_pair_kernel<KIND, BLAYOUT>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kPSmemBytes) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  kern<<<grid, kPThreads, kPSmemBytes, st>>>(ta, tb, p);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

}  // namespace

// Launches the CTA-pair kernel; the caller has validated the arguments (see qwx_gemm_q8).
int gemm_q8_pair_launch(const void* a, const void* b, int code_dtype, int b_layout, int64_t M,
                        int64_t N, int64_t K, const void* sa, const void* sb, int scale_dtype,
                        void* out, int out_dtype, int epilogue, int32_t* error_flag, int sms,
                        cudaStream_t st) {
  CUtensorMap ta, tb;
  if (!get_encode_tiled()) return QWX_ERR_NO_DEVICE;
  if (!encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)M, (uint64_t)K, PM, PK))
    return QWX_ERR_LAUNCH;
  const bool ok_b = b_layout == QWX_B_NK
                        ? encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)N, (uint64_t)K, PNH, PK)
                        : encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)K, (uint64_t)N, PK, PNH);
  if (!ok_b) return QWX_ERR_LAUNCH;
  PairParams p;
  p.M = M; p.N = N; p.K = K;
  p.sa = sa; p.sb = sb; p.scale_dtype = scale_dtype;
  p.out = out; p.out_dtype = out_dtype; p.epilogue = epilogue;
  p.error_flag = error_flag;
  p.tiles_m = (int)((M + 2 * PM - 1) / (2 * PM));
  p.tiles_n = (int)((N + PN - 1) / PN);
  const int64_t num_tiles = (int64_t)p.tiles_m * p.tiles_n;
  if (num_tiles > INT32_MAX / 2) return QWX_ERR_SHAPE;
  const int64_t pairs = num_tiles < sms / 2 ? num_tiles : sms / 2;
  const int grid = (int)(2 * pairs);
  if (code_dtype == QWX_S8) {
    return b_layout == QWX_B_NK ? launch_pair<MmaKind::kI8, QWX_B_NK>(ta, tb, p, grid, st)
                                : launch_pair<MmaKind::kI8, QWX_B_KN>(ta, tb, p, grid, st);
  }
  return b_layout == QWX_B_NK ? launch_pair<MmaKind::kF8F6F4, QWX_B_NK>(ta, tb, p, grid, st)
                              : launch_pair<MmaKind::kF8F6F4, QWX_B_KN>(ta, tb, p, grid, st);
}

}  // namespace qwx
