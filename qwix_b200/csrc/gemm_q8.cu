// Quantized GEMM for 8-bit codes on tcgen05 tensor cores with the dequant fused in the
// epilogue: the device side of dot_general._fast_dot_general (dot_general.py:135-261).
//
//   out[m, n] = convert( acc[m, n] * sa[m] * sb[n] ),  acc = sum_k a[m, k] * b[k, n]
//
// int8 x int8 -> int32 (kind::i8) and e4m3 x e4m3 -> float32 (kind::f8f6f4).
//
// Structure (one persistent CTA per SM, 256 threads):
//   warp 0      TMA producer: A [128 x 128B] and B [256 x 128B] tiles, 128-byte swizzle, into a
//               4-stage shared-memory ring guarded by full/empty mbarriers
//   warp 1      MMA issuer: one elected thread issues 4 x tcgen05.mma (M128 N256 K32) per stage,
//               accumulating in tensor memory; tcgen05.commit releases the stage
//   warp 2      allocates / frees the 512 tensor-memory columns (two 128x256 accumulators)
//   warps 4-7   epilogue: tcgen05.ld 32 lanes x 32 columns at a time, scale, convert, store;
//               runs on accumulator i while the MMA warp fills accumulator i^1
// B may be [N, K] (K-major operand) or qwix's native [K, N] (MN-major operand, no repack).
#include "common.cuh"
#include "sm100.cuh"

namespace qwx {
namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;       // bytes == elements for 8-bit codes: one 128-byte swizzle row
constexpr int UMMA_K = 32;    // K per tcgen05.mma for 8-bit operands
constexpr int kStages = 4;
constexpr int kABytes = BM * BK;
constexpr int kBBytes = BN * BK;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kAccCols = BN;  // 32-bit accumulator columns per tile
constexpr int kTmemCols = 2 * kAccCols;
constexpr int kGemmThreads = 256;
constexpr int kEpiWarp0 = 4;

struct Control {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t epi_done, fin_done;   // split-K: hand-over between the four epilogue warps
  uint32_t tmem_base;
  int abort;
  int finalize;
  float sb[4][2][BN];  // per epilogue warp, per accumulator
};

constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + sizeof(Control);

struct GemmParams {
  int64_t M, N, K;
  const void* sa;
  const void* sb;
  int scale_dtype;
  void* out;
  int out_dtype;
  int epilogue;
  int32_t* error_flag;
  int tiles_m, tiles_n;
  int splits;          // K is cut in `splits` ranges; 1 = every CTA owns whole tiles
  uint32_t* ws;        // splits > 1: [splits][tiles][BN][BM] partial sums (int32 or float32 bits)
  int* counters;       // splits > 1: [tiles][2], zero on entry
};

__device__ __forceinline__ float load_scale(const void* p, int dtype, int64_t i) {
  if (dtype == QWX_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == QWX_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ float round_out(float v, int out_dtype) {
  if (out_dtype == QWX_BF16) return round_to<BF16>(v);
  if (out_dtype == QWX_F16) return round_to<F16>(v);
  return v;
}

// Polls a global counter (written with atomics by other CTAs of this cooperative launch) until
// it reaches `target`; bounded like every other wait of this file.
__device__ __forceinline__ bool wait_count(const int* ctr, int target, volatile int* abort) {
  const long long t0 = clock64();
#pragma unroll 1
  for (uint32_t it = 1;; ++it) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if (v >= target) return true;
    __nanosleep(64);
    if ((it & 63u) == 0) {
      if (*abort) return false;
      if (clock64() - t0 > kWaitBudgetCycles) {
        *abort = 1;
        return false;
      }
    }
  }
}

template <MmaKind KIND, int BLAYOUT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_q8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  Control* ctl = reinterpret_cast<Control*>(smem_raw + (tiles - smem_u32(smem_raw)) +
                                            (size_t)kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Work items: (tile, K range).  With splits == 1 an item is a whole output tile; decode-shaped
  // problems with fewer tiles than SMs cut K so that every SM streams a share of the weight.
  const int kblocks = (int)((p.K + BK - 1) / BK);
  const int num_tiles = p.tiles_m * p.tiles_n * p.splits;
  volatile int* abort = &ctl->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->acc_full[a]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[a]), 4);
    }
    mbar_init(smem_u32(&ctl->epi_done), 128);
    mbar_init(smem_u32(&ctl->fin_done), 1);
    ctl->abort = 0;
    ctl->finalize = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    long issued = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int split = tile % p.splits, t = tile / p.splits;
      const int m0 = (t % p.tiles_m) * BM;
      const int n0 = (t / p.tiles_m) * BN;
      const int kb0 = (int)((int64_t)kblocks * split / p.splits);
      const int kb1 = (int)((int64_t)kblocks * (split + 1) / p.splits);
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort);
          if (ok) {
            const uint32_t bar = smem_u32(&ctl->full[stage]);
            const uint32_t sa = tiles + stage * kStageBytes;
            const uint32_t sb = sa + kABytes;
            mbar_expect_tx(bar, kStageBytes);
            tma_load_2d(sa, &tma_a, kb * BK, m0, bar);
            if (BLAYOUT == QWX_B_NK) {
              tma_load_2d(sb, &tma_b, kb * BK, n0, bar);
            } else {
              tma_load_2d(sb, &tma_b, n0, kb * BK, bar);
              tma_load_2d(sb + BK * 128, &tma_b, n0 + 128, kb * BK, bar);
            }
            ++issued;
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (lane == 0 && *abort) {
      // Let copies that are still in flight land before the CTA gives up its shared memory.
      long pending = issued < kStages ? issued : kStages;
      int s = stage;
      uint32_t ph = phase;
      for (long i = 0; i < pending; ++i) {
        if (--s < 0) { s = kStages - 1; ph ^= 1u; }
        for (int it = 0; it < 100000; ++it)
          if (mbar_try_wait(smem_u32(&ctl->full[s]), ph)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc =
        KIND == MmaKind::kI8
            ? make_idesc(2, 1, 1, 0, BLAYOUT == QWX_B_KN ? 1 : 0, BM, BN)
            : make_idesc(1, 0, 0, 0, BLAYOUT == QWX_B_KN ? 1 : 0, BM, BN);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort);
        tc_fence_after();
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      const int split = tile % p.splits;
      const int kb0 = (int)((int64_t)kblocks * split / p.splits);
      const int kb1 = (int)((int64_t)kblocks * (split + 1) / p.splits);
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&ctl->full[stage]), phase, abort);
          if (ok) {
            tc_fence_after();
            const uint32_t sa = tiles + stage * kStageBytes;
            const uint32_t sb = sa + kABytes;
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              // A, K-major: 8-row groups 1024 B apart; step 32 B inside the swizzled row.
              const uint64_t da = make_smem_desc(sa + kk * UMMA_K, 16, 1024);
              // B, K-major: same as A.  B, MN-major ([K, N] rows of 128 N-bytes): 8 K-rows
              // per 1024 B group, the second 128 columns BK*128 B further; step 32 K-rows.
              const uint64_t db = BLAYOUT == QWX_B_NK
                                      ? make_smem_desc(sb + kk * UMMA_K, 16, 1024)
                                      : make_smem_desc(sb + kk * UMMA_K * 128, BK * 128, 1024);
              mma_ss<KIND>(tmem_base + acc * kAccCols, da, db, idesc, kb != kb0 || kk != 0);
            }
            mma_commit(smem_u32(&ctl->empty[stage]));
            if (kb == kb1 - 1) mma_commit(smem_u32(&ctl->acc_full[acc]));
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  } else if (warp >= kEpiWarp0) {
    // ---------------- epilogue ----------------
    const int q = warp - kEpiWarp0;           // tensor-memory lane quarter of this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool reference = p.epilogue == QWX_EPI_REFERENCE;
    uint32_t epi_phase = 0, fin_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int t = tile / p.splits;
      const int m0 = (t % p.tiles_m) * BM;
      const int n0 = (t / p.tiles_m) * BN;
      // Each warp stages this tile's column scales for itself (no cross-warp barrier, so a
      // warp that gives up on a wait cannot strand the others).
      for (int j = lane; j < BN; j += 32) {
        const int64_t n = (int64_t)n0 + j;
        ctl->sb[q][acc][j] = (p.sb && n < p.N) ? load_scale(p.sb, p.scale_dtype, n) : 1.0f;
      }
      __syncwarp();
      const int64_t m = (int64_t)m0 + q * 32 + lane;
      const float sa = (p.sa && m < p.M) ? load_scale(p.sa, p.scale_dtype, m) : 1.0f;

      if (lane == 0) ok = mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();

      // Scale, convert and store 32 consecutive columns of row m (r: raw accumulator bits).
      auto emit32 = [&](const uint32_t (&r)[32], int64_t m, float sa, int64_t ncol, const float* sbv) {
        if (p.out_dtype == QWX_S32) {
          int32_t* o = reinterpret_cast<int32_t*>(p.out) + m * p.N + ncol;
          if (ncol + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<uint4*>(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
          } else {
            for (int j = 0; j < 32 && ncol + j < p.N; ++j) o[j] = (int32_t)r[j];
          }
          return;
        }
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float a = KIND == MmaKind::kI8 ? (float)(int32_t)r[j] : __uint_as_float(r[j]);
          if (reference) {
            a = round_out(a, p.out_dtype);
            a = round_out(__fmul_rn(a, sa), p.out_dtype);
            a = round_out(__fmul_rn(a, sbv[j]), p.out_dtype);
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
      };

      // The same for 8 consecutive columns (the split-K finish).
      auto emit8 = [&](const uint32_t (&r)[8], int64_t m, float sa, int64_t ncol, const float* sbv) {
        const bool full = ncol + 8 <= p.N;
        if (p.out_dtype == QWX_S32) {
          int32_t* o = reinterpret_cast<int32_t*>(p.out) + m * p.N + ncol;
          if (full && (p.N & 3) == 0) {
            *reinterpret_cast<uint4*>(o) = make_uint4(r[0], r[1], r[2], r[3]);
            *reinterpret_cast<uint4*>(o + 4) = make_uint4(r[4], r[5], r[6], r[7]);
          } else {
            for (int j = 0; j < 8 && ncol + j < p.N; ++j) o[j] = (int32_t)r[j];
          }
          return;
        }
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float a = KIND == MmaKind::kI8 ? (float)(int32_t)r[j] : __uint_as_float(r[j]);
          if (reference) {
            a = round_out(a, p.out_dtype);
            a = round_out(__fmul_rn(a, sa), p.out_dtype);
            a = round_out(__fmul_rn(a, sbv[j]), p.out_dtype);
          } else {
            a = __fmul_rn(__fmul_rn(a, sa), sbv[j]);
          }
          v[j] = a;
        }
        if (p.out_dtype == QWX_F32) {
          float* o = reinterpret_cast<float*>(p.out) + m * p.N + ncol;
          if (full && (p.N & 3) == 0) {
            *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
          } else {
            for (int j = 0; j < 8 && ncol + j < p.N; ++j) o[j] = v[j];
          }
        } else {
          uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + m * p.N + ncol;
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (p.out_dtype == QWX_BF16) {
              __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
              w[j] = *reinterpret_cast<uint32_t*>(&h);
            } else {
              __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
              w[j] = *reinterpret_cast<uint32_t*>(&h);
            }
          }
          if (full && (p.N & 7) == 0) {
            *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
          } else {
            for (int j = 0; j < 8 && ncol + j < p.N; ++j) o[j] = (uint16_t)(w[j >> 1] >> ((j & 1) * 16));
          }
        }
      };

      // Split-K: this item's partial sums go to a private slab, laid out as the accumulator
      // comes out of tensor memory ([column][tile row]) so that every store is coalesced.
      uint32_t* slab = nullptr;
      if (p.splits > 1)
        slab = p.ws + ((size_t)(tile % p.splits) * (p.tiles_m * p.tiles_n) + t) * (size_t)(BM * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * kAccCols + c * 32, r);
        tmem_ld_wait();
        const int64_t ncol = (int64_t)n0 + c * 32;
        if (m >= p.M || ncol >= p.N) continue;
        if (p.splits == 1) {
          emit32(r, m, sa, ncol, &ctl->sb[q][acc][c * 32]);
        } else {
          uint32_t* w = slab + (size_t)(c * 32) * BM + q * 32 + lane;
#pragma unroll
          for (int j = 0; j < 32; ++j) __stcg(w + j * BM, r[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));

      if (p.splits > 1) {
        // Publish this K range, wait until every range of the tile has been published (the
        // launch is cooperative: all CTAs are resident), then finish a share of the tile:
        // CTA `split` takes the 32-column chunks c = split, split + splits, ...; warp q the
        // eight columns q * 8 .. q * 8 + 7 of each, every lane one row, adding the ranges'
        // slabs in range order (so float sums do not depend on timing).
        const int split = tile % p.splits;
        int* arrived = p.counters + 2 * t;
        __threadfence();
        mbar_arrive(smem_u32(&ctl->epi_done));
        if (q == 0 && lane == 0) {
          if (mbar_wait(smem_u32(&ctl->epi_done), epi_phase, abort)) atomicAdd(arrived, 1);
          mbar_arrive(smem_u32(&ctl->fin_done));
        }
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&ctl->fin_done), fin_phase, abort);
          if (ok) ok = wait_count(arrived, p.splits, abort);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        epi_phase ^= 1u;
        fin_phase ^= 1u;
        if (!ok) break;
        __threadfence();

        const int64_t rows_left = p.M - m0;
        const int groups = (int)(rows_left >= BM ? BM / 32 : (rows_left + 31) / 32);
        const size_t split_stride = (size_t)(p.tiles_m * p.tiles_n) * (size_t)(BM * BN);
        const uint32_t* base = p.ws + (size_t)t * (size_t)(BM * BN);
#pragma unroll 1
        for (int c = split; c < BN / 32; c += p.splits) {
          const int64_t ncol = (int64_t)n0 + c * 32 + q * 8;
          if (ncol >= p.N) break;
#pragma unroll 1
          for (int g = 0; g < groups; ++g) {
            const int64_t mr = (int64_t)m0 + g * 32 + lane;
            if (mr >= p.M) continue;
            const uint32_t* w = base + (size_t)(c * 32 + q * 8) * BM + g * 32 + lane;
            uint32_t r[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) r[j] = __ldcg(w + j * BM);
#pragma unroll 4
            for (int sp = 1; sp < p.splits; ++sp) {
              w += split_stride;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint32_t v = __ldcg(w + j * BM);
                if (KIND == MmaKind::kI8) r[j] += v;
                else r[j] = __float_as_uint(__fadd_rn(__uint_as_float(r[j]), __uint_as_float(v)));
              }
            }
            const float sar = p.sa ? load_scale(p.sa, p.scale_dtype, mr) : 1.0f;
            emit8(r, mr, sar, ncol, &ctl->sb[q][acc][c * 32 + q * 8]);
          }
        }
        // The CTA that leaves the tile last clears its two counters for the next launch.
        __syncwarp();
        mbar_arrive(smem_u32(&ctl->epi_done));
        if (q == 0 && lane == 0) {
          if (mbar_wait(smem_u32(&ctl->epi_done), epi_phase, abort)) {
            if (atomicAdd(arrived + 1, 1) + 1 == p.splits) {
              arrived[0] = 0;
              arrived[1] = 0;
            }
          }
        }
        epi_phase ^= 1u;
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && ctl->abort && p.error_flag) atomicExch(p.error_flag, QWX_ERR_DEVICE_WAIT);
}

template <MmaKind KIND, int BLAYOUT>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
           cudaStream_t st) {
  auto kern = gemm_q8_kernel<KIND, BLAYOUT>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) !=
        cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  if (p.splits > 1) {
    // the CTAs of a tile wait for one another: a cooperative launch guarantees that all of
    // them are resident (the grid is at most one CTA per SM)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, ta, tb, p) != cudaSuccess) {
      (void)cudaGetLastError();
      return QWX_ERR_LAUNCH;
    }
    return QWX_OK;
  }
  kern<<<grid, kGemmThreads, kSmemBytes, st>>>(ta, tb, p);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return v;
  }();
  return n;
}

}  // namespace
}  // namespace qwx

namespace qwx {
// gemm_q8_narrow.cu
int narrow_tile_width(int64_t N, int64_t K, int sms);
int gemm_q8_narrow_launch(const void* a, const void* b, const void* sa, const void* sb, int scale_dtype,
                          int64_t M, int64_t N, int64_t K, int code_dtype, void* out, int out_dtype,
                          int epilogue, int bn, int32_t* error_flag, cudaStream_t st);
int gemm_q8_pair_launch(const void* a, const void* b, int code_dtype, int b_layout, int64_t M,
                        int64_t N, int64_t K, const void* sa, const void* sb, int scale_dtype,
                        void* out, int out_dtype, int epilogue, int32_t* error_flag, int sms,
                        cudaStream_t st);
}

using namespace qwx;

// Split-K is worth it when the tiles cannot occupy the SMs: cut K so that tiles x splits comes
// close to the SM count, keeping at least four 128-wide K blocks per range.
// The workspace opens with two int32 counters per tile (ranges published, CTAs finished; rounded
// up to 256 bytes), zero between calls; the partial-sum slabs follow and need no initialisation.
// The region has one size for every shape: callers reuse one workspace for calls with different
// tile counts, and the slabs of one call must never lie where another call keeps its counters
// (K is only cut when the tiles fill at most half of the SMs, so 1 KB holds all counters).
static size_t counter_bytes(int64_t tiles) {
  const size_t need = (size_t)tiles * 8;
  return need <= 1024 ? 1024 : ((need + 255) & ~(size_t)255);
}

static int choose_splits(int64_t tiles, int kblocks, int sms) {
  if (tiles * 2 > sms) return 1;
  int64_t s = sms / tiles;
  if (s > kblocks / 4) s = kblocks / 4;
  return s < 1 ? 1 : (int)s;
}

extern "C" size_t qwx_gemm_q8_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int sms = sm_count() > 0 ? sm_count() : 148;
  const int splits = choose_splits(tiles, (int)((K + BK - 1) / BK), sms);
  if (splits == 1) return 0;
  return counter_bytes(tiles) + (size_t)splits * tiles * BM * BN * 4;
}

static int gemm_q8_impl(const void* a, const void* b, int code_dtype, int b_layout, int64_t M,
                        int64_t N, int64_t K, int64_t k_tile, const void* sa, int sa_tiled,
                        const void* sb, int sb_tiled, int scale_dtype, void* out, int out_dtype,
                        int epilogue, void* workspace, size_t workspace_bytes,
                        int workspace_is_zero, int32_t* error_flag, qwx_stream_t stream) {
  if (!a || !b || !out) return QWX_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (M > INT32_MAX - BM || N > INT32_MAX - BN || K > INT32_MAX - BK) return QWX_ERR_SHAPE;
  if (code_dtype != QWX_S8 && code_dtype != QWX_E4M3) return QWX_ERR_DTYPE;
  if (b_layout != QWX_B_KN && b_layout != QWX_B_NK) return QWX_ERR_SHAPE;
  if (k_tile != 0 && k_tile != K)  // scales change along K: the kernel with running sums
    return qwx_gemm_q8_tiled(a, b, code_dtype, b_layout, M, N, K, k_tile, sa, sa_tiled, sb, sb_tiled,
                             scale_dtype, nullptr, nullptr, out, out_dtype, epilogue, error_flag,
                             stream);
  if (out_dtype == QWX_S32) {
    if (code_dtype != QWX_S8 || sa || sb) return QWX_ERR_DTYPE;
  } else if (out_dtype != QWX_BF16 && out_dtype != QWX_F32 && out_dtype != QWX_F16) {
    return QWX_ERR_DTYPE;
  }
  if ((sa || sb) && scale_dtype != QWX_F32 && scale_dtype != QWX_BF16 && scale_dtype != QWX_F16)
    return QWX_ERR_DTYPE;
  if (epilogue != QWX_EPI_F32 && epilogue != QWX_EPI_REFERENCE) return QWX_ERR_SHAPE;
  // TMA: 16-byte aligned bases and row pitches.
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return QWX_ERR_ALIGN;
  if (K % 16) return QWX_ERR_ALIGN;
  if (b_layout == QWX_B_KN && (N % 16)) return QWX_ERR_ALIGN;
  const int elem = out_dtype == QWX_F32 || out_dtype == QWX_S32 ? 4 : 2;
  if (reinterpret_cast<uintptr_t>(out) & 15) return QWX_ERR_ALIGN;
  (void)elem;

  CUtensorMap ta, tb;
  if (!get_encode_tiled()) return QWX_ERR_NO_DEVICE;
  if (!encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)M, (uint64_t)K, BM, BK))
    return QWX_ERR_LAUNCH;
  const bool ok_b = b_layout == QWX_B_NK
                        ? encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)N, (uint64_t)K, BN, BK)
                        : encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)K, (uint64_t)N, BK, 128);
  if (!ok_b) return QWX_ERR_LAUNCH;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.sa = sa; p.sb = sb; p.scale_dtype = scale_dtype;
  p.out = out; p.out_dtype = out_dtype; p.epilogue = epilogue;
  p.error_flag = error_flag;
  p.tiles_m = (int)((M + BM - 1) / BM);
  p.tiles_n = (int)((N + BN - 1) / BN);
  int64_t num_tiles = (int64_t)p.tiles_m * p.tiles_n;
  if (num_tiles > INT32_MAX / 64) return QWX_ERR_SHAPE;
  const int sms = sm_count();
  if (sms <= 0) return QWX_ERR_NO_DEVICE;
  cudaStream_t st = (cudaStream_t)stream;
  p.splits = 1;
  p.ws = nullptr;
  p.counters = nullptr;
  if (workspace != nullptr) {
    const int splits = choose_splits(num_tiles, (int)((K + BK - 1) / BK), sms);
    if (splits > 1) {
      const size_t need = counter_bytes(num_tiles) + (size_t)splits * num_tiles * BM * BN * 4;
      if (workspace_bytes < need) return QWX_ERR_WORKSPACE;
      if (reinterpret_cast<uintptr_t>(workspace) & 15) return QWX_ERR_ALIGN;
      if (!workspace_is_zero &&
          cudaMemsetAsync(workspace, 0, counter_bytes(num_tiles), st) != cudaSuccess)
        return QWX_ERR_LAUNCH;
      p.splits = splits;
      p.counters = (int*)workspace;
      p.ws = (uint32_t*)((char*)workspace + counter_bytes(num_tiles));
      num_tiles *= splits;
    }
  }
  // Few rows against a K-major weight with a handful of 256-wide column tiles: narrow column
  // tiles, one per SM, instead of cutting K (no partial sums through global memory; a workspace
  // that was passed has been checked above as for the K cut, and stays untouched).
  if (M <= BM && b_layout == QWX_B_NK && K % BK == 0) {
    const int bn = narrow_tile_width(N, K, sms);
    if (bn > 0)
      return gemm_q8_narrow_launch(a, b, sa, sb, scale_dtype, M, N, K, code_dtype, out, out_dtype, epilogue, bn,
                                   error_flag, st);
  }
  // Two or more 128-row tiles: the CTA-pair kernel, which moves a third less data per SM.
  if (p.splits == 1 && M > BM)
    return gemm_q8_pair_launch(a, b, code_dtype, b_layout, M, N, K, sa, sb, scale_dtype, out,
                               out_dtype, epilogue, error_flag, sms, st);
  const int grid = (int)(num_tiles < sms ? num_tiles : sms);
  if (code_dtype == QWX_S8) {
    return b_layout == QWX_B_NK ? launch<MmaKind::kI8, QWX_B_NK>(ta, tb, p, grid, st)
                                : launch<MmaKind::kI8, QWX_B_KN>(ta, tb, p, grid, st);
  }
  return b_layout == QWX_B_NK ? launch<MmaKind::kF8F6F4, QWX_B_NK>(ta, tb, p, grid, st)
                              : launch<MmaKind::kF8F6F4, QWX_B_KN>(ta, tb, p, grid, st);
}

extern "C" int qwx_gemm_q8(const void* a, const void* b, int code_dtype, int b_layout, int64_t M,
                           int64_t N, int64_t K, int64_t k_tile, const void* sa, int sa_tiled,
                           const void* sb, int sb_tiled, int scale_dtype, void* out,
                           int out_dtype, int epilogue, int32_t* error_flag,
                           qwx_stream_t stream) {
  return gemm_q8_impl(a, b, code_dtype, b_layout, M, N, K, k_tile, sa, sa_tiled, sb, sb_tiled,
                      scale_dtype, out, out_dtype, epilogue, nullptr, 0, 0, error_flag, stream);
}

extern "C" int qwx_gemm_q8_ws(const void* a, const void* b, int code_dtype, int b_layout, int64_t M,
                              int64_t N, int64_t K, int64_t k_tile, const void* sa, int sa_tiled,
                              const void* sb, int sb_tiled, int scale_dtype, void* out,
                              int out_dtype, int epilogue, void* workspace,
                              size_t workspace_bytes, int workspace_is_zero, int32_t* error_flag,
                              qwx_stream_t stream) {
  return gemm_q8_impl(a, b, code_dtype, b_layout, M, N, K, k_tile, sa, sa_tiled, sb, sb_tiled,
                      scale_dtype, out, out_dtype, epilogue, workspace, workspace_bytes,
                      workspace_is_zero, error_flag, stream);
}

extern "C" size_t qwx_quant_gemm_q8_workspace_bytes(int64_t M, int64_t K) {
  if (M <= 0 || K <= 0) return 0;
  return (size_t)(M * K) + (size_t)((M * 2 + 255) / 256 * 256);
}

// Per-token quantization of the bf16 activations followed by the GEMM, as one call.  The two
// kernels run back to back on `stream`; the codes ([M, K], 1 byte each) are written once and
// read by the GEMM while most of them are still in the 126 MB L2.  Quantizing inside the
// GEMM's producer instead would repeat the division and rounding of every activation once per
// column of output tiles (N / 256 times) and needs the row's absmax first, i.e. a second read
// of the bf16 rows, so the separate pass is the cheaper form on this part.
extern "C" int qwx_quant_gemm_q8(const void* a, int64_t M, int64_t K, const void* wq,
                                 const void* sw, int64_t N, int code_dtype, int b_layout,
                                 int rounding, void* out, int out_dtype, int epilogue,
                                 void* workspace, size_t workspace_bytes, int32_t* error_flag,
                                 qwx_stream_t stream) {
  if (!a || !wq || !sw || !out || !workspace) return QWX_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (code_dtype != QWX_S8 && code_dtype != QWX_E4M3) return QWX_ERR_DTYPE;
  if (workspace_bytes < qwx_quant_gemm_q8_workspace_bytes(M, K)) return QWX_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return QWX_ERR_ALIGN;
  void* sa = workspace;                                     // [M] bf16 row scales
  void* aq = (char*)workspace + (M * 2 + 255) / 256 * 256;  // [M, K] codes
  int rc = qwx_quantize(a, QWX_BF16, 1, M, K, 1, 1, K, QWX_ABSMAX, 0, 0.0, code_dtype, rounding,
                        aq, sa, nullptr, nullptr, 0, stream);
  if (rc) return rc;
  return gemm_q8_impl(aq, wq, code_dtype, b_layout, M, N, K, 0, sa, 0, sw, 0, QWX_BF16, out,
                      out_dtype, epilogue, nullptr, 0, 0, error_flag, stream);
}
