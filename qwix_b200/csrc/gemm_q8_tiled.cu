// Quantized GEMM with scales that change along K and with zero-point corrections, sm_100a.
//
//   out[m, n] = sum_t ( acc_t[m, n] - corr_row[m, t] * corr_col[t, n] ) * sa[m, t] * sb[t, n]
//   acc_t[m, n] = sum_{k in K tile t} a[m, k] * b[k, n]          (int32 or float32, tcgen05)
//
// This is the general form of the reference's dequantize-on-output contraction
// (qwix/_src/core/dot_general.py:135-261): a tiled contracting axis becomes (count, size), the
// count axis rides along as a batch axis of the integer dot (:187-203, :220), the zero point of
// an asymmetric operand is removed with one more integer dot against the other operand's codes
// (:228-253), every tile's result is multiplied by the two scales (:255-258) and the tiles are
// summed (:259).  Here the loop over K tiles stays inside one kernel, like the reference's
// Pallas form (dot_general.py:278-399): the tensor cores fill one of two accumulators in tensor
// memory per K tile while the epilogue warps drain the other, apply the rank-1 integer
// correction and the scales, and keep the running float32 sums in registers.  That bounds the
// tile to 128 x 128 (128 running sums per thread).
//
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer, warp 2 owns the tensor-memory allocation,
// warps 4-11 epilogue (two per tensor-memory lane quarter, 64 columns each: with 128-wide K
// tiles the epilogue, not the MMA, sets the pace).  Every wait is bounded.

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

constexpr int TM = 128;
constexpr int TN = 128;
constexpr int TK = 128;        // bytes == elements for 8-bit codes
constexpr int UMMA_K8 = 32;
constexpr int kStagesT = 6;
constexpr int kStageBytesT = (TM + TN) * TK;
constexpr int kThreadsT = 384;      // 4 control warps + 8 epilogue warps
constexpr int kEpiWarpT = 4;

struct ControlT {
  uint64_t full[kStagesT];
  uint64_t empty[kStagesT];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort;
  float sb[8][2][TN / 2];  // per epilogue warp (64 columns each), double-buffered per K tile
  int32_t zc[8][2][TN / 2];
};

constexpr size_t kSmemBytesT = 1024 + (size_t)kStagesT * kStageBytesT + sizeof(ControlT);

struct TiledParams {
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
  int epilogue;
  int fast_i2f;             // |acc| < 2^22 guaranteed: convert with the magic-number add
  int32_t* error_flag;
  int tiles_m, tiles_n;
};

__device__ __forceinline__ float load_scale_t(const void* p, int dtype, int64_t i) {
  if (dtype == QWX_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == QWX_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ float round_out_t(float v, int out_dtype) {
  if (out_dtype == QWX_BF16) return round_to<BF16>(v);
  if (out_dtype == QWX_F16) return round_to<F16>(v);
  return v;
}

template <MmaKind KIND, int BLAYOUT>
__global__ void __launch_bounds__(kThreadsT, 1)
gemm_q8_tiled_kernel(const __grid_constant__ CUtensorMap tma_a,
                     const __grid_constant__ CUtensorMap tma_b, const TiledParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  ControlT* ctl = reinterpret_cast<ControlT*>(smem_raw + (tiles - smem_u32(smem_raw)) +
                                              (size_t)kStagesT * kStageBytesT);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = p.T * p.kb_per_tile;
  volatile int* abort = &ctl->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesT; ++s) {
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
    tmem_alloc(smem_u32(&ctl->tmem_base), 2 * TN);
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
      const int m0 = (tile % p.tiles_m) * TM;
      const int n0 = (tile / p.tiles_m) * TN;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort);
          if (ok) {
            const uint32_t bar = smem_u32(&ctl->full[stage]);
            const uint32_t sa = tiles + stage * kStageBytesT;
            const uint32_t sb = sa + TM * TK;
            mbar_expect_tx(bar, kStageBytesT);
            tma_load_2d(sa, &tma_a, kb * TK, m0, bar);
            if (BLAYOUT == QWX_B_NK) tma_load_2d(sb, &tma_b, kb * TK, n0, bar);
            else tma_load_2d(sb, &tma_b, n0, kb * TK, bar);
            ++issued;
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == kStagesT) { stage = 0; phase ^= 1u; }
      }
    }
    if (lane == 0 && *abort) {
      // Let copies that are still in flight land before the CTA gives up its shared memory.
      long pending = issued < kStagesT ? issued : kStagesT;
      int s = stage;
      uint32_t ph = phase;
      for (long i = 0; i < pending; ++i) {
        if (--s < 0) { s = kStagesT - 1; ph ^= 1u; }
        for (int it = 0; it < 100000; ++it)
          if (mbar_try_wait(smem_u32(&ctl->full[s]), ph)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: one accumulator per (output tile, K tile) ----------------
    constexpr uint32_t idesc =
        KIND == MmaKind::kI8 ? make_idesc(2, 1, 1, 0, BLAYOUT == QWX_B_KN ? 1 : 0, TM, TN)
                             : make_idesc(1, 0, 0, 0, BLAYOUT == QWX_B_KN ? 1 : 0, TM, TN);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
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
              const uint32_t sa = tiles + stage * kStageBytesT;
              const uint32_t sb = sa + TM * TK;
#pragma unroll
              for (int kk = 0; kk < TK / UMMA_K8; ++kk) {
                const uint64_t da = make_smem_desc(sa + kk * UMMA_K8, 16, 1024);
                const uint64_t db = BLAYOUT == QWX_B_NK
                                        ? make_smem_desc(sb + kk * UMMA_K8, 16, 1024)
                                        : make_smem_desc(sb + kk * UMMA_K8 * 128, TK * 128, 1024);
                mma_ss<KIND>(tmem_base + acc * TN, da, db, idesc, kb != 0 || kk != 0);
              }
              mma_commit(smem_u32(&ctl->empty[stage]));
              if (kb == p.kb_per_tile - 1) mma_commit(smem_u32(&ctl->acc_full[acc]));
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (++stage == kStagesT) { stage = 0; phase ^= 1u; }
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp >= kEpiWarpT) {
    // ---------------- epilogue: drain one accumulator per K tile, keep running sums ----------------
    const int ew = warp - kEpiWarpT;          // epilogue warp 0..7
    const int q = ew & 3;                     // tensor-memory lane quarter of this warp
    const int ch = ew >> 2;                   // which 64 columns of the tile
    const bool reference = p.epilogue == QWX_EPI_REFERENCE;
    const bool has_corr = p.corr_row != nullptr && p.corr_col != nullptr;
    const bool fast_i2f = p.fast_i2f != 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;

    // Scales and correction factors of one (output tile, K tile): four columns per lane for
    // the warp's shared copy, one row value per lane.
    struct Prefetch {
      float sb[2];
      int32_t zc[2];
      float sa;
      int32_t zr;
    };
    auto fetch = [&](int tile, int t) {
      Prefetch f;
      const int m0 = (tile % p.tiles_m) * TM;
      const int n0 = (tile / p.tiles_m) * TN;
      const int64_t m = (int64_t)m0 + q * 32 + lane;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int64_t n = (int64_t)n0 + ch * 64 + lane + 32 * i;
        const bool in = n < p.N;
        f.sb[i] = (p.sb && in) ? load_scale_t(p.sb, p.scale_dtype, (p.sb_tiled ? (int64_t)t * p.N : 0) + n)
                               : 1.0f;
        f.zc[i] = (has_corr && in) ? __ldg(p.corr_col + (int64_t)t * p.N + n) : 0;
      }
      const bool rin = m < p.M;
      f.sa = (p.sa && rin) ? load_scale_t(p.sa, p.scale_dtype, p.sa_tiled ? m * p.T + t : m) : 1.0f;
      f.zr = (has_corr && rin) ? __ldg(p.corr_row + m * p.T + t) : 0;
      return f;
    };

    int tile = blockIdx.x, t = 0, it = 0;
    bool have = tile < num_tiles;
    Prefetch pf;
    if (have) pf = fetch(tile, t);
    float v[TN / 2];

    while (have && ok) {
      const int buf = it & 1;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        ctl->sb[ew][buf][lane + 32 * i] = pf.sb[i];
        ctl->zc[ew][buf][lane + 32 * i] = pf.zc[i];
      }
      const float sa = pf.sa;
      const int32_t zr = pf.zr;
      __syncwarp();
      int ntile = tile, nt = t + 1;
      if (nt == p.T) { nt = 0; ntile += gridDim.x; }
      const bool nhave = ntile < num_tiles;
      if (nhave) pf = fetch(ntile, nt);   // in flight while this K tile is drained

      if (lane == 0) ok = mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();

      if (t == 0) {
#pragma unroll
        for (int j = 0; j < TN / 2; ++j) v[j] = 0.0f;
      }
      const float* sbv = ctl->sb[ew][buf];
      const int32_t* zcv = ctl->zc[ew][buf];
#pragma unroll
      for (int c = 0; c < TN / 64; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * TN + ch * 64 + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float f;
          if (KIND == MmaKind::kI8) {
            int32_t x = (int32_t)r[j];
            if (has_corr) x -= zr * zcv[c * 32 + j];
            f = fast_i2f ? __int_as_float(0x4B400000 + x) - 12582912.0f : (float)x;
          } else {
            f = __uint_as_float(r[j]);
          }
          const float s = sbv[c * 32 + j];
          if (reference) {
            f = round_out_t(f, p.out_dtype);
            f = round_out_t(__fmul_rn(f, sa), p.out_dtype);
            f = round_out_t(__fmul_rn(f, s), p.out_dtype);
            v[c * 32 + j] = __fadd_rn(v[c * 32 + j], f);
          } else {
            v[c * 32 + j] = __fmaf_rn(__fmul_rn(f, sa), s, v[c * 32 + j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));

      if (t == p.T - 1) {
        const int m0 = (tile % p.tiles_m) * TM;
        const int n0 = (tile / p.tiles_m) * TN;
        const int64_t m = (int64_t)m0 + q * 32 + lane;
        if (m < p.M) {
#pragma unroll
          for (int c = 0; c < TN / 64; ++c) {
            const int64_t ncol = (int64_t)n0 + ch * 64 + c * 32;
            if (ncol >= p.N) break;
            const float* vc = v + c * 32;
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

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * TN);
  }
  if (threadIdx.x == 0 && ctl->abort && p.error_flag) atomicExch(p.error_flag, QWX_ERR_DEVICE_WAIT);
}

template <MmaKind KIND, int BLAYOUT>
int launch_tiled(const CUtensorMap& ta, const CUtensorMap& tb, const TiledParams& p, int grid,
                 cudaStream_t st) {
  auto kern = gemm_q8_tiled_kernel<KIND, BLAYOUT>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kSmemBytesT) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  kern<<<grid, kThreadsT, kSmemBytesT, st>>>(ta, tb, p);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

// Sums of 8-bit codes over each K tile.  K_MINOR: codes [R, K], one warp per (row, K tile).
__global__ void code_sums_k_minor_kernel(const int8_t* __restrict__ src, int64_t R, int64_t K,
                                         int64_t k_tile, int T, int t_major, int32_t* out) {
  const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= R * T) return;
  const int64_t r = w / T;
  const int t = (int)(w % T);
  const int8_t* row = src + r * K + (int64_t)t * k_tile;
  int32_t s = 0;
  if ((k_tile & 15) == 0 && (K & 15) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    for (int64_t k = lane * 16; k < k_tile; k += 32 * 16) {
      const int4 u = __ldg(reinterpret_cast<const int4*>(row + k));
      s = __dp4a(u.x, 0x01010101, s);
      s = __dp4a(u.y, 0x01010101, s);
      s = __dp4a(u.z, 0x01010101, s);
      s = __dp4a(u.w, 0x01010101, s);
    }
  } else {
    for (int64_t k = lane; k < k_tile; k += 32) s += row[k];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[t_major ? (int64_t)t * R + r : r * T + t] = s;
}

// K_MAJOR: codes [K, N], one thread per (K tile, column).
__global__ void code_sums_k_major_kernel(const int8_t* __restrict__ src, int64_t K, int64_t N,
                                         int64_t k_tile, int T, int t_major, int32_t* out) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int t = blockIdx.y;
  if (n >= N) return;
  const int8_t* col = src + (int64_t)t * k_tile * N + n;
  int32_t s = 0;
  for (int64_t k = 0; k < k_tile; ++k) s += col[k * N];
  out[t_major ? (int64_t)t * N + n : n * T + t] = s;
}

int sm_count_t() {
  static int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return v;
  }();
  return n;
}

}  // namespace

// gemm_q8_tiled_pair.cu
int gemm_q8_tiled_pair_launch(const void* a, const void* b, int code_dtype, int b_layout,
                              int64_t M, int64_t N, int64_t K, int64_t k_tile, const void* sa,
                              int sa_tiled, const void* sb, int sb_tiled, int scale_dtype,
                              const int32_t* corr_row, const int32_t* corr_col, void* out,
                              int out_dtype, int epilogue, int32_t* error_flag, int sms,
                              cudaStream_t st);

}  // namespace qwx

using namespace qwx;

extern "C" int qwx_code_sums(const void* codes, int64_t rows, int64_t cols, int k_axis,
                             int64_t k_tile, int t_major, int32_t* out, qwx_stream_t stream) {
  if (!codes || !out) return QWX_ERR_NULL;
  if (rows <= 0 || cols <= 0 || (k_axis != 0 && k_axis != 1)) return QWX_ERR_SHAPE;
  const int64_t K = k_axis == 1 ? cols : rows;
  const int64_t other = k_axis == 1 ? rows : cols;
  if (k_tile == 0) k_tile = K;
  if (k_tile < 0 || K % k_tile) return QWX_ERR_SHAPE;
  const int64_t T = K / k_tile;
  if (T > 65535 || other * T > (int64_t)INT32_MAX * 8) return QWX_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int8_t* src = reinterpret_cast<const int8_t*>(codes);
  if (k_axis == 1) {
    const int64_t warps = other * T;
    const int64_t blocks = (warps * 32 + 255) / 256;
    code_sums_k_minor_kernel<<<(unsigned)blocks, 256, 0, st>>>(src, other, K, k_tile, (int)T, t_major, out);
  } else {
    dim3 grid((unsigned)((other + 255) / 256), (unsigned)T);
    code_sums_k_major_kernel<<<grid, 256, 0, st>>>(src, K, other, k_tile, (int)T, t_major, out);
  }
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

extern "C" int qwx_gemm_q8_tiled(const void* a, const void* b, int code_dtype, int b_layout,
                                 int64_t M, int64_t N, int64_t K, int64_t k_tile, const void* sa,
                                 int sa_tiled, const void* sb, int sb_tiled, int scale_dtype,
                                 const int32_t* corr_row, const int32_t* corr_col, void* out,
                                 int out_dtype, int epilogue, int32_t* error_flag,
                                 qwx_stream_t stream) {
  if (!a || !b || !out) return QWX_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (M > INT32_MAX - TM || N > INT32_MAX - TN || K > INT32_MAX - TK) return QWX_ERR_SHAPE;
  if (code_dtype != QWX_S8 && code_dtype != QWX_E4M3) return QWX_ERR_DTYPE;
  if (b_layout != QWX_B_KN && b_layout != QWX_B_NK) return QWX_ERR_SHAPE;
  if (k_tile == 0) k_tile = K;
  if (k_tile < 0 || K % k_tile) return QWX_ERR_SHAPE;
  // The scale tile must be whole 128-wide K blocks unless it is all of K.
  if (k_tile != K && (k_tile % TK)) return QWX_ERR_UNSUPPORTED;
  if (out_dtype != QWX_BF16 && out_dtype != QWX_F32 && out_dtype != QWX_F16) return QWX_ERR_DTYPE;
  if ((sa || sb) && scale_dtype != QWX_F32 && scale_dtype != QWX_BF16 && scale_dtype != QWX_F16)
    return QWX_ERR_DTYPE;
  if ((corr_row == nullptr) != (corr_col == nullptr)) return QWX_ERR_NULL;
  if (corr_row && code_dtype != QWX_S8) return QWX_ERR_DTYPE;  // zero points exist for integer codes only
  if (epilogue != QWX_EPI_F32 && epilogue != QWX_EPI_REFERENCE) return QWX_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return QWX_ERR_ALIGN;
  if (K % 16) return QWX_ERR_ALIGN;
  if (b_layout == QWX_B_KN && (N % 16)) return QWX_ERR_ALIGN;
  if (reinterpret_cast<uintptr_t>(out) & 15) return QWX_ERR_ALIGN;

  // More than one 128-row tile: 256 x 256 tiles on CTA pairs.
  if (M > TM) {
    const int sms_pair = sm_count_t();
    if (sms_pair <= 0) return QWX_ERR_NO_DEVICE;
    return gemm_q8_tiled_pair_launch(a, b, code_dtype, b_layout, M, N, K, k_tile, sa, sa_tiled, sb,
                                     sb_tiled, scale_dtype, corr_row, corr_col, out, out_dtype,
                                     epilogue, error_flag, sms_pair, (cudaStream_t)stream);
  }

  CUtensorMap ta, tb;
  if (!get_encode_tiled()) return QWX_ERR_NO_DEVICE;
  if (!encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)M, (uint64_t)K, TM, TK))
    return QWX_ERR_LAUNCH;
  const bool ok_b = b_layout == QWX_B_NK
                        ? encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)N, (uint64_t)K, TN, TK)
                        : encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)K, (uint64_t)N, TK, TN);
  if (!ok_b) return QWX_ERR_LAUNCH;

  TiledParams p;
  p.M = M; p.N = N; p.K = K;
  p.T = (int)(K / k_tile);
  p.kb_per_tile = (int)((k_tile + TK - 1) / TK);
  p.sa = sa; p.sb = sb;
  p.sa_tiled = sa_tiled && p.T > 1; p.sb_tiled = sb_tiled && p.T > 1;
  p.scale_dtype = scale_dtype;
  p.corr_row = corr_row; p.corr_col = corr_col;
  p.out = out; p.out_dtype = out_dtype; p.epilogue = epilogue;
  // int8 products over at most 128 codes stay below 2^21 in magnitude: the magic-number
  // conversion is exact there.  A zero-point correction can double that, so it keeps cvt.
  p.fast_i2f = (code_dtype == QWX_S8 && k_tile <= 128 && !corr_row) ? 1 : 0;
  p.error_flag = error_flag;
  p.tiles_m = (int)((M + TM - 1) / TM);
  p.tiles_n = (int)((N + TN - 1) / TN);
  const int64_t num_tiles = (int64_t)p.tiles_m * p.tiles_n;
  if (num_tiles > INT32_MAX / 2) return QWX_ERR_SHAPE;
  const int sms = sm_count_t();
  if (sms <= 0) return QWX_ERR_NO_DEVICE;
  const int grid = (int)(num_tiles < sms ? num_tiles : sms);
  cudaStream_t st = (cudaStream_t)stream;
  if (code_dtype == QWX_S8) {
    return b_layout == QWX_B_NK ? launch_tiled<MmaKind::kI8, QWX_B_NK>(ta, tb, p, grid, st)
                                : launch_tiled<MmaKind::kI8, QWX_B_KN>(ta, tb, p, grid, st);
  }
  return b_layout == QWX_B_NK ? launch_tiled<MmaKind::kF8F6F4, QWX_B_NK>(ta, tb, p, grid, st)
                              : launch_tiled<MmaKind::kF8F6F4, QWX_B_KN>(ta, tb, p, grid, st);
}
