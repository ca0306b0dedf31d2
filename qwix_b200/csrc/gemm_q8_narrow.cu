// Quantized GEMM for few rows (decode): up to 128 token rows against a weight [N, K],
//
//   out[m, n] = convert( acc[m, n] * sa[m] * sb[n] ),  acc = sum_k a[m, k] * b[n, k]
//
// the same product and epilogue as gemm_q8.cu (dot_general.py:135-261), cut differently.  A
// decode-shaped problem has one row tile and few 256-wide column tiles, so the wide kernel cuts
// K across CTAs and pays for it: partial sums through global memory, a fence, a counter, a poll,
// a second pass -- about 4 us of a 14 us call.  Here the weight is cut along N alone, into as
// many narrow column tiles (32 .. 256 wide) as there are SMs: every CTA streams whole rows of
// the weight over all of K and finishes its own tile.  An M128 MMA costs the same 46 clocks for
// N = 32 as for N = 64, which wastes tensor pipe that a weight stream at HBM rate does not need
// (4 KB of weight per 184 clocks and SM = 22 B/clk; HBM gives an SM 24).
//
// One tile per CTA, 256 threads: warp 0 TMA producer (only the token rows that exist are
// fetched: the MMA reads 128 rows, the rest is whatever the ring holds there, and an output
// row depends on its own operand row alone), warp 1 MMA issuer, warp 2 owns tensor memory,
// warps 4-7 epilogue of 32 rows each.  A stage holds 1, 2 or 4 K blocks of (token rows + BN) x
// 128 bytes, each operand's blocks brought by ONE three-dimensional TMA copy (a copy of 4 KB
// costs the TMA unit about what one of 32 KB does: with a copy per block and operand a 32-wide
// tile streamed at 11 B/clk); the ring is as deep as shared memory allows.  K must be a multiple
// of 128.  Every wait is bounded.
#include "common.cuh"
#include "sm100.cuh"

namespace qwx {
namespace {

using namespace sm100;

constexpr int NM = 128;        // rows of the MMA
constexpr int NK = 128;        // bytes == elements per stage: one 128-byte swizzle row
constexpr int NUMMA_K = 32;
constexpr int kNMaxStages = 24;
constexpr int kNThreads = 256;
constexpr int kNEpiWarp0 = 4;
constexpr int kNTailBytes = NM * NK;     // the MMA reads 128 rows from a stage's A base: room behind the last stage
constexpr size_t kNRingBytes = 196 * 1024;

struct ControlN {
  uint64_t full[kNMaxStages];
  uint64_t empty[kNMaxStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort;
  float sb[4][256];     // per epilogue warp
};

constexpr size_t kNSmemBytes = 1024 + kNRingBytes + kNTailBytes + sizeof(ControlN);
static_assert(kNSmemBytes <= 227 * 1024, "shared memory of the narrow kernel");

struct NarrowParams {
  int64_t M, N, K;
  const void* sa;
  const void* sb;
  int scale_dtype;
  void* out;
  int out_dtype;
  int epilogue;
  int32_t* error_flag;
  int bn;              // columns per tile: a multiple of 32, at most 256
  int rows;            // token rows fetched per stage: M rounded up to 8
  int stages;
  int kbc;             // K blocks of 128 per stage: 1, 2 or 4
  int tmem_cols;       // power of two >= bn, at least 32
};

// [rows, K] bytes seen as [K / 128][rows][128]: box [kbc][box_rows][128], 128-byte swizzle per row.
bool encode_blocks(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows,
                   uint32_t kbc) {
  EncodeTiledFn fn = get_encode_tiled();
  if (!fn) return false;
  cuuint64_t dims[3] = {128, rows, K / 128};
  cuuint64_t strides[2] = {K, 128};
  cuuint32_t box[3] = {128, box_rows, kbc};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, int c0, int c1, int c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ float load_scale_n(const void* p, int dtype, int64_t i) {
  if (dtype == QWX_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == QWX_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ float round_out_n(float v, int out_dtype) {
  if (out_dtype == QWX_BF16) return round_to<BF16>(v);
  if (out_dtype == QWX_F16) return round_to<F16>(v);
  return v;
}

template <MmaKind KIND, int KBC>
__global__ void __launch_bounds__(kNThreads, 1)
gemm_q8_narrow_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const NarrowParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  ControlN* ctl = reinterpret_cast<ControlN*>(smem_raw + (tiles - smem_u32(smem_raw)) + kNRingBytes + kNTailBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (int)(p.K / NK);
  const int kstages = (kblocks + KBC - 1) / KBC;
  const int n0 = blockIdx.x * p.bn;
  const uint32_t a_bytes = (uint32_t)p.rows * NK, b_bytes = (uint32_t)p.bn * NK;    // per K block
  const uint32_t stage_bytes = (uint32_t)KBC * (a_bytes + b_bytes);                  // [A blocks][B blocks]
  volatile int* abort = &ctl->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    mbar_init(smem_u32(&ctl->acc_full), 1);
    ctl->abort = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&ctl->tmem_base), (uint32_t)p.tmem_cols);
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
    for (int ks = 0; ks < kstages && ok; ++ks) {
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort);
        if (ok) {
          const uint32_t bar = smem_u32(&ctl->full[stage]);
          const uint32_t sa = tiles + stage * stage_bytes;
          mbar_expect_tx(bar, stage_bytes);          // blocks past K arrive as zeros and count
          tma_load_3d(sa, &tma_a, 0, 0, ks * KBC, bar);
          tma_load_3d(sa + KBC * a_bytes, &tma_b, 0, n0, ks * KBC, bar);
          ++issued;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (++stage == p.stages) { stage = 0; phase ^= 1u; }
    }
    if (lane == 0 && *abort) {
      // Let copies that are still in flight land before the CTA gives up its shared memory.
      long pending = issued < p.stages ? issued : p.stages;
      int s = stage;
      uint32_t ph = phase;
      for (long i = 0; i < pending; ++i) {
        if (--s < 0) { s = p.stages - 1; ph ^= 1u; }
        for (int it = 0; it < 100000; ++it)
          if (mbar_try_wait(smem_u32(&ctl->full[s]), ph)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    const uint32_t idesc = KIND == MmaKind::kI8 ? make_idesc(2, 1, 1, 0, 0, NM, (uint32_t)p.bn)
                                                : make_idesc(1, 0, 0, 0, 0, NM, (uint32_t)p.bn);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const uint64_t da0 = make_smem_desc(tiles, 16, 1024);
    const uint64_t step = (uint64_t)(stage_bytes >> 4), a_blk = (uint64_t)(a_bytes >> 4),
                   b_blk = (uint64_t)(b_bytes >> 4), b_off = (uint64_t)((KBC * a_bytes) >> 4);
    uint64_t off = 0;
    for (int ks = 0; ks < kstages && ok; ++ks) {
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&ctl->full[stage]), phase, abort);
        if (ok) {
          tc_fence_after();
          // the issuing thread has 46 clocks per N = 32 MMA: everything unrolled, two adds per MMA
          const int left = kblocks - ks * KBC;
          uint64_t da = da0 + off, db = da0 + off + b_off;
#pragma unroll
          for (int j = 0; j < KBC; ++j, da += a_blk, db += b_blk) {
            if (j >= left) break;
#pragma unroll
            for (int kk = 0; kk < NK / NUMMA_K; ++kk)
              mma_ss<KIND>(tmem_base, da + (uint64_t)(kk * (NUMMA_K >> 4)), db + (uint64_t)(kk * (NUMMA_K >> 4)), idesc,
                           (kk != 0 || j != 0) ? 1u : (uint32_t)(ks != 0));
          }
          mma_commit(smem_u32(&ctl->empty[stage]));
          if (ks == kstages - 1) mma_commit(smem_u32(&ctl->acc_full));
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      off += step;
      if (++stage == p.stages) { stage = 0; phase ^= 1u; off = 0; }
    }
  } else if (warp >= kNEpiWarp0) {
    // ---------------- epilogue: rows q * 32 .. q * 32 + 31 ----------------
    const int q = warp - kNEpiWarp0;
    if (q * 32 < p.M) {
      const bool reference = p.epilogue == QWX_EPI_REFERENCE;
      for (int j = lane; j < p.bn; j += 32) {
        const int64_t n = (int64_t)n0 + j;
        ctl->sb[q][j] = (p.sb && n < p.N) ? load_scale_n(p.sb, p.scale_dtype, n) : 1.0f;
      }
      __syncwarp();
      const int64_t m = (int64_t)q * 32 + lane;
      const float sa = (p.sa && m < p.M) ? load_scale_n(p.sa, p.scale_dtype, m) : 1.0f;
      bool ok = true;
      if (lane == 0) ok = mbar_wait(smem_u32(&ctl->acc_full), 0, abort);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (ok) {
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < p.bn / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + c * 32, r);
          tmem_ld_wait();
          const int64_t ncol = (int64_t)n0 + c * 32;
          if (m >= p.M || ncol >= p.N) continue;
          const float* sbv = &ctl->sb[q][c * 32];
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
              a = round_out_n(a, p.out_dtype);
              a = round_out_n(__fmul_rn(a, sa), p.out_dtype);
              a = round_out_n(__fmul_rn(a, sbv[j]), p.out_dtype);
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
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
  if (threadIdx.x == 0 && ctl->abort && p.error_flag) atomicExch(p.error_flag, QWX_ERR_DEVICE_WAIT);
}

template <MmaKind KIND, int KBC>
int launch_narrow(const CUtensorMap& ta, const CUtensorMap& tb, const NarrowParams& p, int grid, cudaStream_t st) {
  auto kern = gemm_q8_narrow_kernel<KIND, KBC>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kNSmemBytes) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  kern<<<grid, kNThreads, kNSmemBytes, st>>>(ta, tb, p);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

}  // namespace

// Column-tile width for a decode-shaped problem: the narrowest multiple of 32 that covers N with at
// most `sms` tiles; 0 (the wide kernel's cases) where that leaves fewer than half of the SMs
// busy, where N needs more than 256-wide tiles, or where a CTA would issue more than 160 MMAs:
// a narrow tile spends an MMA (about 75 clocks of the issuing thread) per 32 bytes of K, and
// beyond that the K cut of the wide kernel is faster (8192 x 28672 ... 4096 x 4096 measured:
// 22.7 / 12.7 / 10.9 us against 25.5 / 15.4 / 13.6; 4096 x 14336: 28.3 against 19.2).
int narrow_tile_width(int64_t N, int64_t K, int sms) {
  if (K > 160 * NUMMA_K) return 0;
  for (int bn = 32; bn <= 256; bn += 32) {
    const int64_t tiles = (N + bn - 1) / bn;
    if (tiles <= sms) return tiles * 2 >= sms ? bn : 0;
  }
  return 0;
}

// a [M, K] codes, b [N, K] codes (K-major), M <= 128.  The caller has checked the arguments.
int gemm_q8_narrow_launch(const void* a, const void* b, const void* sa, const void* sb, int scale_dtype,
                          int64_t M, int64_t N, int64_t K, int code_dtype, void* out, int out_dtype,
                          int epilogue, int bn, int32_t* error_flag, cudaStream_t st) {
  NarrowParams p;
  p.M = M; p.N = N; p.K = K;
  p.sa = sa; p.sb = sb; p.scale_dtype = scale_dtype;
  p.out = out; p.out_dtype = out_dtype; p.epilogue = epilogue; p.error_flag = error_flag;
  p.bn = bn;
  p.rows = (int)((M + 7) / 8 * 8);
  const size_t block_bytes = (size_t)(p.rows + bn) * NK;
  p.kbc = block_bytes * 4 <= 32 * 1024 ? 4 : (block_bytes * 2 <= 32 * 1024 ? 2 : 1);
  const size_t stage_bytes = block_bytes * p.kbc;
  p.stages = (int)(kNRingBytes / stage_bytes);
  if (p.stages > kNMaxStages) p.stages = kNMaxStages;
  if (p.stages < 2) return QWX_ERR_UNSUPPORTED;
  p.tmem_cols = 32;
  while (p.tmem_cols < bn) p.tmem_cols *= 2;
  CUtensorMap ta, tb;
  if (!get_encode_tiled()) return QWX_ERR_NO_DEVICE;
  if (!encode_blocks(&ta, a, (uint64_t)M, (uint64_t)K, (uint32_t)p.rows, (uint32_t)p.kbc) ||
      !encode_blocks(&tb, b, (uint64_t)N, (uint64_t)K, (uint32_t)bn, (uint32_t)p.kbc))
    return QWX_ERR_LAUNCH;
  const int grid = (int)((N + bn - 1) / bn);
  if (code_dtype == QWX_E4M3) {
    return p.kbc == 4 ? launch_narrow<MmaKind::kF8F6F4, 4>(ta, tb, p, grid, st)
           : p.kbc == 2 ? launch_narrow<MmaKind::kF8F6F4, 2>(ta, tb, p, grid, st)
                        : launch_narrow<MmaKind::kF8F6F4, 1>(ta, tb, p, grid, st);
  }
  return p.kbc == 4 ? launch_narrow<MmaKind::kI8, 4>(ta, tb, p, grid, st)
         : p.kbc == 2 ? launch_narrow<MmaKind::kI8, 2>(ta, tb, p, grid, st)
                      : launch_narrow<MmaKind::kI8, 1>(ta, tb, p, grid, st);
}

}  // namespace qwx
