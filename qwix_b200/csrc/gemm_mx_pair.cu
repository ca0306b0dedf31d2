// Block-scaled GEMM on CTA pairs (tcgen05 cta_group::2), sm_100a: the products of gemm_mx8.cu
// (MXFP8, MXFP4, NVFP4; both operands K-major) for problems with more than 128 rows.  Two CTAs
// of a cluster compute one 256 x 224 output tile: each keeps 128 rows of A, 112 columns of B
// and the scale bytes of its own rows and of all 224 columns in shared memory, 128 accumulator
// rows in its tensor memory, and the even CTA issues one M = 256 MMA for both.  What this buys
// is traffic: 30 KB of operands per 128-byte K stage and SM instead of 44 KB -- the single-CTA
// kernel is held back by the L2 -> shared-memory rate, not by the tensor pipe.
//
// A stage holds two 128-byte K blocks (one barrier round trip between the CTAs per eight MMAs).
//
// Per CTA: warp 0 TMA producer (its own halves and scale groups; every load counts on the even
// CTA's `full` barrier: the scale groups travel as rows of a plain two-dimensional tensor map
// so that they can), warp 1 MMA issuer (even CTA only: tcgen05.cp of the scale groups in both
// CTAs, then the MMAs), warp 2 owns the pair's tensor-memory allocation, warps 4-7 epilogue of
// the CTA's 128 rows.  Barriers as in the int8 pair kernel:
//   full[s]      even CTA: 1 arrival (its producer, with the byte count of both CTAs' loads)
//   empty[s]     each CTA: commit of the MMAs that read stage s (the even CTA commits to both)
//   acc_full[a]  each CTA: commit of a tile's last MMA
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

constexpr int YM = 128;        // rows per CTA (256 per pair)
constexpr int YN = 224;        // columns per pair
constexpr int YNH = 112;       // columns of B held by one CTA
constexpr int YK = 128;        // contracted bytes per stage
constexpr int YUMMA_K = 32;
constexpr int kYHalves = 2;                   // 128-byte K blocks per stage: one barrier round trip per two
constexpr int kYStages = 3;
constexpr int kYABytes = YM * YK;             // 16 KB
constexpr int kYBBytes = YNH * YK;            // 14 KB
constexpr int kYSfGroup = 512;                // scale bytes of 128 rows x 4 blocks
constexpr int kYSfOff = kYHalves * (kYABytes + kYBBytes);   // [A k0][A k1][B k0][B k1][scales of A][scales of B]
constexpr int kYStageBytes = 72 * 1024;       // up to 2 x (4 + 8) scale groups behind the operands
static_assert(kYSfOff + kYHalves * 12 * kYSfGroup <= kYStageBytes, "stage layout");
constexpr int kYSfCol = 2 * YN;               // scale columns behind the two accumulators
constexpr int kYThreads = 256;
constexpr int kYEpiWarp0 = 4;

struct ControlY {
  uint64_t full[kYStages];
  uint64_t empty[kYStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort;
};

constexpr size_t kYSmemBytes = 1024 + (size_t)kYStages * kYStageBytes + sizeof(ControlY);
static_assert(kYSmemBytes <= 227 * 1024, "shared memory of the pair kernel");

struct MxPairParams {
  int64_t M, N, K;         // K: contracted bytes
  void* out;
  int out_dtype;
  int32_t* error_flag;
  int tiles_m, tiles_n;    // 256 x 224 tiles
};

// block-scaled MMAs over the pair
__device__ __forceinline__ void mma_mx_pair(int fmt, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  if (fmt == 0) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
  } else if (fmt == 1) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
  }
}
// the scale copy in both CTAs of the pair, each from its own shared memory
__device__ __forceinline__ void tmem_cp_pair_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// FMT: 0 = MXFP8, 1 = MXFP4, 2 = NVFP4 (as in gemm_mx8.cu)
template <int FMT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kYThreads, 1)
gemm_mx_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ CUtensorMap tma_sfa, const __grid_constant__ CUtensorMap tma_sfb,
                    const MxPairParams p) {
  constexpr int kSfGroups = FMT == 2 ? 4 : (FMT == 1 ? 2 : 1);   // 512-byte scale groups per 128 rows and stage
  constexpr uint32_t kCtaTx = kYHalves * (kYABytes + kYBBytes + kSfGroups * 3 * kYSfGroup);
  static_assert(kYSfCol + 12 * kSfGroups <= 512, "scale columns in tensor memory");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  ControlY* ctl = reinterpret_cast<ControlY*>(smem_raw + (tiles - smem_u32(smem_raw)) +
                                              (size_t)kYStages * kYStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: issues the MMAs
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int kblocks = (int)(p.K / (kYHalves * YK));     // stages of two K blocks (the host checks the fit)
  const int num_tiles = p.tiles_m * p.tiles_n;
  volatile int* abort = &ctl->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kYStages; ++s) {
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
    prefetch_tensormap(&tma_sfa);
    prefetch_tensormap(&tma_sfb);
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

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's halves and scale groups ----------------
    int stage = 0;
    uint32_t phase = 0;
    long issued = 0;
    bool ok = true;
    const uint32_t full0 = map_to_cta(smem_u32(&ctl->full[0]), 0);   // the even CTA's barriers
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const int m0 = tm * (2 * YM) + (int)rank * YM;
      const int n0 = tn * YN + (int)rank * YNH;
      // rows of the scale tensors: 512-byte groups, [128-row tile][stage][group] for A and
      // [224-column tile][stage][group][128-column part] for B
      const int sfa_row0 = ((2 * tm + (int)rank) * kblocks) * kYHalves * kSfGroups;
      const int sfb_row0 = (tn * kblocks) * kYHalves * kSfGroups * 2;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort);
          if (ok) {
            const uint32_t sa = tiles + stage * kYStageBytes;
            const uint32_t sb = sa + kYHalves * kYABytes;
            const uint32_t ssfa = sa + kYSfOff;
            const uint32_t ssfb = ssfa + kYHalves * kSfGroups * kYSfGroup;
            if (rank == 0) mbar_expect_tx(smem_u32(&ctl->full[stage]), 2 * kCtaTx);
            const uint32_t bar = full0 + stage * 8;
#pragma unroll
            for (int h = 0; h < kYHalves; ++h) {
              const int k0 = (kYHalves * kb + h) * YK;
              tma_load_2d_pair(sa + h * kYABytes, &tma_a, k0, m0, bar);
              tma_load_2d_pair(sb + h * kYBBytes, &tma_b, k0, n0, bar);
            }
            // the scale groups of both K blocks are consecutive rows: one box each
            tma_load_2d_pair(ssfa, &tma_sfa, 0, sfa_row0 + kb * kYHalves * kSfGroups, bar);
            tma_load_2d_pair(ssfb, &tma_sfb, 0, sfb_row0 + kb * kYHalves * kSfGroups * 2, bar);
            ++issued;
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == kYStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (lane == 0 && *abort && rank == 0) {
      // Let copies that are still in flight land before the CTA gives up its shared memory.
      long pending = issued < kYStages ? issued : kYStages;
      int s = stage;
      uint32_t ph = phase;
      for (long i = 0; i < pending; ++i) {
        if (--s < 0) { s = kYStages - 1; ph ^= 1u; }
        for (int it = 0; it < 100000; ++it)
          if (mbar_try_wait(smem_u32(&ctl->full[s]), ph)) break;
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ---------------- MMA issuer (even CTA): M = 256 over the pair ----------------
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const uint32_t tsfa = tmem_base + kYSfCol;        // 4 columns per scale group
    const uint32_t tsfb = tsfa + 4 * kSfGroups;       // 8 columns per scale group
    const uint32_t empty_peer = map_to_cta(smem_u32(&ctl->empty[0]), 1);
    const uint32_t acc_full_peer = map_to_cta(smem_u32(&ctl->acc_full[0]), 1);
    // Descriptors of stage 0 once; the stage's offset (in their 16-byte units) as a running sum:
    // the issuing thread's instruction stream is what the MMAs wait for.
    const uint64_t da0 = make_smem_desc(tiles, 16, 1024);
    const uint64_t db0 = make_smem_desc(tiles + kYHalves * kYABytes, 16, 1024);
    const uint64_t dsa0 = make_smem_desc_plain(tiles + kYSfOff, 16, 128);
    const uint64_t dsb0 = dsa0 + (uint64_t)((kYHalves * kSfGroups * kYSfGroup) >> 4);
    constexpr uint64_t kStageStep = kYStageBytes >> 4;
    uint64_t off = 0;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort);
        tc_fence_after();
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      const uint32_t d_tmem = tmem_base + acc * YN;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&ctl->full[stage]), phase, abort);
          if (ok) {
            tc_fence_after();
#pragma unroll
            for (int h = 0; h < kYHalves; ++h) {
              const uint64_t da = da0 + off + (uint64_t)(h * (kYABytes >> 4));
              const uint64_t db = db0 + off + (uint64_t)(h * (kYBBytes >> 4));
              const uint64_t dsa = dsa0 + off + (uint64_t)(h * kSfGroups * (kYSfGroup >> 4));
              const uint64_t dsb = dsb0 + off + (uint64_t)(h * kSfGroups * 2 * (kYSfGroup >> 4));
#pragma unroll
              for (int sg = 0; sg < kSfGroups; ++sg) {
                tmem_cp_pair_32x128b_warpx4(tsfa + 4 * sg, dsa + (uint64_t)(sg * (kYSfGroup >> 4)));
                tmem_cp_pair_32x128b_warpx4(tsfb + 8 * sg, dsb + (uint64_t)(sg * 2 * (kYSfGroup >> 4)));
                tmem_cp_pair_32x128b_warpx4(tsfb + 8 * sg + 4, dsb + (uint64_t)((sg * 2 + 1) * (kYSfGroup >> 4)));
              }
#pragma unroll
              for (int kk = 0; kk < YK / YUMMA_K; ++kk) {
                const uint64_t dak = da + (uint64_t)(kk * (YUMMA_K >> 4));
                const uint64_t dbk = db + (uint64_t)(kk * (YUMMA_K >> 4));
                const uint32_t accumulate = (kk != 0 || h != 0) ? 1u : (uint32_t)(kb != 0);
                if constexpr (FMT == 2) {
                  constexpr uint32_t idesc = make_idesc_mx(1, 1, 0, 0, 2 * YM, YN, 0, /*e8m0_scales=*/0);
                  mma_mx_pair(2, d_tmem, dak, dbk, idesc, tsfa + 4 * kk, tsfb + 8 * kk, accumulate);
                } else if constexpr (FMT == 1) {
                  const uint32_t id = (uint32_t)(kk & 1) * 2u, sg = (uint32_t)(kk >> 1);
                  const uint32_t idesc = make_idesc_mx(1, 1, 0, 0, 2 * YM, YN, id);
                  mma_mx_pair(1, d_tmem, dak, dbk, idesc, (tsfa + 4 * sg) | (id << 30), (tsfb + 8 * sg) | (id << 30),
                              accumulate);
                } else {
                  const uint32_t idesc = make_idesc_mx(0, 0, 0, 0, 2 * YM, YN, kk);
                  mma_mx_pair(0, d_tmem, dak, dbk, idesc, tsfa | ((uint32_t)kk << 30), tsfb | ((uint32_t)kk << 30),
                              accumulate);
                }
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
        off += kStageStep;
        if (++stage == kYStages) { stage = 0; phase ^= 1u; off = 0; }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  } else if (warp >= kYEpiWarp0) {
    // ---------------- epilogue of this CTA's 128 rows ----------------
    const int q = warp - kYEpiWarp0;           // tensor-memory lane quarter of this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const uint32_t acc_empty0 = map_to_cta(smem_u32(&ctl->acc_empty[0]), 0);
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int m0 = (tile % p.tiles_m) * (2 * YM) + (int)rank * YM;
      const int n0 = (tile / p.tiles_m) * YN;
      const int64_t m = (int64_t)m0 + q * 32 + lane;
      if (lane == 0) ok = mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < YN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * YN + c * 32, r);
        tmem_ld_wait();
        const int64_t ncol = (int64_t)n0 + c * 32;
        if (m >= p.M || ncol >= p.N) continue;
        if (p.out_dtype == QWX_F32) {
          float* o = reinterpret_cast<float*>(p.out) + m * p.N + ncol;
          if (ncol + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<uint4*>(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
          } else {
            for (int j = 0; j < 32 && ncol + j < p.N; ++j) o[j] = __uint_as_float(r[j]);
          }
        } else {
          uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + m * p.N + ncol;
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float x = __uint_as_float(r[2 * j]), y = __uint_as_float(r[2 * j + 1]);
            if (p.out_dtype == QWX_BF16) {
              __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
              w[j] = *reinterpret_cast<uint32_t*>(&h);
            } else {
              __half2 h = __floats2half2_rn(x, y);
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

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // neither CTA frees tensor memory or leaves while the other still uses the pair
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
  if (threadIdx.x == 0 && ctl->abort && p.error_flag) atomicExch(p.error_flag, QWX_ERR_DEVICE_WAIT);
}

// Row-major [rows, 128] matrix of 32-bit words (512-byte scale groups), box [box_rows, 128], no
// swizzle, zero fill outside.
bool encode_groups(CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_tiled();
  if (!fn) return false;
  cuuint64_t dims[2] = {128, rows};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count_y() {
  static int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return v;
  }();
  return n;
}

template <int FMT>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                const MxPairParams& p, int grid, cudaStream_t st) {
  auto kern = gemm_mx_pair_kernel<FMT>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kYSmemBytes) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  kern<<<grid, kYThreads, kYSmemBytes, st>>>(ta, tb, tsa, tsb, p);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

}  // namespace

// a [M, kbytes], b [N, kbytes] codes (K-major); sfa / sfb: the packed scale groups that the
// single-CTA kernel reads (same order: 128-row tiles of A, 224-column tiles of B), with their
// sizes in bytes.  fmt: 0 MXFP8, 1 MXFP4, 2 NVFP4.  The caller has checked the arguments.
int gemm_mx_pair_launch(int fmt, const void* a, const void* b, int64_t M, int64_t N, int64_t kbytes,
                        const void* sfa, size_t sfa_bytes, const void* sfb, size_t sfb_bytes, void* out,
                        int out_dtype, int32_t* error_flag, cudaStream_t st) {
  const int groups = fmt == 2 ? 4 : (fmt == 1 ? 2 : 1);
  CUtensorMap ta, tb, tsa, tsb;
  if (!get_encode_tiled()) return QWX_ERR_NO_DEVICE;
  if (!encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)M, (uint64_t)kbytes, YM, YK) ||
      !encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)N, (uint64_t)kbytes, YNH, YK) ||
      !encode_groups(&tsa, sfa, sfa_bytes / 512, (uint32_t)(kYHalves * groups)) ||
      !encode_groups(&tsb, sfb, sfb_bytes / 512, (uint32_t)(kYHalves * 2 * groups)))
    return QWX_ERR_LAUNCH;
  MxPairParams p;
  p.M = M; p.N = N; p.K = kbytes;
  p.out = out; p.out_dtype = out_dtype; p.error_flag = error_flag;
  p.tiles_m = (int)((M + 2 * YM - 1) / (2 * YM));
  p.tiles_n = (int)((N + YN - 1) / YN);
  const int64_t num_tiles = (int64_t)p.tiles_m * p.tiles_n;
  if (num_tiles > INT32_MAX / 2) return QWX_ERR_SHAPE;
  const int sms = sm_count_y();
  if (sms < 2) return QWX_ERR_NO_DEVICE;
  const int pairs = (int)(num_tiles < sms / 2 ? num_tiles : sms / 2);
  if (fmt == 0) return launch_pair<0>(ta, tb, tsa, tsb, p, 2 * pairs, st);
  if (fmt == 1) return launch_pair<1>(ta, tb, tsa, tsb, p, 2 * pairs, st);
  return launch_pair<2>(ta, tb, tsa, tsb, p, 2 * pairs, st);
}

}  // namespace qwx
