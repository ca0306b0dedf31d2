// MXFP8 block-scaled GEMM on tcgen05 tensor cores, sm_100a:
//
//   out[m, n] = sum_j ( sum_{k in block j} a[m, k] * b[k, n] ) * 2^(ea[m, j] - 127) * 2^(eb[j, n] - 127)
//
// a, b: e4m3 codes; one power-of-two scale (E8M0 byte) per 32 contracted elements of every row
// of A and every column of B; float32 accumulation.  This is what the reference reaches through
// jax.nn.scaled_matmul when both operands are microscaled (qwix/_src/core/mxfp_dot.py:24-79);
// here the scaling happens inside the MMA (`tcgen05.mma.kind::mxf8f6f4.block_scale`), with the
// scales staged in tensor memory.
//
// Structure (one persistent CTA per SM, 256 threads, 128 x 224 output tiles so that two
// accumulators and the scale columns fit the 512 columns of tensor memory):
//   warp 0      producer: A [128 x 128 B] and B [224 x 128 B] by TMA (128-byte swizzle), and
//               the stage's scale bytes (512 B for A, 1 KB for B, already in the order
//               tensor memory wants) by bulk copies, into a 4-stage ring
//   warp 1      MMA issuer: three tcgen05.cp (scales: shared -> tensor memory), then four
//               block-scaled MMAs (M128 N224 K32) per stage; tcgen05 operations of one thread
//               execute in order, so the copies of stage s+1 wait for the MMAs of stage s
//   warp 2      owns the tensor-memory allocation
//   warps 4-7   epilogue: float32 accumulator -> output dtype, while the other accumulator fills
// Every wait is bounded.
//
// The same kernel serves MXFP4 (e2m1 codes packed two per byte, both operands K-major):
// `tcgen05.mma.kind::mxf4.block_scale.scale_vec::2X`, 64 contracted elements (32 bytes) per
// MMA with two scale bytes each, so a 128-byte stage holds 256 elements and eight scale blocks
// per row: two 512-byte scale groups per 128 rows and stage, six tcgen05.cp.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qwix_b200.h"
#include "common.cuh"
#include "sm100.cuh"

namespace qwx {

// gemm_mx_pair.cu: the CTA-pair form for more than 128 rows (both operands K-major, the
// contracted bytes a multiple of 256)
int gemm_mx_pair_launch(int fmt, const void* a, const void* b, int64_t M, int64_t N, int64_t kbytes,
                        const void* sfa, size_t sfa_bytes, const void* sfb, size_t sfb_bytes, void* out,
                        int out_dtype, int32_t* error_flag, cudaStream_t st);

namespace {

using namespace sm100;

constexpr int XM = 128;
constexpr int XN = 224;
constexpr int XK = 128;        // contracted elements (bytes) per stage: four 32-wide scale blocks
constexpr int XUMMA_K = 32;
constexpr int kXStages = 4;
constexpr int kXABytes = XM * XK;            // 16 KB
constexpr int kXBBytes = 256 * XK;           // room for two 128-column halves of a [K, N] tile
constexpr int kXSfaBytes = 512;              // 128 rows x 4 blocks
constexpr int kXSfbBytes = 1024;             // two 128-row groups
constexpr int kXStageBytes = 50 * 1024;      // A + B + scales, rounded up to the swizzle alignment
static_assert(kXABytes + kXBBytes + kXSfaBytes + kXSfbBytes <= kXStageBytes, "stage layout");
// 4-bit codes: twice the scale blocks per stage; B is [N, K] only (224 rows of 128 bytes)
constexpr int kX4BBytes = XN * XK;
static_assert(kXABytes + kX4BBytes + 2 * kXSfaBytes + 2 * kXSfbBytes <= kXStageBytes, "stage layout, 4-bit");
constexpr int kXAccCols = XN;
constexpr int kXSfCol = 2 * kXAccCols;       // scale columns behind the two accumulators: 4 (A) + 8 (B)
constexpr int kXThreads = 256;
constexpr int kXEpiWarp0 = 4;

struct ControlX {
  uint64_t full[kXStages];
  uint64_t empty[kXStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort;
};

constexpr size_t kXSmemBytes = 1024 + (size_t)kXStages * kXStageBytes + sizeof(ControlX);
static_assert(kXSmemBytes <= 227 * 1024, "shared memory of the MX GEMM");

struct MxParams {
  int64_t M, N, K;
  const uint8_t* sfa;      // [tiles_m][K / 128][512]
  const uint8_t* sfb;      // [tiles_n][K / 128][1024]
  void* out;
  int out_dtype;
  int32_t* error_flag;
  int tiles_m, tiles_n;
};

// FMT: 0 = e4m3 codes, E8M0 scale per 32 (MXFP8); 1 = e2m1 codes, E8M0 scale per 32 (MXFP4);
// 2 = e2m1 codes, e4m3 scale per 16 (NVFP4)
template <int BLAYOUT, int FMT>
__global__ void __launch_bounds__(kXThreads, 1)
gemm_mx8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                const MxParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  ControlX* ctl = reinterpret_cast<ControlX*>(smem_raw + (tiles - smem_u32(smem_raw)) +
                                              (size_t)kXStages * kXStageBytes);
  constexpr bool FP4 = FMT != 0;
  static_assert(!FP4 || BLAYOUT == QWX_B_NK, "4-bit operands are K-major");
  constexpr int kSfGroups = FMT == 2 ? 4 : (FMT == 1 ? 2 : 1);   // 512-byte scale groups per 128 rows and stage
  static_assert(kXABytes + (FP4 ? kX4BBytes : kXBBytes) + kSfGroups * (kXSfaBytes + kXSfbBytes) <= kXStageBytes,
                "stage layout");
  static_assert(kXSfCol + 12 * kSfGroups <= 512, "scale columns in tensor memory");
  constexpr int kSfaStage = kSfGroups * kXSfaBytes;
  constexpr int kSfbStage = kSfGroups * kXSfbBytes;
  constexpr int kBStage = FP4 ? kX4BBytes : kXBBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (int)(p.K / XK);                    // p.K: contracted bytes
  const int num_tiles = p.tiles_m * p.tiles_n;
  volatile int* abort = &ctl->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kXStages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->acc_full[a]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[a]), 4);
    }
    ctl->abort = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ---------------- producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    long issued = 0;
    bool ok = true;
    constexpr uint32_t kStageTx =
        kXABytes + (BLAYOUT == QWX_B_NK ? XN * XK : 2 * 128 * XK) + kSfaStage + kSfbStage;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const int m0 = tm * XM, n0 = tn * XN;
      const uint8_t* sfa = p.sfa + (size_t)tm * kblocks * kSfaStage;
      const uint8_t* sfb = p.sfb + (size_t)tn * kblocks * kSfbStage;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort);
          if (ok) {
            const uint32_t bar = smem_u32(&ctl->full[stage]);
            const uint32_t sa = tiles + stage * kXStageBytes;
            const uint32_t sb = sa + kXABytes;
            const uint32_t ssfa = sb + kBStage;
            const uint32_t ssfb = ssfa + kSfaStage;
            mbar_expect_tx(bar, kStageTx);
            tma_load_2d(sa, &tma_a, kb * XK, m0, bar);
            if (BLAYOUT == QWX_B_NK) {
              tma_load_2d(sb, &tma_b, kb * XK, n0, bar);
            } else {
              tma_load_2d(sb, &tma_b, n0, kb * XK, bar);
              tma_load_2d(sb + XK * 128, &tma_b, n0 + 128, kb * XK, bar);
            }
            bulk_load(ssfa, sfa + (size_t)kb * kSfaStage, kSfaStage, bar);
            bulk_load(ssfb, sfb + (size_t)kb * kSfbStage, kSfbStage, bar);
            ++issued;
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == kXStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (lane == 0 && *abort) {
      // Let copies that are still in flight land before the CTA gives up its shared memory.
      long pending = issued < kXStages ? issued : kXStages;
      int s = stage;
      uint32_t ph = phase;
      for (long i = 0; i < pending; ++i) {
        if (--s < 0) { s = kXStages - 1; ph ^= 1u; }
        for (int it = 0; it < 100000; ++it)
          if (mbar_try_wait(smem_u32(&ctl->full[s]), ph)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const uint32_t tsfa = tmem_base + kXSfCol;        // 4 columns per scale group
    const uint32_t tsfb = tsfa + 4 * kSfGroups;       // 8 columns per scale group
    // The issuing thread's own instruction stream is what bounds this kernel (a lone thread
    // issues an instruction every several cycles; four M128 N224 MMAs take 448), so nothing is
    // computed per MMA that can be computed once: descriptors of stage 0 here, the stage's offset
    // (in the descriptors' 16-byte units) as a running sum.
    const uint64_t da0 = make_smem_desc(tiles, 16, 1024);
    const uint64_t db0 = BLAYOUT == QWX_B_NK ? make_smem_desc(tiles + kXABytes, 16, 1024)
                                              : make_smem_desc(tiles + kXABytes, XK * 128, 1024);
    const uint64_t dsa0 = make_smem_desc_plain(tiles + kXABytes + kBStage, 16, 128);
    const uint64_t dsb0 = dsa0 + (uint64_t)(kSfaStage >> 4);
    constexpr uint64_t kStageStep = kXStageBytes >> 4;
    constexpr uint64_t kKStep = BLAYOUT == QWX_B_NK ? (XUMMA_K >> 4) : ((XUMMA_K * 128) >> 4);
    uint64_t off = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort);
        tc_fence_after();
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      const uint32_t d_tmem = tmem_base + acc * kXAccCols;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&ctl->full[stage]), phase, abort);
          if (ok) {
            tc_fence_after();
            const uint64_t da = da0 + off, db = db0 + off, dsa = dsa0 + off, dsb = dsb0 + off;
            // scale bytes: 32 rows of 16 B per 128 operand rows, four 8-row core matrices 128 B apart
#pragma unroll
            for (int sg = 0; sg < kSfGroups; ++sg) {
              tmem_cp_32x128b_warpx4(tsfa + 4 * sg, dsa + (uint64_t)(sg * (kXSfaBytes >> 4)));
              tmem_cp_32x128b_warpx4(tsfb + 8 * sg, dsb + (uint64_t)(sg * (kXSfbBytes >> 4)));
              tmem_cp_32x128b_warpx4(tsfb + 8 * sg + 4, dsb + (uint64_t)(sg * (kXSfbBytes >> 4) + (512 >> 4)));
            }
#pragma unroll
            for (int kk = 0; kk < XK / XUMMA_K; ++kk) {
              const uint64_t dak = da + (uint64_t)(kk * (XUMMA_K >> 4));
              const uint64_t dbk = db + (uint64_t)kk * kKStep;
              const uint32_t accumulate = kk != 0 ? 1u : (uint32_t)(kb != 0);
              if constexpr (FMT == 2) {
                // four scale bytes per MMA: a word each
                constexpr uint32_t idesc = make_idesc_mx(1, 1, 0, 0, XM, XN, 0, /*e8m0_scales=*/0);
                mma_nvf4_ss(d_tmem, dak, dbk, idesc, tsfa + 4 * kk, tsfb + 8 * kk, accumulate);
              } else if constexpr (FMT == 1) {
                // two scale bytes per MMA: bytes 0-1 or 2-3 of the word, a word per two MMAs
                const uint32_t id = (uint32_t)(kk & 1) * 2u, sg = (uint32_t)(kk >> 1);
                const uint32_t idesc = make_idesc_mx(1, 1, 0, 0, XM, XN, id);
                mma_mx4_ss(d_tmem, dak, dbk, idesc, (tsfa + 4 * sg) | (id << 30), (tsfb + 8 * sg) | (id << 30),
                           accumulate);
              } else {
                const uint32_t idesc = make_idesc_mx(0, 0, 0, BLAYOUT == QWX_B_KN ? 1 : 0, XM, XN, kk);
                // which of the word's four bytes: in the descriptor and in the two top bits of the addresses
                mma_mx_ss(d_tmem, dak, dbk, idesc, tsfa | ((uint32_t)kk << 30), tsfb | ((uint32_t)kk << 30),
                          accumulate);
              }
            }
            mma_commit(smem_u32(&ctl->empty[stage]));
            if (kb == kblocks - 1) mma_commit(smem_u32(&ctl->acc_full[acc]));
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        off += kStageStep;
        if (++stage == kXStages) { stage = 0; phase ^= 1u; off = 0; }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  } else if (warp >= kXEpiWarp0) {
    // ---------------- epilogue ----------------
    const int q = warp - kXEpiWarp0;           // tensor-memory lane quarter of this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile % p.tiles_m) * XM;
      const int n0 = (tile / p.tiles_m) * XN;
      const int64_t m = (int64_t)m0 + q * 32 + lane;
      if (lane == 0) ok = mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < XN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * kXAccCols + c * 32, r);
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
      if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && ctl->abort && p.error_flag) atomicExch(p.error_flag, QWX_ERR_DEVICE_WAIT);
}

// Scales (powers of two in a float dtype) -> E8M0 bytes in the order the kernel stages them:
// per operand tile of `tile_rows` rows and per 128 contracted elements, groups of 128 rows, each
// 512 bytes: byte (r % 32) * 16 + (r / 32) * 4 + j for row r of the group and 32-wide block j.
// `k_major`: scale array is [K / 32, rows] (a [K, N] weight) instead of [rows, K / 32].
// `stage_groups`: 512-byte groups per 128 rows and stage: 1 (four blocks per stage, 8-bit codes)
// or 2 (eight blocks per stage, 4-bit codes; the stage's groups of one operand tile lie
// [group][128-row part]).
__global__ void mx_pack_scales_kernel(const void* __restrict__ scale, int dtype, int64_t rows,
                                      int64_t blocks, int k_major, int tile_rows, int stage_groups,
                                      int e4m3_bytes, uint8_t* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * blocks) return;
  // consecutive threads read consecutive elements of the scale array
  const int64_t r = k_major ? i % rows : i / blocks;
  const int64_t j = k_major ? i / rows : i % blocks;
  float s;
  if (dtype == QWX_F32) s = reinterpret_cast<const float*>(scale)[i];
  else if (dtype == QWX_BF16) s = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(scale)[i]);
  else s = __half2float(reinterpret_cast<const __half*>(scale)[i]);
  // the biased exponent of a power of two, or the e4m3 byte of a scale that is an e4m3 value
  const uint8_t e = e4m3_bytes ? (uint8_t)__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3)
                               : (uint8_t)((__float_as_uint(s) >> 23) & 0xffu);
  const int groups = (tile_rows + 127) / 128;
  const int64_t tile = r / tile_rows, rr = r % tile_rows;
  const int64_t g = rr / 128, r128 = rr % 128;
  const int64_t kb = j / (4 * stage_groups), sg = (j / 4) % stage_groups, jj = j % 4;
  const int64_t kblocks = blocks / (4 * stage_groups);
  out[(((tile * kblocks + kb) * stage_groups + sg) * groups + g) * 512 + (r128 % 32) * 16 +
      (r128 / 32) * 4 + jj] = e;
}

// The row-major case ([rows, blocks], an activation: packed on every call) four blocks per thread:
// one vector load of four scales, one 32-bit store of their bytes.
template <typename S>
__global__ void mx_pack_scales_rows_kernel(const S* __restrict__ scale, int64_t rows, int64_t quads,
                                           int tile_rows, int stage_groups, int e4m3_bytes,
                                           uint32_t* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * quads) return;
  const int64_t r = i / quads, jq = i % quads;          // row, group of four blocks
  float s[4];
  if constexpr (sizeof(S) == 4) {
    const float4 v = reinterpret_cast<const float4*>(scale)[i];
    s[0] = v.x; s[1] = v.y; s[2] = v.z; s[3] = v.w;
  } else {
    const uint2 v = reinterpret_cast<const uint2*>(scale)[i];
    const uint32_t w[2] = {v.x, v.y};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint16_t h = (uint16_t)(w[k >> 1] >> (16 * (k & 1)));
      if constexpr (std::is_same<S, __nv_bfloat16>::value) s[k] = __uint_as_float((uint32_t)h << 16);
      else s[k] = __half2float(__ushort_as_half(h));
    }
  }
  uint32_t word = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t e = e4m3_bytes ? (uint32_t)__nv_cvt_float_to_fp8(s[k], __NV_SATFINITE, __NV_E4M3)
                                  : ((__float_as_uint(s[k]) >> 23) & 0xffu);
    word |= e << (8 * k);
  }
  const int groups = (tile_rows + 127) / 128;
  const int64_t tile = r / tile_rows, rr = r % tile_rows;
  const int64_t g = rr / 128, r128 = rr % 128;
  const int64_t kb = jq / stage_groups, sg = jq % stage_groups;
  const int64_t kblocks = quads / stage_groups;
  out[((((tile * kblocks + kb) * stage_groups + sg) * groups + g) * 512 + (r128 % 32) * 16 + (r128 / 32) * 4) >> 2] = word;
}

// Packs `scale` ([rows, blocks] or, k_major, [blocks, rows]) into the kernels' staging order.
int pack_scales(const void* scale, int scale_dtype, int64_t rows, int64_t blocks, int k_major,
                int tile_rows, int stage_groups, int e4m3_bytes, void* out, size_t need, cudaStream_t st) {
  // rows past the operand read a zero byte (2^-127, or e4m3 zero) against zero-filled codes
  // (nothing is left unwritten when whole 128-row groups are packed)
  if ((rows % tile_rows != 0 || tile_rows % 128 != 0) && cudaMemsetAsync(out, 0, need, st) != cudaSuccess)
    return QWX_ERR_LAUNCH;
  if (!k_major && blocks % 4 == 0 && !(reinterpret_cast<uintptr_t>(scale) & 15)) {
    const int64_t quads = blocks / 4, n = rows * quads;
    const unsigned grid = (unsigned)((n + 255) / 256);
    if (scale_dtype == QWX_F32)
      mx_pack_scales_rows_kernel<float><<<grid, 256, 0, st>>>((const float*)scale, rows, quads, tile_rows,
                                                              stage_groups, e4m3_bytes, (uint32_t*)out);
    else if (scale_dtype == QWX_BF16)
      mx_pack_scales_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          (const __nv_bfloat16*)scale, rows, quads, tile_rows, stage_groups, e4m3_bytes, (uint32_t*)out);
    else
      mx_pack_scales_rows_kernel<__half><<<grid, 256, 0, st>>>((const __half*)scale, rows, quads, tile_rows,
                                                               stage_groups, e4m3_bytes, (uint32_t*)out);
  } else {
    const int64_t n = rows * blocks;
    mx_pack_scales_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
        scale, scale_dtype, rows, blocks, k_major, tile_rows, stage_groups, e4m3_bytes, (uint8_t*)out);
  }
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

int sm_count_x() {
  static int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return v;
  }();
  return n;
}

// Unpacked 4-bit codes (one per byte) -> two per byte along K (even index in the low nibble),
// rows K-major: out[r, k / 2].  `k_major`: the codes are [K, rows] (a [K, N] weight).
__global__ void mx4_pack_codes_kernel(const uint8_t* __restrict__ codes, int64_t rows, int64_t K,
                                      int k_major, uint8_t* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // output byte
  const int64_t kh = K / 2;
  if (i >= rows * kh) return;
  if (k_major) {
    // consecutive threads take consecutive rows: both reads run along the fast axis
    const int64_t r = i % rows, k2 = i / rows;
    const uint8_t lo = codes[(2 * k2) * rows + r], hi = codes[(2 * k2 + 1) * rows + r];
    out[r * kh + k2] = (uint8_t)((lo & 0xf) | (hi << 4));
  } else {
    const uchar2 c = reinterpret_cast<const uchar2*>(codes)[i];
    out[i] = (uint8_t)((c.x & 0xf) | (c.y << 4));
  }
}

// The row-major case sixteen codes at a time (an activation: packed on every call).
__global__ void mx4_pack_codes_vec_kernel(const uint4* __restrict__ codes, int64_t nvec,
                                          uint2* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const uint4 c = codes[i];
  // bytes b0 b1 b2 b3 of a word -> (b0 | b1 << 4) and (b2 | b3 << 4) in its low two bytes
  auto squeeze = [](uint32_t w) {
    const uint32_t t = (w & 0x000f000fu) | ((w >> 4) & 0x00f000f0u);   // bytes 0 and 2 hold the pairs
    return (t & 0xffu) | ((t >> 8) & 0xff00u);
  };
  out[i] = make_uint2(squeeze(c.x) | (squeeze(c.y) << 16), squeeze(c.z) | (squeeze(c.w) << 16));
}

template <int BLAYOUT, int FMT>
int launch_mx(const CUtensorMap& ta, const CUtensorMap& tb, const MxParams& p, int grid, cudaStream_t st) {
  auto kern = gemm_mx8_kernel<BLAYOUT, FMT>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kXSmemBytes) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  kern<<<grid, kXThreads, kXSmemBytes, st>>>(ta, tb, p);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

int tile_rows_of(int operand) { return operand == 0 ? XM : XN; }

}  // namespace
}  // namespace qwx

using namespace qwx;

extern "C" size_t qwx_mx_scales_packed_bytes(int operand, int64_t rows, int64_t K) {
  if (rows <= 0 || K <= 0 || K % XK || (operand != 0 && operand != 1)) return 0;
  const int tr = tile_rows_of(operand);
  const int64_t tiles = (rows + tr - 1) / tr;
  return (size_t)tiles * (size_t)(K / XK) * (size_t)((tr + 127) / 128) * 512;
}

extern "C" int qwx_mx_pack_scales(int operand, const void* scale, int scale_dtype, int64_t rows,
                                  int64_t K, int k_major, void* out, size_t out_bytes,
                                  qwx_stream_t stream) {
  if (!scale || !out) return QWX_ERR_NULL;
  if (operand != 0 && operand != 1) return QWX_ERR_SHAPE;
  if (rows <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (K % XK) return QWX_ERR_UNSUPPORTED;
  if (scale_dtype != QWX_F32 && scale_dtype != QWX_BF16 && scale_dtype != QWX_F16) return QWX_ERR_DTYPE;
  const size_t need = qwx_mx_scales_packed_bytes(operand, rows, K);
  if (out_bytes < need) return QWX_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(out) & 15) return QWX_ERR_ALIGN;
  return pack_scales(scale, scale_dtype, rows, K / 32, k_major ? 1 : 0, tile_rows_of(operand), 1, 0, out, need,
                     (cudaStream_t)stream);
}

extern "C" int qwx_gemm_mx8(const void* a, const void* b, int b_layout, int64_t M, int64_t N,
                            int64_t K, const void* sfa_packed, const void* sfb_packed, void* out,
                            int out_dtype, int32_t* error_flag, qwx_stream_t stream) {
  if (!a || !b || !sfa_packed || !sfb_packed || !out) return QWX_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (M > INT32_MAX - XM || N > INT32_MAX - 256 || K > INT32_MAX - XK) return QWX_ERR_SHAPE;
  if (b_layout != QWX_B_KN && b_layout != QWX_B_NK) return QWX_ERR_SHAPE;
  if (K % XK) return QWX_ERR_UNSUPPORTED;      // whole stages of four scale blocks
  if (out_dtype != QWX_BF16 && out_dtype != QWX_F32 && out_dtype != QWX_F16) return QWX_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) ||
      (reinterpret_cast<uintptr_t>(sfa_packed) & 15) || (reinterpret_cast<uintptr_t>(sfb_packed) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return QWX_ERR_ALIGN;
  if (b_layout == QWX_B_KN && (N % 16)) return QWX_ERR_ALIGN;
  if (b_layout == QWX_B_NK && M > XM && K % 256 == 0)
    return gemm_mx_pair_launch(0, a, b, M, N, K, sfa_packed, qwx_mx_scales_packed_bytes(0, M, K), sfb_packed,
                               qwx_mx_scales_packed_bytes(1, N, K), out, out_dtype, error_flag,
                               (cudaStream_t)stream);

  CUtensorMap ta, tb;
  if (!get_encode_tiled()) return QWX_ERR_NO_DEVICE;
  if (!encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)M, (uint64_t)K, XM, XK))
    return QWX_ERR_LAUNCH;
  const bool ok_b = b_layout == QWX_B_NK
                        ? encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)N, (uint64_t)K, XN, XK)
                        : encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)K, (uint64_t)N, XK, 128);
  if (!ok_b) return QWX_ERR_LAUNCH;

  MxParams p;
  p.M = M; p.N = N; p.K = K;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa_packed);
  p.sfb = reinterpret_cast<const uint8_t*>(sfb_packed);
  p.out = out; p.out_dtype = out_dtype; p.error_flag = error_flag;
  p.tiles_m = (int)((M + XM - 1) / XM);
  p.tiles_n = (int)((N + XN - 1) / XN);
  const int64_t num_tiles = (int64_t)p.tiles_m * p.tiles_n;
  if (num_tiles > INT32_MAX / 2) return QWX_ERR_SHAPE;
  const int sms = sm_count_x();
  if (sms <= 0) return QWX_ERR_NO_DEVICE;
  const int grid = (int)(num_tiles < sms ? num_tiles : sms);
  cudaStream_t st = (cudaStream_t)stream;
  return b_layout == QWX_B_NK ? launch_mx<QWX_B_NK, 0>(ta, tb, p, grid, st)
                              : launch_mx<QWX_B_KN, 0>(ta, tb, p, grid, st);
}

// ---- MXFP4: e2m1 codes, two per byte, 256 contracted elements per stage ----------------------

extern "C" size_t qwx_mx4_scales_packed_bytes(int operand, int64_t rows, int64_t K) {
  if (rows <= 0 || K <= 0 || K % (2 * XK) || (operand != 0 && operand != 1)) return 0;
  const int tr = tile_rows_of(operand);
  const int64_t tiles = (rows + tr - 1) / tr;
  return (size_t)tiles * (size_t)(K / (2 * XK)) * 2 * (size_t)((tr + 127) / 128) * 512;
}

extern "C" int qwx_mx4_pack_scales(int operand, const void* scale, int scale_dtype, int64_t rows,
                                   int64_t K, int k_major, void* out, size_t out_bytes,
                                   qwx_stream_t stream) {
  if (!scale || !out) return QWX_ERR_NULL;
  if (operand != 0 && operand != 1) return QWX_ERR_SHAPE;
  if (rows <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (K % (2 * XK)) return QWX_ERR_UNSUPPORTED;
  if (scale_dtype != QWX_F32 && scale_dtype != QWX_BF16 && scale_dtype != QWX_F16) return QWX_ERR_DTYPE;
  const size_t need = qwx_mx4_scales_packed_bytes(operand, rows, K);
  if (out_bytes < need) return QWX_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(out) & 15) return QWX_ERR_ALIGN;
  return pack_scales(scale, scale_dtype, rows, K / 32, k_major ? 1 : 0, tile_rows_of(operand), 2, 0, out, need,
                     (cudaStream_t)stream);
}

extern "C" int qwx_mx4_pack_codes(const void* codes, int64_t rows, int64_t K, int k_major, void* out,
                                  qwx_stream_t stream) {
  if (!codes || !out) return QWX_ERR_NULL;
  if (rows <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (K % 2) return QWX_ERR_UNSUPPORTED;
  if (!k_major && (reinterpret_cast<uintptr_t>(codes) & 1)) return QWX_ERR_ALIGN;
  const int64_t n = rows * (K / 2);
  if (!k_major && (rows * K) % 16 == 0 && !(reinterpret_cast<uintptr_t>(codes) & 15) &&
      !(reinterpret_cast<uintptr_t>(out) & 7)) {
    const int64_t nvec = rows * K / 16;
    mx4_pack_codes_vec_kernel<<<(unsigned)((nvec + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (const uint4*)codes, nvec, (uint2*)out);
    QWX_CHECK_LAUNCH();
    return QWX_OK;
  }
  mx4_pack_codes_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)codes, rows, K, k_major ? 1 : 0, (uint8_t*)out);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

namespace {
template <int FMT>
int gemm_fp4(const void* a_packed, const void* b_packed, int64_t M, int64_t N, int64_t K,
             const void* sfa_packed, const void* sfb_packed, void* out, int out_dtype,
             int32_t* error_flag, qwx_stream_t stream) {
  if (!a_packed || !b_packed || !sfa_packed || !sfb_packed || !out) return QWX_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (M > INT32_MAX - XM || N > INT32_MAX - 256 || K > INT32_MAX - 2 * XK) return QWX_ERR_SHAPE;
  if (K % (2 * XK)) return QWX_ERR_UNSUPPORTED;      // whole 128-byte stages
  if (out_dtype != QWX_BF16 && out_dtype != QWX_F32 && out_dtype != QWX_F16) return QWX_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(a_packed) & 15) || (reinterpret_cast<uintptr_t>(b_packed) & 15) ||
      (reinterpret_cast<uintptr_t>(sfa_packed) & 15) || (reinterpret_cast<uintptr_t>(sfb_packed) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return QWX_ERR_ALIGN;
  const int64_t kbytes = K / 2;
  if (M > XM && kbytes % 256 == 0) {
    const size_t na = FMT == 2 ? qwx_nvfp4_scales_packed_bytes(0, M, K) : qwx_mx4_scales_packed_bytes(0, M, K);
    const size_t nb = FMT == 2 ? qwx_nvfp4_scales_packed_bytes(1, N, K) : qwx_mx4_scales_packed_bytes(1, N, K);
    return gemm_mx_pair_launch(FMT, a_packed, b_packed, M, N, kbytes, sfa_packed, na, sfb_packed, nb, out,
                               out_dtype, error_flag, (cudaStream_t)stream);
  }
  CUtensorMap ta, tb;
  if (!get_encode_tiled()) return QWX_ERR_NO_DEVICE;
  if (!encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_packed, (uint64_t)M, (uint64_t)kbytes, XM, XK) ||
      !encode_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_packed, (uint64_t)N, (uint64_t)kbytes, XN, XK))
    return QWX_ERR_LAUNCH;
  MxParams p;
  p.M = M; p.N = N; p.K = kbytes;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa_packed);
  p.sfb = reinterpret_cast<const uint8_t*>(sfb_packed);
  p.out = out; p.out_dtype = out_dtype; p.error_flag = error_flag;
  p.tiles_m = (int)((M + XM - 1) / XM);
  p.tiles_n = (int)((N + XN - 1) / XN);
  const int64_t num_tiles = (int64_t)p.tiles_m * p.tiles_n;
  if (num_tiles > INT32_MAX / 2) return QWX_ERR_SHAPE;
  const int sms = sm_count_x();
  if (sms <= 0) return QWX_ERR_NO_DEVICE;
  const int grid = (int)(num_tiles < sms ? num_tiles : sms);
  return launch_mx<QWX_B_NK, FMT>(ta, tb, p, grid, (cudaStream_t)stream);
}
}  // namespace

extern "C" int qwx_gemm_mx4(const void* a_packed, const void* b_packed, int64_t M, int64_t N,
                            int64_t K, const void* sfa_packed, const void* sfb_packed, void* out,
                            int out_dtype, int32_t* error_flag, qwx_stream_t stream) {
  return gemm_fp4<1>(a_packed, b_packed, M, N, K, sfa_packed, sfb_packed, out, out_dtype, error_flag, stream);
}

// ---- NVFP4: e2m1 codes, an e4m3 scale per 16 contracted elements ------------------------------

extern "C" size_t qwx_nvfp4_scales_packed_bytes(int operand, int64_t rows, int64_t K) {
  if (rows <= 0 || K <= 0 || K % (2 * XK) || (operand != 0 && operand != 1)) return 0;
  const int tr = tile_rows_of(operand);
  const int64_t tiles = (rows + tr - 1) / tr;
  return (size_t)tiles * (size_t)(K / (2 * XK)) * 4 * (size_t)((tr + 127) / 128) * 512;
}

extern "C" int qwx_nvfp4_pack_scales(int operand, const void* scale, int scale_dtype, int64_t rows,
                                     int64_t K, int k_major, void* out, size_t out_bytes,
                                     qwx_stream_t stream) {
  if (!scale || !out) return QWX_ERR_NULL;
  if (operand != 0 && operand != 1) return QWX_ERR_SHAPE;
  if (rows <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (K % (2 * XK)) return QWX_ERR_UNSUPPORTED;
  if (scale_dtype != QWX_F32 && scale_dtype != QWX_BF16 && scale_dtype != QWX_F16) return QWX_ERR_DTYPE;
  const size_t need = qwx_nvfp4_scales_packed_bytes(operand, rows, K);
  if (out_bytes < need) return QWX_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(out) & 15) return QWX_ERR_ALIGN;
  return pack_scales(scale, scale_dtype, rows, K / 16, k_major ? 1 : 0, tile_rows_of(operand), 4, 1, out, need,
                     (cudaStream_t)stream);
}

extern "C" int qwx_gemm_nvfp4(const void* a_packed, const void* b_packed, int64_t M, int64_t N,
                              int64_t K, const void* sfa_packed, const void* sfb_packed, void* out,
                              int out_dtype, int32_t* error_flag, qwx_stream_t stream) {
  return gemm_fp4<2>(a_packed, b_packed, M, N, K, sfa_packed, sfb_packed, out, out_dtype, error_flag, stream);
}
