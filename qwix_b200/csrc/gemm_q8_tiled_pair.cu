// Quantized GEMM with scales that change along K and zero-point corrections, on CTA pairs
// (tcgen05 cta_group::2), sm_100a.  Same contract as the single-CTA form in gemm_q8_tiled.cu:
//
//   out[m, n] = sum_t ( acc_t[m, n] - corr_row[m, t] * corr_col[t, n] ) * sa[m, t] * sb[t, n]
//   acc_t[m, n] = sum_{k in K tile t} a[m, k] * b[k, n]
//
// (qwix/_src/core/dot_general.py:187-203 tiled contraction, :228-253 zero-point terms, :255-259
// scale and sum over tiles, :278-399 the loop form.)  Two CTAs on the two SMs of a TPC compute
// one 256 x 256 output tile: each holds 128 rows of A and 128 columns of B per K block (the
// 32 KB a 128 x 128 tile needs, for twice the products per SM), and 128 accumulator rows x
// 256 columns in tensor memory, twice: the tensor cores fill one accumulator with K tile t+1
// while the epilogue warps drain K tile t from the other.
//
// The epilogue is the pace-setter when the K tile is short, so it is written for issue slots
// and for the float32 pipe (three float operations and one integer add per value on 128 lanes
// per clock: 1024 clocks per K tile is its floor, twice the 512 the MMAs of a 128-wide K tile take):
//   * eight epilogue warps per CTA, two per tensor-memory lane quarter, 128 columns each; a
//     thread owns one output row and keeps 128 running float32 sums in registers (the CTA's
//     registers are re-split with setmaxnreg: 232 per epilogue thread, 40 per control thread,
//     which adds up to the 168 per thread the CTA was launched with).  A warp's tensor-memory
//     loads complete one after the other, about 95 clocks per 32 x 32 words with no MMA
//     running, so one register buffer serves.  Sixteen warps of 64 columns (112 / 24
//     registers, which spills) measured twice as slow at a 128-wide K tile;
//   * the variant is a template parameter, not a run-time branch in the inner loop;
//   * int8 with |acc| <= 2^22 guaranteed: int32 -> float32 by the exact magic-number add,
//     for 128-wide K tiles alternating with cvt, which runs on another pipe (527 -> 459 us at
//     4096 x 8192 x 8192; with 256-wide tiles the plain form is ahead, 308 vs 319 us)
//     (starting the accumulators at the magic bits, restored with tcgen05.st after each drain,
//     saves the integer add but measured slower: the hand-back then waits for the stores);
//   * the three float operations per value (subtract, times sa, multiply-add with sb) are
//     the packed two-lane forms (add/mul/fma .f32x2): half the issue slots, same rounding;
//   * the scales of the next K tile are fetched and this one's staged in shared memory while
//     the first tensor-memory load is in flight;
//   * the hand-back of an accumulator is a relaxed arrive: what it orders is the tensor-memory
//     traffic, which tcgen05.wait and tcgen05.fence order; a release at cluster scope would
//     also wait for the scale loads in flight, once per K tile.
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
// A stage holds two 128-wide K blocks ([A k0][A k1][B k0][B k1]): one round trip between the two
// CTAs' barriers per eight MMAs.  With one block per stage (six stages of 32 KB) the round trips
// were what wide K tiles waited for.
constexpr int kQHalves = 2;
constexpr int kQStages = 3;
constexpr int kQABytes = QM * QK;
constexpr int kQBBytes = QNH * QK;
constexpr int kQStageBytes = kQHalves * (kQABytes + kQBBytes);
#ifndef QWX_TP_EPI_WARPS
#define QWX_TP_EPI_WARPS 8
#endif
constexpr int kQEpiWarp0 = 4;
constexpr int kQEpiWarps = QWX_TP_EPI_WARPS;        // 8 or 16: two or four per tensor-memory lane quarter
constexpr int kQThreads = 32 * (kQEpiWarp0 + kQEpiWarps);   // one control warpgroup + the epilogue warpgroups
constexpr int QCW = QN / (kQEpiWarps / 4);          // columns one epilogue warp drains (128 or 64)
constexpr int QVPL = QCW / 32;                      // scale values a lane stages per K tile
// setmaxnreg moves registers inside what the CTA was launched with (threads x the launch count,
// 168 for 384 threads, 96 for 640): control threads give up what the epilogue threads claim.
constexpr int kQRegsControl = kQEpiWarps == 8 ? 40 : 24;
constexpr int kQRegsEpilogue = kQEpiWarps == 8 ? 232 : 112;
constexpr int kQRegsLaunch = kQEpiWarps == 8 ? 168 : 96;
static_assert(128 * kQRegsControl + 32 * kQEpiWarps * kQRegsEpilogue <= kQThreads * kQRegsLaunch,
              "the claim would wait for registers that are never released");

// Epilogue variants (template parameter).
constexpr int kModeFast = 0;       // int8, |acc| < 2^22, no zero points: magic-number conversion
constexpr int kModeCvt = 1;        // cvt (int8) or float accumulators, no zero points
constexpr int kModeCorr = 2;       // int8 with the rank-1 zero-point term, cvt
constexpr int kModeRef = 3;        // the reference's rounding after every step
constexpr int kModeRefCorr = 4;
constexpr int kModeMix = 5;        // as kModeFast, every other group of four through cvt: the two
                                   // conversions run on different pipes, and with a 128-wide K tile
                                   // the epilogue is what the tile waits for

struct ControlQ {
  uint64_t full[kQStages];
  uint64_t empty[kQStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort;
  alignas(16) float sb[kQEpiWarps][QCW];    // per epilogue warp: the scales of the K tile being drained
  alignas(16) int32_t zc[kQEpiWarps][QCW];
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
  int scale_vec;            // four scales / corrections of consecutive columns load as one vector
};

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

constexpr uint32_t kMagicBits = 0x4B400000u;      // float32 1.5 * 2^23
constexpr float kMagic = 12582912.0f;

// tcgen05.wait::ld that names the registers the load fills, so that no use of them is
// scheduled ahead of it.
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                 "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]),
                 "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]),
                 "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                 "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]),
                 "+r"(r[31])
               :
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
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
    } else if (MODE == kModeFast || (MODE == kModeMix && (g & 1))) {
      // |acc| <= 2^22: the bits kMagicBits + acc are the float32 value kMagic + acc, exactly
      const float2 magic = make_float2(-kMagic, -kMagic);
      f0 = __fadd2_rn(make_float2(__uint_as_float(kMagicBits + r[4 * g]), __uint_as_float(kMagicBits + r[4 * g + 1])), magic);
      f1 = __fadd2_rn(make_float2(__uint_as_float(kMagicBits + r[4 * g + 2]), __uint_as_float(kMagicBits + r[4 * g + 3])), magic);
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
  const int kstages = (kblocks + kQHalves - 1) / kQHalves;
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
        for (int sb2 = 0; sb2 < kstages && ok; ++sb2) {
          if (lane == 0) {
            ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort);
            if (ok) {
              const uint32_t sa = tiles + stage * kQStageBytes;
              const uint32_t sb = sa + kQHalves * kQABytes;
              if (rank == 0) mbar_expect_tx(smem_u32(&ctl->full[stage]), 2 * kQStageBytes);
              const uint32_t bar = full0 + stage * 8;
#pragma unroll
              for (int h = 0; h < kQHalves; ++h) {
                const int k0 = (kQHalves * sb2 + h) * QK;     // past K (an odd count of blocks): zeros
                tma_load_2d_pair(sa + h * kQABytes, &tma_a, k0, m0, bar);
                if (BLAYOUT == QWX_B_NK) tma_load_2d_pair(sb + h * kQBBytes, &tma_b, k0, n0, bar);
                else tma_load_2d_pair(sb + h * kQBBytes, &tma_b, n0, k0, bar);
              }
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
        int kb = 0;                 // K block inside the scale tile
        for (int sb2 = 0; sb2 < kstages && ok; ++sb2) {
          if (lane == 0) {
            ok = mbar_wait(smem_u32(&ctl->full[stage]), phase, abort);
            if (ok) {
              tc_fence_after();
#pragma unroll
              for (int h = 0; h < kQHalves; ++h) {
                if (kQHalves * sb2 + h >= kblocks) break;    // the zero block behind an odd count
                if (kb == 0) {
                  // a scale tile starts: its accumulator has to be drained
                  ok = mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort);
                  if (!ok) break;
                  tc_fence_after();
                }
                const uint32_t sa = tiles + stage * kQStageBytes + h * kQABytes;
                const uint32_t sb = tiles + stage * kQStageBytes + kQHalves * kQABytes + h * kQBBytes;
#pragma unroll
                for (int kk = 0; kk < QK / QUMMA_K; ++kk) {
                  const uint64_t da = make_smem_desc(sa + kk * QUMMA_K, 16, 1024);
                  const uint64_t db = BLAYOUT == QWX_B_NK
                                          ? make_smem_desc(sb + kk * QUMMA_K, 16, 1024)
                                          : make_smem_desc(sb + kk * QUMMA_K * 128, QK * 128, 1024);
                  mma_ss_pair<KIND>(tmem_base + acc * QN, da, db, idesc, kb != 0 || kk != 0);
                }
                if (++kb == p.kb_per_tile) {
                  kb = 0;
                  mma_commit_pair(smem_u32(&ctl->acc_full[acc]));
                  mma_commit_pair(acc_full_peer + acc * 8);
                  if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                }
              }
              if (ok) {
                mma_commit_pair(smem_u32(&ctl->empty[stage]));
                mma_commit_pair(empty_peer + stage * 8);
              }
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          acc = __shfl_sync(0xffffffffu, acc, 0);
          acc_phase = __shfl_sync(0xffffffffu, acc_phase, 0);
          kb = __shfl_sync(0xffffffffu, kb, 0);
          if (++stage == kQStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    // ---------------- epilogue: drain one accumulator per K tile, keep running sums -----------
    regs_claim<kQRegsEpilogue>();
    const int ew = warp - kQEpiWarp0;         // epilogue warp
    const int q = warp & 3;                   // tensor-memory lane quarter of this warp
    const int ch = ew >> 2;                   // which QCW columns of the tile
    constexpr bool kCorr = MODE == kModeCorr || MODE == kModeRefCorr;
    const uint32_t acc_empty0 = map_to_cta(smem_u32(&ctl->acc_empty[0]), 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;

    const uint32_t tmem_warp = tmem_base + ((uint32_t)(q * 32) << 16) + ch * QCW;   // + acc * QN

    // Scales and correction factors of one (output tile, K tile): QVPL consecutive columns
    // per lane for the warp's shared copy, one row value per lane.
    // What is kept between the prefetch and its use one K tile later is the loaded bits
    // themselves: a conversion right behind a load makes the (in-order) warp wait for that load
    // on the spot, once per K tile (16-bit scales measured 110 us more per 4096 x 8192 x 8192
    // call that way).  Representations: 0 = float32 bits, 1 = two bfloat16 per word, 2 = one
    // 16-bit value of p.scale_dtype per word.
    struct Prefetch {
      uint32_t sb[QVPL];
      int32_t zc[QVPL];
      uint32_t sa;
      int32_t zr;
    };
    struct Where {      // what a lane reads for one output tile
      int m, n;         // its row; the first of its columns
      bool rin, nin;
    };
    auto where = [&](int tile) {
      Where w;
      w.m = (tile % p.tiles_m) * (2 * QM) + (int)rank * QM + q * 32 + lane;
      w.n = (tile / p.tiles_m) * QN + ch * QCW + lane * QVPL;
      w.rin = w.m < p.M;
      w.nin = w.n < p.N;
      return w;
    };
    const bool vec = p.scale_vec != 0;
    const bool f32s = p.scale_dtype == QWX_F32;
    const int sb_rep = (!p.sb || f32s) ? 0 : ((vec && p.scale_dtype == QWX_BF16) ? 1 : 2);
    const int sa_rep = (!p.sa || f32s) ? 0 : 2;
    const uint32_t one16 = p.scale_dtype == QWX_BF16 ? 0x3F80u : 0x3C00u;
    const uint32_t sb_one = sb_rep == 0 ? 0x3F800000u : (sb_rep == 1 ? 0x3F803F80u : one16);
    const uint32_t sa_one = sa_rep == 0 ? 0x3F800000u : one16;
    auto raw = [&](const void* ptr, int64_t i) -> uint32_t {
      return f32s ? __float_as_uint(__ldg(reinterpret_cast<const float*>(ptr) + i))
                  : (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(ptr) + i);
    };
    auto widen = [&](uint32_t bits, int rep) -> float {
      if (rep == 0) return __uint_as_float(bits);
      if (p.scale_dtype == QWX_BF16) return __uint_as_float(bits << 16);
      return __half2float(__ushort_as_half((unsigned short)bits));
    };
    auto fetch = [&](const Where& w, int t) {
      Prefetch f;
#pragma unroll
      for (int k = 0; k < QVPL; ++k) { f.sb[k] = sb_one; f.zc[k] = 0; }
      const int64_t at = (int64_t)t * p.N + w.n;
      if (p.sb && w.nin) {
        const int64_t i = p.sb_tiled ? at : (int64_t)w.n;
        if (vec && f32s) {
          const float* src = reinterpret_cast<const float*>(p.sb) + i;
          if (QVPL == 4) {
            const uint4 u = __ldg(reinterpret_cast<const uint4*>(src));
            f.sb[0] = u.x; f.sb[1] = u.y; f.sb[QVPL - 2] = u.z; f.sb[QVPL - 1] = u.w;
          } else {
            const uint2 u = __ldg(reinterpret_cast<const uint2*>(src));
            f.sb[0] = u.x; f.sb[1] = u.y;
          }
        } else if (sb_rep == 1) {
          const uint16_t* src = reinterpret_cast<const uint16_t*>(p.sb) + i;
          if (QVPL == 4) {
            const uint2 u = __ldg(reinterpret_cast<const uint2*>(src));
            f.sb[0] = u.x; f.sb[1] = u.y;
          } else {
            f.sb[0] = __ldg(reinterpret_cast<const uint32_t*>(src));
          }
        } else {
#pragma unroll
          for (int k = 0; k < QVPL; ++k)
            if (w.n + k < p.N) f.sb[k] = raw(p.sb, i + k);
        }
      }
      if (kCorr && w.nin) {
        if (vec && QVPL == 4) {
          const int4 u = __ldg(reinterpret_cast<const int4*>(p.corr_col + at));
          f.zc[0] = u.x; f.zc[1] = u.y; f.zc[QVPL - 2] = u.z; f.zc[QVPL - 1] = u.w;
        } else if (vec) {
          const int2 u = __ldg(reinterpret_cast<const int2*>(p.corr_col + at));
          f.zc[0] = u.x; f.zc[1] = u.y;
        } else {
#pragma unroll
          for (int k = 0; k < QVPL; ++k)
            if (w.n + k < p.N) f.zc[k] = __ldg(p.corr_col + at + k);
        }
      }
      f.sa = (p.sa && w.rin) ? raw(p.sa, p.sa_tiled ? (int64_t)w.m * p.T + t : (int64_t)w.m) : sa_one;
      f.zr = (kCorr && w.rin) ? __ldg(p.corr_row + (int64_t)w.m * p.T + t) : 0;
      return f;
    };
    // the staged float32 scales of a lane's columns, from the kept bits
    auto widen_sb = [&](const Prefetch& f, float (&o)[QVPL]) {
      if (sb_rep == 1) {
#pragma unroll
        for (int k = 0; k < QVPL / 2; ++k) {
          o[2 * k] = __uint_as_float(f.sb[k] << 16);
          o[2 * k + 1] = __uint_as_float(f.sb[k] & 0xffff0000u);
        }
      } else {
#pragma unroll
        for (int k = 0; k < QVPL; ++k) o[k] = widen(f.sb[k], sb_rep);
      }
    };

    int tile = pair, t = 0;
    bool have = tile < num_tiles;
    Prefetch pf;
    Where wh = where(tile);
    if (have) pf = fetch(wh, t);
    float2 v[QCW / 2];

    while (have && ok) {
      // all lanes try once (the accumulator is usually there already); lane 0 waits otherwise
      if (!mbar_try_wait(smem_u32(&ctl->acc_full[acc]), acc_phase)) {
        if (lane == 0) ok = mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      tc_fence_after();
      const uint32_t tacc = tmem_warp + acc * QN;
      uint32_t r[32];
      tmem_ld_32x32b_x32(tacc, r);

      // while the first load is in flight: this K tile's scales into shared memory, the
      // next K tile's on their way from global memory
      float sbf[QVPL];
      widen_sb(pf, sbf);
      if (QVPL == 4) {
        *reinterpret_cast<float4*>(&ctl->sb[ew][lane * QVPL]) = make_float4(sbf[0], sbf[1], sbf[QVPL - 2], sbf[QVPL - 1]);
        if (kCorr) *reinterpret_cast<int4*>(&ctl->zc[ew][lane * QVPL]) = make_int4(pf.zc[0], pf.zc[1], pf.zc[QVPL - 2], pf.zc[QVPL - 1]);
      } else {
        *reinterpret_cast<float2*>(&ctl->sb[ew][lane * QVPL]) = make_float2(sbf[0], sbf[1]);
        if (kCorr) *reinterpret_cast<int2*>(&ctl->zc[ew][lane * QVPL]) = make_int2(pf.zc[0], pf.zc[1]);
      }
      const float sa = widen(pf.sa, sa_rep);
      const int32_t zr = pf.zr;
      __syncwarp();
      const Where wh_now = wh;
      int ntile = tile, nt = t + 1;
      if (nt == p.T) { nt = 0; ntile += num_pairs; wh = where(ntile); }
      const bool nhave = ntile < num_tiles;
      if (nhave) pf = fetch(wh, nt);

      if (t == 0) {
#pragma unroll
        for (int j = 0; j < QCW / 2; ++j) v[j] = make_float2(0.0f, 0.0f);
      }
      const float* sbv = ctl->sb[ew];
      const int32_t* zcv = ctl->zc[ew];
      // A warp's tensor-memory loads complete one after the other (two in flight take twice
      // as long as one), so one register buffer serves; the other warps of the SM sub-partition
      // fill the time.
#pragma unroll
      for (int c = 0; c < QCW / 32; ++c) {
        if (c) tmem_ld_32x32b_x32(tacc + c * 32, r);
        tmem_ld_wait_for(r);
        if (c == QCW / 32 - 1) {
          // the accumulator goes back before the last chunk is folded: its values are in registers
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster_relaxed(acc_empty0 + acc * 8);
        }
        fold_chunk<KIND, MODE>(r, sbv + c * 32, zcv + c * 32, sa, zr, p.out_dtype, v + c * 16);
      }
      __syncwarp();      // every lane is done with the staged scales before the next K tile's are written

      if (t == p.T - 1) {
        const int64_t m = wh_now.m;
        const int64_t n0 = wh_now.n - lane * QVPL;
        if (m < p.M) {
#pragma unroll
          for (int c = 0; c < QCW / 32; ++c) {
            const int64_t ncol = n0 + c * 32;
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
  {
    const uintptr_t esz = scale_dtype == QWX_F32 ? 4 : 2;
    p.scale_vec = (N % 4 == 0) && (!sb || reinterpret_cast<uintptr_t>(sb) % (4 * esz) == 0) &&
                  (!corr_col || reinterpret_cast<uintptr_t>(corr_col) % 16 == 0) &&
                  (!sb || scale_dtype == QWX_F32 || scale_dtype == QWX_BF16);
  }
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
    if (fast && k_tile <= 128)
      return launch_tiled_pair_layout<MmaKind::kI8, kModeMix>(b_layout, ta, tb, p, grid, st);
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
