// int8 x int8 GEMM for the decode step of a served model: a handful of token rows (at most
// 128) against a large weight held [N, K] (K contiguous),
//
//   out[m, n] = (sum_k a[m, k] * w[n, k]) * sa[m] * sb[n]       (dot_general.py:220, :255-258)
//
// The problem is the weight's bytes: every one of them crosses HBM once and is used by all
// tokens.  The operands are therefore swapped on the tensor core: 128 output CHANNELS are the
// M of a tcgen05.mma (kind::i8), the tokens its N (32, 64 or 128), so a tile is [128 channels
// x tokens], the accumulator takes `tokens` columns of tensor memory and the epilogue reads one
// tcgen05.ld per 32 tokens.  A stage of the shared-memory ring holds 256 K of 128 channels
// (32 KB) plus the same K of the tokens (8 KB at 32 tokens), both fetched by TMA.
//
// Work is cut stream-K style: the (channel tile, K stage) units are numbered tile-major and
// every CTA takes an equal contiguous run of them, so all SMs stream the same number of bytes
// whatever the tile count (32 tiles for a 4096-channel projection, 1002 for a vocabulary of
// 128256).  A tile that is shared by several CTAs is summed in a zeroed int32 scratch slot with
// red.global.add (exact, order-free); whoever adds last (a counter says so) scales, converts,
// stores and clears the slot.  Nobody waits for another CTA: no cooperative launch, no spin.
// A CTA that owns a whole tile skips the scratch.
//
// Where the time of a small launch goes (4096 x 4096 weight, 32 tokens, 16.7 MB = 2.6 us of HBM
// time; measured with %globaltimer probes): about 1.8 us between two kernels of a CUDA graph,
// 0.9 us until the first TMA issue, 1.8 us until its data arrives, 1.9 us of streaming and MMAs
// (a tcgen05.mma of N = 32 costs about as much as one of N = 256: 0.5 us per 32 KB stage, i.e.
// at most 60 GB/s per SM, so every SM has to take part), then the reduction of shared tiles:
// adds + fence 1.3 us, counter 0.7 us, finishing loads and stores 2.5 us in the CTA that adds
// last.  Programmatic dependent launch hides the first 2.7 us behind the previous kernel.
//
// Roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer and tensor-memory owner, warps
// 2-5 epilogue (two accumulators ping-pong, so the epilogue of one segment overlaps the MMAs
// of the next).  Every mbarrier wait is bounded (sm100.cuh).
#include "common.cuh"
#include "sm100.cuh"

namespace qwx {
namespace {

using namespace sm100;

constexpr int DT = 128;          // channels per tile: the MMA's M
constexpr int DBK = 128;         // one 128-byte swizzle row of K
constexpr int DSK = 2;           // swizzle rows per stage: 256 K
constexpr int DUK = 32;          // K per tcgen05.mma for 8-bit codes
constexpr int kDecThreads = 192;
constexpr int kMaxGrid = 256;    // scratch slots: one per CTA

template <int NT>
struct DecCfg {
  static constexpr int kStages = NT <= 32 ? 5 : (NT <= 64 ? 4 : 3);
  static constexpr int kWBytes = DT * DBK * DSK;
  static constexpr int kABytes = NT * DBK * DSK;
  static constexpr int kStageBytes = kWBytes + kABytes;
  static constexpr int kTmemCols = 2 * NT;     // two accumulators; 64 / 128 / 256 columns
};

struct DecControl {
  uint64_t full[5];
  uint64_t empty[5];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t epi_bar;       // the four epilogue warps meet here (bounded, unlike bar.sync)
  uint32_t tmem_base;
  int abort;
  int last;
  float sa[128];
};

template <int NT>
constexpr size_t dec_smem_bytes() {
  return 1024 + (size_t)DecCfg<NT>::kStages * DecCfg<NT>::kStageBytes + sizeof(DecControl);
}

struct DecParams {
  int M;
  int64_t N, K;
  const void* sa;
  const void* sb;
  int scale_dtype;
  void* out;
  int out_dtype;
  int epilogue;
  int32_t* error_flag;
  int kstages;            // stages of 256 K per tile
  long long units;        // tiles * kstages
  int32_t* ws;            // [grid][NT][128] partial sums, zero on entry, left zero
  int* counters;          // [grid], zero on entry, left zero
};

__device__ __forceinline__ float dec_scale(const void* p, int dtype, int64_t i) {
  if (dtype == QWX_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == QWX_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ float dec_round(float v, int out_dtype) {
  if (out_dtype == QWX_BF16) return round_to<BF16>(v);
  if (out_dtype == QWX_F16) return round_to<F16>(v);
  return v;
}

// The CTA whose unit range [c * U / G, (c + 1) * U / G) contains unit u.
__device__ __forceinline__ int cta_of_unit(long long u, long long G, long long U) {
  return (int)(((u + 1) * G - 1) / U);
}

template <int NT>
__global__ void __launch_bounds__(kDecThreads, 1)
gemm_q8_decode_kernel(const __grid_constant__ CUtensorMap tma_w,
                      const __grid_constant__ CUtensorMap tma_a, const DecParams p) {
  using Cfg = DecCfg<NT>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  DecControl* ctl = reinterpret_cast<DecControl*>(smem_raw + (ring - smem_u32(smem_raw)) +
                                                  (size_t)Cfg::kStages * Cfg::kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort = &ctl->abort;
  const long long G = gridDim.x, U = p.units;
  const long long u_begin = (long long)blockIdx.x * U / G;
  const long long u_end = (long long)(blockIdx.x + 1) * U / G;
  const int S = p.kstages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->acc_full[a]), 1);
      mbar_init(smem_u32(&ctl->acc_empty[a]), 4);
    }
    mbar_init(smem_u32(&ctl->epi_bar), 4);
    ctl->abort = 0;
    ctl->last = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_w);
    prefetch_tensormap(&tma_a);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), Cfg::kTmemCols);
    tmem_relinquish();
  }
  griddep_launch_dependents();
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
    // The weight does not depend on the kernel before this one: the first pass through the
    // ring fetches its weight halves at once, the token halves follow the dependency wait.
    const long long ahead = (u_end - u_begin) < Cfg::kStages ? (u_end - u_begin) : Cfg::kStages;
    if (lane == 0) {
      for (long long i = 0; i < ahead; ++i) {
        const long long u = u_begin + i;
        const int tile = (int)(u / S), ks = (int)(u % S);
        const uint32_t bar = smem_u32(&ctl->full[i]);
        const uint32_t sw = ring + (uint32_t)i * Cfg::kStageBytes;
        mbar_expect_tx(bar, Cfg::kStageBytes);
#pragma unroll
        for (int j = 0; j < DSK; ++j)
          tma_load_2d(sw + j * (DT * DBK), &tma_w, (ks * DSK + j) * DBK, tile * DT, bar);
      }
      griddep_wait();
      for (long long i = 0; i < ahead; ++i) {
        const int ks = (int)((u_begin + i) % S);
        const uint32_t bar = smem_u32(&ctl->full[i]);
        const uint32_t sact = ring + (uint32_t)i * Cfg::kStageBytes + Cfg::kWBytes;
#pragma unroll
        for (int j = 0; j < DSK; ++j)
          tma_load_2d(sact + j * (NT * DBK), &tma_a, (ks * DSK + j) * DBK, 0, bar);
      }
      issued = (long)ahead;
    }
    stage = (int)(ahead % Cfg::kStages);
    phase = ahead == Cfg::kStages ? 1u : 0u;
    for (long long u = u_begin + ahead; u < u_end && ok; ++u) {
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort);
        if (ok) {
          const int tile = (int)(u / S), ks = (int)(u % S);
          const uint32_t bar = smem_u32(&ctl->full[stage]);
          const uint32_t sw = ring + stage * Cfg::kStageBytes;
          const uint32_t sact = sw + Cfg::kWBytes;
          mbar_expect_tx(bar, Cfg::kStageBytes);
#pragma unroll
          for (int j = 0; j < DSK; ++j) {
            const int k0 = (ks * DSK + j) * DBK;
            tma_load_2d(sw + j * (DT * DBK), &tma_w, k0, tile * DT, bar);
            tma_load_2d(sact + j * (NT * DBK), &tma_a, k0, 0, bar);
          }
          ++issued;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
    }
    if (lane == 0 && *abort) {
      // Let copies that are still in flight land before the CTA gives up its shared memory.
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
    constexpr uint32_t idesc = make_idesc(2, 1, 1, 0, 0, DT, NT);   // s32 += s8 x s8, both K-major
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
          for (int j = 0; j < DSK; ++j) {
#pragma unroll
            for (int kk = 0; kk < DBK / DUK; ++kk) {
              // K-major operands: 8-row groups 1024 B apart, 32 B steps inside the swizzled row
              const uint64_t da = make_smem_desc(sw + j * (DT * DBK) + kk * DUK, 16, 1024);
              const uint64_t db = make_smem_desc(sact + j * (NT * DBK) + kk * DUK, 16, 1024);
              mma_ss<MmaKind::kI8>(tmem_base + acc * NT, da, db, idesc,
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
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;                     // tensor-memory lane quarter this warp may read
    const int nl = q * 32 + lane;               // channel inside the tile
    // Scales come from the kernel before this one, and nothing may be written before it has
    // finished.  Every epilogue warp stages the token scales (same values: a benign overlap).
    griddep_wait();
    for (int m = lane; m < NT; m += 32)
      ctl->sa[m] = (p.sa && m < p.M) ? dec_scale(p.sa, p.scale_dtype, m) : 1.0f;
    __syncwarp();
    int acc = 0;
    uint32_t acc_phase = 0, epi_phase = 0;
    bool ok = true;
    const bool reference = p.epilogue == QWX_EPI_REFERENCE;

    auto emit = [&](int m, int64_t n, int32_t v, float sb) {
      const int64_t o = (int64_t)m * p.N + n;
      if (p.out_dtype == QWX_S32) {
        reinterpret_cast<int32_t*>(p.out)[o] = v;
        return;
      }
      float a = (float)v;
      const float sa = ctl->sa[m];
      if (reference) {
        a = dec_round(a, p.out_dtype);
        a = dec_round(__fmul_rn(a, sa), p.out_dtype);
        a = dec_round(__fmul_rn(a, sb), p.out_dtype);
      } else {
        a = __fmul_rn(__fmul_rn(a, sa), sb);
      }
      if (p.out_dtype == QWX_F32) reinterpret_cast<float*>(p.out)[o] = a;
      else if (p.out_dtype == QWX_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(a);
      else reinterpret_cast<__half*>(p.out)[o] = __float2half_rn(a);
    };
    // all four epilogue warps reach this point (bounded)
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
      const int c_first = cta_of_unit(t_begin, G, U);
      const int nseg = cta_of_unit(t_end - 1, G, U) - c_first + 1;
      const int64_t n = (int64_t)tile * DT + nl;
      const bool n_ok = n < p.N;
      const float sb = (p.sb && n_ok) ? dec_scale(p.sb, p.scale_dtype, n) : 1.0f;
      int32_t* slot = p.ws + (size_t)c_first * (NT * DT) + nl;

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
            if (c * 32 + j < p.M) emit(c * 32 + j, n, (int32_t)r[j], sb);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c * 32 + j < p.M) atomicAdd(slot + (c * 32 + j) * DT, (int32_t)r[j]);
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
            // all loads first (one L2 round trip for the lot), then the clears, then the stores
#pragma unroll 1
            for (int c = 0; c * 32 < p.M; ++c) {
              int32_t v[32];
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] = c * 32 + j < p.M ? __ldcg(slot + (c * 32 + j) * DT) : 0;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (c * 32 + j < p.M) __stcg(slot + (c * 32 + j) * DT, 0);
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (c * 32 + j < p.M) emit(c * 32 + j, n, v[j], sb);
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

template <int NT>
int launch_decode(const CUtensorMap& tw, const CUtensorMap& ta, const DecParams& p, int grid,
                  cudaStream_t st) {
  auto kern = gemm_q8_decode_kernel<NT>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)dec_smem_bytes<NT>()) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured.mark();
  }
  if (launch_dependent(kern, dim3(grid), dim3(kDecThreads), dec_smem_bytes<NT>(), st, tw, ta, p) !=
      cudaSuccess) {
    (void)cudaGetLastError();
    return QWX_ERR_LAUNCH;
  }
  return QWX_OK;
}

int dec_token_tile(int64_t M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }

int dec_sm_count() {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return v;
}

}  // namespace
}  // namespace qwx

using namespace qwx;

extern "C" size_t qwx_gemm_q8_decode_workspace_bytes(int64_t M, int64_t N) {
  if (M <= 0 || M > 128 || N <= 0) return 0;
  return 1024 + (size_t)kMaxGrid * dec_token_tile(M) * DT * sizeof(int32_t);
}

extern "C" int qwx_gemm_q8_decode(const void* a, const void* w, int64_t M, int64_t N, int64_t K,
                                  const void* sa, const void* sb, int scale_dtype, void* out,
                                  int out_dtype, int epilogue, void* workspace,
                                  size_t workspace_bytes, int workspace_is_zero,
                                  int32_t* error_flag, qwx_stream_t stream) {
  if (!a || !w || !out || !workspace) return QWX_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (M > 128) return QWX_ERR_UNSUPPORTED;
  if (N > INT32_MAX - DT || K > INT32_MAX - DBK * DSK) return QWX_ERR_SHAPE;
  if (out_dtype == QWX_S32) {
    if (sa || sb) return QWX_ERR_DTYPE;
  } else if (out_dtype != QWX_BF16 && out_dtype != QWX_F32 && out_dtype != QWX_F16) {
    return QWX_ERR_DTYPE;
  }
  if ((sa || sb) && scale_dtype != QWX_F32 && scale_dtype != QWX_BF16 && scale_dtype != QWX_F16)
    return QWX_ERR_DTYPE;
  if (epilogue != QWX_EPI_F32 && epilogue != QWX_EPI_REFERENCE) return QWX_ERR_SHAPE;
  // TMA: 16-byte aligned bases and row pitches
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (K % 16))
    return QWX_ERR_ALIGN;
  if (reinterpret_cast<uintptr_t>(workspace) & 15) return QWX_ERR_ALIGN;
  const size_t need = qwx_gemm_q8_decode_workspace_bytes(M, N);
  if (workspace_bytes < need) return QWX_ERR_WORKSPACE;
  const int nt = dec_token_tile(M);
  const int sms = dec_sm_count();
  if (sms <= 0) return QWX_ERR_NO_DEVICE;
  if (!get_encode_tiled()) return QWX_ERR_NO_DEVICE;
  CUtensorMap tw, ta;
  if (!encode_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w, (uint64_t)N, (uint64_t)K, DT, DBK) ||
      !encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)M, (uint64_t)K, nt, DBK))
    return QWX_ERR_LAUNCH;
  cudaStream_t st = (cudaStream_t)stream;
  if (!workspace_is_zero && cudaMemsetAsync(workspace, 0, need, st) != cudaSuccess)
    return QWX_ERR_LAUNCH;

  DecParams p;
  p.M = (int)M; p.N = N; p.K = K;
  p.sa = sa; p.sb = sb; p.scale_dtype = scale_dtype;
  p.out = out; p.out_dtype = out_dtype; p.epilogue = epilogue;
  p.error_flag = error_flag;
  const int64_t tiles = (N + DT - 1) / DT;
  p.kstages = (int)((K + DBK * DSK - 1) / (DBK * DSK));
  p.units = (long long)tiles * p.kstages;
  p.counters = (int*)workspace;
  p.ws = (int32_t*)((char*)workspace + 1024);
  int grid = sms < kMaxGrid ? sms : kMaxGrid;
  if (p.units < grid) grid = (int)p.units;
  switch (nt) {
    case 32: return launch_decode<32>(tw, ta, p, grid, st);
    case 64: return launch_decode<64>(tw, ta, p, grid, st);
    default: return launch_decode<128>(tw, ta, p, grid, st);
  }
}
