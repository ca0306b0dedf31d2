// Weight-only int4 GEMM for decode-shaped problems (few tokens, huge weight): the device
// side of dot_general._slow_dot_general (dot_general.py:264-275) for a bf16 activation and an
// int4 sub-channel-quantized weight,
//
//   out[m, n] = sum_k a[m, k] * W~[k, n],   W~[k, n] = bf16( q[k, n] * s[k / tile, n] )
//
// without ever writing W~ to global memory.  The kernel is HBM-bound on the packed weight:
// K*N/2 bytes are streamed exactly once.
//
// Operands are swapped so that the 128 output channels of a tile are the M dimension of
// tcgen05.mma (kind::f16, bf16 x bf16 -> f32 in tensor memory) and the (padded) token count is
// its N dimension.  Work is cut into units of (128 channels x 128 K) and dealt to one
// persistent CTA per SM as contiguous ranges (stream-K), so all SMs stream for the same time;
// a tile split between CTAs is summed with float atomics in a caller-provided workspace and
// converted by the CTA that contributes last.
//
//   warps 4-15    weight stream + unpack, in up to three groups of four warps that take the
//                 units round-robin: every thread owns one channel row (64 bytes, 128 codes) of
//                 its group's units and keeps three of them in flight with 16-byte
//                 cp.async copies into a private slice of a shared-memory ring (the LSU path: a
//                 single TMA bulk stream per SM was measured at a third of the HBM rate); then
//                 int4 -> bf16 (magic-number conversion), scale, store into the swizzled
//                 K-major operand layout; group 0 also runs the epilogue of each tile segment
//   warp 0        TMA tile loads of the activations (small, L2-resident), one per unit
//   warps 1-3     MMA issuers (8 x M128 N{16..128} K16 per unit), units taken round-robin;
//                 warp 1 also owns the tensor-memory allocation
#include "common.cuh"
#include "sm100.cuh"
#include <algorithm>

namespace qwx {
namespace {

using namespace sm100;

constexpr int W4_BN = 128;          // channels per tile
constexpr int W4_BK = 128;          // K per unit
constexpr int kUnitBytes = W4_BN * W4_BK / 2;
constexpr int kGroupThreads = 128;  // one unpack group = 4 warps = one thread per channel row
constexpr int kRawStageBytes = kUnitBytes + kGroupThreads * 4;   // + one scale word per thread
constexpr int kMaxSlots = 3;        // operand slots = unpack groups = MMA issuers, upper bound
constexpr int kWSlotBytes = W4_BN * W4_BK * 2;   // two 16 KB swizzle atoms
constexpr int kUnpackWarp0 = 4;
constexpr int kW4Threads = (kUnpackWarp0 + 4 * kMaxSlots) * 32;   // 512

struct W4Control {
  uint64_t ready[kMaxSlots];   // 128 unpack arrivals + the activation tile's bytes
  uint64_t free_[kMaxSlots];   // tcgen05.commit of the unit that used the slot
  uint64_t acc_full[2], acc_free[2];
  uint64_t epi_done, fin_done;
  uint32_t tmem_base;
  int abort;
  int finalize;
};

struct W4Params {
  const uint8_t* wp;      // packed units, [n_tiles][k_blocks][8 KB]
  const void* scale;      // [K / tile, N], f32 or bf16
  int scale_dtype;
  int64_t M, N, K;
  int tile;               // scale tile along K (multiple of 128)
  int mpad;               // tokens padded to 16 / 32 / 64 / 128: the MMA N extent
  int slots;              // operand slots in use = unpack groups = MMA issuers in use
  int depth;              // packed-weight units each group keeps in flight (3)
  void* out;
  int out_dtype;
  float* ws;              // [M, N] partial sums, zero on entry, left zero
  int* counters;          // [n_tiles], zero on entry, left zero
  int32_t* error_flag;
  int n_tiles, k_blocks;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7])
      : "r"(taddr)
      : "memory");
}

// Eight offset-binary nibbles (value + 8), stored in the order k0 k2 k4 k6 k1 k3 k5 k7, to four
// bf16x2 words (k0 k1)(k2 k3)(k4 k5)(k6 k7), each multiplied by the bf16 scale.  0x4300 | u is
// the bf16 number 128 + u; subtracting 136 gives the signed code exactly.
__device__ __forceinline__ void unpack8(uint32_t w, __nv_bfloat162 s2, uint32_t (&o)[4]) {
  const __nv_bfloat162 bias = __floats2bfloat162_rn(136.f, 136.f);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t v = ((w >> (4 * j)) & 0x000f000fu) | 0x43004300u;
    __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&v);
    h = __hmul2(__hsub2(h, bias), s2);
    o[j] = *reinterpret_cast<uint32_t*>(&h);
  }
}

// Does issuer `t` own a unit of the segment that starts `first_local` units into the CTA's
// range and is `units` long?  (Units go to issuers round-robin by their local index.)
__device__ __forceinline__ bool issuer_in_segment(int t, int issuers, int first_local, int units) {
  if (units >= issuers) return true;
  int d = t - first_local % issuers;
  if (d < 0) d += issuers;
  return d < units;
}

__global__ void __launch_bounds__(kW4Threads, 1)
gemm_w4_kernel(const __grid_constant__ CUtensorMap tma_act, const W4Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t act_bytes = 2u * p.mpad * 128u;   // activation tile of one unit (two atoms)
  const uint32_t w_off = 0;
  const uint32_t act_off = w_off + p.slots * kWSlotBytes;
  const uint32_t raw_off = act_off + p.slots * act_bytes;
  const uint32_t ctl_off = raw_off + p.slots * p.depth * kRawStageBytes;
  W4Control* ctl = reinterpret_cast<W4Control*>(base_ptr + ctl_off);
  volatile int* abort = &ctl->abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Units are numbered tile-major; the host guarantees that the count fits 31 bits, so all the
  // per-unit bookkeeping below is 32-bit and incremental (no divisions in the loops).
  const int total_units = p.n_tiles * p.k_blocks;
  const int g_begin = (int)((int64_t)total_units * blockIdx.x / gridDim.x);
  const int g_end = (int)((int64_t)total_units * (blockIdx.x + 1) / gridDim.x);
  const int kb_begin = g_begin % p.k_blocks, tile_begin = g_begin / p.k_blocks;
  // Tensor memory: [2 segment buffers][issuers][mpad columns] of float32 accumulators.
  const uint32_t set_cols = (uint32_t)(p.slots * p.mpad);
  uint32_t tmem_cols = 32;
  while (tmem_cols < 2 * set_cols) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxSlots; ++s) {
      mbar_init(smem_u32(&ctl->ready[s]), kGroupThreads + 1);
      mbar_init(smem_u32(&ctl->free_[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->acc_full[a]), p.slots);
      mbar_init(smem_u32(&ctl->acc_free[a]), kGroupThreads / 32);
    }
    mbar_init(smem_u32(&ctl->epi_done), kGroupThreads);
    mbar_init(smem_u32(&ctl->fin_done), 1);
    ctl->abort = 0;
    ctl->finalize = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_act);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ---------------- activation tiles: one per unit, into the unit's operand slot ----------
    if (lane == 0) {
      int u = 0, kb = kb_begin;
      uint32_t uphase = 0;
      for (int g = g_begin; g < g_end; ++g) {
        if (!mbar_wait(smem_u32(&ctl->free_[u]), uphase ^ 1u, abort)) break;
        const uint32_t bar = smem_u32(&ctl->ready[u]);
        const uint32_t dst = base + act_off + u * act_bytes;
        mbar_expect_tx(bar, act_bytes);
        tma_load_2d(dst, &tma_act, kb * W4_BK, 0, bar);
        tma_load_2d(dst + p.mpad * 128, &tma_act, kb * W4_BK + 64, 0, bar);
        if (++u == p.slots) { u = 0; uphase ^= 1u; }
        if (++kb == p.k_blocks) kb = 0;
      }
      if (*abort) {
        // give copies in flight time to land before the CTA retires
        for (int s = 0; s < p.slots; ++s)
          for (int it = 0; it < 20000; ++it)
            if (mbar_try_wait(smem_u32(&ctl->ready[s]), 0) || mbar_try_wait(smem_u32(&ctl->ready[s]), 1)) break;
      }
    }
    __syncwarp();
  } else if (warp <= p.slots) {
    // ---------------- MMA issuers ----------------
    // An issuing thread pays a few hundred cycles per mbarrier wait and per commit, far more
    // than the eight MMAs of a unit cost the tensor pipe, so several warps issue: issuer j
    // serves operand slot j (every unit whose local index is j mod slots) and adds into its own
    // accumulator columns.  Because a slot has one issuer, that thread observes every phase of
    // the slot's barrier in order (a parity wait must never skip a phase).  Per unit: one wait,
    // eight MMAs, one commit.  Descriptors are built once and advanced by adding to their low word
    // (the start-address field cannot carry into the next field below 256 KB).
    const int me = warp - 1;
    if (lane == 0) {
      const uint32_t idesc = make_idesc(1, 1, 1, 0, 0, W4_BN, (uint32_t)p.mpad);
      const uint64_t wdesc0 = make_smem_desc(base + w_off, 16, 1024);
      const uint64_t adesc0 = make_smem_desc(base + act_off, 16, 1024);
      const uint32_t act_atom = (uint32_t)(p.mpad * 128) >> 4;
      const uint32_t bar_ready = smem_u32(&ctl->ready[0]), bar_free = smem_u32(&ctl->free_[0]);
      int u = 0, acc = 0, kb = kb_begin;
      uint32_t uphase = 0, acc_phase = 0;
      bool mine_in_segment = false;
      for (int g = g_begin; g < g_end; ++g) {
        const int seg_first = max(g_begin, g - kb);
        const int seg_last = min(g_end - 1, g + (p.k_blocks - 1 - kb));
        // every issuer watches every segment's accumulator hand-over, in order
        if (g == seg_first && !mbar_wait(smem_u32(&ctl->acc_free[acc]), acc_phase ^ 1u, abort)) break;
        if (u == me) {
          const bool first_of_mine = g - p.slots < seg_first;
          if (!mbar_wait(bar_ready + u * 8, uphase, abort)) break;
          tc_fence_after();
          const uint64_t da = wdesc0 + (uint64_t)(u * (kWSlotBytes >> 4));
          const uint64_t db = adesc0 + (uint64_t)(u * (act_bytes >> 4));
          const uint32_t d_tmem = tmem_base + acc * set_cols + me * p.mpad;
#pragma unroll
          for (int kk = 0; kk < W4_BK / 16; ++kk) {
            const uint32_t atom = kk >> 2, sub = ((kk & 3) * 32) >> 4;
            mma_ss<MmaKind::kF16>(d_tmem, da + atom * ((W4_BN * 128) >> 4) + sub,
                                  db + atom * act_atom + sub, idesc, !(first_of_mine && kk == 0));
          }
          mma_commit(bar_free + u * 8);
          mine_in_segment = true;
        }
        if (g == seg_last) {
          // every issuer reports on the segment: a commit if it has MMAs in it, else an arrive
          if (mine_in_segment) mma_commit(smem_u32(&ctl->acc_full[acc]));
          else mbar_arrive(smem_u32(&ctl->acc_full[acc]));
          mine_in_segment = false;
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (++u == p.slots) { u = 0; uphase ^= 1u; }
        if (++kb == p.k_blocks) kb = 0;
      }
    }
    __syncwarp();
  } else if (warp >= kUnpackWarp0 && warp < kUnpackWarp0 + 4 * p.slots) {
    // ---------------- weight stream, unpack, epilogue ----------------
    // Group j (4 warps, one thread per channel row) owns every unit whose local index is
    // j mod slots and always fills operand slot j.  While one group sits in a barrier wait or
    // a proxy fence the others convert, which is what keeps the issue slots busy.  Group 0
    // additionally runs the epilogue of every tile segment.
    const int group = (warp - kUnpackWarp0) >> 2;
    const int n = threadIdx.x & 127;                  // channel row inside the tile
    const int quarter = warp & 3;                     // tensor-memory lane quarter (group 0)
    const int scale_elem = p.scale_dtype == QWX_F32 ? 4 : 2;
    const uint32_t my_off = n * 16;                   // chunk j of this row: + j * 2048
    const uint32_t bar_free = smem_u32(&ctl->free_[group]);
    const uint32_t bar_ready = smem_u32(&ctl->ready[group]);

    // Prefetch cursor over this group's units (local index group, group + slots, ...): one
    // commit group per unit = the row's four 16-byte chunks + the 4-byte word holding the
    // channel's scale for the unit's K tile (two bf16 scales share a word).
    const int blocks_per_scale = p.tile / W4_BK;
    const int64_t scale_row_bytes = p.N * scale_elem;
    const int64_t scale_col_bytes = scale_elem == 4 ? (int64_t)n * 4 : (int64_t)(n & ~1) * 2;
    int f_g = g_begin + group;
    int f_kb = kb_begin + group, f_tile = tile_begin;
    while (f_kb >= p.k_blocks) { f_kb -= p.k_blocks; ++f_tile; }
    int f_stage = 0;
    auto fetch = [&]() {
      if (f_g < g_end) {
        const uint8_t* src = p.wp + (int64_t)f_g * kUnitBytes + my_off;
        const uint32_t dst = base + raw_off + (group * p.depth + f_stage) * kRawStageBytes;
#pragma unroll
        for (int j = 0; j < 4; ++j) cp_async16(dst + my_off + j * 2048, src + j * 2048);
        const char* sp = reinterpret_cast<const char*>(p.scale) +
                         (int64_t)(f_kb / blocks_per_scale) * scale_row_bytes +
                         (int64_t)f_tile * W4_BN * scale_elem + scale_col_bytes;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + kUnitBytes + n * 4),
                     "l"(sp) : "memory");
        f_g += p.slots;
        f_kb += p.slots;
        while (f_kb >= p.k_blocks) { f_kb -= p.k_blocks; ++f_tile; }
      }
      if (++f_stage == p.depth) f_stage = 0;
      cp_async_commit();
    };
    for (int d = 0; d < p.depth; ++d) fetch();

    int rs = 0, acc = 0, owner = 0;
    uint32_t uphase = 0, acc_phase = 0, epi_phase = 0;
    int seg_units = 0, seg_first_local = 0;
    bool ok = true;
    int tile = tile_begin, kb = kb_begin;
    for (int g = g_begin; g < g_end && ok; ++g, kb = (kb + 1 == p.k_blocks ? (++tile, 0) : kb + 1)) {
      const bool first = (g == g_begin) || kb == 0;
      const bool last = (g == g_end - 1) || kb == p.k_blocks - 1;
      if (first) { seg_units = 0; seg_first_local = g - g_begin; }
      ++seg_units;

      if (owner == group) {
        // this thread's own copies of the unit have landed once at most depth - 1 groups pend
        cp_async_wait<2>();   // depth is 3
        const uint8_t* raw = base_ptr + raw_off + (group * p.depth + rs) * kRawStageBytes;
        uint32_t words[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 c = *reinterpret_cast<const uint4*>(raw + my_off + j * 2048);
          words[4 * j] = c.x; words[4 * j + 1] = c.y; words[4 * j + 2] = c.z; words[4 * j + 3] = c.w;
        }
        const uint32_t sw = *reinterpret_cast<const uint32_t*>(raw + kUnitBytes + n * 4);
        fetch();                       // refill the slice just read
        if (++rs == p.depth) rs = 0;

        ok = mbar_wait(bar_free, uphase ^ 1u, abort);
        if (!ok) break;
        uphase ^= 1u;
        __nv_bfloat16 sb;  // the scale as bf16 (f32 scales are rounded)
        if (scale_elem == 4) sb = __float2bfloat16_rn(__uint_as_float(sw));
        else sb = __ushort_as_bfloat16((unsigned short)((n & 1) ? (sw >> 16) : (sw & 0xffffu)));
        const __nv_bfloat162 s2 = __halves2bfloat162(sb, sb);
        uint8_t* wrow = base_ptr + w_off + group * kWSlotBytes + (n >> 3) * 1024 + (n & 7) * 128;
#pragma unroll
        for (int c = 0; c < 16; ++c) {   // words 0-7: K 0..63 (atom 0), words 8-15: atom 1
          uint32_t o[4];
          unpack8(words[c], s2, o);
          *reinterpret_cast<uint4*>(wrow + (c >> 3) * (W4_BN * 128) + (((c & 7) ^ (n & 7)) * 16)) =
              make_uint4(o[0], o[1], o[2], o[3]);
        }
        fence_proxy_async();
        mbar_arrive(bar_ready);
      }
      if (++owner == p.slots) owner = 0;

      if (!last || group != 0) continue;
      // ---- epilogue of the segment (tile, kb - seg_units + 1 .. kb), by group 0 ----
      ok = mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort);
      if (!ok) break;
      tc_fence_after();
      const bool whole = seg_units == p.k_blocks;
      const int64_t channel = (int64_t)tile * W4_BN + quarter * 32 + lane;
      for (int col = 0; col < p.mpad; col += 8) {
        float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int t = 0; t < p.slots; ++t) {   // add up the issuers' partial accumulators
          if (!issuer_in_segment(t, p.slots, seg_first_local, seg_units)) continue;
          uint32_t r[8];
          tmem_ld_32x32b_x8(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * set_cols +
                                t * p.mpad + col, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) sum[j] += __uint_as_float(r[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int64_t m = col + j;
          if (m >= p.M) continue;
          const float v = sum[j];
          if (whole) {
            if (p.out_dtype == QWX_BF16)
              reinterpret_cast<__nv_bfloat16*>(p.out)[m * p.N + channel] = __float2bfloat16_rn(v);
            else
              reinterpret_cast<float*>(p.out)[m * p.N + channel] = v;
          } else {
            atomicAdd(p.ws + m * p.N + channel, v);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_free[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }

      if (!whole) {
        // Count this CTA's K blocks for the tile; whoever completes the tile converts it.
        __threadfence();
        mbar_arrive(smem_u32(&ctl->epi_done));
        if (n == 0) {
          ok = mbar_wait(smem_u32(&ctl->epi_done), epi_phase, abort);
          if (ok) {
            const int old = atomicAdd(p.counters + tile, seg_units);
            __threadfence();
            ctl->finalize = (old + seg_units == p.k_blocks) ? 1 : 0;
            if (ctl->finalize) p.counters[tile] = 0;
          }
          mbar_arrive(smem_u32(&ctl->fin_done));
        }
        ok = mbar_wait(smem_u32(&ctl->fin_done), epi_phase, abort);
        epi_phase ^= 1u;
        if (!ok) break;
        if (ctl->finalize) {
          for (int64_t m = 0; m < p.M; ++m) {
            float* wsp = p.ws + m * p.N + channel;
            const float v = __ldcg(wsp);
            *wsp = 0.f;
            if (p.out_dtype == QWX_BF16)
              reinterpret_cast<__nv_bfloat16*>(p.out)[m * p.N + channel] = __float2bfloat16_rn(v);
            else
              reinterpret_cast<float*>(p.out)[m * p.N + channel] = v;
          }
        }
      }
    }
    cp_async_wait<0>();  // nothing of this thread may still be landing when the CTA retires
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
  if (threadIdx.x == 0 && ctl->abort && p.error_flag) atomicExch(p.error_flag, QWX_ERR_DEVICE_WAIT);
}

// Logical codes q[K, N] (one sign-extended int4 per byte) -> packed units.
__global__ void pack_w4_kernel(const int8_t* __restrict__ q, int64_t K, int64_t N, int k_blocks,
                               uint32_t* __restrict__ out, int64_t total_words) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total_words) return;
  // word index inside a unit: ((j * 128 + n) * 4 + w); unit index: tile * k_blocks + kb
  const int w = (int)(t & 3);
  const int n = (int)((t >> 2) & 127);
  const int j = (int)((t >> 9) & 3);
  const int64_t unit = t >> 11;
  const int64_t tile = unit / k_blocks, kb = unit % k_blocks;
  const int64_t col = tile * W4_BN + n;
  const int64_t k0 = kb * W4_BK + j * 32 + w * 8;
  uint32_t word = 0;
  const int order[8] = {0, 2, 4, 6, 1, 3, 5, 7};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t k = k0 + order[i];
    int v = (col < N && k < K) ? (int)q[k * N + col] : 0;
    word |= (uint32_t)((v + 8) & 0xf) << (4 * i);
  }
  out[t] = word;
}

int sm_count_w4() {
  static int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return v;
  }();
  return n;
}

// Operand slots (= unpack groups = issuing warps) and prefetch depth per token count: what fits
// 227 KB of shared memory and 512 tensor-memory columns (2 segment buffers x slots x mpad).
void w4_config(int mpad, int* slots, int* depth) {
  if (mpad <= 64) { *slots = 3; *depth = 3; }
  else { *slots = 2; *depth = 3; }
}

size_t w4_smem_bytes(int mpad) {
  int slots, depth;
  w4_config(mpad, &slots, &depth);
  return 1024 + (size_t)slots * (kWSlotBytes + 2 * mpad * 128) +
         (size_t)slots * depth * kRawStageBytes + sizeof(W4Control);
}

}  // namespace
}  // namespace qwx

using namespace qwx;

extern "C" {

size_t qwx_w4_packed_bytes(int64_t K, int64_t N) {
  if (K <= 0 || N <= 0 || K % W4_BK) return 0;
  const int64_t n_tiles = (N + W4_BN - 1) / W4_BN;
  return (size_t)(n_tiles * (K / W4_BK) * kUnitBytes);
}

int qwx_pack_w4(const void* q, int64_t K, int64_t N, void* packed, qwx_stream_t stream) {
  if (!q || !packed) return QWX_ERR_NULL;
  if (K <= 0 || N <= 0 || K % W4_BK) return QWX_ERR_SHAPE;
  const int64_t n_tiles = (N + W4_BN - 1) / W4_BN;
  const int64_t words = n_tiles * (K / W4_BK) * (kUnitBytes / 4);
  pack_w4_kernel<<<(unsigned)((words + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const int8_t*)q, K, N, (int)(K / W4_BK), (uint32_t*)packed, words);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

size_t qwx_gemm_a16w4_workspace_bytes(int64_t M, int64_t N) {
  if (M <= 0 || N <= 0) return 0;
  const int64_t n_tiles = (N + W4_BN - 1) / W4_BN;
  return (size_t)(M * N * 4 + n_tiles * 4);
}

int qwx_gemm_a16w4(const void* a, const void* w_packed, const void* scale, int scale_dtype,
                   int64_t M, int64_t N, int64_t K, int64_t k_tile, void* out, int out_dtype,
                   void* workspace, size_t workspace_bytes, int workspace_is_zero,
                   int32_t* error_flag, qwx_stream_t stream) {
  if (!a || !w_packed || !scale || !out || !workspace) return QWX_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0) return QWX_ERR_SHAPE;
  if (M > 128) return QWX_ERR_UNSUPPORTED;            // larger batches: call per 128 rows
  if (K % W4_BK || N % W4_BN) return QWX_ERR_UNSUPPORTED;
  if (k_tile <= 0 || K % k_tile || k_tile % W4_BK) return QWX_ERR_UNSUPPORTED;
  if (scale_dtype != QWX_F32 && scale_dtype != QWX_BF16) return QWX_ERR_DTYPE;
  if (out_dtype != QWX_BF16 && out_dtype != QWX_F32) return QWX_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w_packed) & 15) ||
      (reinterpret_cast<uintptr_t>(scale) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 15))
    return QWX_ERR_ALIGN;
  if (workspace_bytes < qwx_gemm_a16w4_workspace_bytes(M, N)) return QWX_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (!workspace_is_zero &&
      cudaMemsetAsync(workspace, 0, qwx_gemm_a16w4_workspace_bytes(M, N), st) != cudaSuccess)
    return QWX_ERR_LAUNCH;

  const int mpad = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  CUtensorMap ta;
  if (!get_encode_tiled()) return QWX_ERR_NO_DEVICE;
  if (!encode_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, (uint64_t)M, (uint64_t)K, mpad, 64))
    return QWX_ERR_LAUNCH;

  W4Params p;
  p.wp = (const uint8_t*)w_packed;
  p.scale = scale; p.scale_dtype = scale_dtype;
  p.M = M; p.N = N; p.K = K; p.tile = (int)k_tile; p.mpad = mpad;
  p.out = out; p.out_dtype = out_dtype;
  p.ws = (float*)workspace;
  p.counters = (int*)((char*)workspace + M * N * 4);
  p.error_flag = error_flag;
  w4_config(mpad, &p.slots, &p.depth);
  p.n_tiles = (int)(N / W4_BN);
  p.k_blocks = (int)(K / W4_BK);

  const size_t smem = w4_smem_bytes(mpad);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_w4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)std::max(w4_smem_bytes(16), w4_smem_bytes(64))) != cudaSuccess)
      return QWX_ERR_LAUNCH;
    configured = true;
  }
  const int sms = sm_count_w4();
  if (sms <= 0) return QWX_ERR_NO_DEVICE;
  const int64_t units = (int64_t)p.n_tiles * p.k_blocks;
  if (units > (1 << 30)) return QWX_ERR_UNSUPPORTED;
  const int grid = (int)(units < sms ? units : sms);
  gemm_w4_kernel<<<grid, kW4Threads, smem, st>>>(ta, p);
  QWX_CHECK_LAUNCH();
  return QWX_OK;
}

}  // extern "C"
