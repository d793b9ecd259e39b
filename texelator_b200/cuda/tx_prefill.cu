// Prefill GEMM for tokens >= prefill_threshold: Y[T, M] = X[T, K] * Wq[M, K]^T on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in TMEM).
//
// Reference counterpart: the five CUTLASS 2.x tiles whose B iterator gathers BC4 texels
// (texelator/cuda/cutlass_texture_mainloop.cu:61-249, _t1/_t2/_t3/_smalln.cu; sm_80 mma.sync,
// two-stage register-staged pipeline).  B200 design, one CTA per MT*128 output rows x BN tokens:
//
//   pre-pass   one small kernel rescales the activations per token by an exact power of two and stores
//              them as fp16 (the decode GEMV's staging) in the chunk-major order of the B operand;
//   warps 0-15 producers: 128-bit loads of the tiled BC4 payload (one 8-row half of a 16-row tile per
//              warp), decode in registers exactly like the decode GEMV (masked index fields + HFMA2 ->
//              exact numerators n * 2^-16, n = 7*e0 + g*(e1-e0), as fp16) and store the A tile into shared
//              memory in the canonical K-major core-matrix layout (no swizzle);
//   warp 16    one lane issues the TMA load of the staged X tile (BN tokens x BK columns) per stage
//              through a 3-D tensor map whose rows are 512 contiguous bytes (no multicast);
//   warp 17    allocates TMEM, and one lane issues MT * BK/16 tcgen05.mma kind::f16 (M=128, N=BN, K=16)
//              per stage, committing to the stage's "empty" barrier;
//   warps 0-15 epilogue: tcgen05.ld of the fp32 accumulators, * scale_m * 2^s * 65536/889, + bias, one bf16
//              rounding, store.
//
// Numerics are those of the decode GEMV: products of exact integers and exactly rescaled activations,
// fp32 accumulation, weights never rounded to bf16 (the reference rounds bf16(pal*scale); the outputs
// differ by that rounding only, rel-RMS about 1e-3).
//
// Output rows are the MMA M (TMEM lanes) and tokens the MMA N (TMEM columns), so every weight tile
// is decoded once per CTA for all BN tokens.  K is consumed in the same 16-column steps and the
// same order by every tile candidate, so candidates are bitwise identical to each other (the
// reference's admission rule, texelator/autotune.py:160-168).
//
// Every mbarrier wait is bounded: when a wait runs out, the thread records a code in a device status
// word, raises a CTA-wide abort flag, the roles leave their loops, outstanding TMA copies are waited
// for (bounded again), TMEM is freed and the CTA returns.
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "tx_common.cuh"
#include "tx_decode.cuh"

namespace tx {

constexpr int kMmaM = 128;               // rows of one tcgen05.mma (TMEM lanes)
constexpr int kASbo = 128;               // byte stride between 8-row groups of the A tile
// Sixteen producer warps, one 8-row half of a 16-row tile each, all on every pipeline stage.  Measured and not
// adopted: two groups of eight warps taking alternate stages with a whole tile per warp (same speed at 32 and
// 128 tokens, 2-4 % slower at 512), a four-unit register look-ahead (same / 10 % slower), a 128 x 32 tile with a
// five-stage ring against the 128 x 64 tile with four stages at 32 tokens (same).
constexpr int kProducerWarps = 16;              // 8: one 16-row tile per warp; 16: one 8-row half of a tile per warp
constexpr int kTileWarps = 8;                   // 16-row tiles of one 128-row accumulator
constexpr int kGroups = 1;                      // groups of producer warps that take alternate units
constexpr int kHalvesPerWarp = 16 * kGroups / kProducerWarps;
constexpr int kTmaWarp = kProducerWarps, kMmaWarp = kProducerWarps + 1;
constexpr int kPrefillThreads = (kProducerWarps + 2) * 32;   // producer/epilogue warps + TMA warp + MMA warp
static_assert(kProducerWarps == 8 || kProducerWarps == 16, "producer warps split tiles whole or by halves");
constexpr unsigned kSpinLimit = 1u << 22;

// One tile shape: MT x 128 output rows (MT accumulators side by side in TMEM), BN tokens, BK columns
// per pipeline stage.  Per FLOP the X tile is re-read 1/(128*MT) times, so tall tiles relieve L2; the
// BC4 side costs a quarter of a byte per weight either way.
template <int MT, int BN, int BK> struct TileConfig {
  static constexpr int rows = MT * kMmaM;
  static constexpr int chunks = BK / 8;                       // 16-byte K chunks per stage
  static constexpr int a_lbo = MT * 16 * kASbo + 16;          // chunk stride (+16: conflict-free stores)
  static constexpr int a_stage = chunks * a_lbo;
  static constexpr int b_lbo = BN * 16;
  static constexpr int b_stage = chunks * b_lbo;
  static constexpr int fixed = 1024 + 16 /*alignment*/ + 256 /*barriers*/;
  static constexpr int fit = (220 * 1024 - fixed) / (a_stage + b_stage);
  static constexpr int stages = fit > 4 ? 4 : fit;
  static constexpr size_t smem = fixed + size_t(stages) * (a_stage + b_stage);
  static constexpr int used_columns = MT * BN;
  // allocations are powers of two (a 192-token tile takes 256 columns)
  static constexpr int tmem_columns = used_columns <= 32 ? 32 : used_columns <= 64 ? 64 : used_columns <= 128 ? 128 : used_columns <= 256 ? 256 : 512;
  static_assert(stages >= 2, "tile does not fit two pipeline stages");
  static_assert(BN % 32 == 0, "the activation box is made of 32-token runs");
  static_assert(used_columns <= 512 && BN % 16 == 0 && BN <= 256, "accumulators must fit 512 TMEM columns; N is a multiple of 16 up to 256");
};

struct PrefillParams {
  const uint4 *tiles;
  const uint8_t *flags;
  const float *scales;
  const __nv_bfloat16 *bias;
  const float *xmul;   // per-token multiplier 2^s * 65536/889 of the staged activations
  __nv_bfloat16 *y;
  int *status;
  int M, K, KI, MT, T;
  int palette;
  int half_io;   // bias and y are fp16 (the staged activations are fp16 either way)
  float *partial;   // gridDim.z > 1: K is cut into gridDim.z ranges of units and the scaled fp32 sums go to partial[range][T][M]
};

// ---- PTX wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait; returns false (after recording `code`) when the limit is reached or the CTA aborted.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int *abort_flag, int *status, int code) {
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  atomicCAS(status, 0, code);
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap *map, unsigned bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                          unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// K-major, no-swizzle shared-memory matrix descriptor: 8-row groups `sbo` bytes apart, 16-byte K chunks
// `lbo` bytes apart (canonical layout ((8,m),(8,2)):((16B,SBO),(2B,LBO)) for 16-bit elements).
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr, unsigned lbo, unsigned sbo) {
  return (unsigned long long)((addr >> 4) & 0x3FFF) | ((unsigned long long)((lbo >> 4) & 0x3FFF) << 16) |
         ((unsigned long long)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}

// Activation staging for the GEMM: per token an exact power-of-two rescale to fp16 (the decode GEMV's
// arithmetic), stored chunk-major -- out[(chunk * padded_tokens + token) * 8 .. +8], padded_tokens a
// multiple of 32 -- which is the K-major core-matrix order of the B operand.  A TMA box then copies
// runs of 32 tokens x 16 bytes = 512 contiguous bytes; with the row-major layout every 16-byte piece
// was a TMA row of its own and the load, not the tensor pipe, set the pace of the wide tiles.
// One CTA of 1024 threads stages eight tokens: four warps find the scaling of each token, then all
// threads convert and write 128-byte runs (eight tokens of one chunk).
constexpr int kStageThreads = 1024;
__global__ void __launch_bounds__(kStageThreads) stage_activations_kernel(const __nv_bfloat16 *__restrict__ x, __half *__restrict__ out,
                                                                          float *__restrict__ xmul, int K, int KP, int tokens,
                                                                          int padded_tokens, int half_in) {
  __shared__ unsigned warp_max[32];
  grid_launch_dependents();      // the tile kernel may set up (barriers, TMEM, first weight loads) while this one runs
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = K / 8, padded = KP / 8;
  const int first = blockIdx.x * 8;
  {
    const int tok = first + (warp >> 2);
    unsigned m = 0;
    if (tok < tokens && !half_in) {
      const uint4 *src = reinterpret_cast<const uint4 *>(x + size_t(tok) * K);
      for (int i = (warp & 3) * 32 + lane; i < chunks; i += 128) m = max(m, chunk_absmax(src[i]));
      m = __reduce_max_sync(0xffffffffu, m);
    }
    if (lane == 0) warp_max[warp] = m;
  }
  __syncthreads();
  const int j = threadIdx.x & 7, tok = first + j;
  const unsigned m = max(max(warp_max[4 * j], warp_max[4 * j + 1]), max(warp_max[4 * j + 2], warp_max[4 * j + 3]));
  float mult, inverse;
  token_scaling(m, mult, inverse);
  if (half_in) inverse = 1.f;   // fp16 activations (x then points to fp16) are the operand as they are
  if (threadIdx.x < 8 && tok < tokens && blockIdx.y == 0) xmul[tok] = inverse * kNumeratorScale;
  uint4 *dst = reinterpret_cast<uint4 *>(out);
  const uint4 *src = reinterpret_cast<const uint4 *>(x + size_t(tok < tokens ? tok : 0) * K);
  // few tokens give few CTAs: blockIdx.y cuts the conversion (not the scan above) into column slices
  const int per_slice = (padded + int(gridDim.y) - 1) / int(gridDim.y);
  const int slice_end = min(padded, (int(blockIdx.y) + 1) * per_slice);
  for (int chunk = int(blockIdx.y) * per_slice + (threadIdx.x >> 3); chunk < slice_end; chunk += kStageThreads / 8)
    dst[size_t(chunk) * padded_tokens + tok] =
        (tok < tokens && chunk < chunks) ? (half_in ? src[chunk] : convert_chunk(src[chunk], mult)) : make_uint4(0, 0, 0, 0);
}

template <int MT, int BN, int BK>
__global__ void __launch_bounds__(kPrefillThreads, 1)
prefill_umma_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap x_map) {
  using Cfg = TileConfig<MT, BN, BK>;
  constexpr int S = Cfg::stages;
  constexpr int kSubs = 128 / BK;            // pipeline stages per 128-column unit of the payload (1 or 2)
  extern __shared__ uint8_t smem_raw[];
  const unsigned sbase = unsigned(__cvta_generic_to_shared(smem_raw));
  const unsigned bars_s = (sbase + 15) & ~15u;          // barriers + small state (256 bytes)
  uint8_t *bars_g = smem_raw + (bars_s - sbase);
  const unsigned full_a = bars_s, full_b = bars_s + 8 * S, empty = bars_s + 16 * S, accum = bars_s + 24 * S;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars_g + 200);
  unsigned *tmem_slot = reinterpret_cast<unsigned *>(bars_g + 208);
  const unsigned tiles_s = (bars_s + 256 + 1023) & ~1023u;   // A stages then B stages, 1 KiB aligned
  uint8_t *tiles_g = smem_raw + (tiles_s - sbase);
  const unsigned a_s = tiles_s, b_s = tiles_s + S * Cfg::a_stage;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // Launched with programmatic stream serialisation behind the staging kernel: everything up to the first read
  // of the staged activations (the TMA lane) or of the token multipliers (the epilogue) touches only the
  // immutable payload and this CTA's own memory and may run while the staging kernel is still at work.
  grid_launch_dependents();
  // this CTA's range of 128-column units (the whole row unless the launch cuts K)
  const int u0 = int(blockIdx.z) * p.KI / int(gridDim.z), u1 = (int(blockIdx.z) + 1) * p.KI / int(gridDim.z);
  const int KT = (u1 - u0) * kSubs;                      // pipeline stages over this range
  const int row0 = blockIdx.x * Cfg::rows, tok0 = blockIdx.y * BN;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_a + 8 * s, kProducerWarps / kGroups);
      mbar_init(full_b + 8 * s, 1);
      mbar_init(empty + 8 * s, 1);
    }
    mbar_init(accum, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(bars_s + 208), "r"(unsigned(Cfg::tmem_columns)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp < kProducerWarps) {
    // ---------------- producers: BC4 -> fp16 A tile; warp w owns 16-row tiles w, w+8, ... of the CTA ----------------
    const int g = lane >> 2, t = lane & 3;
    const int tile_warp = warp % kTileWarps;
    const int group = kGroups > 1 ? warp / kTileWarps : 0, half0 = kGroups > 1 ? 0 : warp / kTileWarps;   // half0 is 0 with eight producers
    const uint4 *src[MT];
    const uint8_t *fl[MT];
    bool live[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int rt = blockIdx.x * (Cfg::rows / 16) + m * kTileWarps + tile_warp;
      live[m] = rt < p.MT;
      src[m] = p.tiles + (size_t(live[m] ? rt : 0) * p.KI) * 64 + half0 * 32 + lane;
      fl[m] = p.flags + size_t(live[m] ? rt : 0) * p.KI;
    }
    // kLook units of every tile in flight per warp as register loads.  One is enough: four measured the same at
    // 32 tokens (the pace there is set by the stage hand-over, not by DRAM latency) and 10 % slower at 512 tokens
    constexpr int kLook = 1;
    uint4 q[kLook][MT][kHalvesPerWarp];
    unsigned flag[kLook][MT];
#pragma unroll
    for (int slot = 0; slot < kLook; ++slot)
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (u0 + group + slot * kGroups < u1) {
#pragma unroll
          for (int h = 0; h < kHalvesPerWarp; ++h) q[slot][m][h] = ldg_stream(src[m] + size_t(u0 + group + slot * kGroups) * 64 + h * 32);
          flag[slot][m] = fl[m][u0 + group + slot * kGroups];
        }
      }
    bool ok = true;
    for (int base = u0 + group; base < u1 && ok; base += kLook * kGroups) {
#pragma unroll
     for (int slot = 0; slot < kLook; ++slot) {
      const int unit = base + slot * kGroups;
      if (unit >= u1 || !ok) break;                      // warp-uniform
      uint4 cq[MT][kHalvesPerWarp];
      unsigned cflag[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        cflag[m] = flag[slot][m];
#pragma unroll
        for (int h = 0; h < kHalvesPerWarp; ++h) cq[m][h] = q[slot][m][h];
        if (unit + kLook * kGroups < u1) {               // refill the slot with this warp's next unit
#pragma unroll
          for (int h = 0; h < kHalvesPerWarp; ++h) q[slot][m][h] = ldg_stream(src[m] + size_t(unit + kLook * kGroups) * 64 + h * 32);
          flag[slot][m] = fl[m][unit + kLook * kGroups];
        }
      }
#pragma unroll
      for (int part = 0; part < kSubs; ++part) {
        const int kt = (unit - u0) * kSubs + part, s = kt % S;
        if (kt >= S && !mbar_wait(empty + 8 * s, ((kt / S) - 1) & 1, abort_flag, p.status, 1)) {
          ok = false;
          break;
        }
        uint8_t *stage = tiles_g + s * Cfg::a_stage;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
#pragma unroll
          for (int h = 0; h < kHalvesPerWarp; ++h) {
            const uint4 u = cq[m][h];
            const int half = half0 + h;
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
              if (kSubs == 2 && sub != part) continue;   // 64-column stages take one block column of the unit each
              unsigned packed[8];                                   // exact numerators n * 2^-16 as fp16x2
              if (p.palette == TX_PALETTE_HARDWARE) {               // uniform
                if (sub == 0) decode_duo_first<true>(u, packed); else decode_duo_second<true>(u, packed);
              } else {
                if (sub == 0) decode_duo_first(u, packed); else decode_duo_second(u, packed);
              }
              if (cflag[m] && duo_block_is_low(u, sub)) decode_block_slow(u, sub, packed, p.palette);
              // block kb of the stage -> K chunks 2kb, 2kb+1; row = (m*8 + tile_warp)*16 + half*8 + g
              const int kb = (kSubs == 2 ? 0 : sub * 4) + t;
              uint8_t *dst = stage + (2 * kb) * Cfg::a_lbo + ((m * kTileWarps + tile_warp) * 2 + half) * kASbo + g * 16;
              // (row tiles past the end of the matrix decode tile 0 again: their accumulator rows are never stored)
              *reinterpret_cast<uint4 *>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              *reinterpret_cast<uint4 *>(dst + Cfg::a_lbo) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(full_a + 8 * s);
      }
     }
    }
  } else if (warp == kTmaWarp) {
    // ---------------- TMA: staged X tile [BN tokens x BK columns] per stage ----------------
    if (lane == 0) {
      grid_dependency_wait();              // the staged activations are complete
      int issued = 0;
      for (int kt = 0; kt < KT; ++kt) {
        const int s = kt % S;
        if (kt >= S && !mbar_wait(empty + 8 * s, ((kt / S) - 1) & 1, abort_flag, p.status, 2)) break;
        mbar_expect_tx(full_b + 8 * s, Cfg::b_stage);
        tma_load_3d(b_s + s * Cfg::b_stage, &x_map, full_b + 8 * s, 0, tok0 / 32, (u0 * kSubs + kt) * Cfg::chunks);
        issued = kt + 1;
      }
      if (*abort_flag) {
        // wait (bounded) for copies that were issued but never consumed, so none lands after exit
        for (int kt = issued > S ? issued - S : 0; kt < issued; ++kt)
          for (unsigned spin = 0; spin < (1u << 20) && !mbar_try_wait(full_b + 8 * (kt % S), (kt / S) & 1); ++spin) {}
      }
    }
  } else {
    // ---------------- MMA issue ----------------
    if (lane == 0) {
      // D = f32 (bits 4-5 = 1), A = B = f16 (format 0), both K-major, N at bit 17, M at bit 24
      const unsigned idesc = (1u << 4) | (unsigned(BN >> 3) << 17) | (unsigned(kMmaM >> 4) << 24);
      bool ok = true;
      for (int kt = 0; kt < KT && ok; ++kt) {
        const int s = kt % S;
        const unsigned parity = (kt / S) & 1;
        ok = mbar_wait(full_a + 8 * s, parity, abort_flag, p.status, 3) && mbar_wait(full_b + 8 * s, parity, abort_flag, p.status, 4);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int j = 0; j < BK / 16; ++j) {
            const unsigned long long adesc = smem_desc(a_s + s * Cfg::a_stage + m * 16 * kASbo + j * 2 * Cfg::a_lbo, Cfg::a_lbo, kASbo);
            const unsigned long long bdesc = smem_desc(b_s + s * Cfg::b_stage + j * 2 * Cfg::b_lbo, Cfg::b_lbo, 128);
            umma_bf16(tmem_base + unsigned(m * BN), adesc, bdesc, idesc, (kt | j) ? 1u : 0u);
          }
        umma_commit(empty + 8 * s);        // frees the stage when these MMAs have read it
      }
      if (ok) umma_commit(accum);          // accumulators complete
    }
  }

  // ---------------- epilogue: TMEM -> registers -> y ----------------
  if (warp < kProducerWarps) {
    grid_dependency_wait();                // xmul comes from the staging kernel
    const bool ready = mbar_wait(accum, 0, abort_flag, p.status, 5);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ready) {
      const int quarter = warp & 3;
      // the warps of one lane quarter share its MT x (BN/32) accumulator chunks
      for (int item = warp >> 2; item < MT * (BN / 32); item += kProducerWarps / 4) {
        const int m = item / (BN / 32), c = item % (BN / 32);
        const int row = row0 + m * kMmaM + quarter * 32 + lane;
        const float bias = (row < p.M && p.bias)
                               ? (p.half_io ? __half2float(reinterpret_cast<const __half *>(p.bias)[row]) : __bfloat162float(p.bias[row]))
                               : 0.f;
        const float row_scale = row < p.M ? p.scales[row] : 0.f;
        unsigned v[32];
        tmem_load32(tmem_base + (unsigned(quarter * 32) << 16) + unsigned(m * BN + c * 32), v);
        if (row < p.M) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int tok = tok0 + c * 32 + j;
            if (tok < p.T && gridDim.z > 1) {
              p.partial[(size_t(blockIdx.z) * p.T + tok) * p.M + row] = __uint_as_float(v[j]) * (row_scale * __ldg(p.xmul + tok));
            } else if (tok < p.T) {
              const float value = fmaf(__uint_as_float(v[j]), row_scale * __ldg(p.xmul + tok), bias);
              if (p.half_io) reinterpret_cast<__half *>(p.y)[size_t(tok) * p.M + row] = __float2half_rn(value);
              else p.y[size_t(tok) * p.M + row] = __float2bfloat16(value);
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(unsigned(Cfg::tmem_columns)) : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled_entry() {
  static EncodeTiled entry = [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query) != cudaSuccess ||
        query != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeTiled>(fn);
  }();
  return entry;
}

// Tile candidates behind the reference's backend ids 5..9 (texelator/autotune.py:16-22):
//   5: 128 rows x 256 tokens (baseline)   6: 256 x 256   7: 128 x 128   8: 128 x 64   9: 128 x 192
// (192 tokens: 5120-row matrices at 512+ tokens launch 120 CTAs instead of 80 or 160 on the 148 SMs)
// Tall tiles re-read the activations less often (tensor-bound prompts); narrow ones suit short prompts
// where the weight stream is the bound.
struct TileShape {
  int mt, bn, bk;
};
static TileShape backend_shape(int backend) {
  switch (backend) {
    case 5: return {1, 256, 128};
    case 6: return {2, 256, 64};
    case 7: return {1, 128, 128};
    case 8: return {1, 64, 128};
    case 9: return {1, 192, 128};
    default: return {0, 0, 0};
  }
}

bool prefill_tile_eligible(const Handle *h, int backend, int tokens) {
  return backend_shape(backend).mt != 0 && tokens >= 1 && h->K % 16 == 0 && encode_tiled_entry() != nullptr;
}

// Short prompts on matrices with few rows leave most SMs without a CTA (5120 rows = 40 CTAs of 128 rows): K is
// then cut into ranges, one CTA per (row block, token block, range), fp32 sums combined by a second kernel.  The
// number of ranges depends on the matrix and the token count only -- never on the tile -- so that all tiles keep
// adding in the same order and stay bitwise identical to each other (the autotuner's admission rule).
static int prefill_k_ranges(const Handle *h, int tokens, const Workspace *ws) {
  const int blocks = ((h->M + 127) / 128) * ((tokens + 127) / 128);
  int ranges = std::min(std::min(ws->sm_count / std::max(blocks, 1), 8), h->KI / 4);
  while (ranges > 1 && size_t(ranges) * tokens * h->M > ws->partial_floats) --ranges;
  return std::max(ranges, 1);
}

template <int MT, int BN, int BK>
static int launch_tile(const Handle *h, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream, bool half_io) {
  using Cfg = TileConfig<MT, BN, BK>;
  Workspace *ws = workspace_for(h->device);
  if (!ws) return TX_ECUDA;
  static std::mutex guard;
  static std::map<int, bool> configured;
  {
    std::lock_guard<std::mutex> lock(guard);
    if (!configured[h->device]) {
      TX_CUDA(cudaFuncSetAttribute(prefill_umma_kernel<MT, BN, BK>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(Cfg::smem)));
      configured[h->device] = true;
    }
  }
  // Activations are staged once as fp16 after an exact per-token power-of-two rescale (the decode GEMV's
  // arithmetic), in chunks of tokens that fit the per-device scratch.
  const int KP = h->KI * 128;
  const int capacity = int(std::min<size_t>(ws->xprep_halfs / size_t(KP), 65536)) & ~31;   // staged tokens are padded to 32
  if (capacity < 32) return fail(TX_EINVAL, "K is too large for the prefill activation scratch");
  for (int t0 = 0; t0 < tokens; t0 += capacity) {
    const int n = std::min(capacity, tokens - t0);
    const int padded_tokens = (n + 31) & ~31;
    const int slices = std::max(1, std::min(16, ws->sm_count / (padded_tokens / 8)));
    stage_activations_kernel<<<dim3(padded_tokens / 8, slices), kStageThreads, 0, stream>>>(x + size_t(t0) * h->K, ws->xprep, ws->xmul, h->K, KP, n,
                                                                    padded_tokens, half_io ? 1 : 0);
    count_launch();
    // staged X viewed as [KP/8 chunks][padded_tokens/32][32 tokens x 8 elements]: a box is BN/32 runs of
    // 512 contiguous bytes per chunk and lands as BN-token core-matrix columns
    CUtensorMap map;
    cuuint64_t dims[3] = {256, cuuint64_t(padded_tokens / 32), cuuint64_t(KP / 8)};
    cuuint64_t strides[2] = {512, cuuint64_t(padded_tokens) * 16};
    cuuint32_t box[3] = {256, cuuint32_t(BN / 32), cuuint32_t(Cfg::chunks)};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult cr = encode_tiled_entry()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, ws->xprep, dims, strides, box, elem,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(TX_ECUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(cr)));
    PrefillParams p{};
    p.tiles = reinterpret_cast<const uint4 *>(h->tiles);
    p.flags = h->unit_flags;
    p.scales = h->scales;
    p.bias = h->bias;
    p.xmul = ws->xmul;
    p.y = y + size_t(t0) * h->M;
    p.status = ws->status;
    p.M = h->M;
    p.K = h->K;
    p.KI = h->KI;
    p.MT = h->MT;
    p.T = n;
    p.palette = h->palette;
    p.half_io = half_io ? 1 : 0;
    p.partial = ws->partial;
    const int ranges = prefill_k_ranges(h, n, ws);
    dim3 grid((h->M + Cfg::rows - 1) / Cfg::rows, (n + BN - 1) / BN, ranges);
    TX_CUDA(launch_pdl(prefill_umma_kernel<MT, BN, BK>, grid, dim3(kPrefillThreads), Cfg::smem, stream, p, map));
    count_launch();
    if (ranges > 1) {
      int rc = launch_combine(ws->partial, ranges, h->bias, y + size_t(t0) * h->M, n, h->M, half_io, ws->sm_count, stream);
      if (rc != TX_OK) return rc;
    }
  }
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

// `half_io`: x, y and the handle's bias are fp16 (the reference multiplies fp16(pal*scale) with cuBLAS there,
// texelator_cuda.cu:996-1046; this kernel multiplies the exact numerators and scales in the epilogue)
int launch_prefill_tile(const Handle *h, int backend, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream,
                        bool half_io) {
  switch (backend) {
    case 5: return launch_tile<1, 256, 128>(h, x, y, tokens, stream, half_io);
    case 6: return launch_tile<2, 256, 64>(h, x, y, tokens, stream, half_io);
    case 7: return launch_tile<1, 128, 128>(h, x, y, tokens, stream, half_io);
    case 8: return launch_tile<1, 64, 128>(h, x, y, tokens, stream, half_io);
    case 9: return launch_tile<1, 192, 128>(h, x, y, tokens, stream, half_io);
    default: return fail(TX_EINVAL, "backend is not a tensor-core tile candidate");
  }
}

template <int MT, int BN, int BK>
static int tile_info(int64_t out[9]) {
  using Cfg = TileConfig<MT, BN, BK>;
  cudaFuncAttributes attributes{};
  TX_CUDA(cudaFuncGetAttributes(&attributes, prefill_umma_kernel<MT, BN, BK>));
  TX_CUDA(cudaFuncSetAttribute(prefill_umma_kernel<MT, BN, BK>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(Cfg::smem)));
  int active = 0;
  TX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&active, prefill_umma_kernel<MT, BN, BK>, kPrefillThreads, Cfg::smem));
  out[0] = attributes.numRegs;
  out[1] = int64_t(attributes.sharedSizeBytes);
  out[2] = int64_t(attributes.localSizeBytes);
  out[3] = attributes.maxThreadsPerBlock;
  out[4] = int64_t(Cfg::smem);
  out[5] = Cfg::rows;   // output rows per CTA
  out[6] = BN;          // tokens per CTA
  out[7] = BK;          // columns per pipeline stage
  out[8] = active;
  return TX_OK;
}

int prefill_kernel_info(int backend, int64_t out[9]) {
  switch (backend) {
    case 5: return tile_info<1, 256, 128>(out);
    case 6: return tile_info<2, 256, 64>(out);
    case 7: return tile_info<1, 128, 128>(out);
    case 8: return tile_info<1, 64, 128>(out);
    case 9: return tile_info<1, 192, 128>(out);
    default: return fail(TX_EINVAL, "backend is not a tensor-core tile candidate");
  }
}

}  // namespace tx
