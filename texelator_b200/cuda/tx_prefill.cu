// Prefill GEMM for tokens >= prefill_threshold: Y[T, M] = X[T, K] * Wq[M, K]^T on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in TMEM).
//
// Reference counterpart: the five CUTLASS 2.x tiles whose B iterator gathers BC4 texels
// (texelator/cuda/cutlass_texture_mainloop.cu:61-249, _t1/_t2/_t3/_smalln.cu; sm_80 mma.sync,
// two-stage register-staged pipeline).  B200 design, one CTA per 128 output rows x BN tokens:
//
//   pre-pass   one small kernel rescales the activations per token by an exact power of two and stores
//              them as fp16 (the decode GEMV's staging), so that both operands are fp16;
//   warps 0-7  producers: 128-bit loads of the tiled BC4 payload (one 16-row tile per warp), decode
//              in registers exactly like the decode GEMV (pair table + HFMA2 -> exact integer
//              numerators n = 7*e0 + g*(e1-e0) as fp16) and store the 128 x 128 A tile into shared
//              memory in the canonical K-major core-matrix layout (no swizzle);
//   warp 8     one lane issues the TMA load of the staged X tile (BN tokens x 128 columns) per stage
//              through a 3-D tensor map that lands in the same core-matrix layout (no multicast);
//   warp 9     allocates TMEM, and one lane issues eight tcgen05.mma kind::f16 (M=128, N=BN, K=16) per
//              stage, committing to the stage's "empty" barrier;
//   warps 0-7  epilogue: tcgen05.ld of the fp32 accumulators, * scale_m * 2^s/889, + bias, one bf16
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

constexpr int kBM = 128;                 // output rows per CTA (TMEM lanes)
constexpr int kBK = 128;                 // columns per stage = one unit of the tiled payload
constexpr int kChunks = kBK / 8;         // 16-byte K chunks (core-matrix columns) per stage
constexpr int kALbo = 2064;              // byte stride between K chunks of the A tile (2048 + 16: bank spread)
constexpr int kASbo = 128;               // byte stride between 8-row groups
constexpr int kAStage = kChunks * kALbo; // 33024
constexpr int kProducerWarps = 8;
constexpr int kPrefillThreads = 320;     // 8 producer/epilogue warps + TMA warp + MMA warp
constexpr unsigned kSpinLimit = 1u << 22;

template <int BN> struct TileConfig {
  static constexpr int stages = BN == 256 ? 2 : (BN == 128 ? 3 : 4);
  static constexpr int b_stage = BN * kBK * 2;
  static constexpr int b_lbo = BN * 16;
  static constexpr size_t smem = 1024 /*align*/ + kLutBytes * 2 + 256 /*barriers*/ + size_t(stages) * (kAStage + b_stage);
};

struct PrefillParams {
  const uint4 *tiles;
  const uint8_t *flags;
  const float *scales;
  const __nv_bfloat16 *bias;
  const float *xmul;   // per-token multiplier 2^s/889 of the staged activations
  __nv_bfloat16 *y;
  int *status;
  int M, K, KI, MT, T;
  int palette;
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

template <int BN>
__global__ void __launch_bounds__(kPrefillThreads, 1)
prefill_umma_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap x_map) {
  using Cfg = TileConfig<BN>;
  constexpr int S = Cfg::stages;
  extern __shared__ uint8_t smem_raw[];
  const unsigned sbase = unsigned(__cvta_generic_to_shared(smem_raw));
  const unsigned lut_s = (sbase + kLutBytes - 1) & ~unsigned(kLutBytes - 1);
  uint8_t *lut_g = smem_raw + (lut_s - sbase);
  const unsigned bars_s = lut_s + kLutBytes;            // barriers + small state (256 bytes)
  uint8_t *bars_g = lut_g + kLutBytes;
  const unsigned full_a = bars_s, full_b = bars_s + 8 * S, empty = bars_s + 16 * S, accum = bars_s + 24 * S;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars_g + 200);
  unsigned *tmem_slot = reinterpret_cast<unsigned *>(bars_g + 208);
  const unsigned tiles_s = (bars_s + 256 + 1023) & ~1023u;   // A stages then B stages, 1 KiB aligned
  uint8_t *tiles_g = smem_raw + (tiles_s - sbase);
  const unsigned a_s = tiles_s, b_s = tiles_s + S * kAStage;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int KT = p.KI;                                   // stages of 128 columns
  const int row0 = blockIdx.x * kBM, tok0 = blockIdx.y * BN;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_a + 8 * s, kProducerWarps);
      mbar_init(full_b + 8 * s, 1);
      mbar_init(empty + 8 * s, 1);
    }
    mbar_init(accum, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  fill_pair_table(lut_g, tid, kPrefillThreads, p.palette);
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(bars_s + 208), "r"(unsigned(BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp < kProducerWarps) {
    // ---------------- producers: BC4 -> bf16 A tile ----------------
    const int g = lane >> 2, t = lane & 3;
    const int rt = blockIdx.x * (kBM / 16) + warp;       // this warp's 16-row tile
    const bool live = rt < p.MT;
    const unsigned lut_lane = lut_s + lane * 4;
    const uint4 *src = p.tiles + (size_t(live ? rt : 0) * p.KI) * 64 + lane;
    const uint8_t *fl = p.flags + size_t(live ? rt : 0) * p.KI;
    uint4 q = ldg_stream(src), r = ldg_stream(src + 32);
    unsigned flag = fl[0];
    for (int kt = 0; kt < KT; ++kt) {
      const int s = kt % S;
      const uint4 cq = q, cr = r;
      const unsigned cflag = flag;
      if (kt + 1 < KT) {                                 // next unit in flight while this one is decoded
        q = ldg_stream(src + size_t(kt + 1) * 64);
        r = ldg_stream(src + size_t(kt + 1) * 64 + 32);
        flag = fl[kt + 1];
      }
      if (kt >= S && !mbar_wait(empty + 8 * s, ((kt / S) - 1) & 1, abort_flag, p.status, 1)) break;
      uint8_t *stage = tiles_g + s * kAStage;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint4 u = half ? cr : cq;
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          const unsigned lo = sub ? u.z : u.x, hi = sub ? u.w : u.y;
          unsigned packed[8];
          decode_block_fast(lo, hi, lut_lane, packed);          // exact integer numerators as fp16x2
          if (cflag && block_is_low(lo)) decode_block_slow(lo, hi, packed, p.palette);
          // block kb = sub*4 + t of the stage -> K chunks 2kb, 2kb+1; row = warp*16 + half*8 + g
          uint8_t *dst = stage + (2 * (sub * 4 + t)) * kALbo + (warp * 2 + half) * kASbo + g * 16;
          *reinterpret_cast<uint4 *>(dst) = live ? make_uint4(packed[0], packed[1], packed[2], packed[3]) : make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4 *>(dst + kALbo) = live ? make_uint4(packed[4], packed[5], packed[6], packed[7]) : make_uint4(0, 0, 0, 0);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(full_a + 8 * s);
    }
  } else if (warp == 8) {
    // ---------------- TMA: X tile [BN tokens x 128 columns] per stage ----------------
    if (lane == 0) {
      int issued = 0;
      for (int kt = 0; kt < KT; ++kt) {
        const int s = kt % S;
        if (kt >= S && !mbar_wait(empty + 8 * s, ((kt / S) - 1) & 1, abort_flag, p.status, 2)) break;
        mbar_expect_tx(full_b + 8 * s, Cfg::b_stage);
        tma_load_3d(b_s + s * Cfg::b_stage, &x_map, full_b + 8 * s, 0, tok0, kt * kChunks);
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
      const unsigned idesc = (1u << 4) | (unsigned(BN >> 3) << 17) | (unsigned(kBM >> 4) << 24);
      bool ok = true;
      for (int kt = 0; kt < KT && ok; ++kt) {
        const int s = kt % S;
        const unsigned parity = (kt / S) & 1;
        ok = mbar_wait(full_a + 8 * s, parity, abort_flag, p.status, 3) && mbar_wait(full_b + 8 * s, parity, abort_flag, p.status, 4);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int j = 0; j < kBK / 16; ++j) {
          const unsigned long long adesc = smem_desc(a_s + s * kAStage + j * 2 * kALbo, kALbo, kASbo);
          const unsigned long long bdesc = smem_desc(b_s + s * Cfg::b_stage + j * 2 * Cfg::b_lbo, Cfg::b_lbo, 128);
          umma_bf16(tmem_base, adesc, bdesc, idesc, (kt | j) ? 1u : 0u);
        }
        umma_commit(empty + 8 * s);        // frees the stage when these MMAs have read it
      }
      if (ok) umma_commit(accum);          // accumulators complete
    }
  }

  // ---------------- epilogue: TMEM -> registers -> y ----------------
  if (warp < kProducerWarps) {
    const bool ready = mbar_wait(accum, 0, abort_flag, p.status, 5);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ready) {
      const int quarter = warp & 3;
      const int row = row0 + quarter * 32 + lane;
      const float bias = (row < p.M && p.bias) ? __bfloat162float(p.bias[row]) : 0.f;
      const float row_scale = row < p.M ? p.scales[row] : 0.f;
      for (int c = warp >> 2; c < BN / 32; c += 2) {
        unsigned v[32];
        tmem_load32(tmem_base + (unsigned(quarter * 32) << 16) + unsigned(c * 32), v);
        if (row < p.M) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int tok = tok0 + c * 32 + j;
            if (tok < p.T)
              p.y[size_t(tok) * p.M + row] = __float2bfloat16(fmaf(__uint_as_float(v[j]), row_scale * __ldg(p.xmul + tok), bias));
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 9) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(unsigned(BN)) : "memory");
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

// Tile candidates behind the reference's backend ids 5..9 (texelator/autotune.py:16-22): token-tile
// widths of the tcgen05 kernel; id 9 is the streamed mma.sync path (handled by the dispatcher).
static int backend_tokens(int backend) {
  switch (backend) {
    case 5: return 256;
    case 6: return 128;
    case 7: return 64;
    case 8: return 32;
    default: return 0;
  }
}

bool prefill_tile_eligible(const Handle *h, int backend, int tokens) {
  return backend_tokens(backend) != 0 && tokens >= 1 && h->K % 16 == 0 && encode_tiled_entry() != nullptr;
}

template <int BN>
static int launch_tile(const Handle *h, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream) {
  Workspace *ws = workspace_for(h->device);
  if (!ws) return TX_ECUDA;
  static std::mutex guard;
  static std::map<int, bool> configured;
  {
    std::lock_guard<std::mutex> lock(guard);
    if (!configured[h->device]) {
      TX_CUDA(cudaFuncSetAttribute(prefill_umma_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(TileConfig<BN>::smem)));
      configured[h->device] = true;
    }
  }
  // Activations are staged once as fp16 after an exact per-token power-of-two rescale (the decode GEMV's
  // arithmetic), in chunks of tokens that fit the per-device scratch.
  const int KP = h->KI * 128;
  const int chunk_tokens = int(std::min<size_t>(std::min<size_t>(ws->xprep_halfs / size_t(KP), 65536), size_t(tokens)));
  if (chunk_tokens < 1) return fail(TX_EINVAL, "K is too large for the prefill activation scratch");
  for (int t0 = 0; t0 < tokens; t0 += chunk_tokens) {
    const int n = std::min(chunk_tokens, tokens - t0);
    int rc = launch_activation_prepass(x + size_t(t0) * h->K, ws->xprep, ws->xmul, n, h->K, KP, stream);
    if (rc != TX_OK) return rc;
    // staged X viewed as [KP/8 chunks][n tokens][8 elements]: one box lands as BN-token core-matrix columns
    CUtensorMap map;
    cuuint64_t dims[3] = {8, cuuint64_t(n), cuuint64_t(KP / 8)};
    cuuint64_t strides[2] = {cuuint64_t(KP) * 2, 16};
    cuuint32_t box[3] = {8, cuuint32_t(BN), cuuint32_t(kChunks)};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult cr = encode_tiled_entry()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, ws->xprep, dims, strides, box, elem,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
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
    dim3 grid((h->M + kBM - 1) / kBM, (n + BN - 1) / BN);
    prefill_umma_kernel<BN><<<grid, kPrefillThreads, TileConfig<BN>::smem, stream>>>(p, map);
    count_launch();
  }
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

int launch_prefill_tile(const Handle *h, int backend, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream) {
  if (tokens > 65535 * 32) return fail(TX_EINVAL, "token grid exceeds CUDA grid.y limit");
  switch (backend_tokens(backend)) {
    case 256: return launch_tile<256>(h, x, y, tokens, stream);
    case 128: return launch_tile<128>(h, x, y, tokens, stream);
    case 64: return launch_tile<64>(h, x, y, tokens, stream);
    case 32: return launch_tile<32>(h, x, y, tokens, stream);
    default: return fail(TX_EINVAL, "backend is not a tensor-core tile candidate");
  }
}

template <int BN>
static int tile_info(int64_t out[9]) {
  cudaFuncAttributes attributes{};
  TX_CUDA(cudaFuncGetAttributes(&attributes, prefill_umma_kernel<BN>));
  TX_CUDA(cudaFuncSetAttribute(prefill_umma_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(TileConfig<BN>::smem)));
  int active = 0;
  TX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&active, prefill_umma_kernel<BN>, kPrefillThreads, TileConfig<BN>::smem));
  out[0] = attributes.numRegs;
  out[1] = int64_t(attributes.sharedSizeBytes);
  out[2] = int64_t(attributes.localSizeBytes);
  out[3] = attributes.maxThreadsPerBlock;
  out[4] = int64_t(TileConfig<BN>::smem);
  out[5] = kBM;   // output rows per CTA
  out[6] = BN;    // tokens per CTA
  out[7] = kBK;   // columns per pipeline stage
  out[8] = active;
  return TX_OK;
}

int prefill_kernel_info(int backend, int64_t out[9]) {
  switch (backend_tokens(backend)) {
    case 256: return tile_info<256>(out);
    case 128: return tile_info<128>(out);
    case 64: return tile_info<64>(out);
    case 32: return tile_info<32>(out);
    default: return gemv_kernel_info(out);   // id 9: the streamed mma.sync path
  }
}

}  // namespace tx
