// Decode GEMV for tokens < prefill_threshold (reference: texelator_bc4_bf16_kernel,
// texelator/cuda/texelator_cuda.cu:141-199, one warp per output row through the texture unit).
//
// B200 design.  A persistent CTA walks 16-row tiles of the tiled BC4 payload; its eight warps split
// the tile's 1 KiB units (16 rows x 128 columns) round-robin, keep LOOKAHEAD units in flight as
// 128-bit loads, and turn each unit into eight mma.sync m16n8k16 A fragments entirely in registers:
//
//   * the payload stores, per weight, the interpolation index g as a 3-bit field placed inside the
//     mantissa of an fp16 half ("duo" layout, tx_common.cuh), so one AND per pair of weights yields
//     the fp16x2 pair (g_even, g_odd) * 2^(offset-24) -- no table, no shared-memory access;
//   * per block, the two endpoint bytes become fp16x2 constants base = 7*e0 * 2^-16 and
//     delta * 2^(8-offset) (byte-permute into the fp16 "1024+u" encoding, HSUB2, HFMA2, three HMUL2);
//   * one HFMA2 per pair gives the exact numerators n * 2^-16, n = 7*e0 + g*(e1-e0), |n| <= 889.
//
// Activations are converted once per CTA to fp16 after an exact power-of-two scaling per token
// (so any bf16 range is safe), the tensor core accumulates n*x in fp32, and the epilogue applies
// scale_m * 2^s * 65536/889 and the bias before the single bf16 rounding.  The weights are therefore
// never rounded to bf16: the result is the un-rounded BC4 linear, which differs from the
// reference's bf16(pal*scale) arithmetic by that rounding only (rel-RMS about 1e-3).
// Blocks in the low palette mode (e0 <= e1) are rare; units that contain one are flagged at pack
// time and take a warp-uniform slow path with per-weight arithmetic.
//
// The warps of a CTA combine their fp32 partial tiles through shared memory in warp order, so
// results are deterministic; the only waits in this file are CTA barriers.
#include <map>
#include <mutex>
#include <tuple>

#include "tx_common.cuh"
#include "tx_decode.cuh"

namespace tx {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kMaxTokenTiles = 4;          // 8 tokens per tile
constexpr int kXChunks = 9;                // 8-element activation chunks a thread keeps in registers while staging
constexpr int kXsPad = 16;                 // bytes added to the shared token stride (bank spread)
constexpr size_t kSmemBudget = 200 * 1024; // dynamic shared memory we allow one CTA to take
constexpr int kSmallBytes = 512;           // token multipliers, reduction words, a block of zeros

struct GemvParams {
  const uint4 *tiles;
  const uint8_t *flags;
  const float *scales;
  const __nv_bfloat16 *bias;
  const __nv_bfloat16 *x;   // [T, K]
  __nv_bfloat16 *y;         // [T, M]
  const __half *xprep;      // [T, KP] pre-scaled fp16 activations (PRE) or null
  const float *xmul;        // [T] 2^s * 65536/889 per token (PRE)
  int M, K, KI, T, MT;
  int KP;                   // KI * 128
  int palette;              // TX_PALETTE_* in the low byte; kHalfIO: bias and y are fp16 (the activations then come through xprep)
  // fused prologue (FUSE & 1): x is the residual stream; a = rmsnorm(bf16(x + delta)) * gamma feeds the linear
  // The pre-pass variants (PRE) have no fused prologue and reuse two of its fields (the parameter block stays
  // at its size): K is cut into `splits` ranges, CTA c takes range c % splits of row tiles c / splits, ... and
  // stages only its range of the activations; with splits > 1 the scaled fp32 sums go to partial[split][T][M].
  union {
    const __nv_bfloat16 *delta;   // [T, K] or null
    float *partial;
  };
  const __nv_bfloat16 *gamma;   // [K]
  __nv_bfloat16 *residual_out;  // [T, K] or null: receives bf16(x + delta); must not alias x
  union {
    float eps;
    int splits;
  };
};

// extras of the single-token kernel (kept out of GemvParams: the general kernel measured 4 % slower with
// the larger parameter block)
struct SoloExtras {
  const uint8_t *staged;        // the token in staged form (tx_decode.cuh) or null: stage p.x in the kernel
  float *y_partial;             // [splits][partial_stride] fp32 row sums of the K ranges, or null: bf16 to y
  size_t partial_stride;
  int splits;                   // K ranges per row tile (divides KI); 1 unless y_partial is used
  PeerPush push;                // world > 0: the bf16 result goes as packets into every rank's inbox
};

constexpr int kHalfIO = 0x100;   // flag in GemvParams::palette (a field of its own would grow the parameter block)
constexpr int kFuseNorm = 1;     // residual add + RMSNorm in the activation staging
constexpr int kFuseSwiglu = 2;   // rows are (gate, up) pairs: y[t, i] = silu(gate_i) * up_i

// Pre-pass for larger token counts: one CTA per token writes scaled fp16 activations and the
// per-token multiplier 2^s * 65536/889 to scratch.  fp16 activations (HALF) already are what the
// tensor core takes: they are copied with the row padded to whole units, multiplier 65536/889.
template <bool HALF>
__global__ void __launch_bounds__(kGemvThreads) gemv_xprep_kernel(const void *__restrict__ x, __half *__restrict__ xprep,
                                                                 float *__restrict__ xmul, int K, int KP) {
  __shared__ unsigned warp_max[kGemvWarps];
  grid_launch_dependents();      // the main kernel's first weight loads may overlap this pass
  grid_dependency_wait();
  int tok = blockIdx.x;
  const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(x) + size_t(tok) * K);
  int chunks = K / 8, padded = KP / 8;
  if (HALF) {
    if (threadIdx.x == 0) xmul[tok] = kNumeratorScale;
    uint4 *copy = reinterpret_cast<uint4 *>(xprep + size_t(tok) * KP);
    for (int i = threadIdx.x; i < padded; i += kGemvThreads) copy[i] = i < chunks ? __ldcg(src + i) : make_uint4(0, 0, 0, 0);
    return;
  }
  unsigned m = 0;
  for (int i = threadIdx.x; i < chunks; i += kGemvThreads) m = max(m, chunk_absmax(__ldcg(src + i)));
  m = __reduce_max_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  m = 0;
#pragma unroll
  for (int w = 0; w < kGemvWarps; ++w) m = max(m, warp_max[w]);
  float mult, inverse;
  token_scaling(m, mult, inverse);
  if (threadIdx.x == 0) xmul[tok] = inverse * kNumeratorScale;
  uint4 *dst = reinterpret_cast<uint4 *>(xprep + size_t(tok) * KP);
  for (int i = threadIdx.x; i < padded; i += kGemvThreads)
    dst[i] = i < chunks ? convert_chunk(__ldcg(src + i), mult) : make_uint4(0, 0, 0, 0);
}

// ------------------------------------------------------------------------------------------
// Decode GEMV, one 16-row tile per CTA iteration.  A persistent CTA walks row tiles
// blockIdx.x, blockIdx.x + gridDim.x, ...; its warps split the tile's column units round-robin
// (unit ki = warp, warp + WS, ...), keep LOOKAHEAD units in flight across tile boundaries, and
// combine their fp32 partial tiles through shared memory (double-buffered, one named barrier per
// tile).  No global scratch, no atomics, deterministic summation order.
// ------------------------------------------------------------------------------------------
template <int LOOKAHEAD, int NT, bool PRE, bool LOWMODE, int FUSE = 0>
__global__ void __launch_bounds__(kGemvThreads, (NT == 1 && LOOKAHEAD <= 2) ? 3 : (NT <= 2 ? 2 : 1))
gemv_tile_kernel(const GemvParams p) {
  static_assert(FUSE == 0 || (NT == 1 && !PRE), "fused variants stage their activations in the CTA");
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const unsigned sbase = unsigned(__cvta_generic_to_shared(smem_raw));
  float *tokmul = reinterpret_cast<float *>(smem_raw);                  // 32 floats
  unsigned *red = reinterpret_cast<unsigned *>(smem_raw + 128);         // 8 words (+ 8 floats of the fused norm)
  uint4 *zero_g = reinterpret_cast<uint4 *>(smem_raw + 256);            // 256 zero bytes
  float *part_g = reinterpret_cast<float *>(smem_raw + kSmallBytes);    // [2][8 warps][NT*128] partial tiles
  constexpr int kPartBytes = 2 * kGemvWarps * NT * 128 * 4;
  uint8_t *xs_g = smem_raw + kSmallBytes + kPartBytes;
  const unsigned zero_s = sbase + 256;
  const unsigned xs_s = sbase + kSmallBytes + kPartBytes;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // same value, but known to be warp-uniform
  const int g = lane >> 2, t = lane & 3;
  const int KI = p.KI, MT = p.MT;
  // this CTA's range of column units [kbeg, kbeg + KR) and its first row tile (the whole row without PRE)
  const int S = PRE ? p.splits : 1;
  const int split = PRE ? int(blockIdx.x) % S : 0;
  const int kbeg = PRE ? split * KI / S : 0;
  const int KR = PRE ? (split + 1) * KI / S - kbeg : KI;
  const int tile0 = PRE ? int(blockIdx.x) / S : int(blockIdx.x);
  const int tile_stride = PRE ? int(gridDim.x) / S : int(gridDim.x);
  const unsigned xs_stride = (PRE ? unsigned((KI + S - 1) / S) * 256 : unsigned(p.KP) * 2) + kXsPad;
  const int WS = KR < kGemvWarps ? KR : kGemvWarps;   // warps that own column units
  const bool worker = warp < WS;
  const int per_tile = worker ? (KR - warp + WS - 1) / WS : 0;   // units of this warp in every tile

  // -- first loads, issued before anything else.  The prefetch pointer walks this warp's units
  //    (ki = kbeg + warp, + WS, ... of tiles tile0, + tile_stride, ...) and stops at the end of the payload.
  // The walk is kept as a 32-bit unit index (payloads stay far below 2^32 units) and stops loading at the
  // end of the payload.
  const unsigned unit_limit = unsigned(MT) * unsigned(KI);
  unsigned unext = unsigned(tile0) * unsigned(KI) + unsigned(kbeg + warp);
  const unsigned step_unit = WS, step_tile = unsigned(tile_stride) * unsigned(KI) - unsigned(per_tile - 1) * unsigned(WS);
  int pcount = 0;
  uint4 pend[LOOKAHEAD][2];
  unsigned pflag[LOOKAHEAD];
  auto prefetch = [&](int slot) {
    if (unext < unit_limit) {                  // (one shared padding unit would be a hot spot for every warp's tail)
      const uint4 *src = p.tiles + size_t(unext) * 64 + lane;
      pend[slot][0] = ldg_stream(src);
      pend[slot][1] = ldg_stream(src + 32);
      if (LOWMODE) pflag[slot] = p.flags[unext];
    }
    const bool wrap = pcount == per_tile - 1;
    unext += wrap ? step_tile : step_unit;
    pcount = wrap ? 0 : pcount + 1;
  };
#pragma unroll
  for (int i = 0; i < LOOKAHEAD; ++i) prefetch(i);

  if (tid < 16) zero_g[tid] = make_uint4(0, 0, 0, 0);
  // Everything above touched only the immutable payload and shared memory; the activations below are
  // produced by the previous kernel on the stream.
  grid_launch_dependents();
  grid_dependency_wait();

  // -- activations -> fp16 in shared memory
  const int chunks = p.K / 8, padded = p.KP / 8;
  if (PRE) {
    const int range_chunks = KR * 16;
    for (int tok = 0; tok < p.T; ++tok) {
      const uint4 *xp = reinterpret_cast<const uint4 *>(p.xprep + size_t(tok) * p.KP) + kbeg * 16;
      uint4 *dst = reinterpret_cast<uint4 *>(xs_g + size_t(tok) * xs_stride);
      for (int i = tid; i < range_chunks; i += kGemvThreads) dst[i] = __ldcg(xp + i);
    }
    if (tid < p.T) tokmul[tid] = __ldcg(p.xmul + tid);
  } else {
    for (int tok = 0; tok < p.T; ++tok) {
      // one trip to global memory: the first kXChunks*256 chunks stay in registers between the
      // magnitude scan and the conversion (covers K <= 18432); longer rows re-read the rest
      const uint4 *xp = reinterpret_cast<const uint4 *>(p.x + size_t(tok) * p.K);
      uint4 held[kXChunks];
      unsigned m = 0;
      if (FUSE & kFuseNorm) {
        // residual add and RMSNorm with the rounding points of separate kernels: r = bf16(x + delta),
        // a = bf16(r * inv * gamma).  Every CTA computes the row (K <= 18432 stays in registers); CTA 0
        // also stores r.  Rows longer than that are rejected by the launcher.
        const uint4 *dp = p.delta ? reinterpret_cast<const uint4 *>(p.delta + size_t(tok) * p.K) : nullptr;
        uint4 *rp = (p.residual_out && blockIdx.x == 0) ? reinterpret_cast<uint4 *>(p.residual_out + size_t(tok) * p.K) : nullptr;
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < kXChunks; ++c) {
          const int i = tid + c * kGemvThreads;
          if (i < chunks) {
            uint4 v = __ldcg(xp + i);
            __nv_bfloat162 *pv = reinterpret_cast<__nv_bfloat162 *>(&v);
            if (dp) {
              const uint4 d = __ldcg(dp + i);
              const __nv_bfloat162 *pd = reinterpret_cast<const __nv_bfloat162 *>(&d);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 a = __bfloat1622float2(pv[e]), b = __bfloat1622float2(pd[e]);
                pv[e] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
              }
            }
            if (rp) rp[i] = v;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 a = __bfloat1622float2(pv[e]);
              ss += a.x * a.x + a.y * a.y;
            }
            held[c] = v;
          }
        }
#pragma unroll
        for (int d = 16; d; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
        float *ss_part = reinterpret_cast<float *>(red + kGemvWarps);
        if (lane == 0) ss_part[warp] = ss;
        __syncthreads();
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kGemvWarps; ++w) total += ss_part[w];
        const float inv = rsqrtf(total / float(p.K) + p.eps);
        const uint4 *gp = reinterpret_cast<const uint4 *>(p.gamma);
#pragma unroll
        for (int c = 0; c < kXChunks; ++c) {
          const int i = tid + c * kGemvThreads;
          if (i < chunks) {
            uint4 v = held[c];
            const uint4 gw = gp[i];
            __nv_bfloat162 *pv = reinterpret_cast<__nv_bfloat162 *>(&v);
            const __nv_bfloat162 *pg = reinterpret_cast<const __nv_bfloat162 *>(&gw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 a = __bfloat1622float2(pv[e]), gm = __bfloat1622float2(pg[e]);
              pv[e] = __floats2bfloat162_rn(a.x * inv * gm.x, a.y * inv * gm.y);
            }
            held[c] = v;
            m = max(m, chunk_absmax(v));
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < kXChunks; ++c) {
          const int i = tid + c * kGemvThreads;
          if (i < chunks) {
            held[c] = __ldcg(xp + i);   // L2 read: another kernel wrote these moments ago
            m = max(m, chunk_absmax(held[c]));
          }
        }
        for (int i = tid + kXChunks * kGemvThreads; i < chunks; i += kGemvThreads) m = max(m, chunk_absmax(__ldcg(xp + i)));
      }
      m = __reduce_max_sync(0xffffffffu, m);
      if (lane == 0) red[warp] = m;
      __syncthreads();
      m = 0;
#pragma unroll
      for (int w = 0; w < kGemvWarps; ++w) m = max(m, red[w]);
      float mult, inverse;
      token_scaling(m, mult, inverse);
      if (tid == 0) tokmul[tok] = inverse * kNumeratorScale;
      uint4 *dst = reinterpret_cast<uint4 *>(xs_g + size_t(tok) * xs_stride);
#pragma unroll
      for (int c = 0; c < kXChunks; ++c) {
        const int i = tid + c * kGemvThreads;
        if (i < padded) dst[i] = i < chunks ? convert_chunk(held[c], mult) : make_uint4(0, 0, 0, 0);
      }
      for (int i = tid + kXChunks * kGemvThreads; i < padded; i += kGemvThreads)
        dst[i] = i < chunks ? convert_chunk(__ldcg(xp + i), mult) : make_uint4(0, 0, 0, 0);
      __syncthreads();
    }
  }
  __syncthreads();
  if (!worker || tile0 >= MT) return;

  // shared address of this lane's activations per token tile (token = 8*nt + g); lanes whose token
  // does not exist read a block of zeros instead and never advance
  unsigned xs_lane[NT], xs_step[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    bool ok = nt * 8 + g < p.T;
    xs_lane[nt] = ok ? xs_s + unsigned(nt * 8 + g) * xs_stride + t * 32 : zero_s + t * 32;
    xs_step[nt] = ok ? 0xffffffffu : 0u;
  }

  // output elements this thread finalises: e = wtid + j*workers, e = (nt*4 + qd)*32 + lane'
  const int workers = WS * 32;
  constexpr int kElems = NT * 128;
  constexpr int kPerThread = (kElems + 31) / 32;   // upper bound (one worker warp)
  float row_scale[kPerThread], row_bias[kPerThread];
  constexpr int kPairConstants = (FUSE & kFuseSwiglu) ? kPerThread : 1;
  float up_scale[kPairConstants], up_bias[kPairConstants];   // SwiGLU: constants of the paired up row (tile row + 8)
  bool row_live[kPerThread];   // this thread's element exists (row < M, token < T)
  auto load_row_constants = [&](int rt) {
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
      if (j * workers >= kElems) break;        // uniform: with eight worker warps only j = 0 exists
      int e = tid + j * workers;
      int row = rt * 16 + ((e >> 6) & 1) * 8 + ((e & 31) >> 2);
      int tok = (e >> 7) * 8 + 2 * (e & 3) + ((e >> 5) & 1);
      bool ok = e < kElems && row < p.M && tok < p.T;
      if (FUSE & kFuseSwiglu) ok = ok && ((e >> 6) & 1) == 0;   // the gate element's thread finishes the pair
      row_live[j] = ok;
      row_scale[j] = ok ? p.scales[row] : 0.f;
      row_bias[j] = ok && p.bias ? __bfloat162float(p.bias[row]) : 0.f;
      if (PRE && (p.palette & kHalfIO) && ok && p.bias) row_bias[j] = __half2float(reinterpret_cast<const __half *>(p.bias)[row]);
      if (FUSE & kFuseSwiglu) {
        up_scale[j] = ok ? p.scales[row + 8] : 0.f;
        up_bias[j] = ok && p.bias ? __bfloat162float(p.bias[row + 8]) : 0.f;
      }
    }
  };

  // two independent accumulator chains halve the mma latency chain
  float acc[NT][4], acc2[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[nt][q] = acc2[nt][q] = 0.f;

  uint4 bsolo[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};   // B fragments of the NT == 1 path
  int tile = tile0, done = 0, buf = 0;
  unsigned xoff = unsigned(warp) * 256;
  const unsigned xoff_step = unsigned(WS) * 256;
  load_row_constants(tile);
  while (true) {
#pragma unroll
    for (int slot = 0; slot < LOOKAHEAD; ++slot) {
      const uint4 q = pend[slot][0], r = pend[slot][1];   // duos of rows g and g+8
      const unsigned flag = pflag[slot];
      // ---- one unit: blocks (ki*8 + t) [sub 0] and (ki*8 + 4 + t) [sub 1] of rows g and g+8
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        unsigned aq[8], ar[8];
        if (LOWMODE && (p.palette & 0xff) == TX_PALETTE_HARDWARE) {   // uniform
          if (sub == 0) { decode_duo_first<true>(q, aq); decode_duo_first<true>(r, ar); }
          else { decode_duo_second<true>(q, aq); decode_duo_second<true>(r, ar); }
        } else {
          if (sub == 0) { decode_duo_first(q, aq); decode_duo_first(r, ar); }
          else { decode_duo_second(q, aq); decode_duo_second(r, ar); }
        }
        if (LOWMODE && __any_sync(0xffffffffu, flag != 0)) {   // rare, warp-uniform: redo the low-mode blocks
          if (duo_block_is_low(q, sub)) decode_block_slow(q, sub, aq, p.palette & 0xff);
          if (duo_block_is_low(r, sub)) decode_block_slow(r, sub, ar, p.palette & 0xff);
        }
        if (NT == 1) {
          // One token tile: lanes whose token does not exist skip the load (their MMA columns are never
          // stored, so whatever their registers hold is fine).  With a single token only four lanes of
          // the warp touch shared memory: one wavefront per load instead of five.
          if (xs_step[0]) {
            const unsigned xa = xs_lane[0] + xoff + sub * 128;
            bsolo[0] = lds128(xa);
            bsolo[1] = lds128(xa + 16);
          }
          mma_f16(acc[0], aq[0], ar[0], aq[1], ar[1], bsolo[0].x, bsolo[0].y);
          mma_f16(acc2[0], aq[2], ar[2], aq[3], ar[3], bsolo[0].z, bsolo[0].w);
          mma_f16(acc[0], aq[4], ar[4], aq[5], ar[5], bsolo[1].x, bsolo[1].y);
          mma_f16(acc2[0], aq[6], ar[6], aq[7], ar[7], bsolo[1].z, bsolo[1].w);
        }
#pragma unroll
        for (int nt = 0; nt < (NT == 1 ? 0 : NT); ++nt) {
          const unsigned xa = xs_lane[nt] + (xoff & xs_step[nt]) + sub * 128;
          const uint4 b0 = lds128(xa), b1 = lds128(xa + 16);
          mma_f16(acc[nt], aq[0], ar[0], aq[1], ar[1], b0.x, b0.y);
          mma_f16(acc2[nt], aq[2], ar[2], aq[3], ar[3], b0.z, b0.w);
          mma_f16(acc[nt], aq[4], ar[4], aq[5], ar[5], b1.x, b1.y);
          mma_f16(acc2[nt], aq[6], ar[6], aq[7], ar[7], b1.z, b1.w);
        }
      }
      prefetch(slot);   // refill the slot only now: its registers are free, so no copies are needed
      xoff += xoff_step;
      if (++done == per_tile) {
        // ---- this warp's share of the tile is done: publish the partial, combine, store
        float *mine = part_g + (buf * kGemvWarps + warp) * kElems + lane;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int qd = 0; qd < 4; ++qd) {
            mine[(nt * 4 + qd) * 32] = acc[nt][qd] + acc2[nt][qd];
            acc[nt][qd] = acc2[nt][qd] = 0.f;
          }
        asm volatile("bar.sync 1, %0;" ::"r"(workers) : "memory");
#pragma unroll
        for (int j = 0; j < kPerThread; ++j) {
          if (j * workers >= kElems) break;    // uniform
          const int e = tid + j * workers;
          if (row_live[j]) {
            const float *src = part_g + buf * kGemvWarps * kElems + e;
            float sum = 0.f;
            if (WS == kGemvWarps) {              // the usual case, unrolled; same order either way
#pragma unroll
              for (int w = 0; w < kGemvWarps; ++w) sum += src[w * kElems];
            } else {
              for (int w = 0; w < WS; ++w) sum += src[w * kElems];
            }
            const int c = e >> 5, ln = e & 31;
            const int row = tile * 16 + ((c >> 1) & 1) * 8 + (ln >> 2);
            const int tok = (c >> 2) * 8 + 2 * (ln & 3) + (c & 1);
            if (FUSE & kFuseSwiglu) {
              // element e + 64 is the up row of this gate row; both are rounded to bf16 first, like the
              // outputs of an unfused linear, then combined with silu_mul's arithmetic
              float up_sum = 0.f;
              if (WS == kGemvWarps) {
#pragma unroll
                for (int w = 0; w < kGemvWarps; ++w) up_sum += src[w * kElems + 64];
              } else {
                for (int w = 0; w < WS; ++w) up_sum += src[w * kElems + 64];
              }
              const float gate = __bfloat162float(__float2bfloat16(fmaf(sum, row_scale[j] * tokmul[tok], row_bias[j])));
              const float up = __bfloat162float(__float2bfloat16(fmaf(up_sum, up_scale[j] * tokmul[tok], up_bias[j])));
              p.y[size_t(tok) * (p.M / 2) + tile * 8 + (ln >> 2)] = __float2bfloat16(gate / (1.f + __expf(-gate)) * up);
            } else if (PRE && S > 1) {
              p.partial[(size_t(split) * p.T + tok) * p.M + row] = sum * (row_scale[j] * tokmul[tok]);
            } else if (PRE && (p.palette & kHalfIO)) {
              reinterpret_cast<__half *>(p.y)[size_t(tok) * p.M + row] = __float2half_rn(fmaf(sum, row_scale[j] * tokmul[tok], row_bias[j]));
            } else {
              p.y[size_t(tok) * p.M + row] = __float2bfloat16(fmaf(sum, row_scale[j] * tokmul[tok], row_bias[j]));
            }
          }
        }
        buf ^= 1;
        tile += tile_stride;
        if (tile >= MT) return;
        done = 0;
        xoff = unsigned(warp) * 256;
        load_row_constants(tile);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Single-token decode GEMV (tokens == 1, software palette, no low-mode block): the same walk over the
// payload as gemv_tile_kernel, but the per-weight HFMA2 is gone.  With one token seven of the eight
// MMA columns are idle, so they are used to keep the eight blocks of a unit apart:
//
//   * A operand = the masked index fields themselves (one AND per pair of weights): fp16x2 subnormals
//     g * 2^(offset-24).  K slots (2t, 2t+1) of MMA i carry pair i of the lane's first block (block t
//     of the unit), slots (2t+8, 2t+9) pair i of its second block (block t+4).
//   * B operand: column 2t holds the activations of block t, column 2t+1 those of block t+4, zeros
//     elsewhere -- so only the eight lanes g = 2t / g = 2t+1 ever load activations.  The activations
//     are staged with the factor 2^-offset of the field they meet, so every product is g*x * 2^-24.
//   * ten MMAs (pairs 0-6, pair 7 + spare-bit plane 0, planes 1 and 2; two accumulator chains,
//     summed afterwards) leave in the C fragment of lane
//     (g, t) the four sums G = sum_k g_k x_k of its own four blocks (rows g, g+8 x blocks t, t+4);
//     four FFMAs add delta * G to the lane's two row accumulators.
//   * the base term sum_b 7*e0_b * S_b (S_b = sum of the block's activations) is one more MMA per unit
//     into a persistent accumulator: A = the endpoints e0 as exact fp16 integers, B = 7*S_b * 2^-24
//     split into an fp16 high and low part (K slots 0-7 and 8-15), column 0 only.
//
// Per unit: 42 logic instructions for the fields, 4 byte-permutes and 8 half-precision operations for
// the endpoints, 11 MMAs, 4 FFMAs -- about half the instructions of the generic kernel.  Row sums are
// combined over the four lanes of a row by shuffles and over the warps through shared memory in warp
// order (deterministic; independent of LOOKAHEAD and of the number of rows of the matrix).
// ------------------------------------------------------------------------------------------
#ifndef TX_SOLO_MIN_CTAS
#define TX_SOLO_MIN_CTAS 2   // resident CTAs per SM the compiler must leave registers for (build-time tuning knob)
#endif
constexpr int kSoloSmallBytes = 256;                               // token multiplier, reduction words
constexpr int kSoloPartBytes = 2 * kGemvWarps * 16 * 4;            // [2][8 warps][16 rows]

__device__ __forceinline__ uint2 lds64(unsigned addr) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ unsigned hadd2_u(unsigned a, unsigned b) {
  unsigned d;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ void mma_f16_zero(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Work items: an item is one 16-row tile, or with e.splits > 1 the s-th of `splits` equal K ranges of
// a tile (item = tile * splits + s).  K-split items make matrices with few row tiles (5120 rows = 320
// tiles on 296 resident CTAs) fill the machine evenly; their fp32 row sums go to p.y_partial[s][row]
// and whoever consumes the linear adds the `splits` vectors in split order (the residual add + RMSNorm
// kernel does).  Units of item `it` are it * KIs .. it * KIs + KIs - 1 of the payload (KIs = KI / splits).
template <int LOOKAHEAD, bool SWIGLU>
__global__ void __launch_bounds__(kGemvThreads, TX_SOLO_MIN_CTAS) gemv_solo_kernel(const GemvParams p, const SoloExtras e) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const unsigned sbase = unsigned(__cvta_generic_to_shared(smem_raw));
  float *tokmul = reinterpret_cast<float *>(smem_raw);
  unsigned *red = reinterpret_cast<unsigned *>(smem_raw + 128);
  float *part_g = reinterpret_cast<float *>(smem_raw + kSoloSmallBytes);          // [2][8 warps][16 rows]
  uint8_t *stab_g = smem_raw + kSoloSmallBytes + kSoloPartBytes;                  // KI * 32 bytes
  uint8_t *xs_g = stab_g + size_t(p.KI) * 32;                                     // KP fp16 values
  const unsigned stab_s = sbase + kSoloSmallBytes + kSoloPartBytes;
  const unsigned xs_s = stab_s + unsigned(p.KI) * 32;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int g = lane >> 2, t = lane & 3;
  const int KI = p.KI, S = e.splits, KIs = KI / S, items = p.MT * S;
  const int WS = KIs < kGemvWarps ? KIs : kGemvWarps;
  const bool worker = warp < WS;
  const int per_item = worker ? (KIs - warp + WS - 1) / WS : 0;

  const int item_stride = gridDim.x;
  const unsigned unit_limit = unsigned(items) * unsigned(KIs);
  unsigned unext = unsigned(blockIdx.x) * unsigned(KIs) + unsigned(warp);
  const unsigned step_unit = WS, step_item = unsigned(item_stride) * unsigned(KIs) - unsigned(per_item - 1) * unsigned(WS);
  int pcount = 0;
  uint4 pend[LOOKAHEAD][2];
  auto prefetch = [&](int slot) {
    if (unext < unit_limit) {
      const uint4 *src = p.tiles + size_t(unext) * 64 + lane;
      pend[slot][0] = ldg_stream(src);
      pend[slot][1] = ldg_stream(src + 32);
    }
    const bool wrap = pcount == per_item - 1;
    unext += wrap ? step_item : step_unit;
    pcount = wrap ? 0 : pcount + 1;
  };
#pragma unroll
  for (int i = 0; i < LOOKAHEAD; ++i) prefetch(i);
  grid_launch_dependents();
  grid_dependency_wait();

  // -- the token -> scaled fp16 activations and block sums in shared memory
  {
    const int chunks = p.K / 8, padded = p.KP / 8;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    if (e.staged) {
      // the kernel that produced the activations wrote them in staged form (tx_decode.cuh): copy
      const uint4 *src = reinterpret_cast<const uint4 *>(e.staged + kStagedHeader);
      uint4 *dst = reinterpret_cast<uint4 *>(stab_g);
      const int total = KI * 18;
      for (int i = tid; i < total; i += kGemvThreads) dst[i] = __ldcg(src + i);
      if (tid == 0) tokmul[0] = __ldcg(reinterpret_cast<const float *>(e.staged));
    } else {
      const uint4 *xp = reinterpret_cast<const uint4 *>(p.x);
      uint4 held[kXChunks];
      unsigned m = 0;
#pragma unroll
      for (int c = 0; c < kXChunks; ++c) {
        const int i = tid + c * kGemvThreads;
        held[c] = i < chunks ? __ldcg(xp + i) : zero4;     // L2 read: another kernel wrote these moments ago
        m = max(m, chunk_absmax(held[c]));
      }
      for (int i = tid + kXChunks * kGemvThreads; i < chunks; i += kGemvThreads) m = max(m, chunk_absmax(__ldcg(xp + i)));
      m = __reduce_max_sync(0xffffffffu, m);
      if (lane == 0) red[warp] = m;
      __syncthreads();
      m = 0;
#pragma unroll
      for (int w = 0; w < kGemvWarps; ++w) m = max(m, red[w]);
      float mult, inverse;
      token_scaling(m, mult, inverse);
      if (tid == 0) tokmul[0] = inverse * kSoloScale;
#pragma unroll
      for (int c = 0; c < kXChunks; ++c) {
        const int i = tid + c * kGemvThreads;
        if (i - lane < padded) solo_stage_chunk(i, held[c], mult, xs_g, stab_g, i < padded);   // whole warps enter
      }
      for (int i0 = kXChunks * kGemvThreads + (tid - lane); i0 < padded; i0 += kGemvThreads) {
        const int i = i0 + lane;
        solo_stage_chunk(i, i < chunks ? __ldcg(xp + i) : zero4, mult, xs_g, stab_g, i < padded);
      }
    }
  }
  __syncthreads();
  if (!worker || int(blockIdx.x) >= items) return;

  // lanes that feed the B operand: g == 2t supplies block t (column 2t), g == 2t+1 block t+4 (column 2t+1)
  const bool feeds_first = g == 2 * t, feeds_second = g == 2 * t + 1, feeds_base = g == 0;
  const unsigned xs_first = xs_s + t * 32, xs_second = xs_s + 128 + t * 32, stab_lane = stab_s + t * 8;
  unsigned xb0[8], xb1[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) xb0[i] = xb1[i] = 0u;
  uint2 sb = make_uint2(0u, 0u);

  // finalising threads: tid < 16 own row tile*16 + tid (SWIGLU: tid < 8 own the pair (tid, tid + 8))
  float row_scale = 0.f, row_bias = 0.f, up_scale = 0.f, up_bias = 0.f;
  bool row_live = false;
  auto load_row_constants = [&](int item) {
    const int row = (item / S) * 16 + tid;
    row_live = tid < (SWIGLU ? 8 : 16) && row < p.M;
    row_scale = row_live ? p.scales[row] : 0.f;
    row_bias = row_live && p.bias && (item % S) == 0 ? __bfloat162float(p.bias[row]) : 0.f;
    if (SWIGLU) {
      up_scale = row_live ? p.scales[row + 8] : 0.f;
      up_bias = row_live && p.bias ? __bfloat162float(p.bias[row + 8]) : 0.f;
    }
  };

  const unsigned epoch = e.push.world ? __ldcg(e.push.epoch_word) + 1u : 0u;   // after the dependency wait: the previous
                                                                               // exchange's consumer advanced the word
  float acc0 = 0.f, acc1 = 0.f;                    // rows g and g+8: sum over this lane's blocks of delta * G
  float base[4] = {0.f, 0.f, 0.f, 0.f};            // base term, column 0 (lanes t == 0: base[0] row g, base[2] row g+8)
  int item = blockIdx.x, done = 0, buf = 0;
  unsigned unit = unsigned(item % S) * unsigned(KIs) + unsigned(warp);   // unit within the row: selects activations
  const int workers = WS * 32;
  load_row_constants(item);
  while (true) {
#pragma unroll
    for (int slot = 0; slot < LOOKAHEAD; ++slot) {
      const uint4 q = pend[slot][0], r = pend[slot][1];   // duos of rows g and g+8
      // ---- activations of this unit for the lanes that feed B; block sums for the base MMA
      const unsigned xoff = unit * 256;
      if (feeds_first) {
        const uint4 v0 = lds128(xs_first + xoff), v1 = lds128(xs_first + xoff + 16);
        xb0[0] = v0.x; xb0[1] = v0.y; xb0[2] = v0.z; xb0[3] = v0.w; xb0[4] = v1.x; xb0[5] = v1.y; xb0[6] = v1.z; xb0[7] = v1.w;
      }
      if (feeds_second) {
        const uint4 v0 = lds128(xs_second + xoff), v1 = lds128(xs_second + xoff + 16);
        xb1[0] = v0.x; xb1[1] = v0.y; xb1[2] = v0.z; xb1[3] = v0.w; xb1[4] = v1.x; xb1[5] = v1.y; xb1[6] = v1.z; xb1[7] = v1.w;
      }
      if (feeds_base) sb = lds64(stab_lane + unit * 32);
      const unsigned plane1 = hadd2_u(xb1[7], xb1[7]), plane2 = hadd2_u(plane1, plane1);
      // ---- endpoints: (e0 first | e0 second) as exact fp16 integers, (delta first | delta second)
      const unsigned q0 = __byte_perm(q.w, 0x64646464u, 0x4240), q1 = __byte_perm(q.w, 0x64646464u, 0x4341);
      const unsigned r0 = __byte_perm(r.w, 0x64646464u, 0x4240), r1 = __byte_perm(r.w, 0x64646464u, 0x4341);
      const unsigned e0q = hadd2_u(q0, 0xE480E480u), e0r = hadd2_u(r0, 0xE480E480u);   // - (1024 + 128)
      const unsigned dq = hsub2_u(q1, q0), dr = hsub2_u(r1, r0);
      mma_f16(base, e0q, e0r, e0q, e0r, sb.x, sb.y);
      // ---- G = sum g * x per block: ten MMAs in two independent accumulator chains
      const unsigned qs0 = q.x >> 10, qs1 = q.y >> 10, qs2 = q.z >> 10;
      const unsigned rs0 = r.x >> 10, rs1 = r.y >> 10, rs2 = r.z >> 10;
      float ca[4], cb[4];
      mma_f16_zero(ca, q.x & kField0, r.x & kField0, qs1 & kField0, rs1 & kField0, xb0[0], xb1[0]);
      mma_f16_zero(cb, q.x & kField3, r.x & kField3, qs1 & kField3, rs1 & kField3, xb0[1], xb1[1]);
      mma_f16(ca, q.x & kField6, r.x & kField6, q.z & kField0, r.z & kField0, xb0[2], xb1[2]);
      mma_f16(cb, qs0 & kField0, rs0 & kField0, q.z & kField3, r.z & kField3, xb0[3], xb1[3]);
      mma_f16(ca, qs0 & kField3, rs0 & kField3, q.z & kField6, r.z & kField6, xb0[4], xb1[4]);
      mma_f16(cb, q.y & kField0, r.y & kField0, qs2 & kField0, rs2 & kField0, xb0[5], xb1[5]);
      mma_f16(ca, q.y & kField3, r.y & kField3, qs2 & kField3, rs2 & kField3, xb0[6], xb1[6]);
      mma_f16(cb, q.y & kField6, r.y & kField6, q.x & kFieldSpare, r.x & kFieldSpare, xb0[7], xb1[7]);
      mma_f16(ca, 0u, 0u, q.y & kFieldSpare, r.y & kFieldSpare, 0u, plane1);
      mma_f16(cb, 0u, 0u, q.z & kFieldSpare, r.z & kFieldSpare, 0u, plane2);
      const float g0 = ca[0] + cb[0], g1 = ca[1] + cb[1], g2 = ca[2] + cb[2], g3 = ca[3] + cb[3];
      {
        const __half2 hq = *reinterpret_cast<const __half2 *>(&dq), hr = *reinterpret_cast<const __half2 *>(&dr);
        const float2 fq = __half22float2(hq), fr = __half22float2(hr);
        acc0 = fmaf(fq.x, g0, acc0);
        acc0 = fmaf(fq.y, g1, acc0);
        acc1 = fmaf(fr.x, g2, acc1);
        acc1 = fmaf(fr.y, g3, acc1);
      }
      prefetch(slot);
      unit += unsigned(WS);
      if (++done == per_item) {
        // ---- this warp's share of the item is done: rows over the lane quad, then over the warps
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
        if (t == 0) {
          float *mine = part_g + (buf * kGemvWarps + warp) * 16;
          mine[g] = acc0 + base[0];
          mine[g + 8] = acc1 + base[2];
        }
        acc0 = acc1 = 0.f;
        base[0] = base[1] = base[2] = base[3] = 0.f;
        asm volatile("bar.sync 1, %0;" ::"r"(workers) : "memory");
        if (e.push.world) {
          // tensor-parallel partial: packets of four consecutive rows into every rank's inbox (warp 0)
          if (tid < 32) {
            unsigned bits = 0;
            if (row_live) {
              const float *src = part_g + buf * kGemvWarps * 16 + tid;
              float sum = 0.f;
              for (int w = 0; w < WS; ++w) sum += src[w * 16];
              bits = __bfloat16_as_ushort(__float2bfloat16(fmaf(sum, row_scale * tokmul[0], row_bias)));
            }
            const unsigned b1 = __shfl_down_sync(0xffffffffu, bits, 1), b2 = __shfl_down_sync(0xffffffffu, bits, 2);
            const unsigned b3 = __shfl_down_sync(0xffffffffu, bits, 3);
            const int row = (item / S) * 16 + tid;
            if (tid < 16 && (tid & 3) == 0 && row < p.M) {
              const size_t at = (size_t(epoch & 1u) * e.push.world + e.push.rank) * e.push.packets + (row >> 2);
              for (int peer = 0; peer < e.push.world; ++peer)
                store_packet(e.push.inbox[peer] + at, bits | (b1 << 16), b2 | (b3 << 16), epoch);
            }
          }
        } else if (row_live) {
          const float *src = part_g + buf * kGemvWarps * 16 + tid;
          float sum = 0.f;
          for (int w = 0; w < WS; ++w) sum += src[w * 16];
          const float tm = tokmul[0];
          const int tile = item / S;
          if (SWIGLU) {
            float up_sum = 0.f;
            for (int w = 0; w < WS; ++w) up_sum += src[w * 16 + 8];
            const float gate = __bfloat162float(__float2bfloat16(fmaf(sum, row_scale * tm, row_bias)));
            const float up = __bfloat162float(__float2bfloat16(fmaf(up_sum, up_scale * tm, up_bias)));
            p.y[tile * 8 + tid] = __float2bfloat16(gate / (1.f + __expf(-gate)) * up);
          } else if (e.y_partial) {
            e.y_partial[size_t(item % S) * e.partial_stride + tile * 16 + tid] = fmaf(sum, row_scale * tm, row_bias);
          } else {
            p.y[tile * 16 + tid] = __float2bfloat16(fmaf(sum, row_scale * tm, row_bias));
          }
        }
        buf ^= 1;
        item += item_stride;
        if (item >= items) return;
        done = 0;
        unit = unsigned(item % S) * unsigned(KIs) + unsigned(warp);
        load_row_constants(item);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Reference-arithmetic GEMV (TX_DECODE_ALU_EXACT): w = bf16(pal*scale), fp32 FMA, one warp per
// row (texelator_cuda.cu:141-199 without the texture unit).  Correctness path, not tuned.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gemv_exact_kernel(const uint8_t *__restrict__ tiles,
                                                         const float *__restrict__ scales,
                                                         const __nv_bfloat16 *__restrict__ bias,
                                                         const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ y,
                                                         int M, int K, int bpr, int KI, int palette) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int row = blockIdx.x * 8 + warp, token = blockIdx.y;
  if (row >= M) return;
  x += size_t(token) * K;
  float scale = scales[row];
  float a0 = 0.f, a1 = 0.f;
  for (int kb = lane; kb < bpr; kb += 32) {
    unsigned long long block = tiled_block(tiles, row, kb, KI);
    int e0 = block_e0(block), e1 = block_e1(block);
#pragma unroll
    for (int p = 0; p < 16; p += 2) {
      float w0 = __bfloat162float(__float2bfloat16(__fmul_rn(palette_value_of(palette, e0, e1, block_selector(block, p)), scale)));
      float w1 = __bfloat162float(__float2bfloat16(__fmul_rn(palette_value_of(palette, e0, e1, block_selector(block, p + 1)), scale)));
      a0 = fmaf(w0, __bfloat162float(x[kb * 16 + p]), a0);
      a1 = fmaf(w1, __bfloat162float(x[kb * 16 + p + 1]), a1);
    }
  }
  float acc = a0 + a1;
  for (int d = 16; d; d >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, d);
  if (lane == 0) y[size_t(token) * M + row] = __float2bfloat16(acc + (bias ? __bfloat162float(bias[row]) : 0.f));
}

int launch_gemv_exact(const Handle *h, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream) {
  for (int t0 = 0; t0 < tokens; t0 += 65535) {
    int n = std::min(tokens - t0, 65535);
    dim3 grid((h->M + 7) / 8, n);
    gemv_exact_kernel<<<grid, 256, 0, stream>>>(h->tiles, h->scales, h->bias,
                                                x + size_t(t0) * h->K, y + size_t(t0) * h->M, h->M, h->K,
                                                h->blocks_per_row, h->KI, h->palette);
    count_launch();
  }
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

// ------------------------------------------------------------------------------------------
// Texture GEMV (TX_DECODE_TEXTURE): signed-BC4 texture object, tex2Dgather, one warp per row.
// Own mapping: lane = block within a 32-block stride, four gathers per block.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gemv_texture_kernel(cudaTextureObject_t texture, const float *__restrict__ scales,
                                                           const __nv_bfloat16 *__restrict__ bias,
                                                           const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ y,
                                                           int M, int K, int bpr) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int row = blockIdx.x * 8 + warp, token = blockIdx.y;
  if (row >= M) return;
  x += size_t(token) * K;
  float scale = scales[row];
  float a0 = 0.f, a1 = 0.f;
  for (int kb = lane; kb < bpr; kb += 32) {
#pragma unroll
    for (int quad = 0; quad < 4; ++quad) {
      int qx = (quad & 1) * 2, qy = (quad >> 1) * 2;
      // gather returns the 2x2 footprint as (w: x0y0, z: x1y0, x: x0y1, y: x1y1)
      float4 v = tex2Dgather<float4>(texture, kb * 4 + qx + 1.f, row * 4 + qy + 1.f, 0);
      int k = kb * 16 + qy * 4 + qx;
      a0 = fmaf(__bfloat162float(__float2bfloat16(__fmul_rn(v.w, scale))), __bfloat162float(x[k]), a0);
      a1 = fmaf(__bfloat162float(__float2bfloat16(__fmul_rn(v.z, scale))), __bfloat162float(x[k + 1]), a1);
      a0 = fmaf(__bfloat162float(__float2bfloat16(__fmul_rn(v.x, scale))), __bfloat162float(x[k + 4]), a0);
      a1 = fmaf(__bfloat162float(__float2bfloat16(__fmul_rn(v.y, scale))), __bfloat162float(x[k + 5]), a1);
    }
  }
  float acc = a0 + a1;
  for (int d = 16; d; d >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, d);
  if (lane == 0) y[size_t(token) * M + row] = __float2bfloat16(acc + (bias ? __bfloat162float(bias[row]) : 0.f));
}

int launch_gemv_texture(const Handle *h, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream) {
  if (!h->texture) return fail(TX_ESTATE, "texture decode path selected but no texture object exists");
  for (int t0 = 0; t0 < tokens; t0 += 65535) {
    int n = std::min(tokens - t0, 65535);
    dim3 grid((h->M + 7) / 8, n);
    gemv_texture_kernel<<<grid, 256, 0, stream>>>(h->texture, h->scales, h->bias, x + size_t(t0) * h->K,
                                                  y + size_t(t0) * h->M, h->M, h->K, h->blocks_per_row);
    count_launch();
  }
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

// ------------------------------------------------------------------------------------------
// Host launcher of the MMA GEMV
// ------------------------------------------------------------------------------------------
using GemvKernel = void (*)(const GemvParams);

// Kernel variants: LOOKAHEAD x token tiles x activation source x "payload has low-mode blocks".
// Matrices without a single low-mode block (the normal case for dense weights) run a variant that
// carries no generic-decode code at all.
template <int NT, bool PRE, bool LOWMODE>
static GemvKernel pick_lookahead(int lookahead) {
  switch (lookahead) {
    case 1: return gemv_tile_kernel<1, NT, PRE, LOWMODE>;
    case 2: return gemv_tile_kernel<2, NT, PRE, LOWMODE>;
    case 3: return gemv_tile_kernel<3, NT, PRE, LOWMODE>;
    case 4: return gemv_tile_kernel<4, NT, PRE, LOWMODE>;
    case 6: return gemv_tile_kernel<6, NT, PRE, LOWMODE>;
    default: return gemv_tile_kernel<8, NT, PRE, LOWMODE>;
  }
}

template <bool LOWMODE>
static GemvKernel pick_tokens(int lookahead, int nt, bool pre) {
  if (!pre) return pick_lookahead<1, false, LOWMODE>(lookahead);
  switch (nt) {
    case 1: return pick_lookahead<1, true, LOWMODE>(lookahead);
    case 2: return pick_lookahead<2, true, LOWMODE>(lookahead);
    default: return pick_lookahead<4, true, LOWMODE>(lookahead);
  }
}

template <bool LOWMODE, int FUSE>
static GemvKernel pick_fused_lookahead(int lookahead) {
  switch (lookahead) {
    case 1: return gemv_tile_kernel<1, 1, false, LOWMODE, FUSE>;
    case 2: return gemv_tile_kernel<2, 1, false, LOWMODE, FUSE>;
    case 3: return gemv_tile_kernel<3, 1, false, LOWMODE, FUSE>;
    case 4: return gemv_tile_kernel<4, 1, false, LOWMODE, FUSE>;
    case 6: return gemv_tile_kernel<6, 1, false, LOWMODE, FUSE>;
    default: return gemv_tile_kernel<8, 1, false, LOWMODE, FUSE>;
  }
}

// fuse: kFuseNorm, kFuseSwiglu or both; fused variants exist for in-CTA staging (one token tile) only
static GemvKernel pick_kernel(int lookahead, int nt, bool pre, bool low_mode, int fuse = 0) {
  switch (fuse) {
    case 0: return low_mode ? pick_tokens<true>(lookahead, nt, pre) : pick_tokens<false>(lookahead, nt, pre);
    case kFuseNorm: return low_mode ? pick_fused_lookahead<true, kFuseNorm>(lookahead) : pick_fused_lookahead<false, kFuseNorm>(lookahead);
    case kFuseSwiglu: return low_mode ? pick_fused_lookahead<true, kFuseSwiglu>(lookahead) : pick_fused_lookahead<false, kFuseSwiglu>(lookahead);
    default:
      return low_mode ? pick_fused_lookahead<true, kFuseNorm | kFuseSwiglu>(lookahead)
                      : pick_fused_lookahead<false, kFuseNorm | kFuseSwiglu>(lookahead);
  }
}

// The lean variant decodes high-mode blocks of the software palette only; low-mode blocks and the
// texture-unit palette's uneven interpolation weights need the variant that carries the extra code.
static bool needs_generic_variant(const Handle *h) { return h->has_low_mode || h->palette == TX_PALETTE_HARDWARE; }

using SoloKernel = void (*)(const GemvParams, const SoloExtras);

template <bool SWIGLU>
static SoloKernel pick_solo(int lookahead) {
  switch (lookahead) {
    case 1: return gemv_solo_kernel<1, SWIGLU>;
    case 2: return gemv_solo_kernel<2, SWIGLU>;
    case 3: return gemv_solo_kernel<3, SWIGLU>;
    case 4: return gemv_solo_kernel<4, SWIGLU>;
    case 6: return gemv_solo_kernel<6, SWIGLU>;
    default: return gemv_solo_kernel<8, SWIGLU>;
  }
}

static size_t solo_smem_bytes(int KI) { return size_t(kSoloSmallBytes) + kSoloPartBytes + size_t(KI) * 32 + size_t(KI) * 256; }

static size_t gemv_smem_bytes(int KP, int tokens, int nt) {
  // small arrays, double-buffered partial tiles, activations
  return size_t(kSmallBytes) + size_t(2 * kGemvWarps * 128 * 4) * nt + size_t(tokens) * (size_t(KP) * 2 + kXsPad);
}

static int token_tiles(int tokens) { return tokens <= 8 ? 1 : (tokens <= 16 ? 2 : 4); }

constexpr int kMaxSplits = 16;
static size_t split_smem_bytes(int KI, int splits, int tokens) {
  return gemv_smem_bytes((KI + splits - 1) / splits * 128, tokens, token_tiles(tokens));
}

// K ranges for a pass that takes its activations from the pre-pass.  Every CTA keeps `tokens` rows of
// its range in shared memory, so the ranges decide how many tokens fit and how many CTAs share an SM;
// the price is splits * tokens * M fp32 sums written and read back.  Fewest ranges that (a) leave room
// for two CTAs per SM, or failing that fit at all, and (b) give every SM two CTAs' worth of work items
// while a range still holds eight units; 0 when `tokens` cannot be staged even with kMaxSplits ranges.
static int choose_splits(const Handle *h, int tokens, int sm_count, size_t partial_floats) {
  const int limit = std::min(kMaxSplits, h->KI);
  int pick = 0;
  for (int s = 1; s <= limit && !pick; ++s)
    if (split_smem_bytes(h->KI, s, tokens) <= kSmemBudget / 2) pick = s;
  for (int s = 1; s <= limit && !pick; ++s)
    if (split_smem_bytes(h->KI, s, tokens) <= kSmemBudget) pick = s;
  if (!pick) return 0;
  while (pick < limit && h->MT * pick < 2 * sm_count && h->KI / (pick + 1) >= 8) ++pick;
  while (pick > 1 && size_t(pick) * tokens * h->M > partial_floats) --pick;
  return split_smem_bytes(h->KI, pick, tokens) <= kSmemBudget ? pick : 0;
}

// Largest number of tokens one pass can take (shared-memory bound with the most K ranges), capped at 32.
static int tokens_per_pass(const Handle *h) {
  int best = 0;
  for (int tokens = 1; tokens <= 8 * kMaxTokenTiles; ++tokens)
    if (split_smem_bytes(h->KI, std::min(kMaxSplits, h->KI), tokens) <= kSmemBudget) best = tokens;
  if (best >= 8) best = best / 8 * 8;   // whole token tiles when possible
  return best;
}

// y[t, m] = round(sum over the K ranges + bias): the second step of a pass with more than one range
__global__ void __launch_bounds__(256) gemv_combine_kernel(const float *__restrict__ partial, int splits, const void *__restrict__ bias,
                                                           void *__restrict__ y, int T, int M, int half_io) {
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t total = size_t(T) * M;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    float sum = 0.f;
    for (int s = 0; s < splits; ++s) sum += __ldcg(partial + size_t(s) * total + i);
    const int row = int(i % M);
    if (half_io) {
      if (bias) sum += __half2float(static_cast<const __half *>(bias)[row]);
      static_cast<__half *>(y)[i] = __float2half_rn(sum);
    } else {
      if (bias) sum += __bfloat162float(static_cast<const __nv_bfloat16 *>(bias)[row]);
      static_cast<__nv_bfloat16 *>(y)[i] = __float2bfloat16(sum);
    }
  }
}

int launch_combine(const float *partial, int ranges, const void *bias, void *y, int tokens, int M, bool half_io, int sm_count,
                   cudaStream_t stream) {
  const int blocks = int(std::min<size_t>((size_t(tokens) * M + 255) / 256, size_t(sm_count) * 8));
  TX_CUDA(launch_pdl(gemv_combine_kernel, dim3(blocks), dim3(256), 0, stream, partial, ranges, bias, y, tokens, M, half_io ? 1 : 0));
  count_launch();
  return TX_OK;
}

struct GemvPlan {
  GemvKernel kernel;
  SoloKernel solo_kernel;
  int nt, grid;
  int splits;   // K ranges (pre-pass variants only)
  bool pre, solo;
  size_t smem;
};

static int plan_gemv(const Handle *h, int tokens, GemvPlan &plan, int fuse = 0, bool single_token_kernel = false, bool force_pre = false,
                     bool allow_splits = true) {
  Workspace *ws = workspace_for(h->device);
  if (!ws) return TX_ECUDA;
  int KP = h->KI * 128;
  plan.nt = token_tiles(tokens);
  // in-CTA activation conversion only while it stays a short prologue
  plan.pre = force_pre || !(tokens <= 2 && size_t(tokens) * h->K <= 36864);
  if (fuse && plan.pre) return fail(TX_EINVAL, "fused linear handles at most 2 tokens with tokens * K <= 36864");
  // The single-token kernel (no per-weight arithmetic) is taken on request only (tx_linear_single): it
  // pays off when its token arrives staged; staging a bf16 row costs it more than the general kernel.
  plan.solo = single_token_kernel;
  plan.splits = 1;
  if (plan.pre && !plan.solo && allow_splits) {
    plan.splits = choose_splits(h, tokens, ws->sm_count, ws->partial_floats);
    if (plan.splits < 1) return fail(TX_EINVAL, "decode GEMV does not fit in shared memory for this K");
  }
  if (plan.solo) {
    plan.pre = false;
    plan.kernel = nullptr;
    plan.solo_kernel = (fuse & kFuseSwiglu) ? pick_solo<true>(h->lookahead) : pick_solo<false>(h->lookahead);
    plan.smem = solo_smem_bytes(h->KI);
  } else {
    plan.kernel = pick_kernel(h->lookahead, plan.nt, plan.pre, needs_generic_variant(h), fuse);
    plan.smem = plan.pre ? split_smem_bytes(h->KI, plan.splits, tokens) : gemv_smem_bytes(KP, tokens, plan.nt);
  }
  // attribute + occupancy queries are cached per (device, kernel, shared bytes)
  static std::mutex guard;
  static std::map<std::tuple<int, const void *, size_t>, int> cache;
  int per_sm = 0;
  {
    std::lock_guard<std::mutex> lock(guard);
    const void *entry = plan.solo ? reinterpret_cast<const void *>(plan.solo_kernel) : reinterpret_cast<const void *>(plan.kernel);
    auto key = std::make_tuple(h->device, entry, plan.smem);
    auto hit = cache.find(key);
    if (hit == cache.end()) {
      TX_CUDA(cudaFuncSetAttribute(entry, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBudget + 1024)));
      TX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, entry, kGemvThreads, plan.smem));
      cache[key] = per_sm;
    } else {
      per_sm = hit->second;
    }
  }
  if (per_sm < 1) return fail(TX_EINVAL, "decode GEMV does not fit in shared memory for this K");
  // persistent CTAs: one resident wave, each walking row tiles with stride gridDim.x
  const int slots = ws->sm_count * std::min(per_sm, 3);
  plan.grid = std::max(1, std::min(h->MT, slots / plan.splits)) * plan.splits;   // a multiple of the K ranges
  return TX_OK;
}

// `half_io`: x, y and the handle's bias are fp16 (the reference's texelator_bc4_kernel,
// texelator_cuda.cu:94-139, which multiplies the un-rounded pal*scale in fp32 -- what this kernel computes
// for either type); the activations then always take the pre-pass, which for fp16 is a padded copy.
int launch_gemv(const Handle *h, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream, bool half_io) {
  Workspace *ws = workspace_for(h->device);
  if (!ws) return TX_ECUDA;
  int KP = h->KI * 128;
  int per_pass = tokens_per_pass(h);
  if (per_pass < 1) return fail(TX_EINVAL, "K is too large for the decode GEMV's shared-memory staging");
  for (int t0 = 0; t0 < tokens; t0 += per_pass) {
    int n = std::min(per_pass, tokens - t0);
    GemvPlan plan;
    int rc = plan_gemv(h, n, plan, 0, false, half_io);
    if (rc != TX_OK) return rc;
    GemvParams p{};
    p.tiles = reinterpret_cast<const uint4 *>(h->tiles);
    p.flags = h->unit_flags;
    p.scales = h->scales;
    p.bias = h->bias;
    p.x = x + size_t(t0) * h->K;
    p.y = y + size_t(t0) * h->M;
    p.M = h->M;
    p.K = h->K;
    p.KI = h->KI;
    p.MT = h->MT;
    p.T = n;
    p.KP = KP;
    p.palette = h->palette | (half_io ? kHalfIO : 0);
    if (plan.pre) {
      // scaled fp16 activations go through the per-device scratch (one pre-pass CTA per token)
      if (size_t(n) * KP > ws->xprep_halfs) return fail(TX_EINVAL, "tokens*K exceeds the activation scratch of the decode GEMV");
      if (half_io) gemv_xprep_kernel<true><<<n, kGemvThreads, 0, stream>>>(p.x, ws->xprep, ws->xmul, h->K, KP);
      else gemv_xprep_kernel<false><<<n, kGemvThreads, 0, stream>>>(p.x, ws->xprep, ws->xmul, h->K, KP);
      count_launch();
      p.xprep = ws->xprep;
      p.xmul = ws->xmul;
      p.splits = plan.splits;
      p.partial = ws->partial;
    }
    TX_CUDA(launch_pdl(plan.kernel, dim3(plan.grid), dim3(kGemvThreads), plan.smem, stream, p));
    count_launch();
    if (plan.pre && plan.splits > 1) {
      rc = launch_combine(ws->partial, plan.splits, h->bias, p.y, n, h->M, half_io, ws->sm_count, stream);
      if (rc != TX_OK) return rc;
    }
  }
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

// Decode linear with fused neighbours: optional residual add + RMSNorm in front (the activation
// staging every CTA does anyway), optional SwiGLU behind (rows packed as gate/up pairs).
int launch_gemv_fused(const Handle *h, const __nv_bfloat16 *x, const __nv_bfloat16 *delta, const __nv_bfloat16 *gamma, float eps,
                      __nv_bfloat16 *residual_out, bool swiglu, __nv_bfloat16 *y, int tokens, cudaStream_t stream) {
  const int fuse = (gamma ? kFuseNorm : 0) | (swiglu ? kFuseSwiglu : 0);
  if (!gamma && (delta || residual_out)) return fail(TX_EINVAL, "delta and residual_out need a norm weight");
  if (gamma && h->K > kXChunks * kGemvThreads * 8) return fail(TX_EINVAL, "fused RMSNorm handles K up to 18432");
  if (residual_out) {
    // CTA 0 stores the new residual while the other CTAs still read x and delta for their own copy of the row
    auto overlaps = [&](const void *other, size_t bytes) {
      const char *a = reinterpret_cast<const char *>(residual_out), *b = static_cast<const char *>(other);
      const size_t mine = size_t(tokens) * h->K * 2;
      return other && a < b + bytes && b < a + mine;
    };
    if (overlaps(x, size_t(tokens) * h->K * 2)) return fail(TX_EINVAL, "residual_out must not alias x");
    if (overlaps(delta, size_t(tokens) * h->K * 2) || overlaps(y, size_t(tokens) * (swiglu ? h->M / 2 : h->M) * 2))
      return fail(TX_EINVAL, "residual_out must not overlap delta or y");
  }
  if (swiglu && h->M % 16) return fail(TX_EINVAL, "SwiGLU pairs need M to be a multiple of 16");
  if (fuse == 0) return launch_gemv(h, x, y, tokens, stream);
  GemvPlan plan;
  int rc = plan_gemv(h, tokens, plan, fuse);
  if (rc != TX_OK) return rc;
  GemvParams p{};
  p.tiles = reinterpret_cast<const uint4 *>(h->tiles);
  p.flags = h->unit_flags;
  p.scales = h->scales;
  p.bias = h->bias;
  p.x = x;
  p.y = y;
  p.M = h->M;
  p.K = h->K;
  p.KI = h->KI;
  p.MT = h->MT;
  p.T = tokens;
  p.KP = h->KI * 128;
  p.palette = h->palette;
  p.delta = delta;
  p.gamma = gamma;
  p.residual_out = residual_out;
  p.eps = eps;
  TX_CUDA(launch_pdl(plan.kernel, dim3(plan.grid), dim3(kGemvThreads), plan.smem, stream, p));
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

bool gemv_single_eligible(const Handle *h) {
  return h->decode_path == TX_DECODE_ALU_MMA && !needs_generic_variant(h) && solo_smem_bytes(h->KI) <= kSmemBudget;
}

// Number of K ranges for a partial-sum launch.  Two ranges help when the row tiles do not fill the resident
// CTAs evenly (5120 rows = 320 tiles on 296 CTAs: the last 24 tiles run alone at a fraction of the
// bandwidth); more ranges cost more in per-item combines than they gain (measured on 5120x17408:
// 1 range 18.4 us, 2 ranges 16.7 us, 4 ranges 18.8 us).
int gemv_suggest_splits(const Handle *h) {
  Workspace *ws = workspace_for(h->device);
  if (!ws || !gemv_single_eligible(h) || h->KI % 2 || h->KI < 16) return 1;
  const int slots = ws->sm_count * 2;
  const double one = double((h->MT + slots - 1) / slots), two = double((2 * h->MT + slots - 1) / slots) / 2.0;
  return two < 0.85 * one ? 2 : 1;
}

// One token through the single-token kernel with its extras: the token may arrive in staged form
// (written by the kernel that produced it), the result may leave as `splits` fp32 partial vectors.
int launch_gemv_single(const Handle *h, const __nv_bfloat16 *x, const uint8_t *staged, bool swiglu, __nv_bfloat16 *y,
                       float *y_partial, int splits, size_t partial_stride, const PeerPush *push, cudaStream_t stream) {
  if (!gemv_single_eligible(h))
    return fail(TX_EUNSUPPORTED, "the single-token kernel needs the ALU decode path, the software palette and a payload without low-mode blocks");
  if ((x == nullptr) == (staged == nullptr)) return fail(TX_EINVAL, "pass the token either as bf16 or in staged form");
  if (int(y != nullptr) + int(y_partial != nullptr) + int(push != nullptr) != 1)
    return fail(TX_EINVAL, "pass either a bf16 output or a partial-sum output");
  if (push && (swiglu || h->M % 4 || push->packets != h->M / 4 || push->world < 1 || push->world > kMaxRanks || push->rank < 0 ||
               push->rank >= push->world || !push->epoch_word))
    return fail(TX_EINVAL, "peer push needs M a multiple of 4, hidden / 4 packets per sender and 1..8 ranks");
  if (swiglu && (y_partial || h->M % 16)) return fail(TX_EINVAL, "SwiGLU needs a bf16 output and M a multiple of 16");
  if (!y_partial) splits = 1;
  if (splits < 1 || h->KI % splits) return fail(TX_EINVAL, "splits must divide the number of 128-column units of a row");
  if (y_partial && partial_stride < size_t(h->M)) return fail(TX_EINVAL, "partial_stride is smaller than M");
  Workspace *ws = workspace_for(h->device);
  if (!ws) return TX_ECUDA;
  GemvPlan plan;
  int rc = plan_gemv(h, 1, plan, swiglu ? kFuseSwiglu : 0, true);
  if (rc != TX_OK) return rc;
  GemvParams p{};
  p.tiles = reinterpret_cast<const uint4 *>(h->tiles);
  p.scales = h->scales;
  p.bias = h->bias;
  p.x = x;
  p.y = y;
  p.M = h->M;
  p.K = h->K;
  p.KI = h->KI;
  p.MT = h->MT;
  p.T = 1;
  p.KP = h->KI * 128;
  p.palette = h->palette;
  SoloExtras e{};
  e.staged = staged;
  e.y_partial = y_partial;
  e.partial_stride = partial_stride;
  e.splits = splits;
  if (push) e.push = *push;
  const int grid = std::max(1, std::min(h->MT * splits, ws->sm_count * 2));
  TX_CUDA(launch_pdl(plan.solo_kernel, dim3(grid), dim3(kGemvThreads), plan.smem, stream, p, e));
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

// ------------------------------------------------------------------------------------------
// Multi-token decode without any allocation.
//
// Some hosts may not allocate device memory at the moment they need a linear: a serving loop that
// has handed all memory to its own pool, or a real-time thread that must not take the allocator lock.  For them the rescaled fp16
// activations of the multi-token decode pass live in a fixed array that is part of the library
// image instead of the per-device workspace that tx_pack_encoded allocates.  Every GPU that loads
// the library carries the array (about 0.5 MiB) until the process exits.
//
// Limits: tokens <= 32 and tokens * K (K rounded up to 128) <= kStaticActivationHalfs, and the
// token group must fit one shared-memory pass.  The pre-pass rewrites every element the main kernel
// reads (including the zero padding), so nothing depends on what an earlier call left behind; but
// all calls on a device share the one array, so two calls that overlap on the GPU race.
// ------------------------------------------------------------------------------------------
constexpr size_t kStaticActivationHalfs = size_t(8) * 32768;
static __device__ __align__(256) __half g_static_activations[kStaticActivationHalfs];
static __device__ __align__(256) float g_static_multipliers[64];

struct StaticScratch {
  __half *activations = nullptr;   // device addresses of the two arrays on one device
  float *multipliers = nullptr;
  int sm_count = 0;
  bool ready = false;
};

// The array names above are host-side stand-ins; the device addresses come from
// cudaGetSymbolAddress, once per device, with that device current.
static int static_scratch_for(int device, StaticScratch **out) {
  static StaticScratch table[64];
  static std::mutex guard;
  if (device < 0 || device >= 64) return fail(TX_EINVAL, "device index outside 0..63");
  std::lock_guard<std::mutex> lock(guard);
  StaticScratch &entry = table[device];
  if (!entry.ready) {
    TX_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&entry.activations), g_static_activations));
    TX_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&entry.multipliers), g_static_multipliers));
    TX_CUDA(cudaDeviceGetAttribute(&entry.sm_count, cudaDevAttrMultiProcessorCount, device));
    entry.ready = true;
  }
  *out = &entry;
  return TX_OK;
}

int launch_gemv_static_scratch(const Handle *h, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream) {
  const int KP = h->KI * 128;
  if (tokens < 1 || tokens > 8 * kMaxTokenTiles)
    return fail(TX_EINVAL, "tx_linear_static_scratch handles 1..32 tokens per call");
  if (size_t(tokens) * KP > kStaticActivationHalfs)
    return fail(TX_EINVAL, "tokens * K exceeds the built-in activation scratch (262144 fp16 values); use tx_linear");
  const int nt = token_tiles(tokens);
  const size_t smem = gemv_smem_bytes(KP, tokens, nt);
  if (smem > kSmemBudget)
    return fail(TX_EINVAL, "this many tokens of this K do not fit one shared-memory pass; use tx_linear");
  StaticScratch *scratch = nullptr;
  int rc = static_scratch_for(h->device, &scratch);
  if (rc != TX_OK) return rc;
  GemvKernel kernel = pick_kernel(h->lookahead, nt, true, needs_generic_variant(h));
  // attribute and occupancy are looked up once per (device, kernel variant, shared bytes): host-side table, no allocation on the device
  static std::mutex guard;
  static std::map<std::tuple<int, const void *, size_t>, int> cache;
  int per_sm = 0;
  {
    std::lock_guard<std::mutex> lock(guard);
    auto key = std::make_tuple(h->device, reinterpret_cast<const void *>(kernel), smem);
    auto hit = cache.find(key);
    if (hit == cache.end()) {
      TX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBudget + 1024)));
      TX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kGemvThreads, smem));
      cache[key] = per_sm;
    } else {
      per_sm = hit->second;
    }
  }
  if (per_sm < 1) return fail(TX_EINVAL, "decode GEMV does not fit in shared memory for this K");
  GemvParams p{};
  p.tiles = reinterpret_cast<const uint4 *>(h->tiles);
  p.flags = h->unit_flags;
  p.scales = h->scales;
  p.bias = h->bias;
  p.x = x;
  p.y = y;
  p.M = h->M;
  p.K = h->K;
  p.KI = h->KI;
  p.MT = h->MT;
  p.T = tokens;
  p.KP = KP;
  p.palette = h->palette;
  p.xprep = scratch->activations;
  p.xmul = scratch->multipliers;
  p.splits = 1;   // whole rows per CTA: no partial-sum scratch
  gemv_xprep_kernel<false><<<tokens, kGemvThreads, 0, stream>>>(x, scratch->activations, scratch->multipliers, h->K, KP);
  count_launch();
  const int grid = std::max(1, std::min(h->MT, scratch->sm_count * std::min(per_sm, 3)));
  kernel<<<grid, kGemvThreads, smem, stream>>>(p);
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

int gemv_kernel_info(int64_t out[9]) {
  cudaFuncAttributes attributes{};
  GemvKernel kernel = gemv_tile_kernel<2, 1, false, false>;
  TX_CUDA(cudaFuncGetAttributes(&attributes, kernel));
  TX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBudget + 1024)));
  int active = 0;
  size_t smem = gemv_smem_bytes(4096, 1, 1);
  TX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&active, kernel, kGemvThreads, smem));
  out[0] = attributes.numRegs;
  out[1] = int64_t(attributes.sharedSizeBytes);
  out[2] = int64_t(attributes.localSizeBytes);
  out[3] = attributes.maxThreadsPerBlock;
  out[4] = int64_t(smem);
  out[5] = 16;   // rows per unit
  out[6] = 8;    // tokens per mma tile
  out[7] = 128;  // columns per unit
  out[8] = active;
  return TX_OK;
}

}  // namespace tx
