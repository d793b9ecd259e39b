// Glue kernels of the batch-1 decode loop around the BC4 linears: residual + RMSNorm, RoPE + KV-cache
// append, single-query grouped-query attention over the cache, SwiGLU.  The reference leaves all of
// this to Hugging Face / PyTorch (texelator/cli.py:189-219); at batch 1 on a B200 those many small
// PyTorch kernels cost more than the weight stream, so the decoder harness replaces them with a few
// fused launches.  No reference counterpart; bf16 in and out, fp32 arithmetic.
#include <cooperative_groups.h>

#include <algorithm>

#include "tx_common.cuh"
#include "tx_decode.cuh"

namespace tx {

__device__ __forceinline__ float warp_sum(float v) {
  for (int d = 16; d; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
  for (int d = 16; d; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}

// h += delta (optional, rounded to bf16 like a PyTorch residual add); y = rmsnorm(h) * weight.
// One CTA per token row; every thread keeps its 8-element chunks in registers between the two passes.
constexpr int kNormThreads = 512;
constexpr int kNormChunks = 4;            // hidden <= 512 * 8 * 4 = 16384 stays in registers

__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_kernel(__nv_bfloat16 *__restrict__ h, const __nv_bfloat16 *__restrict__ delta,
                                                                   const __nv_bfloat16 *__restrict__ weight, __nv_bfloat16 *__restrict__ y,
                                                                   int hidden, float eps) {
  __shared__ float partial[kNormThreads / 32];
  grid_launch_dependents();
  const int row = blockIdx.x, chunks = hidden / 8;
  // the norm weight is immutable: fetch it while the launch in front is still running
  const uint4 *wr = reinterpret_cast<const uint4 *>(weight);
  uint4 gain[kNormChunks];
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int i = threadIdx.x + c * kNormThreads;
    if (i < chunks) gain[c] = wr[i];
  }
  grid_dependency_wait();
  uint4 *hr = reinterpret_cast<uint4 *>(h + size_t(row) * hidden);
  const uint4 *dr = delta ? reinterpret_cast<const uint4 *>(delta + size_t(row) * hidden) : nullptr;
  uint4 keep[kNormChunks];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int i = threadIdx.x + c * kNormThreads;
    if (i < chunks) {
      uint4 v = __ldcg(hr + i);   // inputs come from the previous kernel: read through L2
      __nv_bfloat162 *pv = reinterpret_cast<__nv_bfloat162 *>(&v);
      if (dr) {
        uint4 d = __ldcg(dr + i);
        const __nv_bfloat162 *pd = reinterpret_cast<const __nv_bfloat162 *>(&d);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 a = __bfloat1622float2(pv[e]), b = __bfloat1622float2(pd[e]);
          pv[e] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
        }
        hr[i] = v;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 a = __bfloat1622float2(pv[e]);
        ss += a.x * a.x + a.y * a.y;
      }
      keep[c] = v;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kNormThreads / 32; ++w) total += partial[w];
  const float inv = rsqrtf(total / float(hidden) + eps);
  uint4 *yr = reinterpret_cast<uint4 *>(y + size_t(row) * hidden);
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int i = threadIdx.x + c * kNormThreads;
    if (i < chunks) {
      uint4 v = keep[c], w = gain[c], o;
      const __nv_bfloat162 *pv = reinterpret_cast<const __nv_bfloat162 *>(&v), *pw = reinterpret_cast<const __nv_bfloat162 *>(&w);
      __nv_bfloat162 *po = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 a = __bfloat1622float2(pv[e]), g = __bfloat1622float2(pw[e]);
        po[e] = __floats2bfloat162_rn(a.x * inv * g.x, a.y * inv * g.y);
      }
      yr[i] = o;
    }
  }
}

// The same step for one token with the two extras of the single-token decode path:
//   * delta may arrive as `splits` fp32 partial vectors (the K ranges of a K-split linear,
//     gemv_solo_kernel): they are added in split order and rounded to bf16 like a linear's output;
//   * the normalised activations may also be written in the staged form the single-token decode kernel
//     consumes (tx_decode.cuh), so that the 296 CTAs of the next linear copy 11 KB instead of each
//     scanning, scaling and summing the row.
struct NormExtras {
  const float *partials;      // [splits][partial_stride] or null
  int splits;
  size_t partial_stride;
  uint8_t *staged;            // staged_bytes(KI) bytes or null
  int KI;                     // 128-column units of the consumer's rows (hidden rounded up)
};

__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_single_kernel(__nv_bfloat16 *__restrict__ h, const __nv_bfloat16 *__restrict__ delta,
                                                                          const __nv_bfloat16 *__restrict__ weight,
                                                                          __nv_bfloat16 *__restrict__ y, int hidden, float eps,
                                                                          const NormExtras extra) {
  __shared__ float partial[kNormThreads / 32];
  __shared__ unsigned peak[kNormThreads / 32];
  grid_launch_dependents();
  const int chunks = hidden / 8, lane = threadIdx.x & 31;
  // the norm weight is immutable: fetch it while the launch in front is still running
  const uint4 *wr = reinterpret_cast<const uint4 *>(weight);
  uint4 gain[kNormChunks];
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int i = threadIdx.x + c * kNormThreads;
    if (i < chunks) gain[c] = wr[i];
  }
  grid_dependency_wait();
  uint4 *hr = reinterpret_cast<uint4 *>(h);
  const uint4 *dr = delta ? reinterpret_cast<const uint4 *>(delta) : nullptr;
  uint4 keep[kNormChunks];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int i = threadIdx.x + c * kNormThreads;
    keep[c] = make_uint4(0, 0, 0, 0);
    if (i < chunks) {
      uint4 v = __ldcg(hr + i);
      __nv_bfloat162 *pv = reinterpret_cast<__nv_bfloat162 *>(&v);
      if (dr || extra.partials) {
        __nv_bfloat162 d2[4];
        if (extra.partials) {
          float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int sp = 0; sp < extra.splits; ++sp) {
            const float4 *src = reinterpret_cast<const float4 *>(extra.partials + size_t(sp) * extra.partial_stride) + 2 * i;
            const float4 lo = __ldcg(src), hi = __ldcg(src + 1);
            sum[0] += lo.x; sum[1] += lo.y; sum[2] += lo.z; sum[3] += lo.w;
            sum[4] += hi.x; sum[5] += hi.y; sum[6] += hi.z; sum[7] += hi.w;
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) d2[e] = __floats2bfloat162_rn(sum[2 * e], sum[2 * e + 1]);
        } else {
          const uint4 d = __ldcg(dr + i);
#pragma unroll
          for (int e = 0; e < 4; ++e) d2[e] = reinterpret_cast<const __nv_bfloat162 *>(&d)[e];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = __bfloat1622float2(pv[e]), b = __bfloat1622float2(d2[e]);
          pv[e] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
        }
        hr[i] = v;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = __bfloat1622float2(pv[e]);
        ss += a.x * a.x + a.y * a.y;
      }
      keep[c] = v;
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) partial[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kNormThreads / 32; ++w) total += partial[w];
  const float inv = rsqrtf(total / float(hidden) + eps);
  uint4 *yr = reinterpret_cast<uint4 *>(y);
  unsigned m = 0;
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int i = threadIdx.x + c * kNormThreads;
    if (i < chunks) {
      uint4 v = keep[c], w = gain[c], o;
      const __nv_bfloat162 *pv = reinterpret_cast<const __nv_bfloat162 *>(&v), *pw = reinterpret_cast<const __nv_bfloat162 *>(&w);
      __nv_bfloat162 *po = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = __bfloat1622float2(pv[e]), g = __bfloat1622float2(pw[e]);
        po[e] = __floats2bfloat162_rn(a.x * inv * g.x, a.y * inv * g.y);
      }
      if (yr) yr[i] = o;
      keep[c] = o;
      m = max(m, chunk_absmax(o));
    }
  }
  if (!extra.staged) return;
  // ---- staged form of the normalised row (the arithmetic of gemv_solo_kernel's own staging)
  m = __reduce_max_sync(0xffffffffu, m);
  if (lane == 0) peak[threadIdx.x >> 5] = m;
  __syncthreads();
  m = 0;
#pragma unroll
  for (int w = 0; w < kNormThreads / 32; ++w) m = max(m, peak[w]);
  float mult, inverse;
  token_scaling(m, mult, inverse);
  if (threadIdx.x == 0) *reinterpret_cast<float *>(extra.staged) = inverse * kSoloScale;
  uint8_t *stab = extra.staged + kStagedHeader, *xs = stab + size_t(extra.KI) * 32;
  const int padded = extra.KI * 16;
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int i = threadIdx.x + c * kNormThreads;
    if (i - lane < padded) solo_stage_chunk(i, keep[c], mult, xs, stab, i < padded);   // whole warps enter
  }
}

// ---- all-reduce fused into the residual add + RMSNorm (tensor parallelism, one token) -----------------
// The row-parallel linears (o, down) leave a partial sum on every rank.  Instead of a collective followed
// by the norm kernel, the norm kernel itself exchanges the partials over NVLink peer memory:
//   1. every rank stores its partial into slot [epoch & 1][rank] of every rank's inbox (plain peer stores),
//   2. fences at system scope and writes the epoch number into the matching flag word of every rank,
//   3. waits -- bounded -- until its own flag words of all ranks show this epoch,
//   4. sums the inbox rows in rank order (fp32, one bf16 rounding; every rank gets the same bits) and
//      carries on with h += delta, y = rmsnorm(h) * weight.
// The epoch lives in device memory and advances by one per call, so CUDA-graph replays keep working; two
// inbox slots suffice because a rank can only start epoch e+1 after every peer has contributed to e.
// No multicast objects, no TMA: peer loads and stores only.  A wait that runs out records code 32 in the
// status word and the kernel finishes with whatever the inbox holds (the host sees the status).
struct PeerTable {
  uint4 *inbox[kMaxRanks];        // [2][world][hidden/8] on each rank, addressed from this rank
  unsigned *flags[kMaxRanks];     // [2][world] on each rank
};

__global__ void __launch_bounds__(kNormThreads) allreduce_add_rmsnorm_kernel(__nv_bfloat16 *__restrict__ h,
                                                                             const __nv_bfloat16 *__restrict__ partial,
                                                                             const __nv_bfloat16 *__restrict__ weight,
                                                                             __nv_bfloat16 *__restrict__ y, int hidden, float eps,
                                                                             PeerTable peers, int rank, int world,
                                                                             unsigned *__restrict__ epoch_word, int *__restrict__ status) {
  __shared__ float partial_ss[kNormThreads / 32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int chunks = hidden / 8;
  const unsigned epoch = __ldcg(epoch_word) + 1;
  const unsigned slot = epoch & 1;
  // 1. my partial -> every rank's inbox
  const uint4 *src = reinterpret_cast<const uint4 *>(partial);
  for (int i = threadIdx.x; i < chunks; i += kNormThreads) {
    const uint4 v = __ldcg(src + i);
    for (int p = 0; p < world; ++p) peers.inbox[p][(size_t(slot) * world + rank) * chunks + i] = v;
  }
  __syncthreads();
  // 2. publish: the barrier orders the CTA's stores before thread 0's system-scope fence
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int p = 0; p < world; ++p)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[p] + slot * world + rank), "r"(epoch) : "memory");
  }
  // 3. bounded wait for every rank's contribution to this epoch
  if (threadIdx.x < world) {
    const unsigned *flag = peers.flags[rank] + slot * world + threadIdx.x;
    unsigned seen = 0, spin = 0;
    for (; spin < kPeerSpinLimit; ++spin) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
      if (seen == epoch) break;
    }
    if (seen != epoch && status) atomicCAS(status, 0, 32);
  }
  __syncthreads();
  // 4. delta = sum over ranks (rank order), h += delta, RMSNorm
  const uint4 *inbox = peers.inbox[rank] + size_t(slot) * world * chunks;
  uint4 *hr = reinterpret_cast<uint4 *>(h);
  uint4 keep[kNormChunks];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int i = threadIdx.x + c * kNormThreads;
    if (i < chunks) {
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < world; ++r) {
        const uint4 d = __ldcg(inbox + size_t(r) * chunks + i);     // written by a peer: read at L2
        const __nv_bfloat162 *pd = reinterpret_cast<const __nv_bfloat162 *>(&d);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(pd[e]);
          sum[2 * e] += f.x;
          sum[2 * e + 1] += f.y;
        }
      }
      uint4 v = __ldcg(hr + i);
      __nv_bfloat162 *pv = reinterpret_cast<__nv_bfloat162 *>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = __bfloat1622float2(pv[e]);
        const float2 b = __bfloat1622float2(__floats2bfloat162_rn(sum[2 * e], sum[2 * e + 1]));   // the all-reduced bf16 delta
        pv[e] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
      }
      hr[i] = v;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = __bfloat1622float2(pv[e]);
        ss += a.x * a.x + a.y * a.y;
      }
      keep[c] = v;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) partial_ss[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kNormThreads / 32; ++w) total += partial_ss[w];
  const float inv = rsqrtf(total / float(hidden) + eps);
  const uint4 *wr = reinterpret_cast<const uint4 *>(weight);
  uint4 *yr = reinterpret_cast<uint4 *>(y);
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int i = threadIdx.x + c * kNormThreads;
    if (i < chunks) {
      uint4 v = keep[c], w = wr[i], o;
      const __nv_bfloat162 *pv = reinterpret_cast<const __nv_bfloat162 *>(&v), *pw = reinterpret_cast<const __nv_bfloat162 *>(&w);
      __nv_bfloat162 *po = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = __bfloat1622float2(pv[e]), g = __bfloat1622float2(pw[e]);
        po[e] = __floats2bfloat162_rn(a.x * inv * g.x, a.y * inv * g.y);
      }
      yr[i] = o;
    }
  }
  if (threadIdx.x == 0) *epoch_word = epoch;
}

// ---- consumer of the packet exchange (tx_common.cuh): residual add + RMSNorm over a thread-block cluster ----
// One cluster of up to eight CTAs; CTA c owns a contiguous range of 8-column chunks, one chunk per thread.
// Every thread polls the two packets of its chunk from all `world` senders (all loads issued before any
// is checked), adds them in rank order, rounds to bf16, adds the residual; the sum of squares and the
// peak magnitude travel between the CTAs through distributed shared memory (two cluster barriers).
// With world == 0 the delta comes from memory (or is absent) and the kernel is a multi-SM add_rmsnorm.
constexpr int kReduceThreads = 256;
constexpr int kReduceCluster = 8;

struct ReduceParams {
  __nv_bfloat16 *h;
  const __nv_bfloat16 *delta;      // world == 0 only; may be null
  const __nv_bfloat16 *weight;
  __nv_bfloat16 *y;                // may be null when staged is given
  uint8_t *staged;                 // staged form for tx_linear_single, or null
  const uint4 *inbox;              // this rank's inbox
  unsigned *epoch_word;
  int *status;
  int hidden, KI, world, packets;
  float eps;
};

__global__ void __launch_bounds__(kReduceThreads) peer_reduce_rmsnorm_kernel(const ReduceParams p) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float ss_all[kReduceCluster];
  __shared__ unsigned peak_all[kReduceCluster];
  __shared__ float ss_warp[kReduceThreads / 32];
  __shared__ unsigned peak_warp[kReduceThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ctas = int(cluster.num_blocks()), cta = int(cluster.block_rank());
  grid_launch_dependents();
  const int chunks = p.hidden / 8;
  const int per = (((chunks + ctas - 1) / ctas) + 1) & ~1;            // even: the two chunks of a block stay in one warp
  const int i = cta * per + tid;
  const bool live = tid < per && i < chunks;
  // the norm weight is immutable: fetch it while the launch in front is still running
  const uint4 gain = live ? reinterpret_cast<const uint4 *>(p.weight)[i] : make_uint4(0, 0, 0, 0);
  grid_dependency_wait();
  const unsigned epoch = p.world ? __ldcg(p.epoch_word) + 1u : 0u;

  uint4 v = make_uint4(0, 0, 0, 0);
  float ss = 0.f;
  if (live) {
    v = __ldcg(reinterpret_cast<const uint4 *>(p.h) + i);
    __nv_bfloat162 *pv = reinterpret_cast<__nv_bfloat162 *>(&v);
    __nv_bfloat162 d2[4];
    bool have = false;
    if (p.world) {
      const uint4 *base = p.inbox + (size_t(epoch & 1u) * p.world) * p.packets + 2 * i;
      uint4 a[kMaxRanks], b[kMaxRanks];
      unsigned pending = (1u << p.world) - 1u;
      for (unsigned spin = 0; pending && spin < kPeerSpinLimit; ++spin) {
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (pending & (1u << r)) {
            a[r] = load_packet(base + size_t(r) * p.packets);
            b[r] = load_packet(base + size_t(r) * p.packets + 1);
          }
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if ((pending & (1u << r)) && a[r].y == epoch && a[r].w == epoch && b[r].y == epoch && b[r].w == epoch) pending &= ~(1u << r);
      }
      if (pending && p.status) atomicCAS(p.status, 0, 32);
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < p.world) {
          const unsigned w[4] = {a[r].x, a[r].z, b[r].x, b[r].z};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            sum[2 * e] += __uint_as_float(w[e] << 16);
            sum[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
          }
        }
#pragma unroll
      for (int e = 0; e < 4; ++e) d2[e] = __floats2bfloat162_rn(sum[2 * e], sum[2 * e + 1]);
      have = true;
    } else if (p.delta) {
      const uint4 d = __ldcg(reinterpret_cast<const uint4 *>(p.delta) + i);
#pragma unroll
      for (int e = 0; e < 4; ++e) d2[e] = reinterpret_cast<const __nv_bfloat162 *>(&d)[e];
      have = true;
    }
    if (have) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = __bfloat1622float2(pv[e]), d = __bfloat1622float2(d2[e]);
        pv[e] = __floats2bfloat162_rn(x.x + d.x, x.y + d.y);
      }
      reinterpret_cast<uint4 *>(p.h)[i] = v;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __bfloat1622float2(pv[e]);
      ss += x.x * x.x + x.y * x.y;
    }
  }
  // ---- sum of squares over the cluster
  ss = warp_sum(ss);
  if (lane == 0) ss_warp[warp] = ss;
  __syncthreads();
  if (tid == 0) {
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kReduceThreads / 32; ++w) total += ss_warp[w];
    for (int c = 0; c < ctas; ++c) cluster.map_shared_rank(ss_all, c)[cta] = total;
  }
  cluster.sync();
  float total = 0.f;
  for (int c = 0; c < ctas; ++c) total += ss_all[c];
  const float inv = rsqrtf(total / float(p.hidden) + p.eps);
  uint4 o = make_uint4(0, 0, 0, 0);
  unsigned m = 0;
  if (live) {
    const uint4 w = gain;
    const __nv_bfloat162 *pv = reinterpret_cast<const __nv_bfloat162 *>(&v), *pw = reinterpret_cast<const __nv_bfloat162 *>(&w);
    __nv_bfloat162 *po = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __bfloat1622float2(pv[e]), g = __bfloat1622float2(pw[e]);
      po[e] = __floats2bfloat162_rn(x.x * inv * g.x, x.y * inv * g.y);
    }
    if (p.y) reinterpret_cast<uint4 *>(p.y)[i] = o;
    m = chunk_absmax(o);
  }
  if (cta == 0 && tid == 0 && p.world) *p.epoch_word = epoch;     // every CTA read the word before the barrier above
  if (!p.staged) return;
  // ---- staged form: peak magnitude over the cluster, then the arithmetic of the linear's own staging
  m = __reduce_max_sync(0xffffffffu, m);
  if (lane == 0) peak_warp[warp] = m;
  __syncthreads();
  if (tid == 0) {
    unsigned top = 0;
#pragma unroll
    for (int w = 0; w < kReduceThreads / 32; ++w) top = max(top, peak_warp[w]);
    for (int c = 0; c < ctas; ++c) cluster.map_shared_rank(peak_all, c)[cta] = top;
  }
  cluster.sync();
  m = 0;
  for (int c = 0; c < ctas; ++c) m = max(m, peak_all[c]);
  float mult, inverse;
  token_scaling(m, mult, inverse);
  if (cta == 0 && tid == 0) *reinterpret_cast<float *>(p.staged) = inverse * kSoloScale;
  uint8_t *stab = p.staged + kStagedHeader, *xs = stab + size_t(p.KI) * 32;
  solo_stage_chunk(i, o, mult, xs, stab, live);     // hidden is a multiple of 128 here: no padding chunks
}

// Vocabulary-parallel output head: every rank scored its slice of the vocabulary; one 16-byte packet
// {score bits, epoch, token, epoch} per rank travels to all ranks and the best score wins (ties: lowest
// rank, like an arg-max over the gathered list).  One warp; bounded poll.
__global__ void __launch_bounds__(32) peer_best_token_kernel(const float *__restrict__ local_score, const long long *__restrict__ local_token,
                                                             long long token_offset, PeerPush peers, unsigned *__restrict__ epoch_word,
                                                             long long *__restrict__ next_token, int *__restrict__ status) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x;
  const unsigned epoch = __ldcg(epoch_word) + 1u;
  const size_t slot = size_t(epoch & 1u) * peers.world;
  if (lane < peers.world)
    store_packet(peers.inbox[lane] + slot + peers.rank, __float_as_uint(__ldcg(local_score)), unsigned(__ldcg(local_token) + token_offset), epoch);
  float score = -INFINITY;
  unsigned token = 0;
  if (lane < peers.world) {
    uint4 got = make_uint4(0, 0, 0, 0);
    unsigned spin = 0;
    for (; spin < kPeerSpinLimit; ++spin) {
      got = load_packet(peers.inbox[peers.rank] + slot + lane);
      if (got.y == epoch && got.w == epoch) break;
    }
    if (spin == kPeerSpinLimit && status) atomicCAS(status, 0, 32);
    score = __uint_as_float(got.x);
    token = got.z;
  }
  // arg-max with the lowest rank winning ties
  int best = lane;
#pragma unroll
  for (int d = 16; d; d >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, score, d);
    const int other_rank = __shfl_xor_sync(0xffffffffu, best, d);
    const unsigned other_token = __shfl_xor_sync(0xffffffffu, token, d);
    if (other > score || (other == score && other_rank < best)) {
      score = other;
      best = other_rank;
      token = other_token;
    }
  }
  if (lane == 0) {
    *next_token = (long long)token;
    *epoch_word = epoch;
  }
}

// Rotate q and k of one token in place (rotate-half convention) and append k, v to the cache at the
// position read from device memory.  qkv = [q_rows | kv_rows | kv_rows]; grid = heads (q + 2 kv).
__global__ void __launch_bounds__(64) rope_append_kernel(__nv_bfloat16 *__restrict__ qkv, const float *__restrict__ cos_table,
                                                         const float *__restrict__ sin_table, const long long *__restrict__ position,
                                                         __nv_bfloat16 *__restrict__ k_cache, __nv_bfloat16 *__restrict__ v_cache,
                                                         int q_heads, int kv_heads, int head_dim, int max_len) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int head = blockIdx.x, half = head_dim / 2;
  const long long pos = __ldcg(position);
  __nv_bfloat16 *vec = qkv + size_t(head) * head_dim;
  const int i = threadIdx.x;
  if (head < q_heads + kv_heads) {
    float a = 0.f, b = 0.f;
    if (i < half) {
      const float c = cos_table[pos * half + i], s = sin_table[pos * half + i];
      const float x1 = __bfloat162float(__ldcg(vec + i)), x2 = __bfloat162float(__ldcg(vec + i + half));
      a = x1 * c - x2 * s;
      b = x2 * c + x1 * s;
      vec[i] = __float2bfloat16(a);
      vec[i + half] = __float2bfloat16(b);
      if (head >= q_heads) {
        __nv_bfloat16 *dst = k_cache + (size_t(head - q_heads) * max_len + pos) * head_dim;
        dst[i] = __float2bfloat16(a);
        dst[i + half] = __float2bfloat16(b);
      }
    }
  } else if (i < half) {
    __nv_bfloat16 *dst = v_cache + (size_t(head - q_heads - kv_heads) * max_len + pos) * head_dim;
    dst[i] = __ldcg(vec + i);
    dst[i + half] = __ldcg(vec + i + half);
  }
}

// Single-query attention over cache positions [0, pos], split along the sequence: CTA (split, kv head)
// handles kKeys keys for the G query heads of its group.  Scores: one warp per key, lanes across the
// head dimension (coalesced 256-byte key rows, q in registers).  Values: one thread per head dimension
// and key parity.  Unnormalised partial outputs and (max, sum) go to `partial`.
constexpr int kKeys = 128;
constexpr int kMaxGroup = 8;
constexpr int kHeadDim = 128;
constexpr int kAttnThreads = 256;

__global__ void __launch_bounds__(kAttnThreads) attention_partial_kernel(const __nv_bfloat16 *__restrict__ qkv,
                                                                         const __nv_bfloat16 *__restrict__ k_cache,
                                                                         const __nv_bfloat16 *__restrict__ v_cache,
                                                                         const long long *__restrict__ position, float *__restrict__ partial,
                                                                         int q_heads, int kv_heads, int max_len, float scale) {
  __shared__ float p_s[kMaxGroup][kKeys];
  __shared__ float acc_s[kMaxGroup][kHeadDim];
  const int split = blockIdx.x, kvh = blockIdx.y, splits = gridDim.x;
  const int group = q_heads / kv_heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  grid_launch_dependents();
  grid_dependency_wait();
  const long long last = __ldcg(position);                       // attends to keys 0..last
  const int key0 = split * kKeys;
  const int count = int(max(0ll, min((long long)kKeys, last + 1 - key0)));
  // q: lane owns dimensions 4*lane .. 4*lane+3 of every query head of the group
  float q[kMaxGroup][4];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    if (g < group) {
      uint2 raw = __ldcg(reinterpret_cast<const uint2 *>(qkv + size_t(kvh * group + g) * kHeadDim + 4 * lane));
      float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&raw.x)), b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&raw.y));
      q[g][0] = a.x * scale; q[g][1] = a.y * scale; q[g][2] = b.x * scale; q[g][3] = b.y * scale;
    } else {
      q[g][0] = q[g][1] = q[g][2] = q[g][3] = 0.f;
    }
  }
  // all key rows of this warp are requested before any is used (16 independent 256-byte rows in flight)
  constexpr int kPerWarp = kKeys / (kAttnThreads / 32);
  uint2 key_raw[kPerWarp];
#pragma unroll
  for (int i = 0; i < kPerWarp; ++i) {
    const int j = warp + i * (kAttnThreads / 32);
    key_raw[i] = j < count ? __ldcg(reinterpret_cast<const uint2 *>(k_cache + (size_t(kvh) * max_len + key0 + j) * kHeadDim + 4 * lane))
                           : make_uint2(0, 0);
  }
#pragma unroll
  for (int i = 0; i < kPerWarp; ++i) {
    const int j = warp + i * (kAttnThreads / 32);
    float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&key_raw[i].x));
    float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&key_raw[i].y));
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g)
      if (g < group) {
        float s = warp_sum(a.x * q[g][0] + a.y * q[g][1] + b.x * q[g][2] + b.y * q[g][3]);
        if (lane == 0) p_s[g][j] = j < count ? s : -INFINITY;
      }
  }
  __syncthreads();
  // per head: max and exp-sum over the kKeys scores (warp g handles head g)
  float head_max = -INFINITY, head_sum = 0.f;
  if (warp < group) {
    float m = -INFINITY;
    for (int j = lane; j < kKeys; j += 32) m = fmaxf(m, p_s[warp][j]);
    m = warp_max(m);
    float sum = 0.f;
    for (int j = lane; j < kKeys; j += 32) {
      float e = (j < count) ? __expf(p_s[warp][j] - m) : 0.f;
      p_s[warp][j] = e;
      sum += e;
    }
    head_max = m;
    head_sum = warp_sum(sum);
  }
  __syncthreads();
  const int d = tid & (kHeadDim - 1), parity = tid >> 7;
  float acc[kMaxGroup];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) acc[g] = 0.f;
  const __nv_bfloat16 *vbase = v_cache + (size_t(kvh) * max_len + key0) * kHeadDim + d;
  constexpr int kBatch = 16;                      // value rows requested together
  for (int j0 = parity; j0 < count; j0 += 2 * kBatch) {
    float v[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int j = j0 + 2 * i;
      v[i] = j < count ? __bfloat162float(__ldcg(vbase + size_t(j) * kHeadDim)) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int j = min(j0 + 2 * i, kKeys - 1);
#pragma unroll
      for (int g = 0; g < kMaxGroup; ++g)
        if (g < group) acc[g] += p_s[g][j] * v[i];
    }
  }
  if (parity == 1)
    for (int g = 0; g < group; ++g) acc_s[g][d] = acc[g];
  __syncthreads();
  if (parity == 0)
    for (int g = 0; g < group; ++g) {
      float *out = partial + (size_t(kvh * group + g) * splits + split) * (kHeadDim + 2);
      out[d] = acc[g] + acc_s[g][d];
    }
  if (warp < group && lane == 0) {
    float *out = partial + (size_t(kvh * group + warp) * splits + split) * (kHeadDim + 2);
    out[kHeadDim] = count > 0 ? head_max : -INFINITY;
    out[kHeadDim + 1] = head_sum;
  }
}

__global__ void __launch_bounds__(kHeadDim) attention_combine_kernel(const float *__restrict__ partial, __nv_bfloat16 *__restrict__ out,
                                                                     int splits) {
  grid_launch_dependents();
  grid_dependency_wait();
  __shared__ float weight_s[128];
  const int head = blockIdx.x, tid = threadIdx.x;
  const float *base = partial + size_t(head) * splits * (kHeadDim + 2);
  // thread s fetches (max, sum) of split s; the block maximum and the per-split weights go to shared memory
  float pm = -INFINITY, pl = 0.f;
  if (tid < splits) {
    pm = __ldcg(base + tid * (kHeadDim + 2) + kHeadDim);
    pl = __ldcg(base + tid * (kHeadDim + 2) + kHeadDim + 1);
  }
  __shared__ float red_s[4];
  float m = warp_max(pm);
  if ((tid & 31) == 0) red_s[tid >> 5] = m;
  __syncthreads();
  m = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
  const float w = pm == -INFINITY ? 0.f : __expf(pm - m);
  weight_s[tid] = w;
  float den = warp_sum(w * pl);
  __syncthreads();
  if ((tid & 31) == 0) red_s[tid >> 5] = den;
  __syncthreads();
  den = red_s[0] + red_s[1] + red_s[2] + red_s[3];
  float num = 0.f;
#pragma unroll 8
  for (int s = 0; s < splits; ++s) num += weight_s[s] * __ldcg(base + s * (kHeadDim + 2) + tid);
  out[size_t(head) * kHeadDim + tid] = __float2bfloat16(num / den);
}

// One launch for the attention block of a decode step: RoPE of q and of the new key, append of the new
// key and value to the caches, single-query grouped-query attention over positions 0..pos, and the
// merge of the sequence splits.  CTA (split, kv head) owns kStepKeys cache positions:
//   prologue  rotated q of the GROUP query heads -> shared memory (rounded to bf16 like a stored q);
//             the CTA whose range holds `pos` rotates the new key and writes key and value rows to the
//             caches (visible to the whole CTA after the barrier);
//   loads     every key and value row of the CTA is requested before any arithmetic: keys eight lanes
//             per row (four rows per warp instruction), values one row per warp instruction;
//   scores    16 products per lane, three shuffles per (key, head); soft-max statistics per head;
//   values    p * v accumulated per warp, summed over the eight warps through shared memory;
//   merge     each CTA publishes its unnormalised output and (max, sum); the CTA that arrives last for
//             a kv head (atomic counter, no waiting) merges all splits of that head's query group.
// The arrival counters live in a file-scope array and are reset by the merging CTA, so launches on one
// device must be ordered on one stream, like every other call of this library.
constexpr int kStepKeys = 64;
constexpr int kStepThreads = 256;
constexpr int kStepRow = kHeadDim + 4;          // floats per (head, split) record: output, max, sum, pad
constexpr int kStepMaxSplits = 256;
constexpr int kStepMaxKvHeads = 128;
constexpr int kStepMaxSlots = 4096;             // (sequence, kv head) pairs of one launch
__device__ unsigned g_attention_arrivals[kStepMaxSlots];

__device__ __forceinline__ void unpack_bf16x8(const uint4 &raw, float (&out)[8]) {
  const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <int GROUP>
__global__ void __launch_bounds__(kStepThreads, 2) attention_step_kernel(const __nv_bfloat16 *__restrict__ qkv,
                                                                      const float *__restrict__ cos_table,
                                                                      const float *__restrict__ sin_table,
                                                                      const long long *__restrict__ position,
                                                                      __nv_bfloat16 *__restrict__ k_cache,
                                                                      __nv_bfloat16 *__restrict__ v_cache, float *__restrict__ partial,
                                                                      __nv_bfloat16 *__restrict__ out, int q_heads, int kv_heads,
                                                                      int max_len, int split_capacity, float scale, int merge_here) {
  __shared__ __align__(16) float q_s[GROUP][kHeadDim];
  __shared__ float p_s[GROUP][kStepKeys];
  __shared__ __align__(16) float red_s[kStepThreads / 32][GROUP][kHeadDim];   // per-warp partial sums
  __shared__ float stat_s[GROUP][2];
  __shared__ float weight_s[GROUP][kStepMaxSplits];   // merge weights of the splits
  __shared__ int last_s;
  constexpr int kHalf = kHeadDim / 2, kWarps = kStepThreads / 32;
  const int split = blockIdx.x, kvh = blockIdx.y;
  // batched step: blockIdx.z is the sequence; every array is [sequences][the one-sequence extent]
  const int arrival_slot = int(blockIdx.z) * kv_heads + kvh;
  qkv += size_t(blockIdx.z) * size_t(q_heads + 2 * kv_heads) * kHeadDim;
  position += blockIdx.z;
  k_cache += size_t(blockIdx.z) * kv_heads * max_len * kHeadDim;
  v_cache += size_t(blockIdx.z) * kv_heads * max_len * kHeadDim;
  partial += size_t(blockIdx.z) * q_heads * split_capacity * kStepRow;
  out += size_t(blockIdx.z) * q_heads * kHeadDim;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  grid_launch_dependents();
  // The position and the cache rows below it were written by earlier steps (no launch of this library writes
  // them, and a foreign kernel directly in front would have to finish first), so they are read before the wait
  // for the launch in front -- the qkv linear, whose tail these loads overlap.  Only qkv itself is new.
  const long long pos = __ldcg(position);                       // attends to keys 0..pos; key pos is new
  const int live = int(pos / kStepKeys) + 1;                    // splits that hold at least one key
  if (split >= live) return;
  const int key0 = split * kStepKeys;
  const int count = int(min((long long)kStepKeys, pos + 1 - key0));
  const size_t q_rows = size_t(q_heads) * kHeadDim, kv_rows = size_t(kv_heads) * kHeadDim;

  // ---- all old cache rows of this CTA in flight at once ----
  // keys: lane (r = lane >> 3, j = lane & 7) holds dimensions 8j..8j+7 and 64+8j..64+8j+7 of key
  // warp*8 + batch*4 + r; values: lane holds dimensions 4*lane..4*lane+3 of key warp*8 + i
  const int r = lane >> 3, j = lane & 7;
  uint4 key_raw[2][2];
  uint2 val_raw[8];
#pragma unroll
  for (int b = 0; b < 2; ++b) {
    const int key = warp * 8 + b * 4 + r;
    const uint4 *row = reinterpret_cast<const uint4 *>(k_cache + (size_t(kvh) * max_len + key0 + key) * kHeadDim);
    const bool old_row = key0 + key < pos;
    key_raw[b][0] = old_row ? __ldcg(row + j) : make_uint4(0, 0, 0, 0);
    key_raw[b][1] = old_row ? __ldcg(row + 8 + j) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int key = warp * 8 + i;
    val_raw[i] = key0 + key < pos ? __ldcg(reinterpret_cast<const uint2 *>(v_cache + (size_t(kvh) * max_len + key0 + key) * kHeadDim) + lane)
                                  : make_uint2(0, 0);
  }
  grid_dependency_wait();

  // ---- prologue: rotate-half RoPE of q (and of the new key by its owner) ----
  for (int idx = tid; idx < GROUP * kHalf; idx += kStepThreads) {
    const int g = idx / kHalf, i = idx % kHalf;
    const float c = cos_table[pos * kHalf + i], sn = sin_table[pos * kHalf + i];
    const __nv_bfloat16 *vec = qkv + size_t(kvh * GROUP + g) * kHeadDim;
    const float x1 = __bfloat162float(__ldcg(vec + i)), x2 = __bfloat162float(__ldcg(vec + i + kHalf));
    q_s[g][i] = __bfloat162float(__float2bfloat16(x1 * c - x2 * sn)) * scale;
    q_s[g][i + kHalf] = __bfloat162float(__float2bfloat16(x2 * c + x1 * sn)) * scale;
  }
  if (split == live - 1) {
    if (tid < kHalf) {
      const int i = tid;
      const float c = cos_table[pos * kHalf + i], sn = sin_table[pos * kHalf + i];
      const __nv_bfloat16 *vec = qkv + q_rows + size_t(kvh) * kHeadDim;
      const float x1 = __bfloat162float(__ldcg(vec + i)), x2 = __bfloat162float(__ldcg(vec + i + kHalf));
      __nv_bfloat16 *dst = k_cache + (size_t(kvh) * max_len + pos) * kHeadDim;
      dst[i] = __float2bfloat16(x1 * c - x2 * sn);
      dst[i + kHalf] = __float2bfloat16(x2 * c + x1 * sn);
    } else if (tid < 2 * kHalf) {
      const int i = tid - kHalf;
      const __nv_bfloat162 *vec = reinterpret_cast<const __nv_bfloat162 *>(qkv + q_rows + kv_rows + size_t(kvh) * kHeadDim);
      reinterpret_cast<__nv_bfloat162 *>(v_cache + (size_t(kvh) * max_len + pos) * kHeadDim)[i] = __ldcg(vec + i);
    }
  }
  __syncthreads();

  // ---- the new row (written above by this CTA when it owns the last split) ----
#pragma unroll
  for (int b = 0; b < 2; ++b) {
    const int key = warp * 8 + b * 4 + r;
    if (key0 + key == pos) {
      const uint4 *row = reinterpret_cast<const uint4 *>(k_cache + (size_t(kvh) * max_len + pos) * kHeadDim);
      key_raw[b][0] = __ldcg(row + j);
      key_raw[b][1] = __ldcg(row + 8 + j);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (key0 + warp * 8 + i == pos)
      val_raw[i] = __ldcg(reinterpret_cast<const uint2 *>(v_cache + (size_t(kvh) * max_len + pos) * kHeadDim) + lane);

  // ---- scores (q of one head at a time, so that two CTAs fit the register file of an SM) ----
  {
    float k[2][16];
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      unpack_bf16x8(key_raw[b][0], *reinterpret_cast<float(*)[8]>(&k[b][0]));
      unpack_bf16x8(key_raw[b][1], *reinterpret_cast<float(*)[8]>(&k[b][8]));
    }
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      const float4 *src = reinterpret_cast<const float4 *>(&q_s[g][0]);
      const float4 qa = src[2 * j], qb = src[2 * j + 1], qc = src[16 + 2 * j], qd = src[16 + 2 * j + 1];
      const float q[16] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w, qc.x, qc.y, qc.z, qc.w, qd.x, qd.y, qd.z, qd.w};
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        const int key = warp * 8 + b * 4 + r;
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) dot = fmaf(k[b][e], q[e], dot);
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        if (j == 0) p_s[g][key] = key < count ? dot : -INFINITY;
      }
    }
  }
  __syncthreads();
  // ---- per head: max and exp-sum over the CTA's keys (warp g handles head g; GROUP <= 8 warps) ----
  if (warp < GROUP) {
    const float a = p_s[warp][lane], b = p_s[warp][lane + 32];
    const float m = warp_max(fmaxf(a, b));              // finite: key 0 of a live split exists
    const float ea = __expf(a - m), eb = __expf(b - m);
    p_s[warp][lane] = ea;
    p_s[warp][lane + 32] = eb;
    const float sum = warp_sum(ea + eb);
    if (lane == 0) {
      stat_s[warp][0] = m;
      stat_s[warp][1] = sum;
    }
  }
  __syncthreads();
  // ---- values ----
  {
    float acc[GROUP][4];
#pragma unroll
    for (int g = 0; g < GROUP; ++g) acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float v0 = __uint_as_float(val_raw[i].x << 16), v1 = __uint_as_float(val_raw[i].x & 0xffff0000u);
      const float v2 = __uint_as_float(val_raw[i].y << 16), v3 = __uint_as_float(val_raw[i].y & 0xffff0000u);
#pragma unroll
      for (int g = 0; g < GROUP; ++g) {
        const float pw = p_s[g][warp * 8 + i];
        acc[g][0] = fmaf(pw, v0, acc[g][0]);
        acc[g][1] = fmaf(pw, v1, acc[g][1]);
        acc[g][2] = fmaf(pw, v2, acc[g][2]);
        acc[g][3] = fmaf(pw, v3, acc[g][3]);
      }
    }
#pragma unroll
    for (int g = 0; g < GROUP; ++g)
      *reinterpret_cast<float4 *>(&red_s[warp][g][4 * lane]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
  }
  __syncthreads();
  for (int idx = tid; idx < GROUP * kHeadDim; idx += kStepThreads) {
    const int g = idx / kHeadDim, d = idx % kHeadDim;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) sum += red_s[w][g][d];
    partial[(size_t(kvh * GROUP + g) * split_capacity + split) * kStepRow + d] = sum;
  }
  if (tid < GROUP) {
    float *rec = partial + (size_t(kvh * GROUP + tid) * split_capacity + split) * kStepRow;
    rec[kHeadDim] = stat_s[tid][0];
    rec[kHeadDim + 1] = stat_s[tid][1];
  }
  if (!merge_here) return;      // attention_merge_kernel, the next launch on the stream, merges the splits
  // ---- publish; the CTA that arrives last for this kv head merges ----
  // The barrier makes every thread's stores visible to thread 0, whose device-scope fence orders them
  // before its arrival (the grid-synchronisation idiom); the last arriver fences again before reading.
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned before = atomicAdd(&g_attention_arrivals[arrival_slot], 1u);
    last_s = before == unsigned(live - 1);
    if (last_s) {
      g_attention_arrivals[arrival_slot] = 0;      // every CTA of this launch has arrived: ready for the next launch
      __threadfence();
    }
  }
  __syncthreads();
  if (!last_s) return;
  // merge: warps 0..GROUP-1 turn the (max, sum) records of their head into weights (each record is read
  // once, eight per lane at most); then all warps accumulate weighted outputs over interleaved splits
  // and the CTA adds the eight partial sums
  if (warp < GROUP) {
    const float *base = partial + size_t(kvh * GROUP + warp) * split_capacity * kStepRow;
    constexpr int kPerLane = kStepMaxSplits / 32;
    float2 rec[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int sp = lane + 32 * i;
      rec[i] = sp < live ? __ldcg(reinterpret_cast<const float2 *>(base + size_t(sp) * kStepRow + kHeadDim)) : make_float2(-INFINITY, 0.f);
    }
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) m = fmaxf(m, rec[i].x);
    m = warp_max(m);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int sp = lane + 32 * i;
      const float w = __expf(rec[i].x - m);        // 0 for the padding records
      if (sp < live) weight_s[warp][sp] = w;
      den = fmaf(w, rec[i].y, den);
    }
    den = warp_sum(den);
    if (lane == 0) stat_s[warp][0] = 1.f / den;
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < GROUP; ++g) {
    const float *base = partial + size_t(kvh * GROUP + g) * split_capacity * kStepRow;
    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int sp = warp; sp < live; sp += kWarps) {
      const float w = weight_s[g][sp];
      const float4 v = __ldcg(reinterpret_cast<const float4 *>(base + size_t(sp) * kStepRow) + lane);
      num.x = fmaf(w, v.x, num.x);
      num.y = fmaf(w, v.y, num.y);
      num.z = fmaf(w, v.z, num.z);
      num.w = fmaf(w, v.w, num.w);
    }
    *reinterpret_cast<float4 *>(&red_s[warp][g][4 * lane]) = num;
  }
  __syncthreads();
  for (int idx = tid; idx < GROUP * kHeadDim; idx += kStepThreads) {
    const int g = idx / kHeadDim, d = idx % kHeadDim;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) sum += red_s[w][g][d];
    out[size_t(kvh * GROUP + g) * kHeadDim + d] = __float2bfloat16(sum * stat_s[g][0]);
  }
}

// The same step for long caches: the grid is capped at two resident CTAs per SM and every CTA walks several
// 64-key chunks (chunk = split, split + gridDim.x, ...) with running soft-max statistics.
template <int GROUP>
__global__ void __launch_bounds__(kStepThreads, 2) attention_step_loop_kernel(const __nv_bfloat16 *__restrict__ qkv,
                                                                      const float *__restrict__ cos_table,
                                                                      const float *__restrict__ sin_table,
                                                                      const long long *__restrict__ position,
                                                                      __nv_bfloat16 *__restrict__ k_cache,
                                                                      __nv_bfloat16 *__restrict__ v_cache, float *__restrict__ partial,
                                                                      __nv_bfloat16 *__restrict__ out, int q_heads, int kv_heads,
                                                                      int max_len, int split_capacity, float scale, int merge_here) {
  __shared__ __align__(16) float q_s[GROUP][kHeadDim];
  __shared__ float p_s[GROUP][kStepKeys];
  __shared__ __align__(16) float red_s[kStepThreads / 32][GROUP][kHeadDim];   // per-warp partial sums
  __shared__ float stat_s[GROUP][2];
  __shared__ float rescale_s[GROUP];
  __shared__ float weight_s[GROUP][kStepMaxSplits];   // merge weights of the splits
  __shared__ int last_s;
  constexpr int kHalf = kHeadDim / 2, kWarps = kStepThreads / 32;
  const int split = blockIdx.x, kvh = blockIdx.y;
  // batched step: blockIdx.z is the sequence; every array is [sequences][the one-sequence extent]
  const int arrival_slot = int(blockIdx.z) * kv_heads + kvh;
  qkv += size_t(blockIdx.z) * size_t(q_heads + 2 * kv_heads) * kHeadDim;
  position += blockIdx.z;
  k_cache += size_t(blockIdx.z) * kv_heads * max_len * kHeadDim;
  v_cache += size_t(blockIdx.z) * kv_heads * max_len * kHeadDim;
  partial += size_t(blockIdx.z) * q_heads * split_capacity * kStepRow;
  out += size_t(blockIdx.z) * q_heads * kHeadDim;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  grid_launch_dependents();
  grid_dependency_wait();
  const long long pos = __ldcg(position);                       // attends to keys 0..pos; key pos is new
  const int chunks = int(pos / kStepKeys) + 1;                  // 64-key chunks that hold at least one key
  const int splits = gridDim.x;                                 // CTA `split` takes chunks split, split + splits, ...
  const int live = min(splits, chunks);                         // CTAs with work
  if (split >= live) return;
  const size_t q_rows = size_t(q_heads) * kHeadDim, kv_rows = size_t(kv_heads) * kHeadDim;

  // ---- prologue: rotate-half RoPE of q (and of the new key by its owner) ----
  for (int idx = tid; idx < GROUP * kHalf; idx += kStepThreads) {
    const int g = idx / kHalf, i = idx % kHalf;
    const float c = cos_table[pos * kHalf + i], sn = sin_table[pos * kHalf + i];
    const __nv_bfloat16 *vec = qkv + size_t(kvh * GROUP + g) * kHeadDim;
    const float x1 = __bfloat162float(__ldcg(vec + i)), x2 = __bfloat162float(__ldcg(vec + i + kHalf));
    q_s[g][i] = __bfloat162float(__float2bfloat16(x1 * c - x2 * sn)) * scale;
    q_s[g][i + kHalf] = __bfloat162float(__float2bfloat16(x2 * c + x1 * sn)) * scale;
  }
  if (split == (chunks - 1) % splits) {          // the CTA whose last chunk holds the new position
    if (tid < kHalf) {
      const int i = tid;
      const float c = cos_table[pos * kHalf + i], sn = sin_table[pos * kHalf + i];
      const __nv_bfloat16 *vec = qkv + q_rows + size_t(kvh) * kHeadDim;
      const float x1 = __bfloat162float(__ldcg(vec + i)), x2 = __bfloat162float(__ldcg(vec + i + kHalf));
      __nv_bfloat16 *dst = k_cache + (size_t(kvh) * max_len + pos) * kHeadDim;
      dst[i] = __float2bfloat16(x1 * c - x2 * sn);
      dst[i + kHalf] = __float2bfloat16(x2 * c + x1 * sn);
    } else if (tid < 2 * kHalf) {
      const int i = tid - kHalf;
      const __nv_bfloat162 *vec = reinterpret_cast<const __nv_bfloat162 *>(qkv + q_rows + kv_rows + size_t(kvh) * kHeadDim);
      reinterpret_cast<__nv_bfloat162 *>(v_cache + (size_t(kvh) * max_len + pos) * kHeadDim)[i] = __ldcg(vec + i);
    }
  }
  __syncthreads();

  // ---- all cache rows of a chunk in flight at once ----
  // keys: lane (r = lane >> 3, j = lane & 7) holds dimensions 8j..8j+7 and 64+8j..64+8j+7 of key
  // warp*8 + batch*4 + r; values: lane holds dimensions 4*lane..4*lane+3 of key warp*8 + i
  const int r = lane >> 3, j = lane & 7;
  uint4 key_raw[2][2];
  uint2 val_raw[8];
  auto request_keys = [&](int chunk) {
    const int key0 = chunk * kStepKeys;
    const int count = int(min((long long)kStepKeys, pos + 1 - key0));
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const int key = warp * 8 + b * 4 + r;
      const uint4 *row = reinterpret_cast<const uint4 *>(k_cache + (size_t(kvh) * max_len + key0 + key) * kHeadDim);
      key_raw[b][0] = key < count ? __ldcg(row + j) : make_uint4(0, 0, 0, 0);
      key_raw[b][1] = key < count ? __ldcg(row + 8 + j) : make_uint4(0, 0, 0, 0);
    }
  };
  auto request_values = [&](int chunk) {
    const int key0 = chunk * kStepKeys;
    const int count = int(min((long long)kStepKeys, pos + 1 - key0));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int key = warp * 8 + i;
      val_raw[i] = key < count ? __ldcg(reinterpret_cast<const uint2 *>(v_cache + (size_t(kvh) * max_len + key0 + key) * kHeadDim) + lane)
                               : make_uint2(0, 0);
    }
  };
  request_keys(split);
  request_values(split);

  // Long caches give a CTA several chunks: running soft-max statistics per head (kept by warp g for head
  // g), accumulators rescaled when the maximum moves, the next chunk's rows requested before this one is
  // processed.  With one chunk per CTA (up to about 2300 positions on 8 kv heads) the loop runs once.
  // The next chunk's keys are requested as soon as this chunk's scores are done with the key registers,
  // its values after the value registers are consumed (no second register set: two CTAs per SM).
  float acc[GROUP][4];
#pragma unroll
  for (int g = 0; g < GROUP; ++g) acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
  float run_max = -INFINITY, run_sum = 0.f;
  for (int chunk = split; chunk < chunks; chunk += splits) {
  const int count = int(min((long long)kStepKeys, pos + 1 - (long long)chunk * kStepKeys));
  const bool more = chunk + splits < chunks;                    // uniform
  // ---- scores (q of one head at a time, so that two CTAs fit the register file of an SM) ----
  {
    float k[2][16];
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      unpack_bf16x8(key_raw[b][0], *reinterpret_cast<float(*)[8]>(&k[b][0]));
      unpack_bf16x8(key_raw[b][1], *reinterpret_cast<float(*)[8]>(&k[b][8]));
    }
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      const float4 *src = reinterpret_cast<const float4 *>(&q_s[g][0]);
      const float4 qa = src[2 * j], qb = src[2 * j + 1], qc = src[16 + 2 * j], qd = src[16 + 2 * j + 1];
      const float q[16] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w, qc.x, qc.y, qc.z, qc.w, qd.x, qd.y, qd.z, qd.w};
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        const int key = warp * 8 + b * 4 + r;
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) dot = fmaf(k[b][e], q[e], dot);
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        if (j == 0) p_s[g][key] = key < count ? dot : -INFINITY;
      }
    }
  }
  if (more) request_keys(chunk + splits);
  __syncthreads();
  // ---- per head: max and exp-sum over the CTA's keys (warp g handles head g; GROUP <= 8 warps) ----
  if (warp < GROUP) {
    const float a = p_s[warp][lane], b = p_s[warp][lane + 32];
    const float m = fmaxf(run_max, warp_max(fmaxf(a, b)));     // finite: every chunk of the walk holds a key
    const float ea = __expf(a - m), eb = __expf(b - m);
    p_s[warp][lane] = ea;
    p_s[warp][lane + 32] = eb;
    const float factor = __expf(run_max - m);                   // 0 on the first chunk
    run_sum = fmaf(run_sum, factor, warp_sum(ea + eb));
    run_max = m;
    if (lane == 0) {
      stat_s[warp][0] = m;
      stat_s[warp][1] = run_sum;
      rescale_s[warp] = factor;
    }
  }
  __syncthreads();
  // ---- values ----
  {
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      const float factor = rescale_s[g];
      acc[g][0] *= factor; acc[g][1] *= factor; acc[g][2] *= factor; acc[g][3] *= factor;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float v0 = __uint_as_float(val_raw[i].x << 16), v1 = __uint_as_float(val_raw[i].x & 0xffff0000u);
      const float v2 = __uint_as_float(val_raw[i].y << 16), v3 = __uint_as_float(val_raw[i].y & 0xffff0000u);
#pragma unroll
      for (int g = 0; g < GROUP; ++g) {
        const float pw = p_s[g][warp * 8 + i];
        acc[g][0] = fmaf(pw, v0, acc[g][0]);
        acc[g][1] = fmaf(pw, v1, acc[g][1]);
        acc[g][2] = fmaf(pw, v2, acc[g][2]);
        acc[g][3] = fmaf(pw, v3, acc[g][3]);
      }
    }
  }
  if (more) {
    request_values(chunk + splits);
    __syncthreads();                                            // p_s and rescale_s are rewritten by the next chunk
  }
  }   // chunk loop
#pragma unroll
  for (int g = 0; g < GROUP; ++g)
    *reinterpret_cast<float4 *>(&red_s[warp][g][4 * lane]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
  __syncthreads();
  for (int idx = tid; idx < GROUP * kHeadDim; idx += kStepThreads) {
    const int g = idx / kHeadDim, d = idx % kHeadDim;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) sum += red_s[w][g][d];
    partial[(size_t(kvh * GROUP + g) * split_capacity + split) * kStepRow + d] = sum;
  }
  if (tid < GROUP) {
    float *rec = partial + (size_t(kvh * GROUP + tid) * split_capacity + split) * kStepRow;
    rec[kHeadDim] = stat_s[tid][0];
    rec[kHeadDim + 1] = stat_s[tid][1];
  }
  if (!merge_here) return;      // attention_merge_kernel, the next launch on the stream, merges the splits
  // ---- publish; the CTA that arrives last for this kv head merges ----
  // The barrier makes every thread's stores visible to thread 0, whose device-scope fence orders them
  // before its arrival (the grid-synchronisation idiom); the last arriver fences again before reading.
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned before = atomicAdd(&g_attention_arrivals[arrival_slot], 1u);
    last_s = before == unsigned(live - 1);
    if (last_s) {
      g_attention_arrivals[arrival_slot] = 0;      // every CTA of this launch has arrived: ready for the next launch
      __threadfence();
    }
  }
  __syncthreads();
  if (!last_s) return;
  // merge: warps 0..GROUP-1 turn the (max, sum) records of their head into weights (each record is read
  // once, eight per lane at most); then all warps accumulate weighted outputs over interleaved splits
  // and the CTA adds the eight partial sums
  if (warp < GROUP) {
    const float *base = partial + size_t(kvh * GROUP + warp) * split_capacity * kStepRow;
    constexpr int kPerLane = kStepMaxSplits / 32;
    float2 rec[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int sp = lane + 32 * i;
      rec[i] = sp < live ? __ldcg(reinterpret_cast<const float2 *>(base + size_t(sp) * kStepRow + kHeadDim)) : make_float2(-INFINITY, 0.f);
    }
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) m = fmaxf(m, rec[i].x);
    m = warp_max(m);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int sp = lane + 32 * i;
      const float w = __expf(rec[i].x - m);        // 0 for the padding records
      if (sp < live) weight_s[warp][sp] = w;
      den = fmaf(w, rec[i].y, den);
    }
    den = warp_sum(den);
    if (lane == 0) stat_s[warp][0] = 1.f / den;
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < GROUP; ++g) {
    const float *base = partial + size_t(kvh * GROUP + g) * split_capacity * kStepRow;
    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int sp = warp; sp < live; sp += kWarps) {
      const float w = weight_s[g][sp];
      const float4 v = __ldcg(reinterpret_cast<const float4 *>(base + size_t(sp) * kStepRow) + lane);
      num.x = fmaf(w, v.x, num.x);
      num.y = fmaf(w, v.y, num.y);
      num.z = fmaf(w, v.z, num.z);
      num.w = fmaf(w, v.w, num.w);
    }
    *reinterpret_cast<float4 *>(&red_s[warp][g][4 * lane]) = num;
  }
  __syncthreads();
  for (int idx = tid; idx < GROUP * kHeadDim; idx += kStepThreads) {
    const int g = idx / kHeadDim, d = idx % kHeadDim;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) sum += red_s[w][g][d];
    out[size_t(kvh * GROUP + g) * kHeadDim + d] = __float2bfloat16(sum * stat_s[g][0]);
  }
}

// out[t, i] = silu(gu[t, i]) * gu[t, inter + i]
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16 *__restrict__ gu, __nv_bfloat16 *__restrict__ out,
                                                       int inter, int tokens) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int pairs = inter / 2;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < size_t(tokens) * pairs; i += size_t(gridDim.x) * blockDim.x) {
    const int t = int(i / pairs), c = int(i % pairs) * 2;
    float2 g = __bfloat1622float2(__ldcg(reinterpret_cast<const __nv_bfloat162 *>(gu + size_t(t) * 2 * inter + c)));
    float2 u = __bfloat1622float2(__ldcg(reinterpret_cast<const __nv_bfloat162 *>(gu + size_t(t) * 2 * inter + inter + c)));
    // same rounding points as the PyTorch expression silu(g.float()) * u.float() -> bf16
    float a = g.x / (1.f + __expf(-g.x)) * u.x, b = g.y / (1.f + __expf(-g.y)) * u.y;
    *reinterpret_cast<__nv_bfloat162 *>(out + size_t(t) * inter + c) = __floats2bfloat162_rn(a, b);
  }
}

// the same for rows stored as (gate, up) groups of eight -- the row order of the SwiGLU-fused linear:
// out[t, 8j + e] = silu(gu[t, 16j + e]) * gu[t, 16j + 8 + e]
__global__ void __launch_bounds__(256) silu_mul_pairs_kernel(const __nv_bfloat16 *__restrict__ gu, __nv_bfloat16 *__restrict__ out,
                                                             int inter, int tokens) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int chunks = inter / 8;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < size_t(tokens) * chunks; i += size_t(gridDim.x) * blockDim.x) {
    const int t = int(i / chunks), j = int(i % chunks);
    const uint4 *src = reinterpret_cast<const uint4 *>(gu + size_t(t) * 2 * inter + size_t(j) * 16);
    const uint4 gate = __ldcg(src), up = __ldcg(src + 1);
    const __nv_bfloat162 *pg = reinterpret_cast<const __nv_bfloat162 *>(&gate), *pu = reinterpret_cast<const __nv_bfloat162 *>(&up);
    uint4 result;
    __nv_bfloat162 *pr = reinterpret_cast<__nv_bfloat162 *>(&result);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(pg[e]), u = __bfloat1622float2(pu[e]);
      pr[e] = __floats2bfloat162_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4 *>(out + size_t(t) * inter + size_t(j) * 8) = result;
  }
}

// The merge of the splits as a launch of its own: one CTA per query head and sequence, thread d owns output
// dimension d.  As a programmatic dependent of the step kernel it is resident and waiting when the last split
// finishes, which costs less than the fence -> atomic -> last-CTA chain inside the step kernel (the kernel
// boundary orders the partial records; no arrival counter is needed).
constexpr int kMergeParts = 4;      // thread groups of one CTA that share a head's splits
__global__ void __launch_bounds__(kHeadDim * kMergeParts) attention_merge_kernel(const float *__restrict__ partial,
                                                                                const long long *__restrict__ position,
                                                                                __nv_bfloat16 *__restrict__ out, int q_heads,
                                                                                int split_capacity, int live_cap) {
  __shared__ float weight_s[kStepMaxSplits];
  __shared__ float sum_s[kMergeParts][kHeadDim];
  __shared__ float inverse_s;
  const int head = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int d = tid % kHeadDim, part = tid / kHeadDim;      // output dimension, share of the splits
  grid_launch_dependents();
  const long long pos = __ldcg(position + seq);     // written by an earlier step: safe to read before the wait
  const int live = min(int(pos / kStepKeys) + 1, live_cap);
  const float *base = partial + (size_t(seq) * q_heads + head) * split_capacity * kStepRow;
  grid_dependency_wait();
  // warp 0 turns the (max, sum) records into weights while every group already has its first records in flight
  if (warp == 0) {
    constexpr int kPerLane = kStepMaxSplits / 32;
    float2 rec[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int sp = lane + 32 * i;
      rec[i] = sp < live ? __ldcg(reinterpret_cast<const float2 *>(base + size_t(sp) * kStepRow + kHeadDim)) : make_float2(-INFINITY, 0.f);
    }
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) m = fmaxf(m, rec[i].x);
    m = warp_max(m);
    float den = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int sp = lane + 32 * i;
      const float w = __expf(rec[i].x - m);        // 0 for the padding records
      if (sp < live) weight_s[sp] = w;
      den = fmaf(w, rec[i].y, den);
    }
    den = warp_sum(den);
    if (lane == 0) inverse_s = 1.f / den;
  }
  // this group's records: split part, part + kMergeParts, ... in rounds of eight loads; the first round is issued
  // before the barrier that publishes the weights
  constexpr int kRounds = kStepMaxSplits / kMergeParts / 8;
  float value[8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int sp = part + i * kMergeParts;
    value[i] = sp < live ? __ldcg(base + size_t(sp) * kStepRow + d) : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int sp = part + i * kMergeParts;
    if (sp < live) sum = fmaf(weight_s[sp], value[i], sum);
  }
  for (int round = 1; round < kRounds; ++round) {
    const int first = round * 8 * kMergeParts + part;
    if (first >= live) break;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int sp = first + i * kMergeParts;
      value[i] = sp < live ? __ldcg(base + size_t(sp) * kStepRow + d) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int sp = first + i * kMergeParts;
      if (sp < live) sum = fmaf(weight_s[sp], value[i], sum);
    }
  }
  sum_s[part][d] = sum;
  __syncthreads();
  if (part == 0) {
    float total = sum_s[0][d];
#pragma unroll
    for (int p = 1; p < kMergeParts; ++p) total += sum_s[p][d];
    out[(size_t(seq) * q_heads + head) * kHeadDim + d] = __float2bfloat16(total * inverse_s);
  }
}

// TEXELATOR_B200_ATTENTION_MERGE=inline keeps the merge inside the step kernel (one launch per step instead of
// two; 27B-class decode measured 193.0 tok/s that way against 198.7 with the separate merge)
static bool merge_inline() {
  static const bool value = [] {
    const char *text = std::getenv("TEXELATOR_B200_ATTENTION_MERGE");
    return text && std::string(text) == "inline";
  }();
  return value;
}

template <int GROUP, bool LOOP>
static cudaError_t launch_attention_step(int splits, int kv_heads, int sequences, cudaStream_t s, const __nv_bfloat16 *qkv, const float *cos_table,
                                         const float *sin_table, const long long *position, __nv_bfloat16 *k_cache,
                                         __nv_bfloat16 *v_cache, float *scratch, __nv_bfloat16 *out, int q_heads, int max_len, float scale) {
  const int merge_here = merge_inline() ? 1 : 0;
  cudaError_t status;
  if (LOOP)
    status = launch_pdl(attention_step_loop_kernel<GROUP>, dim3(splits, kv_heads, sequences), dim3(kStepThreads), 0, s, qkv, cos_table, sin_table,
                        position, k_cache, v_cache, scratch, out, q_heads, kv_heads, max_len, splits, scale, merge_here);
  else
    status = launch_pdl(attention_step_kernel<GROUP>, dim3(splits, kv_heads, sequences), dim3(kStepThreads), 0, s, qkv, cos_table, sin_table,
                        position, k_cache, v_cache, scratch, out, q_heads, kv_heads, max_len, splits, scale, merge_here);
  if (status != cudaSuccess || merge_here) return status;
  count_launch();
  return launch_pdl(attention_merge_kernel, dim3(q_heads, sequences), dim3(kHeadDim * kMergeParts), 0, s, static_cast<const float *>(scratch), position, out,
                    q_heads, splits, LOOP ? splits : kStepMaxSplits);
}

}  // namespace tx

using namespace tx;

extern "C" {

int tx_aux_add_rmsnorm(void *h, const void *delta, const void *weight, void *y, int tokens, int hidden, float eps, void *stream) {
  if (!h || !weight || !y || tokens < 1 || hidden < 8 || hidden % 8 || hidden > kNormThreads * 8 * kNormChunks)
    return fail(TX_EINVAL, "tx_aux_add_rmsnorm: hidden must be a multiple of 8 and at most 16384");
  TX_CUDA(launch_pdl(add_rmsnorm_kernel, dim3(tokens), dim3(kNormThreads), 0, static_cast<cudaStream_t>(stream),
                     static_cast<__nv_bfloat16 *>(h), static_cast<const __nv_bfloat16 *>(delta),
                     static_cast<const __nv_bfloat16 *>(weight), static_cast<__nv_bfloat16 *>(y), hidden, eps));
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

int tx_aux_add_rmsnorm_single(void *h, const void *delta, const float *partials, int splits, size_t partial_stride, const void *weight,
                              void *y, void *staged, int hidden, float eps, void *stream) {
  if (!h || !weight || (!y && !staged) || hidden < 8 || hidden % 8 || hidden > kNormThreads * 8 * kNormChunks)
    return fail(TX_EINVAL, "tx_aux_add_rmsnorm_single: hidden must be a multiple of 8 and at most 16384; y or staged must be given");
  if (delta && partials) return fail(TX_EINVAL, "tx_aux_add_rmsnorm_single: pass delta or partials, not both");
  if (partials && (splits < 1 || partial_stride < size_t(hidden) || (reinterpret_cast<uintptr_t>(partials) & 15) || partial_stride % 4))
    return fail(TX_EINVAL, "tx_aux_add_rmsnorm_single: partials need splits >= 1, a 16-byte aligned base and a stride >= hidden that is a multiple of 4");
  NormExtras extra{};
  extra.partials = partials;
  extra.splits = splits;
  extra.partial_stride = partial_stride;
  extra.staged = static_cast<uint8_t *>(staged);
  extra.KI = (hidden + 127) / 128;
  TX_CUDA(launch_pdl(add_rmsnorm_single_kernel, dim3(1), dim3(kNormThreads), 0, static_cast<cudaStream_t>(stream),
                     static_cast<__nv_bfloat16 *>(h), static_cast<const __nv_bfloat16 *>(delta),
                     static_cast<const __nv_bfloat16 *>(weight), static_cast<__nv_bfloat16 *>(y), hidden, eps, extra));
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

int tx_aux_allreduce_add_rmsnorm(void *h, const void *partial, const void *weight, void *y, int hidden, float eps,
                                 void *const *peer_inboxes, void *const *peer_flags, int rank, int world, void *epoch_word,
                                 void *stream) {
  if (!h || !partial || !weight || !y || !peer_inboxes || !peer_flags || !epoch_word)
    return fail(TX_EINVAL, "tx_aux_allreduce_add_rmsnorm: null argument");
  if (hidden < 8 || hidden % 8 || hidden > kNormThreads * 8 * kNormChunks)
    return fail(TX_EINVAL, "tx_aux_allreduce_add_rmsnorm: hidden must be a multiple of 8 and at most 16384");
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(TX_EINVAL, "tx_aux_allreduce_add_rmsnorm: world must be 1..8 and rank inside it");
  PeerTable table{};
  for (int p = 0; p < world; ++p) {
    if (!peer_inboxes[p] || !peer_flags[p]) return fail(TX_EINVAL, "tx_aux_allreduce_add_rmsnorm: null peer buffer");
    table.inbox[p] = static_cast<uint4 *>(peer_inboxes[p]);
    table.flags[p] = static_cast<unsigned *>(peer_flags[p]);
  }
  int device = 0;
  TX_CUDA(cudaGetDevice(&device));
  Workspace *ws = workspace_for(device);
  TX_CUDA(launch_pdl(allreduce_add_rmsnorm_kernel, dim3(1), dim3(kNormThreads), 0, static_cast<cudaStream_t>(stream),
                     static_cast<__nv_bfloat16 *>(h), static_cast<const __nv_bfloat16 *>(partial),
                     static_cast<const __nv_bfloat16 *>(weight), static_cast<__nv_bfloat16 *>(y), hidden, eps, table, rank, world,
                     static_cast<unsigned *>(epoch_word), ws ? ws->status : nullptr));
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

static int peer_table(void *const *peer_inboxes, int rank, int world, int packets, void *epoch_word, PeerPush &out) {
  if (!peer_inboxes || !epoch_word || world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(TX_EINVAL, "peer exchange: world must be 1..8, rank inside it, inboxes and epoch word non-null");
  out = PeerPush{};
  for (int p = 0; p < world; ++p) {
    if (!peer_inboxes[p] || (reinterpret_cast<uintptr_t>(peer_inboxes[p]) & 15)) return fail(TX_EINVAL, "peer exchange: null or unaligned inbox");
    out.inbox[p] = static_cast<uint4 *>(peer_inboxes[p]);
  }
  out.epoch_word = static_cast<const unsigned *>(epoch_word);
  out.rank = rank;
  out.world = world;
  out.packets = packets;
  return TX_OK;
}

int tx_aux_peer_reduce_rmsnorm(void *h, const void *delta, const void *weight, void *y, void *staged, int hidden, float eps,
                               const void *inbox, int world, void *epoch_word, void *stream) {
  if (!h || !weight || (!y && !staged) || hidden < 8 || hidden % 8 || hidden > kReduceThreads * 8 * kReduceCluster)
    return fail(TX_EINVAL, "tx_aux_peer_reduce_rmsnorm: hidden must be a multiple of 8 and at most 16384; y or staged must be given");
  if (staged && hidden % 128) return fail(TX_EINVAL, "tx_aux_peer_reduce_rmsnorm: the staged form needs hidden to be a multiple of 128");
  if (world < 0 || world > kMaxRanks || (world > 0 && (!inbox || !epoch_word || delta || hidden % 4)))
    return fail(TX_EINVAL, "tx_aux_peer_reduce_rmsnorm: with world >= 1 pass the inbox and the epoch word and no delta");
  int device = 0;
  TX_CUDA(cudaGetDevice(&device));
  Workspace *ws = workspace_for(device);
  if (!ws) return TX_ECUDA;
  ReduceParams p{};
  p.h = static_cast<__nv_bfloat16 *>(h);
  p.delta = static_cast<const __nv_bfloat16 *>(delta);
  p.weight = static_cast<const __nv_bfloat16 *>(weight);
  p.y = static_cast<__nv_bfloat16 *>(y);
  p.staged = static_cast<uint8_t *>(staged);
  p.inbox = static_cast<const uint4 *>(inbox);
  p.epoch_word = static_cast<unsigned *>(epoch_word);
  p.status = ws->status;
  p.hidden = hidden;
  p.KI = (hidden + 127) / 128;
  p.world = world;
  p.packets = hidden / 4;
  p.eps = eps;
  // as many CTAs as keep every thread of the cluster busy, at most eight
  int ctas = 1;
  while (ctas < kReduceCluster && hidden / 8 > ctas * kReduceThreads / 2) ctas *= 2;
  if ((hidden / 8 + ctas - 1) / ctas + 1 > kReduceThreads) ctas = kReduceCluster;
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(ctas);
  config.blockDim = dim3(kReduceThreads);
  config.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attributes[2]{};
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = ctas;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = pdl_enabled() ? 2 : 1;
  TX_CUDA(cudaLaunchKernelEx(&config, peer_reduce_rmsnorm_kernel, p));
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

int tx_aux_peer_best_token(const float *local_score, const void *local_token, long long token_offset, void *const *peer_inboxes, int rank,
                           int world, void *epoch_word, void *next_token, void *stream) {
  if (!local_score || !local_token || !next_token) return fail(TX_EINVAL, "tx_aux_peer_best_token: null argument");
  PeerPush peers;
  int rc = peer_table(peer_inboxes, rank, world, 1, epoch_word, peers);
  if (rc != TX_OK) return rc;
  int device = 0;
  TX_CUDA(cudaGetDevice(&device));
  Workspace *ws = workspace_for(device);
  TX_CUDA(launch_pdl(peer_best_token_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), local_score,
                     static_cast<const long long *>(local_token), token_offset, peers, static_cast<unsigned *>(epoch_word),
                     static_cast<long long *>(next_token), ws ? ws->status : nullptr));
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

int tx_linear_single_push(uint64_t handle, const void *x, const void *staged, void *const *peer_inboxes, int rank, int world,
                          void *epoch_word, void *stream) {
  Handle *h = reinterpret_cast<Handle *>(handle);
  if (!h || h->magic != 0x54584234) return fail(TX_EINVAL, "null Texelator handle");
  if (h->bias && h->bias_dtype != TX_DTYPE_BF16) return fail(TX_EINVAL, "input and bias dtypes must match");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(staged)) & 15)
    return fail(TX_EINVAL, "activation pointers must be 16-byte aligned");
  PeerPush peers;
  int rc = peer_table(peer_inboxes, rank, world, h->M / 4, epoch_word, peers);
  if (rc != TX_OK) return rc;
  int current = 0;
  TX_CUDA(cudaGetDevice(&current));
  if (current != h->device) TX_CUDA(cudaSetDevice(h->device));
  rc = launch_gemv_single(h, static_cast<const __nv_bfloat16 *>(x), static_cast<const uint8_t *>(staged), false, nullptr, nullptr, 1, 0,
                          &peers, static_cast<cudaStream_t>(stream));
  if (current != h->device) cudaSetDevice(current);
  return rc;
}

int tx_aux_rope_append(void *qkv, const float *cos_table, const float *sin_table, const void *position, void *k_cache,
                       void *v_cache, int q_heads, int kv_heads, int head_dim, int max_len, void *stream) {
  if (!qkv || !cos_table || !sin_table || !position || !k_cache || !v_cache || head_dim > 128 || head_dim % 2)
    return fail(TX_EINVAL, "tx_aux_rope_append: bad argument");
  TX_CUDA(launch_pdl(rope_append_kernel, dim3(q_heads + 2 * kv_heads), dim3(64), 0, static_cast<cudaStream_t>(stream),
                     static_cast<__nv_bfloat16 *>(qkv), cos_table, sin_table, static_cast<const long long *>(position),
                     static_cast<__nv_bfloat16 *>(k_cache), static_cast<__nv_bfloat16 *>(v_cache), q_heads, kv_heads,
                     head_dim, max_len));
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

int tx_aux_attention_decode(const void *qkv, const void *k_cache, const void *v_cache, const void *position, float *scratch,
                            void *out, int q_heads, int kv_heads, int head_dim, int max_len, float scale, void *stream) {
  if (!qkv || !k_cache || !v_cache || !position || !scratch || !out) return fail(TX_EINVAL, "tx_aux_attention_decode: null argument");
  if (head_dim != kHeadDim || kv_heads < 1 || q_heads % kv_heads || q_heads / kv_heads > kMaxGroup)
    return fail(TX_EUNSUPPORTED, "tx_aux_attention_decode supports head_dim 128 and up to 8 query heads per kv head");
  const int splits = (max_len + kKeys - 1) / kKeys;
  if (splits > 128) return fail(TX_EUNSUPPORTED, "tx_aux_attention_decode supports caches of up to 16384 positions");
  auto s = static_cast<cudaStream_t>(stream);
  TX_CUDA(launch_pdl(attention_partial_kernel, dim3(splits, kv_heads), dim3(kAttnThreads), 0, s,
                     static_cast<const __nv_bfloat16 *>(qkv), static_cast<const __nv_bfloat16 *>(k_cache),
                     static_cast<const __nv_bfloat16 *>(v_cache), static_cast<const long long *>(position), scratch, q_heads,
                     kv_heads, max_len, scale));
  TX_CUDA(launch_pdl(attention_combine_kernel, dim3(q_heads), dim3(kHeadDim), 0, s, static_cast<const float *>(scratch),
                     static_cast<__nv_bfloat16 *>(out), splits));
  count_launch(2);
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

static int attention_step_any(const void *qkv, const float *cos_table, const float *sin_table, const void *position, void *k_cache,
                              void *v_cache, float *scratch, void *out, int sequences, int q_heads, int kv_heads, int head_dim,
                              int max_len, float scale, void *stream) {
  if (!qkv || !cos_table || !sin_table || !position || !k_cache || !v_cache || !scratch || !out)
    return fail(TX_EINVAL, "tx_aux_attention_step: null argument");
  if (head_dim != kHeadDim || kv_heads < 1 || kv_heads > kStepMaxKvHeads || sequences < 1 || sequences * kv_heads > kStepMaxSlots ||
      q_heads % kv_heads || q_heads / kv_heads > kMaxGroup)
    return fail(TX_EUNSUPPORTED, "tx_aux_attention_step supports head_dim 128, up to 128 kv heads, up to 4096 (sequence, kv head) pairs and "
                                 "up to 8 query heads per kv head");
  if (max_len < 1) return fail(TX_EINVAL, "tx_aux_attention_step: max_len must be positive");
  // one CTA per 64-key chunk while that fits two resident CTAs per SM; longer caches give every CTA several chunks
  int device = 0;
  TX_CUDA(cudaGetDevice(&device));
  Workspace *ws = workspace_for(device);
  const int resident = std::max(1, (ws ? 2 * ws->sm_count : 256) / (kv_heads * sequences));
  const int chunks_max = (max_len + kStepKeys - 1) / kStepKeys;
  // up to two waves of one-chunk CTAs (most of them idle while the cache is short) run the leaner variant
  const bool loop = chunks_max > 2 * resident || chunks_max > kStepMaxSplits;
  const int splits = loop ? std::min(std::min(chunks_max, resident), kStepMaxSplits) : chunks_max;
  auto s = static_cast<cudaStream_t>(stream);
  auto q = static_cast<const __nv_bfloat16 *>(qkv);
  auto pos = static_cast<const long long *>(position);
  auto kc = static_cast<__nv_bfloat16 *>(k_cache), vc = static_cast<__nv_bfloat16 *>(v_cache);
  auto o = static_cast<__nv_bfloat16 *>(out);
  cudaError_t err = cudaSuccess;
  switch (q_heads / kv_heads) {
#define TX_STEP_CASE(G)                                                                                                          \
  case G:                                                                                                                        \
    err = loop ? launch_attention_step<G, true>(splits, kv_heads, sequences, s, q, cos_table, sin_table, pos, kc, vc, scratch, o, \
                                                q_heads, max_len, scale)                                                          \
               : launch_attention_step<G, false>(splits, kv_heads, sequences, s, q, cos_table, sin_table, pos, kc, vc, scratch,   \
                                                 o, q_heads, max_len, scale);                                                     \
    break;
    TX_STEP_CASE(1) TX_STEP_CASE(2) TX_STEP_CASE(3) TX_STEP_CASE(4) TX_STEP_CASE(5) TX_STEP_CASE(6) TX_STEP_CASE(7) TX_STEP_CASE(8)
#undef TX_STEP_CASE
    default: return fail(TX_EUNSUPPORTED, "tx_aux_attention_step: unsupported query group");
  }
  TX_CUDA(err);
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

int tx_aux_attention_step(const void *qkv, const float *cos_table, const float *sin_table, const void *position, void *k_cache,
                          void *v_cache, float *scratch, void *out, int q_heads, int kv_heads, int head_dim, int max_len,
                          float scale, void *stream) {
  return attention_step_any(qkv, cos_table, sin_table, position, k_cache, v_cache, scratch, out, 1, q_heads, kv_heads, head_dim, max_len,
                            scale, stream);
}

int tx_aux_attention_step_batch(const void *qkv, const float *cos_table, const float *sin_table, const void *positions, void *k_cache,
                                void *v_cache, float *scratch, void *out, int sequences, int q_heads, int kv_heads, int head_dim,
                                int max_len, float scale, void *stream) {
  return attention_step_any(qkv, cos_table, sin_table, positions, k_cache, v_cache, scratch, out, sequences, q_heads, kv_heads, head_dim,
                            max_len, scale, stream);
}

int tx_aux_silu_mul_pairs(const void *gate_up, void *out, int tokens, int intermediate, void *stream) {
  if (!gate_up || !out || tokens < 1 || intermediate < 8 || intermediate % 8) return fail(TX_EINVAL, "tx_aux_silu_mul_pairs: bad argument");
  size_t chunks = size_t(tokens) * intermediate / 8;
  int grid = int(std::min<size_t>((chunks + 255) / 256, 148 * 8));
  TX_CUDA(launch_pdl(silu_mul_pairs_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                     static_cast<const __nv_bfloat16 *>(gate_up), static_cast<__nv_bfloat16 *>(out), intermediate, tokens));
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

int tx_aux_silu_mul(const void *gate_up, void *out, int tokens, int intermediate, void *stream) {
  if (!gate_up || !out || tokens < 1 || intermediate < 2 || intermediate % 2) return fail(TX_EINVAL, "tx_aux_silu_mul: bad argument");
  size_t pairs = size_t(tokens) * intermediate / 2;
  int grid = int(std::min<size_t>((pairs + 255) / 256, 148 * 8));
  TX_CUDA(launch_pdl(silu_mul_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                     static_cast<const __nv_bfloat16 *>(gate_up), static_cast<__nv_bfloat16 *>(out), intermediate, tokens));
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

}  // extern "C"
