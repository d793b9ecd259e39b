// Glue kernels of the batch-1 decode loop around the BC4 linears: residual + RMSNorm, RoPE + KV-cache
// append, single-query grouped-query attention over the cache, SwiGLU.  The reference leaves all of
// this to Hugging Face / PyTorch (texelator/cli.py:189-219); at batch 1 on a B200 those many small
// PyTorch kernels cost more than the weight stream, so the decoder harness replaces them with a few
// fused launches.  No reference counterpart; bf16 in and out, fp32 arithmetic.
#include "tx_common.cuh"

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
// One CTA per token row.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__nv_bfloat16 *__restrict__ h, const __nv_bfloat16 *__restrict__ delta,
                                                          const __nv_bfloat16 *__restrict__ weight, __nv_bfloat16 *__restrict__ y,
                                                          int hidden, float eps) {
  __shared__ float partial[8];
  const int row = blockIdx.x;
  __nv_bfloat16 *hr = h + size_t(row) * hidden;
  const __nv_bfloat16 *dr = delta ? delta + size_t(row) * hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x * 2; i < hidden; i += 512) {
    float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(hr + i));
    if (dr) {
      float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(dr + i));
      __nv_bfloat162 s = __floats2bfloat162_rn(v.x + d.x, v.y + d.y);
      *reinterpret_cast<__nv_bfloat162 *>(hr + i) = s;
      v = __bfloat1622float2(s);
    }
    ss += v.x * v.x + v.y * v.y;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) total += partial[w];
  const float inv = rsqrtf(total / float(hidden) + eps);
  for (int i = threadIdx.x * 2; i < hidden; i += 512) {
    float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(hr + i));
    float2 w = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(weight + i));
    *reinterpret_cast<__nv_bfloat162 *>(y + size_t(row) * hidden + i) = __floats2bfloat162_rn(v.x * inv * w.x, v.y * inv * w.y);
  }
}

// Rotate q and k of one token in place (rotate-half convention) and append k, v to the cache at the
// position read from device memory.  qkv = [q_rows | kv_rows | kv_rows]; grid = heads (q + 2 kv).
__global__ void __launch_bounds__(64) rope_append_kernel(__nv_bfloat16 *__restrict__ qkv, const float *__restrict__ cos_table,
                                                         const float *__restrict__ sin_table, const long long *__restrict__ position,
                                                         __nv_bfloat16 *__restrict__ k_cache, __nv_bfloat16 *__restrict__ v_cache,
                                                         int q_heads, int kv_heads, int head_dim, int max_len) {
  const int head = blockIdx.x, half = head_dim / 2;
  const long long pos = *position;
  __nv_bfloat16 *vec = qkv + size_t(head) * head_dim;
  const int i = threadIdx.x;
  if (head < q_heads + kv_heads) {
    float a = 0.f, b = 0.f;
    if (i < half) {
      const float c = cos_table[pos * half + i], s = sin_table[pos * half + i];
      const float x1 = __bfloat162float(vec[i]), x2 = __bfloat162float(vec[i + half]);
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
    dst[i] = vec[i];
    dst[i + half] = vec[i + half];
  }
}

// Single-query attention over cache positions [0, pos], split along the sequence: CTA (split, kv head)
// scores kKeys keys for the G query heads of its group, then accumulates p*V with one thread per
// head dimension.  Unnormalised partial outputs and (max, sum) go to `partial`.
constexpr int kKeys = 256;
constexpr int kMaxGroup = 8;
constexpr int kHeadDim = 128;

__global__ void __launch_bounds__(kHeadDim) attention_partial_kernel(const __nv_bfloat16 *__restrict__ qkv,
                                                                     const __nv_bfloat16 *__restrict__ k_cache,
                                                                     const __nv_bfloat16 *__restrict__ v_cache,
                                                                     const long long *__restrict__ position, float *__restrict__ partial,
                                                                     int q_heads, int kv_heads, int max_len, float scale) {
  __shared__ float q_s[kMaxGroup][kHeadDim];
  __shared__ float p_s[kMaxGroup][kKeys];
  __shared__ float red[kMaxGroup][4];
  const int split = blockIdx.x, kvh = blockIdx.y, splits = gridDim.x;
  const int group = q_heads / kv_heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long last = *position;                       // attends to keys 0..last
  const int key0 = split * kKeys;
  const int count = int(min((long long)kKeys, last + 1 - key0));   // may be <= 0
  for (int g = 0; g < group; ++g) q_s[g][tid] = __bfloat162float(qkv[size_t(kvh * group + g) * kHeadDim + tid]) * scale;
  __syncthreads();
  float local_max[kMaxGroup];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) local_max[g] = -INFINITY;
  for (int j = tid; j < kKeys; j += kHeadDim) {
    float dot[kMaxGroup];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) dot[g] = 0.f;
    if (j < count) {
      const uint4 *row = reinterpret_cast<const uint4 *>(k_cache + (size_t(kvh) * max_len + key0 + j) * kHeadDim);
#pragma unroll 4
      for (int c = 0; c < kHeadDim / 8; ++c) {
        uint4 raw = row[c];
        const __nv_bfloat162 *pairs = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 kv = __bfloat1622float2(pairs[e]);
#pragma unroll
          for (int g = 0; g < kMaxGroup; ++g)
            if (g < group) dot[g] += kv.x * q_s[g][c * 8 + 2 * e] + kv.y * q_s[g][c * 8 + 2 * e + 1];
        }
      }
    }
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g)
      if (g < group) {
        float s = j < count ? dot[g] : -INFINITY;
        p_s[g][j] = s;
        local_max[g] = fmaxf(local_max[g], s);
      }
  }
  for (int g = 0; g < group; ++g) {
    float m = warp_max(local_max[g]);
    if (lane == 0) red[g][warp] = m;
  }
  __syncthreads();
  float gmax[kMaxGroup], gsum[kMaxGroup];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    gmax[g] = g < group ? fmaxf(fmaxf(red[g][0], red[g][1]), fmaxf(red[g][2], red[g][3])) : 0.f;
    gsum[g] = 0.f;
  }
  __syncthreads();
  for (int j = tid; j < kKeys; j += kHeadDim)
    for (int g = 0; g < group; ++g) {
      float e = (j < count) ? __expf(p_s[g][j] - gmax[g]) : 0.f;
      p_s[g][j] = e;
      gsum[g] += e;
    }
  for (int g = 0; g < group; ++g) {
    float s = warp_sum(gsum[g]);
    if (lane == 0) red[g][warp] = s;
  }
  __syncthreads();
  float acc[kMaxGroup];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) acc[g] = 0.f;
  const __nv_bfloat16 *vbase = v_cache + (size_t(kvh) * max_len + key0) * kHeadDim + tid;
  for (int j = 0; j < count; ++j) {
    const float v = __bfloat162float(vbase[size_t(j) * kHeadDim]);
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g)
      if (g < group) acc[g] += p_s[g][j] * v;
  }
  for (int g = 0; g < group; ++g) {
    const int head = kvh * group + g;
    float *out = partial + (size_t(head) * splits + split) * (kHeadDim + 2);
    out[tid] = acc[g];
    if (tid == 0) {
      out[kHeadDim] = count > 0 ? gmax[g] : -INFINITY;
      out[kHeadDim + 1] = red[g][0] + red[g][1] + red[g][2] + red[g][3];
    }
  }
}

__global__ void __launch_bounds__(kHeadDim) attention_combine_kernel(const float *__restrict__ partial, __nv_bfloat16 *__restrict__ out,
                                                                     int splits) {
  const int head = blockIdx.x, tid = threadIdx.x;
  const float *base = partial + size_t(head) * splits * (kHeadDim + 2);
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, base[s * (kHeadDim + 2) + kHeadDim]);
  float num = 0.f, den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float *p = base + s * (kHeadDim + 2);
    const float pm = p[kHeadDim];
    if (pm == -INFINITY) continue;
    const float w = __expf(pm - m);
    num += w * p[tid];
    den += w * p[kHeadDim + 1];
  }
  out[size_t(head) * kHeadDim + tid] = __float2bfloat16(num / den);
}

// out[t, i] = silu(gu[t, i]) * gu[t, inter + i]
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16 *__restrict__ gu, __nv_bfloat16 *__restrict__ out,
                                                       int inter, int tokens) {
  const int pairs = inter / 2;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < size_t(tokens) * pairs; i += size_t(gridDim.x) * blockDim.x) {
    const int t = int(i / pairs), c = int(i % pairs) * 2;
    float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(gu + size_t(t) * 2 * inter + c));
    float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(gu + size_t(t) * 2 * inter + inter + c));
    // same rounding points as the PyTorch expression silu(g.float()) * u.float() -> bf16
    float a = g.x / (1.f + __expf(-g.x)) * u.x, b = g.y / (1.f + __expf(-g.y)) * u.y;
    *reinterpret_cast<__nv_bfloat162 *>(out + size_t(t) * inter + c) = __floats2bfloat162_rn(a, b);
  }
}

}  // namespace tx

using namespace tx;

extern "C" {

int tx_aux_add_rmsnorm(void *h, const void *delta, const void *weight, void *y, int tokens, int hidden, float eps, void *stream) {
  if (!h || !weight || !y || tokens < 1 || hidden < 2 || hidden % 2) return fail(TX_EINVAL, "tx_aux_add_rmsnorm: bad argument");
  add_rmsnorm_kernel<<<tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16 *>(h), static_cast<const __nv_bfloat16 *>(delta), static_cast<const __nv_bfloat16 *>(weight),
      static_cast<__nv_bfloat16 *>(y), hidden, eps);
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

int tx_aux_rope_append(void *qkv, const float *cos_table, const float *sin_table, const void *position, void *k_cache,
                       void *v_cache, int q_heads, int kv_heads, int head_dim, int max_len, void *stream) {
  if (!qkv || !cos_table || !sin_table || !position || !k_cache || !v_cache || head_dim > 128 || head_dim % 2)
    return fail(TX_EINVAL, "tx_aux_rope_append: bad argument");
  rope_append_kernel<<<q_heads + 2 * kv_heads, 64, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16 *>(qkv), cos_table, sin_table, static_cast<const long long *>(position),
      static_cast<__nv_bfloat16 *>(k_cache), static_cast<__nv_bfloat16 *>(v_cache), q_heads, kv_heads, head_dim, max_len);
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
  auto s = static_cast<cudaStream_t>(stream);
  attention_partial_kernel<<<dim3(splits, kv_heads), kHeadDim, 0, s>>>(
      static_cast<const __nv_bfloat16 *>(qkv), static_cast<const __nv_bfloat16 *>(k_cache),
      static_cast<const __nv_bfloat16 *>(v_cache), static_cast<const long long *>(position), scratch, q_heads, kv_heads, max_len, scale);
  attention_combine_kernel<<<q_heads, kHeadDim, 0, s>>>(scratch, static_cast<__nv_bfloat16 *>(out), splits);
  count_launch(2);
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

int tx_aux_silu_mul(const void *gate_up, void *out, int tokens, int intermediate, void *stream) {
  if (!gate_up || !out || tokens < 1 || intermediate < 2 || intermediate % 2) return fail(TX_EINVAL, "tx_aux_silu_mul: bad argument");
  size_t pairs = size_t(tokens) * intermediate / 2;
  int grid = int(std::min<size_t>((pairs + 255) / 256, 148 * 8));
  silu_mul_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16 *>(gate_up),
                                                                      static_cast<__nv_bfloat16 *>(out), intermediate, tokens);
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

}  // extern "C"
