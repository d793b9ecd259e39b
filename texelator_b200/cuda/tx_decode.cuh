// Register-level BC4 decode shared by the decode GEMV and the prefill GEMM producers.
#pragma once

#include "tx_common.cuh"

namespace tx {

constexpr int kLutBytes = 8192;   // 64 selector-pair entries x 32 lanes x 4 bytes, 8 KiB aligned

__device__ __forceinline__ unsigned lds32(unsigned addr) {
  unsigned v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_f16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                        unsigned b0, unsigned b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned hfma2_u(unsigned a, unsigned b, unsigned c) {
  unsigned d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// (a & mask) | c as one LOP3
__device__ __forceinline__ unsigned and_or(unsigned a, unsigned mask, unsigned c) {
  unsigned d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(c));
  return d;
}
__device__ __forceinline__ unsigned hsub2_u(unsigned a, unsigned b) {
  unsigned d;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Eight fp16x2 numerator pairs of one block (positions 2i, 2i+1 in pair i), fast high-mode path.
__device__ __forceinline__ void decode_block_fast(unsigned lo, unsigned hi, unsigned lut_lane, unsigned (&a)[8]) {
  unsigned u = lo ^ 0x8080u;                               // endpoints as biased bytes e+128
  unsigned e0m = __byte_perm(u, 0x64646464u, 0x4040);      // fp16x2 (1024+u0, 1024+u0)
  unsigned e1m = __byte_perm(u, 0x64646464u, 0x4141);
  unsigned delta = hsub2_u(e1m, e0m);                      // e1 - e0
  unsigned base = hfma2_u(e0m, 0x47004700u, 0xEFE0EFE0u);  // 7*(1024+u0) - 8064 = 7*e0
  unsigned f[8];
  f[0] = lo >> 9;                                          // selector bits start at bit 16 of the block
  f[1] = lo >> 15;
  f[2] = __funnelshift_r(lo, hi, 21);
  f[3] = hi << 5;
  f[4] = hi >> 1;
  f[5] = hi >> 7;
  f[6] = hi >> 13;
  f[7] = hi >> 19;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    unsigned g2 = lds32(and_or(f[i], 0x1F80u, lut_lane));
    a[i] = hfma2_u(g2, delta, base);
  }
}

// Generic path: any mode, per-weight fp32 arithmetic, value = 889 * palette rounded to fp16.
__device__ __forceinline__ void decode_block_slow(unsigned lo, unsigned hi, unsigned (&a)[8]) {
  unsigned long long block = (unsigned long long)lo | ((unsigned long long)hi << 32);
  int e0 = block_e0(block), e1 = block_e1(block);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float v[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      int s = block_selector(block, 2 * i + q);
      if (e0 > e1) {
        int g = s == 0 ? 0 : (s == 1 ? 7 : s - 1);
        v[q] = float((7 - g) * e0 + g * e1);
      } else if (s >= 6) {
        v[q] = s == 6 ? -889.0f : 889.0f;
      } else {
        int g = s == 0 ? 0 : (s == 1 ? 5 : s - 1);
        v[q] = float((5 - g) * e0 + g * e1) * 1.4f;       // 889/635
      }
    }
    __half2 h = __floats2half2_rn(v[0], v[1]);
    a[i] = *reinterpret_cast<unsigned *>(&h);
  }
}

__device__ __forceinline__ bool block_is_low(unsigned lo) {
  return int(int8_t(lo & 0xff)) <= int(int8_t((lo >> 8) & 0xff));
}

// Selector-pair table: entry idx holds fp16x2 (g(idx & 7), g(idx >> 3)) with g the interpolation
// index of the high palette mode (0,7,1..6), replicated for every lane so that bank == lane.
__device__ __forceinline__ void fill_pair_table(uint8_t *lut, int tid, int threads) {
  for (int i = tid; i < 64 * 32; i += threads) {
    int idx = i >> 5, s0 = idx & 7, s1 = idx >> 3;
    float g0 = s0 == 0 ? 0.f : (s0 == 1 ? 7.f : float(s0 - 1));
    float g1 = s1 == 0 ? 0.f : (s1 == 1 ? 7.f : float(s1 - 1));
    reinterpret_cast<__half2 *>(lut)[i] = __floats2half2_rn(g0, g1);
  }
}

}  // namespace tx
