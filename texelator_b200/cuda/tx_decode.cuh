// Register-level BC4 decode shared by the decode GEMV and the prefill GEMM producers.
#pragma once

#include "tx_common.cuh"

namespace tx {

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

__device__ __forceinline__ unsigned hmul2_u(unsigned a, unsigned b) {
  unsigned d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// ---------------------------------------------------------------------------------------------
// Numerators.  Every decode kernel hands the tensor core the exact integers n = 7*e0 + g*(e1-e0)
// (|n| <= 889) scaled by 2^-16, as fp16: n * 2^-16 is a multiple of 2^-24 below 2^-6, hence exact in
// fp16 (subnormal below 2^-14; HFMA2 and the tensor cores take subnormal fp16 operands at full
// speed).  The epilogues multiply by kNumeratorScale * scale_m * (token scaling).
//
// Per block: base = 7*e0 * 2^-16 and three multipliers delta * 2^(8-p) for the field offsets p = 0, 3, 6
// (a field at offset p, masked in place, reads as g * 2^(p-24); the product with delta * 2^(8-p) is
// g*delta * 2^-16; delta * 256 <= 65024 still fits fp16).  Fields at offsets 10 and 13 come down to 0
// and 3 with one shift.  The pair kept in the spare bits is summed from its three bit planes with
// multipliers delta/2, delta, 2*delta (bit 9 reads as 2^-15).
// ---------------------------------------------------------------------------------------------
constexpr float kNumeratorScale = 65536.0f / 889.0f;   // numerators are n * 2^-16, palette value = n / 889

constexpr unsigned kField0 = 0x00070007u, kField3 = 0x00380038u, kField6 = 0x01C001C0u, kFieldSpare = 0x02000200u;

struct BlockConstants {
  unsigned base, d0, d3, d6, delta;   // fp16x2, both halves equal
};

// TEXTURE_WEIGHTS: the texture unit's interpolation weights are {0,36,72,114,144,186,222,258}/258 for
// g = 0..7, i.e. (36*g + 6*majority(bits of g))/258; the fast path then uses delta * 252/258 per g step
// plus delta * 42/258 per majority bit, both rounded to fp16 (relative error <= 2^-11; the 16-bit
// widening of the endpoints, 3e-5, is neglected -- tx_dequant and the exact kernels evaluate the
// texture palette exactly).
template <bool TEXTURE_WEIGHTS>
__device__ __forceinline__ BlockConstants block_constants(unsigned ends, unsigned sel_e0, unsigned sel_e1) {
  const unsigned e0m = __byte_perm(ends, 0x64646464u, sel_e0);   // fp16x2 (1024+u0, 1024+u0)
  const unsigned e1m = __byte_perm(ends, 0x64646464u, sel_e1);
  BlockConstants c;
  c.base = hfma2_u(e0m, 0x07000700u /* 7 * 2^-16 */, 0xAFE0AFE0u /* -8064 * 2^-16 */);   // 7*(u0-128) * 2^-16
  unsigned delta = hsub2_u(e1m, e0m);                              // e1 - e0, exact
  if (TEXTURE_WEIGHTS) delta = hmul2_u(delta, 0x3BD03BD0u);        // * 252/258 = 0.976744 -> fp16 0x3BD0
  c.delta = delta;
  c.d0 = hmul2_u(delta, 0x5C005C00u);                              // * 256
  c.d3 = hmul2_u(delta, 0x50005000u);                              // * 32
  c.d6 = hmul2_u(delta, 0x44004400u);                              // * 4
  return c;
}

// majority of the three bits of every field, left at the field's lowest bit (texture weights only)
__device__ __forceinline__ unsigned field_majority(unsigned w, unsigned low_bits) {
  unsigned m;
  const unsigned w1 = w >> 1, w2 = w >> 2;
  asm("lop3.b32 %0, %1, %2, %3, 0xE8;" : "=r"(m) : "r"(w), "r"(w1), "r"(w2));
  return m & low_bits;
}

template <bool TEXTURE_WEIGHTS>
__device__ __forceinline__ unsigned numerators(unsigned word, unsigned mask, unsigned multiplier, unsigned base, unsigned low_bits) {
  unsigned n = hfma2_u(word & mask, multiplier, base);
  if (TEXTURE_WEIGHTS)   // + majority * delta * 42/258; multiplier already carries 252/258: 42/252 = 1/6
    n = hfma2_u(field_majority(word, low_bits), hmul2_u(multiplier, 0x31553155u /* 1/6 */), n);
  return n;
}

// The eight fp16x2 numerator pairs (weights 2i, 2i+1 in pair i) of the first / second block of a duo.
// High palette mode only; blocks with e0 <= e1 are redone by decode_block_slow.
template <bool TEXTURE_WEIGHTS = false>
__device__ __forceinline__ void decode_duo_first(const uint4 duo, unsigned (&a)[8]) {
  const BlockConstants c = block_constants<TEXTURE_WEIGHTS>(duo.w, 0x4040, 0x4141);
  const unsigned s0 = duo.x >> 10;
  a[0] = numerators<TEXTURE_WEIGHTS>(duo.x, kField0, c.d0, c.base, 0x00010001u);
  a[1] = numerators<TEXTURE_WEIGHTS>(duo.x, kField3, c.d3, c.base, 0x00080008u);
  a[2] = numerators<TEXTURE_WEIGHTS>(duo.x, kField6, c.d6, c.base, 0x00400040u);
  a[3] = numerators<TEXTURE_WEIGHTS>(s0, kField0, c.d0, c.base, 0x00010001u);
  a[4] = numerators<TEXTURE_WEIGHTS>(s0, kField3, c.d3, c.base, 0x00080008u);
  a[5] = numerators<TEXTURE_WEIGHTS>(duo.y, kField0, c.d0, c.base, 0x00010001u);
  a[6] = numerators<TEXTURE_WEIGHTS>(duo.y, kField3, c.d3, c.base, 0x00080008u);
  a[7] = numerators<TEXTURE_WEIGHTS>(duo.y, kField6, c.d6, c.base, 0x00400040u);
}

template <bool TEXTURE_WEIGHTS = false>
__device__ __forceinline__ void decode_duo_second(const uint4 duo, unsigned (&a)[8]) {
  const BlockConstants c = block_constants<TEXTURE_WEIGHTS>(duo.w, 0x4242, 0x4343);
  const unsigned s1 = duo.y >> 10, s2 = duo.z >> 10;
  a[0] = numerators<TEXTURE_WEIGHTS>(s1, kField0, c.d0, c.base, 0x00010001u);
  a[1] = numerators<TEXTURE_WEIGHTS>(s1, kField3, c.d3, c.base, 0x00080008u);
  a[2] = numerators<TEXTURE_WEIGHTS>(duo.z, kField0, c.d0, c.base, 0x00010001u);
  a[3] = numerators<TEXTURE_WEIGHTS>(duo.z, kField3, c.d3, c.base, 0x00080008u);
  a[4] = numerators<TEXTURE_WEIGHTS>(duo.z, kField6, c.d6, c.base, 0x00400040u);
  a[5] = numerators<TEXTURE_WEIGHTS>(s2, kField0, c.d0, c.base, 0x00010001u);
  a[6] = numerators<TEXTURE_WEIGHTS>(s2, kField3, c.d3, c.base, 0x00080008u);
  // pair 7: bit k of both g values is the spare bit of word k (reads as 2^-15 per set bit)
  unsigned n = hfma2_u(duo.x & kFieldSpare, hmul2_u(c.delta, 0x38003800u /* 1/2 */), c.base);
  n = hfma2_u(duo.y & kFieldSpare, c.delta, n);
  n = hfma2_u(duo.z & kFieldSpare, hmul2_u(c.delta, 0x40004000u /* 2 */), n);
  if (TEXTURE_WEIGHTS) {
    // majority of the three planes, at the spare bit: * delta * (1/2) * (1/6)
    unsigned m;
    asm("lop3.b32 %0, %1, %2, %3, 0xE8;" : "=r"(m) : "r"(duo.x), "r"(duo.y), "r"(duo.z));
    n = hfma2_u(m & kFieldSpare, hmul2_u(c.delta, 0x2D552D55u /* 1/12 */), n);
  }
  a[7] = n;
}

// Generic path: any mode and palette, per-weight fp32 arithmetic on the canonical block,
// value = palette * 889 * 2^-16 rounded to fp16.  Kept out of line (it runs only for the rare low-mode
// blocks); the eight results travel by value.
struct BlockNumerators {
  uint4 first, second;
};
static __device__ __noinline__ BlockNumerators decode_block_generic(unsigned lo, unsigned hi, int palette) {
  unsigned long long block = (unsigned long long)lo | ((unsigned long long)hi << 32);
  int e0 = block_e0(block), e1 = block_e1(block);
  unsigned a[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float v0 = palette_value_of(palette, e0, e1, block_selector(block, 2 * i)) * (889.0f / 65536.0f);
    float v1 = palette_value_of(palette, e0, e1, block_selector(block, 2 * i + 1)) * (889.0f / 65536.0f);
    __half2 h = __floats2half2_rn(v0, v1);
    a[i] = *reinterpret_cast<unsigned *>(&h);
  }
  BlockNumerators out;
  out.first = make_uint4(a[0], a[1], a[2], a[3]);
  out.second = make_uint4(a[4], a[5], a[6], a[7]);
  return out;
}
__device__ __forceinline__ void decode_block_slow(const uint4 duo, int second, unsigned (&a)[8], int palette) {
  const unsigned long long block = duo_extract(duo, second);
  BlockNumerators n = decode_block_generic(unsigned(block), unsigned(block >> 32), palette);
  a[0] = n.first.x; a[1] = n.first.y; a[2] = n.first.z; a[3] = n.first.w;
  a[4] = n.second.x; a[5] = n.second.y; a[6] = n.second.z; a[7] = n.second.w;
}

// e0 <= e1 for block `second` of a duo (biased bytes compare like the signed endpoints)
__device__ __forceinline__ bool duo_block_is_low(const uint4 duo, int second) {
  const unsigned ends = duo.w >> (16 * second);
  return (ends & 0xffu) <= ((ends >> 8) & 0xffu);
}

// amax of |x| over one token row, as the integer order of bf16 magnitudes
__device__ __forceinline__ unsigned chunk_absmax(uint4 c) {
  unsigned m = 0;
  unsigned w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m = max(m, w[i] & 0x7fffu);
    m = max(m, (w[i] >> 16) & 0x7fffu);
  }
  return m;
}

// power-of-two scaling that brings a row with bf16 magnitude pattern `amax_bits` below 2^15
__device__ __forceinline__ void token_scaling(unsigned amax_bits, float &mult, float &inverse) {
  int ex = int(amax_bits >> 7) & 0xff;
  if (amax_bits == 0) ex = 141;
  ex = min(max(ex, 15), 254);
  mult = __int_as_float((268 - ex) << 23);      // 2^(14 - (ex-127))
  inverse = __int_as_float((ex - 14) << 23);    // 2^((ex-127) - 14)
}

__device__ __forceinline__ uint4 convert_chunk(uint4 c, float mult) {
  unsigned w[4] = {c.x, c.y, c.z, c.w};
  unsigned o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float lo = __uint_as_float(w[i] << 16) * mult;
    float hi = __uint_as_float(w[i] & 0xffff0000u) * mult;
    __half2 h = __floats2half2_rn(lo, hi);
    o[i] = *reinterpret_cast<unsigned *>(&h);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// ---------------------------------------------------------------------------------------------
// Staged form of one token for the single-token decode kernel (gemv_solo_kernel): a 16-byte slot with
// the fp32 multiplier 2^s * 2^24/889, then per 128-column unit and lane quad t the four fp16 values
// (hi_t, hi_{t+4}, lo_t, lo_{t+4}) of 7 * S_block * 2^-24 (32 bytes per unit), then the activations as
// fp16 with the factor 2^-offset of the index field they meet (256 bytes per unit).  The kernel stages
// a bf16 token itself, or copies this form when the producer of the activations wrote it.
// ---------------------------------------------------------------------------------------------
constexpr int kStagedHeader = 16;
__host__ __device__ inline size_t staged_bytes(int KI) { return kStagedHeader + size_t(KI) * (32 + 256); }
constexpr float kSoloScale = 16777216.0f / 889.0f;   // sums are (n * x) * 2^-24, palette value = n / 889

// exponent of the staging factor 2^-e for pair i of the first / second block of a duo (tx_common.cuh)
__device__ __forceinline__ int solo_pair_exponent(int second, int pair) {
  // first: offsets 0,3,6,10->0,13->3 (word 0), 0,3,6 (word 1); second: 10->0,13->3 (word 1), 0,3,6,0,3 (word 2), spare bit 9
  const unsigned table = second ? 0x93063030u : 0x63030630u;       // nibble i = exponent of pair i
  return int((table >> (4 * pair)) & 15u);
}

// Stages one token for gemv_solo_kernel: xs[column] = fp16(x * mult * 2^-e(column)), and per unit and
// lane quad t the four fp16 values (hi_t, hi_{t+4}, lo_t, lo_{t+4}) of 7 * S_block * 2^-24.
// `i` is the 8-column chunk index; chunks 2b and 2b+1 of block b sit in neighbouring lanes.
__device__ __forceinline__ void solo_stage_chunk(int i, uint4 raw, float mult, uint8_t *xs_g, uint8_t *stab_g, bool inside) {
  const int pair0 = 4 * (i & 1), second = (i >> 3) & 1;            // block b = i >> 1, second half of the unit when b & 4
  unsigned w[4] = {raw.x, raw.y, raw.z, raw.w}, o[4];
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = solo_pair_exponent(second, pair0 + j);
    const float down = __int_as_float((127 - e) << 23), up = __int_as_float((127 + e) << 23);
    const float lo = __uint_as_float(w[j] << 16) * mult * down;
    const float hi = __uint_as_float(w[j] & 0xffff0000u) * mult * down;
    const __half2 h = __floats2half2_rn(lo, hi);
    o[j] = *reinterpret_cast<const unsigned *>(&h);
    const float2 back = __half22float2(h);                          // the value the tensor core will see
    sum += (back.x + back.y) * up;
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);                      // both chunks of the block
  if (inside) {
    reinterpret_cast<uint4 *>(xs_g)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    if ((i & 1) == 0) {
      const int block = i >> 1, unit = block >> 3, t = block & 3, high = (block >> 2) & 1;
      const float v = sum * (7.0f / 16777216.0f);
      const __half hi = __float2half_rn(v);
      const __half lo = __float2half_rn(v - __half2float(hi));
      __half *entry = reinterpret_cast<__half *>(stab_g + size_t(unit) * 32 + t * 8);
      entry[high] = hi;
      entry[2 + high] = lo;
    }
  }
}

}  // namespace tx
