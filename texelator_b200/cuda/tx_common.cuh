// Shared declarations of the texelator_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/texelator_b200.h"

namespace tx {

// ---------------------------------------------------------------------------------------------
// Device layout of the BC4 payload ("tiled"): every block keeps its 64 bits of information (only an
// endpoint of -128 is stored as -127, which decodes identically under BC4-SNORM), but blocks are
// re-ordered so that one warp-wide pair of 128-bit loads fetches a 16-row x 128-column unit as 1 KiB
// of consecutive memory, and the two blocks a lane fetches with one load are bit-shuffled into a
// "duo" (below):
//
//   unit(rt, ki)  = 16 output rows [16rt, 16rt+16)  x  8 blocks [8ki, 8ki+8)      -> 1024 bytes
//   duo offset    = (rt*KI + ki)*1024 + half*512 + lane*16
//   lane = g*4+t  holds row 16rt + 8*half + g, blocks 8ki + t (first) and 8ki + 4 + t (second)
//
// This is the mma.sync m16n8k16 A-fragment ownership (lane (g,t) owns rows g and g+8), so decoded
// weights go from registers to the tensor core with no shuffle.  Rows are padded to 16 and blocks
// to 8 per row with a benign high-mode block (e0=1, e1=0, selectors 0); padded columns meet
// zero activations and padded rows are never stored.
// ---------------------------------------------------------------------------------------------
constexpr int kUnitRows = 16;
constexpr int kUnitBlocks = 8;
constexpr int kUnitBytes = 1024;
constexpr int kPadUnits = 8;   // readable units behind the payload (unguarded prefetch of the decode GEMV)
constexpr unsigned long long kPadBlock = 0x0000000000000001ull;  // e0=1, e1=0, selectors 0

// ---------------------------------------------------------------------------------------------
// The 16 bytes a lane loads -- blocks kb = 8ki+t ("first") and 8ki+4+t ("second") of one row -- are
// one "duo": the same 128 bits of information as the two 8-byte blocks, re-arranged at pack time so
// that the decode kernels need one logic instruction per pair of weights and no table:
//
//   word 3     the four endpoints as biased bytes u = e + 128: first e0, first e1, second e0, second e1
//   words 0-2  for every weight the interpolation index g in place of the selector (high palette
//              mode: selector 0,1,2..7 -> g 0,7,1..6, so that value = ((7-g)*e0 + g*e1)/7; the same
//              bijection is applied to low-mode blocks and undone by the generic decoder).
//              Each 16-bit half of a word holds five 3-bit fields at bits 0, 3, 6, 10, 13 and a spare
//              bit 9; the low half carries the even position of a pair of weights, the high half the
//              odd position, at the same offset.  A masked word is therefore an fp16x2 whose halves
//              are the subnormal numbers g * 2^(offset-24) -- the offsets 0, 3, 6 need no shift at
//              all, 10 and 13 share one shift by 10 -- and one HFMA2 with a per-block multiplier
//              turns it into the exact numerators (7*e0 + g*(e1-e0)) * 2^-16 of both weights.
//              Pairs 0-4 of the first block sit in word 0, pairs 5-7 in word 1 (offsets 0, 3, 6);
//              pairs 0-1 of the second block in word 1 (offsets 10, 13), pairs 2-6 in word 2, and
//              pair 7 in the three spare bits: bit k of its g values is bit 9 / bit 25 of word k.
//
// duo_build / duo_extract convert between this form and the canonical blocks of the file format
// (texelator/encoder.py:105-117); every kernel that is not speed critical goes through duo_extract.
// ---------------------------------------------------------------------------------------------
__host__ __device__ inline unsigned selector_to_g(unsigned s) { return s == 0 ? 0u : (s == 1 ? 7u : s - 1u); }
__host__ __device__ inline unsigned g_to_selector(unsigned g) { return g == 0 ? 0u : (g == 7 ? 1u : g + 1u); }

// where pair `pair` (weights 2*pair, 2*pair+1) of block `second` lives: word index and bit offset of the
// even weight's field (the odd weight's is 16 higher); offset -1 = the spare-bit planes
__host__ __device__ inline void duo_slot(int second, int pair, int &word, int &offset) {
  const int offsets[5] = {0, 3, 6, 10, 13};
  if (!second) {
    word = pair < 5 ? 0 : 1;
    offset = offsets[pair < 5 ? pair : pair - 5];
  } else if (pair < 2) {
    word = 1;
    offset = offsets[3 + pair];
  } else if (pair < 7) {
    word = 2;
    offset = offsets[pair - 2];
  } else {
    word = 0;
    offset = -1;
  }
}

__host__ __device__ inline unsigned biased_endpoint(unsigned long long byte) {
  unsigned u = (unsigned(byte) & 0xffu) ^ 0x80u;   // e + 128
  return u == 0 ? 1u : u;                          // BC4-SNORM reads -128 as -127
}

__host__ __device__ inline uint4 duo_build(unsigned long long first, unsigned long long second) {
  unsigned w[4] = {0, 0, 0, 0};
  for (int b = 0; b < 2; ++b) {
    const unsigned long long block = b ? second : first;
    w[3] |= (biased_endpoint(block) | (biased_endpoint(block >> 8) << 8)) << (16 * b);
    for (int pair = 0; pair < 8; ++pair) {
      const unsigned even = selector_to_g(unsigned(block >> (16 + 6 * pair)) & 7u);
      const unsigned odd = selector_to_g(unsigned(block >> (19 + 6 * pair)) & 7u);
      int word, offset;
      duo_slot(b, pair, word, offset);
      if (offset >= 0) {
        w[word] |= (even << offset) | (odd << (offset + 16));
      } else {
        for (int k = 0; k < 3; ++k) w[k] |= (((even >> k) & 1u) << 9) | (((odd >> k) & 1u) << 25);
      }
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// canonical block (endpoint -128 already stored as -127) number `second` of a duo
__host__ __device__ inline unsigned long long duo_extract(const uint4 duo, int second) {
  const unsigned w[3] = {duo.x, duo.y, duo.z};
  const unsigned ends = (duo.w >> (16 * second)) & 0xffffu;
  unsigned long long block = (unsigned long long)((ends ^ 0x8080u) & 0xffffu);
  for (int pair = 0; pair < 8; ++pair) {
    int word, offset;
    duo_slot(second, pair, word, offset);
    unsigned even = 0, odd = 0;
    if (offset >= 0) {
      even = (w[word] >> offset) & 7u;
      odd = (w[word] >> (offset + 16)) & 7u;
    } else {
      for (int k = 0; k < 3; ++k) {
        even |= ((w[k] >> 9) & 1u) << k;
        odd |= ((w[k] >> 25) & 1u) << k;
      }
    }
    block |= (unsigned long long)g_to_selector(even) << (16 + 6 * pair);
    block |= (unsigned long long)g_to_selector(odd) << (19 + 6 * pair);
  }
  return block;
}

// byte offset of the duo that holds block kb of `row`; (kb >> 2) & 1 says which of its two blocks it is
__host__ __device__ inline size_t tiled_duo_offset(int row, int kb, int KI) {
  int rt = row >> 4, half = (row >> 3) & 1, g = row & 7;
  int ki = kb >> 3, t = kb & 3;
  return (size_t(rt) * KI + ki) * kUnitBytes + half * 512 + (g * 4 + t) * 16;
}
__device__ __forceinline__ unsigned long long tiled_block(const uint8_t *tiles, int row, int kb, int KI) {
  const uint4 duo = *reinterpret_cast<const uint4 *>(tiles + tiled_duo_offset(row, kb, KI));
  return duo_extract(duo, (kb >> 2) & 1);
}

struct Handle {
  uint32_t magic = 0x54584234;  // "TXB4"
  int M = 0, K = 0, blocks_per_row = 0, device = 0;
  int MT = 0, KI = 0;           // row tiles of 16, k iterations of 128 columns
  int lookahead = 2;            // texelator_cuda.cu:48 default
  int prefill_threshold = 16, prefill_tile_rows = 1024, prefill_backend = 0;
  int decode_path = TX_DECODE_ALU_MMA;
  int palette = TX_PALETTE_SOFTWARE;   // which table the payload was encoded against
  uint8_t *tiles = nullptr;     // MT*KI*1024 bytes
  uint8_t *unit_flags = nullptr;  // MT*KI bytes: 1 if the unit holds a low-mode (e0<=e1) block
  bool has_low_mode = false;      // any unit flag set
  float *scales = nullptr;      // M
  __nv_bfloat16 *bias = nullptr;  // M or null
  int bias_dtype = TX_DTYPE_BF16;
  // texture path (created on demand)
  cudaArray_t array = nullptr;
  cudaTextureObject_t texture = 0;
};

// Per-device scratch shared by every handle of the process on that device.
struct Workspace {
  __half *xprep = nullptr;        // scaled fp16 activations of multi-token decode passes
  size_t xprep_halfs = 0;
  float *xmul = nullptr;          // per-token multipliers, one per staged token
  float *partial = nullptr;       // fp32 sums of the K ranges of a multi-token decode pass, [splits][tokens][M]
  size_t partial_floats = 0;
  int *status = nullptr;          // first non-zero code a kernel recorded when a bounded wait ran out
  int sm_count = 0;
};

// ---------------------------------------------------------------------------------------------
// Tensor-parallel exchange of one token's partial row (row-parallel linears: o, down).  Every rank owns
// an inbox in peer-mapped memory, [2 slots][world senders][hidden / 4 packets] of 16 bytes.  A packet is
// {two bf16, epoch, two bf16, epoch}: it is written with ONE 16-byte store, and a reader that sees the
// current epoch in both flag words has the four values -- no fence, no separate flag, one NVLink
// latency.  The linear's epilogue writes its packets into the inboxes of all ranks (its own included) as
// its row tiles finish, so the transfer overlaps the rest of the weight stream; the residual add +
// RMSNorm kernel that consumes the sum polls the packets, adds them in rank order (fp32, one bf16
// rounding: every rank gets the same bits) and advances the epoch word.  Slots alternate with the
// epoch; a rank can be at most one exchange ahead of a peer, so two suffice.  Every poll is bounded and
// records code 32 in the device status word when it runs out.
// ---------------------------------------------------------------------------------------------
constexpr int kMaxRanks = 8;
constexpr unsigned kPeerSpinLimit = 1u << 21;
struct PeerPush {
  uint4 *inbox[kMaxRanks];        // every rank's inbox as addressable from this rank
  const unsigned *epoch_word;     // this rank's epoch counter (the consumer kernel advances it)
  int rank, world, packets;       // packets per sender = hidden / 4
};
__device__ __forceinline__ void store_packet(uint4 *dst, unsigned lo, unsigned hi, unsigned epoch) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(lo), "r"(epoch), "r"(hi), "r"(epoch) : "memory");
}
__device__ __forceinline__ uint4 load_packet(const uint4 *src) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
  return v;
}

void set_error(const std::string &message);
int fail(int code, const std::string &message);
Workspace *workspace_for(int device);  // allocates on first use (never inside a launch path)
void count_launch(int n = 1);

#define TX_CUDA(call)                                                                      \
  do {                                                                                     \
    cudaError_t tx_status_ = (call);                                                       \
    if (tx_status_ != cudaSuccess)                                                         \
      return ::tx::fail(TX_ECUDA, std::string(#call) + ": " + cudaGetErrorString(tx_status_)); \
  } while (0)

// ---------------------------------------------------------------------------------------------
// Exact software-palette decode of one selector (BC4-SNORM interpolation, each value rounded once to fp32):
// value = RN( ((7-g)*e0 + g*e1) / 889 ) in the high mode (e0 > e1),
//         RN( ((5-g)*e0 + g*e1) / 635 ) in the low mode, selectors 6/7 -> -1/+1.
// n*c followed by one fused residual correction is the correctly rounded quotient for every
// numerator in [-889, 889] (checked exhaustively on the CPU), so no division is issued.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float rn_div_const(float n, float den, float rcp) {
  float q = n * rcp;
  float r = fmaf(-q, den, n);
  return fmaf(r, rcp, q);
}

__device__ __forceinline__ float palette_value(int e0, int e1, int sel) {
  e0 = max(e0, -127);
  e1 = max(e1, -127);
  if (e0 > e1) {
    int g = sel == 0 ? 0 : (sel == 1 ? 7 : sel - 1);
    int n = (7 - g) * e0 + g * e1;
    return rn_div_const(float(n), 889.0f, 1.0f / 889.0f);
  }
  if (sel == 6) return -1.0f;
  if (sel == 7) return 1.0f;
  int g = sel == 0 ? 0 : (sel == 1 ? 5 : sel - 1);
  int n = (5 - g) * e0 + g * e1;
  return rn_div_const(float(n), 635.0f, 1.0f / 635.0f);
}

__device__ __forceinline__ int block_selector(unsigned long long block, int p) {
  return int((block >> (16 + 3 * p)) & 7ull);
}
__device__ __forceinline__ int block_e0(unsigned long long block) { return int(int8_t(block & 0xff)); }
__device__ __forceinline__ int block_e1(unsigned long long block) { return int(int8_t((block >> 8) & 0xff)); }

// Exact texture-unit ("hardware") palette, the table NVIDIA texture units return for signed BC4 and
// the reference measures (texelator_cuda.cu:1540-1595): endpoints widened to 16-bit snorm by bit
// replication, interpolants = nearer endpoint + {36,72,144}*(e1-e0) (8-value mode) or {48,96}*(e1-e0)
// (6-value mode), value = I/32767 rounded to fp32 (same correctly rounded quotient trick).
__device__ __forceinline__ int widen_snorm8(int e) {
  int m = abs(e);
  int w = (m << 8) | (m << 1) | (m >> 6);
  return e < 0 ? -w : w;
}
__device__ __forceinline__ float hardware_palette_value(int e0, int e1, int sel) {
  e0 = max(e0, -127);
  e1 = max(e1, -127);
  const int x0 = widen_snorm8(e0), x1 = widen_snorm8(e1), d = e1 - e0;
  int v;
  if (sel == 0) v = x0;
  else if (sel == 1) v = x1;
  else if (e0 > e1) {
    switch (sel) {
      case 2: v = x0 + 36 * d; break;
      case 3: v = x0 + 72 * d; break;
      case 4: v = x1 - 144 * d; break;
      case 5: v = x0 + 144 * d; break;
      case 6: v = x1 - 72 * d; break;
      default: v = x1 - 36 * d; break;
    }
  } else {
    switch (sel) {
      case 2: v = x0 + 48 * d; break;
      case 3: v = x0 + 96 * d; break;
      case 4: v = x1 - 96 * d; break;
      case 5: v = x1 - 48 * d; break;
      case 6: v = -32767; break;
      default: v = 32767; break;
    }
  }
  return rn_div_const(float(v), 32767.0f, 1.0f / 32767.0f);
}
__device__ __forceinline__ float palette_value_of(int palette, int e0, int e1, int sel) {
  return palette == TX_PALETTE_HARDWARE ? hardware_palette_value(e0, e1, sel) : palette_value(e0, e1, sel);
}

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch.  Kernels of the decode step are short (a few microseconds), so the
// launch gap and the prologue of each kernel matter.  Launched with the programmatic-serialisation
// attribute, a kernel may start while its predecessor on the stream is still draining; everything it
// does before `grid_dependency_wait()` must therefore only read immutable data (weights, tables) and
// write nothing outside the CTA.  `grid_dependency_wait()` returns once all earlier work on the stream
// is complete and visible (a no-op for ordinary launches).  Data that an earlier kernel produced must
// then be read through L2 (`__ldcg` / ld.global.cg): a CTA that started early shares its SM's L1 with
// kernels that may have cached the old lines (observed on B200 as stale activations under CUDA-graph
// replay).  TEXELATOR_B200_NO_PDL=1 turns the attribute off.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool pdl_enabled();

template <typename... KernelArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, KernelArgs(args)...);
}

// launchers implemented in the other translation units
int launch_retile(const uint8_t *rowmajor_dev, Handle *h, cudaStream_t stream);
int launch_untile(const Handle *h, uint8_t *rowmajor_dev, cudaStream_t stream);
int launch_dequant(const Handle *h, void *out, int what, cudaStream_t stream);
int launch_gemv(const Handle *h, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream, bool half_io = false);
int launch_gemv_fused(const Handle *h, const __nv_bfloat16 *x, const __nv_bfloat16 *delta, const __nv_bfloat16 *gamma, float eps,
                      __nv_bfloat16 *residual_out, bool swiglu, __nv_bfloat16 *y, int tokens, cudaStream_t stream);
bool gemv_single_eligible(const Handle *h);
int gemv_suggest_splits(const Handle *h);
int launch_gemv_single(const Handle *h, const __nv_bfloat16 *x, const uint8_t *staged, bool swiglu, __nv_bfloat16 *y,
                       float *y_partial, int splits, size_t partial_stride, const PeerPush *push, cudaStream_t stream);
int launch_gemv_static_scratch(const Handle *h, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream);
int launch_gemv_exact(const Handle *h, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream);
int launch_gemv_texture(const Handle *h, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens, cudaStream_t stream);
int launch_prefill_tile(const Handle *h, int backend, const __nv_bfloat16 *x, __nv_bfloat16 *y, int tokens,
                        cudaStream_t stream, bool half_io = false);
// y = round(sum of `ranges` fp32 partial results [ranges][tokens][M] + bias): second step of a launch that cut K
int launch_combine(const float *partial, int ranges, const void *bias, void *y, int tokens, int M, bool half_io, int sm_count,
                   cudaStream_t stream);
bool prefill_tile_eligible(const Handle *h, int backend, int tokens);
int gemv_kernel_info(int64_t out[9]);
int prefill_kernel_info(int backend, int64_t out[9]);
int texture_supported(int device);                       // 1 / 0
int create_texture(Handle *h);                           // builds array + BC4 view from the tiled copy
int probe_texture_palette(int device, float *out_host);  // TX_EUNSUPPORTED when views cannot be made
int probe_software_palette(int device, float *out_host, int palette);

}  // namespace tx
