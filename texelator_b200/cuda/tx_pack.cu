// Packing (row-major BC4 -> tiled device layout), exact dequantisation, palette tables and the
// CUDA texture probe.
#include <vector>

#include "tx_common.cuh"

namespace tx {

// ------------------------------------------------------------------------------------------
// retile: one thread per destination duo (two blocks of one row, tx_common.cuh).  Reference
// counterpart: the cudaMemcpy2DToArray upload of texelator_cuda.cu:1296-1299 (a cudaArray is an
// opaque swizzled layout as well).
// ------------------------------------------------------------------------------------------
__global__ void retile_kernel(const unsigned long long *__restrict__ src, uint4 *__restrict__ dst,
                              uint8_t *__restrict__ unit_flags, int M, int bpr, int MT, int KI) {
  size_t total = size_t(MT) * KI * 64;  // destination duos
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    size_t unit = i >> 6;
    int in_unit = int(i & 63);
    int half = in_unit >> 5, lane = in_unit & 31;
    int rt = int(unit / KI), ki = int(unit % KI);
    int row = rt * 16 + half * 8 + (lane >> 2);
    unsigned long long blocks[2];
#pragma unroll
    for (int second = 0; second < 2; ++second) {
      int kb = ki * 8 + second * 4 + (lane & 3);
      unsigned long long block = kPadBlock;
      if (row < M && kb < bpr) {
        block = src[size_t(row) * bpr + kb];
        // BC4-SNORM reads -128 as -127: compare the endpoints the decoders will see
        int e0 = max(block_e0(block), -127), e1 = max(block_e1(block), -127);
        if (e0 <= e1) unit_flags[unit] = 1;  // benign race: all writers store 1
      }
      blocks[second] = block;
    }
    dst[i] = duo_build(blocks[0], blocks[1]);
  }
}

__global__ void untile_kernel(const uint8_t *__restrict__ tiles, unsigned long long *__restrict__ dst,
                              int M, int bpr, int KI) {
  size_t total = size_t(M) * bpr;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    int row = int(i / bpr), kb = int(i % bpr);
    dst[i] = tiled_block(tiles, row, kb, KI);
  }
}

__global__ void any_flag_kernel(const uint8_t *__restrict__ flags, size_t units, int *__restrict__ result) {
  int seen = 0;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < units; i += size_t(gridDim.x) * blockDim.x) seen |= flags[i];
  if (__any_sync(0xffffffffu, seen) && (threadIdx.x & 31) == 0) atomicOr(result, 1);
}

int launch_retile(const uint8_t *rowmajor_dev, Handle *h, cudaStream_t stream) {
  size_t units = size_t(h->MT) * h->KI;
  TX_CUDA(cudaMemsetAsync(h->unit_flags, 0, units, stream));
  size_t total = units * 64;
  int grid = int(std::min<size_t>((total + 255) / 256, 148 * 16));
  retile_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const unsigned long long *>(rowmajor_dev),
                                          reinterpret_cast<uint4 *>(h->tiles), h->unit_flags, h->M,
                                          h->blocks_per_row, h->MT, h->KI);
  count_launch();
  TX_CUDA(cudaGetLastError());
  // does the payload contain any low-mode block at all?  (decides the decode kernel variant)
  Workspace *ws = workspace_for(h->device);
  if (!ws) return TX_ECUDA;
  TX_CUDA(cudaMemsetAsync(ws->status + 1, 0, sizeof(int), stream));
  any_flag_kernel<<<int(std::min<size_t>((units + 255) / 256, 592)), 256, 0, stream>>>(h->unit_flags, units, ws->status + 1);
  count_launch();
  int any = 0;
  TX_CUDA(cudaMemcpyAsync(&any, ws->status + 1, sizeof(int), cudaMemcpyDeviceToHost, stream));
  TX_CUDA(cudaStreamSynchronize(stream));
  h->has_low_mode = any != 0;
  return TX_OK;
}

int launch_untile(const Handle *h, uint8_t *rowmajor_dev, cudaStream_t stream) {
  size_t total = size_t(h->M) * h->blocks_per_row;
  int grid = int(std::min<size_t>((total + 255) / 256, 148 * 16));
  untile_kernel<<<grid, 256, 0, stream>>>(h->tiles, reinterpret_cast<unsigned long long *>(rowmajor_dev), h->M,
                                          h->blocks_per_row, h->KI);
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

// ------------------------------------------------------------------------------------------
// dequant: one thread per block, 16 outputs each.  Bit-exact to the software palette; the scaled
// forms follow texelator_cuda.cu:141-152 (fp32 pal*scale, then one bf16 rounding).
// ------------------------------------------------------------------------------------------
template <int WHAT>
__global__ void dequant_kernel(const uint8_t *__restrict__ tiles, const float *__restrict__ scales,
                               void *__restrict__ out, int M, int bpr, int KI, int palette) {
  size_t total = size_t(M) * bpr;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    int row = int(i / bpr), kb = int(i % bpr);
    unsigned long long block = tiled_block(tiles, row, kb, KI);
    int e0 = block_e0(block), e1 = block_e1(block);
    float scale = WHAT == TX_DEQUANT_PALETTE_F32 ? 1.0f : scales[row];
    float v[16];
#pragma unroll
    for (int p = 0; p < 16; ++p) {
      float pal = palette_value_of(palette, e0, e1, block_selector(block, p));
      v[p] = WHAT == TX_DEQUANT_PALETTE_F32 ? pal : __fmul_rn(pal, scale);
    }
    size_t base = size_t(row) * bpr * 16 + size_t(kb) * 16;
    if (WHAT == TX_DEQUANT_SCALED_BF16) {
      __nv_bfloat162 packed[8];
#pragma unroll
      for (int p = 0; p < 8; ++p) packed[p] = __floats2bfloat162_rn(v[2 * p], v[2 * p + 1]);
      uint4 *dst = reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(out) + base);
      dst[0] = reinterpret_cast<uint4 *>(packed)[0];
      dst[1] = reinterpret_cast<uint4 *>(packed)[1];
    } else {
      float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(out) + base);
#pragma unroll
      for (int p = 0; p < 4; ++p) dst[p] = make_float4(v[4 * p], v[4 * p + 1], v[4 * p + 2], v[4 * p + 3]);
    }
  }
}

int launch_dequant(const Handle *h, void *out, int what, cudaStream_t stream) {
  size_t total = size_t(h->M) * h->blocks_per_row;
  int grid = int(std::min<size_t>((total + 127) / 128, 148 * 32));
  const uint8_t *tiles = h->tiles;
  switch (what) {
    case TX_DEQUANT_PALETTE_F32:
      dequant_kernel<TX_DEQUANT_PALETTE_F32><<<grid, 128, 0, stream>>>(tiles, h->scales, out, h->M, h->blocks_per_row, h->KI, h->palette);
      break;
    case TX_DEQUANT_SCALED_F32:
      dequant_kernel<TX_DEQUANT_SCALED_F32><<<grid, 128, 0, stream>>>(tiles, h->scales, out, h->M, h->blocks_per_row, h->KI, h->palette);
      break;
    case TX_DEQUANT_SCALED_BF16:
      dequant_kernel<TX_DEQUANT_SCALED_BF16><<<grid, 128, 0, stream>>>(tiles, h->scales, out, h->M, h->blocks_per_row, h->KI, h->palette);
      break;
    default:
      return fail(TX_EINVAL, "tx_dequant: unknown output selector");
  }
  count_launch();
  TX_CUDA(cudaGetLastError());
  return TX_OK;
}

// ------------------------------------------------------------------------------------------
// Palette tables.  Probe blocks are the ones the reference builds in texelator_cuda.cu:1551-1564:
// block (x=e0+127, y=e1+127), position p carries selector p & 7.
// ------------------------------------------------------------------------------------------
static void build_probe_blocks(std::vector<unsigned long long> &host) {
  host.resize(255 * 255);
  unsigned long long selectors = 0;
  for (int p = 0; p < 16; ++p) selectors |= (unsigned long long)(p & 7) << (3 * p);
  for (int y = 0; y < 255; ++y)
    for (int x = 0; x < 255; ++x) {
      unsigned long long e0 = (unsigned long long)(uint8_t)(int8_t)(x - 127);
      unsigned long long e1 = (unsigned long long)(uint8_t)(int8_t)(y - 127);
      host[size_t(y) * 255 + x] = e0 | (e1 << 8) | (selectors << 16);
    }
}

__global__ void software_palette_kernel(const unsigned long long *__restrict__ blocks, float *__restrict__ out, int pairs,
                                        int palette) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  unsigned long long block = blocks[i];
  for (int s = 0; s < 8; ++s) out[size_t(i) * 8 + s] = palette_value_of(palette, block_e0(block), block_e1(block), block_selector(block, s));
}

int probe_software_palette(int device, float *out_host, int palette) {
  TX_CUDA(cudaSetDevice(device));
  constexpr int pairs = 255 * 255;
  std::vector<unsigned long long> host;
  build_probe_blocks(host);
  unsigned long long *blocks = nullptr;
  float *out = nullptr;
  TX_CUDA(cudaMalloc(&blocks, size_t(pairs) * 8));
  TX_CUDA(cudaMalloc(&out, size_t(pairs) * 8 * sizeof(float)));
  TX_CUDA(cudaMemcpy(blocks, host.data(), size_t(pairs) * 8, cudaMemcpyHostToDevice));
  software_palette_kernel<<<(pairs + 255) / 256, 256>>>(blocks, out, pairs, palette);
  count_launch();
  cudaError_t status = cudaGetLastError();
  if (status == cudaSuccess) status = cudaMemcpy(out_host, out, size_t(pairs) * 8 * sizeof(float), cudaMemcpyDeviceToHost);
  cudaFree(blocks);
  cudaFree(out);
  if (status != cudaSuccess) return fail(TX_ECUDA, std::string("software palette: ") + cudaGetErrorString(status));
  return TX_OK;
}

// ------------------------------------------------------------------------------------------
// CUDA texture objects with a signed-BC4 resource view (texelator_cuda.cu:1296-1312).  No graphics
// API is involved: these are CUDA runtime calls.  Whether the device accepts such a view is a
// run-time fact, so creation failures are reported as TX_EUNSUPPORTED, never fatal.
// ------------------------------------------------------------------------------------------
static cudaError_t make_bc4_texture(cudaArray_t *array, cudaTextureObject_t *texture, const void *src,
                                    cudaMemcpyKind kind, int blocks_per_row, int rows) {
  cudaChannelFormatDesc description = cudaCreateChannelDesc<uint2>();
  cudaError_t status = cudaMallocArray(array, &description, blocks_per_row, rows);
  if (status != cudaSuccess) return status;
  status = cudaMemcpy2DToArray(*array, 0, 0, src, size_t(blocks_per_row) * 8, size_t(blocks_per_row) * 8, rows, kind);
  if (status != cudaSuccess) return status;
  cudaResourceDesc resource{};
  resource.resType = cudaResourceTypeArray;
  resource.res.array.array = *array;
  cudaResourceViewDesc view{};
  view.format = cudaResViewFormatSignedBlockCompressed4;
  view.width = size_t(blocks_per_row) * 4;
  view.height = size_t(rows) * 4;
  cudaTextureDesc description_t{};
  description_t.addressMode[0] = cudaAddressModeClamp;
  description_t.addressMode[1] = cudaAddressModeClamp;
  description_t.filterMode = cudaFilterModePoint;
  description_t.readMode = cudaReadModeElementType;
  return cudaCreateTextureObject(texture, &resource, &description_t, &view);
}

__global__ void texture_palette_kernel(cudaTextureObject_t texture, float *__restrict__ out, int pairs) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  int x = i % 255, y = i / 255;
  for (int s = 0; s < 8; ++s)
    out[size_t(i) * 8 + s] = tex2D<float>(texture, x * 4 + (s & 3) + 0.5f, y * 4 + (s >> 2) + 0.5f);
}

int probe_texture_palette(int device, float *out_host) {
  TX_CUDA(cudaSetDevice(device));
  constexpr int pairs = 255 * 255;
  std::vector<unsigned long long> host;
  build_probe_blocks(host);
  cudaArray_t array = nullptr;
  cudaTextureObject_t texture = 0;
  cudaError_t status = make_bc4_texture(&array, &texture, host.data(), cudaMemcpyHostToDevice, 255, 255);
  if (status != cudaSuccess) {
    cudaGetLastError();
    if (texture) cudaDestroyTextureObject(texture);
    if (array) cudaFreeArray(array);
    return fail(TX_EUNSUPPORTED, std::string("signed-BC4 texture view unavailable: ") + cudaGetErrorString(status));
  }
  float *out = nullptr;
  status = cudaMalloc(&out, size_t(pairs) * 8 * sizeof(float));
  if (status == cudaSuccess) {
    texture_palette_kernel<<<(pairs + 255) / 256, 256>>>(texture, out, pairs);
    count_launch();
    status = cudaGetLastError();
  }
  if (status == cudaSuccess) status = cudaMemcpy(out_host, out, size_t(pairs) * 8 * sizeof(float), cudaMemcpyDeviceToHost);
  if (out) cudaFree(out);
  cudaDestroyTextureObject(texture);
  cudaFreeArray(array);
  if (status != cudaSuccess) return fail(TX_ECUDA, std::string("texture palette probe: ") + cudaGetErrorString(status));
  return TX_OK;
}

int texture_supported(int device) {
  static int cached[64];
  static bool known[64];
  if (device < 0 || device >= 64) return 0;
  if (known[device]) return cached[device];
  int previous = 0;
  cudaGetDevice(&previous);
  cudaSetDevice(device);
  unsigned long long block = kPadBlock;
  cudaArray_t array = nullptr;
  cudaTextureObject_t texture = 0;
  cudaError_t status = make_bc4_texture(&array, &texture, &block, cudaMemcpyHostToDevice, 1, 1);
  if (status != cudaSuccess) cudaGetLastError();
  if (texture) cudaDestroyTextureObject(texture);
  if (array) cudaFreeArray(array);
  cudaSetDevice(previous);
  cached[device] = status == cudaSuccess ? 1 : 0;
  known[device] = true;
  return cached[device];
}

int create_texture(Handle *h) {
  if (h->texture) return TX_OK;
  if (!texture_supported(h->device)) return fail(TX_EUNSUPPORTED, "signed-BC4 texture views are unavailable on this device");
  uint8_t *linear = nullptr;
  size_t bytes = size_t(h->M) * h->blocks_per_row * 8;
  TX_CUDA(cudaMalloc(&linear, bytes));
  int rc = launch_untile(h, linear, 0);
  if (rc == TX_OK && cudaStreamSynchronize(0) != cudaSuccess) rc = fail(TX_ECUDA, "untile failed");
  if (rc == TX_OK) {
    cudaError_t status = make_bc4_texture(&h->array, &h->texture, linear, cudaMemcpyDeviceToDevice, h->blocks_per_row, h->M);
    if (status != cudaSuccess) {
      cudaGetLastError();
      if (h->texture) cudaDestroyTextureObject(h->texture);
      if (h->array) cudaFreeArray(h->array);
      h->texture = 0;
      h->array = nullptr;
      rc = fail(TX_EUNSUPPORTED, std::string("BC4 texture creation failed: ") + cudaGetErrorString(status));
    }
  }
  cudaFree(linear);
  return rc;
}

}  // namespace tx
