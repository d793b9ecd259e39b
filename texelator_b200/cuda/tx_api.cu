// C ABI of texelator_b200: handle life cycle, dispatcher, setters and info calls.
// Reference counterparts: texelator/cuda/extension.cpp:7-48 (binding) and
// texelator/cuda/texelator_cuda.cu:1260-1538 (implementation).
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "tx_common.cuh"
#include "tx_decode.cuh"

namespace tx {

static thread_local std::string g_error;
static std::atomic<long long> g_launches{0};
static std::mutex g_workspace_guard;
static std::map<int, Workspace> g_workspaces;

void set_error(const std::string &message) { g_error = message; }
int fail(int code, const std::string &message) {
  g_error = message;
  return code;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
bool pdl_enabled() {
  static const bool enabled = [] {
    const char *value = std::getenv("TEXELATOR_B200_NO_PDL");
    return !(value && value[0] && value[0] != '0');
  }();
  return enabled;
}

// The scratch is sized once per device: 48 Mi scaled fp16 activations (96 MiB; multi-token decode
// passes use the first 32 tokens' worth, the prefill GEMM stages whole token chunks) plus one
// multiplier per staged token, and 16 Mi floats (64 MiB) for the K-range sums of multi-token decode passes.
Workspace *workspace_for(int device) {
  std::lock_guard<std::mutex> lock(g_workspace_guard);
  auto found = g_workspaces.find(device);
  if (found != g_workspaces.end()) return &found->second;
  int previous = 0;
  cudaGetDevice(&previous);
  Workspace ws;
  cudaError_t status = cudaSetDevice(device);
  if (status == cudaSuccess) status = cudaDeviceGetAttribute(&ws.sm_count, cudaDevAttrMultiProcessorCount, device);
  ws.xprep_halfs = size_t(48) << 20;
  if (status == cudaSuccess) status = cudaMalloc(&ws.xprep, ws.xprep_halfs * sizeof(__half));
  if (status == cudaSuccess) status = cudaMalloc(&ws.xmul, 65536 * sizeof(float));
  ws.partial_floats = size_t(16) << 20;
  if (status == cudaSuccess) status = cudaMalloc(&ws.partial, ws.partial_floats * sizeof(float));
  if (status == cudaSuccess) status = cudaMalloc(&ws.status, 2 * sizeof(int));   // [0] kernel status, [1] pack-time scratch
  if (status == cudaSuccess) status = cudaMemset(ws.status, 0, 2 * sizeof(int));
  cudaSetDevice(previous);
  if (status != cudaSuccess) {
    g_error = std::string("workspace allocation failed: ") + cudaGetErrorString(status);
    return nullptr;
  }
  return &g_workspaces.emplace(device, ws).first->second;
}

static Handle *as_handle(uint64_t value) {
  auto *h = reinterpret_cast<Handle *>(value);
  if (!h || h->magic != 0x54584234) return nullptr;
  return h;
}

static void destroy(Handle *h) {
  int previous = 0;
  cudaGetDevice(&previous);
  cudaSetDevice(h->device);
  if (h->texture) cudaDestroyTextureObject(h->texture);
  if (h->array) cudaFreeArray(h->array);
  if (h->tiles) cudaFree(h->tiles);
  if (h->unit_flags) cudaFree(h->unit_flags);
  if (h->scales) cudaFree(h->scales);
  if (h->bias) cudaFree(h->bias);
  h->magic = 0;
  delete h;
  cudaSetDevice(previous);
}

static int pack_common(const uint8_t *blocks, size_t src_pitch_blocks, const float *scales, int rows, int bpr,
                       const void *bias_dev, int bias_dtype, int device, uint64_t *out) {
  if (bias_dev && bias_dtype != TX_DTYPE_BF16 && bias_dtype != TX_DTYPE_F16) return fail(TX_EINVAL, "bias must be CUDA FP16 or BF16 [M]");
  int previous = 0;
  cudaGetDevice(&previous);
  cudaError_t status = cudaSetDevice(device);
  if (status != cudaSuccess) return fail(TX_ECUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(status));
  if (!workspace_for(device)) {
    cudaSetDevice(previous);
    return TX_ECUDA;
  }
  auto *h = new Handle;
  h->M = rows;
  h->blocks_per_row = bpr;
  h->K = bpr * 16;
  h->device = device;
  h->MT = (rows + 15) / 16;
  h->KI = (bpr + 7) / 8;
  size_t units = size_t(h->MT) * h->KI;
  uint8_t *staging = nullptr;
  int rc = TX_OK;
  auto check = [&](cudaError_t s, const char *what) {
    if (s != cudaSuccess && rc == TX_OK) rc = fail(TX_ECUDA, std::string(what) + ": " + cudaGetErrorString(s));
  };
  check(cudaMalloc(&h->tiles, (units + kPadUnits) * kUnitBytes), "cudaMalloc(tiles)");
  check(cudaMalloc(&h->unit_flags, units + kPadUnits), "cudaMalloc(flags)");
  if (rc == TX_OK) check(cudaMemset(h->tiles + units * kUnitBytes, 0, size_t(kPadUnits) * kUnitBytes), "cudaMemset(pad)");
  if (rc == TX_OK) check(cudaMemset(h->unit_flags + units, 0, kPadUnits), "cudaMemset(pad flags)");
  check(cudaMalloc(&h->scales, size_t(rows) * sizeof(float)), "cudaMalloc(scales)");
  check(cudaMalloc(&staging, size_t(rows) * bpr * 8), "cudaMalloc(staging)");
  if (rc == TX_OK)
    check(cudaMemcpy2D(staging, size_t(bpr) * 8, blocks, src_pitch_blocks * 8, size_t(bpr) * 8, rows, cudaMemcpyDefault),
          "cudaMemcpy2D(blocks)");
  if (rc == TX_OK) check(cudaMemcpy(h->scales, scales, size_t(rows) * sizeof(float), cudaMemcpyDefault), "cudaMemcpy(scales)");
  if (rc == TX_OK) rc = launch_retile(staging, h, 0);
  if (rc == TX_OK && bias_dev) {
    check(cudaMalloc(&h->bias, size_t(rows) * 2), "cudaMalloc(bias)");
    if (rc == TX_OK) check(cudaMemcpy(h->bias, bias_dev, size_t(rows) * 2, cudaMemcpyDeviceToDevice), "cudaMemcpy(bias)");
    h->bias_dtype = bias_dtype;
  }
  if (rc == TX_OK) check(cudaDeviceSynchronize(), "pack synchronise");
  if (staging) cudaFree(staging);
  if (rc != TX_OK) {
    destroy(h);
    cudaSetDevice(previous);
    return rc;
  }
  cudaSetDevice(previous);
  *out = reinterpret_cast<uint64_t>(h);
  return TX_OK;
}

}  // namespace tx

using namespace tx;

extern "C" {

const char *tx_last_error(void) { return g_error.c_str(); }

int64_t tx_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int tx_runtime_info(int device, int64_t out[4]) {
  if (!out) return fail(TX_EINVAL, "tx_runtime_info: null output");
  int sms = 0;
  TX_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  out[0] = 1;
  out[1] = 100;
  out[2] = sms;
  out[3] = texture_supported(device);
  return TX_OK;
}

int tx_pack_encoded(const uint8_t *blocks, size_t nbytes, const float *scales, int M, const void *bias_dev,
                    int bias_dtype, int device, uint64_t *out_handle) {
  if (!blocks || !scales || !out_handle) return fail(TX_EINVAL, "tx_pack_encoded: null argument");
  // texelator_cuda.cu:1266-1269
  if (M <= 0 || nbytes == 0 || nbytes % (size_t(M) * 8) != 0) return fail(TX_EINVAL, "invalid encoded size");
  int bpr = int(nbytes / (size_t(M) * 8));
  return pack_common(blocks, bpr, scales, M, bpr, bias_dev, bias_dtype, device, out_handle);
}

int tx_pack_encoded_shard(const uint8_t *blocks, size_t nbytes, const float *scales, int M, int K, int row_begin,
                          int row_end, int kblock_begin, int kblock_end, const void *bias_dev, int bias_dtype,
                          int device, uint64_t *out_handle) {
  if (!blocks || !scales || !out_handle) return fail(TX_EINVAL, "tx_pack_encoded_shard: null argument");
  if (M <= 0 || K <= 0 || K % 16 || nbytes != size_t(M) * (K / 16) * 8) return fail(TX_EINVAL, "invalid encoded size");
  int bpr = K / 16;
  if (row_begin < 0 || row_end > M || row_begin >= row_end || kblock_begin < 0 || kblock_end > bpr || kblock_begin >= kblock_end)
    return fail(TX_EINVAL, "shard range is empty or outside the matrix");
  const uint8_t *first = blocks + (size_t(row_begin) * bpr + kblock_begin) * 8;
  const void *bias = bias_dev ? static_cast<const uint8_t *>(bias_dev) + size_t(row_begin) * 2 : nullptr;
  return pack_common(first, bpr, scales + row_begin, row_end - row_begin, kblock_end - kblock_begin, bias, bias_dtype,
                     device, out_handle);
}

int tx_linear(uint64_t handle, const void *x, void *y, int tokens, int dtype, void *stream_ptr) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (!x || !y) return fail(TX_EINVAL, "input must be contiguous CUDA FP16 or BF16");
  if (dtype != TX_DTYPE_BF16 && dtype != TX_DTYPE_F16) return fail(TX_EINVAL, "input must be contiguous CUDA FP16 or BF16");
  if (tokens <= 0) return fail(TX_EINVAL, "input shape/device mismatch");
  if (h->bias && h->bias_dtype != dtype) return fail(TX_EINVAL, "input and bias dtypes must match");   // texelator_cuda.cu:1449
  const bool half_io = dtype == TX_DTYPE_F16;
  if (half_io && h->decode_path != TX_DECODE_ALU_MMA)
    return fail(TX_EUNSUPPORTED, "the exact-arithmetic and texture decode paths restate the reference's bf16 kernel; fp16 runs on the default path");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15)
    return fail(TX_EINVAL, "activation and output pointers must be 16-byte aligned");
  auto stream = static_cast<cudaStream_t>(stream_ptr);
  auto xb = static_cast<const __nv_bfloat16 *>(x);
  auto yb = static_cast<__nv_bfloat16 *>(y);
  int current = 0;
  TX_CUDA(cudaGetDevice(&current));
  if (current != h->device) TX_CUDA(cudaSetDevice(h->device));
  int rc;
  // texelator_cuda.cu:1341 -- tokens >= threshold takes the prefill side of the dispatcher
  if (tokens >= h->prefill_threshold && h->prefill_backend >= 5 && prefill_tile_eligible(h, h->prefill_backend, tokens)) {
    rc = launch_prefill_tile(h, h->prefill_backend, xb, yb, tokens, stream, half_io);
  } else if (h->decode_path == TX_DECODE_ALU_EXACT) {
    rc = launch_gemv_exact(h, xb, yb, tokens, stream);
  } else if (h->decode_path == TX_DECODE_TEXTURE && tokens < h->prefill_threshold) {
    rc = launch_gemv_texture(h, xb, yb, tokens, stream);
  } else {
    rc = launch_gemv(h, xb, yb, tokens, stream, half_io);
  }
  if (current != h->device) cudaSetDevice(current);
  return rc;
}

// the entry points below read the bias as bf16
static bool bias_is_bf16(const Handle *h) { return !h->bias || h->bias_dtype == TX_DTYPE_BF16; }

int tx_linear_static_scratch(uint64_t handle, const void *x, void *y, int tokens, int dtype, void *stream_ptr) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (!x || !y || dtype != TX_DTYPE_BF16) return fail(TX_EINVAL, "input must be contiguous CUDA BF16");
  if (!bias_is_bf16(h)) return fail(TX_EINVAL, "input and bias dtypes must match");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15)
    return fail(TX_EINVAL, "activation and output pointers must be 16-byte aligned");
  int current = 0;
  TX_CUDA(cudaGetDevice(&current));
  if (current != h->device) TX_CUDA(cudaSetDevice(h->device));
  int rc = launch_gemv_static_scratch(h, static_cast<const __nv_bfloat16 *>(x), static_cast<__nv_bfloat16 *>(y), tokens,
                                      static_cast<cudaStream_t>(stream_ptr));
  if (current != h->device) cudaSetDevice(current);
  return rc;
}

int tx_linear_single(uint64_t handle, const void *x, const void *staged, int swiglu, void *y, float *y_partial, int splits,
                     size_t partial_stride, void *stream_ptr) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (!bias_is_bf16(h)) return fail(TX_EINVAL, "input and bias dtypes must match");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(staged) | reinterpret_cast<uintptr_t>(y) |
       reinterpret_cast<uintptr_t>(y_partial)) & 15)
    return fail(TX_EINVAL, "activation and output pointers must be 16-byte aligned");
  int current = 0;
  TX_CUDA(cudaGetDevice(&current));
  if (current != h->device) TX_CUDA(cudaSetDevice(h->device));
  int rc = launch_gemv_single(h, static_cast<const __nv_bfloat16 *>(x), static_cast<const uint8_t *>(staged), swiglu != 0,
                              static_cast<__nv_bfloat16 *>(y), y_partial, splits, partial_stride, nullptr, static_cast<cudaStream_t>(stream_ptr));
  if (current != h->device) cudaSetDevice(current);
  return rc;
}

int tx_linear_single_info(uint64_t handle, int64_t out[3]) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (!out) return fail(TX_EINVAL, "tx_linear_single_info: null output");
  out[0] = gemv_single_eligible(h) ? 1 : 0;
  out[1] = gemv_suggest_splits(h);
  out[2] = int64_t(staged_bytes(h->KI));
  return TX_OK;
}

int tx_linear_fused(uint64_t handle, const void *x, const void *delta, const void *norm_weight, float eps, void *residual_out,
                    int swiglu, void *y, int tokens, int dtype, void *stream_ptr) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (!x || !y || dtype != TX_DTYPE_BF16) return fail(TX_EINVAL, "input must be contiguous CUDA BF16");
  if (!bias_is_bf16(h)) return fail(TX_EINVAL, "input and bias dtypes must match");
  if (tokens < 1) return fail(TX_EINVAL, "tokens must be positive");
  if (h->decode_path != TX_DECODE_ALU_MMA) return fail(TX_EUNSUPPORTED, "fused linear runs on the ALU mma decode path only");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(delta) |
       reinterpret_cast<uintptr_t>(norm_weight) | reinterpret_cast<uintptr_t>(residual_out)) & 15)
    return fail(TX_EINVAL, "activation, norm and output pointers must be 16-byte aligned");
  int current = 0;
  TX_CUDA(cudaGetDevice(&current));
  if (current != h->device) TX_CUDA(cudaSetDevice(h->device));
  int rc = launch_gemv_fused(h, static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(delta),
                             static_cast<const __nv_bfloat16 *>(norm_weight), eps, static_cast<__nv_bfloat16 *>(residual_out),
                             swiglu != 0, static_cast<__nv_bfloat16 *>(y), tokens, static_cast<cudaStream_t>(stream_ptr));
  if (current != h->device) cudaSetDevice(current);
  return rc;
}

int tx_set_lookahead(uint64_t handle, int lookahead) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (lookahead != 1 && lookahead != 2 && lookahead != 3 && lookahead != 4 && lookahead != 6 && lookahead != 8)
    return fail(TX_EINVAL, "lookahead must be one of 1,2,3,4,6,8");
  h->lookahead = lookahead;
  return TX_OK;
}

int tx_set_prefill(uint64_t handle, int threshold, int tile_rows) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (threshold < 1) return fail(TX_EINVAL, "prefill threshold must be positive");
  if (tile_rows < 16 || tile_rows % 16) return fail(TX_EINVAL, "prefill tile rows must be a positive multiple of 16");
  h->prefill_threshold = threshold;
  h->prefill_tile_rows = tile_rows;
  return TX_OK;
}

int tx_set_prefill_backend(uint64_t handle, int backend) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (backend < 0 || backend > 9) return fail(TX_EINVAL, "prefill backend must be in 0..9");
  h->prefill_backend = backend;
  return TX_OK;
}

int tx_set_decode_path(uint64_t handle, int path) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (path != TX_DECODE_ALU_MMA && path != TX_DECODE_ALU_EXACT && path != TX_DECODE_TEXTURE)
    return fail(TX_EINVAL, "unknown decode path");
  if (path == TX_DECODE_TEXTURE) {
    int current = 0;
    TX_CUDA(cudaGetDevice(&current));
    TX_CUDA(cudaSetDevice(h->device));
    // palette gate (tuning.py:38-41): the texture unit must reproduce the encoder's palette bit for bit
    static std::mutex guard;
    static std::map<std::pair<int, int>, int> verdict;  // (device, palette) -> 1 match, 0 mismatch, -1 unsupported
    int state;
    {
      std::lock_guard<std::mutex> lock(guard);
      auto key = std::make_pair(h->device, h->palette);
      auto found = verdict.find(key);
      if (found == verdict.end()) {
        std::vector<float> hw(65025 * 8), sw(65025 * 8);
        int rc = probe_texture_palette(h->device, hw.data());
        if (rc == TX_EUNSUPPORTED) state = -1;
        else if (rc != TX_OK) { cudaSetDevice(current); return rc; }
        else {
          rc = probe_software_palette(h->device, sw.data(), h->palette);
          if (rc != TX_OK) { cudaSetDevice(current); return rc; }
          state = std::memcmp(hw.data(), sw.data(), hw.size() * sizeof(float)) == 0 ? 1 : 0;
        }
        verdict[key] = state;
      } else {
        state = found->second;
      }
    }
    int rc = TX_OK;
    if (state < 0) rc = fail(TX_EUNSUPPORTED, "signed-BC4 texture views are unavailable on this device");
    else if (state == 0) rc = fail(TX_ESTATE, "model BC4 palette does not match this GPU; the ALU decode path stays in force");
    else rc = create_texture(h);
    cudaSetDevice(current);
    if (rc != TX_OK) return rc;
  }
  h->decode_path = path;
  return TX_OK;
}

int tx_handle_info(uint64_t handle, int64_t out[7]) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  out[0] = h->M;
  out[1] = h->K;
  out[2] = h->prefill_threshold;
  out[3] = h->prefill_tile_rows;
  out[4] = h->prefill_backend;
  out[5] = h->decode_path;
  out[6] = h->lookahead + 16 * h->palette;
  return TX_OK;
}

int tx_kernel_info(int backend, int64_t out[9]) {
  if (!out) return fail(TX_EINVAL, "tx_kernel_info: null output");
  if (backend == 0) return gemv_kernel_info(out);
  if (backend >= 5 && backend <= 9) return prefill_kernel_info(backend, out);
  return fail(TX_EINVAL, "kernel info exists for backend 0 and 5..9");
}

int tx_kernel_status(int device, int clear) {
  Workspace *ws = workspace_for(device);
  if (!ws) return TX_ECUDA;
  int current = 0, value = 0;
  TX_CUDA(cudaGetDevice(&current));
  TX_CUDA(cudaSetDevice(device));
  cudaError_t status = cudaDeviceSynchronize();      // also orders against non-blocking streams, which a plain copy does not
  if (status == cudaSuccess) status = cudaMemcpy(&value, ws->status, sizeof(int), cudaMemcpyDeviceToHost);
  if (status == cudaSuccess && clear && value) status = cudaMemset(ws->status, 0, sizeof(int));
  cudaSetDevice(current);
  if (status != cudaSuccess) return fail(TX_ECUDA, std::string("tx_kernel_status: ") + cudaGetErrorString(status));
  return value;
}

int tx_free(uint64_t handle) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  destroy(h);
  return TX_OK;
}

int tx_palette_probe(int device, float *out_host) {
  if (!out_host) return fail(TX_EINVAL, "tx_palette_probe: null output");
  return probe_texture_palette(device, out_host);
}

int tx_software_palette(int device, float *out_host) {
  if (!out_host) return fail(TX_EINVAL, "tx_software_palette: null output");
  return probe_software_palette(device, out_host, TX_PALETTE_SOFTWARE);
}

int tx_hardware_palette(int device, float *out_host) {
  if (!out_host) return fail(TX_EINVAL, "tx_hardware_palette: null output");
  return probe_software_palette(device, out_host, TX_PALETTE_HARDWARE);
}

int tx_set_palette(uint64_t handle, int palette) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (palette != TX_PALETTE_SOFTWARE && palette != TX_PALETTE_HARDWARE) return fail(TX_EINVAL, "unknown palette");
  if (palette != h->palette && h->decode_path == TX_DECODE_TEXTURE)
    return fail(TX_ESTATE, "leave the texture decode path before changing the palette");
  h->palette = palette;
  return TX_OK;
}

int tx_dequant(uint64_t handle, void *out, int what, void *stream_ptr) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (!out || (reinterpret_cast<uintptr_t>(out) & 15)) return fail(TX_EINVAL, "tx_dequant: output must be 16-byte aligned");
  int current = 0;
  TX_CUDA(cudaGetDevice(&current));
  if (current != h->device) TX_CUDA(cudaSetDevice(h->device));
  int rc = launch_dequant(h, out, what, static_cast<cudaStream_t>(stream_ptr));
  if (current != h->device) cudaSetDevice(current);
  return rc;
}

int tx_unpack_blocks(uint64_t handle, uint8_t *out_host) {
  Handle *h = as_handle(handle);
  if (!h) return fail(TX_EINVAL, "null Texelator handle");
  if (!out_host) return fail(TX_EINVAL, "tx_unpack_blocks: null output");
  int current = 0;
  TX_CUDA(cudaGetDevice(&current));
  TX_CUDA(cudaSetDevice(h->device));
  size_t bytes = size_t(h->M) * h->blocks_per_row * 8;
  uint8_t *linear = nullptr;
  TX_CUDA(cudaMalloc(&linear, bytes));
  int rc = launch_untile(h, linear, 0);
  if (rc == TX_OK) {
    cudaError_t status = cudaMemcpy(out_host, linear, bytes, cudaMemcpyDeviceToHost);
    if (status != cudaSuccess) rc = fail(TX_ECUDA, std::string("cudaMemcpy: ") + cudaGetErrorString(status));
  }
  cudaFree(linear);
  cudaSetDevice(current);
  return rc;
}

}  // extern "C"
