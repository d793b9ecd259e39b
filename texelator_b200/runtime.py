"""Python operator surface of the BC4 weight-linear path.

Mirrors ``texelator/runtime.py`` of the reference (``extension()`` :27-63,
``TexelatorLinear`` :133-145, ``DecodeOnlyLinear`` :148-157, ``pack_entry`` :168-176,
``pack_entry_handles`` :179-207, ``install`` :210-239, ``install_standalone``
:242-263, ``free`` :266-274) with the same names, argument meaning and error
behaviour, but the object returned by ``extension()`` drives the sm_100a C-ABI
library ``texelator_b200/cuda/libtexelator_b200.so`` through ctypes instead of a
pybind11 torch extension.  PyTorch is used for device memory and streams only.

There is no CPU fallback: if the CUDA library is missing and cannot be built,
``extension()`` raises.
"""
from __future__ import annotations

import ctypes
import gc
import json
import os
from pathlib import Path

import numpy as np
import torch
from torch import nn

from .adapters import resolve_parent

PACKAGE_ROOT = Path(__file__).resolve().parent
LIBRARY_PATH = PACKAGE_ROOT / "cuda" / "libtexelator_b200.so"
_EXTENSION = None
PREFILL_THRESHOLD = int(os.environ.get("TEXELATOR_PREFILL_THRESHOLD", "16"))
PREFILL_TILE_ROWS = int(os.environ.get("TEXELATOR_PREFILL_TILE_ROWS", "1024"))

DTYPE_F16, DTYPE_BF16 = 0, 1
DECODE_ALU_MMA, DECODE_ALU_EXACT, DECODE_TEXTURE = 0, 1, 2
DEQUANT_PALETTE_F32, DEQUANT_SCALED_F32, DEQUANT_SCALED_BF16 = 0, 1, 2
PALETTE_SOFTWARE, PALETTE_HARDWARE = 0, 1
TX_EUNSUPPORTED = -3

# every symbol include/texelator_b200.h declares: name -> (restype, argtypes)
_u64, _i32, _i64p = ctypes.c_uint64, ctypes.c_int, ctypes.POINTER(ctypes.c_int64)
_vp, _sz = ctypes.c_void_p, ctypes.c_size_t
C_API = {
    "tx_last_error": (ctypes.c_char_p, []),
    "tx_runtime_info": (_i32, [_i32, _i64p]),
    "tx_pack_encoded": (_i32, [_vp, _sz, _vp, _i32, _vp, _i32, _i32, ctypes.POINTER(_u64)]),
    "tx_pack_encoded_shard": (_i32, [_vp, _sz, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _i32,
                                     ctypes.POINTER(_u64)]),
    "tx_linear": (_i32, [_u64, _vp, _vp, _i32, _i32, _vp]),
    "tx_linear_static_scratch": (_i32, [_u64, _vp, _vp, _i32, _i32, _vp]),
    "tx_linear_fused": (_i32, [_u64, _vp, _vp, _vp, ctypes.c_float, _vp, _i32, _vp, _i32, _i32, _vp]),
    "tx_set_lookahead": (_i32, [_u64, _i32]),
    "tx_set_prefill": (_i32, [_u64, _i32, _i32]),
    "tx_set_prefill_backend": (_i32, [_u64, _i32]),
    "tx_set_decode_path": (_i32, [_u64, _i32]),
    "tx_handle_info": (_i32, [_u64, _i64p]),
    "tx_kernel_info": (_i32, [_i32, _i64p]),
    "tx_free": (_i32, [_u64]),
    "tx_palette_probe": (_i32, [_i32, _vp]),
    "tx_software_palette": (_i32, [_i32, _vp]),
    "tx_hardware_palette": (_i32, [_i32, _vp]),
    "tx_set_palette": (_i32, [_u64, _i32]),
    "tx_dequant": (_i32, [_u64, _vp, _i32, _vp]),
    "tx_unpack_blocks": (_i32, [_u64, _vp]),
    "tx_kernel_status": (_i32, [_i32, _i32]),
    "tx_aux_add_rmsnorm": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, ctypes.c_float, _vp]),
    "tx_aux_rope_append": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "tx_aux_attention_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, ctypes.c_float, _vp]),
    "tx_aux_allreduce_add_rmsnorm": (_i32, [_vp, _vp, _vp, _vp, _i32, ctypes.c_float, _vp, _vp, _i32, _i32, _vp, _vp]),
    "tx_aux_attention_step": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, ctypes.c_float, _vp]),
    "tx_aux_silu_mul": (_i32, [_vp, _vp, _i32, _i32, _vp]),
    "tx_aux_silu_mul_pairs": (_i32, [_vp, _vp, _i32, _i32, _vp]),
    "tx_aux_attention_step_batch": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, ctypes.c_float, _vp]),
    "tx_launch_count": (ctypes.c_int64, []),
    "tx_linear_single": (_i32, [_u64, _vp, _vp, _i32, _vp, _vp, _i32, ctypes.c_size_t, _vp]),
    "tx_linear_single_info": (_i32, [_u64, _vp]),
    "tx_aux_add_rmsnorm_single": (_i32, [_vp, _vp, _vp, _i32, ctypes.c_size_t, _vp, _vp, _vp, _i32, ctypes.c_float, _vp]),
    "tx_encode": (_i32, [_vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp]),
    "tx_linear_single_push": (_i32, [_u64, _vp, _vp, _vp, _i32, _i32, _vp, _vp]),
    "tx_aux_peer_reduce_rmsnorm": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, ctypes.c_float, _vp, _i32, _vp, _vp]),
    "tx_aux_peer_best_token": (_i32, [_vp, _vp, ctypes.c_longlong, _vp, _i32, _i32, _vp, _vp, _vp]),
}


def load_library(path: Path | None = None) -> ctypes.CDLL:
    """dlopen the C-ABI library and bind every declared symbol (raises if one is missing)."""
    library = ctypes.CDLL(str(path or os.environ.get("TEXELATOR_B200_LIBRARY") or LIBRARY_PATH))
    for name, (restype, argtypes) in C_API.items():
        function = getattr(library, name)
        function.restype = restype
        function.argtypes = argtypes
    return library


class _Extension:
    """The module-like object the reference gets from ``extension()``
    (texelator/cuda/extension.cpp:27-48): same function names and semantics."""

    def __init__(self, library: ctypes.CDLL):
        self._lib = library
        self._shapes: dict[int, tuple[int, int, int]] = {}   # handle -> (M, K, device)

    # -- helpers -------------------------------------------------------------
    def _check(self, status: int) -> None:
        if status != 0:
            message = self._lib.tx_last_error().decode(errors="replace")
            raise RuntimeError(message or f"texelator_b200 call failed with status {status}")

    @staticmethod
    def _device_index(device: torch.device | int | None) -> int:
        if device is None:
            return torch.cuda.current_device()
        if isinstance(device, int):
            return device
        return device.index if device.index is not None else torch.cuda.current_device()

    # -- reference surface ---------------------------------------------------
    def pack_encoded(self, blocks: torch.Tensor, scales: torch.Tensor, bias: torch.Tensor | None = None) -> int:
        if blocks.is_cuda or blocks.dtype != torch.uint8 or not blocks.is_contiguous():
            raise RuntimeError("blocks must be contiguous CPU uint8")
        if scales.is_cuda or scales.dtype != torch.float32 or not scales.is_contiguous():
            raise RuntimeError("scales must be contiguous CPU float32")
        m = scales.numel()
        device = torch.cuda.current_device()
        bias_ptr, bias_dtype = self._bias_argument(bias, m, device)
        handle = _u64(0)
        self._check(self._lib.tx_pack_encoded(blocks.data_ptr(), blocks.numel(), scales.data_ptr(), m,
                                              bias_ptr, bias_dtype, device, ctypes.byref(handle)))
        k = 16 * (blocks.numel() // (8 * m))
        self._shapes[handle.value] = (m, k, device)
        return handle.value

    def pack_encoded_device(self, blocks: torch.Tensor, scales: torch.Tensor, bias: torch.Tensor | None = None) -> int:
        """``pack_encoded`` for blocks/scales that already live on the current CUDA device (an
        encoder that runs on the GPU); same layout and semantics otherwise."""
        if not blocks.is_cuda or blocks.dtype != torch.uint8 or not blocks.is_contiguous():
            raise RuntimeError("blocks must be contiguous CUDA uint8")
        if not scales.is_cuda or scales.dtype != torch.float32 or not scales.is_contiguous():
            raise RuntimeError("scales must be contiguous CUDA float32")
        m = scales.numel()
        device = blocks.get_device()
        torch.cuda.current_stream(device).synchronize()
        bias_ptr, bias_dtype = self._bias_argument(bias, m, device)
        handle = _u64(0)
        self._check(self._lib.tx_pack_encoded(blocks.data_ptr(), blocks.numel(), scales.data_ptr(), m,
                                              bias_ptr, bias_dtype, device, ctypes.byref(handle)))
        self._shapes[handle.value] = (m, 16 * (blocks.numel() // (8 * m)), device)
        return handle.value

    def pack_encoded_shard(self, blocks: torch.Tensor, scales: torch.Tensor, m: int, k: int,
                           rows: tuple[int, int], kblocks: tuple[int, int],
                           bias: torch.Tensor | None = None) -> int:
        """Tensor-parallel pack: rows ``[rows[0], rows[1])`` and 16-column blocks
        ``[kblocks[0], kblocks[1])`` of a full ``m x k`` matrix (no reference counterpart)."""
        if blocks.is_cuda or blocks.dtype != torch.uint8 or not blocks.is_contiguous():
            raise RuntimeError("blocks must be contiguous CPU uint8")
        if scales.is_cuda or scales.dtype != torch.float32 or not scales.is_contiguous():
            raise RuntimeError("scales must be contiguous CPU float32")
        device = torch.cuda.current_device()
        bias_ptr, bias_dtype = self._bias_argument(bias, m, device)
        handle = _u64(0)
        self._check(self._lib.tx_pack_encoded_shard(blocks.data_ptr(), blocks.numel(), scales.data_ptr(), m, k,
                                                    rows[0], rows[1], kblocks[0], kblocks[1], bias_ptr, bias_dtype,
                                                    device, ctypes.byref(handle)))
        self._shapes[handle.value] = (rows[1] - rows[0], 16 * (kblocks[1] - kblocks[0]), device)
        return handle.value

    @staticmethod
    def _bias_argument(bias, m, device):
        if bias is None or bias.numel() == 0:
            return None, DTYPE_BF16
        contiguous = bias.detach().contiguous()
        if not contiguous.is_cuda or contiguous.dtype not in (torch.float16, torch.bfloat16) or contiguous.numel() != m:
            raise RuntimeError("bias must be CUDA FP16 or BF16 [M]")
        # keep the tensor alive until the (synchronous) copy inside the call is done
        _Extension._bias_keepalive = contiguous
        return contiguous.data_ptr(), (DTYPE_BF16 if contiguous.dtype == torch.bfloat16 else DTYPE_F16)

    def _activation(self, handle: int, x: torch.Tensor) -> tuple[int, int, int, int]:
        """The checks of texelator_cuda.cu:1332-1337 on an activation tensor; returns (M, K, device, tokens)."""
        shape = self._shapes.get(handle)
        if shape is None:
            raise RuntimeError("null Texelator handle")
        m, k, device = shape
        if not x.is_cuda or x.dtype not in (torch.float16, torch.bfloat16) or not x.is_contiguous():
            raise RuntimeError("input must be contiguous CUDA FP16 or BF16")
        if x.size(-1) != k or x.get_device() != device:
            raise RuntimeError("input shape/device mismatch")
        return m, k, device, x.numel() // k

    @staticmethod
    def _dtype_flag(x: torch.Tensor) -> int:
        return DTYPE_BF16 if x.dtype == torch.bfloat16 else DTYPE_F16

    def linear(self, handle: int, x: torch.Tensor) -> torch.Tensor:
        m, k, device, tokens = self._activation(handle, x)
        y = torch.empty(x.shape[:-1] + (m,), dtype=x.dtype, device=x.device)
        if tokens:
            self._check(self._lib.tx_linear(handle, x.data_ptr(), y.data_ptr(), tokens, self._dtype_flag(x),
                                            torch.cuda.current_stream(device).cuda_stream))
        return y

    def linear_out(self, handle: int, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        """``linear`` into a caller-provided output (static buffers for CUDA graphs)."""
        m, k, device, tokens = self._activation(handle, x)
        if y.numel() != tokens * m or y.dtype != x.dtype or not y.is_contiguous() or y.device != x.device:
            raise RuntimeError("input shape/device mismatch")
        self._check(self._lib.tx_linear(handle, x.data_ptr(), y.data_ptr(), tokens, self._dtype_flag(x),
                                        torch.cuda.current_stream(device).cuda_stream))
        return y

    def linear_static_scratch(self, handle: int, x: torch.Tensor) -> torch.Tensor:
        """``linear`` for a small token group through the entry point that allocates nothing on the
        device: its activation scratch is a fixed array inside the library (for callers whose memory
        is all in their own pool, or who must not take the allocator lock).  Raises for requests beyond
        32 tokens or 262144 activation values.  Calls on one device must not overlap on the GPU."""
        m, k, device = self._shapes[handle]
        if not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.size(-1) != k:
            raise RuntimeError("input must be contiguous CUDA BF16 [..., K]")
        y = torch.empty(x.shape[:-1] + (m,), dtype=x.dtype, device=x.device)
        stream = torch.cuda.current_stream(device).cuda_stream
        self._check(self._lib.tx_linear_static_scratch(handle, x.data_ptr(), y.data_ptr(), x.numel() // k, DTYPE_BF16, stream))
        return y

    def linear_fused_out(self, handle: int, x: torch.Tensor, y: torch.Tensor, *, norm_weight: torch.Tensor | None = None,
                         delta: torch.Tensor | None = None, eps: float = 1e-6, residual_out: torch.Tensor | None = None,
                         swiglu: bool = False) -> None:
        """Decode linear with fused neighbours, written into ``y``: with ``norm_weight`` the input is the
        residual stream (``x + delta`` is rounded to bf16, stored to ``residual_out`` and RMS-normalised
        first); with ``swiglu`` the handle's rows are (gate, up) pairs (``interleave_gate_up`` order) and
        ``y`` is ``[tokens, M/2]``.  At most two tokens."""
        m, k, device, tokens = self._activation(handle, x)
        for tensor in (x, y, norm_weight, delta, residual_out):
            if tensor is not None and (not tensor.is_cuda or tensor.dtype != torch.bfloat16 or not tensor.is_contiguous()
                                       or tensor.get_device() != device):
                raise RuntimeError("fused linear tensors must be contiguous CUDA BF16 on the handle's device")
        if y.numel() != tokens * (m // 2 if swiglu else m):
            raise RuntimeError("output has the wrong size for this handle")
        ptr = lambda t: t.data_ptr() if t is not None else None
        self._check(self._lib.tx_linear_fused(handle, x.data_ptr(), ptr(delta), ptr(norm_weight), float(eps), ptr(residual_out),
                                              int(swiglu), y.data_ptr(), tokens, DTYPE_BF16,
                                              torch.cuda.current_stream(device).cuda_stream))

    def set_lookahead(self, handle: int, lookahead: int) -> None:
        self._check(self._lib.tx_set_lookahead(handle, int(lookahead)))

    def set_prefill(self, handle: int, threshold: int, tile_rows: int) -> None:
        self._check(self._lib.tx_set_prefill(handle, int(threshold), int(tile_rows)))

    def set_prefill_backend(self, handle: int, backend: int) -> None:
        self._check(self._lib.tx_set_prefill_backend(handle, int(backend)))

    def handle_info(self, handle: int) -> list[int]:
        out = (ctypes.c_int64 * 7)()
        self._check(self._lib.tx_handle_info(handle, out))
        return list(out)

    def kernel_info(self, backend: int) -> list[int]:
        out = (ctypes.c_int64 * 9)()
        self._check(self._lib.tx_kernel_info(int(backend), out))
        return list(out)

    # the reference exposes one info function per tile (extension.cpp:36-42)
    def cutlass_texture_kernel_info(self) -> list[int]:
        return self.kernel_info(5)

    def cutlass_t1_kernel_info(self) -> list[int]:
        return self.kernel_info(6)

    def cutlass_t2_kernel_info(self) -> list[int]:
        return self.kernel_info(7)

    def cutlass_t3_kernel_info(self) -> list[int]:
        return self.kernel_info(8)

    def cutlass_smalln_kernel_info(self) -> list[int]:
        return self.kernel_info(9)

    def free(self, handle: int) -> None:
        self._shapes.pop(handle, None)
        self._check(self._lib.tx_free(handle))

    def palette_probe(self) -> torch.Tensor:
        """CPU float32 ``[65025, 8]``, row ``(e1+127)*255 + (e0+127)`` measured through a
        signed-BC4 CUDA texture (texelator_cuda.cu:1540-1595).  Raises when the device has no
        BC4 texture views."""
        out = torch.empty((255 * 255, 8), dtype=torch.float32)
        self._check(self._lib.tx_palette_probe(torch.cuda.current_device(), out.data_ptr()))
        return out

    # -- additions -----------------------------------------------------------
    def software_palette(self) -> torch.Tensor:
        """The same table produced by the library's ALU decoder."""
        out = torch.empty((255 * 255, 8), dtype=torch.float32)
        self._check(self._lib.tx_software_palette(torch.cuda.current_device(), out.data_ptr()))
        return out

    def hardware_palette(self) -> torch.Tensor:
        """The ALU decoder's table for the texture-unit palette (closed form)."""
        out = torch.empty((255 * 255, 8), dtype=torch.float32)
        self._check(self._lib.tx_hardware_palette(torch.cuda.current_device(), out.data_ptr()))
        return out

    def set_palette(self, handle: int, palette: int) -> None:
        """Declare the palette the handle's payload was encoded against (``PALETTE_*``)."""
        self._check(self._lib.tx_set_palette(handle, int(palette)))

    def texture_supported(self) -> bool:
        return bool(self.runtime_info()[3])

    def runtime_info(self, device: int | None = None) -> list[int]:
        out = (ctypes.c_int64 * 4)()
        self._check(self._lib.tx_runtime_info(self._device_index(device), out))
        return list(out)

    def set_decode_path(self, handle: int, path: int) -> None:
        self._check(self._lib.tx_set_decode_path(handle, int(path)))

    def dequant(self, handle: int, what: int = DEQUANT_SCALED_BF16) -> torch.Tensor:
        m, k, device = self._shapes[handle]
        dtype = torch.bfloat16 if what == DEQUANT_SCALED_BF16 else torch.float32
        out = torch.empty((m, k), dtype=dtype, device=torch.device("cuda", device))
        stream = torch.cuda.current_stream(device).cuda_stream
        self._check(self._lib.tx_dequant(handle, out.data_ptr(), int(what), stream))
        return out

    def unpack_blocks(self, handle: int) -> torch.Tensor:
        m, k, _ = self._shapes[handle]
        out = torch.empty(m * k // 2, dtype=torch.uint8)
        self._check(self._lib.tx_unpack_blocks(handle, out.data_ptr()))
        return out

    # -- decode-loop glue kernels (see include/texelator_b200.h) ----------------
    @staticmethod
    def _stream(tensor: torch.Tensor) -> int:
        return torch.cuda.current_stream(tensor.device).cuda_stream

    def add_rmsnorm(self, h: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, y: torch.Tensor, eps: float) -> None:
        tokens, hidden = h.shape
        self._check(self._lib.tx_aux_add_rmsnorm(h.data_ptr(), delta.data_ptr() if delta is not None else None,
                                                 weight.data_ptr(), y.data_ptr(), tokens, hidden, eps, self._stream(h)))

    def rope_append(self, qkv, cos, sin, position, k_cache, v_cache, q_heads: int, kv_heads: int, head_dim: int) -> None:
        self._check(self._lib.tx_aux_rope_append(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), position.data_ptr(),
                                                 k_cache.data_ptr(), v_cache.data_ptr(), q_heads, kv_heads, head_dim,
                                                 k_cache.shape[1], self._stream(qkv)))

    def attention_decode(self, qkv, k_cache, v_cache, position, scratch, out, q_heads: int, kv_heads: int, head_dim: int) -> None:
        self._check(self._lib.tx_aux_attention_decode(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), position.data_ptr(),
                                                      scratch.data_ptr(), out.data_ptr(), q_heads, kv_heads, head_dim,
                                                      k_cache.shape[1], float(head_dim) ** -0.5, self._stream(qkv)))

    def allreduce_add_rmsnorm(self, h: torch.Tensor, partial: torch.Tensor, weight: torch.Tensor, y: torch.Tensor, eps: float,
                              peers) -> None:
        """``h += all_reduce(partial)``; ``y = rmsnorm(h) * weight`` for one token in one launch; ``peers`` is a
        ``tp.PeerExchange`` (peer-mapped inboxes and flags of all ranks)."""
        if h.numel() != weight.numel() or partial.numel() != h.numel():
            raise RuntimeError("fused all-reduce handles exactly one token")
        self._check(self._lib.tx_aux_allreduce_add_rmsnorm(h.data_ptr(), partial.data_ptr(), weight.data_ptr(), y.data_ptr(),
                                                           h.numel(), float(eps), peers.inbox_ptrs, peers.flag_ptrs, peers.rank,
                                                           peers.world, peers.epoch.data_ptr(), self._stream(h)))

    @staticmethod
    def attention_step_scratch_floats(q_heads: int, max_len: int) -> int:
        """Size of the fp32 scratch ``attention_step`` needs for caches of ``max_len`` positions."""
        return q_heads * ((max_len + 63) // 64) * 132

    def attention_step(self, qkv, cos, sin, position, k_cache, v_cache, scratch, out, q_heads: int, kv_heads: int,
                       head_dim: int) -> None:
        """RoPE + cache append + single-query attention + split merge of one token in one launch."""
        if scratch.numel() < self.attention_step_scratch_floats(q_heads, k_cache.shape[1]):
            raise ValueError("attention_step scratch is too small for this cache length")
        self._check(self._lib.tx_aux_attention_step(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), position.data_ptr(),
                                                    k_cache.data_ptr(), v_cache.data_ptr(), scratch.data_ptr(), out.data_ptr(),
                                                    q_heads, kv_heads, head_dim, k_cache.shape[1], float(head_dim) ** -0.5,
                                                    self._stream(qkv)))

    def attention_step_batch(self, qkv, cos, sin, positions, k_cache, v_cache, scratch, out, q_heads: int, kv_heads: int,
                             head_dim: int) -> None:
        """``attention_step`` for one token of each sequence of a batch in one launch: ``qkv [B, ...]``, ``positions``
        int64 ``[B]``, caches ``[B, kv_heads, max_len, head_dim]``, ``out [B, q_heads * head_dim]``."""
        sequences, max_len = k_cache.shape[0], k_cache.shape[2]
        if qkv.shape[0] != sequences or positions.numel() != sequences or not (k_cache.is_contiguous() and v_cache.is_contiguous()):
            raise ValueError("attention_step_batch: one qkv row, one position and one contiguous cache per sequence")
        if scratch.numel() < sequences * self.attention_step_scratch_floats(q_heads, max_len):
            raise ValueError("attention_step scratch is too small for this batch and cache length")
        self._check(self._lib.tx_aux_attention_step_batch(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), positions.data_ptr(),
                                                          k_cache.data_ptr(), v_cache.data_ptr(), scratch.data_ptr(), out.data_ptr(),
                                                          sequences, q_heads, kv_heads, head_dim, max_len, float(head_dim) ** -0.5,
                                                          self._stream(qkv)))

    def silu_mul_pairs(self, gate_up: torch.Tensor, out: torch.Tensor) -> None:
        """``silu_mul`` for rows in ``interleave_gate_up`` order (gate and up rows in alternating groups of eight)."""
        tokens, two_i = gate_up.shape
        self._check(self._lib.tx_aux_silu_mul_pairs(gate_up.data_ptr(), out.data_ptr(), tokens, two_i // 2, self._stream(gate_up)))

    def silu_mul(self, gate_up: torch.Tensor, out: torch.Tensor) -> None:
        tokens, two_i = gate_up.shape
        self._check(self._lib.tx_aux_silu_mul(gate_up.data_ptr(), out.data_ptr(), tokens, two_i // 2, self._stream(gate_up)))

    def encode(self, weight: torch.Tensor, hdiag: torch.Tensor, lut: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """The reference's E3 encoder (``encode_linear_e3``, texelator/encoder.py:120-157) on the GPU, byte-identical:
        CUDA fp32 ``weight [M, K]``, ``hdiag [K]``, ``lut [255, 255, 8]`` -> (uint8 blocks ``[M*K/2]``, fp32 scales ``[M]``)."""
        if not (weight.is_cuda and hdiag.is_cuda and lut.is_cuda) or weight.dim() != 2:
            raise RuntimeError("encode needs CUDA tensors: weight [M, K], hdiag [K], lut [255, 255, 8]")
        m, k = weight.shape
        if hdiag.numel() != k or lut.numel() != 255 * 255 * 8:
            raise RuntimeError("encode: hdiag must have K elements and lut 255*255*8")
        weight, hdiag, lut = weight.float().contiguous(), hdiag.float().contiguous(), lut.float().contiguous()
        blocks = torch.empty(m * k // 2, dtype=torch.uint8, device=weight.device)
        scales = torch.empty(m, dtype=torch.float32, device=weight.device)
        with torch.cuda.device(weight.device):
            self._check(self._lib.tx_encode(weight.data_ptr(), hdiag.data_ptr(), lut.data_ptr(), m, k, blocks.data_ptr(),
                                            scales.data_ptr(), self._stream(weight)))
        return blocks, scales

    def linear_single_info(self, handle: int) -> tuple[bool, int, int]:
        """(eligible for the single-token kernel, suggested K splits, bytes of a staged token)."""
        out = (ctypes.c_int64 * 3)()
        self._check(self._lib.tx_linear_single_info(handle, out))
        return bool(out[0]), int(out[1]), int(out[2])

    def linear_single(self, handle: int, x: torch.Tensor | None, y: torch.Tensor | None, *, staged: torch.Tensor | None = None,
                      swiglu: bool = False, partials: torch.Tensor | None = None) -> None:
        """One token through the single-token decode kernel: input ``x`` (bf16 ``[1, K]``) or ``staged``
        (uint8 buffer written by ``add_rmsnorm_single``); output ``y`` (bf16) or ``partials`` (fp32
        ``[splits, stride]``)."""
        source = next((t for t in (x, staged, y, partials) if t is not None), None)
        if source is None:
            raise RuntimeError("pass the token either as bf16 or in staged form")
        splits, stride = (partials.shape[0], partials.stride(0)) if partials is not None else (1, 0)
        self._check(self._lib.tx_linear_single(handle, x.data_ptr() if x is not None else None,
                                               staged.data_ptr() if staged is not None else None, int(swiglu),
                                               y.data_ptr() if y is not None else None,
                                               partials.data_ptr() if partials is not None else None, splits, stride,
                                               self._stream(source)))

    def add_rmsnorm_single(self, h: torch.Tensor, weight: torch.Tensor, eps: float, *, delta: torch.Tensor | None = None,
                           partials: torch.Tensor | None = None, y: torch.Tensor | None = None,
                           staged: torch.Tensor | None = None) -> None:
        """``h += delta`` (bf16 ``delta`` or fp32 ``partials [splits, stride]``); ``y`` / ``staged`` = rmsnorm(h) * weight."""
        splits, stride = (partials.shape[0], partials.stride(0)) if partials is not None else (0, 0)
        self._check(self._lib.tx_aux_add_rmsnorm_single(h.data_ptr(), delta.data_ptr() if delta is not None else None,
                                                        partials.data_ptr() if partials is not None else None, splits, stride,
                                                        weight.data_ptr(), y.data_ptr() if y is not None else None,
                                                        staged.data_ptr() if staged is not None else None, h.numel(), float(eps),
                                                        self._stream(h)))

    def linear_single_push(self, handle: int, x: torch.Tensor | None, peers, *, staged: torch.Tensor | None = None) -> None:
        """Row-parallel linear of one token whose bf16 partial row goes straight into every rank's packet
        inbox (``peers``: a ``tp.PeerExchange``)."""
        source = x if x is not None else staged
        self._check(self._lib.tx_linear_single_push(handle, x.data_ptr() if x is not None else None,
                                                    staged.data_ptr() if staged is not None else None, peers.packet_ptrs,
                                                    peers.rank, peers.world, peers.packet_epoch.data_ptr(), self._stream(source)))

    def peer_reduce_rmsnorm(self, h: torch.Tensor, weight: torch.Tensor, eps: float, *, peers=None, delta: torch.Tensor | None = None,
                            y: torch.Tensor | None = None, staged: torch.Tensor | None = None) -> None:
        """``h += sum over ranks of the packets in this rank's inbox`` (``peers`` given) or ``h += delta``;
        ``y`` / ``staged`` = rmsnorm(h) * weight.  One thread-block cluster."""
        self._check(self._lib.tx_aux_peer_reduce_rmsnorm(
            h.data_ptr(), delta.data_ptr() if delta is not None else None, weight.data_ptr(),
            y.data_ptr() if y is not None else None, staged.data_ptr() if staged is not None else None, h.numel(), float(eps),
            peers.packet_inbox.data_ptr() if peers is not None else None, peers.world if peers is not None else 0,
            peers.packet_epoch.data_ptr() if peers is not None else None, self._stream(h)))

    def peer_best_token(self, score: torch.Tensor, token: torch.Tensor, offset: int, peers, next_token: torch.Tensor) -> None:
        """Vocabulary-parallel arg-max: this rank's (score fp32, token int64 + offset) against all ranks'."""
        self._check(self._lib.tx_aux_peer_best_token(score.data_ptr(), token.data_ptr(), int(offset), peers.token_ptrs, peers.rank,
                                                     peers.world, peers.token_epoch.data_ptr(), next_token.data_ptr(),
                                                     self._stream(score)))

    def kernel_status(self, clear: bool = False, device: int | None = None) -> int:
        """0 when no kernel of this library ever gave up on a bounded wait on this device."""
        value = self._lib.tx_kernel_status(self._device_index(device), int(clear))
        if value < 0:
            self._check(value)
        return value

    def launch_count(self) -> int:
        return int(self._lib.tx_launch_count())


def extension(verbose: bool = False):
    """Load (building in-tree with nvcc if needed) the CUDA library.  Like the reference
    (runtime.py:27-63) this raises instead of degrading when no native code is available;
    ``TEXELATOR_DISABLE_JIT`` forbids the nvcc build."""
    global _EXTENSION
    if _EXTENSION is None:
        if not LIBRARY_PATH.exists():
            if os.environ.get("TEXELATOR_DISABLE_JIT", "").upper() in {"1", "ON", "YES", "TRUE"}:
                raise RuntimeError(
                    "the prebuilt Texelator CUDA library is unavailable and JIT compilation is disabled")
            from .cuda.build import build
            build(verbose=verbose)
        try:
            _EXTENSION = _Extension(load_library())
        except (OSError, AttributeError) as error:
            raise RuntimeError(f"the Texelator CUDA library could not be loaded: {error}") from error
    return _EXTENSION


class TexelatorLinear(nn.Module):
    """Drop-in for an ``nn.Linear`` whose weight lives in one or more BC4 handles (the reference's module of
    the same name, texelator/runtime.py:133-145; it splits outputs taller than a texture allows into
    several handles, and lists of handles keep that shape here).  Each handle yields a slice of the output
    features; ``bias`` is only used when the handles themselves carry none."""

    def __init__(self, handles: list[int], bias: nn.Parameter | None = None):
        super().__init__()
        if not handles:
            raise ValueError("TexelatorLinear requires at least one texture handle")
        self.handles = list(handles)
        self.bias = bias

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ext = extension()
        x = x.contiguous()
        if len(self.handles) == 1:
            y = ext.linear(self.handles[0], x)
        else:
            y = torch.cat([ext.linear(handle, x) for handle in self.handles], dim=-1)
        return y if self.bias is None else y + self.bias


class DecodeOnlyLinear(nn.Module):
    """Single-token calls go to the BC4 module, everything else to the dense original
    (texelator/runtime.py:148-157: the opt-in "fp16 prefill" mode)."""

    def __init__(self, original: nn.Module, quantized: nn.Module):
        super().__init__()
        self.original = original
        self.quantized = quantized

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        one_token = x.numel() == x.shape[-1]
        return (self.quantized if one_token else self.original)(x)


def palette_of(weights: Path) -> int:
    """Which palette the artefact under ``weights`` was encoded against, from the ``palette_sha256`` its
    ``metadata.json`` records (texelator/converter.py:204): the published texture-unit hash selects
    ``PALETTE_HARDWARE``, anything else the software palette (the tuner's gate still checks the hash)."""
    from .hardware import REFERENCE_TEXTURE_PALETTE_SHA256
    try:
        recorded = json.loads((Path(weights) / "metadata.json").read_text()).get("palette_sha256")
    except (OSError, ValueError):
        recorded = None
    return PALETTE_HARDWARE if recorded == REFERENCE_TEXTURE_PALETTE_SHA256 else PALETTE_SOFTWARE


class _EncodedMatrix:
    """The two files of one ``metadata.json`` entry (``<key>.bc4`` row-major blocks, ``<key>.scales.f32``),
    memory-mapped, handed out as row slabs."""

    def __init__(self, weights: Path, entry: dict):
        self.m, self.k = int(entry["M"]), int(entry["K"])
        self.blocks = np.memmap(Path(weights) / entry["blocks_file"], dtype=np.uint8, mode="r", shape=(self.m, self.k // 2))
        self.scales = np.memmap(Path(weights) / entry["scales_file"], dtype="<f4", mode="r", shape=(self.m,))

    def slabs(self, rows: int):
        for first in range(0, self.m, rows):
            last = min(first + rows, self.m)
            yield (first, last, torch.from_numpy(np.array(self.blocks[first:last]).reshape(-1)),
                   torch.from_numpy(np.array(self.scales[first:last])))


def pack_entry_handles(weights: Path, entry: dict, bias: torch.Tensor | None = None, lookahead: int = 1,
                       max_texture_rows: int = 32768, palette: int | None = None) -> list[int]:
    """Handles for one encoded matrix, one per slab of ``max_texture_rows`` output rows (the reference
    splits at the texture height limit, texelator/runtime.py:179-207; the split is kept so that handle
    lists look the same).  Every handle gets the look-ahead, the default prefill settings and the palette
    the artefact was encoded against."""
    if max_texture_rows <= 0:
        raise ValueError("max_texture_rows must be positive")
    ext = extension()
    palette = palette_of(weights) if palette is None else palette
    handles: list[int] = []
    try:
        for first, last, blocks, scales in _EncodedMatrix(weights, entry).slabs(max_texture_rows):
            handle = ext.pack_encoded(blocks, scales, None if bias is None else bias[first:last])
            handles.append(handle)
            ext.set_lookahead(handle, lookahead)
            ext.set_prefill(handle, PREFILL_THRESHOLD, PREFILL_TILE_ROWS)
            ext.set_palette(handle, palette)
    except Exception:
        free(handles)
        raise
    return handles


def pack_entry(weights: Path, entry: dict, bias: torch.Tensor | None = None, lookahead: int = 1) -> int:
    """One handle for the whole matrix (texelator/runtime.py:168-176)."""
    return pack_entry_handles(weights, entry, bias, lookahead, max_texture_rows=int(entry["M"]))[0]


def _swap_linears(model: nn.Module, weights: Path, entries: list[dict], lookahead: int, locate, wrap) -> list[int]:
    """Pack every entry and put ``wrap(original, handles)`` in the place ``locate(entry)`` names; on any
    failure the handles made so far are released."""
    handles: list[int] = []
    try:
        for entry in entries:
            parent, child = resolve_parent(model, locate(entry))
            original = getattr(parent, child)
            made = wrap(original, entry)
            setattr(parent, child, made[0])
            handles.extend(made[1])
    except Exception:
        free(handles)
        raise
    model._texelator_handles = handles
    return handles


def install(model: nn.Module, weights: Path, lookahead: int = 1, fp16_prefill: bool = False) -> list[int]:
    """Replace the linears listed in ``weights/metadata.json`` of a CUDA-resident model
    (texelator/runtime.py:210-239).  The handles take over the original bias."""
    weights = Path(weights)

    def wrap(original, entry):
        device = original.weight.device
        if device.type != "cuda":
            raise RuntimeError(f"{entry['module_name']} is on {device}; selected linears must be CUDA resident")
        with torch.cuda.device(device):
            made = pack_entry_handles(weights, entry, bias=getattr(original, "bias", None), lookahead=lookahead)
        module = TexelatorLinear(made)
        return (DecodeOnlyLinear(original, module) if fp16_prefill else module), made

    handles = _swap_linears(model, weights, json.loads((weights / "metadata.json").read_text())["entries"], lookahead,
                            lambda entry: entry["module_name"], wrap)
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return handles


def install_standalone(model: nn.Module, weights: Path, entries: list[dict], name_mapper, lookahead: int = 1) -> list[int]:
    """Replace meta-initialised linears that never had dense weights (texelator/runtime.py:242-263); the
    bias stays a module parameter because it is loaded after the handles are made."""
    weights = Path(weights)

    def wrap(original, entry):
        made = pack_entry_handles(weights, entry, lookahead=lookahead)
        return TexelatorLinear(made, bias=getattr(original, "bias", None)), made

    return _swap_linears(model, weights, entries, lookahead, lambda entry: name_mapper(entry["module_name"]), wrap)


def free(handles: list[int]) -> None:
    """Release handles after the device has finished with them (texelator/runtime.py:266-274)."""
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    ext = extension()
    for handle in handles:
        ext.free(handle)
