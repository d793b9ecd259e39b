"""CPU restatement of the reference's BC4 weight-linear arithmetic.

TEST INFRASTRUCTURE ONLY -- see ``oracle/__init__.py``.  The product never
imports this module.

Every function cites the reference file:line (paths inside the hp0303/Texelator
tree) whose behaviour it restates.  The restatement is pinned two ways:

* ``tests/golden/*.npz`` were produced by ``tests/golden/make_golden.py``, which
  imports the reference's own ``texelator/encoder.py`` and records its outputs
  on seeded inputs; ``tests/test_oracle.py`` replays them against this file.
* The reference ships no golden vectors and no palette file for this path (its
  palette is measured on a GPU texture unit at install time), so the palette
  here is the *software* BC4-SNORM palette defined in ``software_palette``.
"""
from __future__ import annotations

import hashlib

import numpy as np

# Remapped interpolation index g(s) for the two BC4 modes.
# texelator/encoder.py:53-70 -- selector 0 -> endpoint0, 1 -> endpoint1,
# 2..7 -> ((8-s)*E0+(s-1)*E1)/7 when e0>e1, else 2..5 -> ((6-s)*E0+(s-1)*E1)/5,
# 6 -> -1, 7 -> +1.
G8 = np.array([0, 7, 1, 2, 3, 4, 5, 6], dtype=np.int32)
G6 = np.array([0, 5, 1, 2, 3, 4, 0, 0], dtype=np.int32)
DEN8 = 7 * 127
DEN6 = 5 * 127


def software_palette() -> np.ndarray:
    """The software BC4-SNORM palette as the ``[255, 255, 8]`` fp32 table the
    reference encoder indexes as ``lut[e1 + 127, e0 + 127, selector]``
    (texelator/encoder.py:11-20; row order of the probe,
    texelator/cuda/texelator_cuda.cu:1542-1564).

    Each entry is the exact rational BC4-SNORM value rounded once to fp32:
    ``((7-g)*e0 + g*e1) / 889`` for ``e0 > e1`` and ``((5-g)*e0 + g*e1) / 635``
    otherwise (selectors 6/7 give -1/+1 there).  Numerators are exact integers,
    so one IEEE division defines every entry without op-order ambiguity.
    """
    e = np.arange(-127, 128, dtype=np.int32)
    e0 = e[None, :, None]
    e1 = e[:, None, None]
    n8 = (7 - G8)[None, None, :] * e0 + G8[None, None, :] * e1
    n6 = (5 - G6)[None, None, :] * e0 + G6[None, None, :] * e1
    p8 = n8.astype(np.float32) / np.float32(DEN8)
    p6 = n6.astype(np.float32) / np.float32(DEN6)
    p6[:, :, 6] = -1.0
    p6[:, :, 7] = 1.0
    return np.where(e0 > e1, p8, p6).astype(np.float32)


# SHA-256 of the texture-unit palette the reference publishes for RTX 4060 / 4080 SUPER / 5080
# (WINDOWS_VALIDATION.md:13-14; research/results/paper/environment.json:32-36).
REFERENCE_TEXTURE_PALETTE_SHA256 = "34670bd1c521c26b14ea88ed6f2d8f16c55720f20915909ac621dcabe0f3ed47"


def hardware_palette() -> np.ndarray:
    """The palette NVIDIA texture units produce for signed BC4 (what the reference measures with
    texelator/cuda/texelator_cuda.cu:1540-1595 and encodes its published models against), as a
    closed form.  Endpoints are widened to 16-bit snorm by bit replication,
    ``X(e) = sign(e) * ((|e|<<8) | (|e|<<1) | (|e|>>6))``; interpolated entries add integer multiples
    of ``d = e1 - e0`` to the nearer endpoint (36, 72, 144 in the 8-value mode; 48, 96 in the 6-value
    mode); the result is ``I / 32767`` rounded to fp32.  The table reproduces the published SHA-256
    bit for bit (``REFERENCE_TEXTURE_PALETTE_SHA256``) and equals what a B200 returns."""
    e = np.arange(-127, 128, dtype=np.int64)
    mag = np.abs(e)
    wide = np.sign(e) * ((mag << 8) | (mag << 1) | (mag >> 6))
    x0 = np.broadcast_to(wide[None, :], (255, 255))
    x1 = np.broadcast_to(wide[:, None], (255, 255))
    d = e[:, None] - e[None, :]
    high = [x0, x1, x0 + 36 * d, x0 + 72 * d, x1 - 144 * d, x0 + 144 * d, x1 - 72 * d, x1 - 36 * d]
    low = [x0, x1, x0 + 48 * d, x0 + 96 * d, x1 - 96 * d, x1 - 48 * d,
           np.full((255, 255), -32767), np.full((255, 255), 32767)]
    table = np.where((e[None, :] > e[:, None])[:, :, None], np.stack(high, -1), np.stack(low, -1))
    return (table.astype(np.float64) / 32767.0).astype(np.float32)


def palette_sha256(lut: np.ndarray) -> str:
    """SHA-256 of ``palette.bin`` (65 025 x 8 little-endian fp32) -- the value
    the reference compares in texelator/tuning.py:38-41 and
    texelator/artifacts.py:16-21."""
    return hashlib.sha256(np.ascontiguousarray(lut, dtype="<f4").tobytes()).hexdigest()


def unpack_blocks(blocks: np.ndarray, rows: int):
    """Inverse of ``pack_blocks`` (texelator/encoder.py:105-117).

    ``blocks`` is the raw ``<key>.bc4`` byte stream: per output row ``K/16``
    blocks of 8 bytes -- int8 endpoint0, int8 endpoint1, 48-bit little-endian
    selector word with weight ``p`` at bits ``3p..3p+2``.  Returns
    ``(e0, e1, sel)`` shaped ``[rows, K/16]``, ``[rows, K/16]``,
    ``[rows, K/16, 16]``.
    """
    raw = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(rows, -1, 8)
    e0 = raw[:, :, 0].view(np.int8).astype(np.int32)
    e1 = raw[:, :, 1].view(np.int8).astype(np.int32)
    word = np.zeros(raw.shape[:2], dtype=np.uint64)
    for byte in range(6):
        word |= raw[:, :, 2 + byte].astype(np.uint64) << np.uint64(8 * byte)
    shifts = (3 * np.arange(16, dtype=np.uint64))[None, None, :]
    sel = ((word[:, :, None] >> shifts) & np.uint64(7)).astype(np.int32)
    return e0, e1, sel


def pack_blocks(e0: np.ndarray, e1: np.ndarray, sel: np.ndarray) -> np.ndarray:
    """Byte layout of texelator/encoder.py:105-117 from ``[n]`` endpoints and
    ``[n, 16]`` selectors; returns ``[n, 8]`` uint8."""
    e0 = np.asarray(e0).reshape(-1)
    e1 = np.asarray(e1).reshape(-1)
    sel = np.asarray(sel).reshape(-1, 16).astype(np.uint64)
    word = np.zeros(sel.shape[0], dtype=np.uint64)
    for p in range(16):
        word |= sel[:, p] << np.uint64(3 * p)
    out = np.empty((sel.shape[0], 8), dtype=np.uint8)
    out[:, 0] = e0.astype(np.int8).view(np.uint8)
    out[:, 1] = e1.astype(np.int8).view(np.uint8)
    for byte in range(6):
        out[:, 2 + byte] = ((word >> np.uint64(8 * byte)) & np.uint64(255)).astype(np.uint8)
    return out


def palette_values(lut: np.ndarray, e0: np.ndarray, e1: np.ndarray, sel: np.ndarray) -> np.ndarray:
    """``lut[e1+127, e0+127][sel]`` (texelator/encoder.py:19-20,31).  An
    endpoint of -128 is read as -127, the BC4-SNORM rule the texture unit
    applies; the reference encoder never emits it (encoder.py:48-49,92-93)."""
    i0 = np.maximum(e0, -127) + 127
    i1 = np.maximum(e1, -127) + 127
    pal = lut[i1, i0]                                  # [..., 8]
    return np.take_along_axis(pal, sel.astype(np.int64), axis=-1)


def dequant_palette(blocks: np.ndarray, rows: int, lut: np.ndarray) -> np.ndarray:
    """Unscaled reconstructed weights ``[rows, K]`` fp32 (what the texture unit
    returns per texel, texelator/cuda/texelator_cuda.cu:85-90)."""
    e0, e1, sel = unpack_blocks(blocks, rows)
    return palette_values(lut, e0, e1, sel).reshape(rows, -1).astype(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 (round to nearest even) -> fp32, i.e. ``__float2bfloat16``
    followed by ``__bfloat162float`` (texelator_cuda.cu:141-152)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    rounded = (bits + np.uint64(0x7FFF) + ((bits >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)
    out = (rounded.astype(np.uint32) << np.uint32(16)).view(np.float32)
    nan = np.isnan(x)
    if nan.any():
        out = out.copy()
        out[nan] = np.nan
    return out


def dequant_weights(blocks: np.ndarray, scales: np.ndarray, lut: np.ndarray,
                    round_bf16: bool = True) -> np.ndarray:
    """The matrix the reference multiplies by: ``pal * scale_m`` in fp32, then
    rounded to bf16 for the bf16 operator (texelator_cuda.cu:141-152;
    cutlass_texture_mainloop.cu:162-170).  Returns fp32 ``[M, K]``."""
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    q = dequant_palette(blocks, scales.shape[0], lut) * scales[:, None]
    return bf16_round(q) if round_bf16 else q.astype(np.float32)


def linear_bf16(x_bf16_as_f32: np.ndarray, blocks: np.ndarray, scales: np.ndarray,
                lut: np.ndarray, bias: np.ndarray | None = None,
                bias_after_store: bool = False) -> np.ndarray:
    """Dequantise-then-matmul oracle for the bf16 operator.

    ``y = bf16( sum_k f32(bf16(pal*scale)) * f32(x) + f32(bias) )`` -- the decode
    GEMV contract (texelator_cuda.cu:141-199).  With ``bias_after_store`` the
    bias is added after a first bf16 store and rounded again, which is what the
    reference's tensor-core prefill does (cutlass_texture_mainloop.cu:190-199,
    241-247).  Accumulation here is fp64 so the result is the correctly
    rounded target the fp32-accumulating kernels are compared against with a
    tolerance.  Input and output are fp32 arrays holding bf16-representable
    values; ``x`` is ``[T, K]``, result ``[T, M]``.
    """
    w = dequant_weights(blocks, scales, lut, round_bf16=True).astype(np.float64)
    acc = np.asarray(x_bf16_as_f32, dtype=np.float64) @ w.T
    if bias is None:
        return bf16_round(acc.astype(np.float32))
    b = np.asarray(bias, dtype=np.float64)[None, :]
    if bias_after_store:
        first = bf16_round(acc.astype(np.float32)).astype(np.float64)
        return bf16_round((first + b).astype(np.float32))
    return bf16_round((acc + b).astype(np.float32))


def linear_f16(x_f16_as_f32: np.ndarray, blocks: np.ndarray, scales: np.ndarray, lut: np.ndarray,
               bias: np.ndarray | None = None, prefill: bool = False) -> np.ndarray:
    """Oracle for the fp16 operator.  Decode (texelator_bc4_kernel, texelator_cuda.cu:77-139):
    ``y = f16( sum_k f32(pal*scale) * f32(x) + f32(bias) )`` -- the weight is *not* rounded.  With ``prefill``
    (texelator_prefill, :996-1046): the weight is rounded to fp16 (texelator_decode_tile), cuBLAS accumulates in
    fp32 and stores fp16, and the bias is added to that with ``__hadd`` (:630-634).  Accumulation here is fp64, as
    in ``linear_bf16``.  Input and output are fp32 arrays holding fp16-representable values."""
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    w = dequant_palette(blocks, scales.shape[0], lut) * scales[:, None]
    if prefill:
        w = w.astype(np.float16)
    acc = np.asarray(x_f16_as_f32, dtype=np.float64) @ w.astype(np.float64).T
    if bias is None:
        return acc.astype(np.float16).astype(np.float32)
    b = np.asarray(bias, dtype=np.float64)[None, :]
    if prefill:
        return (acc.astype(np.float16).astype(np.float64) + b).astype(np.float16).astype(np.float32)
    return (acc + b).astype(np.float16).astype(np.float32)


def row_scales(weight: np.ndarray) -> np.ndarray:
    """``scale_m = max(|W[m,:]|, 1e-12)`` (texelator/encoder.py:140)."""
    return np.maximum(np.abs(np.asarray(weight, dtype=np.float32)).max(axis=1), np.float32(1e-12)).astype(np.float32)


# --------------------------------------------------------------------------
# Encoder restatement (texelator/encoder.py:23-102,120-157).  torch CPU ops are
# used, in the reference's evaluation order, because bit-identical blocks need
# the same fp32 reductions; the structure (table-driven coefficients, candidate
# list) is this file's own.
# --------------------------------------------------------------------------

def _nearest(values, palette):
    """First-lowest-index nearest palette entry (texelator/encoder.py:23-31:
    strict ``<`` keeps the earliest selector on ties)."""
    import torch
    best = torch.full_like(values, float("inf"))
    chosen = torch.zeros(values.shape, dtype=torch.uint8)
    for s in range(8):
        dist = (values - palette[:, s:s + 1]).abs()
        take = dist < best
        best = torch.where(take, dist, best)
        chosen = torch.where(take, torch.full_like(chosen, s), chosen)
    return chosen, torch.gather(palette, 1, chosen.long())


def encode_rows(weight, hdiag, scale, lut):
    """One row chunk of the "E3" endpoint search (texelator/encoder.py:34-102):
    min/max start, activation-weighted 2x2 least squares on the selector
    coefficients, then the 3x3 integer neighbourhood, first-best wins."""
    import torch
    with torch.inference_mode():
        lut_t = torch.as_tensor(lut)
        m, k = weight.shape
        nblk = k // 16
        v = (weight.float() / scale[:, None]).clamp(-1, 1).reshape(-1, 16)
        h = hdiag.float().reshape(nblk, 16).repeat(m, 1)
        e0 = torch.round(v.max(1).values * 127).clamp(-127, 127).to(torch.int16)
        e1 = torch.round(v.min(1).values * 127).clamp(-127, 127).to(torch.int16)
        pal = lut_t[(e1 + 127).long(), (e0 + 127).long()]
        sel, _ = _nearest(v, pal)

        # coefficient tables: value = a*u + b*z + c  (encoder.py:53-70)
        ta8 = torch.tensor([1.0, 0.0] + [(8 - s) / 7 for s in range(2, 8)], dtype=torch.float32)
        tb8 = torch.tensor([0.0, 1.0] + [(s - 1) / 7 for s in range(2, 8)], dtype=torch.float32)
        ta6 = torch.tensor([1.0, 0.0] + [(6 - s) / 5 for s in range(2, 6)] + [0.0, 0.0], dtype=torch.float32)
        tb6 = torch.tensor([0.0, 1.0] + [(s - 1) / 5 for s in range(2, 6)] + [0.0, 0.0], dtype=torch.float32)
        tc6 = torch.tensor([0.0] * 6 + [-1.0, 1.0], dtype=torch.float32)
        high = (e0 > e1)[:, None]
        idx = sel.long()
        a = torch.where(high, ta8[idx], ta6[idx])
        b = torch.where(high, tb8[idx], tb6[idx])
        c = torch.where(high, torch.zeros_like(v), tc6[idx])

        t = v - c
        saa = (h * a * a).sum(1)
        sbb = (h * b * b).sum(1)
        sab = (h * a * b).sum(1)
        say = (h * a * t).sum(1)
        sby = (h * b * t).sum(1)
        det = saa * sbb - sab * sab
        keep = det.abs() < 1e-12
        safe = det.clamp_min(1e-12)
        u = ((say * sbb - sby * sab) / safe).clamp(-1, 1)
        z = ((sby * saa - say * sab) / safe).clamp(-1, 1)
        u = torch.where(keep, e0.float() / 127, u)
        z = torch.where(keep, e1.float() / 127, z)
        c0 = torch.round(u * 127).to(torch.int16)
        c1 = torch.round(z * 127).to(torch.int16)

        best = torch.full((v.shape[0],), float("inf"))
        out0, out1, outs = e0, e1, sel
        for d0 in (-1, 0, 1):
            for d1 in (-1, 0, 1):
                q0 = (c0 + d0).clamp(-127, 127)
                q1 = (c1 + d1).clamp(-127, 127)
                qpal = lut_t[(q1 + 127).long(), (q0 + 127).long()]
                qsel, qv = _nearest(v, qpal)
                err = (h * (v - qv).square()).sum(1)
                win = err < best
                best = torch.where(win, err, best)
                out0 = torch.where(win, q0, out0)
                out1 = torch.where(win, q1, out1)
                outs = torch.where(win[:, None], qsel, outs)
        return out0.numpy(), out1.numpy(), outs.numpy()


def encode_linear(weight, hdiag, lut, rows_per_chunk: int = 128):
    """In-memory form of ``encode_linear_e3`` (texelator/encoder.py:120-157):
    returns ``(blocks_u8 [M*K/16*8], scales_f32 [M])`` -- the contents of the
    ``.bc4`` and ``.scales.f32`` files."""
    import torch
    weight = torch.as_tensor(weight)
    hdiag = torch.as_tensor(hdiag)
    m, k = map(int, weight.shape)
    if k % 16:
        raise ValueError(f"unsupported K={k}; BC4 needs K % 16 == 0")
    out_blocks, out_scales = [], []
    for start in range(0, m, rows_per_chunk):
        rows = weight[start:start + rows_per_chunk].detach().float()
        sc = rows.abs().amax(1).clamp_min(1e-12)
        q0, q1, qs = encode_rows(rows, hdiag, sc, lut)
        out_blocks.append(pack_blocks(q0, q1, qs).reshape(-1))
        out_scales.append(sc.numpy().astype("<f4"))
    return np.concatenate(out_blocks), np.concatenate(out_scales)


def encode_minmax(weight: np.ndarray, lut: np.ndarray):
    """Cheap encoder for throughput-only inputs: the min/max initialisation of
    texelator/encoder.py:46-51 without the endpoint search.  Produces valid
    BC4 blocks with the same byte statistics; parity tests never use it."""
    w = np.asarray(weight, dtype=np.float32)
    sc = row_scales(w)
    v = np.clip(w / sc[:, None], -1, 1).reshape(-1, 16)
    e0 = np.clip(np.rint(v.max(1) * 127), -127, 127).astype(np.int32)
    e1 = np.clip(np.rint(v.min(1) * 127), -127, 127).astype(np.int32)
    pal = lut[e1 + 127, e0 + 127]                      # [n, 8]
    dist = np.abs(v[:, :, None] - pal[:, None, :])
    sel = dist.argmin(axis=2)
    return pack_blocks(e0, e1, sel).reshape(-1), sc


# --------------------------------------------------------------------------
# Tensor-parallel slicing (byte slicing only; no re-encode).
# --------------------------------------------------------------------------

def shard_rows(blocks: np.ndarray, scales: np.ndarray, rank: int, world: int):
    """Column-parallel shard: output rows ``[r*M/P, (r+1)*M/P)``."""
    m = scales.shape[0]
    per = m // world
    raw = np.asarray(blocks, dtype=np.uint8).reshape(m, -1)
    return raw[rank * per:(rank + 1) * per].reshape(-1).copy(), scales[rank * per:(rank + 1) * per].copy()


def shard_kblocks(blocks: np.ndarray, scales: np.ndarray, rank: int, world: int):
    """Row-parallel shard: K-block range ``[r*K/(16P), (r+1)*K/(16P))`` of every
    row, with the full per-row scale vector."""
    m = scales.shape[0]
    raw = np.asarray(blocks, dtype=np.uint8).reshape(m, -1, 8)
    per = raw.shape[1] // world
    return raw[:, rank * per:(rank + 1) * per].reshape(-1).copy(), scales.copy()


def rel_rms(got: np.ndarray, ref: np.ndarray) -> float:
    """Relative RMS error used by the reference's gates
    (texelator/prefill.py:98-107; texelator/autotune.py:62-75)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.sqrt(np.mean((got - ref) ** 2)) / max(np.sqrt(np.mean(ref ** 2)), 1e-30))
