"""Generate the golden fixtures in this directory from the REFERENCE encoder.

Run once, in a container where the hp0303/Texelator tree is mounted:

    python tests/golden/make_golden.py /path/to/Texelator

It imports the reference's own ``texelator/encoder.py`` (CPU torch) and records
what it emits for seeded inputs under the software BC4 palette.  The committed
``.npz``/``.json`` files are what the test-suite replays; this script is not
imported by anything and the reference tree is not needed at test time.
"""
from __future__ import annotations

import hashlib
import json
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle import bc4_oracle as O  # noqa: E402  (only for the palette table)


def seeded_case(seed: int, m: int, k: int, tokens: int, calib: int = 64, std: float = 0.02):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(m, k, generator=g) * std
    xc = torch.randn(calib, k, generator=g)
    h = (xc * xc).mean(0)
    x = torch.randn(tokens, k, generator=g).bfloat16()
    return w, h, x


def edge_matrix(seed: int, m: int = 32, k: int = 128):
    """Rows that force the e0<=e1 palette mode and the clamps: zeros, constants,
    +-max, a 90%-sparse row, single spikes."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(m, k, generator=g) * 0.02
    w[0] = 0.0
    w[1] = 0.05
    w[2] = -0.05
    w[3, :64] = 0.0
    w[4] = torch.where(torch.rand(k, generator=g) < 0.9, torch.zeros(k), w[4])
    w[5, ::16] = 0.3
    w[6, 16:32] = w[6].abs().max()
    w[7, 32:48] = -w[7].abs().max()
    w[8] = torch.where(torch.rand(k, generator=g) < 0.5, torch.full((k,), 0.01), torch.full((k,), -0.01))
    w[9, :16] = torch.linspace(-0.04, 0.04, 16)
    h = torch.rand(k, generator=g) + 0.1
    x = torch.randn(5, k, generator=g).bfloat16()
    return w, h, x


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from texelator import encoder as R  # the reference, unmodified

    lut_np = O.software_palette()
    lut = torch.from_numpy(lut_np)
    manifest = {"palette_sha256": O.palette_sha256(lut_np), "cases": {}}

    def run_reference(w, h):
        with tempfile.TemporaryDirectory() as tmp:
            info = R.encode_linear_e3(w, h, lut, Path(tmp) / "a.bc4", Path(tmp) / "a.scales.f32")
            blocks = np.fromfile(Path(tmp) / "a.bc4", dtype=np.uint8)
            scales = np.fromfile(Path(tmp) / "a.scales.f32", dtype="<f4")
        return info, blocks, scales

    def dequant_by_reference(blocks, scales):
        # palette lookup exactly as the reference performs it (encoder.py:19-31)
        m = scales.shape[0]
        raw = blocks.reshape(m, -1, 8)
        e0 = torch.from_numpy(raw[:, :, 0].copy().view(np.int8).astype(np.int16)).reshape(-1)
        e1 = torch.from_numpy(raw[:, :, 1].copy().view(np.int8).astype(np.int16)).reshape(-1)
        word = np.zeros(raw.shape[:2], dtype=np.uint64)
        for b in range(6):
            word |= raw[:, :, 2 + b].astype(np.uint64) << np.uint64(8 * b)
        sel = np.stack([(word >> np.uint64(3 * p)) & np.uint64(7) for p in range(16)], -1).astype(np.int64)
        pal = R.actual_palette(lut, e0, e1)
        vals = torch.gather(pal, 1, torch.from_numpy(sel.reshape(-1, 16)))
        return vals.reshape(m, -1).numpy()

    small = {
        "small_48x256": seeded_case(1234, 48, 256, 3),
        "odd_24x48": seeded_case(77, 24, 48, 2),
        "edge_32x128": edge_matrix(5),
        "tall_130x64": seeded_case(9, 130, 64, 1),
    }
    for name, (w, h, x) in small.items():
        info, blocks, scales = run_reference(w, h)
        pal = dequant_by_reference(blocks, scales)
        np.savez_compressed(
            HERE / f"{name}.npz",
            weight=w.numpy(), hdiag=h.numpy(), x_bf16=x.float().numpy(),
            blocks=blocks, scales=scales, palette_values=pal.astype(np.float32))
        manifest["cases"][name] = {k: info[k] for k in ("M", "K", "blocks_bytes", "blocks_sha256", "scales_bytes", "scales_sha256")}

    # configuration-1 sized case: hashes only (8 MiB of blocks is not committed)
    w, h, x = seeded_case(20260827, 4096, 4096, 1)
    info, blocks, scales = run_reference(w, h)
    manifest["cases"]["cfg1_4096x4096"] = {k: info[k] for k in ("M", "K", "blocks_bytes", "blocks_sha256", "scales_bytes", "scales_sha256")}
    manifest["cases"]["cfg1_4096x4096"]["seed"] = 20260827
    manifest["cases"]["cfg1_4096x4096"]["first_blocks_hex"] = blocks[:128].tobytes().hex()
    e0 = blocks.reshape(-1, 8)[:, 0].view(np.int8)
    e1 = blocks.reshape(-1, 8)[:, 1].view(np.int8)
    manifest["cases"]["cfg1_4096x4096"]["low_mode_blocks"] = int((e0 <= e1).sum())

    # reference `pack_blocks` / `nearest` on handcrafted inputs
    q0 = torch.tensor([127, -127, 5, 0, -1, 126, 3], dtype=torch.int16)
    q1 = torch.tensor([-127, 127, 5, 0, 0, 126, -3], dtype=torch.int16)
    sel = torch.stack([torch.arange(16) % 8, (torch.arange(16) * 3) % 8, torch.zeros(16, dtype=torch.long),
                       torch.full((16,), 7), torch.ones(16, dtype=torch.long), torch.full((16,), 7),
                       (torch.arange(16) // 2)]).to(torch.uint8)
    packed = R.pack_blocks(q0, q1, sel)
    np.savez_compressed(HERE / "handcrafted_blocks.npz", e0=q0.numpy(), e1=q1.numpy(), sel=sel.numpy(), packed=packed)
    (HERE / "manifest.json").write_text(json.dumps(manifest, indent=2, sort_keys=True) + "\n")
    print(json.dumps(manifest, indent=2))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of hp0303/Texelator>")
    main(sys.argv[1])
