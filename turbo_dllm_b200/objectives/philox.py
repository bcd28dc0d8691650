"""Host twin of the device noising generator (csrc/noising.cu): Philox4x32-10, 24-bit uniforms.

`uniform01(seed, offset, n)` returns the same numbers the kernel draws for token indices 0..n-1,
and `corrupt_reference` applies the same masking rules with them, so CPU runs and GPU runs see
identical corrupted batches for equal (seed, offset)."""
from __future__ import annotations

import numpy as np
import torch

M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
MASK32 = 0xFFFFFFFF


def uniform01(seed: int, offset: int, n: int) -> np.ndarray:
    idx = np.arange(n, dtype=np.uint64)
    c0 = (idx & MASK32).astype(np.uint64)
    c1 = (idx >> np.uint64(32)).astype(np.uint64)
    c2 = np.full(n, offset & MASK32, dtype=np.uint64)
    c3 = np.full(n, (offset >> 32) & MASK32, dtype=np.uint64)
    k0, k1 = seed & MASK32, (seed >> 32) & MASK32
    for _ in range(10):
        p0 = np.uint64(M0) * c0
        p1 = np.uint64(M1) * c2
        n0 = ((p1 >> np.uint64(32)) ^ c1 ^ np.uint64(k0)) & np.uint64(MASK32)
        n1 = p1 & np.uint64(MASK32)
        n2 = ((p0 >> np.uint64(32)) ^ c3 ^ np.uint64(k1)) & np.uint64(MASK32)
        n3 = p0 & np.uint64(MASK32)
        c0, c1, c2, c3 = n0, n1, n2, n3
        k0, k1 = (k0 + W0) & MASK32, (k1 + W1) & MASK32
    return ((c0 >> np.uint64(8)).astype(np.float32) * np.float32(1.0 / 16777216.0))


def corrupt_reference(x0: torch.Tensor, t: torch.Tensor, eligible, block_size: int, views: int, shift: bool,
                      mask_id: int, seed: int, offset: int):
    b, l = x0.shape
    u = torch.from_numpy(uniform01(seed, offset, b * l)).view(b, l)
    tj = t.cpu().repeat_interleave(block_size, dim=1)
    el = torch.ones(b, l, dtype=torch.bool) if eligible is None else eligible.cpu().bool()
    sampled = (u < tj) if views == 2 else (u <= tj)
    masks = torch.stack([sampled & el] + ([(~sampled) & el] if views == 2 else []), dim=1)
    xv = x0.cpu()[:, None].expand(-1, views, -1)
    xt = torch.where(masks, torch.full_like(xv, mask_id), xv)
    tgt = torch.where(masks, xv, torch.full_like(xv, -100))
    if shift:
        labels = torch.full_like(tgt, -100)
        labels[:, :, :-1] = tgt[:, :, 1:]
    else:
        labels = tgt
    return xt, labels
