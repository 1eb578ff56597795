"""Q8_0, the public GGML block format: 32 consecutive elements share one fp16 scale d = max|x| / 127, each element is
stored as the signed byte round(x / d); a block is the little-endian scale followed by the 32 bytes (34 bytes), and the
value read back is fp32(d) * q. The engine only names the type (include/gguf.hpp:28; docs/gguf.md lists the id), so
this module is the writer for seed-generated models and the fp32 dequantiser that checks are made against."""
from __future__ import annotations

import numpy as np

BLOCK = 32
BLOCK_BYTES = 34


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    """fp32 / fp16 array [..., n] (n a multiple of 32) -> uint8 array [..., n/32*34]."""
    w = np.asarray(w, dtype=np.float32)
    if w.shape[-1] % BLOCK:
        raise ValueError("the last dimension must be a multiple of 32")
    blocks = w.reshape(*w.shape[:-1], w.shape[-1] // BLOCK, BLOCK)
    amax = np.abs(blocks).max(axis=-1, keepdims=True)
    d = amax / np.float32(127.0)
    inv = np.where(d > 0, np.float32(1.0) / np.where(d > 0, d, 1), np.float32(0.0)).astype(np.float32)
    # roundf: half away from zero
    scaled = blocks * inv
    q = (np.sign(scaled) * np.floor(np.abs(scaled) + np.float32(0.5))).astype(np.int8)
    out = np.empty(blocks.shape[:-1] + (BLOCK_BYTES,), dtype=np.uint8)
    out[..., :2] = d.astype(np.float16).view(np.uint8).reshape(*d.shape[:-1], 2)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(*w.shape[:-1], -1)


def dequantize_q8_0(blocks: np.ndarray) -> np.ndarray:
    """uint8 [..., n/32*34] -> fp32 [..., n] (fp32(d) * q, exact in fp32)."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    b = b.reshape(*b.shape[:-1], b.shape[-1] // BLOCK_BYTES, BLOCK_BYTES)
    d = b[..., :2].copy().view(np.float16).astype(np.float32)
    q = b[..., 2:].view(np.int8).astype(np.float32)
    return (d * q).reshape(*blocks.shape[:-1], -1)


def repack_q8_0_tiled(blocks: np.ndarray) -> np.ndarray:
    """uint8 [rows, n/32*34] -> the tiled layout of attn_repack_q8_0_tiled, uint8 [ceil(rows/16), n/32, 544]: per
    group of 16 rows and per block, lane L = 4 g + t owns 16 bytes = the words {row g, k-step 0}, {row g+8, k-step 0},
    {row g, k-step 1}, {row g+8, k-step 1}, a word = the row's elements 16 s + 4 t + (0, 2, 1, 3) of the block as
    bytes q + 128; the fp16 scales of rows (g, g+8) follow at 512 + 4 g. Rows past the end are zeros (bytes 0x80)."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    rows, nb = b.shape[0], b.shape[1] // BLOCK_BYTES
    groups = (rows + 15) // 16
    padded = np.zeros((groups * 16, nb, BLOCK_BYTES), dtype=np.uint8)
    padded[:, :, 2:] = 0  # q = 0
    padded[:rows] = b.reshape(rows, nb, BLOCK_BYTES)
    q = padded[:, :, 2:] ^ np.uint8(0x80)               # [R, nb, 32] biased bytes
    q[rows:] = 0x80
    q = q.reshape(groups, 2, 8, nb, 2, 4, 4)            # [rg, half, g, blk, s, t, e]
    q = q[..., [0, 2, 1, 3]]                            # byte order inside a word
    q = q.transpose(0, 3, 2, 5, 4, 1, 6)                # [rg, blk, g, t, s, half, e]
    out = np.empty((groups, nb, 16 * BLOCK_BYTES), dtype=np.uint8)
    out[:, :, :512] = q.reshape(groups, nb, 512)
    sc = padded[:, :, :2].reshape(groups, 2, 8, nb, 2)  # [rg, half, g, blk, byte]
    out[:, :, 512:] = sc.transpose(0, 3, 2, 1, 4).reshape(groups, nb, 32)
    return out


def quantize_q8_0_torch(w):
    """The same writer on torch tensors of any device: [..., n] float -> uint8 [..., n/32*34]."""
    import torch
    w = w.float()
    blocks = w.reshape(*w.shape[:-1], w.shape[-1] // BLOCK, BLOCK)
    amax = blocks.abs().amax(dim=-1, keepdim=True)
    d = amax / 127.0
    inv = torch.where(d > 0, 1.0 / torch.where(d > 0, d, torch.ones_like(d)), torch.zeros_like(d))
    scaled = blocks * inv
    q = (torch.sign(scaled) * torch.floor(scaled.abs() + 0.5)).to(torch.int8)
    out = torch.empty(blocks.shape[:-1] + (BLOCK_BYTES,), dtype=torch.uint8, device=w.device)
    out[..., :2] = d.half().view(torch.uint8).reshape(*d.shape[:-1], 2)
    out[..., 2:] = q.view(torch.uint8)
    return out.reshape(*w.shape[:-1], -1)
