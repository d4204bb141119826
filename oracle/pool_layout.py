"""numpy codec of the 3-bit page chunk layout (test infrastructure).

Restates the bit layout the kernels use (one chunk = 16 tokens of one kv head, K or V:
192 uint32 words of codes + 16 fp16 norms = 800 bytes), independently of the CUDA code,
so that the pool the kernels write can be decoded and compared code by code.
"""

from __future__ import annotations

import numpy as np

CHUNK_BYTES = 800
CHUNK_WORDS = 192


def k_slot(slot: int, coord: int) -> tuple[int, int]:
    """(unit index, code index in unit) of a K code."""
    return slot * 4 + coord // 32, coord % 32


def v_slot(slot: int, coord: int) -> tuple[int, int]:
    p, g = slot // 2, coord // 16
    ui = 4 * g + p if p < 4 else 32 + 4 * g + (p - 4)
    return ui, 2 * (coord % 16) + (slot % 2)


def get_code(words: np.ndarray, ui: int, e: int) -> int:
    """Unit = words[ui], words[64+ui], words[128+ui]; codes 0..23 one per nibble, codes
    24..31 spread over bit 3 of the nibbles (bit b of the code in word b)."""
    if e < 24:
        return int(words[(e // 8) * 64 + ui] >> (4 * (e % 8))) & 7
    sh = 4 * (e - 24) + 3
    return sum(((int(words[b * 64 + ui]) >> sh) & 1) << b for b in range(3))


def decode_chunk(chunk: np.ndarray, which: int) -> tuple[np.ndarray, np.ndarray]:
    """chunk: uint8[800] -> (codes uint8 [16, 128], norms float32 [16])."""
    words = chunk[:768].view(np.uint32)
    norms = chunk[768:].view(np.float16).astype(np.float32)
    codes = np.zeros((16, 128), dtype=np.uint8)
    for slot in range(16):
        for c in range(128):
            ui, e = k_slot(slot, c) if which == 0 else v_slot(slot, c)
            codes[slot, c] = get_code(words, ui, e)
    return codes, norms


def encode_chunk(codes: np.ndarray, norms: np.ndarray, which: int) -> np.ndarray:
    """Inverse of decode_chunk (codes [16,128] in 0..7, norms float [16])."""
    words = np.zeros(CHUNK_WORDS, dtype=np.uint32)
    for slot in range(16):
        for c in range(128):
            ui, e = k_slot(slot, c) if which == 0 else v_slot(slot, c)
            code = int(codes[slot, c])
            if e < 24:
                words[(e // 8) * 64 + ui] |= np.uint32(code << (4 * (e % 8)))
            else:
                for b in range(3):
                    words[b * 64 + ui] |= np.uint32(((code >> b) & 1) << (4 * (e - 24) + 3))
    out = np.zeros(CHUNK_BYTES, dtype=np.uint8)
    out[:768] = words.view(np.uint8)
    out[768:] = np.asarray(norms, dtype=np.float16).view(np.uint8)
    return out


def nibbles_to_codes(packed: np.ndarray) -> np.ndarray:
    """Reference nibble format (..., 64) uint8 -> codes (..., 128)."""
    lo, hi = packed & 0xF, packed >> 4
    return np.stack([lo, hi], axis=-1).reshape(*packed.shape[:-1], -1)
