"""Shared inputs of the parity tests: exhaustive block patterns, seeded layers, configs.

The block-pattern generators follow the coverage the reference's GPU kernel tests describe
(picoforge tests/test_qwen4_fast_kernels.py:1565-1624): every scale/min field value at every
position, every code at every column, every codebook index and sign word, and every finite
fp16 scale, cycled over 65536 blocks.
"""
from __future__ import annotations

import numpy as np

from picoforge_b200 import abi, synth


def finite_halfs() -> np.ndarray:
    patterns = np.arange(65536, dtype=np.uint16)
    return patterns[(patterns & 0x7C00) != 0x7C00]


def pattern_blocks(gguf_type: int, count: int = 65536) -> np.ndarray:
    """`count` blocks (uint8 [count, block bytes]) sweeping every field of the format."""
    finite = finite_halfs()
    rows = np.arange(count)
    if gguf_type == abi.Q4_K:
        packed = np.zeros((count, 144), np.uint8)
        packed[:, 0:2] = finite[rows % len(finite)].view(np.uint8).reshape(-1, 2)
        packed[:, 2:4] = finite[(rows * 7919) % len(finite)].view(np.uint8).reshape(-1, 2)
        packed[:, 4:16] = (rows[:, None] + 17 * np.arange(12)) % 256
        packed[:, 16:144] = (rows[:, None] * 29 + 7 * np.arange(128)) % 256
    elif gguf_type == abi.Q2_K:
        packed = np.zeros((count, 84), np.uint8)
        packed[:, :16] = (rows[:, None] + 17 * np.arange(16)) % 256
        packed[:, 16:80] = (rows[:, None] * 29 + 7 * np.arange(64)) % 256
        packed[:, 80:82] = finite[rows % len(finite)].view(np.uint8).reshape(-1, 2)
        packed[:, 82:84] = finite[(rows * 7919) % len(finite)].view(np.uint8).reshape(-1, 2)
    elif gguf_type == abi.IQ2_XXS:
        start, sign_id, scale = rows % 256, rows // 256 % 128, (rows + rows // 256) % 16
        words = (sign_id * (1 | 1 << 7 | 1 << 14 | 1 << 21) | scale << 28).astype("<u4")
        packed = np.zeros((count, 66), np.uint8)
        packed[:, :2] = finite[rows % len(finite)].view(np.uint8).reshape(-1, 2)
        for g in range(8):
            packed[:, 2 + 8 * g:6 + 8 * g] = (start[:, None] + 4 * g + np.arange(4)) % 256
            packed[:, 6 + 8 * g:10 + 8 * g] = words.view(np.uint8).reshape(-1, 4)
    elif gguf_type == abi.Q8_0:
        packed = np.zeros((count, 34), np.uint8)
        packed[:, :2] = finite[rows % len(finite)].view(np.uint8).reshape(-1, 2)
        packed[:, 2:] = (rows[:, None] * 13 + 5 * np.arange(32)) % 256
    elif gguf_type == abi.MXFP4:
        packed = np.zeros((count, 17), np.uint8)
        packed[:, 0] = rows % 253                     # 253, 254 overflow with the largest codes; 255 is Inf/NaN
        packed[:, 1:] = (rows[:, None] // 253 * 17 + 31 * np.arange(16) + rows[:, None]) % 256
    elif gguf_type == abi.F16:
        packed = finite[rows % len(finite)].view(np.uint8).reshape(-1, 2).copy()
    elif gguf_type == abi.BF16:
        values = (rows % 65536).astype(np.uint16)
        values = values[(values & 0x7F80) != 0x7F80] if count >= 65536 else values
        values = np.resize(values, count)
        values[(values & 0x7F80) == 0x7F80] = 0x3F80
        packed = values.view(np.uint8).reshape(-1, 2).copy()
    elif gguf_type == abi.F32:
        rng = np.random.default_rng(4100)
        bits = rng.integers(0, 2**32, count, dtype=np.uint64).astype(np.uint32)
        bits[(bits & 0x7F800000) == 0x7F800000] ^= 0x40000000
        packed = bits.view(np.uint8).reshape(-1, 4).copy()
    else:
        raise ValueError(gguf_type)
    return np.ascontiguousarray(packed)


def small_layer(seed: int, routed: int = abi.Q4_K, shared: int = abi.Q4_K, experts: int = 16, top_k: int = 4,
                hidden: int = 512, inter: int = 256, shared_inter: int = 256, **kw):
    return synth.make_layer(seed, routed_type=routed, shared_type=shared, experts=experts, top_k=top_k,
                            hidden=hidden, inter=inter, shared_inter=shared_inter, **kw)


def float_layer(seed: int, hidden=8, experts=4, top_k=2, inter=5, shared_inter=3, down_physical=None, norm=True,
                sigma=0.5):
    """All-F32 layer with odd shapes, as the reference's lifecycle fixtures use
    (picoforge tests/test_qwen4_moe.c:234-242)."""
    from picoforge_b200.layer import LayerSpec
    spec = LayerSpec(hidden, experts, top_k, inter, shared_inter, down_physical or inter, norm, (abi.F32,) * 8)
    rng = np.random.default_rng(seed)
    spec.tensors = [np.ascontiguousarray((rng.standard_normal(n * ex * k) * sigma).astype(np.float32)).view(np.uint8)
                    for (k, _, n, ex) in spec.shapes()]
    return spec
