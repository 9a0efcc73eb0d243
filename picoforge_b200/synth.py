"""Seeded synthetic Qwen4 MoE layers and activations for tests and benchmarks.

Weights: FP32 masters N(0, 0.02) drawn per tensor from a counter-based generator and
encoded to the requested GGUF block format by this project's own encoders (csrc/synth.c;
picoforge has no quantiser).  Router tensors stay F32.  Activations: FP32 N(0, 1).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

from . import abi
from .layer import LayerSpec

_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        path = Path(__file__).resolve().parent / "libqw4synth.so"
        if not path.exists():
            raise FileNotFoundError(f"{path} is missing: run python -m picoforge_b200.build")
        _LIB = C.CDLL(str(path))
        _LIB.qw4s_tensor.argtypes = [C.c_uint32, C.c_uint64, C.c_uint64, C.c_float, C.c_size_t, C.c_size_t,
                                     C.c_void_p, C.c_int]
        _LIB.qw4s_tensor.restype = C.c_int
        _LIB.qw4s_tensor_rows.argtypes = [C.c_uint32, C.c_uint64, C.c_uint64, C.c_float, C.c_size_t, C.c_size_t, C.c_size_t,
                                          C.c_void_p, C.c_int]
        _LIB.qw4s_tensor_rows.restype = C.c_int
        _LIB.qw4s_encode_rows.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]
        _LIB.qw4s_encode_rows.restype = C.c_int
        _LIB.qw4s_normal.argtypes = [C.c_uint64, C.c_uint64, C.c_float, C.c_void_p, C.c_size_t, C.c_size_t]
        _LIB.qw4s_normal.restype = None
    return _LIB


def threads() -> int:
    return max(1, min(64, len(os.sched_getaffinity(0))))


def tensor(gguf_type: int, seed: int, stream: int, rows: int, k: int, sigma: float = 0.02, row0: int = 0,
           out: np.ndarray | None = None) -> np.ndarray:
    """Rows [row0, row0 + rows) of a tensor of k-weight rows ~ N(0, sigma) encoded as gguf_type;
    returns the packed bytes (a shard has the same bytes as that slice of the whole tensor).  `out`: an
    array of the right size to write into (first-touch page faults of a fresh one can cost more than
    the generation)."""
    size = rows * abi.row_bytes(gguf_type, k)
    if out is None or out.size != size or out.dtype != np.uint8:
        out = np.empty(size, np.uint8)
    if _lib().qw4s_tensor_rows(gguf_type, seed, stream, sigma, row0, rows, k, out.ctypes.data, threads()):
        raise ValueError(f"cannot synthesise type {gguf_type} with k={k}")
    return out


def encode(gguf_type: int, masters: np.ndarray) -> np.ndarray:
    masters = np.ascontiguousarray(masters, np.float32)
    rows, k = masters.shape
    out = np.empty(rows * abi.row_bytes(gguf_type, k), np.uint8)
    if _lib().qw4s_encode_rows(gguf_type, masters.ctypes.data, rows, k, out.ctypes.data):
        raise ValueError(f"cannot encode type {gguf_type} with k={k}")
    return out


def normal(seed: int, stream: int, rows: int, k: int, sigma: float = 1.0) -> np.ndarray:
    out = np.empty((rows, k), np.float32)
    _lib().qw4s_normal(seed, stream, sigma, out.ctypes.data, rows, k)
    return out


def make_layer(seed: int, layer: int = 0, routed_type: int = abi.Q4_K, shared_type: int = abi.Q4_K,
               hidden: int = 2048, experts: int = 512, top_k: int = 10, inter: int = 512,
               shared_inter: int = 512, down_type: int | None = None, norm: bool = True,
               shard: tuple | None = None, fabricated: bool = False, reuse: LayerSpec | None = None,
               down_physical: int | None = None) -> LayerSpec:
    """One synthetic layer.  Stream ids: layer * 8 + tensor index.  shard = (first_expert,
    local_experts) generates only that slice of the routed expert tensors.  fabricated: the
    quantised tensors are random valid blocks with scales set for a spread of about 0.02 (as the
    reference's kernel tests make theirs) instead of encoded Gaussians: some twenty times
    faster to make, for stacks of many layers.  reuse: a spec of the same shapes whose arrays are
    overwritten and returned in the new spec (the old spec must not be used afterwards).
    down_physical: stored K of the routed down projection when it is padded beyond `inter`."""
    down_type = routed_type if down_type is None else down_type
    types = (abi.F32, routed_type, routed_type, down_type, shared_type, shared_type, shared_type, abi.F32)
    spec = LayerSpec(hidden, experts, top_k, inter, shared_inter, down_physical or inter, norm, types)
    if shard is not None:
        spec.first_expert, spec.local_experts = shard
    tensors = []
    for index, (gguf_type, (k_storage, _, n_out, n_experts)) in enumerate(zip(types, spec.shapes())):
        row0 = spec.first_expert * n_out if 1 <= index <= 3 else 0
        sigma = -1.0 if fabricated and gguf_type != abi.F32 else 0.02
        old = reuse.tensors[index] if reuse is not None and len(reuse.tensors) == 8 else None
        tensors.append(tensor(gguf_type, seed, layer * 8 + index, n_out * n_experts, k_storage, sigma=sigma, row0=row0, out=old))
    spec.tensors = tensors
    return spec


def zipf_router_bias(spec: LayerSpec, seed: int, column: int = 0, constant: float = 1.0, exponent: float = 1.1) -> None:
    """Makes expert popularity follow Zipf(exponent): the reference router has no bias term
    (picoforge src/qwen4_moe.c:340-341), so the bias lives in the data.  Router column `column`
    is set to log pmf(rank(e)) / constant and the caller sets x[:, column] = constant."""
    rng = np.random.default_rng([seed, 0x5A1F])
    ranks = rng.permutation(spec.experts) + 1
    pmf = ranks.astype(np.float64) ** -exponent
    pmf /= pmf.sum()
    router = spec.tensors[0].view(np.float32).reshape(spec.experts, spec.hidden)
    router[:, column] = (np.log(pmf) / constant).astype(np.float32)


def activations(seed: int, tokens: int, hidden: int = 2048) -> np.ndarray:
    return normal(seed, 0xAC7, tokens, hidden, 1.0)


def correlated_tokens(x: np.ndarray, seed: int, source: int = 0, target: int = 1, rho: float = 0.9) -> None:
    """x[target] = rho * x[source] + sqrt(1 - rho^2) * n: still N(0, 1), and the two tokens then
    share most of their top-k experts (a multi-token verify step sees nearby hidden states)."""
    noise = normal(seed, 0xC0DE, 1, x.shape[1], 1.0)[0]
    x[target] = (rho * x[source] + np.sqrt(1.0 - rho * rho) * noise).astype(np.float32)
