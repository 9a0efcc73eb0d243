"""Generates tests/golden/golden.npz from the REFERENCE's own CPU objects.

Run in a container where the reference sources are mounted and `make -C oracle ref` has built
oracle/_ref/libqw4ref.so:

    python tests/golden/make_golden.py

The vectors pin the oracle port (and through it the CUDA path) on machines where the
reference objects are absent.  Contents:
  decode_<type>_sha256   SHA-256 of the reference's decode of tests.cases.pattern_blocks(type)
  route_*                seeded logits -> probabilities, ids, weights of qwen4_moe_route
  group_*                seeded ids -> offsets, pair_to_row, row_to_pair of qw4_moe_group_pairs
  fwd_<name>_*           small seeded layers -> y, ids, weights of qwen4_moe_forward
"""
import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import cases  # noqa: E402
import oracle  # noqa: E402
from picoforge_b200 import abi, synth  # noqa: E402
from picoforge_b200.layer import MoeLayer, group_pairs, route  # noqa: E402

FORWARD_CASES = {
    "q4k": dict(seed=11, routed=abi.Q4_K, shared=abi.Q4_K, tokens=5),
    "q2k": dict(seed=12, routed=abi.Q2_K, shared=abi.Q4_K, tokens=3),
    "iq2": dict(seed=13, routed=abi.IQ2_XXS, shared=abi.Q4_K, tokens=4),
    "f32": dict(seed=14, routed=None, shared=None, tokens=7),
}


def forward_case(name):
    case = FORWARD_CASES[name]
    if case["routed"] is None:
        spec = cases.float_layer(case["seed"], hidden=24, experts=6, top_k=3, inter=10, shared_inter=7)
        x = np.random.default_rng(case["seed"]).standard_normal((case["tokens"], 24)).astype(np.float32)
    else:
        spec = cases.small_layer(case["seed"], case["routed"], case["shared"])
        x = synth.activations(case["seed"], case["tokens"], spec.hidden)
    return spec, x


def main():
    ref = oracle.reference_api()
    out = {}
    for gguf_type in (abi.Q4_K, abi.Q2_K, abi.IQ2_XXS, abi.Q8_0, abi.MXFP4, abi.F16, abi.BF16, abi.F32):
        blocks = cases.pattern_blocks(gguf_type)
        k = abi.FORMATS[gguf_type][1]
        decoded = oracle.reference_decode_rows(gguf_type, blocks.reshape(-1), len(blocks), k)
        out[f"decode_{gguf_type}_sha256"] = np.frombuffer(hashlib.sha256(decoded.tobytes()).digest(), np.uint8)
    for seed, (t, e, k) in enumerate([(33, 512, 10), (64, 17, 5), (5, 4, 2), (16, 64, 64)]):
        rng = np.random.default_rng(3811 + seed)
        logits = rng.standard_normal((t, e)).astype(np.float32) * 3
        logits[0, : min(e, 4)] = 1.5                   # exact ties
        for norm in (0, 1):
            probs, ids, weights = route(ref, logits, k, bool(norm))
            tag = f"route_{seed}_{norm}"
            out[tag + "_logits"], out[tag + "_probs"], out[tag + "_ids"], out[tag + "_weights"] = logits, probs, ids, weights
    for seed, (t, e, k) in enumerate([(37, 512, 10), (9, 4, 2), (128, 16, 4)]):
        rng = np.random.default_rng(3812 + seed)
        ids = np.stack([rng.permutation(e)[:k] for _ in range(t)]).astype(np.uint32)
        offsets, p2r, r2p = group_pairs(ref, ids, e)
        tag = f"group_{seed}"
        out[tag + "_ids"], out[tag + "_offsets"], out[tag + "_p2r"], out[tag + "_r2p"] = ids, offsets, p2r, r2p
    for name in FORWARD_CASES:
        spec, x = forward_case(name)
        with MoeLayer(ref, spec, len(x)) as layer:
            y, ids, weights = layer.forward(x)
        out[f"fwd_{name}_y"], out[f"fwd_{name}_ids"], out[f"fwd_{name}_weights"] = y, ids, weights
    np.savez_compressed(Path(__file__).parent / "golden.npz", **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
