"""A GGUF v3 file holding one synthetic MoE layer (plus a few unrelated entries), written from scratch:
header, metadata key/values, tensor table, alignment padding, payloads.  Test infrastructure."""
import struct

import numpy as np

ROLE_SUFFIX = ["ffn_gate_inp.weight", "ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight",
               "ffn_gate_shexp.weight", "ffn_up_shexp.weight", "ffn_down_shexp.weight", "ffn_gate_inp_shexp.weight"]


def _string(text: str) -> bytes:
    raw = text.encode()
    return struct.pack("<Q", len(raw)) + raw


def _kv(key: str, kind: int, payload: bytes) -> bytes:
    return _string(key) + struct.pack("<I", kind) + payload


def tensor_shapes(spec):
    """GGUF shapes (K first) of the eight tensors, Qwen4MoeWeights order."""
    h, f, fs, ne, dp = spec.hidden, spec.inter, spec.shared_inter, spec.experts, spec.down_physical
    return [(h, ne), (h, f, ne), (h, f, ne), (dp, h, ne), (h, fs), (h, fs), (fs, h), (h,)]


def write_layer(path, spec, layer=0, alignment=32, drop=None, extra_metadata=(), truncate=None, architecture="qwen4exp",
                overrides=None):
    """Writes the file and returns {tensor name: (absolute offset, bytes)}.  `drop`: a role index left out;
    `overrides`: {key: uint32} replacing a config value; `truncate`: cut the file to that many bytes."""
    keys = {"qwen4exp.embedding_length": spec.hidden, "qwen4exp.expert_count": spec.experts,
            "qwen4exp.expert_used_count": spec.top_k, "qwen4exp.expert_feed_forward_length": spec.inter,
            "qwen4exp.expert_shared_feed_forward_length": spec.shared_inter}
    keys.update(overrides or {})
    metadata = [_kv("general.architecture", 8, _string(architecture)), _kv("general.alignment", 4, struct.pack("<I", alignment)),
                _kv("general.name", 8, _string("one synthetic layer")),
                _kv("tokenizer.scores", 9, struct.pack("<IQ", 6, 3) + struct.pack("<3f", 0.5, 1.5, 2.5)),      # an array of f32
                _kv("tokenizer.tokens", 9, struct.pack("<IQ", 8, 2) + _string("a") + _string("bc"))]            # an array of strings
    metadata += [_kv(k, 4, struct.pack("<I", v)) for k, v in keys.items()]
    metadata += list(extra_metadata)
    # an unrelated tensor first, so that the layer's payloads do not start at the data offset
    entries = [("token_embd.weight", 0, (64, 3), np.arange(192, dtype=np.float32).view(np.uint8))]
    for role, (suffix, shape) in enumerate(zip(ROLE_SUFFIX, tensor_shapes(spec))):
        if role != drop:
            entries.append((f"blk.{layer}.{suffix}", spec.types[role], shape, spec.tensors[role]))
    entries.append(("output_norm.weight", 0, (spec.hidden,), np.ones(spec.hidden, np.float32).view(np.uint8)))
    table, payload, offsets = b"", b"", {}
    for name, kind, shape, data in entries:
        payload += b"\0" * (-len(payload) % alignment)
        table += _string(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        table += struct.pack("<IQ", kind, len(payload))
        offsets[name] = (len(payload), data.size)
        payload += data.tobytes()
    head = b"GGUF" + struct.pack("<IQQ", 3, len(entries), len(metadata)) + b"".join(metadata) + table
    head += b"\0" * (-len(head) % alignment)
    blob = head + payload
    with open(path, "wb") as out:
        out.write(blob if truncate is None else blob[:truncate])
    return {name: (len(head) + at, size) for name, (at, size) in offsets.items()}
