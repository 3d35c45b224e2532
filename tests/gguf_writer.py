"""A minimal GGUF v3 writer for the tests: header, typed key-value pairs, tensor infos, aligned data
section — the layout yule-core/src/gguf.rs:271-431 reads."""

import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
MAGIC = 0x46554747


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def _value(v) -> bytes:
    """(type, payload) chosen from the Python type; tuples ``(type_id, value)`` force a type."""
    if isinstance(v, tuple):
        t, x = v
        fmt = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q",
               F64: "<d"}[t]
        return struct.pack("<I", t) + struct.pack(fmt, x)
    if isinstance(v, bool):
        return struct.pack("<IB", BOOL, int(v))
    if isinstance(v, int):
        return struct.pack("<II", U32, v)
    if isinstance(v, float):
        return struct.pack("<If", F32, v)
    if isinstance(v, str):
        return struct.pack("<I", STRING) + _s(v)
    if isinstance(v, list):  # array of strings
        return struct.pack("<IIQ", ARRAY, STRING, len(v)) + b"".join(_s(x) for x in v)
    raise TypeError(type(v))


def build(metadata: dict, tensors: dict, alignment: int = 32, version: int = 3) -> bytes:
    """``tensors``: name → (uint8 array of raw bytes, gguf type id, shape in GGUF order)."""
    out = struct.pack("<IIQQ", MAGIC, version, len(tensors), len(metadata))
    for k, v in metadata.items():
        out += _s(k) + _value(v)
    offset, blobs = 0, []
    for name, (data, type_id, shape) in tensors.items():
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        out += _s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        out += struct.pack("<IQ", type_id, offset)
        blobs.append((offset, data))
        offset = (offset + data.size + alignment - 1) // alignment * alignment
    pad = (-len(out)) % alignment
    out += b"\0" * pad
    body = bytearray(offset)
    for off, data in blobs:
        body[off:off + data.size] = data.tobytes()
    return out + bytes(body)


def llama_metadata(cfg, arch: str = "llama") -> dict:
    moe = {f"{arch}.expert_count": cfg.n_experts, f"{arch}.expert_used_count": cfg.n_experts_used} if cfg.n_experts else {}
    return {**moe, "general.architecture": arch, "general.name": "synthetic", f"{arch}.context_length": cfg.max_seq_len,
            f"{arch}.embedding_length": cfg.dim, f"{arch}.block_count": cfg.n_layers,
            f"{arch}.attention.head_count": cfg.n_heads, f"{arch}.attention.head_count_kv": cfg.n_kv_heads,
            f"{arch}.attention.layer_norm_rms_epsilon": float(cfg.norm_eps), f"{arch}.rope.freq_base": float(cfg.rope_freq_base),
            "tokenizer.ggml.vocab_size": cfg.vocab_size}


def model_file(cfg, weights: dict, arch: str = "llama") -> bytes:
    """A GGUF image of a synthetic model: ``weights`` as produced by ``synth.synthetic_model``."""
    shapes = {**cfg.tensor_shapes(True), **cfg.tensor_shapes(False)} if cfg.n_experts else cfg.tensor_shapes()
    tensors = {}
    for name, (data, dt) in weights.items():
        if name in shapes:
            rows, cols = shapes[name]
            tensors[name] = (data, int(dt), (cols, rows))
        else:
            tensors[name] = (data, int(dt), (cfg.dim,))
    return build(llama_metadata(cfg, arch), tensors)
