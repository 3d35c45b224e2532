"""GGUF reader over the C ABI (no GPU needed).  The first nine cases are the reference's own parser tests
(yule-core/src/gguf.rs:629-790) rebuilt with this repository's writer; the rest cover the remaining checks
of parse_bytes (bounds, overlap, alignment, value types) and the model description."""

import dataclasses
import struct

import numpy as np
import pytest

from yule_b200 import GgufFile, ModelConfig, YuleGpuError, synth, DType

import gguf_writer as gw

MAX_STRING, MAX_TENSORS, MAX_KV = 1024 * 1024, 100_000, 100_000


def minimal() -> bytearray:
    return bytearray(struct.pack("<IIQQ", gw.MAGIC, 3, 0, 0))


def rejects(image, needle: str):
    with pytest.raises(YuleGpuError) as e:
        GgufFile.parse(bytes(image))
    assert needle in str(e.value), str(e.value)


def test_parse_minimal_gguf(native_libs):  # gguf.rs:643-653
    g = GgufFile.parse(minimal())
    assert (g.version, g.n_tensors, g.n_kv) == (3, 0, 0)


def test_reject_bad_magic(native_libs):  # gguf.rs:655-666
    img = minimal()
    img[0] = 0xFF
    rejects(img, "invalid magic")


def test_reject_bad_version(native_libs):  # gguf.rs:668-679
    img = minimal()
    img[4:8] = struct.pack("<I", 99)
    rejects(img, "unsupported version 99")


def test_reject_excessive_tensor_count(native_libs):  # gguf.rs:681-689
    img = minimal()
    img[8:16] = struct.pack("<Q", MAX_TENSORS + 1)
    rejects(img, "tensor count")


def test_reject_excessive_kv_count(native_libs):  # gguf.rs:691-698
    img = minimal()
    img[16:24] = struct.pack("<Q", MAX_KV + 1)
    rejects(img, "KV count")


def test_reject_truncated_file(native_libs):  # gguf.rs:700-706
    rejects(bytes(8), "gguf")


def test_parse_with_metadata(native_libs):  # gguf.rs:708-733
    g = GgufFile.parse(gw.build({"general.architecture": "llama"}, {}))
    assert g.get_str("general.architecture") == "llama"
    assert g.get_str("missing") is None and g.get_u32("general.architecture") is None


def test_parse_with_tensor(native_libs):  # gguf.rs:735-772 (a smaller F32 tensor, same structure)
    data = np.zeros(64 * 48, np.float32)
    g = GgufFile.parse(gw.build({}, {"output.weight": (data, 0, (64, 48))}))
    t = g.tensor(0)
    assert (t.name, t.shape, t.gguf_type, t.size_bytes) == ("output.weight", (64, 48), 0, 64 * 48 * 4)
    assert g.data_offset % 32 == 0


def test_reject_string_too_long(native_libs):  # gguf.rs:774-789
    img = struct.pack("<IIQQ", gw.MAGIC, 3, 0, 1) + struct.pack("<Q", MAX_STRING + 1)
    rejects(img, "exceeds maximum")


def test_value_types_and_widening(native_libs):
    """as_u32 takes u8/u16/u32 and non-negative i32; as_f64 takes f32/f64 (gguf.rs:53-103)."""
    meta = {"a": (gw.U8, 7), "b": (gw.U16, 300), "c": (gw.I32, 12), "d": (gw.I32, -1), "e": (gw.U64, 5), "f": (gw.F64, 2.5),
            "g": 1.5, "h": True, "i": (gw.I8, -3), "j": (gw.I16, -300), "k": (gw.I64, -5), "toks": ["x", "yy", "zzz"]}
    g = GgufFile.parse(gw.build(meta, {}))
    assert [g.get_u32(k) for k in "abcde"] == [7, 300, 12, None, None]
    assert g.get_f64("f") == 2.5 and g.get_f64("g") == 1.5 and g.get_f64("a") is None
    assert g.n_kv == len(meta)


def test_unknown_value_type_and_dtype(native_libs):
    img = struct.pack("<IIQQ", gw.MAGIC, 3, 0, 1) + gw._s("k") + struct.pack("<I", 13)
    rejects(img, "unknown GGUF value type")
    rejects(gw.build({}, {"t": (np.zeros(4, np.uint8), 31, (4,))}), "unknown GGUF dtype")


def test_quantized_sizes_and_alignment(native_libs):
    q4k = synth.random_blocks(DType.Q4_K, 1, 3 * 2)    # 3 rows of 512 columns
    q80 = synth.random_blocks(DType.Q8_0, 2, 5)        # 160 weights
    g = GgufFile.parse(gw.build({"general.alignment": 64}, {"a": (q4k, 12, (512, 3)), "b": (q80, 8, (160,))}, alignment=64))
    a, b = g.tensor(0), g.tensor(1)
    assert a.size_bytes == 6 * 144 and b.size_bytes == 5 * 34
    assert g.alignment == 64 and g.data_offset % 64 == 0 and b.offset % 64 == 0
    assert np.array_equal(g.tensor_bytes("a"), q4k) and np.array_equal(g.tensor_bytes("b"), q80)


def test_reject_tensor_out_of_bounds_and_overlap(native_libs):
    img = bytearray(gw.build({}, {"t": (np.zeros(256, np.float32), 0, (256,))}))
    rejects(img[:-64], "out of bounds")
    # two tensors whose byte ranges overlap: rewrite the second offset to 16
    img = bytearray(gw.build({}, {"a": (np.zeros(64, np.float32), 0, (64,)), "b": (np.zeros(64, np.float32), 0, (64,))}))
    pos = img.index(b"b\x01\x00\x00\x00") + 1 + 4 + 8 + 4  # name, n_dims, dim, dtype → offset field
    img[pos:pos + 8] = struct.pack("<Q", 16)
    rejects(img, "overlapping tensors")


def test_reject_too_many_dimensions_and_shape_overflow(native_libs):
    head = struct.pack("<IIQQ", gw.MAGIC, 3, 1, 0) + gw._s("t")
    rejects(head + struct.pack("<I", 9), "dimensions")
    rejects(head + struct.pack("<IQQIQ", 2, 2 ** 40, 2 ** 40, 0, 0), "shape")


def test_model_description(native_libs):
    """to_loaded_model + GpuTransformerRunner::new (gguf.rs:493-586, gpu_runner.rs:86-122)."""
    cfg = ModelConfig(dim=256, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=32, vocab_size=512, ff_dim=768, max_seq_len=64,
                      norm_eps=1e-6, rope_freq_base=500000.0)
    weights = synth.synthetic_model(cfg, seed=3)
    g = GgufFile.parse(gw.model_file(cfg, weights))
    got = g.model_config()
    assert got.norm_eps == pytest.approx(cfg.norm_eps, rel=1e-6)  # carried as f32
    assert dataclasses.replace(got, norm_eps=cfg.norm_eps) == cfg
    assert g.model_config(max_seq_len=16).max_seq_len == 16
    assert g.n_tensors == len(weights)
    # defaults: no eps / theta / kv heads / vocab keys → 1e-5, 1e4, kv = heads, vocab from the embedding table
    meta = {"general.architecture": "llama", "llama.embedding_length": 256, "llama.block_count": 2, "llama.attention.head_count": 8}
    cfg2 = ModelConfig(dim=256, n_layers=2, n_heads=8, n_kv_heads=8, head_dim=32, vocab_size=512, ff_dim=768, max_seq_len=4096)
    w2 = synth.synthetic_model(cfg2, seed=4)
    shapes = cfg2.tensor_shapes()
    tensors = {n: (d, int(t), (shapes[n][1], shapes[n][0]) if n in shapes else (256,)) for n, (d, t) in w2.items()}
    got2 = GgufFile.parse(gw.build(meta, tensors)).model_config()
    assert dataclasses.replace(got2, norm_eps=cfg2.norm_eps) == cfg2 and got2.norm_eps == pytest.approx(1e-5, rel=1e-6)
    # architectures outside the dense transformer path are refused, not mis-run
    for arch in ("mamba", "rwkv6", "mixtral", "bert"):
        with pytest.raises(YuleGpuError):
            GgufFile.parse(gw.model_file(cfg, weights, arch=arch)).model_config()


def test_architecture_variants_from_metadata(native_libs):
    """The variant fields RunnerConfig derives (yule-infer/src/model_runner.rs:417-460, gguf.rs:553-560)."""
    cfg = ModelConfig(dim=256, n_layers=1, n_heads=8, n_kv_heads=2, head_dim=32, vocab_size=64, ff_dim=256, max_seq_len=64,
                      norm_eps=1e-6)
    weights = synth.synthetic_model(cfg, seed=6)

    def parsed(arch, extra):
        shapes = cfg.tensor_shapes()
        tensors = {n: (d, int(t), (shapes[n][1], shapes[n][0]) if n in shapes else (cfg.dim,)) for n, (d, t) in weights.items()}
        meta = gw.llama_metadata(cfg, arch)
        meta.update(extra)
        return GgufFile.parse(gw.build(meta, tensors)).model_config()

    got = parsed("mistral", {"mistral.attention.sliding_window": 16})
    assert got.sliding_window == 16 and got.rotary_dim == 0 and not got.geglu and got.norm_weight_offset == 0.0
    got = parsed("phi3", {"phi3.rope.dimension_count": 16})
    assert got.rotary_dim == 16
    assert parsed("phi3", {"phi3.rope.dimension_count": 32}).rotary_dim == 0  # the whole head: no partial rotation
    got = parsed("gemma2", {"gemma2.attn_logit_softcapping": (gw.F64, 30.0), "gemma2.attention.attn_logit_softcapping": (gw.F64, 50.0)})
    assert got.geglu and got.norm_weight_offset == 1.0 and got.logit_softcap == 30.0 and got.attn_logit_softcap == 50.0
    # mixture of experts (model_runner.rs:395-407): the counts come from the metadata; a nonsensical pair is refused
    got = parsed("llama", {"llama.expert_count": 8, "llama.expert_used_count": 2})
    assert got.n_experts == 8 and got.n_experts_used == 2
    with pytest.raises(YuleGpuError, match="experts"):
        parsed("llama", {"llama.expert_count": 8, "llama.expert_used_count": 9})
    with pytest.raises(YuleGpuError, match="experts"):
        parsed("llama", {"llama.expert_count": 4})
    # default epsilon of Qwen / Phi / Gemma files that carry none: 1e-6 (model_runner.rs:414-417)
    shapes = cfg.tensor_shapes()
    tensors = {n: (d, int(t), (shapes[n][1], shapes[n][0]) if n in shapes else (cfg.dim,)) for n, (d, t) in weights.items()}
    meta = {k: v for k, v in gw.llama_metadata(cfg, "qwen2").items() if not k.endswith("layer_norm_rms_epsilon")}
    assert GgufFile.parse(gw.build(meta, tensors)).model_config().norm_eps == pytest.approx(1e-6, rel=1e-6)


def test_open_maps_a_file(native_libs, tmp_path):
    cfg = ModelConfig(dim=256, n_layers=1, n_heads=8, n_kv_heads=2, head_dim=32, vocab_size=64, ff_dim=256, max_seq_len=32)
    weights = synth.synthetic_model(cfg, seed=5)
    path = tmp_path / "m.gguf"
    path.write_bytes(gw.model_file(cfg, weights))
    g = GgufFile.open(str(path))
    assert dataclasses.replace(g.model_config(), norm_eps=cfg.norm_eps) == cfg
    assert np.array_equal(g.tensor_bytes("blk.0.ffn_down.weight"), np.asarray(weights["blk.0.ffn_down.weight"][0]).view(np.uint8))
    g.close()
    with pytest.raises(YuleGpuError):
        GgufFile.open(str(tmp_path / "absent.gguf"))
