"""Host-side mirror of the reference's loader interface: validation and error behaviour (no GPU)."""
import numpy as np
import pytest
import torch

import oracle
from scratchy_b200 import AffineQuantLinear, Fp8Linear, GpuWeights, LinearLayer, ScratchyCudaError, synth
from scratchy_b200.layers import affine_packed_cols, load_layered_linear_affine_quant


def _ckpt(N=16, K=128, prefix="model.layers.0.self_attn.q_proj", scale_dtype=torch.bfloat16):
    w, s, b = synth.affine_int4_weights(N, K, 64, 3)
    return {
        f"{prefix}.weight": torch.from_numpy(w.view(np.int32)),
        f"{prefix}.scales": torch.from_numpy(s.view(np.int16)).view(torch.bfloat16).to(scale_dtype),
        f"{prefix}.biases": torch.from_numpy(b.view(np.int16)).view(torch.bfloat16).to(scale_dtype),
    }


def test_affine_packed_cols_law():
    # crates/targets/metal/src/layers_quant.rs:46-48
    assert affine_packed_cols(3072, 4) == 384 and affine_packed_cols(64, 4) == 8


def test_load_rejects_wrong_in_features():
    gw = GpuWeights(_ckpt())
    with pytest.raises(ValueError, match="in_features=128.*expects in_features=256"):
        LinearLayer.load_affine_quant(gw, "model.layers.0.self_attn.q_proj", 64, 4, 256)


def test_load_rejects_unpinned_or_mismatched_scale_dtype():
    with pytest.raises(ValueError, match="no scale dtype pinned"):
        AffineQuantLinear.load(GpuWeights(_ckpt(), scale_dtype=None), "model.layers.0.self_attn.q_proj", 64, 4, 128)
    with pytest.raises(ValueError, match="on disk"):
        AffineQuantLinear.load(GpuWeights(_ckpt(scale_dtype=torch.float16)), "model.layers.0.self_attn.q_proj",
                               64, 4, 128)


def test_load_missing_tensor_is_a_key_error():
    with pytest.raises(KeyError, match="not found"):
        AffineQuantLinear.load(GpuWeights({}), "nope", 64, 4, 128)


def test_cpu_tensors_are_refused_there_is_no_cpu_path():
    gw = GpuWeights(_ckpt())
    with pytest.raises(ScratchyCudaError, match="no CPU path"):
        AffineQuantLinear.load(gw, "model.layers.0.self_attn.q_proj", 64, 4, 128)
    with pytest.raises(ScratchyCudaError, match="no CPU path"):
        Fp8Linear.from_tensors(torch.zeros((16, 128), dtype=torch.uint8), torch.ones(16))


def test_only_the_four_bit_preset_is_lowered():
    ck = _ckpt()
    with pytest.raises(ScratchyCudaError):
        AffineQuantLinear.from_tensors(ck["model.layers.0.self_attn.q_proj.weight"],
                                       ck["model.layers.0.self_attn.q_proj.scales"],
                                       ck["model.layers.0.self_attn.q_proj.biases"], 64, 8)


def test_layered_loader_walks_root_i_suffix():
    tensors = {}
    for i in range(2):
        tensors.update(_ckpt(prefix=f"model.layers.{i}.mlp.up_proj"))
    gw = GpuWeights(tensors)
    with pytest.raises(ScratchyCudaError):      # reaches the repack of layer 0, which needs a device
        load_layered_linear_affine_quant(gw, 2, "model.layers", "mlp.up_proj", 64, 4, 128)
    assert not gw.contains("model.layers.0.mlp.up_proj.weight")   # layer 0 was taken
    assert gw.contains("model.layers.1.mlp.up_proj.weight")


def test_synthetic_weight_packing_matches_the_checkpoint_nibble_order():
    # element k of a row sits at bits [4*(k%8), +4) of word k//8 == low nibble first in the byte stream
    w, s, b = synth.affine_int4_weights(4, 64, 64, 5)
    packed = w.view(np.uint8).reshape(-1)
    codes = np.empty(4 * 64, np.uint8)
    codes[0::2] = packed & 0xF
    codes[1::2] = packed >> 4
    words = w.reshape(-1)
    for idx in (0, 1, 7, 8, 63, 64, 255):
        assert codes[idx] == (int(words[idx // 8]) >> (4 * (idx % 8))) & 0xF
    scale_one = np.full(4, 0x3F80, np.uint16)
    zero = np.zeros(4, np.uint16)
    wd = oracle.affine_dequant_b4(packed, scale_one, zero, 4, 64, 64)
    assert np.array_equal(oracle.bf16_bits_to_f32(wd).reshape(-1).astype(np.uint8), codes)


# ---- `load_rows_concat` (crates/targets/metal/src/layers_quant.rs:363-450): the checks run before any upload
def _qkv_ckpt(**kw):
    ck = {}
    for name, rows in (("q_proj", 32), ("k_proj", 16), ("v_proj", 16)):
        ck.update(_ckpt(N=rows, K=128, prefix=f"a.{name}", **kw))
    return ck


def test_rows_concat_refuses_an_empty_list_a_bias_and_mismatched_parts():
    with pytest.raises(ValueError, match="empty prefix list"):
        AffineQuantLinear.load_rows_concat(GpuWeights(_qkv_ckpt()), [], 64, 4, 128)
    ck = _qkv_ckpt()
    ck["a.k_proj.bias"] = torch.zeros(16)
    with pytest.raises(ValueError, match="carries no bias"):
        AffineQuantLinear.load_rows_concat(GpuWeights(ck), ["a.q_proj", "a.k_proj"], 64, 4, 128)
    with pytest.raises(ValueError, match="not a bits=4 packing of in_features=256"):
        AffineQuantLinear.load_rows_concat(GpuWeights(_qkv_ckpt()), ["a.q_proj"], 64, 4, 256)
    with pytest.raises(ValueError, match="on disk"):
        AffineQuantLinear.load_rows_concat(GpuWeights(_qkv_ckpt(scale_dtype=torch.float16)), ["a.q_proj"], 64, 4, 128)
    with pytest.raises(ValueError, match="no scale dtype pinned"):
        AffineQuantLinear.load_rows_concat(GpuWeights(_qkv_ckpt(), scale_dtype=None), ["a.q_proj"], 64, 4, 128)
    ck = _qkv_ckpt()
    ck["a.v_proj.scales"] = ck["a.v_proj.scales"][:8]
    with pytest.raises(ValueError, match=r"are not \[16, 2\]"):
        AffineQuantLinear.load_rows_concat(GpuWeights(ck), ["a.q_proj", "a.v_proj"], 64, 4, 128)


def test_rows_concat_leaves_the_parts_in_the_store():
    gw = GpuWeights(_qkv_ckpt())
    with pytest.raises(ScratchyCudaError, match="no CPU path"):        # validation passed; the upload refuses CPU tensors
        AffineQuantLinear.load_rows_concat(gw, ["a.q_proj", "a.k_proj", "a.v_proj"], 64, 4, 128)
    assert gw.contains("a.q_proj.weight") and gw.contains("a.v_proj.biases")


def test_decode_rope_tables_and_checkpoint_shapes():
    from scratchy_b200 import decode
    cos, sin = decode.rope_tables(8, 64, 10000.0)
    assert cos.shape == (8, 64) and np.allclose(cos[0], 1.0) and np.allclose(sin[0], 0.0)
    assert np.allclose(cos[3, :32], np.cos(3.0 / 10000.0 ** (np.arange(32) * 2 / 64)), atol=1e-6)
    assert np.array_equal(cos[:, :32], cos[:, 32:])
    cfg = decode.LlamaConfig(hidden=128, n_layers=1, n_q_heads=2, n_kv_heads=1, head_dim=64, intermediate=256, vocab=64)
    ck = decode.synthetic_checkpoint(cfg, 0)
    assert ck["model.layers.0.self_attn.q_proj.weight"].shape == (128, 16)
    assert ck["model.layers.0.self_attn.k_proj.scales"].shape == (64, 2)
    assert ck["model.layers.0.mlp.down_proj.weight"].shape == (128, 32)
    assert ck["lm_head.weight"].shape == (64, 16) and ck["model.embed_tokens.weight"].shape == (64, 128)
    with pytest.raises(ScratchyCudaError, match="no CPU path"):
        decode.LlamaDecoder(cfg, ck, "cpu")


# ---- checkpoint files (crates/layers/src/weights.rs:473-520, 847-880)
def test_safetensors_round_trip_single_file_and_index(tmp_path):
    import json
    from scratchy_b200.weights import CheckpointWeights, SafetensorsFile, write_safetensors
    w, s, b = synth.affine_int4_weights(16, 128, 64, 1)
    e4 = np.arange(32, dtype=np.uint8).reshape(4, 8)
    one = tmp_path / "one"
    one.mkdir()
    write_safetensors(str(one / "model.safetensors"),
                      {"a.weight": w, "a.scales": (s, "BF16"), "a.biases": (b, "BF16"), "f.weight": (e4, "F8_E4M3"),
                       "f.weight_scale": np.linspace(0.1, 0.4, 4, dtype=np.float32)}, {"format": "pt"})
    f = SafetensorsFile(str(one / "model.safetensors"))
    assert f.entries["a.weight"][:2] == ("U32", (16, 16)) and f.metadata == {"format": "pt"}
    gw = CheckpointWeights.from_dir(str(one), "cpu")
    assert gw.contains("a.scales") and not gw.contains("a.bias")
    t = gw.take("a.scales")
    assert t.dtype == torch.bfloat16 and np.array_equal(t.view(torch.int16).numpy().view(np.uint16), s)
    assert np.array_equal(gw.peek("a.weight").numpy().view(np.uint32), w) and gw.contains("a.weight")
    assert np.array_equal(gw.take("a.weight").numpy().view(np.uint32), w) and not gw.contains("a.weight")
    assert gw.take("f.weight").dtype == torch.uint8
    with pytest.raises(KeyError, match="not found"):
        gw.take("a.weight")
    # sharded: an index routes names to shards
    two = tmp_path / "two"
    two.mkdir()
    write_safetensors(str(two / "model-00001-of-00002.safetensors"), {"a.weight": w})
    write_safetensors(str(two / "model-00002-of-00002.safetensors"), {"a.scales": (s, "BF16"), "a.biases": (b, "BF16")})
    (two / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {
        "a.weight": "model-00001-of-00002.safetensors", "a.scales": "model-00002-of-00002.safetensors",
        "a.biases": "model-00002-of-00002.safetensors"}}))
    gw = CheckpointWeights.from_dir(str(two), "cpu")
    assert gw.names() == ["a.biases", "a.scales", "a.weight"]
    with pytest.raises(ValueError, match="in_features=128.*expects in_features=256"):
        LinearLayer.load_affine_quant(gw, "a", 64, 4, 256)
    # unindexed shards are found too; an empty directory is refused like the reference does
    os_dir = tmp_path / "three"
    os_dir.mkdir()
    write_safetensors(str(os_dir / "part.safetensors"), {"x": np.zeros(3, np.float32)})
    assert CheckpointWeights.from_dir(str(os_dir), "cpu").contains("x")
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(FileNotFoundError, match="No safetensors files found"):
        CheckpointWeights.from_dir(str(empty), "cpu")


def test_safetensors_refuses_a_header_that_lies(tmp_path):
    import json
    import struct
    from scratchy_b200.weights import SafetensorsFile
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p = tmp_path / "bad.safetensors"
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + bytes(8))
    with pytest.raises(ValueError, match="spans 8 bytes, its shape needs 16"):
        SafetensorsFile(str(p))
    p.write_bytes(bytes([1, 2]))
    with pytest.raises(ValueError, match="too short"):
        SafetensorsFile(str(p))
