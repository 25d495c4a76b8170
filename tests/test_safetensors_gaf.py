"""Host-side loader for converted checkpoints (CPU): header parsing, the reference's bits / group-size
inference rule, views into the memory map, error cases."""
import json
import struct

import numpy as np
import pytest

from talu_b200.safetensors_gaf import (GafFormatError, SafetensorsGaf, infer_bits_and_group, write_safetensors)


def _quantized(oracle, N, K, G, bits, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K), dtype=np.float32) * 0.02).astype(np.float32)
    return oracle.quantize(w, G, bits)


def test_inference_rule_matches_the_reference_loader():
    # models/load/transforms.zig:119-139: group sizes 32 / 64 / 128 are the plausible ones
    assert infer_bits_and_group(512, 64) == (8, 32)            # both readings plausible, nothing expected: not 4-bit
    assert infer_bits_and_group(512, 64, expected_dim=4096) == (4, 64)
    assert infer_bits_and_group(512, 64, expected_dim=2048) == (8, 32)
    assert infer_bits_and_group(512, 64, expected_bits=8) == (8, 32)
    assert infer_bits_and_group(1024, 32) == (8, 128)          # 4-bit reading: 256 per group, not plausible
    assert infer_bits_and_group(128, 32) == (4, 32)            # 8-bit reading: 16 per group, not plausible
    with pytest.raises(GafFormatError):
        infer_bits_and_group(100, 3)


def test_round_trip_of_a_converted_checkpoint(tmp_path, oracle):
    specs = {"model.layers.0.mlp.gate_proj": (96, 256, 64, 4), "model.layers.0.mlp.down_proj": (64, 512, 128, 4),
             "model.embed_tokens": (50, 128, 32, 8)}
    tensors, truth = {}, {}
    for i, (base, (N, K, G, bits)) in enumerate(specs.items()):
        p, s, b = _quantized(oracle, N, K, G, bits, i)
        truth[base] = (p, s, b, bits, G)
        tensors[base + ".weight"] = ("U32", p)
        tensors[base + ".scales"] = ("BF16", s)
        tensors[base + ".biases"] = ("BF16", b)
    tensors["model.norm.weight"] = ("F32", np.ones(128, np.float32))   # a tensor that is not quantized
    path = tmp_path / "model.safetensors"
    write_safetensors(path, tensors, metadata={"format": "pt"})
    with SafetensorsGaf(path) as st:
        assert sorted(st.gaf_bases()) == sorted(specs)
        assert st.metadata == {"format": "pt"}
        for base, (p, s, b, bits, G) in truth.items():
            # expected_dim disambiguates like the reference's loader does for mixed 4 / 8-bit models
            t = st.tensor(base, expected_dim=p.shape[1] * (32 // bits))
            assert (t.bits, t.group, t.scales_dtype) == (bits, G, 1)
            assert (t.N, t.K) == (p.shape[0], p.shape[1] * (32 // bits))
            assert np.array_equal(t.packed, p) and np.array_equal(t.scales, s) and np.array_equal(t.biases, b)
            # what the loader hands over dequantizes to the same bits as the source arrays
            assert np.array_equal(oracle.dequant_f32(t.packed, t.scales, t.biases, t.group, t.bits),
                                  oracle.dequant_f32(p, s, b, G, bits))


def test_config_quantization_decides_ambiguous_shapes(tmp_path, oracle):
    p, s, b = _quantized(oracle, 32, 512, 64, 8, 5)            # 8-bit, G = 64: packed width 128, 8 groups
    path = tmp_path / "m.safetensors"
    write_safetensors(path, {"w.weight": ("U32", p), "w.scales": ("BF16", s), "w.biases": ("BF16", b)})
    with SafetensorsGaf(path, config={"quantization": {"bits": 8, "group_size": 64}}) as st:
        t = st.tensor("w")
        assert (t.bits, t.group, t.K) == (8, 64, 512)
    with SafetensorsGaf(path, config={"quantization": {"bits": 4, "group_size": 128}}) as st:
        t = st.tensor("w")                                      # the other plausible reading of the same shapes
        assert (t.bits, t.group, t.K) == (4, 128, 1024)


def test_malformed_files_are_rejected(tmp_path, oracle):
    p, s, b = _quantized(oracle, 16, 128, 32, 4, 9)
    good = tmp_path / "g.safetensors"
    write_safetensors(good, {"w.weight": ("U32", p), "w.scales": ("BF16", s), "w.biases": ("F16", b)})
    with SafetensorsGaf(good) as st, pytest.raises(GafFormatError):
        st.tensor("w")                                          # scales and biases of different types
    write_safetensors(good, {"w.weight": ("U32", p), "w.scales": ("BF16", s[:, :2]), "w.biases": ("BF16", b)})
    with SafetensorsGaf(good) as st, pytest.raises(GafFormatError):
        st.tensor("w")                                          # sizes disagree
    bad = tmp_path / "b.safetensors"
    bad.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(GafFormatError):
        SafetensorsGaf(bad)
    hdr = json.dumps({"w.weight": {"dtype": "U32", "shape": [16, 16], "data_offsets": [0, 4096]}}).encode()
    bad.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with SafetensorsGaf(bad) as st, pytest.raises((GafFormatError, KeyError)):
        st.tensor("w")
