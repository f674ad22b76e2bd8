"""CPU-only: the converter's naming, storage-type and sanitisation rules against the reference's own unit tests
(src/quantize/qwen35_moe/bq4.rs:149-168, common.rs:425-443) and, where the reference tree is present, against
every entry of its name table."""
import json
import os

import numpy as np
import pytest

from moe_infer_b200 import quantize as qz

REF_TABLE = "/root/reference/src/quantize/qwen35_moe/name_mapping.json"


def test_storage_types_of_the_reference_unit_tests():
    L0 = "language_model.model.layers.0."
    assert qz.storage_type(L0 + "self_attn.q_proj.weight", [8192, 2048], "bq4") == "bf16"
    assert qz.storage_type(L0 + "mlp.switch_mlp.gate_up_proj.weight", [256, 2048], "bq4") == "int4"
    assert qz.storage_type(L0 + "input_layernorm.weight", [2048], "bq4") == "bf16"
    assert qz.storage_type(L0 + "linear_attn.A_log", [128], "bq4") == "f32"
    assert qz.storage_type("language_model.model.embed_tokens.scales", [32, 32], "bq4") == "bf16"
    assert qz.storage_type("language_model.lm_head.weight", [1000, 2048], "bq4") == "int8"
    assert qz.storage_type(L0 + "mlp.gate.weight", [256, 2048], "bq4") == "bf16"
    assert qz.storage_type(L0 + "mlp.shared_expert_gate.weight", [1, 2048], "bq4") == "int4"
    # the INT4 scheme packs every matrix
    for name in ("self_attn.q_proj.weight", "mlp.gate.weight"):
        assert qz.storage_type(L0 + name, [256, 2048], "int4") == "int4"
    assert qz.storage_type("language_model.lm_head.weight", [1000, 2048], "int4") == "int4"
    assert qz.storage_type(L0 + "linear_attn.conv1d.weight", [8, 4, 1], "int4") == "bf16"
    assert qz.storage_type(L0 + "linear_attn.dt_bias", [32], "int4") == "bf16"


def test_block_names():
    assert qz._block_of("language_model.model.layers.3.self_attn.q_proj") == "self_attn.q_proj"
    assert qz._block_of("language_model.lm_head") == "lm_head"
    assert qz._block_of("mtp.layers.0.mlp.gate") == "mlp.gate"
    assert qz._block_of("mtp.fc") == "fc"


def test_layer_numbers():
    assert qz.layer_of("model.language_model.layers.17.mlp.experts.down_proj") == 17
    assert qz.layer_of("mtp.layers.0.mlp.experts.gate_up_proj") == 0
    assert qz.layer_of("lm_head.weight") is None
    assert qz.layer_of("players.x.layers.4.w") == 4


def test_zero_centred_norms():
    yes = ["language_model.model.layers.1.input_layernorm.weight", "language_model.model.layers.1.post_attention_layernorm.weight",
           "language_model.model.layers.3.self_attn.q_norm.weight", "language_model.model.layers.3.self_attn.k_norm.weight",
           "mtp.pre_fc_norm_hidden.weight", "mtp.pre_fc_norm_embedding.weight", "language_model.model.norm.weight", "mtp.norm.weight"]
    no = ["language_model.model.layers.0.linear_attn.norm.weight", "language_model.model.layers.0.mlp.gate.weight"]
    assert all(qz.is_zero_centred_norm(n) for n in yes) and not any(qz.is_zero_centred_norm(n) for n in no)
    w = np.array([0.5, -0.25], np.float32)
    assert np.array_equal(qz.sanitise(yes[0], w, "3.6"), w + 1) and np.array_equal(qz.sanitise(yes[0], w, "3.5"), w)
    assert np.array_equal(qz.sanitise(no[0], w, "3.6"), w)


def test_conv1d_axes():
    v = np.arange(2 * 3 * 4, dtype=np.float32).reshape(2, 3, 4)
    out = qz.sanitise("language_model.model.layers.0.linear_attn.conv1d.weight", v, "3.5")
    assert out.shape == (2, 4, 3) and out[1, 2, 0] == v[1, 0, 2] and out.flags["C_CONTIGUOUS"]


def test_manifest_config_block():
    cfg = qz.manifest_config({"hidden_size": 2048, "num_hidden_layers": 8, "mtp_num_hidden_layers": 1, "num_experts": 256,
                              "rope_parameters": {"rope_theta": 5e6, "partial_rotary_factor": 0.5}})
    assert cfg["num_hidden_layers"] == 9 and cfg["mtp_num_hidden_layers"] == 1
    assert cfg["layer_types"] == ["linear_attention"] * 3 + ["full_attention"] + ["linear_attention"] * 3 + ["full_attention"] * 2
    assert cfg["rope_theta"] == 5e6 and cfg["partial_rotary_factor"] == 0.5 and cfg["rms_norm_eps"] == 1e-6
    assert cfg["linear_num_value_heads"] == 32 and cfg["linear_num_key_heads"] == 16


@pytest.mark.skipif(not os.path.exists(REF_TABLE), reason="the reference tree is not on this machine")
def test_name_rules_reproduce_the_reference_table():
    table = json.load(open(REF_TABLE))
    checked = 0
    for hf, want in table.items():
        for token, values in (("{L}", (0, 7, 39)), ("{B}", (0, 26)), ("", (None,))):
            if token and token not in hf:
                continue
            if not token and ("{L}" in hf or "{B}" in hf):
                continue
            for v in values:
                a, b = (hf.replace(token, str(v)), want.replace(token, str(v))) if token else (hf, want)
                # the table also lists the scale / bias names of already-quantised (MLX) expert tensors, whose
                # abbreviated HF-side keys no safetensors checkpoint carries
                if ".mlp.experts.do." in a or ".mlp.experts.gate_." in a:
                    continue
                assert qz.manifest_name(a) == b, (a, b)
                checked += 1
    assert checked > 300
