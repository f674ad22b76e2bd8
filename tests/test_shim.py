"""The `_moe_infer_rs` mirror: CPU-side behaviour (formats, argument checks, error classes)."""
import json
import os

import numpy as np
import pytest

from moe_infer_b200 import _moe_infer_rs as rs
from moe_infer_b200.modeldir import ModelDir, ModelDirWriter


def _tiny_dir(tmp_path, arch="Qwen3_5MoeForConditionalGeneration_Stripped"):
    cfg = {"architectures": [arch], "text_config": {"hidden_size": 2048, "num_hidden_layers": 1, "vocab_size": 100,
                                                    "num_experts": 4, "num_experts_per_tok": 4,
                                                    "moe_intermediate_size": 512,
                                                    "shared_expert_intermediate_size": 512}}
    w = ModelDirWriter(str(tmp_path), cfg, {"scheme": "bq4"})
    w.add_bf16("model.layers.0.post_attention_layernorm.weight", np.full(2048, 0x3F80, np.uint16))
    w.add_q4("model.layers.0.mlp.shared_expert_gate", np.arange(256, dtype=np.uint32).reshape(1, 256),
             np.ones((1, 32), np.uint16), np.ones((1, 32), np.uint16))
    w.close()
    return str(tmp_path)


def test_model_dir_round_trip(tmp_path):
    d = ModelDir(_tiny_dir(tmp_path))
    assert d.get_usize("hidden_size") == 2048 and d.architecture.endswith("_Stripped")
    man = json.load(open(os.path.join(str(tmp_path), "model_weights.json")))
    assert all(t["offset"] % 64 == 0 for t in man["tensors"].values())          # src/quantize.rs:251-256
    assert man["tensors"]["model.layers.0.mlp.shared_expert_gate.weight"]["dtype"] == "u32"  # "u32" means 4-bit words
    w, s, b = d.q4("model.layers.0.mlp.shared_expert_gate")
    assert w.shape == (1, 256) and w[0, 5] == 5 and s.dtype == np.uint16
    assert d.tensor("model.layers.0.nope") is None


def test_model_errors(tmp_path):
    with pytest.raises(RuntimeError):
        rs.Model(str(tmp_path / "missing"))
    m = rs.Model(_tiny_dir(tmp_path))
    assert "1 layers" in repr(m)
    with pytest.raises(ValueError, match="Unknown engine"):
        rs.Engine(m, "NoSuchMode")
    with pytest.raises(ValueError, match="num_active_experts"):
        rs.Engine(m, "Qwen35MoEFusedExp2", 5)  # > num_experts_per_tok


def test_cache_save_load(tmp_path):
    m = rs.Model(_tiny_dir(tmp_path))
    c = rs.Cache(m)
    c.pos = 7
    c.save(str(tmp_path / "c.bin"), str(tmp_path / "c.json"))
    c2 = rs.Cache.load(str(tmp_path / "c.bin"), str(tmp_path / "c.json"))
    assert c2.pos == 7 and c2.cpu_dirty
    c2.reset()
    assert c2.pos == 0
    with pytest.raises(IOError):
        rs.Cache.load(str(tmp_path / "nope.bin"), str(tmp_path / "nope.json"))


def test_quantize_argument_checks(tmp_path):
    with pytest.raises(ValueError):
        rs.qwen35_moe_quantize(str(tmp_path), str(tmp_path / "o"), version="3.4")
    with pytest.raises(ValueError):
        rs.qwen35_moe_quantize(str(tmp_path), str(tmp_path / "o"), version="3.6", scheme="fp4")
    with pytest.raises(NotImplementedError):
        rs.gemma4_moe_quantize("a", "b")
    rs.record_engine_telemetry(False)
