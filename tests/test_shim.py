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


# ─── the mirror as a drop-in for the reference's extension module ─────────────

REF_CORE = "/root/reference/moe_infer/_core.py"


def _load_reference_core():
    """Imports the reference's own wrapper module (numpy-only) with the mirror registered under the extension
    module's top-level name, exactly as `import _moe_infer_rs as _rs` (moe_infer/_core.py:14) expects it."""
    import importlib.util
    import sys
    sys.modules["_moe_infer_rs"] = rs
    spec = importlib.util.spec_from_file_location("ref_core_under_test", REF_CORE)
    mod = importlib.util.module_from_spec(spec)
    try:
        spec.loader.exec_module(mod)
    except ModuleNotFoundError as e:
        # the file ends with re-exports from the package `moe_infer.qwen35_moe` (tokenizer / vision tooling), which is
        # not importable as a package here; the wrapper classes above that line are already defined
        assert "moe_infer" in str(e)
    return mod


@pytest.mark.skipif(not os.path.exists(REF_CORE), reason="the reference tree is not on this machine")
def test_reference_wrappers_bind_to_the_mirror(tmp_path):
    core = _load_reference_core()
    m = core.Model(_tiny_dir(tmp_path))
    assert isinstance(m._inner, rs.Model) and "1 layers" in repr(m)
    c = core.Cache(m)
    c.reset()
    assert c.pos == 0 and "Cache(pos=0)" in repr(c)
    # every name the reference's wrappers and pipeline reach through __getattr__ exists on the mirror
    for name in ("embed_lookup", "forward", "forward_hidden", "forward_batched", "upload_cache", "download_cache",
                 "telemetry", "last_h_pre_norm", "mtp_forward", "mtp_reset", "mtp_rollback", "snapshot_state",
                 "restore_snapshot"):
        assert callable(getattr(rs.Engine, name)), name
    for name in ("record_engine_telemetry", "qwen35_moe_quantize", "qwen35_dense_quantize", "gemma4_moe_quantize",
                 "gemma4_dense_quantize", "PyHfRepo", "PyEngineSnapshot"):
        assert hasattr(rs, name), name
    with pytest.raises(ValueError, match="Unknown engine"):
        core.Engine(m, "NoSuchMode")
    with pytest.raises(NotImplementedError):
        core.HfRepo("Qwen/none")


def test_head_tensors_are_required_for_logits(tmp_path):
    """A directory without embedding table / final norm / lm_head: the logits entry points name what is missing
    instead of returning zeros; checked on the class without a device."""
    e = rs.Engine.__new__(rs.Engine)
    e._missing_head = ["model.embed_tokens", "lm_head"]
    with pytest.raises(RuntimeError, match="model.embed_tokens"):
        e.embed_lookup(np.array([1], np.int64))
    with pytest.raises(RuntimeError, match="lm_head"):
        e._need_head("model.norm.weight", "lm_head")
    e._need_head("model.norm.weight")


def test_model_dir_int8_and_reference_names(tmp_path):
    cfg = {"architectures": ["Qwen3_5MoeForConditionalGeneration_Stripped"], "text_config": {"hidden_size": 2048}}
    w = ModelDirWriter(str(tmp_path), cfg, {"scheme": "bq4"})
    q = (np.arange(4 * 64, dtype=np.int32).reshape(4, 64) % 255 - 127).astype(np.int8)
    w.add_int8("language_model.lm_head", q, np.array([0.5, 1, 2, 4], np.float32))
    w.add_bf16("language_model.model.norm.weight", np.full(2048, 0x3F80, np.uint16), flat=True)
    w.close()
    d = ModelDir(str(tmp_path))
    man = json.load(open(os.path.join(str(tmp_path), "model_weights.json")))["tensors"]
    assert man["language_model.lm_head.weight"]["dtype"] == "u8" and man["language_model.lm_head.scales"]["dtype"] == "f32"
    got = d.tensor("lm_head.weight")          # found under the reference's "language_model." prefix
    assert got.dtype == np.uint8 and np.array_equal(got.view(np.int8), q)
    assert d.tensor("lm_head.scales").dtype == np.float32 and d.tensor("model.norm.weight").shape == (2048,)
