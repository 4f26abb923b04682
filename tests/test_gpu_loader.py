"""lthn_model_load_dir: a checkpoint directory loaded by the library gives the model that uploading
the same tensors through lthn_model_upload_* gives (model.Load, model/load.go:19-108, followed by
the engine's binding of model.LoadedModel)."""
import json
import os

import numpy as np
import pytest

from checkpoint_util import effective_norms, write_checkpoint
from decoder_util import MID, SMALL, build_device, build_oracle, synth_weights, widen_linears

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("norm_dtype,shards,prefix,nest", [("BF16", 1, "", False), ("F32", 3, "language_model.", True),
                                                           ("F16", 2, "", False)])
def test_loaded_checkpoint_equals_uploaded_tensors(oracle, tmp_path, norm_dtype, shards, prefix, nest):
    import lthn
    cfg = SMALL
    w, norms = synth_weights(oracle, lthn, cfg, seed=31, random_norms=True)
    d = str(tmp_path / "ck")
    write_checkpoint(d, cfg, w, norms, norm_dtype=norm_dtype, shards=shards, prefix=prefix, nest_text_config=nest)
    loaded = lthn.Model.load_dir(d, max_len=96)
    # the uploaded twin gets the norm weights the (1+w) fold produces from what the file stores
    eff = effective_norms(oracle, norms, norm_dtype)
    up = build_device(lthn, cfg, w, eff, 96)
    ids = np.random.default_rng(2).integers(0, cfg["vocab"], 20).astype(np.int32)
    a, b = loaded.open_session(), up.open_session()
    a.prefill(ids)
    la = a.logits()
    ta = a.decode_greedy(16)
    b.prefill(ids)
    assert np.array_equal(la, b.logits())
    assert np.array_equal(ta, b.decode_greedy(16))
    # and the CPU reference decoder on the folded norms agrees with the loaded model
    od = build_oracle(oracle, cfg, w, eff, 96)
    want_logits = od.forward(ids)
    rms = float(np.sqrt(np.mean(want_logits.astype(np.float64) ** 2)))
    assert float(np.max(np.abs(la - want_logits))) <= 1e-2 * rms
    a.close(); b.close(); loaded.close(); up.close()


def test_mixed_precision_checkpoint_loads(oracle, tmp_path, monkeypatch):
    """A QAT pack whose quantization block overrides the MLP projections to 8 bits (model/quant_config.go:39-88):
    the loaded model equals the one built from the same tensors by upload, and follows the CPU decoder (the 20-row
    prompt on the f32-grade kernels: LTHN_CUDA_BATCH_F32=1 keeps the 8-bit projections off the bf16-contract GEMM)."""
    import lthn
    monkeypatch.setenv("LTHN_CUDA_BATCH_F32", "1")
    cfg = SMALL
    w, norms = synth_weights(oracle, lthn, cfg, seed=31, random_norms=True)
    w = widen_linears(oracle, lthn, cfg, w, seed=31)
    d = str(tmp_path / "ck")
    write_checkpoint(d, cfg, w, norms, shards=2)
    loaded = lthn.Model.load_dir(d, max_len=96)
    eff = effective_norms(oracle, norms, "BF16")
    up = build_device(lthn, cfg, w, eff, 96)
    assert loaded.weight_bytes == up.weight_bytes
    ids = np.random.default_rng(2).integers(0, cfg["vocab"], 20).astype(np.int32)
    a, b = loaded.open_session(), up.open_session()
    a.prefill(ids)
    la = a.logits()
    ta = a.decode_greedy(16)
    b.prefill(ids)
    assert np.array_equal(la, b.logits())
    assert np.array_equal(ta, b.decode_greedy(16))
    od = build_oracle(oracle, cfg, w, eff, 96)
    want_logits = od.forward(ids)
    rms = float(np.sqrt(np.mean(want_logits.astype(np.float64) ** 2)))
    assert float(np.max(np.abs(la - want_logits))) <= 1e-2 * rms
    a.close(); b.close(); loaded.close(); up.close()


def test_load_rejects_what_the_engine_does_not_serve(oracle, tmp_path):
    import lthn
    cfg = SMALL
    w, norms = synth_weights(oracle, lthn, cfg, seed=31)
    d = str(tmp_path / "ck")
    # an 8-bit per-module override outside the MLP projections: named and refused
    w8 = widen_linears(oracle, lthn, cfg, w, seed=31, roles=("q",), layers=[1])
    write_checkpoint(d, cfg, w8, norms)
    with pytest.raises(lthn.LthnError) as e:
        lthn.Model.load_dir(d, max_len=32)
    assert "model.layers.1.self_attn.q_proj" in str(e.value) and "8-bit" in str(e.value)
    # an override the tensor does not follow
    write_checkpoint(d, cfg, w, norms, quant_extra={"model.layers.1.mlp.down_proj": {"group_size": 64, "bits": 8}})
    with pytest.raises(lthn.LthnError) as e:
        lthn.Model.load_dir(d, max_len=32)
    assert "model.layers.1.mlp.down_proj" in str(e.value) and "geometry" in str(e.value)
    # a missing tensor
    write_checkpoint(d, cfg, w, norms)
    import checkpoint_util as cu
    t = cu.checkpoint_tensors(cfg, w, norms)
    del t["model.layers.0.self_attn.k_norm.weight"]
    cu.write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(lthn.LthnError) as e:
        lthn.Model.load_dir(d, max_len=32)
    assert "k_norm" in str(e.value)
    # sliding-window layers follow gemma3's pattern; uniform_attention runs every block with full attention.
    # With a window of 8 the two differ once the prompt is longer than the window.
    write_checkpoint(d, cfg, w, norms, extra_config={"sliding_window": 8, "sliding_window_pattern": 2, "rope_local_base_freq": 10000.0})
    ids = (np.arange(24, dtype=np.int32) * 37) % cfg["vocab"]
    outs = []
    for uniform in (False, True):
        m = lthn.Model.load_dir(d, max_len=48, uniform_attention=uniform)
        s = m.open_session()
        s.prefill(ids)
        outs.append(s.logits().copy())
        assert len(s.decode_greedy(3)) == 3
        s.close(); m.close()
    assert float(np.max(np.abs(outs[0] - outs[1]))) > 1e-3
    # geometry that contradicts the quantization block
    cfgj = json.load(open(os.path.join(d, "config.json")))
    cfgj["quantization"]["language_model.model.layers.0.mlp.gate_proj"] = {"group_size": 32, "bits": 4}
    json.dump(cfgj, open(os.path.join(d, "config.json"), "w"))
    with pytest.raises(lthn.LthnError) as e:
        lthn.Model.load_dir(d, max_len=32, uniform_attention=True)
    assert "geometry" in str(e.value) and "gate_proj" in str(e.value)
    # a checkpoint quantised at another group size altogether
    del cfgj["quantization"]["language_model.model.layers.0.mlp.gate_proj"]
    cfgj["quantization"]["group_size"] = 32
    json.dump(cfgj, open(os.path.join(d, "config.json"), "w"))
    with pytest.raises(lthn.LthnError) as e:
        lthn.Model.load_dir(d, max_len=32, uniform_attention=True)
    assert "group-64" in str(e.value)
