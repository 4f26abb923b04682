"""Host half of the checkpoint loader (config.json + safetensors directory parsing), no GPU:
lthn_checkpoint_inspect on synthetic gemma3-style checkpoints and on malformed ones. The rules are
the reference's: model/load.go:19-108, model/safetensors/header_parse.go, sharded.go,
model/quant_config.go:39-88."""
import json
import os
import struct

import numpy as np
import pytest

from checkpoint_util import write_checkpoint, write_safetensors
from decoder_util import SMALL, synth_weights


@pytest.fixture(scope="module")
def small_model(oracle):
    import lthn
    return synth_weights(oracle, lthn, SMALL, seed=4, random_norms=True)


def test_inspect_reads_dimensions_quantization_and_shards(small_model, tmp_path):
    import lthn
    w, norms = small_model
    write_checkpoint(str(tmp_path / "one"), SMALL, w, norms)
    info = lthn.checkpoint_inspect(str(tmp_path / "one"))
    assert (info["layers"], info["hidden"], info["q_heads"], info["kv_heads"], info["head_dim"], info["ffn"], info["vocab"]) == \
           (SMALL["layers"], SMALL["hidden"], SMALL["q_heads"], SMALL["kv_heads"], SMALL["head_dim"], SMALL["ffn"], SMALL["vocab"])
    assert (info["group_size"], info["bits"], info["shards"], info["overrides"]) == (64, 4, 1, 0)
    assert info["tensors"] == SMALL["layers"] * (7 * 3 + 6) + 3 + 1
    # sharded, the text fields nested under text_config, names under language_model., one per-module override
    write_checkpoint(str(tmp_path / "three"), SMALL, w, norms, shards=3, prefix="language_model.", nest_text_config=True,
                     quant_extra={"language_model.model.layers.0.mlp.down_proj": {"group_size": 64, "bits": 8}})
    info3 = lthn.checkpoint_inspect(str(tmp_path / "three"))
    assert info3["shards"] == 3 and info3["tensors"] == info["tensors"] and info3["overrides"] == 1
    assert info3["model_type"] == "gemma3" and info3["hidden"] == SMALL["hidden"]


def test_inspect_infers_dimensions_the_config_omits(small_model, tmp_path):
    """vocab_size and head_dim missing from config.json are taken from the weight shapes
    (InferFromWeights, model/load.go:63)."""
    import lthn
    w, norms = small_model
    d = str(tmp_path / "ck")
    write_checkpoint(d, SMALL, w, norms)
    cfg = json.load(open(os.path.join(d, "config.json")))
    del cfg["vocab_size"], cfg["head_dim"]
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    info = lthn.checkpoint_inspect(d)
    assert info["vocab"] == SMALL["vocab"] and info["head_dim"] == SMALL["head_dim"]


def test_inspect_rejects_malformed_checkpoints(small_model, tmp_path):
    import lthn
    w, norms = small_model
    d = str(tmp_path / "ck")
    write_checkpoint(d, SMALL, w, norms)
    good_cfg = open(os.path.join(d, "config.json")).read()
    good_st = open(os.path.join(d, "model.safetensors"), "rb").read()

    def expect(msg_part):
        with pytest.raises(lthn.LthnError) as e:
            lthn.checkpoint_inspect(d)
        assert msg_part in str(e.value), str(e.value)

    with pytest.raises(lthn.LthnError):
        lthn.checkpoint_inspect(str(tmp_path / "missing"))
    open(os.path.join(d, "config.json"), "w").write(good_cfg.replace('"gemma3_text"', '"llama"'))
    expect("model_type")
    open(os.path.join(d, "config.json"), "w").write(good_cfg[:-5])
    expect("config.json")
    cfg = json.loads(good_cfg)
    del cfg["quantization"]
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    expect("quantization")
    cfg = json.loads(good_cfg)
    cfg["quantization"]["mode"] = "mxfp4"
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    expect("affine")
    open(os.path.join(d, "config.json"), "w").write(good_cfg)
    # header length beyond the file, truncated data, offsets outside the file
    open(os.path.join(d, "model.safetensors"), "wb").write(struct.pack("<Q", 1 << 40) + good_st[8:])
    expect("header length")
    open(os.path.join(d, "model.safetensors"), "wb").write(good_st[:len(good_st) // 2])
    expect("outside the file")
    write_safetensors(os.path.join(d, "model.safetensors"), {"model.norm.weight": ("BF16", np.zeros(4, np.uint16))})
    raw = open(os.path.join(d, "model.safetensors"), "rb").read()
    open(os.path.join(d, "model.safetensors"), "wb").write(raw.replace(b'"BF16"', b'"F32" '))
    expect("bytes for its shape")
    # an index that points outside the directory
    open(os.path.join(d, "model.safetensors"), "wb").write(good_st)
    json.dump({"weight_map": {"model.norm.weight": "../evil.safetensors"}}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    expect("leaves the checkpoint directory")
