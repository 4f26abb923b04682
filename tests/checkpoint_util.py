"""Writes a synthetic gemma3-style MLX-affine checkpoint directory (config.json + safetensors,
optionally sharded) from the tensors decoder_util.synth_weights makes, the way an MLX conversion
lays it out: U32 codes, BF16 scales/biases, norm weights stored as w-1 (the gemma convention)."""
import json
import os
import struct

import numpy as np

from decoder_util import NORMS, ROLES

NORM_NAMES = {"input": "input_layernorm", "post_attn": "post_attention_layernorm", "pre_ff": "pre_feedforward_layernorm",
              "post_ff": "post_feedforward_layernorm", "q_norm": "self_attn.q_norm", "k_norm": "self_attn.k_norm"}
LINEAR_NAMES = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
                "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}


def write_safetensors(path, tensors, metadata=None):
    """8-byte little-endian header length, JSON directory, tensor bytes (model/safetensors/write.go)."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, (dtype, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)


def checkpoint_tensors(cfg, w, norms, norm_dtype="BF16", prefix=""):
    """name -> (dtype, array). Norm weights are stored as (effective - 1) in norm_dtype."""
    t = {}

    def put_norm(name, eff):
        stored = (np.asarray(eff, dtype=np.float32) - np.float32(1.0)).astype(np.float32)
        if norm_dtype == "F32":
            t[prefix + name] = ("F32", stored)
        elif norm_dtype == "F16":
            t[prefix + name] = ("F16", stored.astype(np.float16))
        else:
            t[prefix + name] = ("BF16", bf16_bits(stored))

    for li in range(cfg["layers"]):
        base = f"model.layers.{li}."
        for role in ROLES:
            p, s, b = w[(li, role)][:3]
            n = prefix + base + LINEAR_NAMES[role]
            t[n + ".weight"], t[n + ".scales"], t[n + ".biases"] = ("U32", p), ("BF16", s), ("BF16", b)
        for role in NORMS:
            put_norm(base + NORM_NAMES[role] + ".weight", norms[(li, role)])
    p, s, b = w["embed"]
    n = prefix + "model.embed_tokens"
    t[n + ".weight"], t[n + ".scales"], t[n + ".biases"] = ("U32", p), ("BF16", s), ("BF16", b)
    put_norm("model.norm.weight", norms["final"])
    return t


def effective_norms(oracle, norms, norm_dtype):
    """What the loader's (1+w) fold yields from the stored tensors, in f32: bf16 storage rounds w-1 and
    the sum to bf16 (model/norm_bias.go:22-49), f16 storage is first widened to bf16, f32 is exact."""
    out = {}
    for k, eff in norms.items():
        stored = (np.asarray(eff, dtype=np.float32) - np.float32(1.0)).astype(np.float32)
        if norm_dtype == "F32":
            out[k] = (stored + np.float32(1.0)).astype(np.float32)
        else:
            if norm_dtype == "F16":
                stored = stored.astype(np.float16).astype(np.float32)
            sb = oracle.bf16_to_f32(bf16_bits(stored))
            out[k] = oracle.bf16_to_f32(bf16_bits((sb + np.float32(1.0)).astype(np.float32)))
    return out


def write_checkpoint(path, cfg, w, norms, norm_dtype="BF16", shards=1, prefix="", nest_text_config=False, quant_extra=None,
                     extra_config=None):
    os.makedirs(path, exist_ok=True)
    text = {"model_type": "gemma3_text", "hidden_size": cfg["hidden"], "num_hidden_layers": cfg["layers"],
            "intermediate_size": cfg["ffn"], "num_attention_heads": cfg["q_heads"], "num_key_value_heads": cfg["kv_heads"],
            "head_dim": cfg["head_dim"], "vocab_size": cfg["vocab"], "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
            "max_position_embeddings": 8192}
    if extra_config:
        text.update(extra_config)
    quant = {"group_size": 64, "bits": 4, "mode": "affine"}
    for key, val in w.items():   # linears that carry their own code width get a per-module override
        if key != "embed" and len(val) == 4:
            quant[f"model.layers.{key[0]}.{LINEAR_NAMES[key[1]]}"] = {"group_size": 64, "bits": int(val[3])}
    if quant_extra:
        quant.update(quant_extra)
    config = {"model_type": "gemma3", "text_config": text, "quantization": quant} if nest_text_config else dict(text, quantization=quant)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f)
    tensors = checkpoint_tensors(cfg, w, norms, norm_dtype, prefix)
    if shards == 1:
        write_safetensors(os.path.join(path, "model.safetensors"), tensors, {"format": "mlx"})
        return
    names = list(tensors)
    weight_map = {}
    for i in range(shards):
        part = {n: tensors[n] for n in names[i::shards]}
        fname = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        write_safetensors(os.path.join(path, fname), part)
        weight_map.update({n: fname for n in part})
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": 0}, "weight_map": weight_map}, f)
