"""Generates tests/golden/mlxaffine_dequant_golden.npz.

Run once where the reference checkout is available:
    python tests/golden/make_golden.py /path/to/reference
It imports the reference's own independent dequantiser (tools/mlxaffine_dequant.py),
feeds it a small safetensors file holding packed U32 codes and BF16 scales/biases,
and stores its f32 output next to the inputs. The inputs are quantised by the
oracle from deterministic formula weights (synthWeight of
go/model/quant/mlxaffine/mlxaffine_test.go:13-26 and a seeded normal tensor), so
the file pins: oracle quantiser output -> reference tool's dequantised values."""
import importlib.util
import json
import math
import os
import struct
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as o  # noqa: E402


def synth_weight(out_dim, in_dim):
    w = np.zeros((out_dim, in_dim), dtype=np.float32)
    for r in range(out_dim):
        amp = np.float32(0.01) + np.float32(0.5) * np.float32(r + 1) / np.float32(out_dim)
        bias = np.float32(0.1) * np.float32(r % 3 - 1)
        for c in range(in_dim):
            w[r, c] = bias + amp * np.float32(math.sin(float(r * 7 + c) * 0.013))
    return w


def write_safetensors(path, tensors):
    header, blobs, off = {}, [], 0
    for name, (dtype, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def main(ref_root):
    spec = importlib.util.spec_from_file_location("mlxaffine_dequant", os.path.join(ref_root, "tools", "mlxaffine_dequant.py"))
    tool = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tool)
    out = {}
    cases = {
        "synth_b4_g64": (synth_weight(8, 512), 4, 64),
        "synth_b8_g32": (synth_weight(3, 128), 8, 32),
        "synth_b2_g64": (synth_weight(5, 640), 2, 64),
        "normal_b4_g64": ((np.random.default_rng(0).standard_normal((16, 2304)) * 0.02).astype(np.float32), 4, 64),
    }
    with tempfile.TemporaryDirectory() as d:
        for name, (w, bits, gs) in cases.items():
            p, s, b = o.quantize(w, bits, gs)
            write_safetensors(os.path.join(d, "model.safetensors"),
                              {"t.weight": ("U32", p), "t.scales": ("BF16", s), "t.biases": ("BF16", b)})
            ref = tool.dequantise(__import__("pathlib").Path(d), "t", gs, bits)
            out[name + ".packed"], out[name + ".scales"], out[name + ".biases"] = p, s, b
            out[name + ".dequant"] = np.asarray(ref, dtype=np.float32)
            out[name + ".meta"] = np.array([bits, gs], dtype=np.int32)
    np.savez_compressed(os.path.join(HERE, "mlxaffine_dequant_golden.npz"), **out)
    print("wrote", len(cases), "cases")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a checkout of the reference (holds tools/mlxaffine_dequant.py)>")
    main(sys.argv[1])
