"""Builds the same Gemma-style decoder on the CPU oracle and on the device."""
import ctypes as C

import numpy as np

ROLES = ("q", "k", "v", "o", "gate", "up", "down")
NORMS = ("input", "post_attn", "pre_ff", "post_ff", "q_norm", "k_norm")


def linear_shapes(cfg):
    D, H, F = cfg["head_dim"], cfg["hidden"], cfg["ffn"]
    return {"q": (cfg["q_heads"] * D, H), "k": (cfg["kv_heads"] * D, H), "v": (cfg["kv_heads"] * D, H),
            "o": (H, cfg["q_heads"] * D), "gate": (F, H), "up": (F, H), "down": (H, F)}


def synth_weights(oracle, lthn, cfg, seed, sigma=0.02, random_norms=False):
    """Every tensor of the model from the shared synthetic source (identical to
    lthn_model_synthesize), quantised by the oracle. Norms are 1 unless random_norms."""
    w = {}
    shapes = linear_shapes(cfg)
    for li in range(cfg["layers"]):
        for ri, role in enumerate(ROLES):
            n, k = shapes[role]
            dense = oracle.synth_normal(lthn.tensor_seed(seed, li, ri), 0, n * k, sigma).reshape(n, k)
            w[(li, role)] = oracle.quantize(dense)
    dense = oracle.synth_normal(lthn.tensor_seed(seed, -1, 0), 0, cfg["vocab"] * cfg["hidden"], sigma)
    w["embed"] = oracle.quantize(dense.reshape(cfg["vocab"], cfg["hidden"]))
    rng = np.random.default_rng(seed + 17)
    norms = {}
    for li in range(cfg["layers"]):
        for role in NORMS:
            n = cfg["head_dim"] if role in ("q_norm", "k_norm") else cfg["hidden"]
            # effective weight = 1 + stored weight (model/norm_bias.go fold), stored ~ N(0, 0.1)
            norms[(li, role)] = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32) if random_norms \
                else np.ones(n, dtype=np.float32)
    norms["final"] = (1.0 + 0.1 * rng.standard_normal(cfg["hidden"])).astype(np.float32) if random_norms \
        else np.ones(cfg["hidden"], dtype=np.float32)
    return w, norms


def widen_linears(oracle, lthn, cfg, w, seed, roles=("gate", "up", "down"), layers=None, sigma=0.02):
    """A mixed-precision pack: the named projections re-quantised at 8 bits (group 64) from the same dense
    source, as the per-module overrides of a QAT checkpoint keep them. Entries become (packed, scales, biases, 8)."""
    shapes = linear_shapes(cfg)
    out = dict(w)
    for li in (range(cfg["layers"]) if layers is None else layers):
        for role in roles:
            n, k = shapes[role]
            dense = oracle.synth_normal(lthn.tensor_seed(seed, li, ROLES.index(role)), 0, n * k, sigma).reshape(n, k)
            out[(li, role)] = (*oracle.quantize(dense, bits=8), 8)
    return out


def synth_weights_from_device(lthn, cfg, seed, sigma=0.02):
    """The same tensors for models too large to generate on the CPU in seconds: drawn and quantised
    by the device generator (tests/test_gpu_codec.py holds it bit-identical to the oracle's) and
    downloaded. Norm weights are 1, as lthn_model_synthesize sets them."""
    w = {}
    shapes = linear_shapes(cfg)
    for li in range(cfg["layers"]):
        for ri, role in enumerate(ROLES):
            n, k = shapes[role]
            q = lthn.QuantWeight.synth(lthn.tensor_seed(seed, li, ri), sigma, n, k)
            w[(li, role)] = q.to_host()
            q.free()
    q = lthn.QuantWeight.synth(lthn.tensor_seed(seed, -1, 0), sigma, cfg["vocab"], cfg["hidden"])
    w["embed"] = q.to_host()
    q.free()
    norms = {(li, role): np.ones(cfg["head_dim"] if role in ("q_norm", "k_norm") else cfg["hidden"], dtype=np.float32)
             for li in range(cfg["layers"]) for role in NORMS}
    norms["final"] = np.ones(cfg["hidden"], dtype=np.float32)
    return w, norms


def build_oracle(oracle, cfg, w, norms, max_len, prefill_bf16=0, sliding=None):
    embed_scale = float(oracle.bf16_to_f32(oracle.f32_to_bf16(np.array([np.sqrt(cfg["hidden"])], dtype=np.float32)))[0])
    oc = oracle.DecoderConfig(layers=cfg["layers"], hidden=cfg["hidden"], q_heads=cfg["q_heads"],
                              kv_heads=cfg["kv_heads"], head_dim=cfg["head_dim"], ffn=cfg["ffn"], vocab=cfg["vocab"],
                              gs=64, bits=4, max_len=max_len, eps=1e-6, rope_base=10000.0,
                              attn_scale=float(np.float32(1.0 / np.sqrt(cfg["head_dim"]))), embed_scale=embed_scale,
                              kv_bf16=1, prefill_bf16=prefill_bf16)
    if sliding:   # (window, pattern, local rope base)
        oc.sliding_window, oc.sliding_pattern, oc.rope_local_base = sliding
    d = oracle.Decoder(oc)
    for li in range(cfg["layers"]):
        for role in ROLES:
            d.set_linear(li, role, *w[(li, role)])
        for role in NORMS:
            d.set_norm(li, role, norms[(li, role)])
    d.set_linear(-1, 0, *w["embed"])
    d.set_norm(-1, 0, norms["final"])
    return d


def build_device(lthn, cfg, w, norms, max_len, max_lanes=1, tp_rank=0, tp_size=1, comm=None, sliding=None):
    mc = lthn.make_config(cfg["layers"], cfg["hidden"], cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["ffn"],
                          cfg["vocab"], max_len, max_lanes, tp_rank=tp_rank, tp_size=tp_size)
    if sliding:
        mc.sliding_window, mc.sliding_pattern, mc.rope_local_base = sliding
    m = lthn.Model(mc)
    for li in range(cfg["layers"]):
        for role in ROLES:
            m.upload_linear(li, role, *w[(li, role)])
        for role in NORMS:
            m.upload_norm(li, role, norms[(li, role)])
    m.upload_linear(-1, 0, *w["embed"])
    m.upload_norm(-1, 0, norms["final"])
    if comm is not None:
        m.set_comm(comm)
    m.finalize()
    return m


SMALL = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1024)
MID = dict(layers=3, hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=4096)
# the 26-layer decoder of the single-GPU decode benchmark: hidden 2304, 8 q / 4 kv heads x 256, GeGLU 9216, vocab 262144
GEMMA_2B = dict(layers=26, hidden=2304, q_heads=8, kv_heads=4, head_dim=256, ffn=9216, vocab=262144)
# the 62-layer decoder of the tensor-parallel benchmark: hidden 5376, 32 q / 16 kv heads x 128, GeGLU 21504, vocab 262144
GEMMA_27B = dict(layers=62, hidden=5376, q_heads=32, kv_heads=16, head_dim=128, ffn=21504, vocab=262144)
