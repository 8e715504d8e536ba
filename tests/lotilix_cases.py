"""Small Lotilix configurations and weights for the tests.

The weights are drawn here, by tensor name and shape as the design names them (not from the library's
parameter table), with scales that make faults show: matrices of scale 1/sqrt(inputs) give scores and
pre-activations of order one (sharp softmax rows, decays and gates spread over their range), convolution
taps and biases of order one.  All values are exactly representable in bfloat16, so the same folder serves
both number formats.
"""
import json
import os

import numpy as np
import torch

from plain_lotilix import to_bf16

# every size differs from layer to layer; values that a model could make equal (heads and key/value heads,
# key and value widths, rotated dimensions and the head, the two low ranks) are equal in one layer and
# different in another; masks shorter than the prompts, one of exactly a page, one absent
CASE_A = {
    "architecture": "Lotilix", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "token_side": {"dim": 8},
    "layers": [
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 4},
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 16, "rot_dim": 8, "vdim": 24, "q_rank": 24, "kv_rank": 40,
                                               "scale": 0.9, "rot": {"base": 10000.0, "dims": 8}, "mask": {"size": 37}},
         "mlp": None},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 1.1,
                                        "rot": {"base": 300.0, "dims": 8,
                                                "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 40}},
                                        "mask": {"size": 50}},
         "mlp": {"kind": "dense", "ff": 48}},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 8, "rot_dim": 8, "vdim": 8, "q_rank": 16, "kv_rank": 56,
                                               "scale": 1.4, "rot": {"base": 50.0, "dims": 8}, "mask": {"size": 64}},
         "mlp": {"kind": "dense", "ff": 24}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.6,
                                        "rot": {"base": 1000.0, "dims": 32}, "mask": {"size": 64}},
         "mlp": None},
        {"type": "channel_delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 40, "vdim": 136, "conv": 2},
         "mlp": {"kind": "dense", "ff": 16}},
    ],
}
LOW_RANKS_A = {0: (6, 10), 5: (8, 8)}  # layer -> (rows of a1, rows of g1)

# sizes that are no multiples of 8 anywhere: rows of no whole 16-byte pieces, so every kernel takes its
# number-by-number path and the products the library's; a convolution of one tap; no mask in one mixer
CASE_B = {
    "architecture": "Lotilix", "vocab": 61, "width": 50, "norm": {"eps": 1e-6}, "token_side": {"dim": 5},
    "layers": [
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 10, "rot_dim": 6, "vdim": 12, "q_rank": 14, "kv_rank": 20,
                                               "scale": 1.2, "rot": {"base": 77.0, "dims": 6}, "mask": {"size": 30}},
         "mlp": {"kind": "dense", "ff": 18}},
        {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 20, "vdim": 36, "conv": 1}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 20, "vdim": 20, "scale": 0.8,
                                        "rot": {"base": 9.0, "dims": 10}, "mask": {"size": 23}},
         "mlp": {"kind": "dense", "ff": 10}},
        {"type": "latent_attention", "mixer": {"heads": 1, "dim": 6, "rot_dim": 2, "vdim": 7, "q_rank": 5, "kv_rank": 9,
                                               "scale": 2.0, "rot": {"base": 4.0, "dims": 2}},
         "mlp": {"kind": "dense", "ff": 10}},
    ],
}
LOW_RANKS_B = {1: (3, 7)}

# key rows in multiples of 16 (the tensor-core kernel for runs of new tokens takes these), masks shorter than
# the prompts, no per-token input, a chunk that is no multiple of a page and a window longer than two
CASE_C = {
    "architecture": "Lotilix", "vocab": 150, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.7,
                                        "rot": {"base": 5000.0, "dims": 16,
                                                "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}},
                                        "mask": {"size": 70}},
         "mlp": {"kind": "dense", "ff": 64}},
        {"type": "latent_attention", "mixer": {"heads": 4, "dim": 16, "rot_dim": 16, "vdim": 32, "q_rank": 32, "kv_rank": 48,
                                               "scale": 0.8, "rot": {"base": 200.0, "dims": 16}, "mask": {"size": 150}},
         "mlp": {"kind": "dense", "ff": 32}},
        {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 32, "conv": 3},
         "mlp": {"kind": "dense", "ff": 32}},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 32, "rot_dim": 32, "vdim": 16, "q_rank": 48, "kv_rank": 96,
                                               "scale": 0.5, "rot": {"base": 1e6, "dims": 32}, "mask": {"size": 33}},
         "mlp": None},
    ],
}
LOW_RANKS_C = {2: (16, 16)}

# latents wider than the tensor-core kernel's key rows: runs of new tokens in bfloat16 take per-head keys and values
# made from the cached rows; with and without a window, behind cached tokens and from the first token on
CASE_D = {
    "architecture": "Lotilix", "vocab": 120, "width": 64, "norm": {"eps": 1e-6}, "token_side": {"dim": 16},
    "layers": [
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 16, "rot_dim": 16, "vdim": 32, "q_rank": 24, "kv_rank": 272,
                                               "scale": 0.8, "rot": {"base": 300.0, "dims": 16}, "mask": {"size": 40}},
         "mlp": {"kind": "dense", "ff": 32}},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 32, "rot_dim": 16, "vdim": 16, "q_rank": 32, "kv_rank": 304,
                                               "scale": 0.6, "rot": {"base": 1e4, "dims": 16}},
         "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 16, "rot_dim": 16, "vdim": 32, "q_rank": 24, "kv_rank": 272,
                                               "scale": 0.8, "rot": {"base": 300.0, "dims": 16}, "mask": {"size": 40}},
         "mlp": {"kind": "dense", "ff": 32}},
    ],
}

CASES = {"A": (CASE_A, LOW_RANKS_A), "B": (CASE_B, LOW_RANKS_B), "C": (CASE_C, LOW_RANKS_C), "D": (CASE_D, {})}


def tensor_shapes(cfg: dict, low_ranks: dict) -> dict:
    """Every tensor of the design by name, from the configuration (and the ranks that only the tensors fix)."""
    W, V = cfg["width"], cfg["vocab"]
    t = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    side = (cfg.get("token_side") or {}).get("dim", 0)
    if side:
        t["side.embed"] = (V, side * len(cfg["layers"]))
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        t[p + "norm1"] = (W,)
        if layer["type"] == "latent_attention":
            H, d, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"], t[p + "mix.uq"] = (m["q_rank"], W), (m["q_rank"],), (H * (d + dr), m["q_rank"])
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = (m["kv_rank"] + dr, W), (m["kv_rank"],)
            t[p + "mix.uk"], t[p + "mix.uv"] = (H * d, m["kv_rank"]), (H * dv, m["kv_rank"])
            t[p + "mix.g"], t[p + "mix.o"] = (H, W), (W, H * dv)
        elif layer["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.o"] = (H * d, W), (G * d, W), (W, H * d)
        else:
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = low_ranks[i]
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                t[p + f"mix.{n}"], t[p + f"mix.{n}.conv"] = (rows, W), (rows, taps)
            t[p + "mix.b"], t[p + "mix.A_log"], t[p + "mix.norm"] = (H, W), (H,), (dv,)
            t[p + "mix.a1"], t[p + "mix.a2"], t[p + "mix.dt_bias"] = (ra, W), (H * d, ra), (H * d,)
            t[p + "mix.g1"], t[p + "mix.g2"], t[p + "mix.o"] = (rg, W), (H * dv, rg), (W, H * dv)
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = (ff, W), (ff, W), (W, ff)
        if side:
            t[p + "side.gate"], t[p + "side.proj"], t[p + "side.norm"] = (side, W), (W, side), (W,)
    return t


def draw_weights(cfg: dict, low_ranks: dict, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, low_ranks).items():
        last = name.split(".")[-1]
        if last.startswith("norm") or name.endswith(".norm"):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "embed":
            a = rng.standard_normal(shape)
        elif last == "conv":
            a = rng.standard_normal(shape) * 0.7
        elif last == "A_log":
            a = rng.standard_normal(shape) - 1.0
        elif last == "dt_bias":
            a = rng.standard_normal(shape) - 1.0
        elif last in ("b", "g"):
            a = rng.standard_normal(shape) * 2.0 / np.sqrt(shape[-1])  # inputs have unit rms: pre-activations of size 2
        else:
            a = rng.standard_normal(shape) * 1.3 / np.sqrt(shape[-1])
        out[name] = to_bf16(a.astype(np.float64))
    return out


def write_folder(folder: str, cfg: dict, weights: dict, storage: str = "bfloat16") -> str:
    from bitnet_c_b200.weights import write_safetensors
    os.makedirs(folder, exist_ok=True)
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[storage]
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(n, torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dt)) for n, a in weights.items()])
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return folder
