"""Small Fesorax configurations and weights for the tests.

The weights are drawn here, by tensor name and shape as the design names them (not from the
library's parameter table), with scales that make faults show: unit-norm queries and keys with a
large score scale give sharp softmax rows, the distance-bias tables have entries of size one, the
gates' biases spread over several units.  All values are exactly representable in bfloat16, so the
same folder serves both number formats.
"""
import json
import os

import numpy as np
import torch

import plain_llama

# every size differs from layer to layer; values that a model could make equal (heads and key/value
# heads, key and value widths, top and the number of experts, the two limits) are equal in one layer
# and different in another
CASE_A = {
    "architecture": "Fesorax", "vocab": 97, "width": 64, "postln_alpha": 1.7, "norm": {"eps": 1e-5},
    "embedding": {"scale": 3.0},
    "layers": [
        {"type": "mlstm", "mixer": {"heads": 2, "dim": 16, "vdim": 24, "gate_cap": 5.0},
         "mlp": {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 40, "limit": 1.0},
                 "shared": {"ff": 24, "limit": 2.0}}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.9, "bias_max": 50,
                                        "mask": {"size": 37, "keep_first": 3}}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.6, "bias_max": 90,
                                        "kv_from": 1, "mask": {"size": 70, "keep_first": 9}},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 1}, "expert": {"ff": 16, "limit": 0.7}}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 40, "scale": 0.5, "bias_max": 33},
         "mlp": {"kind": "moe", "router": {"experts": 4, "top": 4}, "expert": {"ff": 24, "limit": 1.2},
                 "shared": {"ff": 24, "limit": 1.2}}},
        {"type": "mlstm", "mixer": {"heads": 1, "dim": 40, "vdim": 136, "gate_cap": 30.0}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 40, "scale": 0.8, "bias_max": 8,
                                        "kv_from": 3, "mask": {"size": 9, "keep_first": 0}},
         "mlp": {"kind": "moe", "router": {"experts": 2, "top": 1}, "expert": {"ff": 8, "limit": 3.0},
                 "shared": {"ff": 56, "limit": 0.5}}},
    ],
}
REL_ROWS_A = {1: 12, 2: 16, 3: 8, 5: 10}

# attention first, a window of exactly one page, kept tokens that fill more than a page, alpha 1
CASE_B = {
    "architecture": "Fesorax", "vocab": 131, "width": 48, "postln_alpha": 1.0, "norm": {"eps": 1e-6},
    "embedding": {"scale": 1.0},
    "layers": [
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 48, "vdim": 16, "scale": 0.35, "bias_max": 200,
                                        "mask": {"size": 64, "keep_first": 70}},
         "mlp": {"kind": "moe", "router": {"experts": 6, "top": 3}, "expert": {"ff": 32, "limit": 1.5},
                 "shared": {"ff": 16, "limit": 1.5}}},
        {"type": "mlstm", "mixer": {"heads": 3, "dim": 8, "vdim": 8, "gate_cap": 2.0},
         "mlp": {"kind": "moe", "router": {"experts": 2, "top": 2}, "expert": {"ff": 8, "limit": 9.0}}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 48, "vdim": 16, "scale": 0.2, "bias_max": 17,
                                        "kv_from": 0, "mask": {"size": 1000, "keep_first": 1}}, "mlp": None},
    ],
}
REL_ROWS_B = {0: 30, 2: 6}


# key and value heads of one width (the tensor-core kernel for runs of new tokens takes these), windows
# shorter than the prompts with and without kept tokens, a reader with a wider window than its owner
CASE_C = {
    "architecture": "Fesorax", "vocab": 150, "width": 96, "postln_alpha": 3.0, "norm": {"eps": 1e-6},
    "embedding": {"scale": 8.0},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.5, "bias_max": 100,
                                        "mask": {"size": 70, "keep_first": 5}},
         "mlp": {"kind": "moe", "router": {"experts": 4, "top": 1}, "expert": {"ff": 32, "limit": 1.5},
                 "shared": {"ff": 32, "limit": 1.5}}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.3, "bias_max": 60,
                                        "kv_from": 0, "mask": {"size": 100, "keep_first": 20}}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 80, "vdim": 80, "scale": 0.4, "bias_max": 40,
                                        "mask": {"size": 33, "keep_first": 0}},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 16, "limit": 2.0}}},
    ],
}
REL_ROWS_C = {0: 32, 1: 20, 2: 24}


# sizes that are no multiples of 8 anywhere: rows of no whole 16-byte pieces, so every kernel takes its
# number-by-number path and the products the library's
CASE_D = {
    "architecture": "Fesorax", "vocab": 61, "width": 50, "postln_alpha": 2.0, "norm": {"eps": 1e-5},
    "embedding": {"scale": 5.0},
    "layers": [
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 20, "vdim": 12, "scale": 0.7, "bias_max": 25,
                                        "mask": {"size": 30, "keep_first": 2}},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 18, "limit": 1.0},
                 "shared": {"ff": 10, "limit": 1.0}}},
        {"type": "mlstm", "mixer": {"heads": 2, "dim": 20, "vdim": 36, "gate_cap": 8.0}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 20, "vdim": 12, "scale": 0.7, "bias_max": 25,
                                        "kv_from": 0},
         "mlp": {"kind": "moe", "router": {"experts": 2, "top": 1}, "expert": {"ff": 6, "limit": 2.0}}},
    ],
}
REL_ROWS_D = {0: 10, 2: 14}


def tensor_shapes(cfg: dict, rel_rows: dict) -> dict:
    """Every tensor of the design by name, from the configuration alone."""
    W = cfg["width"]
    t = {"embed": (cfg["vocab"], W), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        t[p + "norm1"] = (W,)
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"] = (H * d, W)
            if m.get("kv_from") is None:
                t[p + "mix.k"], t[p + "mix.v"] = (G * d, W), (G * dv, W)
            t[p + "mix.rel"], t[p + "mix.g"], t[p + "mix.o"] = (rel_rows[i], H), (H, W), (W, H * dv)
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"] = (H * d, W), (H * d, W)
            t[p + "mix.v"], t[p + "mix.g"], t[p + "mix.o"], t[p + "mix.norm"] = (H * dv, W), (H * dv, W), (W, H * dv), (H * dv,)
            for g in ("i", "f"):
                t[p + f"mix.{g}"], t[p + f"mix.{g}.b"] = (H, W), (H,)
        mlp = layer.get("mlp")
        if mlp:
            t[p + "norm2"] = (W,)
            t[p + "mlp.router"] = (mlp["router"]["experts"], W)
            names = [(f"e{e}", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                names.append(("shared", mlp["shared"]["ff"]))
            for n, ff in names:
                t[p + f"mlp.{n}.gate"], t[p + f"mlp.{n}.up"], t[p + f"mlp.{n}.down"] = (ff, W), (ff, W), (W, ff)
    return t


def draw_weights(cfg: dict, rel_rows: dict, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    out = {}
    for name, shape in tensor_shapes(cfg, rel_rows).items():
        last = name.split(".")[-1]
        if "norm" in last:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "rel":
            a = rng.standard_normal(shape)
        elif last == "b":
            a = 1.5 * rng.standard_normal(shape) + (2.0 if name.endswith("f.b") else 0.0)
        elif last == "embed":
            a = rng.standard_normal(shape)
        elif last in ("router", "i", "f", "g"):
            a = rng.standard_normal(shape) * 1.5 / np.sqrt(W)  # inputs have unit rms: pre-activations of size 1.5
        else:
            a = rng.standard_normal(shape) / np.sqrt(shape[-1])
        out[name] = plain_llama.to_bf16(a.astype(np.float64))
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
