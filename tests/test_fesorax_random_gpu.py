"""Fesorax configurations drawn at random by fixed seeds from all that its config.json allows (layer
orders, head counts and sizes, windows with and without kept tokens, shared keys and values, experts and
how many a token uses, layers without a feed-forward), each stepped whole, token by token and in unequal
batches against the plain statement, in both number formats."""
import numpy as np
import pytest

import bitnet_c_b200 as bn
import fesorax_cases as fc
import plain_fesorax as pf
from helpers import TOL_F32, compare, random_tokens, replay, trace_batches, trace_chunks, trace_tail, trace_whole
from test_fesorax_gpu import _check, _poison

pytestmark = pytest.mark.gpu


def draw_config(seed: int):
    rng = np.random.default_rng(seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]
    width = pick([32, 48, 64, 72, 96, 128])
    layers, rel_rows, owners = [], {}, []
    for i in range(int(rng.integers(1, 8))):
        if rng.random() < 0.6:
            src = pick(owners) if owners and rng.random() < 0.4 else None
            if src is not None:
                m0 = layers[src]["mixer"]
                m = {k: m0[k] for k in ("heads", "kv_heads", "dim", "vdim")}
                m["kv_from"] = src
            else:
                g = pick([1, 2, 3])
                m = {"heads": g * pick([1, 2, 3]), "kv_heads": g, "dim": pick([16, 24, 32, 48, 64, 96]),
                     "vdim": pick([8, 16, 32, 40, 48, 64])}
                owners.append(i)
            rel_rows[i] = pick([8, 12, 16, 32])
            m["scale"] = float(rng.uniform(0.2, 1.0))
            m["bias_max"] = int(rng.integers(rel_rows[i] // 2 + 1, 300))
            if rng.random() < 0.8:
                m["mask"] = {"size": int(rng.integers(3, 150)), "keep_first": int(rng.integers(0, 70)) if rng.random() < 0.7 else 0}
            layer = {"type": "attention", "mixer": m}
        else:
            layer = {"type": "mlstm", "mixer": {"heads": pick([1, 2, 3, 4]), "dim": pick([8, 16, 20, 32, 64]),
                                                "vdim": pick([8, 16, 24, 48, 64, 136]), "gate_cap": float(rng.uniform(2, 20))}}
        if rng.random() < 0.8:
            experts = int(rng.integers(1, 10))
            mlp = {"kind": "moe", "router": {"experts": experts, "top": int(rng.integers(1, min(experts, 3) + 1))},
                   "expert": {"ff": pick([8, 16, 24, 40, 64]), "limit": float(rng.uniform(0.5, 3.0))}}
            if rng.random() < 0.7:
                mlp["shared"] = {"ff": pick([8, 16, 32]), "limit": float(rng.uniform(0.5, 3.0))}
            layer["mlp"] = mlp
        else:
            layer["mlp"] = None
        layers.append(layer)
    cfg = {"architecture": "Fesorax", "vocab": int(rng.integers(50, 300)), "width": width,
           "postln_alpha": float(rng.uniform(1.0, 3.0)), "norm": {"eps": pick([1e-5, 1e-6])},
           "embedding": {"scale": float(rng.uniform(0.5, 10.0))}, "layers": layers}
    return cfg, rel_rows


@pytest.mark.parametrize("seed", range(12))
def test_a_configuration_drawn_at_random_steps_like_the_plain_statement(tmp_path, cuda_device, seed):
    cfg, rel_rows = draw_config(1000 + seed)
    w = fc.draw_weights(cfg, rel_rows, seed=seed)
    folder = fc.write_folder(str(tmp_path / "m"), cfg, w)
    V = cfg["vocab"]
    reqs = {"a": random_tokens(seed, 160, V), "b": random_tokens(seed + 50, 1, V), "c": random_tokens(seed + 99, 70, V)}
    plain = {r: pf.forward(cfg, w, t) for r, t in reqs.items()}
    for dtype in ("float32", "bfloat16") if seed % 3 == 0 else ("float32",):
        model = bn.load_model(folder, dtype=dtype)
        cache = model.new_cache(max_tokens=64 * 8, max_seqs=3)
        _poison(cache)
        for what, steps in (("whole", trace_whole(reqs)), ("last 25 one by one", trace_tail(reqs, 25)),
                            ("pieces", trace_chunks(reqs, pieces=(3, 64, 17, 1))),
                            ("an unequal batch", trace_batches([{"a": (reqs["a"], 12), "c": (reqs["c"], 30), "b": (reqs["b"], 0)}]))):
            _check(replay(model, cache, steps), cfg, w, reqs, plain, dtype, f"seed {seed}: {what}, {dtype}")
        model.check_kernels()
