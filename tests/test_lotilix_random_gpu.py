"""Lotilix configurations drawn at random by fixed seeds from all that its config.json allows (layer orders,
head counts and sizes, ranks, rotated dimensions with and without frequency scaling, windows and chunks
below and above a cache page or absent, convolutions of one to five taps, layers without a feed-forward,
with and without the per-token input), each stepped whole, token by token, in pieces and in unequal
batches against the plain statement, in both number formats."""
import numpy as np
import pytest

import bitnet_c_b200 as bn
import lotilix_cases as lc
import plain_lotilix as pl
from helpers import TOL_F32, random_tokens, replay, trace_batches, trace_chunks, trace_tail, trace_whole
from test_lotilix_gpu import _check, _poison

pytestmark = pytest.mark.gpu


def draw_config(seed: int):
    rng = np.random.default_rng(seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]
    width = pick([32, 40, 48, 64, 72, 96, 128])
    layers, ranks = [], {}
    for i in range(int(rng.integers(1, 8))):
        kind = pick(["latent_attention", "attention", "channel_delta"])
        mask = {"mask": {"size": int(rng.integers(2, 200))}} if rng.random() < 0.85 else {}
        if kind == "latent_attention":
            rot = pick([2, 4, 8, 16, 32, 64])
            m = {"heads": pick([1, 2, 3, 4, 6]), "dim": pick([4, 8, 16, 24, 32, 64]), "rot_dim": rot, "vdim": pick([8, 12, 16, 32, 48]),
                 "q_rank": pick([8, 12, 24, 48]), "kv_rank": pick([8, 16, 24, 48, 96, 200, 300]), "scale": float(rng.uniform(0.3, 1.5)),
                 "rot": {"base": float(pick([10.0, 1e3, 1e4, 1e6])), "dims": rot}, **mask}
        elif kind == "attention":
            g, d = pick([1, 2, 3]), pick([8, 16, 20, 32, 48, 64, 96])
            rot = {"base": float(pick([10.0, 500.0, 5e5])), "dims": pick([x for x in (2, 4, 8, 16, 20, 32, 48, 64, 96) if x <= d])}
            if rng.random() < 0.5:
                low = float(pick([1.0, 2.0]))
                rot["scaling"] = {"factor": float(pick([2.0, 8.0, 32.0])), "low": low, "high": low * float(pick([2.0, 4.0])),
                                  "original": int(pick([16, 64, 256, 1024]))}
            m = {"heads": g * pick([1, 2, 4]), "kv_heads": g, "dim": d, "vdim": d, "scale": float(rng.uniform(0.2, 1.2)), "rot": rot, **mask}
        else:
            g = pick([1, 2, 3])
            m = {"heads": g * pick([1, 2, 3]), "kv_heads": g, "dim": pick([8, 16, 20, 32, 64, 100]), "vdim": pick([8, 16, 24, 40, 64, 136]),
                 "conv": int(rng.integers(1, 6))}
            ranks[i] = (int(rng.integers(1, 20)), int(rng.integers(1, 20)))
        layer = {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": pick([8, 12, 24, 40, 64, 100])} if rng.random() < 0.8 else None}
        layers.append(layer)
    cfg = {"architecture": "Lotilix", "vocab": int(rng.integers(50, 300)), "width": width, "norm": {"eps": pick([1e-5, 1e-6])},
           "layers": layers}
    if rng.random() < 0.75:
        cfg["token_side"] = {"dim": pick([1, 4, 8, 12, 16, 32])}
    return cfg, ranks


@pytest.mark.parametrize("seed", range(14))
def test_a_configuration_drawn_at_random_steps_like_the_plain_statement(tmp_path, cuda_device, seed):
    cfg, ranks = draw_config(2000 + seed)
    w = lc.draw_weights(cfg, ranks, seed=seed)
    folder = lc.write_folder(str(tmp_path / "m"), cfg, w)
    V = cfg["vocab"]
    reqs = {"a": random_tokens(seed, 230, V), "b": random_tokens(seed + 50, 1, V), "c": random_tokens(seed + 99, 70, V)}
    plain = {r: pl.forward(cfg, w, t) for r, t in reqs.items()}
    # a model drawn at random may answer single-precision rounding at single places with far more than 1e-4 of
    # its logits (a unit norm or a sharp softmax row behind a nearly empty state): how much, place by place, shows
    # when the plain statement runs with weights moved by 1e-7 of their size; float32 is allowed 30 times that
    rng = np.random.default_rng(seed)
    moved = {k: a * (1.0 + 1e-7 * rng.standard_normal(a.shape)) for k, a in w.items()}
    slack = {r: 30.0 * np.abs(pl.forward(cfg, moved, t) - plain[r]).max(axis=1) for r, t in reqs.items()}
    for dtype in ("float32", "bfloat16") if seed % 2 == 0 else ("float32",):
        model = bn.load_model(folder, dtype=dtype)
        cache = model.new_cache(max_tokens=64 * 10, max_seqs=3)
        _poison(cache)
        for what, steps in (("whole", trace_whole(reqs)), ("last 25 one by one", trace_tail(reqs, 25)),
                            ("pieces", trace_chunks(reqs, pieces=(3, 64, 17, 1))),
                            ("an unequal batch", trace_batches([{"a": (reqs["a"], 12), "c": (reqs["c"], 30), "b": (reqs["b"], 0)}]))):
            got = replay(model, cache, steps)
            if dtype == "bfloat16":
                _check(got, cfg, w, reqs, plain, dtype, f"seed {seed}: {what}, {dtype}", rough_ok=True)
                continue
            for r, per_pos in got.items():
                for p, row in sorted(per_pos.items()):
                    err = float(np.abs(row.astype(np.float64) - plain[r][p]).max())
                    assert err <= TOL_F32 * max(1.0, float(np.abs(plain[r]).max())) + slack[r][p], \
                        f"seed {seed}: {what}: request {r} position {p}: max |diff| {err:.3e}"
        model.check_kernels()
