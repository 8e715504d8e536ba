"""The plain statement of the Lotilix mechanisms checked against itself (closed forms, and faults that must
show), and the library's host side for this design: configuration, tensor names, what the cache keeps."""
import copy
import math

import numpy as np
import pytest

import lotilix_cases as lc
import plain_lotilix as pl
from helpers import random_tokens


def test_masks_are_causal_windows_and_chunks_counted_from_position_zero():
    assert pl.sees_window(10, 10, 3) and pl.sees_window(10, 8, 3) and not pl.sees_window(10, 7, 3)
    assert not pl.sees_window(3, 4, 0) and pl.sees_window(500, 0, 0)
    assert pl.sees_chunk(10, 10, 4) and pl.sees_chunk(10, 8, 4) and not pl.sees_chunk(10, 7, 4)
    assert pl.sees_chunk(11, 8, 4) and not pl.sees_chunk(12, 11, 4) and not pl.sees_chunk(8, 9, 4) and pl.sees_chunk(500, 0, 0)


def test_rotation_of_pairs_depends_on_the_distance_only_and_leaves_the_rest():
    rng = np.random.default_rng(0)
    rot = {"base": 100.0, "dims": 4}
    f = pl.rotary_frequencies(rot)
    assert np.allclose(f, [1.0, 0.1])
    q, k = rng.standard_normal((1, 1, 6)), rng.standard_normal((1, 1, 6))
    a = (pl.rotate_pairs(q, [7], f) * pl.rotate_pairs(k, [3], f)).sum()
    b = (pl.rotate_pairs(q, [104], f) * pl.rotate_pairs(k, [100], f)).sum()
    assert abs(a - b) < 1e-9
    assert np.array_equal(pl.rotate_pairs(q, [9], f)[..., 4:], q[..., 4:])
    # the pair (1, 0) at position p and frequency 1 becomes (cos p, sin p): dimension 2i pairs with 2i + 1
    e = np.zeros((1, 1, 4))
    e[..., 0] = 1.0
    assert np.allclose(pl.rotate_pairs(e, [2], f)[0, 0], [math.cos(2), math.sin(2), 0, 0])


def test_long_wavelengths_are_slowed_and_the_band_between_is_blended():
    rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    plain = pl.rotary_frequencies({"base": 10000.0, "dims": 16})
    f = pl.rotary_frequencies(rot)
    wl = 2 * math.pi / plain
    assert np.array_equal(f[wl < 16], plain[wl < 16]) and np.allclose(f[wl > 64], plain[wl > 64] / 8)
    mid = (wl >= 16) & (wl <= 64)
    assert mid.any() and np.all(f[mid] < plain[mid]) and np.all(f[mid] > plain[mid] / 8)


def test_short_convolution_is_causal_and_its_last_column_is_the_current_token():
    x = np.arange(1.0, 6.0)[:, None] * np.array([[1.0, 10.0]])
    taps = np.array([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])
    y = pl.short_convolution(x, taps)
    assert np.array_equal(y[:, 0], x[:, 0]) and np.array_equal(y[:, 1], [0, 0, 10, 20, 30])


def test_delta_rule_writes_before_it_reads_and_forgets_by_channel():
    rng = np.random.default_rng(1)
    T, d, dv = 7, 3, 2
    q, k, v = rng.standard_normal((T, d)), rng.standard_normal((T, d)), rng.standard_normal((T, dv))
    k /= np.linalg.norm(k, axis=1, keepdims=True)
    # without decay and with beta 1 the state answers the key it has just stored with the stored value
    o, S = pl.delta_rule(k, k, v, np.ones((T, d)), np.ones(T))
    assert np.allclose(o, v)
    # a decay of zero on every channel leaves only the current token: o_t = beta_t v_t (k_t . q_t)
    beta = rng.uniform(0.2, 1.0, T)
    o, _ = pl.delta_rule(q, k, v, np.zeros((T, d)), beta)
    assert np.allclose(o, beta[:, None] * v * (k * q).sum(1, keepdims=True))
    # the unrolled form of two steps with a decay per channel
    g = rng.uniform(0.3, 1.0, (T, d))
    o, _ = pl.delta_rule(q, k, v, g, beta)
    S0 = np.outer(k[0], beta[0] * v[0])
    S1 = g[1][:, None] * S0
    S1 = S1 + np.outer(k[1], beta[1] * (v[1] - S1.T @ k[1]))
    assert np.allclose(o[1], S1.T @ q[1])


@pytest.mark.parametrize("case", ["A", "B", "C", "D"])
def test_faults_in_the_mechanisms_move_the_logits_of_the_test_models(case):
    """The models of the engine tests are sharp enough: each of these faults moves some logit by far more than
    the engine's float32 tolerance, so a test that passes excludes them."""
    cfg, ranks = lc.CASES[case]
    w = lc.draw_weights(cfg, ranks, seed=5)
    toks = random_tokens(4, 150, cfg["vocab"])
    ref = pl.forward(cfg, w, toks)
    assert 1.0 < np.abs(ref).max() < 200.0

    def moved(change_cfg=None, change_w=None):
        c, ww = copy.deepcopy(cfg), dict(w)
        if change_cfg:
            change_cfg(c)
        if change_w:
            change_w(ww)
        return float(np.abs(pl.forward(c, ww, toks) - ref).max())

    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", l["mixer"]
        if m.get("mask") and m["mask"]["size"] < 150:
            size = m["mask"]["size"]
            assert moved(lambda c: c["layers"][i]["mixer"]["mask"].update(size=size + 1)) > 1e-2, f"mask of layer {i}"
            assert moved(lambda c: c["layers"][i]["mixer"]["mask"].update(size=size - 1)) > 1e-2, f"mask of layer {i}"
        if l["type"] in ("latent_attention", "attention"):
            assert moved(lambda c: c["layers"][i]["mixer"].update(scale=m["scale"] * 1.1)) > 1e-2, f"scale of layer {i}"
            if m["rot"]["dims"] > 2:  # the first pair's frequency is 1 whatever the base
                assert moved(lambda c: c["layers"][i]["mixer"]["rot"].update(base=m["rot"]["base"] * 1.5)) > 1e-3, f"base of layer {i}"
            if m["rot"].get("scaling"):
                assert moved(lambda c: c["layers"][i]["mixer"]["rot"].pop("scaling")) > 1e-3, f"frequency scaling of layer {i}"
        if l["type"] == "latent_attention":
            assert moved(change_w=lambda ww: ww.update({p + "g": np.zeros_like(w[p + "g"])})) > 1e-2, f"gate of layer {i}"
            assert moved(change_w=lambda ww: ww.update({p + "dkv.norm": np.ones_like(w[p + "dkv.norm"])})) > 1e-2, f"latent norm of layer {i}"
        if l["type"] == "channel_delta":
            assert moved(change_w=lambda ww: ww.update({p + "A_log": w[p + "A_log"] + 0.5})) > 1e-2, f"decay of layer {i}"
            assert moved(change_w=lambda ww: ww.update({p + "dt_bias": w[p + "dt_bias"] + 0.5})) > 1e-2, f"decay bias of layer {i}"
            assert moved(change_w=lambda ww: ww.update({p + "b": np.zeros_like(w[p + "b"])})) > 1e-2, f"beta of layer {i}"
            if m["conv"] > 1:
                assert moved(change_w=lambda ww: ww.update({p + "k.conv": w[p + "k.conv"][:, ::-1]})) > 1e-2, f"taps of layer {i}"
        if l.get("mlp"):
            assert moved(change_w=lambda ww: ww.update({f"l{i}.mlp.up": 1.1 * w[f"l{i}.mlp.up"]})) > 1e-2, f"feed-forward of layer {i}"
    if cfg.get("token_side"):
        assert moved(change_w=lambda ww: ww.update({"side.embed": np.roll(w["side.embed"], 1, axis=1)})) > 1e-2
        assert moved(change_w=lambda ww: ww.update({"l1.side.norm": 1.5 * w["l1.side.norm"]})) > 1e-2
    assert moved(lambda c: c["norm"].update(eps=0.5)) > 1e-2


# ---- the library's host side ---------------------------------------------------------------------
def test_the_configuration_is_read_key_by_key_and_builds_the_parameter_table_of_the_design():
    import bitnet_c_b200 as bn
    from bitnet_c_b200.config import ConfigError, architecture_of
    from bitnet_c_b200.engine.model import parameter_table
    assert "Lotilix" in bn.known_architectures()
    for cfg_dict, ranks in lc.CASES.values():
        shapes = lc.tensor_shapes(cfg_dict, ranks)
        arch = architecture_of(cfg_dict)
        cfg = arch.read_config(arch.complete_config(cfg_dict, shapes))
        spec = arch.to_spec(cfg)
        table = {}
        for p, s in parameter_table(spec).items():
            table.setdefault(arch.tensor_name(p), set()).add(tuple(s.shape))
        assert {n: next(iter(v)) for n, v in table.items()} == shapes and all(len(v) == 1 for v in table.values())
        assert arch.read_config(arch.config_to_dict(cfg)) == cfg
    arch = architecture_of(lc.CASE_A)
    spec = arch.to_spec(arch.read_config(arch.complete_config(lc.CASE_A, lc.tensor_shapes(lc.CASE_A, lc.LOW_RANKS_A))))
    m0, m1, m2 = spec.blocks[0].mixer, spec.blocks[1].mixer, spec.blocks[2].mixer
    assert (m0.kind, m0.conv_taps, m0.decay_rank, m0.gate_rank) == ("delta_rule", 4, 6, 10)
    assert (m1.kind, m1.window, m1.kv_rank, m1.rot_dim, m1.position.base) == ("latent_attention", 37, 40, 8, 10000.0)
    assert (m2.kind, m2.chunk, m2.window, m2.values_are_keys, m2.position.scaling) == ("bias_attention", 50, 0, True, (4.0, 1.0, 3.0, 40.0))
    assert spec.blocks[1].ffn is None and spec.blocks[0].ffn.activation == "gelu_tanh"
    assert [b.side.column for b in spec.blocks] == [0, 8, 16, 24, 32, 40] and spec.blocks[0].side.table_width == 48
    for bad, what in ((lambda c: c["layers"][0].update(type="conv"), "type"),
                      (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
                      (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6), "rot_dim"),
                      (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "kv_heads"),
                      (lambda c: c["layers"][2]["mixer"].update(vdim=8), "vdim"),
                      (lambda c: c["layers"][0]["mixer"].update(conv=0), "conv"),
                      (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
                      (lambda c: c["norm"].pop("eps"), "eps")):
        c = copy.deepcopy(lc.CASE_A)
        bad(c)
        with pytest.raises(ConfigError, match=what):
            arch.read_config(c)


def test_a_chunked_plane_keeps_the_pages_of_the_chunk_a_sequence_is_in():
    from bitnet_c_b200.cache import Cache
    from bitnet_c_b200.parts import KvRequest
    c = Cache([KvRequest(2, 16, chunk=150)], [None], [None], 64 * 12, 4096, None, None, allocate=False)
    s = c.open()
    c.reserve(s, 500)  # one step over several chunks: every query needs its own chunk
    assert sorted(c.groups[0].held[s]) == list(range(8))
    c.advance(s, 500)
    assert sorted(c.groups[0].held[s]) == [7]  # position 500 looks back to 450, which lies in page 7
    for _ in range(99):
        c.reserve(s, 1)
        c.advance(s, 1)
    assert sorted(c.groups[0].held[s]) == [7, 8, 9]  # 599 tokens: the next token still sees 450..598
    c.reserve(s, 1)
    c.advance(s, 1)
    assert sorted(c.groups[0].held[s]) == [9]  # 600 tokens: the next token opens the chunk at 600, in page 9
    c.reserve(s, 3)  # 600..602 see nothing before 600
    assert sorted(c.groups[0].held[s]) == [9]
    c.advance(s, 3)
    c.close(s)
    c.check()
    assert c.groups[0].pool.n_free == 12


def test_a_plane_whose_values_lie_in_the_key_rows_has_no_value_plane():
    from bitnet_c_b200.cache import Cache
    from bitnet_c_b200.parts import KvRequest
    c = Cache([KvRequest(1, 48, window=37, v_head_dim=40, values_in_keys=True), KvRequest(1, 48, window=37, v_head_dim=40)],
              [None, None], [None, None], 64 * 4, 4096, None, None, allocate=False)
    assert len(c.groups) == 2
    assert c.groups[0].bytes_per_token(2) == 96 and c.groups[1].bytes_per_token(2) == 176
