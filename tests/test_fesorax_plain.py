"""The plain statement of the Fesorax mechanisms checked against itself (closed forms, and faults that
must show), and the library's host side for this design: configuration, tensor names, cache retention."""
import copy
import math

import numpy as np
import pytest

import fesorax_cases as fc
import plain_fesorax as pf
from helpers import random_tokens


def test_distance_buckets_are_the_distance_then_logarithmic_then_the_last():
    b = [pf.distance_bucket(n, 12, 50) for n in range(80)]
    assert b[:6] == list(range(6)) and b[6] == 6 and b[50:] == [11] * 30
    assert all(x <= y for x, y in zip(b, b[1:])) and set(b) == set(range(12))
    # the first distance of a logarithmic bucket k is 6 * (50/6)^((k-6)/6), rounded up
    for k in range(7, 11):
        assert b.index(k) == math.ceil(6 * (50 / 6) ** ((k - 6) / 6))


def test_visibility_is_causal_windowed_and_keeps_the_first():
    assert pf.visible(10, 10, 3, 0) and pf.visible(10, 8, 3, 0) and not pf.visible(10, 7, 3, 0)
    assert pf.visible(10, 1, 3, 2) and not pf.visible(10, 2, 3, 2) and not pf.visible(3, 4, 0, 9)
    assert pf.visible(500, 0, 0, 0)


def test_mlstm_recurrence_equals_its_unrolled_sum():
    rng = np.random.default_rng(0)
    T, H, d, dv = 9, 2, 3, 4
    q, k, v = rng.standard_normal((T, H, d)), rng.standard_normal((T, H, d)), rng.standard_normal((T, H, dv))
    i, f = rng.standard_normal((T, H)) * 3, -np.abs(rng.standard_normal((T, H)))
    got = pf.mlstm_recurrence(q, k, v, i, f)
    for h in range(H):
        F = np.cumsum(f[:, h])
        for t in range(T):
            # weights in the logarithm: log w_s = F_t - F_s + i_s; the stabiliser is the largest of them and F_t
            lw = F[t] - F[:t + 1] + i[:t + 1, h]
            m = max(lw.max(), F[t])
            w = np.exp(lw - m)
            num = (w[:, None] * v[:t + 1, h] * (k[:t + 1, h] @ q[t, h])[:, None]).sum(0)
            den = max(abs(float((w * (k[:t + 1, h] @ q[t, h])).sum())), math.exp(-m)) + 1e-6
            assert np.allclose(got[t, h], num / den, rtol=1e-10, atol=1e-12)


def test_router_takes_the_largest_scores_and_keeps_them_unnormalised():
    h = np.array([[1.0, 0.0], [0.0, 1.0]])
    w = np.array([[2.0, -1.0], [0.5, 3.0], [1.0, 1.0]])
    idx, s = pf.route(h, w, 2)
    assert idx.tolist() == [[0, 2], [1, 2]]
    assert np.allclose(s, 1 / (1 + np.exp(-np.array([[2.0, 1.0], [3.0, 1.0]]))))


def test_expert_clamps_gate_above_and_up_on_both_sides():
    w = {"gate": np.eye(3), "up": np.eye(3), "down": np.eye(3)}
    y = pf.expert(np.array([[5.0, -5.0, 0.5]]), w, "", 1.0)[0]
    s = lambda z: 1 / (1 + math.exp(-1.702 * z))
    assert np.allclose(y, [1.0 * s(1.0) * 2.0, -5.0 * s(-5.0) * 0.0, 0.5 * s(0.5) * 1.5])


@pytest.mark.parametrize("case", ["A", "B", "C"])
def test_faults_in_the_mechanisms_move_the_logits_of_the_test_models(case):
    """The models of the engine tests are sharp enough: each of these faults moves some logit by far
    more than the engine's float32 tolerance, so a test that passes excludes them."""
    cfg, rows = {"A": (fc.CASE_A, fc.REL_ROWS_A), "B": (fc.CASE_B, fc.REL_ROWS_B), "C": (fc.CASE_C, fc.REL_ROWS_C)}[case]
    w = fc.draw_weights(cfg, rows, seed=5)
    toks = random_tokens(4, 150, cfg["vocab"])
    ref = pf.forward(cfg, w, toks)
    assert 1.0 < np.abs(ref).max() < 100.0

    def moved(change_cfg=None, change_w=None):
        c, ww = copy.deepcopy(cfg), dict(w)
        if change_cfg:
            change_cfg(c)
        if change_w:
            change_w(ww)
        return float(np.abs(pf.forward(c, ww, toks) - ref).max())

    att = [i for i, l in enumerate(cfg["layers"]) if l["type"] == "attention" and l["mixer"].get("mask")]
    for i in att:
        m = cfg["layers"][i]["mixer"]["mask"]
        if m["size"] < 150:
            assert moved(lambda c: c["layers"][i]["mixer"]["mask"].update(size=m["size"] + 1)) > 1e-2, f"window of layer {i}"
            assert moved(lambda c: c["layers"][i]["mixer"]["mask"].update(size=m["size"] - 1)) > 1e-2, f"window of layer {i}"
            if m["keep_first"]:
                assert moved(lambda c: c["layers"][i]["mixer"]["mask"].update(keep_first=m["keep_first"] - 1)) > 1e-2, f"kept tokens of layer {i}"
            assert moved(lambda c: c["layers"][i]["mixer"]["mask"].update(keep_first=m["keep_first"] + 1)) > 1e-2, f"kept tokens of layer {i}"
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}.mix."
        if l["type"] == "attention":
            assert moved(change_w=lambda ww: ww.update({p + "rel": np.zeros_like(w[p + "rel"])})) > 1e-2, f"bias of layer {i}"
            assert moved(lambda c: c["layers"][i]["mixer"].update(bias_max=l["mixer"]["bias_max"] + 7)) > 1e-3, f"bias_max of layer {i}"
            assert moved(lambda c: c["layers"][i]["mixer"].update(scale=l["mixer"]["scale"] * 1.1)) > 1e-2, f"scale of layer {i}"
            assert moved(change_w=lambda ww: ww.update({p + "g": np.zeros_like(w[p + "g"])})) > 1e-2, f"gate of layer {i}"
        else:
            assert moved(lambda c: c["layers"][i]["mixer"].update(gate_cap=l["mixer"]["gate_cap"] * 2)) > 1e-3, f"gate cap of layer {i}"
            assert moved(change_w=lambda ww: ww.update({p + "f.b": w[p + "f.b"] + 1.0})) > 1e-2, f"forget gate of layer {i}"
        if l.get("mlp"):
            assert moved(lambda c: c["layers"][i]["mlp"]["expert"].update(limit=l["mlp"]["expert"]["limit"] * 0.1)) > 1e-2, f"limit of layer {i}"
    assert moved(lambda c: c.update(postln_alpha=cfg["postln_alpha"] + 0.3)) > 1e-2
    assert moved(lambda c: c["embedding"].update(scale=cfg["embedding"]["scale"] * 2)) > 1e-3


# ---- the library's host side ---------------------------------------------------------------------
def test_the_configuration_is_read_key_by_key_and_builds_the_parameter_table_of_the_design():
    import bitnet_c_b200 as bn
    from bitnet_c_b200.config import ConfigError, architecture_of
    from bitnet_c_b200.engine.model import parameter_table
    assert "Fesorax" in bn.known_architectures()
    shapes = fc.tensor_shapes(fc.CASE_A, fc.REL_ROWS_A)
    arch = architecture_of(fc.CASE_A)
    cfg = arch.read_config(arch.complete_config(fc.CASE_A, shapes))
    spec = arch.to_spec(cfg)
    assert [e.cache_of for e in spec.schedule] == [None, None, 1, None, None, 3]
    assert spec.embedding_scale == 3.0 and spec.blocks[0].alpha == 1.7 and spec.blocks[1].ffn is None
    m = spec.blocks[2].mixer
    assert (m.window, m.keep_first, m.bias_buckets, m.bias_max_distance, m.own_kv, m.scale) == (70, 9, 16, 90, False, 0.6)
    assert (spec.blocks[3].mixer.window, spec.blocks[3].ffn.top, spec.blocks[0].ffn.shared_limit) == (0, 4, 2.0)
    table = {arch.tensor_name(p): tuple(s.shape) for p, s in parameter_table(spec).items() if not s.optional}
    assert table == shapes
    assert arch.read_config(arch.config_to_dict(cfg)) == cfg
    for bad, what in ((lambda c: c["layers"][2]["mixer"].update(kv_from=4), "kv_from"),
                      (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "kv_from"),
                      (lambda c: c["layers"][0].update(type="conv"), "type"),
                      (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
                      (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
                      (lambda c: c.pop("postln_alpha"), "postln_alpha")):
        c = copy.deepcopy(fc.CASE_A)
        bad(c)
        with pytest.raises(ConfigError, match=what):
            arch.read_config(c)


def test_a_windowed_cache_keeps_the_first_pages_and_what_its_readers_see():
    import bitnet_c_b200 as bn
    from bitnet_c_b200.config import architecture_of
    arch = architecture_of(fc.CASE_B)
    cfg = arch.read_config(arch.complete_config(fc.CASE_B, fc.tensor_shapes(fc.CASE_B, fc.REL_ROWS_B)))
    model = bn.Model(arch.to_spec(cfg), dtype="float32", device=None)
    cache = model.new_cache(max_tokens=64 * 40, allocate=False)
    # layer 2 reads layer 0's plane with a window of 1000: the plane keeps that, and the 70 first positions
    (g,) = cache.groups
    assert (g.request.window, g.request.keep_first, g.entries) == (1000, 70, [0])
    # the same mixer alone: window 64, first 70 positions (two pages) kept
    from bitnet_c_b200.cache import Cache
    from bitnet_c_b200.parts import KvRequest
    c = Cache([KvRequest(3, 48, window=64, v_head_dim=16, keep_first=70)], [None], [None], 64 * 12, 4096, None, None,
              allocate=False)
    s = c.open()
    c.reserve(s, 700)
    assert sorted(c.groups[0].held[s]) == list(range(11))
    c.advance(s, 700)
    assert sorted(c.groups[0].held[s]) == [0, 1, 9, 10]  # positions 0..127 and 637..699
    free = c.groups[0].pool.n_free
    t = c.open()
    c.reserve(t, 64 * 7)  # the pages given back serve another sequence
    c.advance(t, 64 * 7)
    c.check()
    for _ in range(70):
        c.reserve(s, 1)
        c.advance(s, 1)
    assert sorted(c.groups[0].held[s]) == [0, 1, 11, 12]
    c.close(s)
    c.close(t)
    c.check()
    assert c.groups[0].pool.n_free == 12 and free == 8
