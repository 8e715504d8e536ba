"""The Lotilix design on the GPU against its plain statement (tests/plain_lotilix.py): every kernel it brought
alone, then whole models of small sizes (tests/lotilix_cases.py) through the step function, the cache and
state manager, the generation loop and the replay program."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import bitnet_c_b200 as bn
import lotilix_cases as lc
import plain_lotilix as pl
from helpers import (BF16_GAP_FACTOR, TOL_F32, collect_trace_output, compare, random_tokens, replay, steps_to_jsonl,
                     trace_batches, trace_chunks, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to("cuda", dtype)


def ints(a):
    return torch.tensor(list(a), dtype=torch.int32, device="cuda")


bf = pl.to_bf16


# ---- kernels alone -----------------------------------------------------------------------------------
@pytest.mark.parametrize("act,fn", [(0, pl.silu), (1, pl.gelu_tanh)])
@pytest.mark.parametrize("rows", [3, 40, 200])
def test_gated_products_take_the_activation_by_code_on_every_path(cuda_device, act, fn, rows):
    """Few rows (tcgen05 or mma.sync streaming kernels), many rows (the library product and the activation
    kernel, or this library's own product), float32: the same act(gate) * up."""
    from bitnet_c_b200.csrc import ops
    rng = np.random.default_rng(rows + act)
    K, inter = 64, 48
    x, g, u = bf(rng.standard_normal((rows, K))), bf(rng.standard_normal((inter, K)) / 4), bf(rng.standard_normal((inter, K)) / 4)
    want = fn(x @ g.T) * (x @ u.T)
    for t, tol in ((torch.float32, 2e-6), (torch.bfloat16, 2.0 ** -7)):
        w = ops.interleave_gate_up(dev(g, t), dev(u, t))
        got = ops.linear(dev(x, t), w, out_dtype=t, swiglu=True, act=act).float().cpu().numpy()
        assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max())
        was = (ops.USE_TCGEN05, ops.USE_OWN_GEMM)
        try:
            ops.USE_TCGEN05, ops.USE_OWN_GEMM = False, True
            got = ops.linear(dev(x, t), w, out_dtype=t, swiglu=True, act=act).float().cpu().numpy()
        finally:
            ops.USE_TCGEN05, ops.USE_OWN_GEMM = was
        assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("width", [50, 192, 1030])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_kernels_of_the_parallel_block(cuda_device, width, dtype):
    from bitnet_c_b200.csrc import ops
    rng = np.random.default_rng(width)
    t = DT[dtype]
    n = 7
    x, a, b = rng.standard_normal((n, width)), bf(rng.standard_normal((n, width))), rng.standard_normal((n, width))
    xd = dev(x)
    cast = ops.residual_add(xd, dev(a, t), dev(b), cast=t)
    want = x.astype(np.float32).astype(np.float64) + (a + b.astype(np.float32))
    assert np.abs(xd.cpu().numpy() - want).max() < 1e-6 * np.abs(want).max()
    assert np.array_equal(cast.float().cpu().numpy(), xd.cpu().numpy() if dtype == "float32" else bf(xd.cpu().numpy()))
    ops.residual_add(xd, dev(a, t))
    assert np.abs(xd.cpu().numpy() - (want + a)).max() < 1e-6 * np.abs(want).max()
    # a delta that enters through its own norm, and the next norm in the same pass
    y, wy, wn = rng.standard_normal((n, width)) * 3, bf(1 + 0.2 * rng.standard_normal(width)), bf(1 + 0.2 * rng.standard_normal(width))
    xd = dev(x)
    out = ops.add_normed(xd, dev(y), dev(wy, t), 1e-5, dev(wn, t), 1e-6, t)
    x2 = x.astype(np.float32).astype(np.float64) + pl.rms_norm(y.astype(np.float32).astype(np.float64), wy, 1e-5)
    assert np.abs(xd.cpu().numpy() - x2).max() < 1e-6 * np.abs(x2).max()
    tol = 1e-6 if dtype == "float32" else 2.0 ** -8
    assert np.abs(out.float().cpu().numpy() - pl.rms_norm(x2, wn, 1e-6)).max() < tol * 4
    xd = dev(x)
    assert ops.add_normed(xd, dev(y), dev(wy, t), 1e-5) is None
    assert np.abs(xd.cpu().numpy() - x2).max() < 1e-6 * np.abs(x2).max()
    # norms of two slices of a row, each with its gain, the rest of the row untouched
    row = bf(rng.standard_normal((n, width)))
    l0, l1 = width // 3, width // 2
    g0, g1 = bf(1 + 0.2 * rng.standard_normal(l0)), bf(1 + 0.2 * rng.standard_normal(l1))
    rd = dev(row, t)
    ops.rmsnorm_slices(rd, 1e-5, 2, l0, dev(g0, t), 2 + l0, l1, dev(g1, t))
    ref = row.copy()
    ref[:, 2:2 + l0] = pl.rms_norm(row[:, 2:2 + l0], g0, 1e-5)
    ref[:, 2 + l0:2 + l0 + l1] = pl.rms_norm(row[:, 2 + l0:2 + l0 + l1], g1, 1e-5)
    assert np.abs(rd.float().cpu().numpy() - ref).max() < (1e-5 if dtype == "float32" else 2.0 ** -7) * np.abs(ref).max()
    # the gated row of the second embedding; an id outside the table gives zeros
    table, pre = bf(rng.standard_normal((11, 20))), bf(rng.standard_normal((n, 6)))
    toks = [3, 10, 0, 11, 5, 5, 9]
    got = ops.gated_lookup(dev(pre, t), dev(table, t), 7, ints(toks), 5, 1).float().cpu().numpy()
    ref = pl.gelu_tanh(pre[:, :5]) * np.stack([table[k, 7:12] if k < 11 else np.zeros(5) for k in toks])
    assert np.abs(got - ref).max() < (1e-6 if dtype == "float32" else 2.0 ** -7) * max(1.0, np.abs(ref).max())


def _cache_for(lens, n_heads, row, v_row, t, poison=True):
    """A paged cache for sequences of the given lengths in scattered pages, and what a step needs to address it."""
    pages = [(n + 63) // 64 for n in lens]
    order = np.random.default_rng(5).permutation(sum(pages) + 3)
    table = np.zeros((len(lens) + 2, max(pages)), dtype=np.int32)
    at = 0
    for s, p in enumerate(pages):
        table[s + 1, :p] = order[at:at + p]  # sequence s lives in slot s + 1
        at += p
    k = torch.full((sum(pages) + 3, n_heads, 64, row), float("nan") if poison else 0.0, dtype=t, device="cuda")
    v = torch.full((sum(pages) + 3, n_heads, 64, v_row), float("inf") if poison else 0.0, dtype=t, device="cuda") if v_row else None
    return k, v, torch.from_numpy(table).cuda()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,rot,rot_off", [(4, 2, 16, 8, 0), (3, 1, 20, 10, 10), (2, 2, 32, 32, 0)])
def test_pairs_are_rotated_in_place_and_keys_and_unrotated_values_reach_the_cache(cuda_device, dtype, H, G, d, rot, rot_off):
    from bitnet_c_b200.csrc import ops
    rng = np.random.default_rng(H * 100 + d)
    t = DT[dtype]
    lens, new = [70, 5, 130], [3, 5, 66]
    T = sum(new)
    pos = np.concatenate([np.arange(n - c, n) for n, c in zip(lens, new)])
    seq = np.concatenate([np.full(c, i) for i, c in enumerate(new)])
    freqs = pl.rotary_frequencies({"base": 30.0, "dims": rot})
    q, k = bf(rng.standard_normal((T, H, d))), bf(rng.standard_normal((T, G, d)))
    rows = dev(np.concatenate([q.reshape(T, -1), k.reshape(T, -1)], axis=1), t)
    kc, vc, table = _cache_for(lens, G, d, d, t)
    ops.rotary_pairs_append(rows, dev(freqs), ints(pos), q_off=0, n_q_heads=H, q_head_stride=d, q_rot_off=rot_off,
                            k_off=H * d, n_k_heads=G, k_head_stride=d, k_rot_off=rot_off, k_row=d, v_off=H * d, v_head_stride=d,
                            v_row=d, tok_seq=ints(seq), slots=ints([1, 2, 3]), page_table=table, k_cache=kc, v_cache=vc)

    def turned(x):
        out = x.copy()
        out[..., rot_off:rot_off + rot] = pl.rotate_pairs(x[..., rot_off:rot_off + rot], pos, freqs)
        return out

    tol = 2e-5 if dtype == "float32" else 2.0 ** -7
    got = rows.float().cpu().numpy()
    assert np.abs(got[:, :H * d].reshape(T, H, d) - turned(q)).max() < tol * 5
    assert np.abs(got[:, H * d:].reshape(T, G, d) - turned(k)).max() < tol * 5
    tab = table.cpu().numpy()
    for i in range(T):
        page, r = tab[seq[i] + 1, pos[i] // 64], pos[i] % 64
        assert np.abs(kc[page, :, r].float().cpu().numpy() - turned(k)[i]).max() < tol * 5
        assert np.array_equal(vc[page, :, r].float().cpu().numpy(), k[i].astype(np.float32))


def _plain_attention(q, keys, values, pos, scale, rule, size, gate=None):
    """q [H, d] at position pos over keys [n, G, d], values [n, G, dv] by the plain rules."""
    H, G = q.shape[0], keys.shape[1]
    out = np.zeros((H, values.shape[2]))
    seen = np.array([rule(pos, j, size) for j in range(keys.shape[0])])
    for h in range(H):
        g = h // (H // G)
        s = np.where(seen, keys[:, g] @ q[h] * scale, -np.inf)
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ values[:, g]
        if gate is not None:
            out[h] *= pl.sigmoid(gate[h])
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mask,size", [("chunk", 50), ("chunk", 64), ("chunk", 7), ("window", 37), ("window", 64), ("none", 0)])
@pytest.mark.parametrize("H,G", [(4, 2), (8, 2), (3, 1)])
def test_attention_at_the_edges_of_chunks_and_windows_with_one_key_that_stands_out(cuda_device, dtype, mask, size, H, G):
    """Among some hundred keys the one just outside the mask gets a score far above all others, and so does,
    in a second run, the one just inside: the first must not show in the result, the second must own it.
    Both kernels (any mix of tokens; runs of new tokens on the tensor cores), values inside the key rows or in
    a plane of their own, single tokens and runs that cross the edges; two, four and three query heads on a
    key/value head (the general kernel takes them two or four at a time, or one by one)."""
    from bitnet_c_b200.csrc import ops
    t = DT[dtype]
    rng = np.random.default_rng(size + len(mask))
    d, dv = 32, 16
    rule = {"chunk": pl.sees_chunk, "window": pl.sees_window, "none": pl.sees_window}[mask]
    lens, new = [200, 131, 64], [1, 70, 64]
    T = sum(new)
    pos = np.concatenate([np.arange(n - c, n) for n, c in zip(lens, new)])
    seq = np.concatenate([np.full(c, i) for i, c in enumerate(new)])
    starts = np.concatenate([[0], np.cumsum(new)])
    kw = dict(chunk=size) if mask == "chunk" else {}
    window = size if mask == "window" else 0
    for shared_rows in (False, True):
        for which in ("outside", "inside"):
            keys = [bf(rng.standard_normal((n, G, d)) * 0.3) for n in lens]
            vals = [k[..., :dv] if shared_rows else bf(rng.standard_normal((k.shape[0], G, dv))) for k in keys]
            q = bf(rng.standard_normal((T, H, d)) * 0.3)
            gate = bf(rng.standard_normal((T, H)))
            # the token that asks: the last one of sequence 0, and one in the middle of sequence 1's run
            for s, i in ((0, starts[1] - 1), (1, starts[1] + 40)):
                p = int(pos[i])
                lo = (p // size) * size if mask == "chunk" else (max(0, p - size + 1) if mask == "window" else 0)
                j = lo - 1 if which == "outside" else lo
                if j < 0:
                    continue
                keys[s][j] = 0.0
                keys[s][j, :, 0] = 8.0
                q[i, :, 0] = 8.0  # a score of 64 * scale among scores of order one
            kc, vc, table = _cache_for(lens, G, d, 0 if shared_rows else dv, t)
            tab = table.cpu().numpy()
            for s, n in enumerate(lens):
                for p in range(n):
                    kc[tab[s + 1, p // 64], :, p % 64] = dev(keys[s][p], t)
                    if not shared_rows:
                        vc[tab[s + 1, p // 64], :, p % 64] = dev(vals[s][p], t)
            want = np.stack([_plain_attention(q[i], keys[seq[i]][:pos[i] + 1], vals[seq[i]][:pos[i] + 1], int(pos[i]), 0.7, rule,
                                              size, gate[i]) for i in range(T)]).reshape(T, H * dv)
            qd, gd = dev(q.reshape(T, H * d), t), dev(gate, t)
            args = (ints(seq), ints(pos), ints([1, 2, 3]), table, kc, vc)
            extra = dict(gate=gd, gate_stride=H, v_dim=dv if shared_rows else 0, **kw)
            out = torch.empty((T, H * dv), dtype=t, device="cuda")
            ops.attention_general(qd, H * d, out, T, H, G, d, 0.7, window, *args, **extra)
            tol = (2e-5 if dtype == "float32" else 2.0 ** -6) * max(1.0, np.abs(want).max())
            assert np.abs(out.float().cpu().numpy() - want).max() < tol, (mask, size, which, shared_rows, "general")
            if dtype == "bfloat16":
                tiles = [(s, r) for s, c in enumerate(new) for r in range(0, c, 64)]
                out2 = torch.empty_like(out)
                ops.attention_prefill(qd, H * d, out2, H, G, d, 0.7, window, ints([s for s, _ in tiles]), ints([r for _, r in tiles]),
                                      ints(starts), ints([n - c for n, c in zip(lens, new)]), ints([1, 2, 3]), table, kc, vc,
                                      precise=True, **extra)
                assert np.abs(out2.float().cpu().numpy() - want).max() < tol, (mask, size, which, shared_rows, "tiled")


@pytest.mark.parametrize("H,G,d,dv,taps", [(4, 2, 16, 24, 4), (1, 1, 40, 136, 2), (2, 1, 20, 36, 1), (2, 2, 130, 40, 3), (3, 3, 256, 8, 16)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_delta_rule_kernels_alone_and_carrying_their_state(cuda_device, H, G, d, dv, taps, dtype):
    from bitnet_c_b200.csrc import ops
    rng = np.random.default_rng(H * 1000 + d)
    t = DT[dtype]
    lens = [37, 1, 12]
    T = sum(lens)
    n_qk, n_v = G * d, H * dv
    proj = bf(rng.standard_normal((T, 2 * n_qk + n_v + H)))
    conv = bf(rng.standard_normal((2 * n_qk + n_v, taps)) * 0.7)
    a_raw, dt_bias, a_log = rng.standard_normal((T, H * d)), bf(rng.standard_normal(H * d) - 1), bf(rng.standard_normal(H) - 1)
    gate_raw = rng.standard_normal((T, n_v))
    up = dev(np.concatenate([a_raw, gate_raw], axis=1))
    a_raw, gate_raw = a_raw.astype(np.float32).astype(np.float64), gate_raw.astype(np.float32).astype(np.float64)
    starts = np.concatenate([[0], np.cumsum(lens)])
    want = np.zeros((T, H, dv))
    for a, b in zip(starts, starts[1:]):
        x = proj[a:b]
        q = pl.unit_vector(pl.silu(pl.short_convolution(x[:, :n_qk], conv[:n_qk])).reshape(-1, G, d)) * d ** -0.5
        k = pl.unit_vector(pl.silu(pl.short_convolution(x[:, n_qk:2 * n_qk], conv[n_qk:2 * n_qk])).reshape(-1, G, d))
        v = pl.silu(pl.short_convolution(x[:, 2 * n_qk:2 * n_qk + n_v], conv[2 * n_qk:])).reshape(-1, H, dv)
        beta = pl.sigmoid(x[:, 2 * n_qk + n_v:])
        g = np.exp(-np.exp(a_log)[None, :, None] * pl.softplus(a_raw[a:b] + dt_bias).reshape(-1, H, d))
        for h in range(H):
            want[a:b, h], _ = pl.delta_rule(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], g[:, h], beta[:, h])
    want = want.reshape(T, n_v)
    state = torch.zeros((5, ops.delta_state_floats(H, G, d, dv, taps)), dtype=torch.float32, device="cuda")
    state[1].fill_(7.0)  # a slot that is not in the step keeps what it holds
    rows, cw, bias, alog = dev(proj, t), dev(conv, t), dev(dt_bias, t), dev(a_log, t)
    # in three steps: 20 tokens of sequence 0 with all of sequence 1; two more tokens of sequence 0 (fewer than
    # the taps reach back) with sequence 2; the rest of sequence 0 alone
    got = np.zeros((T, n_v), dtype=np.float32)
    for idx, seqs, slots in ((np.r_[0:20, 37:38], [20, 1], [3, 0]), (np.r_[20:22, 38:50], [2, 12], [3, 4]), (np.r_[22:37], [15], [3])):
        o = ops.delta_rule(rows[idx].contiguous(), 0, n_qk, 2 * n_qk, cw, taps, 2 * n_qk + n_v, up[idx].contiguous(), bias, alog, state,
                           ints(np.concatenate([np.full(c, i) for i, c in enumerate(seqs)])), ints(np.concatenate([[0], np.cumsum(seqs)])),
                           ints(slots), len(seqs), H, G, d, dv)
        got[idx] = o.cpu().numpy()
    assert np.abs(got - want).max() < 3e-4 * max(1.0, np.abs(want).max())
    assert bool((state[1] == 7.0).all()) and bool((state[2] == 0.0).all())
    gain = bf(1 + 0.3 * rng.standard_normal(dv))
    y = ops.delta_output(dev(want), dev(gain, t), up[:, H * d:], H, dv, 1e-5, t).float().cpu().numpy()
    ref = (pl.rms_norm(want.astype(np.float32).reshape(T, H, dv).astype(np.float64), gain, 1e-5) * pl.sigmoid(gate_raw).reshape(T, H, dv))
    assert np.abs(y - ref.reshape(T, n_v)).max() < (1e-5 if dtype == "float32" else 2.0 ** -7) * max(1.0, np.abs(ref).max())


# ---- whole models ------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, ranks) in lc.CASES.items():
        w = lc.draw_weights(cfg, ranks, seed=21)
        out[name] = (lc.write_folder(str(tmp_path_factory.mktemp("lotilix") / name), cfg, w), w)
    return out


_ROUNDED = {}


def _check(got, cfg, w, reqs, plain, dtype, what, rough_ok=False):
    """float32: every position within 1e-4 of the plain logits (relative to the largest).  bfloat16: the bound
    of a request is three times what rounding the stored activations does to the plain statement, taken at the
    request's 80th percentile of positions (sharp models answer single roundings in a recurrence or next to
    a mask's edge with gaps several times the typical one, in the engine at other places than in the rounded
    plain statement); at most a fifth of a request's positions may lie beyond it, none beyond three times the
    largest gap.  ``rough_ok``: a request whose bound would exceed a tenth of its largest logit is only looked at
    for non-finite numbers."""
    if dtype == "float32":
        return compare(got, plain, lambda ref: TOL_F32 * max(1.0, float(np.abs(ref).max())), what)
    for r, per_pos in got.items():
        key = (cfg["vocab"], r, tuple(reqs[r]))
        if key not in _ROUNDED:
            _ROUNDED[key] = pl.forward(cfg, w, reqs[r], round_fn=pl.to_bf16)
        gap = np.abs(plain[r] - _ROUNDED[key]).max(axis=1)
        bound = BF16_GAP_FACTOR * float(np.percentile(gap, 80))
        if rough_ok and bound >= 0.1 * float(np.abs(plain[r]).max()):
            # a model drawn at random that answers bfloat16 rounding with a tenth of its logits: only float32 tells
            assert all(np.isfinite(row).all() for row in per_pos.values()), f"{what}: request {r}"
            continue
        assert bound < 0.1 * float(np.abs(plain[r]).max()), "the test model is too rough for bfloat16"
        err = np.array([np.abs(row.astype(np.float64) - plain[r][p]).max() for p, row in sorted(per_pos.items())])
        assert np.isfinite(err).all() and err.max() <= BF16_GAP_FACTOR * float(gap.max()), f"{what}: request {r}"
        beyond = int((err > bound).sum())
        assert beyond <= max(1, len(err) // 5), (f"{what}: request {r}: {beyond} of {len(err)} positions beyond {bound:.3e}; "
                                                 f"first at {sorted(per_pos)[int(np.argmax(err > bound))]}")


def _poison(cache):
    """Pages and state rows that nobody holds may contain anything."""
    for g in cache.groups:
        g.k.fill_(float("nan"))
        if g.v is not None:
            g.v.fill_(float("inf"))
    for s in cache.states.values():
        s.fill_(float("nan"))


@pytest.mark.parametrize("case", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_step_like_the_plain_statement_however_the_tokens_are_cut(folders, cuda_device, case, dtype):
    cfg = lc.CASES[case][0]
    d, w = folders[case]
    V = cfg["vocab"]
    reqs = {"a": random_tokens(1, 210, V), "b": random_tokens(2, 3, V), "c": random_tokens(3, 77, V), "d": random_tokens(4, 131, V)}
    plain = {r: pl.forward(cfg, w, t) for r, t in reqs.items()}
    model = bn.load_model(d, dtype=dtype)
    cache = model.new_cache(max_tokens=64 * 12, max_seqs=4)
    _poison(cache)
    schedules = (
        ("whole", trace_whole(reqs)),
        ("every token alone", trace_tail({"c": reqs["c"], "b": reqs["b"]}, 1000)),
        ("150 tokens decoded one by one", trace_tail({"a": reqs["a"]}, 150)),
        ("pieces down to two tokens", trace_chunks(reqs, pieces=(2, 1, 5, 64, 33))),
        ("pieces of a page and around it", trace_chunks({"a": reqs["a"], "d": reqs["d"]}, pieces=(63, 1, 64, 65), stagger=2)),
        ("unequal batches, slots and pages used again",
         trace_batches([{"a": (reqs["a"], 40), "b": (reqs["b"], 2), "c": (reqs["c"], 9)},
                        {"d": (reqs["d"], 70), "b": (reqs["b"], 1)}, {"c": (reqs["c"], 76), "a": (reqs["a"], 3)}])),
    )
    for what, steps in schedules:
        _check(replay(model, cache, steps), cfg, w, reqs, plain, dtype, f"case {case}, {what}, {dtype}")
        assert cache.slots.n_free == cache.slots.n_slots
    model.check_kernels()


@pytest.mark.parametrize("case", ["A", "C"])
def test_a_request_alone_and_in_a_batch_give_the_same_logits(folders, cuda_device, case):
    """Beyond rounding nothing of the batch around a request reaches it: in float32 the same numbers to 1e-5."""
    cfg = lc.CASES[case][0]
    d, _w = folders[case]
    V = cfg["vocab"]
    reqs = {"a": random_tokens(11, 140, V), "b": random_tokens(12, 66, V), "c": random_tokens(13, 5, V)}
    model = bn.load_model(d, dtype="float32")
    cache = model.new_cache(max_tokens=64 * 10, max_seqs=3)
    alone = replay(model, cache, trace_tail(reqs, 8))
    _poison(cache)
    together = replay(model, cache, trace_batches([{r: (t, min(8, len(t) - 1)) for r, t in reqs.items()}]))
    for r in reqs:
        for p, row in together[r].items():
            assert np.abs(row - alone[r][p]).max() < 1e-5 * max(1.0, np.abs(row).max()), (r, p)


def test_a_long_prompt_and_long_decoding_far_past_every_mask(folders, cuda_device):
    """1,100 tokens in one step and 300 more one by one: pages of windows and chunks are given back and taken
    again many times over, the delta rule's state runs on."""
    cfg = lc.CASES["C"][0]
    d, w = folders["C"]
    toks = random_tokens(7, 1400, cfg["vocab"])
    plain = {"x": pl.forward(cfg, w, toks)}
    model = bn.load_model(d, dtype="float32")
    cache = model.new_cache(max_tokens=64 * 20, max_seqs=2)
    _poison(cache)
    got = replay(model, cache, trace_tail({"x": toks}, 300))
    compare(got, plain, lambda ref: 3 * TOL_F32 * max(1.0, float(np.abs(ref).max())), "long")
    held = max(len(h) for g in cache.groups for h in [g.held])  # nothing is held after the end
    assert held == 0 or all(not h for g in cache.groups for h in g.held.values())


ONE_KIND = {
    "delta": [{"type": "channel_delta", "mixer": {"heads": 3, "kv_heads": 1, "dim": 24, "vdim": 40, "conv": 4},
               "mlp": {"kind": "dense", "ff": 96}}] * 3,
    "latent": [{"type": "latent_attention", "mixer": {"heads": 5, "dim": 24, "rot_dim": 8, "vdim": 16, "q_rank": 40, "kv_rank": 72,
                                                      "scale": 0.3, "rot": {"base": 1e4, "dims": 8}, "mask": {"size": 1}},
                "mlp": None}] * 2,
    "attention": [{"type": "attention", "mixer": {"heads": 6, "kv_heads": 3, "dim": 16, "vdim": 16, "scale": 0.5,
                                                  "rot": {"base": 1e4, "dims": 16}, "mask": {"size": 1}},
                   "mlp": {"kind": "dense", "ff": 96}},
                  {"type": "attention", "mixer": {"heads": 6, "kv_heads": 6, "dim": 16, "vdim": 16, "scale": 0.5,
                                                  "rot": {"base": 1e4, "dims": 2}, "mask": {"size": 100000}},
                   "mlp": {"kind": "dense", "ff": 96}}],
}


@pytest.mark.parametrize("kind", sorted(ONE_KIND))
@pytest.mark.parametrize("side", [True, False])
def test_models_of_one_kind_of_mixer_only(tmp_path, cuda_device, kind, side):
    """No key/value planes at all, or no per-sequence state at all; masks of one position and of more than any
    prompt; the value width of the chunked mixer left out of the configuration; with and without the side input."""
    import copy
    cfg = {"architecture": "Lotilix", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "layers": copy.deepcopy(ONE_KIND[kind])}
    if side:
        cfg["token_side"] = {"dim": 16}
    ranks = {i: (5, 9) for i, l in enumerate(cfg["layers"]) if l["type"] == "channel_delta"}
    w = lc.draw_weights(cfg, ranks, seed=3)
    if kind == "attention":
        cfg["layers"][1]["mixer"].pop("vdim")
    folder = lc.write_folder(str(tmp_path / "m"), cfg, w)
    reqs = {"a": random_tokens(1, 150, 300), "b": random_tokens(2, 70, 300), "c": random_tokens(3, 1, 300)}
    plain = {r: pl.forward(cfg, w, t) for r, t in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        model = bn.load_model(folder, dtype=dtype)
        cache = model.new_cache(max_tokens=64 * 8, max_seqs=3)
        _poison(cache)
        for what, steps in (("whole", trace_whole(reqs)), ("last 30 one by one", trace_tail(reqs, 30)),
                            ("an unequal batch", trace_batches([{"a": (reqs["a"], 20), "b": (reqs["b"], 30), "c": (reqs["c"], 0)}]))):
            _check(replay(model, cache, steps), cfg, w, reqs, plain, dtype, f"{kind} only, {what}, {dtype}", rough_ok=True)
        model.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point_and_the_replay_program(folders, cuda_device, tmp_path, dtype):
    cfg = lc.CASES["A"][0]
    d, w = folders["A"]
    V = cfg["vocab"]
    model = bn.load_model(d, dtype=dtype)
    prompts = [random_tokens(31, 50, V), random_tokens(32, 3, V), random_tokens(33, 120, V)]
    got = bn.generate(model, prompts, max_new_tokens=[70, 20, 24])
    for p, g in zip(prompts, got):
        assert len(g.tokens) in (70, 20, 24) and g.finish_reason == "length"
        seq = list(p) + g.tokens[:-1]
        ref = pl.forward(cfg, w, seq)[len(p) - 1:]
        if dtype == "float32":
            slack = 2 * TOL_F32 * max(1.0, float(np.abs(ref).max()))
        else:
            slack = 2 * BF16_GAP_FACTOR * float(np.abs(pl.forward(cfg, w, seq, round_fn=pl.to_bf16)[len(p) - 1:] - ref).max())
        off = [i for i, t in enumerate(g.tokens) if ref[i, t] < ref[i].max() - slack]
        assert not off, f"tokens {off[:5]} of a prompt of {len(p)} are not the plain statement's"
    # a second call on the same model: slots, pages and state rows are used again
    again = bn.generate(model, prompts[::-1], max_new_tokens=[24, 20, 70])
    assert [g.tokens for g in again[::-1]] == [g.tokens for g in got]
    if dtype != "float32":
        return
    reqs = {"x": prompts[0] + got[0].tokens, "y": prompts[1]}
    steps = trace_tail(reqs, 6)
    out = str(tmp_path / "out")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", out,
                        "--max-tokens", "256"], input=steps_to_jsonl(steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    plain = {k: pl.forward(cfg, w, t) for k, t in reqs.items()}
    compare(collect_trace_output(steps, out, V), plain, lambda ref: TOL_F32 * max(1.0, float(np.abs(ref).max())),
            "through bin/trace_run")


def test_the_command_line_writes_a_random_model_of_the_design_and_generates_from_it(tmp_path, cuda_device):
    import json
    cfgp = tmp_path / "cfg.json"
    cfgp.write_text(json.dumps(lc.CASE_C))
    folder = tmp_path / "m"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "bitnet"), str(folder), "--random-weights", "--config", str(cfgp),
           "--weight-seed", "3", "--dtype", "float32", "--prompt-token-ids", "5,17,3,9,9,1", "--prompt-token-ids", "7",
           "-n", "9", "--repeat-penalty", "1.0", "--token-ids"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [[int(t) for t in l.split(",")] for l in p.stdout.splitlines() if l.strip()]
    assert [len(l) for l in lines] == [9, 9] and "Generation complete tokens=18" in p.stderr
