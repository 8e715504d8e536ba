"""The Fesorax design on the GPU against its plain statement (tests/plain_fesorax.py): every kernel it
brought alone, then whole models of small sizes (tests/fesorax_cases.py) through the step function, the
cache and state manager, the generation loop and the replay program."""
import os
import subprocess
import sys
import types

import numpy as np
import pytest
import torch

import bitnet_c_b200 as bn
import fesorax_cases as fc
import plain_fesorax as pf
import plain_llama
from helpers import (BF16_GAP_FACTOR, TOL_F32, collect_trace_output, compare, random_tokens, replay, steps_to_jsonl,
                     trace_batches, trace_chunks, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to("cuda", dtype)


def bf(a):
    return plain_llama.to_bf16(np.asarray(a, dtype=np.float64))


# ---- kernels alone -----------------------------------------------------------------------------------
@pytest.mark.parametrize("width", [48, 200, 1030])
def test_norm_after_the_sum(cuda_device, width):
    from bitnet_c_b200.csrc import ops
    rng = np.random.default_rng(width)
    x, d, w = rng.standard_normal((7, width)), bf(rng.standard_normal((7, width))), bf(1 + 0.2 * rng.standard_normal(width))
    want = pf.rms_norm(1.75 * x.astype(np.float32).astype(np.float64) + d, w, 1e-5)
    xd = dev(x)
    out = torch.empty((7, width), dtype=torch.bfloat16, device="cuda")
    ops.scaled_add_rmsnorm(xd, 1.75, dev(d, torch.bfloat16), dev(w, torch.bfloat16), 1e-5, out)
    assert np.abs(xd.cpu().numpy() - want).max() < 1e-5 * np.abs(want).max()
    assert np.array_equal(out.float().cpu().numpy(), bf(xd.cpu().numpy()))
    xd = dev(x)
    ops.scaled_add_rmsnorm(xd, 1.75, None, dev(w), 1e-5)  # nothing to add, float32 gain, no copy
    assert np.abs(xd.cpu().numpy() - pf.rms_norm(1.75 * x.astype(np.float32).astype(np.float64), w, 1e-5)).max() < 1e-5 * np.abs(want).max()


@pytest.mark.parametrize("H,d,dv", [(3, 8, 8), (1, 40, 136), (2, 100, 300), (1, 160, 40)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mlstm_kernels_alone_and_carrying_their_state(cuda_device, H, d, dv, dtype):
    from bitnet_c_b200.csrc import ops
    rng = np.random.default_rng(H * 1000 + d)
    width, lens = 40, [37, 1, 12]
    T = sum(lens)
    h = bf(rng.standard_normal((T, width)))
    w = {"i": bf(rng.standard_normal((H, width)) * 0.3), "f": bf(rng.standard_normal((H, width)) * 0.3),
         "i.b": bf(rng.standard_normal(H) * 2), "f.b": bf(rng.standard_normal(H) * 2 + 1)}
    cap = 3.0
    gi, gf = pf.mlstm_gates(h, w, "", {"gate_cap": cap})
    t = DT[dtype]
    gates = ops.mlstm_gates(dev(h, t), dev(np.concatenate([w["i"], w["f"]]), t), dev(np.concatenate([w["i.b"], w["f.b"]]), t), H, cap)
    assert np.abs(gates.cpu().numpy() - np.concatenate([gi, gf], axis=1)).max() < 2e-5
    q, k, v = bf(rng.standard_normal((T, H, d))), bf(rng.standard_normal((T, H, d))), bf(rng.standard_normal((T, H, dv)))
    rows = dev(np.concatenate([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], axis=1), t)
    state = torch.zeros((5, H, ops.mlstm_state_floats(d, dv)), dtype=torch.float32, device="cuda")
    state[1].fill_(7.0)  # a slot that is not in the step keeps what it holds
    slots = torch.tensor([3, 0, 4], dtype=torch.int32, device="cuda")
    starts = np.concatenate([[0], np.cumsum(lens)])
    want = np.concatenate([pf.mlstm_recurrence(q[a:b] * d ** -0.5, k[a:b], v[a:b], gi[a:b], gf[a:b])
                           for a, b in zip(starts, starts[1:])]).reshape(T, H * dv)
    # in two steps: the first 20 tokens of sequence 0 with all of sequence 1, then the rest
    first = [0, 20, 21]
    step1 = np.r_[0:20, 37:38]
    step2 = np.r_[20:37, 38:50]
    got = np.zeros((T, H * dv), dtype=np.float32)
    o = ops.mlstm_recurrence(rows[step1].contiguous(), H * d, 2 * H * d, gates[step1].contiguous(), state,
                             torch.tensor(first, dtype=torch.int32, device="cuda"), slots[:2].contiguous(), 2, H, d, dv, d ** -0.5)
    got[step1] = o.cpu().numpy()
    o = ops.mlstm_recurrence(rows[step2].contiguous(), H * d, 2 * H * d, gates[step2].contiguous(), state,
                             torch.tensor([0, 17, 29], dtype=torch.int32, device="cuda"), slots[[0, 2]].contiguous(), 2, H, d, dv, d ** -0.5)
    got[step2] = o.cpu().numpy()
    assert np.abs(got - want).max() < 2e-4 * max(1.0, np.abs(want).max())
    assert bool((state[1] == 7.0).all()) and bool((state[2] == 0.0).all())
    # the same by chunks of 32 tokens (other order of the sums), in the same two steps, and the states agree
    state2 = torch.zeros_like(state)
    got2 = np.zeros_like(got)
    for rows_of, starts_of, slots_of in ((step1, first, slots[:2]), (step2, [0, 17, 29], slots[[0, 2]])):
        o = ops.mlstm_recurrence(rows[rows_of].contiguous(), H * d, 2 * H * d, gates[rows_of].contiguous(), state2,
                                 torch.tensor(starts_of, dtype=torch.int32, device="cuda"), slots_of.contiguous(), 2, H, d, dv,
                                 d ** -0.5, chunks=True)
        got2[rows_of] = o.cpu().numpy()
    assert np.abs(got2 - want).max() < 5e-4 * max(1.0, np.abs(want).max())
    live = [0, 3, 4]
    # S and n are kept relative to the stabiliser m: compare what they stand for, e^m S
    a, b = state[live].cpu().numpy().astype(np.float64), state2[live].cpu().numpy().astype(np.float64)
    assert np.abs(a[..., -1] - b[..., -1]).max() < 1e-3
    assert np.abs(a[..., :-1] - b[..., :-1] * np.exp(b[..., -1:] - a[..., -1:])).max() < 1e-3 * max(1.0, np.abs(a[..., :-1]).max())
    gain, g = bf(1 + 0.3 * rng.standard_normal(H * dv)), bf(rng.standard_normal((T, H * dv)))
    y = ops.mlstm_output(dev(want), dev(gain, t), dev(g, t), H * dv, H, dv, 1e-5, t).float().cpu().numpy()
    ref = (pf.unit_rms(want.astype(np.float32).reshape(T, H, dv).astype(np.float64), 1e-5).reshape(T, H * dv) * gain * pf.sigmoid(g))
    assert np.abs(y - ref).max() < (1e-5 if dtype == "float32" else 2.0 ** -7) * max(1.0, np.abs(ref).max())


def _ctx(decode=False):
    return types.SimpleNamespace(decode=decode, diag=None, tap=lambda *a, **k: None)


@pytest.mark.parametrize("E,top,ff,shared_ff", [(5, 2, 40, 24), (4, 4, 24, 0), (2, 1, 8, 56), (33, 3, 16, 16)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixture_of_experts_few_rows_and_many_rows(cuda_device, E, top, ff, shared_ff, dtype):
    from bitnet_c_b200.config import MoeSpec
    from bitnet_c_b200.csrc import ops
    from bitnet_c_b200.parts import BuildContext, build_part
    rng = np.random.default_rng(E * 10 + top)
    width, T = 64, 90
    w = {"router": bf(rng.standard_normal((E, width)) * 0.3)}
    names = [(f"e{e}", ff) for e in range(E)] + ([("shared", shared_ff)] if shared_ff else [])
    for n, f in names:
        w[f"{n}.gate"], w[f"{n}.up"] = bf(rng.standard_normal((f, width)) / 8), bf(rng.standard_normal((f, width)) / 8)
        w[f"{n}.down"] = bf(rng.standard_normal((width, f)) / np.sqrt(f))
    h = bf(rng.standard_normal((T, width)))
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": 0.8}}
    if shared_ff:
        mlp["shared"] = {"ff": shared_ff, "limit": 1.3}
    exact = pf.moe(h, w, "", mlp)
    t = DT[dtype]
    # the router: the same experts in the same order, the same scores
    ids, weights = ops.moe_route(dev(h, t), dev(w["router"], t), top)
    ref_ids, ref_s = pf.route(h, w["router"], top)
    assert np.array_equal(ids.cpu().numpy(), ref_ids) and np.abs(weights.cpu().numpy() - ref_s).max() < 1e-6
    part = build_part("ffn", MoeSpec(width=width, n_experts=E, top=top, expert_ff=ff, expert_limit=0.8, shared_ff=shared_ff,
                                     shared_limit=1.3), BuildContext(t, torch.device("cuda")))
    assert {k for k in part.params()} == set(w)
    part.bind({k: dev(a, t) for k, a in w.items()})
    if dtype == "float32":
        tol = 1e-5 * max(1.0, np.abs(exact).max())
    else:
        tol = BF16_GAP_FACTOR * np.abs(exact - pf.moe(h, w, "", mlp, plain_llama.to_bf16)).max()
    many = part.forward(dev(h, t), _ctx()).cpu().numpy()       # sorted by expert, expert by expert
    few = part.forward(dev(h, t), _ctx(decode=True)).cpu().numpy()  # streamed per (token, expert)
    assert np.abs(many - exact).max() < tol and np.abs(few - exact).max() < tol
    one = part.forward(dev(h[5:6], t), _ctx()).cpu().numpy()  # a row alone gives what it gave in the batch
    assert np.abs(one - few[5:6]).max() < 1e-6 * max(1.0, np.abs(exact).max())


# ---- whole models ------------------------------------------------------------------------------------
CASES = {"A": (fc.CASE_A, fc.REL_ROWS_A), "B": (fc.CASE_B, fc.REL_ROWS_B), "C": (fc.CASE_C, fc.REL_ROWS_C),
         "D": (fc.CASE_D, fc.REL_ROWS_D)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, rows) in CASES.items():
        w = fc.draw_weights(cfg, rows, seed=21)
        out[name] = (fc.write_folder(str(tmp_path_factory.mktemp("fesorax") / name), cfg, w), w)
    return out


def _check(got, cfg, w, reqs, plain, dtype, what):
    """float32: every position within 1e-4 of the plain logits (relative to the largest).  bfloat16: the
    bound of a request is three times what rounding the stored activations does to the plain statement
    (at the request's 80th percentile of positions: where rounding flips a router's close call, there
    and in the positions after it, the two differ by whole experts, in the engine at other places than in
    the rounded plain statement); at most a fifth of a request's positions may lie beyond it."""
    if dtype == "float32":
        return compare(got, plain, lambda ref: TOL_F32 * max(1.0, float(np.abs(ref).max())), what)
    for r, per_pos in got.items():
        rounded = _rounded(cfg, w, r, reqs[r])
        gap = np.abs(plain[r] - rounded).max(axis=1)
        bound = BF16_GAP_FACTOR * float(np.percentile(gap, 80))
        assert bound < 0.1 * float(np.abs(plain[r]).max()), "the test model is too rough for bfloat16"
        err = np.array([np.abs(row.astype(np.float64) - plain[r][p]).max() for p, row in sorted(per_pos.items())])
        assert np.isfinite(err).all(), f"{what}: request {r}"
        beyond = int((err > bound).sum())
        assert beyond <= max(1, len(err) // 5), (f"{what}: request {r}: {beyond} of {len(err)} positions beyond {bound:.3e}; "
                                                 f"first at {sorted(per_pos)[int(np.argmax(err > bound))]}")


_ROUNDED = {}


def _rounded(cfg, w, name, tokens):
    key = (cfg["vocab"], name, tuple(tokens))
    if key not in _ROUNDED:
        _ROUNDED[key] = pf.forward(cfg, w, tokens, round_fn=plain_llama.to_bf16)
    return _ROUNDED[key]


def _poison(cache):
    """Pages and state rows that nobody holds may contain anything."""
    for g in cache.groups:
        g.k.fill_(float("nan"))
        g.v.fill_(float("inf"))


@pytest.mark.parametrize("case", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_step_like_the_plain_statement_however_the_tokens_are_cut(folders, cuda_device, case, dtype):
    cfg = CASES[case][0]
    d, w = folders[case]
    V = cfg["vocab"]
    reqs = {"a": random_tokens(1, 210, V), "b": random_tokens(2, 3, V), "c": random_tokens(3, 77, V), "d": random_tokens(4, 131, V)}
    plain = {r: pf.forward(cfg, w, t) for r, t in reqs.items()}
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


@pytest.mark.parametrize("case", ["A", "B"])
def test_a_request_alone_and_in_a_batch_give_the_same_logits(folders, cuda_device, case):
    """Beyond rounding nothing of the batch around a request reaches it: in float32 the same numbers to 1e-5."""
    cfg = CASES[case][0]
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point_and_the_replay_program(folders, cuda_device, tmp_path, dtype):
    cfg = CASES["A"][0]
    d, w = folders["A"]
    V = cfg["vocab"]
    model = bn.load_model(d, dtype=dtype)
    prompts = [random_tokens(31, 50, V), random_tokens(32, 3, V), random_tokens(33, 120, V)]
    got = bn.generate(model, prompts, max_new_tokens=[70, 20, 24])
    for p, g in zip(prompts, got):
        assert len(g.tokens) in (70, 20, 24) and g.finish_reason == "length"
        seq = list(p) + g.tokens[:-1]
        ref = pf.forward(cfg, w, seq)[len(p) - 1:]
        if dtype == "float32":
            slack, allowed = 2 * TOL_F32 * max(1.0, float(np.abs(ref).max())), 0
        else:  # as in ``_check``: a close call of a router may go the other way
            gap = np.abs(pf.forward(cfg, w, seq, round_fn=plain_llama.to_bf16)[len(p) - 1:] - ref).max(axis=1)
            slack, allowed = 2 * BF16_GAP_FACTOR * float(np.percentile(gap, 80)), len(g.tokens) // 5
        off = [i for i, t in enumerate(g.tokens) if ref[i, t] < ref[i].max() - slack]
        assert len(off) <= allowed, f"tokens {off[:5]} of a prompt of {len(p)} are not the plain statement's"
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
    plain = {k: pf.forward(cfg, w, t) for k, t in reqs.items()}
    compare(collect_trace_output(steps, out, V), plain, lambda ref: TOL_F32 * max(1.0, float(np.abs(ref).max())),
            "through bin/trace_run")


def test_the_command_line_writes_a_random_model_of_the_design_and_generates_from_it(tmp_path, cuda_device):
    import json
    cfgp = tmp_path / "cfg.json"
    cfgp.write_text(json.dumps(fc.CASE_C))
    folder = tmp_path / "m"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "bitnet"), str(folder), "--random-weights", "--config", str(cfgp),
           "--weight-seed", "3", "--dtype", "float32", "--prompt-token-ids", "5,17,3,9,9,1", "--prompt-token-ids", "7",
           "-n", "9", "--repeat-penalty", "1.0", "--token-ids"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [[int(t) for t in l.split(",")] for l in p.stdout.splitlines() if l.strip()]
    assert [len(l) for l in lines] == [9, 9] and "Generation complete tokens=18" in p.stderr
    # the folder it wrote: the design's tensor names (the bias tables with the default number of rows), and the
    # tokens are the plain statement's greedy choice
    cfg, w = plain_llama.read_model(str(folder))
    assert w["l0.mix.rel"].shape == (64, 4) and "l1.mix.k" not in w and "l2.mlp.e2.down" in w
    for prompt, toks in zip(([5, 17, 3, 9, 9, 1], [7]), lines):
        ref = pf.forward(cfg, w, prompt + toks[:-1])[len(prompt) - 1:]
        for i, t in enumerate(toks):
            assert ref[i, t] >= ref[i].max() - 2 * TOL_F32 * max(1.0, float(np.abs(ref).max())), (prompt, i)
    # token by token through the same step function gives the same tokens
    p2 = subprocess.run([c for c in cmd if c != "--random-weights"] + ["--no-prefill", "--quiet"], capture_output=True,
                        text=True, timeout=600)
    assert p2.returncode == 0, p2.stderr[-2000:]
    assert [l for l in p2.stderr.splitlines() if l.startswith("token_id=")] == \
           [l for l in p.stderr.splitlines() if l.startswith("token_id=")]
