"""Kodupel on the GPU against the plain numpy restatement in tests/kodupel_oracle.py.

Small configurations of their own (sizes that differ from one another; attention layers with grouped and single
key/value heads, rotated parts smaller than and equal to the head, with and without frequency scaling, shared caches;
delta-rule layers whose head size does and does not have a register kernel; layers without feed-forward; one expert,
every expert chosen), random bfloat16-exact weights.  float32 runs are held to a tight tolerance, bfloat16 runs to a
loose one; the measure is the RMS over the vocabulary of the mean-free difference of the logits, relative to the RMS
of the logits.
"""
import json
import math

import numpy as np
import pytest

from tests import kodupel_oracle as orc

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-4, "bfloat16": 4e-2}


def A(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0, scaling=None, kv_from=None, moe=None):
    mx = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=dict(base=base, dims=rot_dims))
    if scaling:
        mx["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "attention", "mixer": mx, "mlp": moe}


def R(heads, dim, rank, moe=None):
    return {"type": "general_delta", "mixer": dict(heads=heads, dim=dim, decay_rank=rank), "mlp": moe}


def E(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


YARN_A, YARN_C = (4.0, 64, 16.0, 2.0), (3.0, 40, 8.0, 0.5)
CFG_MIXED = {"architecture": "Kodupel", "vocab": 67, "width": 48, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5},
             "layers": [A(4, 2, 12, 8, 0.3, 8, scaling=YARN_A, moe=E(5, 2, 20, 1.5)), R(3, 16, 5),
                        A(4, 2, 12, 8, 0.3, 8, scaling=YARN_A, kv_from=0, moe=E(3, 1, 24, 0.7)), R(2, 24, 7, moe=E(4, 4, 12, 2.0))]}
CFG_ONES = {"architecture": "Kodupel", "vocab": 40, "width": 32, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": [R(1, 32, 3, moe=E(1, 1, 16, 1.0)), A(1, 1, 32, 16, 0.17, 32, base=500.0)]}
CFG_WIDE = {"architecture": "Kodupel", "vocab": 96, "width": 64, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-5},
            "layers": [A(8, 2, 16, 32, 0.25, 4, base=2e5, scaling=YARN_C, moe=E(8, 3, 40, 1.0)), R(2, 64, 8, moe=E(8, 3, 40, 1.0)),
                       A(8, 2, 16, 32, 0.25, 4, base=2e5, scaling=YARN_C, kv_from=0)]}
CONFIGS = {"mixed": CFG_MIXED, "ones": CFG_ONES, "wide": CFG_WIDE}


def row_err(got, want):
    d = np.asarray(got, dtype=np.float64) - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean(-1))


def rel_err(got, want, dtype="float32"):
    """float32: the worst row.  bfloat16: the row at the 90th percentile -- a rounding can flip the choice of an expert
    where two choice scores nearly tie, which moves that token by far more than rounding does and says nothing about
    the kernels; what a float32 run finds at one position only, it finds with the worst-row measure."""
    e = row_err(got, want)
    return float(np.max(e) if dtype == "float32" else np.quantile(e, 0.9))


def make(cfg_dict, dtype, seed=0, max_batch=4, max_seq=400, max_step_tokens=64, **kw):
    from zhilight_b200.kodupel import KodupelConfig, KodupelDecoder
    from zhilight_b200.safetensors_io import f32_to_bf16
    cfg = KodupelConfig.from_dict(cfg_dict)
    W = orc.random_weights(cfg, seed)
    m = KodupelDecoder(cfg, dtype=dtype, max_batch=max_batch, max_seq=max_seq, max_step_tokens=max_step_tokens, **kw)
    m.load_state_dict({k: f32_to_bf16(v) for k, v in W.items()})
    return cfg, {k: v.astype(np.float64) for k, v in W.items()}, m


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg.vocab, n).tolist()


def dev(a, cuda, dtype=None):
    import torch
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(cuda)


def i32(a, cuda):
    import torch
    return torch.tensor(list(a), dtype=torch.int32, device=cuda)


# ---------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gemm_bias_tanh_and_grouped(cuda, lib, dtype):
    import torch
    from zhilight_b200 import ops
    td = getattr(torch, dtype)
    tol = 1e-5 if dtype == "float32" else 1e-2
    rng = np.random.default_rng(0)
    for m, n, k in ((5, 7, 13), (70, 130, 80), (3, 96, 64), (40, 10, 24)):
        x, w, b = (orc.bf16_round(rng.standard_normal(s).astype(np.float32)) for s in ((m, k), (n, k), (n,)))
        ref = x.astype(np.float64) @ w.T.astype(np.float64) + b
        for epi, fn in ((0, lambda r: r), (3, np.tanh)):
            y = ops.gemm_nt_bias(dev(x, cuda, td), dev(w, cuda, td), dev(b, cuda), out_dtype=torch.float32, epilogue=epi)
            assert np.abs(y.cpu().numpy() - fn(ref)).max() < tol * max(1.0, np.abs(ref).max()), (m, n, k, epi)
    # grouped: 5 groups of unequal size (one empty, one larger than a tile), gathered inputs, scattered outputs; then a
    # step of few rows (the kernel that keeps a group's rows in shared memory, one group with more than eight rows)
    for T, sizes in ((47, [0, 70, 3, 1, 67]), (6, [11, 0, 2, 4, 1])):
        _grouped_case(cuda, td, tol, rng, T, sizes)


def _grouped_case(cuda, td, tol, rng, T, sizes):
    import torch
    from zhilight_b200 import ops
    G, K, F, top = 5, 40, 24, 3
    assert sum(sizes) == T * top
    pairs = rng.permutation(T * top)
    off = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
    x = orc.bf16_round(rng.standard_normal((T, K)).astype(np.float32))
    wgu = orc.bf16_round((rng.standard_normal((G, 2 * F, K)) / math.sqrt(K)).astype(np.float32))
    wd = orc.bf16_round((rng.standard_normal((G, K, F)) / math.sqrt(F)).astype(np.float32))
    limit = 0.8
    act = ops.gemm_nt_grouped(dev(x, cuda, td), dev(wgu, cuda, td), dev(off, cuda), T * top, x_rows=i32(pairs // top, cuda),
                              epilogue=ops.GEMM_EPI_GLU_CLAMP, limit=limit, alpha=1.702, beta=1.0)
    out = ops.gemm_nt_grouped(act, dev(wd, cuda, td), dev(off, cuda), T * top, y_rows=i32(pairs, cuda), out_dtype=torch.float32)
    act, out = act.float().cpu().numpy(), out.cpu().numpy()
    for g in range(G):
        for i in range(off[g], off[g + 1]):
            xv = x[pairs[i] // top].astype(np.float64)
            gate, up = wgu[g, 0::2] @ xv, wgu[g, 1::2] @ xv
            gg = np.minimum(gate, limit)
            want = gg * orc.sigmoid(1.702 * gg) * (np.clip(up, -limit, limit) + 1.0)
            assert np.abs(act[i] - want).max() < tol * 4, (g, i)
            assert np.abs(out[pairs[i]] - wd[g].astype(np.float64) @ act[i].astype(np.float64)).max() < tol * 4, (g, i)


def test_rotation_frequencies(lib):
    from zhilight_b200 import ops
    for base, dims, sc in ((10000.0, 8, YARN_A), (2e5, 4, YARN_C), (500.0, 32, None), (1e4, 64, (8.0, 4096, 24.0, 2.0))):
        f, ms = ops.rope_inv_freq_yarn(base, dims, *(sc or ()))
        scd = dict(zip(("factor", "original", "fast", "slow"), sc)) if sc else None
        cos, sin = orc.rotation_tables(2, dims, base, scd)
        mag = math.hypot(cos[1, 0], sin[1, 0])
        assert abs(ms - mag) < 1e-6
        assert np.allclose(np.arctan2(sin[1], cos[1]), f, rtol=1e-12, atol=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_norms_rotation_and_cache_append(cuda, lib, dtype):
    import torch
    from zhilight_b200 import ops
    td = getattr(torch, dtype)
    H, G, d, vd, rot, eps = 3, 1, 20, 12, 6, 1e-5
    rng = np.random.default_rng(1)
    slots, pos = [2, 2, 2, 0, 1], [898, 899, 900, 0, 37]        # far positions: the angle is position * frequency in fp32
    T = len(pos)
    n_in = H * d + G * d + G * vd + 5
    proj = rng.standard_normal((T, n_in)).astype(np.float32)
    qw, kw = (1 + 0.2 * rng.standard_normal(d)).astype(np.float32), (1 + 0.2 * rng.standard_normal(d)).astype(np.float32)
    f, ms = ops.rope_inv_freq_yarn(10000.0, rot, *YARN_A)
    kc = torch.zeros((3, 1000, G * d), dtype=td, device=cuda)
    vc = torch.zeros((3, 1000, G * vd), dtype=td, device=cuda)
    q = ops.qkv_headnorm_rope_append(dev(proj, cuda), 0, H * d, H * d + G * d, H, G, d, vd, dev(qw, cuda), dev(kw, cuda),
                                     dev(f, cuda), rot, ms, eps, kc, vc, ops.slot_table(kc), ops.slot_table(vc), i32(slots, cuda),
                                     i32(pos, cuda), td)
    cos, sin = orc.rotation_tables(1000, rot, 10000.0, dict(zip(("factor", "original", "fast", "slow"), YARN_A)))
    p64 = proj.astype(np.float64)
    tol = 2e-4 if dtype == "float32" else 2e-2
    for t in range(T):
        c, s = cos[pos[t]:pos[t] + 1], sin[pos[t]:pos[t] + 1]
        wq = orc.rotate_pairs((orc.unit_rms(p64[t, :H * d].reshape(1, H, d), eps) * qw), c, s, rot).reshape(-1)
        wk = orc.rotate_pairs((orc.unit_rms(p64[t, H * d:H * d + G * d].reshape(1, G, d), eps) * kw), c, s, rot).reshape(-1)
        wv = orc.unit_rms(p64[t, H * d + G * d:H * d + G * d + G * vd].reshape(G, vd), eps).reshape(-1)
        assert np.abs(q[t].float().cpu().numpy() - wq).max() < tol
        assert np.abs(kc[slots[t], pos[t]].float().cpu().numpy() - wk).max() < tol
        assert np.abs(vc[slots[t], pos[t]].float().cpu().numpy() - wv).max() < tol
    assert float(kc[1, 36].abs().sum()) == 0 and float(kc[1, 38].abs().sum()) == 0       # no other row was touched


@pytest.mark.parametrize("H", [6, 8])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_attention_far_key_sink_and_groups(cuda, lib, dtype, H):
    """700 keys.  One far key is made to carry the softmax of one head (query and that key scaled up), another head's
    scores are pushed far below zero so that the unit sink takes the whole denominator; rows past a token's position
    hold huge values that must not be seen; key splits 1 / 2 / 5 / 23.  Each query row alone and as runs of consecutive rows
    (the tensor-core kernel tiles the tokens of a run; 8 heads on 2 key/value heads fit its tile, 6 do not)."""
    import torch
    from zhilight_b200 import ops
    td = getattr(torch, dtype)
    G, d, vd, n, scale = 2, 16, 24, 700, 0.25
    rng = np.random.default_rng(2)
    q = orc.bf16_round(rng.standard_normal((n, H, d)).astype(np.float32))
    k = orc.bf16_round(rng.standard_normal((n, G, d)).astype(np.float32))
    v = orc.bf16_round(rng.standard_normal((n, G, vd)).astype(np.float32))
    k[13, 0] = orc.bf16_round(np.sign(q[650, 1]) * 2.0)       # head 1 (group 0) of token 650 looks at key 13
    q[650, 1] *= 4
    q[651, 4] = orc.bf16_round(-8.0 * np.sign(k[:652, 1].sum(0)))
    want = orc.unit_sink_attention(q.astype(np.float64), k.astype(np.float64), v.astype(np.float64), scale)
    e = np.exp((k[:651, 0].astype(np.float64) @ q[650, 1]) * scale)
    assert e[13] / (1 + e.sum()) > 0.9                               # the far key does carry that head
    gate = rng.standard_normal((n, H + 3)).astype(np.float32)
    want = want * orc.sigmoid(gate[:, :H].astype(np.float64))[:, :, None]
    rows = [0, 1, 7, 8, 9, 255, 256, 257, 511, 512, 650, 651, 699]
    kc = torch.full((2, n + 5, G * d), 3e4, dtype=td, device=cuda)
    vc = torch.full((2, n + 5, G * vd), 3e4, dtype=td, device=cuda)
    kc[1, :n] = dev(k.reshape(n, -1), cuda, td)
    vc[1, :n] = dev(v.reshape(n, -1), cuda, td)
    tol = 1e-5 if dtype == "float32" else 1e-2
    for splits in (1, 2, 5, 23):
        # every query row alone: its keys end at its own position, the rows behind it are poison
        out = ops.sink_attention(dev(q[rows].reshape(len(rows), -1), cuda, td), ops.slot_table(kc), ops.slot_table(vc),
                                 i32([1] * len(rows), cuda), i32(rows, cuda), scale, H, G, d, vd, gate=dev(gate[rows], cuda),
                                 splits=splits)
        got = out.float().cpu().numpy().reshape(len(rows), H, vd)
        assert np.abs(got - want[rows]).max() < tol, (dtype, splits)
        # the same rows as runs of one row each, then rows 0..9 and 560..699 as two runs
        ones = dict(run_row0=i32(range(len(rows)), cuda), run_len=i32([1] * len(rows), cuda), max_run_len=1)
        out = ops.sink_attention(dev(q[rows].reshape(len(rows), -1), cuda, td), ops.slot_table(kc), ops.slot_table(vc),
                                 i32([1] * len(rows), cuda), i32(rows, cuda), scale, H, G, d, vd, gate=dev(gate[rows], cuda),
                                 splits=splits, **ones)
        assert np.abs(out.float().cpu().numpy().reshape(len(rows), H, vd) - want[rows]).max() < tol, (dtype, splits, "runs of 1")
        seq = list(range(10)) + list(range(560, 700))
        out = ops.sink_attention(dev(q[seq].reshape(len(seq), -1), cuda, td), ops.slot_table(kc), ops.slot_table(vc),
                                 i32([1] * len(seq), cuda), i32(seq, cuda), scale, H, G, d, vd, gate=dev(gate[seq], cuda),
                                 splits=splits, run_row0=i32([0, 10], cuda), run_len=i32([10, 140], cuda), max_run_len=140)
        assert np.abs(out.float().cpu().numpy().reshape(len(seq), H, vd) - want[seq]).max() < tol, (dtype, splits, "two runs")


@pytest.mark.parametrize("dk", [32, 24, 64])
def test_delta_rule_runs_portions_and_slot_reuse(cuda, lib, dk):
    """Two sequences in one step (runs of 19 and 1 rows), then portions of 2, 1 and 9 rows carrying the state, against
    one scan over each whole sequence; then a slot handed to a new sequence that starts at position 0 over the old state."""
    import torch
    from zhilight_b200 import ops
    H, n = 3, 31
    rng = np.random.default_rng(dk)
    seqs = {}
    for name in ("a", "b", "c"):
        r, k, v = (rng.standard_normal((n, H, dk)) for _ in range(3))
        al, wl = rng.standard_normal((n, H, dk)), rng.standard_normal((n, H, dk))
        k[5] *= 1e-4                                           # a key so short that the 1e-6 under the root matters
        seqs[name] = tuple(x.astype(np.float32) for x in (r, k, v, al, wl))
    want = {}
    for name, (r, k, v, al, wl) in seqs.items():
        want[name] = orc.delta_rule_scan(r.astype(np.float64), k.astype(np.float64), v.astype(np.float64),
                                         np.exp(-math.exp(-0.5) * orc.sigmoid(wl.astype(np.float64))), orc.sigmoid(al.astype(np.float64)))
    state = torch.full((3, H, dk, dk), 7.0, dtype=torch.float32, device=cuda)       # stale contents everywhere
    tab = ops.slot_table(state)
    got = {name: [] for name in seqs}
    at = {name: 0 for name in seqs}

    def step(plan, slot_of):
        rows, slots, pos, run0, runlen = [], [], [], [], []
        for name, cnt in plan:
            run0.append(len(slots)); runlen.append(cnt)
            for j in range(cnt):
                rows.append((name, at[name] + j)); slots.append(slot_of[name]); pos.append(at[name] + j)
        pick = lambda idx: dev(np.stack([seqs[nm][idx][p].reshape(-1) for nm, p in rows]), cuda)
        o = ops.delta_rule(pick(0), pick(1), pick(2), pick(3), pick(4), math.exp(-0.5), 1e-6, i32(run0, cuda), i32(runlen, cuda),
                           i32(slots, cuda), i32(pos, cuda), state, tab, H, dk, dk).cpu().numpy()
        i = 0
        for name, cnt in plan:
            got[name].append(o[i:i + cnt]); at[name] += cnt; i += cnt

    slot_of = {"a": 2, "b": 0}
    for plan in ([("a", 19), ("b", 1)], [("b", 2), ("a", 1)], [("a", 9), ("b", 9)], [("b", 19), ("a", 2)]):
        step(plan, slot_of)
    for name in ("a", "b"):
        o, S = want[name]
        assert np.abs(np.concatenate(got[name]).reshape(n, H, dk) - o).max() < 2e-4 * max(1.0, np.abs(o).max()), name
        assert np.abs(state[slot_of[name]].cpu().numpy() - S).max() < 2e-4 * max(1.0, np.abs(S).max()), name
    step([("c", 31)], {"c": 2})                                # slot 2 again, from position 0
    assert np.abs(got["c"][0].reshape(n, H, dk) - want["c"][0]).max() < 2e-4 * max(1.0, np.abs(want["c"][0]).max())


def test_router_choice_and_weights(cuda, lib):
    """The correction decides who is chosen but is not part of the weight; the lists sort the pairs by expert."""
    from zhilight_b200 import ops
    rng = np.random.default_rng(3)
    T, D, E, top = 37, 24, 11, 3
    x = rng.standard_normal((T, D)).astype(np.float32)
    w = (4 * rng.standard_normal((E, D)) / math.sqrt(D)).astype(np.float32)
    corr = rng.standard_normal(E).astype(np.float32)
    corr[4] = 5.0                                                # expert 4 is always chosen, whatever its score
    te, tw, off, lt, lp = (t.cpu().numpy() for t in ops.moe_route(dev(x, cuda), dev(w, cuda), dev(corr, cuda), top))
    chosen, weight = orc.route(x.astype(np.float64), w.astype(np.float64), corr.astype(np.float64), top)
    assert (te == chosen).all() and (te[:, 0] == 4).all()
    assert np.abs(tw - weight).max() < 1e-5 and tw.max() <= 1.0
    assert off[0] == 0 and off[-1] == T * top and (np.diff(off) >= 0).all()
    assert sorted(lp.tolist()) == list(range(T * top)) and (lt == lp // top).all()
    for e in range(E):
        assert (te.reshape(-1)[lp[off[e]:off[e + 1]]] == e).all()


def test_head_norm_gate_and_combine(cuda, lib):
    import torch
    from zhilight_b200 import ops
    rng = np.random.default_rng(4)
    T, H, dv, D, parts, eps = 9, 5, 12, 40, 3, 1e-5
    o = rng.standard_normal((T, H * dv)).astype(np.float32)
    w, g = rng.standard_normal(H * dv).astype(np.float32), rng.standard_normal((T, H * dv)).astype(np.float32)
    got = ops.head_rmsnorm_gate(dev(o, cuda), H, dv, eps, dev(w, cuda), dev(g, cuda)).cpu().numpy()
    want = orc.unit_rms(o.astype(np.float64).reshape(T, H, dv), eps).reshape(T, -1) * w * orc.sigmoid(g.astype(np.float64))
    assert np.abs(got - want).max() < 1e-5
    p = rng.standard_normal((T, parts, D)).astype(np.float32)
    c = rng.random((T, parts)).astype(np.float32)
    nw, x = rng.standard_normal(D).astype(np.float32), rng.standard_normal((T, D)).astype(np.float32)
    xd = dev(x, cuda)
    xa = ops.rmsnorm_residual_combine(dev(p, cuda), dev(c, cuda), dev(nw, cuda), xd, eps, act_dtype=torch.bfloat16)
    s = (p.astype(np.float64) * c[:, :, None]).sum(1)
    want = x + orc.unit_rms(s, eps) * nw
    assert np.abs(xd.cpu().numpy() - want).max() < 1e-5
    assert np.abs(xa.float().cpu().numpy() - want).max() < 2e-2


# ---------------------------------------------------------------------------------------------- the whole model
@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_layers_states_and_logits(cuda, lib, name, dtype):
    cfg, W, m = make(CONFIGS[name], dtype, seed=1, max_step_tokens=128)
    toks = tokens_for(cfg, 97, 5)
    want, streams, states = orc.forward(cfg, W, toks)
    m.capture_layers(True)
    _, logits = m.step(toks, [2] * len(toks), range(len(toks)), range(len(toks)))
    got_streams = m.read_layers(len(toks))
    for i in range(len(cfg.layers)):   # the first layer that differs is the one to look at
        rows = np.abs(got_streams[i] - streams[i]).max(-1) / np.abs(streams[i]).max()
        d = rows.max() if dtype == "float32" else np.quantile(rows, 0.9)
        assert d < (1e-4 if dtype == "float32" else 6e-2), (name, dtype, "layer", i, d)
    for i, S in states.items():
        d = np.abs(m.read_state(i, 2) - S).max() / np.abs(S).max()
        if dtype == "float32":      # in bfloat16 a flipped expert choice upstream moves the state of every later token
            assert d < 1e-4, (name, dtype, "state", i, d)
        else:
            assert np.isfinite(d) and d < 0.5, (name, dtype, "state", i, d)
    assert rel_err(logits, want, dtype) < TOL[dtype]
    m.close()


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_vs_token_by_token_and_portions(cuda, lib, name, dtype):
    """The same prompt whole, token by token, and in portions down to two tokens: every position against the oracle and
    the three runs against one another."""
    from zhilight_b200.engine import Engine
    cfg, W, m = make(CONFIGS[name], dtype, seed=2, max_step_tokens=32)
    eng = Engine(m)
    toks = tokens_for(cfg, 75, 9)
    want = orc.forward(cfg, W, toks)[0]
    runs = {}
    for label, sizes in (("whole", [75]), ("single", [1] * 75), ("portions", [2, 3, 2, 17, 1, 2, 31, 5, 2, 10])):
        assert sum(sizes) == 75
        eng.open(label)
        rows, at = [], 0
        for s in sizes:
            rows.append(eng.forward_step([(label, toks[at:at + s], list(range(s)))])[label][1])
            at += s
        eng.close(label)
        runs[label] = np.concatenate(rows)
        assert rel_err(runs[label], want, dtype) < TOL[dtype], (name, dtype, label)
    cut = 1e-5 if dtype == "float32" else 2e-2      # the cuts change the order of sums, no more
    assert rel_err(runs["single"], runs["whole"].astype(np.float64), dtype) < cut
    assert rel_err(runs["portions"], runs["whole"].astype(np.float64), dtype) < cut
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone_and_slot_reuse(cuda, lib, dtype):
    """Three requests of different lengths share steps (prompt portions next to single decode tokens); afterwards their
    slots -- caches and recurrent states still in them -- are handed to new requests.  Every logit row equals the
    request run alone."""
    from zhilight_b200.engine import Engine
    cfg, W, m = make(CFG_MIXED, dtype, seed=3, max_batch=3, max_step_tokens=16)
    eng = Engine(m)
    prompts = {"a": tokens_for(cfg, 41, 1), "b": tokens_for(cfg, 9, 2), "c": tokens_for(cfg, 26, 3)}
    later = {"d": tokens_for(cfg, 30, 4), "e": tokens_for(cfg, 5, 5)}
    want = {k: orc.forward(cfg, W, v)[0] for k, v in {**prompts, **later}.items()}
    got = {k: [] for k in want}
    at = {k: 0 for k in want}
    for k in prompts:
        eng.open(k)
    plan = [{"a": 7, "b": 2, "c": 1}, {"a": 1, "b": 1, "c": 12}, {"a": 20, "b": 1, "c": 1}, {"a": 1, "b": 5, "c": 2},
            {"a": 12, "c": 10}]
    for step in plan:
        entries = [(k, prompts[k][at[k]:at[k] + n], list(range(n))) for k, n in step.items()]
        res = eng.forward_step(entries)
        for k, n in step.items():
            got[k].append(res[k][1])
            at[k] += n
    assert at == {"a": 41, "b": 9, "c": 26, "d": 0, "e": 0}
    used = {eng.seqs[k].slot for k in prompts}
    for k in prompts:
        eng.close(k)
    for k in later:
        assert eng.open(k).slot in used
    res = eng.forward_step([("d", later["d"][:11], list(range(11))), ("e", later["e"], list(range(5)))])
    got["d"].append(res["d"][1]); got["e"].append(res["e"][1])
    got["d"].append(eng.forward_step([("d", later["d"][11:], list(range(19)))])["d"][1])
    for k in want:
        assert rel_err(np.concatenate(got[k]), want[k], dtype) < TOL[dtype], (dtype, k)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graphs_and_splits(cuda, lib, dtype):
    """A short prompt and then 330 single-token steps: the decode graph, the length buckets (256, 512) and the key splits
    of the attention kernel all change on the way; the recurrent state is carried through 340 updates."""
    cfg, W, m = make(CFG_WIDE, dtype, seed=4, max_batch=2, max_seq=512, max_step_tokens=16)
    toks = tokens_for(cfg, 340, 11)
    want = orc.forward(cfg, W, toks)[0]
    _, first = m.step(toks[:10], [1] * 10, range(10), range(10))
    rows = [first]
    for p in range(10, 340):
        rows.append(m.step([toks[p]], [1], [p], [0])[1])
    assert rel_err(np.concatenate(rows), want, dtype) < TOL[dtype]
    assert m.stats()[1] > 0          # the single-token steps were replayed as graphs
    m.close()


def test_far_token_is_found_through_the_model(cuda, lib):
    """Token 7 of 300 moves the last logits by far more than the float32 tolerance (the oracle says so first), so a key
    lost far back -- through prompt portions or through decoding -- fails the comparison."""
    cfg, W, m = make(CFG_WIDE, "float32", seed=5, max_batch=2, max_seq=320, max_step_tokens=64)
    toks = tokens_for(cfg, 300, 13)
    base = orc.forward(cfg, W, toks)[0][-1]
    other = list(toks)
    other[7] = (toks[7] + 1) % cfg.vocab
    moved = orc.forward(cfg, W, other)[0][-1]
    assert rel_err(moved[None], base[None]) > 10 * TOL["float32"]   # the oracle says token 7 matters at the end
    for seq, want in ((toks, base), (other, moved)):
        for c0 in range(0, 256, 64):
            m.step(seq[c0:c0 + 64], [0] * 64, range(c0, c0 + 64))
        for p in range(256, 299):
            m.step([seq[p]], [0], [p])
        got = m.step([seq[299]], [0], [299], [0])[1]
        assert rel_err(got, want[None]) < TOL["float32"]
    m.close()


def test_greedy_generation_through_the_scheduler(cuda, lib):
    """Engine.generate (admission, portions, mixed steps, retiring, slot reuse: 5 prompts on 2 slots) against greedy
    decoding with the oracle; float32 so that near-ties do not flip."""
    from zhilight_b200.engine import Engine
    cfg, W, m = make(CFG_MIXED, "float32", seed=6, max_batch=2, max_seq=128, max_step_tokens=8)
    prompts = [tokens_for(cfg, n, 20 + n) for n in (3, 19, 1, 11, 6)]
    seen = []
    outs = Engine(m).generate(prompts, max_new_tokens=7, on_step=lambda e: seen.append([len(t) for _, t, _ in e]))
    assert any(len(s) > 1 and max(s) > 1 and min(s) == 1 for s in seen)    # a prompt portion beside a decode token
    for p, out in zip(prompts, outs):
        seq = list(p)
        for tok in out:
            logits = orc.forward(cfg, W, seq)[0][-1]
            top = np.sort(logits)[-2:]
            assert tok == int(np.argmax(logits)) or top[1] - top[0] < 1e-4
            seq.append(tok)
        assert len(out) == 7
    m.close()


def test_model_folder_registry_and_trace_replay(cuda, lib, tmp_path):
    """config.json + model.safetensors on disk -> registry -> trace replay: the written logits are the oracle's.  The
    config on disk does not give the decay path's inner size: it comes from the checkpoint."""
    from zhilight_b200 import registry, safetensors_io, trace
    from zhilight_b200.kodupel import KodupelConfig
    cfg = KodupelConfig.from_dict(CFG_ONES)
    W = orc.random_weights(cfg, 8)
    on_disk = json.loads(json.dumps(CFG_ONES))
    for l in on_disk["layers"]:
        l["mixer"].pop("decay_rank", None)
    (tmp_path / "m").mkdir()
    (tmp_path / "m" / "config.json").write_text(json.dumps(on_disk))
    safetensors_io.save_file({k: safetensors_io.f32_to_bf16(v) for k, v in W.items()}, str(tmp_path / "m" / "model.safetensors"))
    model = registry.load_model(str(tmp_path / "m"), "float32", max_batch=2, max_seq=64, max_step_tokens=8)
    toks = tokens_for(cfg, 21, 3)
    lines = [json.dumps({"step": 0, "entries": [{"id": "x", "tokens": toks[:13], "want": [12, 0, 5]}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "x", "tokens": toks[13:20], "want": []}], "end": []}),
             json.dumps({"step": 2, "entries": [{"id": "x", "tokens": toks[20:], "want": [0]}], "end": ["x"]})]
    said = []
    trace.replay(model, lines, str(tmp_path), emit=said.append)
    assert said == ["done 0", "done 1", "done 2"] and not (tmp_path / "1.f32").exists()
    want = orc.forward(cfg, {k: v.astype(np.float64) for k, v in W.items()}, toks)[0]
    got0 = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(3, cfg.vocab)
    got2 = np.fromfile(tmp_path / "2.f32", dtype="<f4").reshape(1, cfg.vocab)
    assert rel_err(got0, want[[12, 0, 5]]) < TOL["float32"] and rel_err(got2, want[[20]]) < TOL["float32"]
    model.close()
