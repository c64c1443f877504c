"""Dekipel on the GPU against the plain numpy restatement in tests/dekipel_oracle.py.

Small configurations of their own (sizes that are all different from one another, layers of different shapes, a layer
without feed-forward, shared latent caches, taps and groups of 1 and of more), random bfloat16-exact weights.  float32
runs are held to a tight tolerance, bfloat16 runs to a loose one; the measure is the RMS over the vocabulary of the
mean-free difference of the logits, relative to the RMS of the logits.
"""
import json

import numpy as np
import pytest

from tests import dekipel_oracle as orc

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-4, "bfloat16": 4e-2}


def L(heads, dim, vdim, q_rank, kv_rank, scale, ff, kv_from=None):
    mx = dict(heads=heads, dim=dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale)
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mx, "mlp": {"kind": "dense", "ff": ff} if ff else None}


CFG_MIXED = {"architecture": "Dekipel", "vocab": 61, "width": 48, "norm": {"eps": 1e-5, "groups": 3}, "canon": {"taps": 4},
             "layers": [L(3, 8, 12, 20, 24, 0.3, 40), L(2, 16, 8, 12, 24, 0.2, 0, kv_from=0), L(5, 4, 20, 36, 40, 0.5, 72),
                        L(5, 8, 6, 10, 40, 0.25, 24, kv_from=2)]}
CFG_ONES = {"architecture": "Dekipel", "vocab": 33, "width": 32, "norm": {"eps": 1e-6, "groups": 1}, "canon": {"taps": 1},
            "layers": [L(1, 32, 32, 16, 16, 0.17, 64), L(1, 8, 4, 8, 16, 1.0, 0)]}
CFG_WIDE = {"architecture": "Dekipel", "vocab": 96, "width": 64, "norm": {"eps": 1e-5, "groups": 2}, "canon": {"taps": 2},
            "layers": [L(4, 16, 32, 32, 64, 0.25, 128), L(4, 16, 32, 32, 64, 0.25, 128, kv_from=0)]}
CONFIGS = {"mixed": CFG_MIXED, "ones": CFG_ONES, "wide": CFG_WIDE}


def rel_err(got, want):
    d = np.asarray(got, dtype=np.float64) - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float(np.max(np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean(-1))))


def make(cfg_dict, dtype, seed=0, max_batch=4, max_seq=400, max_step_tokens=64, **kw):
    from zhilight_b200.dekipel import DekipelConfig, DekipelDecoder
    from zhilight_b200.safetensors_io import f32_to_bf16
    cfg = DekipelConfig.from_dict(cfg_dict)
    W = orc.random_weights(cfg, seed)
    m = DekipelDecoder(cfg, dtype=dtype, max_batch=max_batch, max_seq=max_seq, max_step_tokens=max_step_tokens, **kw)
    m.load_state_dict({k: f32_to_bf16(v) for k, v in W.items()})
    return cfg, {k: v.astype(np.float64) for k, v in W.items()}, m


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg.vocab, n).tolist()


# ---------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("shape", [(5, 7, 13, 1), (70, 130, 80, 1), (33, 24, 8, 5), (64, 64, 32, 2), (1, 200, 96, 1), (8, 70, 64, 3),
                                   (32, 33, 128, 2), (17, 40, 24, 1), (3, 9, 512, 4)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gemm_nt_any_shape(cuda, lib, shape, dtype):
    import torch
    from zhilight_b200 import ops
    m, n, k, b = shape
    g = torch.Generator().manual_seed(m * 1000 + n)
    td = getattr(torch, dtype)
    x = torch.randn(b, m, k, generator=g).to(td)
    w = torch.randn(b, n, k, generator=g).to(td)
    gate = torch.randn(b, m, n, generator=g)
    ref = torch.einsum("bmk,bnk->bmn", x.double(), w.double())
    tol = 1e-5 if dtype == "float32" else 1e-2
    for epi, fn in ((0, lambda r: r), (1, lambda r: torch.relu(r) ** 2), (2, lambda r: r * torch.sigmoid(gate.double()))):
        y = ops.gemm_nt(x.to(cuda), w.to(cuda), out_dtype=torch.float32, epilogue=epi, gate=gate.to(cuda) if epi == 2 else None)
        want = fn(ref)
        assert float((y.cpu().double() - want).norm() / want.norm()) < tol, (shape, epi)
    if b == 1:   # unbatched call, output in the input type
        y = ops.gemm_nt(x[0].to(cuda), w[0].to(cuda))
        assert y.dtype == td and float((y.cpu().double() - ref[0]).norm() / ref[0].norm()) < 1e-2


@pytest.mark.parametrize("d,groups", [(96, 3), (64, 1), (40, 5), (2048, 2), (7, 7)])
def test_group_rmsnorm_and_residual(cuda, lib, d, groups):
    import torch
    from zhilight_b200 import ops
    rng = np.random.default_rng(d)
    x, y, w = rng.standard_normal((6, d)), rng.standard_normal((6, d)) * 3, rng.uniform(0.5, 1.5, d)
    tx, ty, tw = (torch.tensor(a, dtype=torch.float32, device=cuda) for a in (x, y, w))
    got = ops.group_rmsnorm(tx, tw, groups, 1e-5).cpu().numpy()
    assert np.allclose(got, orc.group_rms_norm(x, w, groups, 1e-5), rtol=2e-5, atol=2e-6)
    ops.group_rmsnorm_residual(ty, tw, tx, groups, 1e-5)
    assert np.allclose(tx.cpu().numpy(), x + orc.group_rms_norm(y, w, groups, 1e-5), rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
def test_causal_conv_with_slot_state(cuda, lib, taps):
    """Two sequences in slots that were used before; portions of 1, 2 and more rows, mixed in one step; every output must
    equal the convolution over the sequence's whole history."""
    import torch
    from zhilight_b200 import ops
    d, n = 24, 23
    rng = np.random.default_rng(taps)
    w = rng.uniform(-1, 1, (d, taps))
    tw = torch.tensor(w, dtype=torch.float32, device=cuda)
    ring = torch.full((3, max(taps - 1, 1), d), 77.0, dtype=torch.float32, device=cuda)   # leftovers of earlier owners
    hist = {1: rng.standard_normal((n, d)), 2: rng.standard_normal((n, d))}
    want = {s: orc.conv_mix(h, w) for s, h in hist.items()}
    at = {1: 0, 2: 0}
    plan = [[(1, 1)], [(2, 2), (1, 1)], [(1, 2)], [(2, 1), (1, 5)], [(1, 1), (2, 1)], [(2, 7)], [(1, 13), (2, 12)]]
    for step in plan:
        rows, slots, poss = [], [], []
        for s, cnt in step:
            rows.append(hist[s][at[s]:at[s] + cnt])
            slots += [s] * cnt
            poss += list(range(at[s], at[s] + cnt))
        h = torch.tensor(np.concatenate(rows), dtype=torch.float32, device=cuda)
        ts = torch.tensor(slots, dtype=torch.int32, device=cuda)
        tp = torch.tensor(poss, dtype=torch.int32, device=cuda)
        u = ops.causal_conv_mix(h, tw, ts, tp, ring if taps > 1 else None).cpu().numpy()
        i = 0
        for s, cnt in step:
            assert np.allclose(u[i:i + cnt], want[s][at[s]:at[s] + cnt], rtol=1e-5, atol=1e-5), (taps, step, s)
            i += cnt
            at[s] += cnt
        # the post-norm kernel is the one that stores the rows into the rings
        x = torch.zeros_like(h)
        ops.group_rmsnorm_residual(torch.ones_like(h), torch.ones(d, device=cuda), x, 1, 1e-5, conv_in=h, slot=ts, pos=tp,
                                   ring=ring if taps > 1 else None, taps=taps)
    assert at == {1: n, 2: n}


@pytest.mark.parametrize("taps,groups", [(1, 1), (2, 3), (3, 2), (4, 6)])
def test_fused_norm_conv_matches_norm_then_conv(cuda, lib, taps, groups):
    """The fused pre-norm + convolution kernel over the same plan of mixed portions, rings carried from step to step."""
    import torch
    from zhilight_b200 import ops
    d, n = 36, 19
    rng = np.random.default_rng(taps * 10 + groups)
    w, nw = rng.uniform(-1, 1, (d, taps)), rng.uniform(0.5, 1.5, d)
    tw, tnw = (torch.tensor(a, dtype=torch.float32, device=cuda) for a in (w, nw))
    ring = torch.full((3, max(taps - 1, 1), d), -55.0, dtype=torch.float32, device=cuda)
    hist = {0: rng.standard_normal((n, d)) * 2, 2: rng.standard_normal((n, d))}
    want = {s: orc.conv_mix(orc.group_rms_norm(x, nw, groups, 1e-5), w) for s, x in hist.items()}
    at = {0: 0, 2: 0}
    for step in [[(0, 2)], [(2, 1), (0, 1)], [(0, 1), (2, 2)], [(2, 3), (0, 7)], [(0, 8), (2, 13)]]:
        rows, slots, poss = [], [], []
        for s, cnt in step:
            rows.append(hist[s][at[s]:at[s] + cnt])
            slots += [s] * cnt
            poss += list(range(at[s], at[s] + cnt))
        x = torch.tensor(np.concatenate(rows), dtype=torch.float32, device=cuda)
        ts = torch.tensor(slots, dtype=torch.int32, device=cuda)
        tp = torch.tensor(poss, dtype=torch.int32, device=cuda)
        h, u = ops.group_norm_conv(x, tnw, tw, ts, tp, ring if taps > 1 else None, groups, 1e-5)
        u = u.cpu().numpy()
        i = 0
        for s, cnt in step:
            assert np.allclose(u[i:i + cnt], want[s][at[s]:at[s] + cnt], rtol=2e-5, atol=2e-5), (taps, groups, step, s)
            i += cnt
            at[s] += cnt
        ops.group_rmsnorm_residual(torch.ones_like(x), torch.ones(d, device=cuda), torch.zeros_like(x), 1, 1e-5, conv_in=h,
                                   slot=ts, pos=tp, ring=ring if taps > 1 else None, taps=taps)
    assert at == {0: n, 2: n}


def _absorbed_attention(qa, c, pos, sink, scale):
    out = np.zeros_like(qa)
    for t in range(qa.shape[0]):
        for h in range(qa.shape[1]):
            s = scale * (c[: pos[t] + 1] @ qa[t, h])
            m = max(s.max(), sink[h])
            e = np.exp(s - m)
            out[t, h] = (e[:, None] * c[: pos[t] + 1]).sum(0) / (e.sum() + np.exp(sink[h] - m))
    return out


@pytest.mark.parametrize("heads,rank", [(3, 24), (8, 128), (5, 40), (1, 7), (40, 128), (6, 192), (4, 320), (17, 512), (2, 64)])
def test_latent_attention_far_key_sink_and_tile_edges(cuda, lib, heads, rank):
    """One query row is lined up with a key far back and scaled so that this key carries the softmax; another row meets
    a sink that outweighs every key; the positions sit on and around the kernel's 32-key tiles; rows after a token's own
    position hold large values that must not be seen.  Every split count must agree."""
    import torch
    from zhilight_b200 import ops
    rng = np.random.default_rng(heads * 100 + rank)
    n_keys, scale = 700, 0.37
    c = rng.standard_normal((n_keys, rank))
    pos = [0, 1, 30, 31, 32, 33, 63, 64, 65, 255, 256, 699, 640, 17]
    qa = rng.standard_normal((len(pos), heads, rank)) * 0.3
    far = 3
    qa[11, :, :] = 60.0 * c[far] / (scale * (c[far] @ c[far]))      # key 3 of 700 wins by e^60 over its own score scale
    sink = rng.uniform(-1, 1, heads)
    sink[0] = 30.0                                                    # head 0: the sink takes nearly all the mass
    cache = np.full((2, n_keys + 40, rank), 1e4)                      # slot 0 unused, rows past the end poisoned
    cache[1, :n_keys] = c
    want = _absorbed_attention(qa, c, pos, sink, scale)
    assert np.allclose(want[11, 1:], c[far], atol=1e-3) and np.abs(want[2, 0]).max() < 1e-9
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        tc = torch.tensor(cache, dtype=dtype, device=cuda)
        cref = tc[1, :n_keys].double().cpu().numpy()
        ref = _absorbed_attention(qa, cref, pos, sink, scale) if dtype != torch.float32 else want
        tab = ops.slot_table(tc)
        args = (torch.tensor(qa, dtype=torch.float32, device=cuda), tc, tab, torch.ones(len(pos), dtype=torch.int32, device=cuda),
                torch.tensor(pos, dtype=torch.int32, device=cuda), torch.tensor(sink, dtype=torch.float32, device=cuda), scale)
        for splits in (1, 2, 5, 23):
            got = ops.latent_attention(*args, splits=splits).double().cpu().numpy()
            assert np.max(np.abs(got - ref)) < tol * max(1.0, np.abs(ref).max()), (dtype, splits)


# ---------------------------------------------------------------------------------------------- the whole model
@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_layers_and_logits(cuda, lib, name, dtype):
    cfg, W, m = make(CONFIGS[name], dtype, seed=1, max_step_tokens=128)
    toks = tokens_for(cfg, 97, 5)
    want, streams = orc.forward(cfg, W, toks)
    m.capture_layers(True)
    _, logits = m.step(toks, [2] * len(toks), range(len(toks)), range(len(toks)))
    got_streams = m.read_layers(len(toks))
    for i in range(len(cfg.layers)):   # the first layer that differs is the one to look at
        d = np.abs(got_streams[i] - streams[i]).max() / np.abs(streams[i]).max()
        assert d < (1e-4 if dtype == "float32" else 6e-2), (name, dtype, "layer", i, d)
    assert rel_err(logits, want) < TOL[dtype]
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
    want, _ = orc.forward(cfg, W, toks)
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
        assert rel_err(runs[label], want) < TOL[dtype], (name, dtype, label)
    cut = 1e-5 if dtype == "float32" else 2e-2      # the cuts change the order of sums, no more
    assert rel_err(runs["single"], runs["whole"].astype(np.float64)) < cut
    assert rel_err(runs["portions"], runs["whole"].astype(np.float64)) < cut
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone_and_slot_reuse(cuda, lib, dtype):
    """Three requests of different lengths share steps (prompt portions next to single decode tokens); afterwards their
    slots are handed to new requests.  Every logit row equals the request run alone in a fresh model."""
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
    for k in later:                                   # the freed slots, with the old owners' rows and states still in them
        assert eng.open(k).slot in used
    res = eng.forward_step([("d", later["d"][:11], list(range(11))), ("e", later["e"], list(range(5)))])
    got["d"].append(res["d"][1]); got["e"].append(res["e"][1])
    got["d"].append(eng.forward_step([("d", later["d"][11:], list(range(19)))])["d"][1])
    for k in want:
        assert rel_err(np.concatenate(got[k]), want[k]) < TOL[dtype], (dtype, k)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graphs_and_splits(cuda, lib, dtype):
    """A short prompt and then 330 single-token steps: the decode graph, the length buckets (256, 512) and the key splits
    of the attention kernel all change on the way; the last steps look back over more than 300 keys."""
    cfg, W, m = make(CFG_WIDE, dtype, seed=4, max_batch=2, max_seq=512, max_step_tokens=16)
    toks = tokens_for(cfg, 340, 11)
    want, _ = orc.forward(cfg, W, toks)
    _, first = m.step(toks[:10], [1] * 10, range(10), range(10))
    rows = [first]
    for p in range(10, 340):
        rows.append(m.step([toks[p]], [1], [p], [0])[1])
    assert rel_err(np.concatenate(rows), want) < TOL[dtype]
    assert m.stats()[1] > 0          # the single-token steps were replayed as graphs
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
    """config.json + model.safetensors on disk -> registry -> trace replay: the written logits are the oracle's."""
    from zhilight_b200 import registry, safetensors_io, trace
    from zhilight_b200.dekipel import DekipelConfig
    cfg = DekipelConfig.from_dict(CFG_ONES)
    W = orc.random_weights(cfg, 8)
    (tmp_path / "m").mkdir()
    (tmp_path / "m" / "config.json").write_text(json.dumps(CFG_ONES))
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
