"""CPU-side pieces of the Dekipel integration: the oracle's own consistency, configuration parsing, the safetensors
reader, the registry, and the engine's scheduling logic over a fake decoder."""
import json

import numpy as np
import pytest

from tests import dekipel_oracle as orc
from zhilight_b200 import registry, safetensors_io
from zhilight_b200.dekipel import DekipelConfig
from zhilight_b200.engine import Engine, SamplingParams, SlotPool, sample_token


def _cfg():
    return {"architecture": "Dekipel", "vocab": 29, "width": 24, "norm": {"eps": 1e-5, "groups": 2}, "canon": {"taps": 3},
            "layers": [{"type": "latent_attention", "mixer": dict(heads=2, dim=6, vdim=10, q_rank=8, kv_rank=12, scale=0.4),
                        "mlp": {"kind": "dense", "ff": 20}},
                       {"type": "latent_attention", "mixer": dict(heads=3, dim=4, vdim=4, q_rank=6, kv_rank=12, scale=0.5, kv_from=0),
                        "mlp": None}]}


def test_oracle_is_causal_and_sink_counts_once():
    cfg = DekipelConfig.from_dict(_cfg())
    W = {k: v.astype(np.float64) for k, v in orc.random_weights(cfg, 0).items()}
    toks = list(range(17))
    full, _ = orc.forward(cfg, W, toks)
    part, _ = orc.forward(cfg, W, toks[:9])
    assert np.allclose(full[:9], part, atol=1e-12)
    # a single key and a sink equal to its score: the value gets exactly half of the weight
    q, k, v = np.ones((1, 1, 4)), np.ones((1, 1, 4)), np.full((1, 1, 2), 6.0)
    assert np.allclose(orc.sink_softmax_attention(q, k, v, np.array([4.0 * 0.5]), 0.5), 3.0)
    # groups of one element normalise every element to +-w (up to eps)
    assert np.allclose(orc.group_rms_norm(np.array([[3.0, -4.0]]), np.array([2.0, 2.0]), 2, 0.0), [[2.0, -2.0]])


def test_config_parse_shapes_and_validation():
    cfg = DekipelConfig.from_dict(_cfg())
    assert cfg.layers[1]["kv_from"] == 0 and cfg.layers[1]["ff"] == 0 and cfg.layers[0]["kv_from"] == -1
    shapes = cfg.tensor_shapes()
    assert shapes["l0.mix.uv"] == (20, 12) and shapes["l1.mix.uk"] == (12, 12) and "l1.mix.dkv" not in shapes
    assert "l1.mlp.up" not in shapes and shapes["l0.canon2"] == (24, 3)
    assert DekipelConfig.from_dict(cfg.to_dict()).layers == cfg.layers
    bad = _cfg()
    bad["layers"][1]["mixer"]["kv_from"] = 1
    with pytest.raises(ValueError):
        DekipelConfig.from_dict(bad)
    bad = _cfg()
    bad["layers"][0]["type"] = "something_else"
    with pytest.raises(ValueError):
        DekipelConfig.from_dict(bad)


def test_safetensors_roundtrip_and_bf16(tmp_path):
    a = np.array([[1.0, -2.5, 3.140625], [1e-3, 65280.0, 0.0]], dtype=np.float32)
    b16 = safetensors_io.f32_to_bf16(a)
    assert safetensors_io.is_bf16(b16) and b16.shape == a.shape
    assert np.allclose(safetensors_io.bf16_to_f32(b16), a, rtol=2 ** -8)
    assert safetensors_io.f32_to_bf16(np.array([1.00390625], np.float32))[0] == 0x3F80          # tie -> even
    assert safetensors_io.f32_to_bf16(np.array([1.01171875], np.float32))[0] == 0x3F82          # tie -> even (up)
    path = str(tmp_path / "t.safetensors")
    safetensors_io.save_file({"w": b16, "i": np.arange(6, dtype=np.int32).reshape(2, 3), "f": a}, path)
    back = safetensors_io.load_file(path)
    assert safetensors_io.is_bf16(back["w"]) and np.array_equal(np.asarray(back["w"]), np.asarray(b16))
    assert np.array_equal(back["i"], np.arange(6).reshape(2, 3)) and np.array_equal(back["f"], a)


def test_registry_picks_the_class_by_config():
    assert registry.architecture_of(_cfg()) == "Dekipel"
    assert registry.architecture_of({"architectures": ["LlamaForCausalLM"]}) == "LlamaForCausalLM"
    assert registry.supported_dtypes(_cfg()) == ("bfloat16", "float32")
    assert "float32" not in registry.supported_dtypes({"model_type": "llama"})
    with pytest.raises(ValueError):
        registry.build_model({"architecture": "nope"})
    assert registry.hf_llama_name("model.layers.3.self_attn.q_proj.weight") == "layers.3.attn.project_q.weight"
    assert registry.hf_llama_name("model.layers.0.mlp.down_proj.qweight") == "layers.0.ff.w_out.qweight"


class FakeModel:
    """Keeps every slot's token history; the 'logits' of a row are a function of the whole history up to it, so any
    row lost, repeated, misplaced or leaked between slots changes the answer."""
    max_batch, max_seq, max_step_tokens, vocab_size = 3, 64, 8, 11

    def __init__(self):
        self.hist = {s: [] for s in range(self.max_batch)}
        self.steps = []

    @staticmethod
    def row(history):
        h = 7
        for t in history:
            h = (h * 31 + t + 1) % 1000003
        out = np.zeros(FakeModel.vocab_size, dtype=np.float32)
        out[h % FakeModel.vocab_size] = 1.0 + (h % 5)
        return out

    def step(self, tokens, slots, positions, want_rows=(), want_logits=True):
        assert 0 < len(tokens) <= self.max_step_tokens
        self.steps.append(list(slots))
        rows = []
        for t, s, p in zip(tokens, slots, positions):
            if p == 0:
                self.hist[s] = []            # a new owner starts at position 0: nothing of the old one is visible
            assert p == len(self.hist[s]), "rows must arrive at consecutive positions"
            self.hist[s].append(t)
            rows.append(self.row(self.hist[s]))
        logits = np.stack([rows[w] for w in want_rows]) if len(want_rows) else np.zeros((0, self.vocab_size), np.float32)
        return logits.argmax(-1).astype(np.int32), (logits if want_logits else None)


def test_slot_pool_gives_back_and_reuses():
    pool = SlotPool(2)
    a, b = pool.alloc("a"), pool.alloc("b")
    assert {a, b} == {0, 1} and pool.alloc("c") is None
    pool.release(a)
    assert pool.alloc("c") == a


def test_forward_step_cuts_portions_and_keeps_rows_in_order():
    model = FakeModel()
    eng = Engine(model)
    eng.open("x"), eng.open("y")
    tx, ty = list(range(1, 20)), [5, 4, 3]
    res = eng.forward_step([("x", tx, [0, 18, 7]), ("y", ty, [2])])
    assert all(len(s) <= 8 for s in model.steps) and len(model.steps) >= 3
    assert np.array_equal(res["x"][1], np.stack([FakeModel.row(tx[:1]), FakeModel.row(tx[:8]), FakeModel.row(tx)]))
    assert np.array_equal(res["y"][1][0], FakeModel.row(ty))
    res = eng.forward_step([("y", [9], [0]), ("x", [2, 2], [])])
    assert np.array_equal(res["y"][1][0], FakeModel.row(ty + [9])) and res["x"][1].shape == (0, 11)
    eng.close("x")
    assert eng.open("z").slot == 0 and eng.open("w") is not None and eng.open("v") is None
    with pytest.raises(ValueError):
        eng.forward_step([("z", [1] * 65, [])])


def test_scheduler_continuous_batching_matches_one_by_one():
    prompts = [[1, 2, 3], list(range(1, 10)) * 2, [4], [7, 7, 7, 7, 7, 7, 7, 7, 7, 7, 7], [3, 1]]

    def alone(p, n):
        seq, out = list(p), []
        for _ in range(n):
            out.append(int(FakeModel.row(seq).argmax()))
            seq.append(out[-1])
        return out
    model = FakeModel()
    outs = Engine(model).generate(prompts, max_new_tokens=6)
    assert outs == [alone(p, 6) for p in prompts]
    assert any(len(set(s)) > 1 for s in model.steps)             # several requests shared a step
    assert max(len(s) for s in model.steps) <= model.max_step_tokens


def test_sampling_is_seeded_and_respects_top_k_top_p():
    logits = np.array([0.0, 3.0, 2.9, -5.0, 1.0])
    rng = np.random.default_rng(0)
    picks = {sample_token(logits, SamplingParams(1.0, top_k=2), rng) for _ in range(200)}
    assert picks == {1, 2}
    picks = {sample_token(logits, SamplingParams(0.5, top_p=0.3), rng) for _ in range(50)}
    assert picks == {1}
    a = [sample_token(logits, SamplingParams(1.0), np.random.default_rng(5)) for _ in range(3)]
    b = [sample_token(logits, SamplingParams(1.0), np.random.default_rng(5)) for _ in range(3)]
    assert a == b and SamplingParams().greedy
