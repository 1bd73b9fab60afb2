"""Kubedra without a GPU: configuration, model description, tensor names, the plain implementation's own
mechanisms, and the engine's host logic (steps, cache, schedule) with the plain kernel references."""
import copy
import json

import pytest
import torch

import plain_kubedra as pk
import tiny_kubedra as tk
from dotllm_b200.config import build_spec, config_from_dict, load_config
from dotllm_b200.engine import StepEntry, run_step
from dotllm_b200.errors import ConfigError, WeightsError
from dotllm_b200.models.decoder import DecoderModel
from dotllm_b200.parts.base import Runtime
from dotllm_b200.weights import load_into

CPU = Runtime(torch.float32, torch.device("cpu"))


def test_configuration_reads_every_key_and_writes_it_back():
    for name in ("P", "Q", "R", "S"):
        cfg = config_from_dict(tk.CONFIGS[name])
        assert cfg.to_dict() == tk.CONFIGS[name]
        assert type(cfg).__name__ == "KubedraConfig"
    cfg = config_from_dict(tk.CONFIGS["P"])
    assert cfg.layer_runs() == [(0, False), (1, False), (0, True), (1, False), (2, False), (3, False)]
    assert config_from_dict(tk.CONFIGS["Q"]).layer_runs() == [(0, False), (1, False), (1, True), (1, True), (2, False)]
    assert config_from_dict(tk.CONFIGS["R"]).layer_runs() == [(0, False), (1, False)]
    for broken, match in ((lambda c: c.pop("width"), "width"), (lambda c: c["layers"][0]["mixer"].pop("heads"), "heads"),
                          (lambda c: c["layers"][1].update(type="conv"), "type"),
                          (lambda c: c.update(loop={"start": 2, "stop": 9, "times": 2}), "loop"),
                          (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind")):
        bad = copy.deepcopy(tk.CONFIGS["P"])
        broken(bad)
        with pytest.raises(ConfigError, match=match):
            config_from_dict(bad)


def test_description_schedule_and_tensor_names():
    spec = build_spec(config_from_dict(tk.CONFIGS["Q"]))
    assert [(e.layer, e.takes_embedding) for e in spec.schedule] == [(0, False), (1, False), (1, True), (1, True), (2, False)]
    assert all(e.cache_of is None for e in spec.schedule)          # every pass keeps a cache of its own
    model = DecoderModel(spec, CPU)
    expected, optional = model.expected_weights()
    assert {"embed", "pos", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.a1", "l0.mix.a2",
            "l0.mix.a2.b", "l0.mix.norm", "l0.mlp.gate", "l1.mix.dq", "l1.mix.dq.norm", "l1.mix.uk", "l1.mix.uv",
            "l1.mlp.e5.down", "l1.mlp.router", "l1.mlp.router.b", "l1.mlp.shared.up"} <= set(expected)
    assert "head.weight" in optional and "head.weight" not in expected         # the head is the embedding table
    needs = model.cache_needs()
    assert [n.kind for n in needs] == ["state", "kv", "kv", "kv", "kv"]
    assert needs[1].window == 130 and needs[4].window is None and needs[0].state_shape == (1, 64, 64)
    # a layer without a feed-forward declares no second pair of norms
    names = set(DecoderModel(build_spec(config_from_dict(tk.CONFIGS["P"])), CPU).expected_weights()[0])
    assert "l2.norm1b" in names and "l2.norm2" not in names and not any(n.startswith("l2.mlp") for n in names)


def test_a_rank_that_only_the_tensors_give(tmp_path):
    folder = tk.make_folder(tmp_path, "R")
    cfg = json.loads((folder / "config.json").read_text())
    del cfg["layers"][0]["mixer"]["decay_rank"]                    # the stored factors are 3 wide, the default is not
    (folder / "config.json").write_text(json.dumps(cfg))
    model = load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder)
    assert model.blocks[0].mixer.decay_rank == 3
    # any other wrong shape is still refused
    cfg["layers"][0]["mixer"]["dim"] = 12
    (folder / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(WeightsError, match="wrong shapes"):
        load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder)


def test_plain_recurrence_continues_from_its_state():
    g = torch.Generator().manual_seed(0)
    q, k, a = (torch.randn(30, 2, 6, generator=g, dtype=torch.float64) for _ in range(3))
    v = torch.randn(30, 2, 5, generator=g, dtype=torch.float64)
    a = torch.sigmoid(a)
    whole, s_whole = pk.gla_recurrence(q, k, v, a)
    first, s = pk.gla_recurrence(q[:11], k[:11], v[:11], a[:11])
    rest, s = pk.gla_recurrence(q[11:], k[11:], v[11:], a[11:], s)
    assert torch.allclose(torch.cat([first, rest]), whole) and torch.allclose(s, s_whole)
    # the closed form: o_t = sum_j (prod_{j < i <= t} alpha_i) . k_j . q_t  v_j
    t = 7
    want = sum(((a[j + 1:t + 1].prod(dim=0) * k[j] * q[t]).sum(-1)[:, None] * v[j]) for j in range(t + 1))
    assert torch.allclose(whole[t], want)


def test_plain_window_and_router():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(9, 1, 4, generator=g, dtype=torch.float64), torch.randn(9, 1, 4, generator=g, dtype=torch.float64)
    v = torch.eye(9, dtype=torch.float64)[:, None, :]              # the output row is the attention weights themselves
    p = pk.windowed_softmax_attention(q, k, v, 1.0, 3)[:, 0]
    for i in range(9):
        seen = [j for j in range(9) if 0 <= i - j < 3]
        assert torch.count_nonzero(p[i]).item() == len(seen) and abs(p[i, seen].sum().item() - 1) < 1e-12
    w = {"r.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]]), "r.router.b": torch.tensor([0.0, 0.0, -0.5])}
    chosen, weight = pk.route(torch.tensor([[2.0, 1.0]], dtype=torch.float64), w, "r.", 2)
    assert chosen.tolist() == [[2, 0]] and torch.allclose(weight, torch.softmax(torch.tensor([[2.5, 2.0]], dtype=torch.float64), -1))


def load(tmp_path, which):
    folder = tk.make_folder(tmp_path, which)
    cfg, weights = tk.read_folder(folder)
    return load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder), cfg, weights


@pytest.mark.parametrize("which", ["P", "Q", "R", "S"])
def test_steps_cuts_and_batches_agree_with_the_plain_implementation(cpu_kernels, tmp_path, which):
    model, cfg, w = load(tmp_path, which)
    a, b = tk.random_tokens(83, cfg["vocab"], 1), tk.random_tokens(21, cfg["vocab"], 2)
    ra, rb = pk.forward(cfg, w, a).float(), pk.forward(cfg, w, b).float()
    cache = model.new_cache(64 * 4)
    cache.fill_free_pages(float("nan"))
    sa, sb = cache.open_sequence(), cache.open_sequence()
    out = run_step(model, cache, [StepEntry(sa, a[:66], [0, 1, 65]), StepEntry(sb, b[:5], [4])])
    assert torch.allclose(out, torch.cat([ra[[0, 1, 65]], rb[[4]]]), atol=2e-4)
    out = run_step(model, cache, [StepEntry(sa, a[66:68], [0, 1]), StepEntry(sb, b[5:19], [13])])       # portions of 2 and 14
    assert torch.allclose(out, torch.cat([ra[[66, 67]], rb[[18]]]), atol=2e-4)
    for t in range(68, 83):
        entries = [StepEntry(sa, [a[t]])] + ([StepEntry(sb, [b[t - 49]])] if t - 49 < 21 else [])
        out = run_step(model, cache, entries)
        assert torch.allclose(out[0], ra[t], atol=2e-4)
        if len(entries) == 2:
            assert torch.allclose(out[1], rb[t - 49], atol=2e-4)
    cache.close_sequence(sa)
    cache.fill_free_pages(float("nan"))
    sc = cache.open_sequence()                           # takes the slot, the state and the pages that a gave back
    out = run_step(model, cache, [StepEntry(sc, b, None)])
    assert torch.allclose(out[0], rb[-1], atol=2e-4)
    cache.check()


def test_trace_replay_of_a_kubedra_folder(cpu_kernels, tmp_path):
    import io
    import numpy as np
    from dotllm_b200.engine.trace import TraceReplayer
    model, cfg, w = load(tmp_path, "R")

    class Wrapped:                                        # what the replayer needs of a Model
        def new_cache(self, n):
            return model.new_cache(n)

        def step(self, cache, entries):
            return run_step(model, cache, entries)

    a = tk.random_tokens(12, cfg["vocab"], 3)
    ref = pk.forward(cfg, w, a).float()
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:9], "want": [0, 8]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[9:10], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": a[10:], "want": [1]}], "end": ["x"]}]
    out = io.StringIO()
    replayer = TraceReplayer(Wrapped(), 128, tmp_path / "out")
    replayer.check_kernels = lambda: None
    replayer.run([json.dumps(s) for s in steps], out)
    assert out.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
    got0 = torch.from_numpy(np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(-1, cfg["vocab"]).copy())
    got2 = torch.from_numpy(np.fromfile(tmp_path / "out" / "2.f32", dtype="<f4").reshape(-1, cfg["vocab"]).copy())
    assert not (tmp_path / "out" / "1.f32").exists()
    assert torch.allclose(got0, ref[[0, 8]], atol=2e-4) and torch.allclose(got2, ref[[11]], atol=2e-4)
    assert not replayer.sequences and not replayer.cache.live
