"""Komulorn without a GPU: configuration, description, tensor names, the rescaled rotary frequencies, what the plain
implementation's mechanisms do, and the engine's host logic (steps, cache, shared caches, replay) against the plain
implementation with the plain kernel references in place of the CUDA kernels."""
import copy
import json
import math

import pytest
import torch

import plain_komulorn as pk
import tiny_komulorn as tk
from dotllm_b200.config import config_from_dict
from dotllm_b200.config.komulorn import DEFAULT_MAX_POSITIONS, KomulornConfig
from dotllm_b200.config.registry import build_spec, load_config
from dotllm_b200.engine.step import StepEntry, run_step
from dotllm_b200.errors import ConfigError
from dotllm_b200.models.decoder import DecoderModel
from dotllm_b200.parts.base import Runtime
from dotllm_b200.parts.rotary import rotary_frequencies, rotary_magnitude
from dotllm_b200.weights.loader import load_into

CPU = Runtime(torch.float32, torch.device("cpu"))


def test_configuration_reads_every_size_and_writes_it_back():
    for name, d in tk.CONFIGS.items():
        cfg = config_from_dict(copy.deepcopy(d))
        assert isinstance(cfg, KomulornConfig) and cfg.max_positions == DEFAULT_MAX_POSITIONS
        assert config_from_dict(cfg.to_dict()) == cfg, name
        for layer, raw in zip(cfg.layers, d["layers"]):
            m = raw["mixer"]
            assert (layer.mixer.heads, layer.mixer.kv_heads, layer.mixer.dim, layer.mixer.vdim) == \
                (m["heads"], m["kv_heads"], m["dim"], m["vdim"])
            assert layer.mixer.scale == m["scale"] and layer.mixer.kv_from == m.get("kv_from")
            assert layer.mixer.rot_dims == (m["rot"]["dims"] if "rot" in m else 0)
            assert (layer.mlp is None) == (raw["mlp"] is None)
    a = config_from_dict(copy.deepcopy(tk.CONFIGS["A"]))
    assert a.logit_softcap == 12.0 and a.layers[0].mlp.shared_ff == 72 and a.layers[1].mlp.shared_ff == 0
    assert config_from_dict(dict(copy.deepcopy(tk.CONFIGS["B"]), max_positions=900)).max_positions == 900


def test_configuration_refuses_what_the_design_does_not_have():
    def broken(change):
        d = copy.deepcopy(tk.CONFIGS["A"])
        change(d)
        with pytest.raises(ConfigError):
            config_from_dict(d)
    broken(lambda d: d["layers"][1]["mixer"].update(kv_from=1))            # itself
    broken(lambda d: d["layers"][1]["mixer"].update(kv_from=2))            # a later layer
    broken(lambda d: d["layers"][3]["mixer"].update(kv_from=1))            # a layer that keeps no keys of its own
    broken(lambda d: d["layers"][1]["mixer"].update(kv_heads=3))           # other key/value heads than the layer it reads
    broken(lambda d: d["layers"][0]["mixer"]["rot"].update(dims=26))       # more rotated channels than the head has
    broken(lambda d: d["layers"][0]["mixer"].update(heads=5))              # 5 query heads over 2 key/value heads
    broken(lambda d: d["layers"][0]["mlp"]["router"].update(top=6))        # more choices than experts
    broken(lambda d: d["layers"][0]["mlp"].update(kind="dense"))
    broken(lambda d: d["layers"][0].update(type="recurrent"))
    broken(lambda d: d.pop("vocab"))


def test_description_names_the_designs_tensors_and_shares_caches():
    spec = build_spec(config_from_dict(copy.deepcopy(tk.CONFIGS["A"])))
    assert [e.cache_of for e in spec.schedule] == [None, 0, None, 0]
    model = DecoderModel(spec, Runtime(torch.float32, torch.device("meta")))
    expected, optional = model.expected_weights()
    names = set(expected)
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.q.b", "l0.mix.k", "l0.mix.k.b",
            "l0.mix.v", "l0.mix.v.b", "l0.mix.g", "l0.mix.o", "l0.mlp.router", "l0.mlp.e0.up", "l0.mlp.e4.down",
            "l0.mlp.shared.up", "l0.mlp.shared.down", "l0.mlp.shared.sg", "l1.mix.q", "l1.mix.q.b", "l1.mix.g", "l1.mix.o"} <= names
    assert not {"l1.mix.k", "l1.mix.v", "l1.mix.k.b", "l1.mix.v.b", "l1.mlp.shared.up", "l2.norm2", "l2.mlp.router",
                "l0.mlp.e0.gate", "l0.mlp.router.b"} & names
    assert "l2.norm2" in optional
    assert tuple(expected["l0.mix.v"].shape) == (2 * 40, 96) and tuple(expected["l0.mix.o"].shape) == (96, 6 * 40)
    assert tuple(expected["l0.mix.g"].shape) == (6, 96) and tuple(expected["l0.mlp.shared.sg"].shape) == (1, 96)
    needs = model.cache_needs()
    assert (needs[0].key_width(), needs[0].value_width(), needs[0].n_kv_heads) == (24, 40, 2)
    cache = model.new_cache(256)
    assert len([g for g in cache.groups if g.kind == "kv"]) == 2          # layers 0 (read by 1 and 3) and 2
    assert cache.groups[0].v.shape[-2:] == (40, 64) and cache.groups[0].k.shape[-2:] == (64, 24)


@pytest.mark.parametrize("dims,base,scaling", [(16, 500.0, (4.0, 64, 8.0, 2.0)), (64, 10000.0, (8.0, 128, 16.0, 1.0)),
                                              (8, 1000.0, (2.0, 32, 4.0, 0.5)), (6, 100.0, None),
                                              (32, 10000.0, (3.0, 4096, 32.0, 1.0)), (4, 10.0, (16.0, 8, 1.0, 1.0))])
def test_rescaled_frequencies_are_the_plain_ones(dims, base, scaling):
    rot = tk.rot(dims, base, scaling)
    want, grow = pk.rotary_frequencies(rot)
    s = None if scaling is None else {"rope_type": "yarn", "factor": scaling[0], "original_max_position_embeddings": scaling[1],
                                      "fast_turns": scaling[2], "slow_turns": scaling[3]}
    got = torch.from_numpy(rotary_frequencies(dims, base, s))
    assert torch.allclose(got, want, rtol=1e-14, atol=0)
    assert rotary_magnitude(s) == pytest.approx(grow, rel=1e-15)
    if scaling:                                                    # the fastest keep their frequency, the slowest are divided
        plain = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        assert bool((got <= plain * (1 + 1e-12)).all()) and bool((got >= plain / scaling[0] * (1 - 1e-12)).all())
        assert grow == pytest.approx(0.1 * math.log(scaling[0]) + 1.0)


def test_plain_mechanisms_alone():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    # the rotation touches the first `dims` channels only, in pairs (i, i + dims/2), and keeps each pair's length but for the factor
    x = r(5, 3, 12)
    rot = tk.rot(8, 100.0, (2.0, 16, 4.0, 1.0))
    y = pk.rotate(x, torch.arange(5), rot)
    grow = pk.rotary_frequencies(rot)[1]
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.allclose(y[0, :, :8], x[0, :, :8] * grow)
    assert torch.allclose(y[..., :4] ** 2 + y[..., 4:8] ** 2, (x[..., :4] ** 2 + x[..., 4:8] ** 2) * grow ** 2)
    # scores depend on the distance between positions only
    q, k = r(1, 1, 12), r(1, 1, 12)
    dot = lambda a, b: float((pk.rotate(q, [a], rot) * pk.rotate(k, [b], rot)).sum())
    assert dot(7, 3) == pytest.approx(dot(104, 100), rel=1e-9) and abs(dot(7, 3) - dot(7, 4)) > 1e-6
    # query head h reads key/value head h // (H / G); a query sees itself and everything before it
    q, k, v = r(6, 4, 5), r(6, 2, 5), r(6, 2, 3)
    o = pk.causal_softmax_attention(q, k, v, 0.7)
    assert torch.allclose(o[0], v[0, [0, 0, 1, 1]])
    w = torch.softmax((k[:4, 1] @ q[3, 2]) * 0.7, dim=0)
    assert torch.allclose(o[3, 2], w @ v[:4, 1])
    assert torch.allclose(pk.causal_softmax_attention(q[4:], k, v, 0.7), o[4:])        # queries are the last positions
    # the router's scores are sigmoids that are not renormalised, ties go to the lower index
    h = r(4, 8)
    wr = r(5, 8)
    wr[3] = wr[1]
    ids, scores = pk.router_choice(h, wr, 3)
    s = torch.sigmoid(h @ wr.T)
    assert torch.allclose(scores, torch.gather(s, 1, ids)) and bool((scores.sum(-1) != 1).all())
    for t in range(4):
        if 1 in ids[t].tolist() and 3 in ids[t].tolist():
            assert ids[t].tolist().index(1) < ids[t].tolist().index(3)
    # the score multiplies what goes into the expert: the square of relu makes that the square of the score on the way out
    up, down = r(7, 8), r(8, 7)
    assert torch.allclose(pk.squared_relu_expert(0.3 * h, up, down), 0.09 * pk.squared_relu_expert(h, up, down))


def load(tmp_path, which):
    folder = tk.make_folder(tmp_path, which)
    cfg, weights = tk.read_folder(folder)
    return load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder), cfg, weights


@pytest.mark.parametrize("which", ["A", "C", "D"])
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
    sc = cache.open_sequence()                           # takes the slot and the pages that a gave back
    out = run_step(model, cache, [StepEntry(sc, b, None)])
    assert torch.allclose(out[0], rb[-1], atol=2e-4)
    cache.check()


def test_a_shared_cache_is_read_and_a_wrong_one_would_show(cpu_kernels, tmp_path):
    """The second layer of the sharpened pair reads the first one's keys and values.  The plain implementation that gives
    it the keys of ANOTHER prompt differs visibly; the engine agrees with the right one, also across a cut."""
    folder = tk.sharp_folder(tmp_path, "sharp_shared")
    cfg, w = tk.read_folder(folder)
    model = load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder)
    tokens = tk.random_tokens(90, cfg["vocab"], 4)
    ref = pk.forward(cfg, w, tokens).float()
    other = copy.deepcopy(cfg)
    del other["layers"][1]["mixer"]["kv_from"]
    w2 = dict(w, **{"l1.mix.k": w["l0.mix.k"].roll(1, 0), "l1.mix.k.b": w["l0.mix.k.b"], "l1.mix.v": w["l0.mix.v"],
                    "l1.mix.v.b": w["l0.mix.v.b"]})
    wrong = pk.forward(other, w2, tokens).float()
    assert float((wrong - ref).abs().max()) > 1e-2
    cache = model.new_cache(256)
    s = cache.open_sequence()
    out = torch.cat([run_step(model, cache, [StepEntry(s, tokens[:70], list(range(70)))]),
                     run_step(model, cache, [StepEntry(s, tokens[70:], list(range(20)))])])
    assert torch.allclose(out, ref, atol=3e-4)


def test_trace_replay_of_a_komulorn_folder(cpu_kernels, tmp_path):
    import io
    import numpy as np
    from dotllm_b200.engine.trace import TraceReplayer
    model, cfg, w = load(tmp_path, "C")

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
    assert not replayer.sequences


@pytest.mark.parametrize("which,layer,width", [("A", 0, 64), ("D", 1, 96)])
def test_heads_laid_out_at_a_common_width_give_the_same_logits(cpu_kernels, tmp_path, which, layer, width):
    """A bfloat16 run lays keys and values of different widths out at one width that the tensor-core kernels take (zeros
    behind each head's own channels).  The logits are those of the true widths, up to bfloat16's rounding."""
    folder = tk.make_folder(tmp_path, which, dtype=torch.bfloat16)
    cfg, w = tk.read_folder(folder)
    model = load_into(DecoderModel(build_spec(load_config(folder)), Runtime(torch.bfloat16, torch.device("cpu"))), folder)
    cache = model.new_cache(256)
    need = model.cache_needs()[layer]
    assert (need.key_width(), need.value_width()) == (width, width)
    mixer = model.blocks[layer].mixer
    assert (mixer.lay_k, mixer.lay_v) == (width, width) and mixer.w_o.shape[1] == mixer.n_heads * width
    if which == "D":                     # twenty query heads on one key/value head are more than those kernels take: true widths
        assert (model.blocks[0].mixer.lay_k, model.blocks[0].mixer.lay_v) == (8, 4)
    tokens = tk.random_tokens(70, cfg["vocab"], 6)
    ref = pk.forward(cfg, w, tokens).float()
    s = cache.open_sequence()
    out = torch.cat([run_step(model, cache, [StepEntry(s, tokens[:66], list(range(66)))]),
                     run_step(model, cache, [StepEntry(s, tokens[66:], list(range(4)))])])
    err = (out - ref).pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt()
    assert float(err.median()) < 2e-2 and float(err.max()) < 0.5          # a router's near-tie may fall the other way in bfloat16
