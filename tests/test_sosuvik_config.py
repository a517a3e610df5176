"""Configuration, registry and schedule of the Sosuvik family, and its plain implementation's pieces (no GPU)."""
import copy
import json
import math

import pytest
import torch

import plain_sosuvik as plain
import tiny_sosuvik as ts


def test_configuration_reads_every_size_and_writes_it_back():
    from rust_mlx_b200.config import SosuvikConfig
    from rust_mlx_b200.registry import build_model_spec, find_architecture
    for raw, _ in ts.CONFIGS.values():
        cfg = SosuvikConfig.from_dict(raw)
        back = json.loads(json.dumps(cfg.to_dict()))
        assert back == {**raw, "logit_scale": raw.get("logit_scale", 1.0)}
        assert find_architecture(raw).name == "Sosuvik"
        spec = build_model_spec(cfg)
        names = {p.name: tuple(p.shape) for p in spec.all_param_specs()}
        width = raw["width"]
        for i, layer in enumerate(raw["layers"]):
            m = layer["mixer"]
            if layer["type"] == "attention":
                assert names[f"l{i}.mix.q"] == (m["heads"] * m["dim"], width) and names[f"l{i}.mix.k"] == (m["kv_heads"] * m["dim"], width)
                assert names[f"l{i}.mix.v"] == (m["kv_heads"] * m["vdim"], width) and names[f"l{i}.mix.o"] == (width, m["heads"] * m["vdim"])
            else:
                assert names[f"l{i}.mix.q"] == (m["heads"] * (m["dim"] + m["rot_dim"]), width)
                assert names[f"l{i}.mix.dkv"] == (m["kv_rank"] + m["rot_dim"], width) and names[f"l{i}.mix.dkv.norm"] == (m["kv_rank"],)
                assert names[f"l{i}.mix.uk"] == (m["heads"] * m["dim"], m["kv_rank"]) and names[f"l{i}.mix.uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
            f = layer["mlp"]
            assert (f"l{i}.norm2" in names) == (f is not None) == (f"l{i}.mlp.router" in names)
            if f:
                e = f["router"]["experts"]
                assert names[f"l{i}.mlp.router"] == (e, width) and names[f"l{i}.mlp.correction"] == (e,)
                assert names[f"l{i}.mlp.e{e - 1}.gate"] == (f["expert"]["ff"], width) and f"l{i}.mlp.e{e}.gate" not in names
        assert ("loop.in" in names) == ("loop" in raw)
        if "loop" in raw:
            assert names["loop.in"] == (width, 2 * width) and names["loop.step"] == (raw["loop"]["times"], width)
        assert names["head"] == (raw["vocab"], width) and names["embed"] == (raw["vocab"], width)


def test_the_schedule_runs_looped_layers_again_with_caches_of_their_own():
    from rust_mlx_b200.config import SosuvikConfig
    from rust_mlx_b200.parts.loop import LoopEntry
    from rust_mlx_b200.registry import build_model_spec
    for raw, _ in ts.CONFIGS.values():
        spec = build_model_spec(SosuvikConfig.from_dict(raw))
        n = len(raw["layers"])
        runs = [(c.layer, c.cache) for c in spec.schedule]
        layers = [layer for layer, _ in runs if layer < n]
        want = plain.order_of_runs(raw)
        assert layers == [i for i, _ in want]
        caches = [cache for layer, cache in runs if layer < n]
        assert caches == list(range(len(caches)))                      # every run of a layer has its own
        entries = [spec.blocks[layer] for layer, _ in runs if layer >= n]
        assert all(isinstance(e, LoopEntry) for e in entries)
        assert [e.index for e in entries] == list(range(raw.get("loop", {}).get("times", 0)))
        # an entry comes right before the first layer of its pass
        for k, (layer, _) in enumerate(runs):
            if layer >= n:
                assert runs[k + 1][0] == raw["loop"]["start"]
        assert spec.embedding.keep_rows == ("loop" in raw)
        # the tensors of a loop are declared once
        assert len([p for p in spec.all_param_specs() if p.name == "loop.in"]) == (1 if "loop" in raw else 0)
    # a latent layer's page row: latent and rotated part, padded to a size the attention kernels take
    spec = build_model_spec(SosuvikConfig.from_dict(ts.S1))
    specs = spec.cache_specs()
    assert specs[1].head_dim == 32 and not specs[1].values and specs[0].head_dim == 24 and specs[0].kv_heads == 2
    spec = build_model_spec(SosuvikConfig.from_dict(ts.S4))
    assert spec.cache_specs()[0].head_dim == 32 and spec.cache_specs()[2].head_dim == 32


def test_every_problem_of_a_configuration_is_reported():
    from rust_mlx_b200.config import ConfigError, SosuvikConfig
    bad = copy.deepcopy(ts.S1)
    del bad["width"]
    bad["layers"][0]["mixer"]["heads"] = 0
    bad["layers"][1]["mixer"].pop("kv_rank")
    bad["layers"].append({"type": "convolution", "mixer": {}, "mlp": None})
    bad["layers"][2]["mlp"] = {"kind": "dense", "ff": 3}
    with pytest.raises(ConfigError) as e:
        SosuvikConfig.from_dict(bad)
    text = str(e.value)
    assert "width" in text and "heads" in text and "convolution" in text and "kv_rank" in text and "'moe'" in text
    bad = copy.deepcopy(ts.S1)
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    bad["layers"][0]["mixer"]["rot"]["dims"] = 18
    bad["layers"][1]["mixer"]["rot"]["dims"] = 4
    bad["layers"][0]["mlp"]["router"]["groups"] = {"count": 4, "keep": 2}
    bad["layers"][1]["mlp"]["router"]["groups"]["keep"] = 1
    bad["loop"]["stop"] = 7
    with pytest.raises(ConfigError) as e:
        SosuvikConfig.from_dict(bad)
    text = str(e.value)
    assert "kv_heads" in text and "beyond the head" in text and "rot_dim" in text and "4 groups" in text and "cannot give 3" in text \
        and "loop" in text


def test_rotation_tables_of_the_package_follow_the_plain_formulas():
    from rust_mlx_b200.config.sosuvik import RotationConfig
    from rust_mlx_b200.parts.position import RotaryEmbedding
    for base, dims, scaling in [(5000.0, 8, (4.0, 64, 8.0, 2.0)), (1e4, 32, None), (2e5, 32, (8.0, 128, 16.0, 1.0)), (300.0, 4, (2.0, 16, 4.0, 1.0)),
                                (1e6, 64, (16.0, 4096, 32.0, 1.0)), (10.0, 6, (3.0, 8, 1.0, 1.0))]:
        rot = ts.rot(base, dims, scaling)
        f, m = plain.frequencies(rot)
        part = RotaryEmbedding(dims + 4, base, rotary_dim=dims, scaling=RotationConfig(base, dims, scaling).scaling_dict(), factor_on="rotated")
        assert torch.allclose(part._table.double(), f, rtol=1e-6, atol=0)
        assert abs(part.magnitude - m) < 1e-12 and part.score_scale == 1.0
    # scaled and unscaled tables differ where they should: the slowest pair is slowed by the factor, the fastest is kept
    f, m = plain.frequencies(ts.rot(1e4, 64, (8.0, 512, 32.0, 1.0)))
    f0, _ = plain.frequencies(ts.rot(1e4, 64))
    assert f[0] == f0[0] and abs(f[-1] - f0[-1] / 8.0) < 1e-18 and abs(m - (0.1 * math.log(8.0) + 1)) < 1e-12


def test_plain_rotation_pairs_halves_or_neighbours():
    x = torch.arange(1.0, 7.0, dtype=torch.float64).view(1, 6)            # one token at position 3, four numbers rotated
    rot = {"base": 100.0, "dims": 4}
    a = [3.0 * 100.0 ** (-2.0 * i / 4) for i in range(2)]
    halves = plain.rotate(x, torch.tensor([3]), rot, False)[0]
    assert torch.allclose(halves, torch.tensor([1 * math.cos(a[0]) - 3 * math.sin(a[0]), 2 * math.cos(a[1]) - 4 * math.sin(a[1]),
                                                3 * math.cos(a[0]) + 1 * math.sin(a[0]), 4 * math.cos(a[1]) + 2 * math.sin(a[1]), 5.0, 6.0],
                                               dtype=torch.float64))
    pairs = plain.rotate(x, torch.tensor([3]), rot, True)[0]
    assert torch.allclose(pairs, torch.tensor([1 * math.cos(a[0]) - 2 * math.sin(a[0]), 2 * math.cos(a[0]) + 1 * math.sin(a[0]),
                                               3 * math.cos(a[1]) - 4 * math.sin(a[1]), 4 * math.cos(a[1]) + 3 * math.sin(a[1]), 5.0, 6.0],
                                              dtype=torch.float64))


def test_plain_chunks_sink_and_cap():
    v = plain.sees(5, 2)
    assert v.tolist() == [[True, False, False, False, False], [True, True, False, False, False],
                          [False, False, True, False, False], [False, False, True, True, False],
                          [False, False, False, False, True]]
    assert plain.sees(3).tolist() == [[True, False, False], [True, True, False], [True, True, True]]
    s = torch.tensor([[0.0, -math.inf], [math.log(3.0), 0.0]], dtype=torch.float64)
    assert torch.allclose(plain.softmax_with_sink(s), torch.tensor([[0.5, 0.0], [0.6, 0.2]], dtype=torch.float64))


def test_plain_router_keeps_the_best_groups_and_weighs_by_uncorrected_scores():
    # six experts in three groups of two; corrected scores by group: (0.9, 0.1), (0.6, 0.55), (0.7, -2.0)
    s = torch.tensor([[0.9, 0.1, 0.6, 0.55, 0.7, 0.5]], dtype=torch.float64)
    z = torch.log(s / (1 - s))
    correction = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, -2.5], dtype=torch.float64)
    router = {"experts": 6, "top": 3, "scale": 2.0, "groups": {"count": 3, "keep": 2}}
    ids, weights = plain.choose_experts(z, correction, router)
    # group worths 1.0, 1.15, -1.3: the third group is out although its first expert would be second best
    assert ids.tolist() == [[0, 2, 3]]
    assert torch.allclose(weights, torch.tensor([[0.9, 0.6, 0.55]], dtype=torch.float64) / 2.05 * 2.0)
    # the correction decides the choice, not the weight
    ids, weights = plain.choose_experts(z, torch.tensor([0.0, 5.0, 0.0, 0.0, 0.0, 0.0], dtype=torch.float64), {"experts": 6, "top": 1, "scale": 1.0})
    assert ids.tolist() == [[1]] and torch.allclose(weights, torch.ones(1, 1, dtype=torch.float64))
    # all corrected scores negative (group worths -5.0, -4.85, -4.8): the first group is out although its first expert has
    # the largest corrected score of all, and experts of a group that is out must not come back in as zeros
    ids, _ = plain.choose_experts(z, torch.full((6,), -3.0, dtype=torch.float64), router)
    assert ids.tolist() == [[4, 2, 3]]


def test_plain_expert_clamps_before_it_multiplies():
    x = torch.tensor([[1.0]], dtype=torch.float64)
    one = torch.ones(1, 1, dtype=torch.float64)
    for g, u, limit in [(3.0, 0.2, 1.0), (-4.0, 5.0, 1.5), (0.3, -9.0, 2.0)]:
        y = plain.clamped_expert(x, one * g, one * u, one, limit).item()
        gc, uc = min(g, limit), max(-limit, min(u, limit))
        assert abs(y - gc / (1 + math.exp(-1.702 * gc)) * (uc + 1)) < 1e-12
