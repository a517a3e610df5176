"""Configuration, registry and schedule of the Reverax family, and its plain implementation's pieces (no GPU)."""
import copy
import json
import math

import pytest
import torch

import plain_reverax as plain
import tiny_reverax as tr


def test_configuration_reads_every_size_and_writes_it_back():
    from rust_mlx_b200.config import ReveraxConfig
    from rust_mlx_b200.registry import build_model_spec, find_architecture
    for raw, _ in tr.CONFIGS.values():
        cfg = ReveraxConfig.from_dict(raw)
        back = json.loads(json.dumps(cfg.to_dict()))
        want = copy.deepcopy(raw)
        want["logit_scale"] = raw.get("logit_scale", 1.0)
        want["norm"]["groups"] = raw["norm"].get("groups", 1)
        assert back == want
        assert find_architecture(raw).name == "Reverax"
        spec = build_model_spec(cfg)
        names = {p.name: tuple(p.shape) for p in spec.all_param_specs()}
        width = raw["width"]
        for i, layer in enumerate(raw["layers"]):
            if "weights_of" in layer:
                assert not any(n.startswith(f"l{i}.") for n in names)       # no tensors of its own
                continue
            m = layer["mixer"]
            a, p = (m, f"l{i}.mix") if layer["type"] == "attention" else (m["left"], f"l{i}.mix.left")
            assert names[f"{p}.q"] == (a["heads"] * a["dim"], width) and names[f"{p}.q.b"] == (a["heads"] * a["dim"],)
            assert names[f"{p}.k"] == (a["kv_heads"] * a["dim"], width) and names[f"{p}.v.b"] == (a["kv_heads"] * a["vdim"],)
            assert names[f"{p}.o"] == (width, a["heads"] * a["vdim"])
            if layer["type"] == "attention":
                assert names[f"{p}.talk"] == (a["heads"], a["heads"])
            else:
                r = m["right"]
                inner = r["heads"] * r["dim"]
                assert names[f"{p}.q.norm"] == (a["dim"],) and names[f"{p}.sink"] == (a["heads"],)
                assert names[f"l{i}.mix.right.w1"] == (r["rank"], width) and names[f"l{i}.mix.right.w2"] == (inner, r["rank"])
                assert names[f"l{i}.mix.right.u"] == (r["heads"], r["dim"]) and names[f"l{i}.mix.right.mu.w"] == (width,)
                assert names[f"l{i}.mix.right.o"] == (width, inner) and names[f"l{i}.mix.right.g"] == (inner, width)
            f = layer["mlp"]
            assert (f"l{i}.norm2" in names) == (f is not None) == (f"l{i}.ls2" in names) and names[f"l{i}.ls1"] == (width,)
            if f and f["kind"] == "moe":
                e = f["router"]["experts"]
                assert names[f"l{i}.mlp.router"] == (e, width) and f"l{i}.mlp.e0.gate" not in names
                assert names[f"l{i}.mlp.e{e - 1}.up"] == (f["expert"]["ff"], width) and f"l{i}.mlp.e{e}.up" not in names
            elif f:
                assert names[f"l{i}.mlp.gate"] == (f["ff"], width) and names[f"l{i}.mlp.down"] == (width, f["ff"])
        assert "head" not in names and names["embed"] == (raw["vocab"], width) and names["final.norm"] == (width,)


def test_a_layer_that_uses_anothers_tensors_runs_that_block_with_caches_of_its_own():
    from rust_mlx_b200.config import ReveraxConfig
    from rust_mlx_b200.registry import build_model_spec
    for raw, _ in tr.CONFIGS.values():
        spec = build_model_spec(ReveraxConfig.from_dict(raw))
        owners = [layer.get("weights_of", i) for i, layer in enumerate(raw["layers"])]
        own = sorted(set(owners))
        assert [c.layer for c in spec.schedule] == [own.index(o) for o in owners]
        ids = [i for c in spec.schedule for i in c.cache_ids()]
        assert ids == list(range(len(ids)))                  # every run has caches of its own
        kinds = [[s.kind for s in spec.blocks[c.layer].cache_specs()] for c in spec.schedule]
        for layer, k in zip(raw["layers"], kinds):
            assert k == (["paged"] if layer["type"] == "attention" else ["paged", "state", "state"])
        specs = spec.cache_specs()
        for c, layer in zip(spec.schedule, raw["layers"]):
            if layer["type"] == "parallel":
                paged, last, state = (specs[i] for i in c.cache_ids())
                left, right = layer["mixer"]["left"], layer["mixer"]["right"]
                assert paged.window == left.get("mask", {}).get("size", 0) and paged.kv_heads == left["kv_heads"]
                assert paged.head_dim >= max(left["dim"], left["vdim"])
                assert last.state_shape == (raw["width"],) and state.state_shape == (right["heads"], right["dim"], right["dim"])
                assert state.state_dtype == "float32"


def test_every_problem_of_a_configuration_is_reported_at_once():
    from rust_mlx_b200.config import ConfigError, ReveraxConfig
    raw = copy.deepcopy(tr.R1)
    raw["layers"][0]["mixer"]["kv_heads"] = 4           # 6 heads over 4
    raw["layers"][1]["mixer"]["left"]["rot"]["dims"] = 7
    raw["layers"][1]["mlp"]["router"]["top"] = 9
    raw["layers"][2]["weights_of"] = 0                   # another kind of layer
    raw["norm"]["groups"] = 5
    del raw["vocab"]
    with pytest.raises(ConfigError) as e:
        ReveraxConfig.from_dict(raw)
    assert "vocab" in str(e.value)
    raw["vocab"] = 10
    with pytest.raises(ConfigError) as e:
        ReveraxConfig.from_dict(raw)
    text = str(e.value)
    for piece in ("6 heads over 4", "dims must be even", "top 9 of 6", "same sizes and constants", "5 equal parts"):
        assert piece in text, piece
    bad = copy.deepcopy(tr.R1)
    bad["layers"][2]["weights_of"] = 2
    with pytest.raises(ConfigError):
        ReveraxConfig.from_dict(bad)
    bad = copy.deepcopy(tr.R1)
    bad["layers"][3]["type"] = "latent"
    with pytest.raises(ConfigError):
        ReveraxConfig.from_dict(bad)


def test_a_size_that_config_json_leaves_out_comes_from_the_checkpoint(tmp_path):
    from rust_mlx_b200.config import ReveraxConfig
    from rust_mlx_b200.registry import build_model_spec, load_config
    folder = tr.make_folder(tmp_path, tr.R1, seed=3)
    raw = json.load(open(f"{folder}/config.json"))
    for layer in raw["layers"]:
        if layer["type"] == "parallel":
            del layer["mixer"]["right"]["rank"]
    json.dump(raw, open(f"{folder}/config.json", "w"))
    cfg = load_config(folder)
    assert [layer.mixer.right.rank for layer in cfg.layers if layer.type == "parallel"] == [5, 5]
    names = {p.name: tuple(p.shape) for p in build_model_spec(cfg).all_param_specs()}
    assert names["l1.mix.right.w1"] == (5, 72)
    with pytest.raises(ValueError):         # without a checkpoint nothing gives the size
        build_model_spec(ReveraxConfig.from_dict(raw))


# ------------------------------------------------------------------------------------------------ the plain pieces

def test_plain_norm_in_groups():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.5, 0.5, 1.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 1.0, 1.0, 1.0, 3.0], dtype=torch.float64)
    got = plain.group_norm(x, w, 0.0, 2)
    a, b = math.sqrt(25.0 / 3), math.sqrt(1.5 / 3)
    assert torch.allclose(got, torch.tensor([[3 / a, 8 / a, 0.0, 0.5 / b, 0.5 / b, 3 / b]], dtype=torch.float64))
    assert torch.allclose(plain.group_norm(x, w, 0.0, 1), x / math.sqrt(x.pow(2).mean()) * w)


def test_plain_rotation_pairs_and_turning_back():
    x = torch.arange(1.0, 9.0, dtype=torch.float64).reshape(1, 1, 8)
    pos = torch.tensor([3])
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    halves = plain.turn(x, pos, 100.0, 4, False)
    assert torch.allclose(halves[0, 0, :4], torch.tensor([1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                                                           3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1)], dtype=torch.float64))
    assert torch.equal(halves[0, 0, 4:], x[0, 0, 4:])
    near = plain.turn(x, pos, 100.0, 4, True)
    assert torch.allclose(near[0, 0, :2], torch.tensor([1 * math.cos(a0) - 2 * math.sin(a0), 2 * math.cos(a0) + 1 * math.sin(a0)], dtype=torch.float64))
    assert torch.allclose(plain.turn(plain.turn(x, pos, 100.0, 8, False), pos, 100.0, 8, False, sign=-1.0), x)


def test_plain_window_and_sink():
    ok = plain.visible(5, 2)
    assert ok.int().tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 1, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 0, 1, 1]]
    assert plain.visible(3, 0).int().tolist() == [[1, 0, 0], [1, 1, 0], [1, 1, 1]]


def test_plain_time_mix_is_the_recurrence_written_out():
    """One head, one channel pair, by hand: o_1 = u k_1 v_1 r_1; o_2 = (k_1 v_1 + u k_2 v_2) r_2, S_2 = w_2 k_1 v_1 + k_2 v_2."""
    D = 2
    w = {f"m.mu.{s}": torch.zeros(D, dtype=torch.float64) for s in "rkvgw"}
    eye = torch.eye(D, dtype=torch.float64)
    w.update({"m.r": eye, "m.k": eye, "m.v": eye, "m.g": 50 * eye, "m.w1": torch.zeros(1, D, dtype=torch.float64),
              "m.w2": torch.zeros(D, 1, dtype=torch.float64), "m.w0": torch.tensor([0.0, 1.0], dtype=torch.float64),
              "m.u": torch.tensor([[0.5, 2.0]], dtype=torch.float64), "m.norm": torch.ones(D, dtype=torch.float64), "m.o": eye})
    h = torch.tensor([[1.0, 2.0], [3.0, 1.0]], dtype=torch.float64)
    states = []
    got = plain.time_mix(h, w, "m", {"heads": 1, "dim": 2}, 0.0, False, state_out=states)
    decay = torch.exp(-torch.exp(w["m.w0"]))
    k1v1 = h[0][:, None] * h[0][None, :]
    k2v2 = h[1][:, None] * h[1][None, :]
    o1 = (w["m.u"][0][:, None] * k1v1).T @ h[0]
    o2 = (k1v1 + w["m.u"][0][:, None] * k2v2).T @ h[1]
    want = torch.stack([o1, o2])
    want = want / want.pow(2).mean(-1, keepdim=True).sqrt()        # gate = silu(50 h) = 50 h for these inputs
    assert torch.allclose(got, want * (50 * h), rtol=1e-9)
    assert torch.allclose(states[0][0], decay[:, None] * k1v1 + k2v2)


def test_plain_experts_read_the_weighted_row():
    g = torch.Generator().manual_seed(0)
    w = {"f.router": torch.randn(3, 4, generator=g, dtype=torch.float64)}
    for e in range(3):
        w[f"f.e{e}.up"] = torch.randn(5, 4, generator=g, dtype=torch.float64)
        w[f"f.e{e}.down"] = torch.randn(4, 5, generator=g, dtype=torch.float64)
    h = torch.randn(6, 4, generator=g, dtype=torch.float64)
    got = plain.squared_relu_experts(h, w, "f", {"router": {"experts": 3, "top": 2}}, False)
    s = torch.sigmoid(h @ w["f.router"].T)
    want = torch.zeros_like(h)
    for t in range(6):
        for e in torch.topk(s[t], 2).indices.tolist():
            # relu(a)^2 of a row times s is s^2 times relu(a)^2 of the row: the weight enters squared, not once
            want[t] += s[t, e] ** 2 * (torch.relu(w[f"f.e{e}.up"] @ h[t]) ** 2 @ w[f"f.e{e}.down"].T)
    assert torch.allclose(got, want, rtol=1e-9)
