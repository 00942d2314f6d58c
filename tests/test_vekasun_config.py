"""Vekasun's configuration on the CPU: reading config.json, refusing what cannot run, the plan of
parts and the order of layer runs, and the tensors the plan asks for."""

import copy

import pytest

import plain_vekasun as PV
import vekasun_configs as VC


def parse(cfg):
    from ninfer_amd_mi50_b200.engine.loading import build_model
    return build_model(cfg)


@pytest.mark.parametrize("name", sorted(VC.CONFIGS))
def test_plan_follows_the_configuration(name):
    cfg, _ = VC.CONFIGS[name]
    typed, model = parse(cfg)
    assert (typed.vocab, typed.width, typed.eps, typed.logit_scale) == (cfg["vocab"], cfg["width"], cfg["norm"]["eps"], cfg["logit_scale"])
    runs = PV.layer_runs(cfg)
    assert typed.runs() == runs
    assert [c.layer for c in model.order] == [i for i, _ in runs]
    assert sorted(c.cache for c in model.order) == list(range(len(runs)))
    assert model.plan.logit_scale == cfg["logit_scale"]
    specs = {s.name: s.shape for s in model.tensor_specs()}
    W = cfg["width"]
    assert specs["embed"] == (cfg["vocab"], W) and specs["head"] == (cfg["vocab"], W) and specs["final.norm"] == (W,)
    assert ("loop.step" in specs) == ("loop" in cfg and cfg["loop"]["stop"] > cfg["loop"]["start"])
    for i, L in enumerate(cfg["layers"]):
        m = L["mixer"]
        assert specs[f"l{i}.norm1"] == (W,)
        assert (f"l{i}.norm2" in specs) == (L["mlp"] is not None)
        if L["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            assert specs[f"l{i}.mix.in"] == (2 * inner + 2 * gn + m["heads"], W)
            assert specs[f"l{i}.mix.conv"] == (inner + 2 * gn, m["conv"]) and specs[f"l{i}.mix.conv.b"] == (inner + 2 * gn,)
            assert specs[f"l{i}.mix.norm"] == (inner,) and specs[f"l{i}.mix.o"] == (W, inner)
            assert specs[f"l{i}.mix.A_log"] == specs[f"l{i}.mix.D"] == specs[f"l{i}.mix.dt_bias"] == (m["heads"],)
        else:
            H = m["heads"]
            assert specs[f"l{i}.mix.dq"] == (m["q_rank"], W) and specs[f"l{i}.mix.uq"] == (H * (m["dim"] + m["rot_dim"]), m["q_rank"])
            assert specs[f"l{i}.mix.dkv"] == (m["kv_rank"] + m["rot_dim"], W) and specs[f"l{i}.mix.dkv.norm"] == (m["kv_rank"],)
            assert specs[f"l{i}.mix.uk"] == (H * m["dim"], m["kv_rank"]) and specs[f"l{i}.mix.uv"] == (H * m["vdim"], m["kv_rank"])
            assert specs[f"l{i}.mix.sink"] == (H,) and specs[f"l{i}.mix.g"] == (H * m["vdim"], W) and specs[f"l{i}.mix.o"] == (W, H * m["vdim"])
        if L["mlp"] is not None:
            ff, E = L["mlp"]["expert"]["ff"], L["mlp"]["router"]["experts"]
            assert specs[f"l{i}.mlp.router"] == (E, W)
            assert specs[f"l{i}.mlp.e{E - 1}.gate"] == (ff, W) and specs[f"l{i}.mlp.e0.down"] == (W, ff)
            assert f"l{i}.mlp.e{E}.gate" not in specs


def test_a_cache_row_holds_the_latent_and_the_rotated_key_and_state_is_fixed():
    cfg, _ = VC.CONFIGS["looped"]
    typed, model = parse(cfg)
    runs = PV.layer_runs(cfg)
    for (i, _), cs, ss in zip(runs, model.cache_specs(), model.state_specs()):
        m = cfg["layers"][i]["mixer"]
        if cfg["layers"][i]["type"] == "latent_attention":
            assert ss is None and cs.row_width == m["kv_rank"] + m["rot_dim"] and cs.kind == "full"
        else:
            channels = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
            assert cs is None and ss.shape == ((m["conv"] - 1) * channels + m["heads"] * m["vdim"] * m["state"],)


def test_what_cannot_run_is_refused():
    from ninfer_amd_mi50_b200.config.model_config import ConfigError
    base, _ = VC.CONFIGS["looped"]

    def broken(change):
        c = copy.deepcopy(base)
        change(c)
        with pytest.raises(ConfigError):
            parse(c)

    broken(lambda c: c["layers"][0].update(type="convolution"))
    broken(lambda c: c["layers"][0]["mixer"].pop("state"))
    broken(lambda c: c["layers"][0]["mixer"].update(groups=4))                 # 6 heads, 4 groups
    broken(lambda c: c["layers"][0]["mixer"].update(norm_groups=7))
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7))
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=32))           # more than the rotated slice
    broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=9))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="dense"))
    broken(lambda c: c["loop"].update(stop=9))
    broken(lambda c: c["loop"].update(times=0))
    broken(lambda c: c.pop("norm"))
    broken(lambda c: c.update(layers=[]))
    broken(lambda c: c.update(architecture="Nobody"))


def test_the_architecture_is_found_under_either_key():
    from ninfer_amd_mi50_b200.registry import architecture_of
    cfg, _ = VC.CONFIGS["straight"]
    assert architecture_of(cfg).name == "Vekasun"
    assert architecture_of({"architectures": ["Vekasun"]}).name == "Vekasun"


def test_random_model_folder_round_trip(tmp_path):
    cfg, seed = VC.CONFIGS["one_pass"]
    d = VC.write_folder(cfg, seed, str(tmp_path / "m"))
    c, w = VC.read_folder(d)
    typed, model = parse(c)
    assert set(w) == {s.name for s in model.tensor_specs()}
    lg = PV.forward(c, w, [3, 1, 4, 1, 5, 9, 2, 6])
    assert lg.shape == (8, cfg["vocab"]) and bool(lg.isfinite().all())
