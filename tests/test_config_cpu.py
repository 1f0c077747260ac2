"""Config system: YAML env substitution and extends, presets, experiment resolution, CLI overrides, patches."""
import os

import pytest
import yaml

from primus_b200.core.config import experiment, overrides, presets, yaml_loader
from primus_b200.core.config.merge import deep_merge, merge_without_override
from primus_b200.core.patches import registry as R


def test_env_substitution_and_coercion(tmp_path, monkeypatch):
    p = tmp_path / "a.yaml"
    p.write_text("a: ${PB_T_INT:7}\nb: ${PB_T_BOOL:false}\nc: pre-${PB_T_STR:x}-post\nd: ${PB_T_F:1.5}\ne: 12\n")
    monkeypatch.setenv("PB_T_STR", "mid")
    d = yaml_loader.load_yaml(p)
    assert d == {"a": 7, "b": False, "c": "pre-mid-post", "d": 1.5, "e": 12}
    monkeypatch.setenv("PB_T_INT", "9")
    assert yaml_loader.load_yaml(p)["a"] == 9


def test_required_env_raises(tmp_path):
    p = tmp_path / "a.yaml"
    p.write_text("a: ${PB_SURELY_UNSET_VAR}\n")
    with pytest.raises(KeyError):
        yaml_loader.load_yaml(p)


def test_extends_chain_and_cycle(tmp_path):
    (tmp_path / "base.yaml").write_text("x: 1\nnested: {a: 1, b: 2}\n")
    (tmp_path / "mid.yaml").write_text("extends: base.yaml\ny: 2\nnested: {b: 3}\n")
    (tmp_path / "top.yaml").write_text("extends: [mid.yaml]\nx: 5\n")
    d = yaml_loader.load_yaml(tmp_path / "top.yaml")
    assert d == {"x": 5, "y": 2, "nested": {"a": 1, "b": 3}}
    (tmp_path / "c1.yaml").write_text("extends: c2.yaml\n")
    (tmp_path / "c2.yaml").write_text("extends: c1.yaml\n")
    with pytest.raises(ValueError):
        yaml_loader.load_yaml(tmp_path / "c1.yaml")


def test_merge_helpers():
    assert deep_merge({"a": {"b": 1}}, {"a": {"c": 2}}) == {"a": {"b": 1, "c": 2}}
    with pytest.raises(KeyError):
        merge_without_override({"a": 1}, {"a": 2})


def test_cli_overrides_forms():
    o = overrides.parse_cli_overrides(["a=1", "--b=2.5", "--c", "hello", "--flag", "x.y.z=[1,2]", "--n", "none"])
    assert o == {"a": 1, "b": 2.5, "c": "hello", "flag": True, "x": {"y": {"z": [1, 2]}}, "n": None}
    with pytest.raises(ValueError):
        overrides.parse_cli_overrides(["positional"])


def test_preset_traversal_guard():
    with pytest.raises((ValueError, FileNotFoundError)):
        presets.preset_path("../../../etc/passwd", "models")
    assert presets.load_preset("megatron/llama3.1_8B.yaml", "models", "megatron")["num_layers"] == 32


def test_every_model_preset_builds_a_config():
    from primus_b200.models.config import TransformerConfig

    root = presets.CONFIG_ROOT / "models"
    names = sorted(p.name for p in root.glob("*.yaml"))
    assert len(names) >= 30
    for n in names:
        cfg = TransformerConfig.from_dict(presets.load_preset(n, "models"))
        assert cfg.num_parameters() > 0, n
    c8 = TransformerConfig.from_dict(presets.load_preset("llama3.1_8B", "models"))
    assert abs(c8.num_parameters() / 1e9 - 8.03) < 0.02
    lite = TransformerConfig.from_dict(presets.load_preset("deepseek_v2_lite", "models"))
    assert 15.0 < lite.num_parameters() / 1e9 < 16.5 and lite.moe_layer_pattern[:2] == [0, 1]
    q = TransformerConfig.from_dict(presets.load_preset("qwen3_30B_A3B", "models"))
    assert 29.5 < q.num_parameters() / 1e9 < 31.5


def test_experiment_resolution_and_alias(tmp_path, monkeypatch):
    exp = tmp_path / "exp.yaml"
    exp.write_text(yaml.safe_dump({
        "work_group": "wg", "user_name": "u", "exp_name": "e", "workspace": str(tmp_path / "out"),
        "env": {"PB_TEST_ENV_BLOCK": 3},
        "modules": {"pre_trainer": {"framework": "megatron", "config": "pre_trainer.yaml", "model": "llama_tiny.yaml",
                                    "overrides": {"train_iters": 3, "lr": 0.5}},
                    "not_a_module": {"x": 1}}}))
    e = experiment.load_experiment(str(exp), {"lr": 0.25, "seq_length": 64}, "pre_trainer")
    m = e.module("pre_trainer")
    assert m.params["train_iters"] == 3 and m.params["lr"] == 0.25 and m.params["seq_length"] == 64
    assert m.params["num_layers"] == 4 and m.trainer_class == "PretrainTrainer"
    assert e.module("post_trainer") is m  # alias
    assert "not_a_module" not in e.modules
    assert e.exp_root_path.endswith(os.path.join("out", "wg", "u", "e"))
    experiment.apply_env_block(e)
    assert os.environ["PB_TEST_ENV_BLOCK"] == "3"
    bad = tmp_path / "bad.yaml"
    bad.write_text("work_group: x\n")
    with pytest.raises(KeyError):
        experiment.load_experiment(str(bad))


def test_example_configs_all_load():
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "configs")
    files = [f for f in os.listdir(root) if f.endswith(".yaml")]
    assert files
    for f in files:
        e = experiment.load_experiment(os.path.join(root, f))
        assert e.modules, f


def test_patch_registry_phases_priority_selection(monkeypatch):
    reg = R.PatchRegistry()
    calls = []
    R.register_patch("t.b", "build_args", priority=20, registry=reg)(lambda c: calls.append("b"))
    R.register_patch("t.a", "build_args", priority=10, registry=reg)(lambda c: calls.append("a"))
    R.register_patch("t.cond", "build_args", condition=lambda c: c.get_param("x") == 1, registry=reg)(
        lambda c: calls.append("cond"))
    R.register_patch("t.setup", "setup", registry=reg)(lambda c: calls.append("setup"))
    ctx = R.PatchContext(phase="build_args", params={"x": 0})
    assert R.run_patches("build_args", ctx, registry=reg) == ["t.a", "t.b"] and calls == ["a", "b"]
    ctx.params["x"] = 1
    assert "t.cond" in R.run_patches("build_args", ctx, registry=reg, dry_run=True)
    monkeypatch.setenv("PRIMUS_PATCHES", "none")
    assert R.run_patches("build_args", ctx, registry=reg) == []
    monkeypatch.setenv("PRIMUS_PATCHES", "t.b")
    assert R.run_patches("build_args", ctx, registry=reg) == ["t.b"]
    with pytest.raises(ValueError):
        reg.register(R.FunctionPatch("t.a", lambda c: None, "build_args"))
    with pytest.raises(ValueError):
        reg.register(R.FunctionPatch("t.z", lambda c: None, "nope"))


def test_version_ranges():
    assert R.version_in_range("0.12.1", ">=0.8,<0.13")
    assert not R.version_in_range("0.13.0", ">=0.8,<0.13")
    assert R.version_in_range("1.2.7", "==1.2.*") and not R.version_in_range("1.3.0", "==1.2.*")


def test_builtin_build_args_patches(tmp_path):
    from primus_b200.core.patches import builtin  # noqa: F401

    params = {"mock_data": True, "vocab_size": None, "data_path": "a b", "num_experts": 4, "num_layers": 3,
              "moe_layer_freq": "([0]*1+[1]*2)", "tensor_model_parallel_size": 1, "sequence_parallel": True,
              "save_interval": 5, "save": None}
    ctx = R.PatchContext(phase="build_args", params=params, extra={"exp_root_path": str(tmp_path)})
    R.run_patches("build_args", ctx)
    assert params["tokenizer_type"] == "NullTokenizer" and params["vocab_size"] == 131072
    assert params["moe_layer_freq"] == [0, 1, 1] and params["sequence_parallel"] is False
    assert params["save"].endswith("checkpoints")
    bad = R.PatchContext(phase="build_args", params={"use_turbo_mega_moe": True, "expert_model_parallel_size": 16})
    with pytest.raises(ValueError):
        R.run_patches("build_args", bad)


def test_schema_check_flags_unknown_keys_with_suggestions(tmp_path):
    from primus_b200.core.config import schema_check
    from primus_b200.core.config.experiment import load_experiment

    known = schema_check.known_keys("pre_trainer.yaml", "llama3.1_8B.yaml")
    assert {"micro_batch_size", "num_layers", "use_turbo_mega_moe", "moe_fused_capacity_factor"} <= known
    recs = schema_check.check_keys(["micro_batch_sizes", "num_layers", "totally_new_key"], known)
    assert [r["key"] for r in recs] == ["micro_batch_sizes", "totally_new_key"]
    assert "micro_batch_size" in recs[0]["suggestions"] and recs[1]["suggestions"] == []
    cfg = tmp_path / "exp.yaml"
    cfg.write_text(
        "work_group: g\nuser_name: u\nexp_name: e\nworkspace: " + str(tmp_path) + "\n"
        "modules:\n  pre_trainer:\n    framework: primus_b200\n    config: pre_trainer.yaml\n    model: llama3.1_8B.yaml\n"
        "    overrides:\n      train_iter: 5\n      micro_batch_size: 1\n")
    exp = load_experiment(str(cfg), {"global_batchsize": 8}, "pre_trainer")
    joined = " ".join(exp.schema_findings)
    assert "train_iter" in joined and "train_iters" in joined and "global_batchsize" in joined
    assert "micro_batch_size'" not in joined


def test_example_configs_pass_the_schema_check():
    """No example recipe uses a key that neither the model / trainer configs nor the presets know."""
    import yaml

    from primus_b200.core.config import schema_check

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "configs")
    files = [os.path.join(d, f) for d, _, fs in os.walk(root) for f in fs if f.endswith(".yaml")]
    assert len(files) > 100
    for f in sorted(files):
        with open(f) as fh:
            raw = yaml.safe_load(fh)
        assert schema_check.check_experiment(raw) == [], f


def test_recipe_book_plans_are_legal_and_fit():
    """Every generated recipe loads, names a plan that the legality check accepts on its node count, and fits the
    memory of the part according to the projection that the generator used."""
    import re

    from primus_b200.core.config.presets import load_preset
    from primus_b200.models.config import TransformerConfig
    from primus_b200.tools import recipes
    from primus_b200.tools.projection.memory import ParallelPlan, project_memory

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "configs", "b200")
    files = sorted(f for f in os.listdir(root) if f.endswith(".yaml"))
    # one BF16 and one MXFP8 recipe per model, except those the index lists as not fitting
    index = open(os.path.join(root, "index.md")).read()
    for m in recipes.model_names():
        for prec in ("BF16", "MXFP8"):
            assert f"{m}-{prec}-pretrain.yaml" in files or f"{m} ({prec})" in index, (m, prec)
    for f in files:
        head = open(os.path.join(root, f)).readline()
        nodes = int(re.search(r"(\d+) node", head).group(1))
        e = experiment.load_experiment(os.path.join(root, f))
        ov = e.modules["pre_trainer"].params
        g = lambda k, d=1: int(ov.get(k) or d)
        d = dict(load_preset(f.split("-")[0], "models"))
        cfg = TransformerConfig.from_dict(d)
        plan = ParallelPlan(world=8 * nodes, tp=g("tensor_model_parallel_size"), pp=g("pipeline_model_parallel_size"),
                            cp=g("context_parallel_size"), ep=g("expert_model_parallel_size"),
                            vpp=g("virtual_pipeline_model_parallel_size"), micro_batch=g("micro_batch_size"),
                            global_batch=g("global_batch_size"), seq=g("seq_length"),
                            recompute_layers=g("recompute_num_layers", 0), sequence_parallel=g("tensor_model_parallel_size") > 1,
                            fused_tp=g("tensor_model_parallel_size") > 1)
        assert plan.validate(cfg) == [], (f, plan.validate(cfg))
        assert project_memory(cfg, plan)["peak_gb"] <= 180.0, f
        if cfg.num_layers % (plan.pp * plan.vpp):
            assert g("decoder_last_pipeline_num_layers", 0) == plan.last_stage_layers(cfg.num_layers), f


def test_every_preset_key_is_read_or_declared_inert():
    """No key may parse and then silently do nothing: a key carried by a module / model preset is a field of the two
    config dataclasses, is consumed somewhere in the package (looked up by name as a quoted string or read as an
    attribute in the Python sources; a mention in a comment or a method of the same name does not count), or is listed
    in ``schema_check.INERT_KEYS`` (setting those is reported)."""
    import dataclasses
    import glob
    import os
    import re

    from primus_b200.core.config import schema_check
    from primus_b200.core.config.presets import load_preset
    from primus_b200.engine.trainer import TrainConfig
    from primus_b200.models.config import TransformerConfig

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "primus_b200")
    keys = set()
    for kind in ("modules", "models"):
        for f in glob.glob(os.path.join(root, "configs", kind, "*.yaml")):
            keys |= set(load_preset(os.path.basename(f), kind))
    fields = {f.name for f in dataclasses.fields(TransformerConfig)} | {f.name for f in dataclasses.fields(TrainConfig)}
    src = ""
    for f in glob.glob(os.path.join(root, "**", "*.py"), recursive=True):
        if not f.endswith(os.path.join("config", "schema_check.py")):
            src += open(f).read()
    words = set(re.findall(r"[\"']([A-Za-z_][A-Za-z0-9_]*)[\"']", src)) | set(re.findall(r"\.([A-Za-z_][A-Za-z0-9_]*)\b(?!\()", src))
    orphan = sorted(k for k in keys if k not in fields and k not in schema_check.EXTRA_KNOWN and k not in words
                    and k not in schema_check.INERT_KEYS)
    assert not orphan, f"preset keys that nothing reads and that are not declared inert: {orphan}"
    stale = sorted(k for k in schema_check.INERT_KEYS if k in fields)
    assert not stale, f"declared inert but now a config field: {stale}"


def test_inert_key_is_reported(tmp_path):
    from primus_b200.core.config import schema_check

    msgs = schema_check.check_inert({"normalization": "LayerNorm", "lr": 1e-3}, "pre_trainer.yaml", "llama3.1_8B.yaml")
    assert len(msgs) == 1 and "normalization" in msgs[0] and "no effect" in msgs[0]
    assert schema_check.check_inert({"normalization": "RMSNorm"}, "pre_trainer.yaml", "llama3.1_8B.yaml") == []
    assert schema_check.check_inert({"hidden_dropout": 0.1}, "pre_trainer.yaml", "llama3.1_8B.yaml") == []   # acted on
