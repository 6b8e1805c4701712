"""Configuration surface: Hydra-style composition of the shipped YAML tree, overrides, group selection, typed views."""
import warnings

import pytest

from aeris_gb_b200.utils import config as C


def _compose(*overrides):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return C.compose("train", list(overrides))


@pytest.mark.parametrize("exp", ["train", "benchmark", "train_6h_hurricane", "b200_1p3b_wp8", "b200_1p3b_wp4_sp2",
                                 "b200_13b_pp2_wp2_sp2", "b200_wp_inference", "tiny_cpu"])
def test_every_shipped_experiment_composes_into_typed_configs(exp):
    cfg = _compose(f"experiment={exp}")
    m, o, d = C.model_config(cfg), C.optim_config(cfg), C.diffusion_config(cfg)
    assert m.n_layers == cfg.model.PP_stages - 2 and m.dim == cfg.model.dim and m.window == tuple(cfg.model.window_size)
    assert o.lr == cfg.optimizer.lr and tuple(o.betas) == tuple(cfg.optimizer.betas)
    assert d.sigma_data == cfg.model.get("sigma_data", 1.0)
    assert m.heads * m.head_dim > 0 and m.param_count() > 0 and m.flops_per_sample() > 0


def test_reference_train_experiment_values():
    cfg = _compose("experiment=train")
    m = C.model_config(cfg)
    assert (m.dim, m.heads, m.head_dim, m.mlp_dim, m.window, m.sublayers, m.n_layers) == (1536, 12, 128, 6144, (60, 60), 3, 8)
    assert cfg.model.SP == 12 and (cfg.model.WP_Y, cfg.model.WP_X) == (4, 4) and cfg.data.gas == 20
    o = C.optim_config(cfg)
    assert o.decay_policy == "custom_decay5" and o.grad_clip and o.grad_clip_max_norm == 20 and o.weight_decay == 0.2
    ch = C.channel_counts(cfg)
    assert ch["model_out"] in (69, 70) and ch["model_in"] == ch["model_out"] + ch["condition"]


def test_overrides_group_selection_and_nested_group_defaults():
    cfg = _compose("experiment=tiny_cpu", "model.dim=64", "trainer.benchmark_steps=3", "+model.extra_key=[1,2]",
                   "optimizer.lr=1e-3")
    assert cfg.model.dim == 64 and cfg.trainer.benchmark_steps == 3 and cfg.model.extra_key == [1, 2]
    assert cfg.optimizer.lr == pytest.approx(1e-3)
    cfg = _compose("data=era5-aurora")
    assert cfg.data.dataset.split == "train" and cfg.data.get("synthetic") is False
    cfg = _compose("optimizer=adam", "experiment=b200_wp_inference")
    assert str(cfg.optimizer.get("_target_")).endswith(("Adam", "AdamW"))


def test_model_tp_and_modes_reach_the_model_config():
    cfg = _compose("experiment=tiny_cpu", "model.TP=2", "model.rit=true", "model.diffusion=false", "model.emb_norm=true",
                   "model.act_ckpt=true", "model.shift_mode=none")
    m = C.model_config(cfg)
    assert m.tp == 2 and m.rit and not m.diffusion and m.emb_norm and m.oracle_checkpoint and m.shift_layers == "none"


def test_keys_without_effect_are_reported_once():
    C._warned = False
    with pytest.warns(UserWarning, match="accepted for compatibility"):
        C.compose("train", ["experiment=train"])
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        C.compose("train", ["experiment=train"])          # second composition: no second warning


def test_unknown_optimizer_target_is_refused():
    cfg = _compose("experiment=tiny_cpu", "optimizer._target_=torch.optim.SGD")
    with pytest.raises(ValueError, match="Adam"):
        C.optim_config(cfg)


def test_run_config_round_trip(tmp_path):
    cfg = _compose("experiment=tiny_cpu", "model.dim=96")
    C.save_run_config(cfg, tmp_path)
    back = C.load_run_config(tmp_path)
    assert back.model.dim == 96 and back.to_dict() == cfg.to_dict()


def test_a_group_file_may_build_on_a_sibling_of_its_group(tmp_path):
    """``defaults: [base]`` inside ``data/site.yaml`` merges ``data/base.yaml`` first, into the same package."""
    (tmp_path / "data").mkdir()
    (tmp_path / "train.yaml").write_text("defaults:\n  - _self_\n  - data: site\nseed: 1\n")
    (tmp_path / "data" / "base.yaml").write_text("workers: 8\ndataset:\n  root: null\n  split: train\n")
    (tmp_path / "data" / "site.yaml").write_text("defaults:\n  - base\ndataset:\n  root: /somewhere\n")
    cfg = C.compose("train", [], config_root=tmp_path)
    assert cfg.data.workers == 8 and cfg.data.dataset.root == "/somewhere" and cfg.data.dataset.split == "train"


def test_numbers_in_scientific_notation_without_a_dot_are_numbers(tmp_path):
    """``eps: 1e-08`` (as the reference's optimizer files write it) and ``optimizer.lr=1e-3`` on the command line."""
    (tmp_path / "optimizer").mkdir()
    (tmp_path / "train.yaml").write_text("defaults:\n  - _self_\n  - optimizer: adam\nseed: 1\n")
    (tmp_path / "optimizer" / "adam.yaml").write_text("lr: 1e-3\neps: 1e-08\nbetas: [0.9, 0.999]\n")
    cfg = C.compose("train", ["optimizer.lr=2e-4"], config_root=tmp_path)
    assert cfg.optimizer.eps == 1e-8 and cfg.optimizer.lr == 2e-4 and isinstance(cfg.optimizer.eps, float)
