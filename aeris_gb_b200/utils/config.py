"""Hydra-compatible configuration surface without Hydra/OmegaConf (neither is a dependency of this package).

Same key names at the global level as the reference's YAML tree (configs/train.yaml composing ``trainer/defaults``,
``optimizer/adamw`` and ``experiment/<name>``; keys listed in the reference at configs/experiment/train.yaml:1-86),
``key=value`` dotted overrides on the command line, ``${name}`` interpolation, and a ``.hydra/config.yaml`` snapshot in
the run directory so that the inference entry points can re-load it (reference: src/aeris/pp_generate.py:539,
src/aeris_wp_inference/inference.py:201). Keys that exist in the reference YAML but are never read by its code are
accepted and reported once (``UNREAD_KEYS``).
"""
from __future__ import annotations

import copy
import os
import re
import time
import warnings
from pathlib import Path
from typing import Any

import yaml

CONFIG_ROOT = Path(__file__).resolve().parent.parent.parent / "configs"

# Present in the reference YAML files, read by no reference code path (accept and warn).
UNREAD_KEYS = {
    "dry_run", "model.emb_init", "model.weight_init", "model.custom_decay2",
    "model.custom_decay3", "model.custom_decay4", "model.custom_decay6", "model.custom_high_wd", "model.P_mean",
    "model.P_std", "model.shift_size", "model.patch_size", "model.depth", "model.fp32_modulation",
    "data.res_fix",
    # read by the reference, without effect here: every rank loads its own block of a sample directly (no scatter, so
    # neither `wp_load` nor `gpu_datamovement` has anything to choose), attention is always the flash kernel, blocks are
    # always pre-norm, the clipping norm is the 2-norm, optimizer hyper-parameters always come from the configuration
    "data.wp_load", "model.gpu_datamovement", "model.attn_fn", "model.norm", "model.grad_clip_norm_type",
    "model.refresh_decay",
}


class Config(dict):
    """dict with attribute access (``cfg.model.dim``), recursively."""

    def __init__(self, d: dict | None = None):
        super().__init__()
        for k, v in (d or {}).items():
            self[k] = self._wrap(v)

    @classmethod
    def _wrap(cls, v):
        if isinstance(v, dict) and not isinstance(v, Config):
            return Config(v)
        if isinstance(v, list):
            return [cls._wrap(i) for i in v]
        return v

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e

    def __setattr__(self, k, v):
        self[k] = self._wrap(v)

    def get_path(self, path: str, default=None):
        cur: Any = self
        for part in path.split("."):
            if not isinstance(cur, dict) or part not in cur:
                return default
            cur = cur[part]
        return cur

    def set_path(self, path: str, value):
        cur = self
        parts = path.split(".")
        for part in parts[:-1]:
            if part not in cur or not isinstance(cur[part], dict):
                cur[part] = Config()
            cur = cur[part]
        cur[parts[-1]] = self._wrap(value)

    def to_dict(self) -> dict:
        def un(v):
            if isinstance(v, dict):
                return {k: un(x) for k, x in v.items()}
            if isinstance(v, list):
                return [un(x) for x in v]
            return v
        return un(self)


def _merge(dst: dict, src: dict) -> dict:
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _merge(dst[k], v)
        else:
            dst[k] = copy.deepcopy(v)
    return dst


def _load_yaml(path: Path) -> dict:
    with open(path) as f:
        return _fix_floats(yaml.safe_load(f) or {})


_SCI = re.compile(r"^[+-]?\d+(\.\d*)?[eE][+-]?\d+$")


def _fix_floats(node):
    """YAML 1.1 reads ``1e-08`` (no dot in the mantissa, as the reference's optimizer files write it) as a string."""
    if isinstance(node, dict):
        return {k: _fix_floats(v) for k, v in node.items()}
    if isinstance(node, list):
        return [_fix_floats(v) for v in node]
    if isinstance(node, str) and _SCI.match(node):
        return float(node)
    return node


def _parse_value(s: str):
    try:
        v = yaml.safe_load(s)
    except yaml.YAMLError:
        return s
    if isinstance(v, str):          # YAML 1.1 reads `1e-3` (no dot) as a string; overrides mean the number
        try:
            return float(v)
        except ValueError:
            pass
    return v


def compose(config_name: str = "train", overrides: list[str] | None = None, config_root: Path | None = None) -> Config:
    """Hydra-style composition: ``<root>/<config_name>.yaml`` with a ``defaults`` list of ``group: option`` entries
    (each merged under the group key unless the file starts with ``# @package _global_``; experiment files are
    global, as the reference intends: the keys its code reads are top-level), then dotted overrides. An override
    ``group=option`` for a defaults group re-selects the option (``experiment=benchmark``)."""
    root = Path(config_root or CONFIG_ROOT)
    overrides = list(overrides or [])
    main = _load_yaml(root / f"{config_name}.yaml")
    defaults = main.pop("defaults", [])
    main.pop("hydra", None)
    group_sel = {}
    for ov in list(overrides):
        k, _, v = ov.partition("=")
        if (root / k).is_dir() and "." not in k:
            group_sel[k] = v
            overrides.remove(ov)
    cfg: dict = {}
    self_merged = False
    for entry in defaults:
        if entry == "_self_":
            _merge(cfg, main)
            self_merged = True
            continue
        (group, option), = entry.items()
        option = group_sel.get(group, option)
        path = root / group / f"{option}.yaml"
        text = path.read_text()
        body = _fix_floats(yaml.safe_load(text) or {})
        nested = body.pop("defaults", None) or []
        m = re.match(r"\s*#\s*@package\s+(\S+)", text)
        package = m.group(1) if m else group
        # a group file may list siblings of its own group that it builds on (`defaults: [defaults]` in
        # configs/data/era5-aurora.yaml): they are merged first, into the same package
        for sib in nested:
            if isinstance(sib, str) and sib != "_self_" and (root / group / f"{sib}.yaml").exists():
                sib_body = _load_yaml(root / group / f"{sib}.yaml")
                sib_body.pop("defaults", None)
                _merge(cfg if package == "_global_" else cfg.setdefault(package, {}), sib_body)
        if package == "_global_":
            _merge(cfg, body)
        else:
            _merge(cfg.setdefault(package, {}), body)
    if not self_merged:
        _merge(cfg, main)
    out = Config(cfg)
    for ov in overrides:
        k, _, v = ov.partition("=")
        out.set_path(k.lstrip("+"), _parse_value(v))
    _interpolate(out, out)
    _warn_unread(out)
    return out


def _interpolate(node, root: Config):
    if isinstance(node, dict):
        for k, v in node.items():
            if isinstance(v, str) and "${" in v:
                node[k] = re.sub(r"\$\{([^}:]+)\}", lambda m: str(root.get_path(m.group(1), m.group(0))), v)
            else:
                _interpolate(v, root)
    elif isinstance(node, list):
        for v in node:
            _interpolate(v, root)


_warned = False


def _warn_unread(cfg: Config):
    global _warned
    if _warned:
        return
    present = [k for k in UNREAD_KEYS if cfg.get_path(k) is not None]
    if present:
        _warned = True
        warnings.warn("config keys accepted for compatibility but not used: " + ", ".join(sorted(present)))


def run_dir(cfg: Config, base: str = "results") -> Path:
    """``results/<experiment_name>/<timestamp>`` (reference: configs/train.yaml:11-15)."""
    return Path(base) / str(cfg.get("experiment_name", "run")) / time.strftime("%Y%m%d_%H%M%S")


def save_run_config(cfg: Config, directory: str | os.PathLike) -> Path:
    d = Path(directory) / ".hydra"
    d.mkdir(parents=True, exist_ok=True)
    p = d / "config.yaml"
    with open(p, "w") as f:
        yaml.safe_dump(cfg.to_dict(), f, sort_keys=False)
    return p


def load_run_config(checkpoint_dir: str | os.PathLike) -> Config:
    return Config(_load_yaml(Path(checkpoint_dir) / ".hydra" / "config.yaml"))


# ---------------------------------------------------------------------------------------------- typed views
def channel_counts(cfg: Config) -> dict:
    """Channel wiring of the reference (src/aeris/train.py:109-128): dataset channels, condition, label, model in/out."""
    m = cfg.model
    if m.get("enhanced_channels4"):
        return dict(dataset=73, condition=74, label=70, model_in=144, model_out=70)
    if m.get("enhanced_channels3"):
        return dict(dataset=72, condition=72, label=69, model_in=141, model_out=69)
    c = int(m.get("channels", 69))
    cond = int(m.get("condition_channels", c))
    if m.get("diffusion", True):
        return dict(dataset=c, condition=cond, label=c, model_in=c + cond, model_out=c)
    return dict(dataset=c, condition=0, label=c, model_in=c, model_out=c)


def model_config(cfg: Config):
    from ..models.aeris import AerisConfig
    m = cfg.model
    ch = channel_counts(cfg)
    img = tuple(m.get("img", (720, 1440)))
    return AerisConfig(
        img=img, window=tuple(m.window_size), in_channels=int(m.get("model_in_channels", ch["model_in"])),
        out_channels=int(m.get("model_out_channels", ch["model_out"])), dim=m.dim, heads=m.heads,
        head_dim=m.head_dim, mlp_dim=m.mlp_dim, n_layers=m.PP_stages - 2, sublayers=m.get("sublayers", 1),
        layerwise_t_emb=bool(m.get("layerwise_t_emb", False)),
        after_mod_norm=bool(m.get("layerwise_t_emb_after_mod_norm", False)),
        max_period=float(m.get("sinusoidal_emb_max_period", 10000)), wp=(m.get("WP_Y", 1), m.get("WP_X", 1)),
        chunk_windows=int(m.get("chunk_windows", 64)), norm_eps=m.get("norm_eps"),
        shift_layers=m.get("shift_mode", "odd"), diffusion=bool(m.get("diffusion", True)),
        rit=bool(m.get("rit", False)), emb_norm=bool(m.get("emb_norm", False)) and bool(m.get("rit", False)),
        tp=int(m.get("TP", 1)),
        # model.act_ckpt: per-block recompute on the PyTorch (CPU / oracle) path; the CUDA blocks always keep only
        # their input
        oracle_checkpoint=bool(m.get("act_ckpt", False)))


def optim_config(cfg: Config):
    from ..engine.optim import OptimConfig
    t, o, m = cfg.trainer, cfg.optimizer, cfg.model
    policy = "custom_decay5" if m.get("custom_decay5") else ("custom_decay" if m.get("custom_decay") else "all")
    target = str(o.get("_target_", "torch.optim.AdamW"))
    if target.rsplit(".", 1)[-1] not in ("AdamW", "Adam"):
        raise ValueError(f"optimizer._target_ = {target}: the fused update implements Adam / AdamW")
    if target.endswith(".Adam") and float(o.weight_decay) != 0.0:
        # torch.optim.Adam adds weight_decay * w to the gradient (L2); the fused kernels decay the weights directly
        warnings.warn("optimizer._target_ is torch.optim.Adam with a non-zero weight_decay: the decoupled (AdamW) "
                      "form of the decay is applied")
    return OptimConfig(
        lr=o.lr, betas=tuple(o.betas), eps=o.eps, weight_decay=o.weight_decay, decay_policy=policy,
        grad_clip=bool(m.get("grad_clip", False)), grad_clip_max_norm=float(m.get("grad_clip_max_norm", 1.0)),
        total_img=int(t.total_kimg * 1000), lr_rampup_img=int(t.lr_rampup_kimg * 1000),
        lr_min_factor=t.lr_min_factor, lr_rampdown_start=int(t.get("lr_rampdown_start", 10 ** 11)),
        lr_rampdown_length=int(t.get("lr_rampdown_length", 1)),
        lr_rampdown_ema_min_ratio=float(t.get("lr_rampdown_ema_min_ratio", 1.0)),
        ema_halflife_img=int(t.ema_halflife_kimg * 1000), ema_rampup_ratio=t.get("ema_rampup_ratio", 0.05),
        use_ema=not bool(m.get("dist_optimizer", False)))


def diffusion_config(cfg: Config):
    from ..engine.trainer import DiffusionConfig
    m = cfg.model
    return DiffusionConfig(sigma_data=m.get("sigma_data", 1.0), sigma_min=m.get("sigma_min", 0.2),
                           sigma_max=m.get("sigma_max", 500), w_lat_add=m.get("w_lat_add", 0.0),
                           noise_law=m.get("noise_law", "loguniform"), cond_channels=channel_counts(cfg)["condition"])
