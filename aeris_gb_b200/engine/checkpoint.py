"""Checkpoint IO in the reference's on-disk format.

Training writes one file per *logical* pipeline stage, ``checkpoint_PP{stage}.pth`` (plus ``it_{it}_checkpoint_PP{stage}
.pth`` every 1000 iterations), each a dict with ``cur_nimg``, ``model_state_dict`` (device-dtype copy),
``main_model_state_dict`` (fp32 master), ``optimizer_state_dict`` and ``ema_state_dict``
(src/aeris/parallelism/parallel_engine.py:1119-1160). Files are loaded with ``weights_only=True``. Because files are
per logical stage they do not depend on how many physical pipeline ranks wrote them.

Inference reads the per-stage files into one monolithic model (``input_stage.* / layers.{i}.* / output_stage.*``),
always from ``ema_state_dict`` (src/aeris_wp_inference/model.py:479-495).
"""
from __future__ import annotations

import os

import torch


def _fname(directory, stage: int, it: int | None = None) -> str:
    name = f"checkpoint_PP{stage}.pth" if it is None else f"it_{it}_checkpoint_PP{stage}.pth"
    return os.path.join(directory, name)


def _n_logical(module) -> int:
    return module.cfg.n_layers + 2


def _stage_ids(module) -> list[int]:
    return list(getattr(module, "stage_ids", range(_n_logical(module))))


def _key_for(module, stage: int, key: str) -> str:
    if stage == 0:
        return f"input_stage.{key}"
    if stage == _n_logical(module) - 1:
        return f"output_stage.{key}"
    return f"layers.{stage - 1}.{key}"


def _logical(module, sd: dict) -> dict[int, dict]:
    """Splits a state dict with ``input_stage.* / layers.{i}.* / output_stage.*`` keys (PipelineStage and AerisModel
    both use them) into one dict per logical pipeline stage with the reference's per-stage key names."""
    out: dict[int, dict] = {}
    last = _n_logical(module) - 1
    for k, v in sd.items():
        if k.startswith("input_stage."):
            out.setdefault(0, {})[k[len("input_stage."):]] = v
        elif k.startswith("output_stage."):
            out.setdefault(last, {})[k[len("output_stage."):]] = v
        elif k.startswith("layers."):
            _, idx, rest = k.split(".", 2)
            out.setdefault(int(idx) + 1, {})[rest] = v
    return out


def _integrity(ckpt: dict) -> dict:
    """Per-tensor float64 sums of every state-dict section: an extra key that the reference's loaders ignore and that
    lets :func:`load_stage_checkpoint` reject a file whose payload was damaged (torch.load does not verify it)."""
    out = {}
    sections = {n: ckpt.get(n, {}) for n in ("model_state_dict", "main_model_state_dict", "ema_state_dict")}
    osd = ckpt.get("optimizer_state_dict", {})
    sections["optimizer/exp_avg"] = osd.get("exp_avg", {})
    sections["optimizer/exp_avg_sq"] = osd.get("exp_avg_sq", {})
    for section, sd in sections.items():
        for k, t in sd.items():
            if torch.is_tensor(t) and t.dtype.is_floating_point:
                out[f"{section}/{k}"] = float(torch.nan_to_num(t.double()).sum())
    return out


def save_stage_checkpoint(directory: str, module, opt, it: int | None = None, write: bool = True) -> list[str]:
    """``module``: a PipelineStage or a whole AerisModel; ``opt``: the optimizer built on it (FlatOptimizer, or the
    sharded optimizer, whose state dicts are gathered collectively: then every rank of its group calls this function
    and ``write`` is True on one of them). Writes one file per logical stage the module holds."""
    if write:
        os.makedirs(directory, exist_ok=True)
    model_sd = _logical(module, module.state_dict())
    master = _logical(module, dict(opt.master_state_dict()))
    ema = _logical(module, dict(opt.ema_state_dict())) if opt.cfg.use_ema else {}
    osd = opt.state_dict()
    exp_avg = _logical(module, osd["exp_avg"])
    exp_avg_sq = _logical(module, osd["exp_avg_sq"])
    written = []
    if not write:
        return written
    for stage, sd in model_sd.items():
        full_master = {k: v.detach().float().cpu().clone() for k, v in sd.items()}     # buffers and frozen params too
        full_master.update({k: v.detach().cpu().clone() for k, v in master.get(stage, {}).items()})
        ckpt = {
            "cur_nimg": int(opt.cur_nimg),
            "model_state_dict": {k: v.detach().cpu().clone() for k, v in sd.items()},
            "main_model_state_dict": full_master,
            "optimizer_state_dict": {"step": int(opt.step_count),
                                     "exp_avg": {k: v.cpu() for k, v in exp_avg.get(stage, {}).items()},
                                     "exp_avg_sq": {k: v.cpu() for k, v in exp_avg_sq.get(stage, {}).items()}},
        }
        if opt.cfg.use_ema:
            full_ema = dict(full_master)
            full_ema.update({k: v.detach().cpu().clone() for k, v in ema.get(stage, {}).items()})
            ckpt["ema_state_dict"] = full_ema
        ckpt["integrity"] = _integrity(ckpt)
        path = _fname(directory, stage, it)
        tmp = path + ".tmp"
        torch.save(ckpt, tmp)
        os.replace(tmp, path)       # a crash mid-write never leaves a truncated checkpoint under the final name
        written.append(path)
    return written


def load_stage_checkpoint(directory: str | None, module, opt, device) -> bool:
    """Loads every logical stage of ``module``; returns False (and leaves everything untouched) if any file is
    missing or unreadable, as the reference's training path does (:1143-1148)."""
    if not directory:
        return False
    loaded = {}
    for stage in _stage_ids(module):
        try:
            ck = torch.load(_fname(directory, stage), map_location="cpu", weights_only=True)
            if "integrity" in ck:
                now = _integrity(ck)
                for k, v in ck["integrity"].items():
                    if not (abs(now.get(k, float("nan")) - v) <= 1e-9 * max(1.0, abs(v))):
                        raise ValueError(f"checkpoint payload damaged: {k}")
            loaded[stage] = ck
        except Exception:
            return False
    model_sd, master, ema, m, v = {}, {}, {}, {}, {}
    for stage, ck in loaded.items():
        for k, t in ck["model_state_dict"].items():
            model_sd[_key_for(module, stage, k)] = t
        for k, t in ck["main_model_state_dict"].items():
            master[_key_for(module, stage, k)] = t
        for k, t in ck.get("ema_state_dict", {}).items():
            ema[_key_for(module, stage, k)] = t
        for k, t in ck["optimizer_state_dict"]["exp_avg"].items():
            m[_key_for(module, stage, k)] = t
        for k, t in ck["optimizer_state_dict"]["exp_avg_sq"].items():
            v[_key_for(module, stage, k)] = t
    first = next(iter(loaded.values()))
    # parameters are views of the optimizer's flat buffers, so loading the masters refreshes the model copies too;
    # buffers and frozen parameters come from the model state dict
    own = module.state_dict()
    managed = set(opt.master_state_dict().keys())
    for k, t in model_sd.items():
        if k in own and k not in managed:
            own[k].copy_(t)
    opt.load_state_dict({"step": first["optimizer_state_dict"]["step"], "cur_nimg": first["cur_nimg"],
                         "exp_avg": m, "exp_avg_sq": v}, master=master, ema=ema or None)
    return True


def convert_inference_checkpoint(path: str, n_logical: int, model, map_location="cpu", use_ema: bool = True,
                                 strict: bool = True) -> dict:
    """Per-stage files -> one state dict for :class:`AerisModel`, then ``model.load_state_dict``. Takes
    ``ema_state_dict`` (or ``model_state_dict``). Keys the monolithic model does not have are skipped (the reference
    drops ``latent_embed*`` and ``*.1.norm*`` the same way, model.py:483,488)."""
    which = "ema_state_dict" if use_ema else "model_state_dict"
    own = model.state_dict()
    new = {}
    for stage in range(n_logical):
        ck = torch.load(_fname(path, stage), map_location=map_location, weights_only=True)
        sd = ck[which] if which in ck else ck["model_state_dict"]
        for k, t in sd.items():
            if stage == 0:
                key = f"input_stage.{k}"
            elif stage == n_logical - 1:
                key = f"output_stage.{k}"
            else:
                key = f"layers.{stage - 1}.{k}"
            if key in own:
                new[key] = t.to(own[key].dtype)
    missing = [k for k in own if k not in new]
    if strict:
        assert not missing, f"checkpoint does not cover the model: missing {missing[:5]}..."
    model.load_state_dict(new, strict=False)
    return new
