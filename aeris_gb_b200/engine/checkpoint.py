"""Checkpoint IO in the reference's on-disk format.

Training writes one file per *logical* pipeline stage, ``checkpoint_PP{stage}.pth`` (plus ``it_{it}_checkpoint_PP{stage}
.pth`` every 1000 iterations), each a dict with ``cur_nimg``, ``model_state_dict`` (device-dtype copy),
``main_model_state_dict`` (fp32 master), ``optimizer_state_dict`` and ``ema_state_dict``
(src/aeris/parallelism/parallel_engine.py:1119-1160). Files are loaded with ``weights_only=True``. Because files are
per logical stage they do not depend on how many physical pipeline ranks wrote them.

``optimizer_state_dict`` has the layout of ``torch.optim.AdamW.state_dict()``, which is what the reference stores
(:1131): ``state`` maps the index of a parameter to ``{"step", "exp_avg", "exp_avg_sq"}`` and ``param_groups`` lists
the indices with the hyper-parameters. Indices count the stage's parameters in ``named_parameters()`` order (the order
of ``main_model.parameters()`` the reference builds its optimizer from, src/aeris/train.py:194-223), one group, or the
reference's (decay, no-decay) pair of groups. Files written here also carry ``param_names`` so that loading does not
depend on the order; a file without it (written by the reference) is mapped by position.

Inference reads the per-stage files into one monolithic model (``input_stage.* / layers.{i}.* / output_stage.*``),
always from ``ema_state_dict`` (src/aeris_wp_inference/model.py:479-495).
"""
from __future__ import annotations

import os

import torch


def _fname(directory, stage: int, it: int | None = None, prefix: str = "") -> str:
    """``prefix``: text in front of the file name, e.g. ``it_5000_`` for a numbered copy (the reference's
    ``--extra-name``, sp_inference_engine.py:552-560)."""
    name = f"{prefix}checkpoint_PP{stage}.pth" if it is None else f"it_{it}_checkpoint_PP{stage}.pth"
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
    state = ckpt.get("optimizer_state_dict", {}).get("state", {})
    sections["optimizer/exp_avg"] = {str(i): st["exp_avg"] for i, st in state.items() if "exp_avg" in st}
    sections["optimizer/exp_avg_sq"] = {str(i): st["exp_avg_sq"] for i, st in state.items() if "exp_avg_sq" in st}
    for section, sd in sections.items():
        for k, t in sd.items():
            if torch.is_tensor(t) and t.dtype.is_floating_point:
                out[f"{section}/{k}"] = float(torch.nan_to_num(t.double()).sum())
    return out


def _torch_optim_state(names: list[str], exp_avg: dict, exp_avg_sq: dict, opt) -> dict:
    """``torch.optim.AdamW.state_dict()`` for one logical stage: ``names`` are all its parameters in order."""
    c = opt.cfg
    state = {}
    for i, n in enumerate(names):
        if n in exp_avg:
            state[i] = {"step": torch.tensor(float(opt.step_count)), "exp_avg": exp_avg[n].cpu(),
                        "exp_avg_sq": exp_avg_sq[n].cpu()}
    group = {"lr": float(getattr(opt, "last_lr", c.lr)), "betas": tuple(c.betas), "eps": c.eps,
             "weight_decay": c.weight_decay, "amsgrad": False, "maximize": False, "foreach": None, "capturable": False,
             "differentiable": False, "fused": None, "params": list(range(len(names)))}
    return {"state": state, "param_groups": [group], "param_names": list(names)}


def _read_optim_state(osd: dict, names: list[str]) -> tuple[int, dict, dict]:
    """(step, exp_avg by name, exp_avg_sq by name) from a ``torch.optim`` state dict of one stage. ``names``: the
    stage's parameters in ``named_parameters()`` order, used when the file does not name them itself."""
    if "state" not in osd or "param_groups" not in osd:
        raise ValueError("optimizer_state_dict is not a torch.optim state dict")
    order = [i for g in osd["param_groups"] for i in g["params"]]
    file_names = osd.get("param_names")
    if file_names is None:
        if len(order) != len(names):
            raise ValueError(f"optimizer state covers {len(order)} parameters, the stage has {len(names)}")
        file_names = names
    by_index = {i: file_names[pos] for pos, i in enumerate(order)}
    m, v, step = {}, {}, 0
    for i, st in osd["state"].items():
        name = by_index[int(i)]
        m[name], v[name] = st["exp_avg"], st["exp_avg_sq"]
        step = max(step, int(float(st["step"])))
    return step, m, v


def _stage_param_names(module) -> dict[int, list[str]]:
    """Per logical stage, the reference-style names of all parameters in registration order."""
    out: dict[int, list[str]] = {}
    last = _n_logical(module) - 1
    for k, _ in module.named_parameters():
        if k.startswith("input_stage."):
            out.setdefault(0, []).append(k[len("input_stage."):])
        elif k.startswith("output_stage."):
            out.setdefault(last, []).append(k[len("output_stage."):])
        elif k.startswith("layers."):
            _, idx, rest = k.split(".", 2)
            out.setdefault(int(idx) + 1, []).append(rest)
    return out


def save_stage_checkpoint(directory: str, module, opt, it: int | None = None, write: bool = True) -> list[str]:
    """``module``: a PipelineStage or a whole AerisModel; ``opt``: the optimizer built on it (FlatOptimizer, or the
    sharded optimizer, whose state dicts are gathered collectively: then every rank of its group calls this function
    and ``write`` is True on one of them). Writes one file per logical stage the module holds."""
    if write:
        os.makedirs(directory, exist_ok=True)
    flat_sd = module.state_dict()
    if getattr(opt, "tp_group", None) is not None:      # tensor-parallel shards are stored as full tensors
        from ..parallel.tensor import full_state_dict
        flat_sd = full_state_dict(flat_sd, opt.tp_group)
    model_sd = _logical(module, flat_sd)
    if hasattr(opt, "host_copies"):
        opt.host_copies = write        # a sharded optimizer gathers collectively; only the writer copies to the host
    master = _logical(module, dict(opt.master_state_dict()))
    ema = _logical(module, dict(opt.ema_state_dict())) if opt.cfg.use_ema else {}
    osd = opt.state_dict()
    if hasattr(opt, "host_copies"):
        opt.host_copies = True
    exp_avg = _logical(module, osd["exp_avg"])
    exp_avg_sq = _logical(module, osd["exp_avg_sq"])
    names = _stage_param_names(module)
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
            "optimizer_state_dict": _torch_optim_state(names.get(stage, []), exp_avg.get(stage, {}),
                                                       exp_avg_sq.get(stage, {}), opt),
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
    names = _stage_param_names(module)
    model_sd, master, ema, m, v = {}, {}, {}, {}, {}
    step = 0
    for stage in _stage_ids(module):
        try:
            ck = torch.load(_fname(directory, stage), map_location="cpu", weights_only=True)
            if "integrity" in ck:
                now = _integrity(ck)
                for k, val in ck["integrity"].items():
                    if not (abs(now.get(k, float("nan")) - val) <= 1e-9 * max(1.0, abs(val))):
                        raise ValueError(f"checkpoint payload damaged: {k}")
            st_step, st_m, st_v = _read_optim_state(ck["optimizer_state_dict"], names.get(stage, []))
            for k, t in ck["model_state_dict"].items():
                model_sd[_key_for(module, stage, k)] = t
            for k, t in ck["main_model_state_dict"].items():
                master[_key_for(module, stage, k)] = t
            for k, t in ck.get("ema_state_dict", {}).items():
                ema[_key_for(module, stage, k)] = t
            for k, t in st_m.items():
                m[_key_for(module, stage, k)] = t
            for k, t in st_v.items():
                v[_key_for(module, stage, k)] = t
            step = max(step, st_step)
            loaded[stage] = ck
        except Exception as e:      # missing, unreadable, damaged or foreign file: nothing has been touched yet
            import logging
            logging.getLogger(__name__).warning("checkpoint of stage %d in %s not loaded: %s", stage, directory, e)
            return False
    first = next(iter(loaded.values()))
    # parameters are views of the optimizer's flat buffers, so loading the masters refreshes the model copies too;
    # buffers and frozen parameters come from the model state dict
    own = module.state_dict()
    managed = set(opt.master_state_dict().keys())
    for k, t in model_sd.items():
        if k in own and k not in managed:
            own[k].copy_(t)
    opt.load_state_dict({"step": step, "cur_nimg": first["cur_nimg"], "exp_avg": m, "exp_avg_sq": v},
                        master=master, ema=ema or None)
    return True


def load_stage_weights(directory: str, module, use_ema: bool = True, tp: int = 1, tp_rank: int = 0,
                       prefix: str = "") -> bool:
    """Inference: only the weights of the module's logical stages, from ``ema_state_dict`` (or ``model_state_dict``),
    as the reference's inference engine does (src/aeris/parallelism/sp_inference_engine.py:552-573). ``tp`` /
    ``tp_rank``: the module holds tensor-parallel shards of the stored full MLP weights."""
    which = "ema_state_dict" if use_ema else "model_state_dict"
    new = {}
    try:
        for stage in _stage_ids(module):
            ck = torch.load(_fname(directory, stage, prefix=prefix), map_location="cpu", weights_only=True)
            for k, t in (ck[which] if which in ck else ck["model_state_dict"]).items():
                new[_key_for(module, stage, k)] = t
    except Exception as e:
        import logging
        logging.getLogger(__name__).warning("weights in %s not loaded: %s", directory, e)
        return False
    own = module.state_dict()
    with torch.no_grad():
        for k, t in new.items():
            if k in own:
                if tp > 1:
                    from ..parallel.tensor import fit_to_shard
                    t = fit_to_shard(k, t, own[k], tp, tp_rank)
                own[k].copy_(t.to(own[k].dtype))
    return True


def convert_inference_checkpoint(path: str, n_logical: int, model, map_location="cpu", use_ema: bool = True,
                                 strict: bool = True, prefix: str = "") -> dict:
    """Per-stage files -> one state dict for :class:`AerisModel`, then ``model.load_state_dict``. Takes
    ``ema_state_dict`` (or ``model_state_dict``). Keys the monolithic model does not have are skipped (the reference
    drops ``latent_embed*`` and ``*.1.norm*`` the same way, model.py:483,488)."""
    which = "ema_state_dict" if use_ema else "model_state_dict"
    own = model.state_dict()
    new = {}
    for stage in range(n_logical):
        ck = torch.load(_fname(path, stage, prefix=prefix), map_location=map_location, weights_only=True)
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
