"""Parameter initialisation policies of the reference (src/aeris/parallelism/parallel_engine.py:1399-1491).

Three policies keyed by ``init_scale_test15`` / ``init_scale_test14`` / neither. All of them touch the *weights* of
every ``nn.Linear`` and ``nn.RMSNorm`` (biases keep PyTorch's default); the base distribution is a truncated normal
with std ``sqrt(2 / (5 dim))``. Modules are recognised by the tags ``is_time_emb`` / ``is_emb`` and by name
(``head``, ``wo``, ``w2``, ``modulation.0``, ``modulation.2``), in that order of precedence.
"""
from __future__ import annotations

import torch.nn as nn


def init_params(model: nn.Module, cfg, policy: dict | None = None) -> None:
    p = dict(init_scale_test15=False, init_scale_test14=False, time_emb_init=0.01, head_init_std=0.6,
             token_emb_init_std=0.3, modulation_0_init=0.001, modulation_2_init=0.0, skip=False)
    p.update(policy or {})
    if p.get("skip"):
        return
    dim = cfg.dim
    base = (2 / (5 * dim)) ** 0.5
    layers = max(cfg.n_layers * cfg.sublayers, 1)
    depth_scale = (1 / (2 * layers)) ** 0.5

    tp, tp_rank = getattr(cfg, "tp", 1), getattr(cfg, "tp_rank", 0)

    def tn(w, std, kind=None):
        if std == 0:
            nn.init.zeros_(w)
        elif kind is not None:
            # a tensor-parallel shard: draw the full-size weight and keep this rank's part, so that the ranks of the
            # group (which share the seed) do not all start from the same values
            import torch
            from ..parallel.tensor import shard_tensor
            shape = (w.shape[0] * tp, w.shape[1]) if kind == "w1" else (w.shape[0], w.shape[1] * tp)
            full = torch.empty(shape, dtype=torch.float32)
            nn.init.trunc_normal_(full, std=std)
            with torch.no_grad():
                w.copy_(shard_tensor(kind, full, tp, tp_rank).to(w.dtype))
        else:
            nn.init.trunc_normal_(w, std=std)

    for name, m in model.named_modules():
        if not isinstance(m, (nn.Linear, nn.RMSNorm)):
            continue
        w = m.weight
        if tp > 1:
            from ..parallel.tensor import tp_kind
            kind = tp_kind(name + ".weight", w)
            if kind is not None:
                scale = depth_scale if (kind == "w2" and p["init_scale_test14"] and not p["init_scale_test15"]) else 1.0
                zero = kind == "w2" and p["init_scale_test15"]
                tn(w, 0 if zero else base * scale, kind)
                continue
        if p["init_scale_test15"] or p["init_scale_test14"]:
            t14 = p["init_scale_test14"] and not p["init_scale_test15"]
            if hasattr(m, "is_time_emb"):
                tn(w, p["time_emb_init"])
            elif "head" in name:
                tn(w, p["head_init_std"]) if t14 else nn.init.zeros_(w)
            elif hasattr(m, "is_emb"):
                tn(w, p["token_emb_init_std"])
            elif "wo" in name or "w2" in name:
                tn(w, base * depth_scale) if t14 else nn.init.zeros_(w)
            elif "modulation.0" in name:
                tn(w, p["modulation_0_init"])
            elif "modulation.2" in name:
                tn(w, p["modulation_2_init"]) if t14 else nn.init.zeros_(w)
            else:
                tn(w, base)
        elif hasattr(m, "is_emb") or "head" in name or "modulation" in name:
            nn.init.zeros_(w)
        else:
            tn(w, base)
