"""Per-linear ratio policy: the reference's JSON schema and its loader.

Schema (policies/qwen3_8b_fixed_ratio0p05_policy_v1.json:1-40): {"metadata": {...}, "summary": {...},
"modules": {"model.layers.<i>.<suffix>": {"ratio", "ratio_continuous", "ratio_projected",
"activation_percentile", "weight_percentile", ...}}} with <suffix> one of TARGET_SUFFIXES.

Loader behaviour follows tools/bench_multimodel_all_layers_policy_fastqf_v29.py:181-216, which takes
`ratio_projected` BEFORE `ratio` (in the shipped policy that turns 0.05 into 0.01).  The precedence is an
explicit argument here: `prefer="projected"` reproduces the reference loader, `prefer="ratio"` reads the
field the file name promises.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict

from .ops import ceil_ratio_count, split_select_params

TARGET_SUFFIXES = (
    "self_attn.q_proj",
    "self_attn.k_proj",
    "self_attn.v_proj",
    "self_attn.o_proj",
    "mlp.gate_proj",
    "mlp.up_proj",
    "mlp.down_proj",
)


def normalize_name(name: str) -> str:
    if name.startswith("model."):
        return name
    if name.startswith("layers."):
        return f"model.{name}"
    return name


def policy_key(layer_idx: int, local_name: str) -> str:
    return f"model.layers.{layer_idx}.{local_name}"


def fixed_cfg(ratio: float) -> dict:
    return {"ratio": float(ratio), "ratio_continuous": float(ratio), "ratio_projected": float(ratio),
            "activation_percentile": 100.0, "weight_percentile": 100.0}


def load_policy(path, force_activation_percentile_100: bool = False, prefer: str = "projected") -> dict:
    """Returns {"path", "summary", "metadata", "modules": {name: {ratio, ratio_continuous,
    ratio_projected, activation_percentile, weight_percentile}}}."""
    if prefer not in ("projected", "ratio"):
        raise ValueError("prefer must be 'projected' or 'ratio'")
    path = Path(path)
    raw = json.loads(path.read_text(encoding="utf-8"))
    modules: Dict[str, dict] = {}
    for name, item in raw.get("modules", {}).items():
        key = normalize_name(name)
        if prefer == "projected":
            ratio = float(item.get("ratio_projected", item.get("ratio", item.get("ratio_continuous", 0.0))))
        else:
            ratio = float(item.get("ratio", item.get("ratio_projected", item.get("ratio_continuous", 0.0))))
        pct = float(item.get("activation_percentile", 100.0))
        if force_activation_percentile_100:
            pct = 100.0
        modules[key] = {
            "ratio": ratio,
            "ratio_continuous": float(item.get("ratio_continuous", ratio)),
            "ratio_projected": ratio,
            "activation_percentile": pct,
            "weight_percentile": float(item.get("weight_percentile", 100.0)),
        }
    return {"path": str(path), "summary": raw.get("summary", {}), "metadata": raw.get("metadata", {}),
            "modules": modules}


def make_fixed_ratio_policy(n_layers: int, ratio: float, model: str = "") -> dict:
    """A policy that gives every target linear the same ratio (tools/make_fixed_ratio_policy_v1.py)."""
    modules = {}
    for i in range(n_layers):
        for s in TARGET_SUFFIXES:
            cfg = fixed_cfg(ratio)
            cfg["module_name"] = policy_key(i, s)
            modules[policy_key(i, s)] = cfg
    return {"metadata": {"model": model, "fixed_ratio": float(ratio)}, "modules": modules}


def select_params_for(entry: dict, K: int):
    """(R, descending_rank) of one policy entry for an input dimension K."""
    R = ceil_ratio_count(K, float(entry["ratio"]))
    _, dr, _ = split_select_params(K, R, float(entry.get("activation_percentile", 100.0)))
    return R, dr


def build_linears(named_weights: Dict[str, "object"], policy: dict, default_ratio: float = 0.0,
                  tail_engine: str = "mma", min_ratio: float = 0.0):
    """One `SplitLinear` per named weight with the ratio and percentile its policy entry gives
    (`policy` as returned by `load_policy`; names as in the policy, e.g. "model.layers.3.mlp.down_proj").
    Entries whose ratio is at most `min_ratio` take the pure W4A4 path (R = 0: no select, no tail operands) --
    the adaptive bypass of tools/bench_qwen3_l18_split_opts_v59_adaptive.py:48-91.  Linears without an
    entry get `default_ratio`."""
    from .linear import SplitLinear
    out = {}
    for name, weight in named_weights.items():
        entry = policy.get("modules", {}).get(normalize_name(name))
        ratio = float(entry["ratio"]) if entry else float(default_ratio)
        pct = float(entry["activation_percentile"]) if entry else 100.0
        if ratio <= min_ratio:
            ratio = 0.0
        out[name] = SplitLinear(weight, ratio=ratio, activation_percentile=pct, tail_engine=tail_engine)
    return out
