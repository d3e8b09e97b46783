"""Checkpoint quantisation-config importers, tried in order: HF flat fp8,
compressed-tensors, NVIDIA ModelOpt. Each turns a config blob into a QuantPlan
or returns ``None`` when the blob is not its format.

Reference: phyai/src/phyai/layers/quant/importers/{fp8,compressed_tensors,modelopt,registry}.py.
"""

from __future__ import annotations

from typing import Any, Callable, Mapping

from .scheme import (FP8_BLOCK_128, FP8_PER_CHANNEL, FP8_PER_TENSOR, NVFP4_BLOCK_16, Granularity, Matcher,
                     QDType, QuantPlan, QuantScheme, Rule, TensorQuant)

Importer = Callable[[Mapping[str, Any]], "QuantPlan | None"]


def _ignore_rules(names) -> tuple[Rule, ...]:
    rules = []
    for n in names or ():
        if n.startswith("re:"):
            rules.append(Rule(Matcher(regex=_from_start(n[3:])), None))
        elif any(ch in n for ch in "*?["):
            rules.append(Rule(Matcher(glob=n), None))
        else:
            rules.append(Rule(Matcher(regex=rf"(^|\.){_esc(n)}($|\.)"), None))
    return tuple(rules)


def _esc(s: str) -> str:
    import re

    return re.escape(s)


def _from_start(pattern: str) -> str:
    """A ``re:`` entry of a checkpoint is matched from the start of the module name (``re.match``), as the libraries
    that write these files and the reference (phyai/src/phyai/layers/quant/plan.py:25-26) do."""
    return pattern if pattern.startswith("^") else f"^(?:{pattern})"


def import_hf_fp8(blob: Mapping[str, Any]) -> QuantPlan | None:
    """``{"quant_method": "fp8", "weight_block_size": [128, 128], "modules_to_not_convert": [...]}``"""
    if blob.get("quant_method") != "fp8":
        return None
    wbs = blob.get("weight_block_size")
    if wbs:
        r, c = int(wbs[0]), int(wbs[1])
        scheme = FP8_BLOCK_128 if (r, c) == (128, 128) else QuantScheme(
            weight=TensorQuant(QDType.FP8_E4M3, Granularity.BLOCK, (r, c)),
            activation=TensorQuant(QDType.FP8_E4M3, Granularity.GROUP, (c,), dynamic=True))
    else:
        scheme = FP8_PER_TENSOR
    return QuantPlan(rules=_ignore_rules(blob.get("ignored_layers") or blob.get("modules_to_not_convert")), default=scheme)


def import_compressed_tensors(blob: Mapping[str, Any]) -> QuantPlan | None:
    if blob.get("quant_method") != "compressed-tensors" and "config_groups" not in blob:
        return None
    rules = list(_ignore_rules(blob.get("ignore")))
    for group in (blob.get("config_groups") or {}).values():
        w = group.get("weights") or {}
        scheme = _ct_scheme(w, group.get("input_activations"))
        for target in group.get("targets", ["Linear"]):
            if target.startswith("re:"):
                rules.append(Rule(Matcher(regex=_from_start(target[3:])), scheme))
            elif target == "Linear":
                rules.append(Rule(Matcher(module_cls="LinearBase"), scheme))
            elif "." not in target and target[:1].isupper():          # a bare CamelCase token names a module class
                rules.append(Rule(Matcher(module_cls=target), scheme))
            else:                                                     # anything else names modules
                rules.append(Rule(Matcher(regex=rf"(^|\.){_esc(target)}($|\.)"), scheme))
    return QuantPlan(rules=tuple(rules), default=None)


def _ct_scheme(w: Mapping[str, Any], act: Mapping[str, Any] | None) -> QuantScheme | None:
    bits, typ, strat = w.get("num_bits"), w.get("type"), w.get("strategy", "tensor")
    if typ == "float" and bits == 8:
        if strat == "block":
            bs = w.get("block_structure") or [128, 128]
            if isinstance(bs, str):
                bs = [int(v) for v in bs.split("x")]
            return QuantScheme(weight=TensorQuant(QDType.FP8_E4M3, Granularity.BLOCK, (int(bs[0]), int(bs[1]))),
                               activation=TensorQuant(QDType.FP8_E4M3, Granularity.GROUP, (int(bs[1]),), dynamic=True))
        return FP8_PER_CHANNEL if strat == "channel" else FP8_PER_TENSOR
    if typ == "float" and bits == 4:
        return NVFP4_BLOCK_16
    return None


def import_modelopt(blob: Mapping[str, Any]) -> QuantPlan | None:
    """``hf_quant_config.json`` (``{"quantization": {"quant_algo": ..., "exclude_modules": [...]}}``) or the same fields
    inline in ``config.json`` under ``quant_method`` modelopt / modelopt_fp8 / modelopt_fp4."""
    q = blob.get("quantization", blob)
    if not isinstance(q, Mapping):
        return None
    algo = q.get("quant_algo")
    if algo is None:
        return None
    table = {"FP8": FP8_PER_TENSOR, "FP8_PER_CHANNEL_PER_TOKEN": FP8_PER_CHANNEL,
             "FP8_PB_WO": FP8_BLOCK_128, "NVFP4": NVFP4_BLOCK_16}
    if algo not in table:
        raise ValueError(f"ModelOpt quant_algo {algo!r} is not supported")
    return QuantPlan(rules=_ignore_rules(q.get("exclude_modules") or q.get("ignore")), default=table[algo])


IMPORTERS: list[Importer] = [import_hf_fp8, import_compressed_tensors, import_modelopt]


def register_importer(fn: Importer, *, first: bool = False) -> None:
    IMPORTERS.insert(0, fn) if first else IMPORTERS.append(fn)


def import_plan(blob: Mapping[str, Any]) -> QuantPlan | None:
    for fn in IMPORTERS:
        plan = fn(blob)
        if plan is not None:
            return plan
    return None


__all__ = ["import_plan", "register_importer", "import_hf_fp8", "import_compressed_tensors", "import_modelopt", "IMPORTERS"]
