"""``python -m paddleformers_b200.cli.docgen > docs/arguments.md``: reference of every configuration key accepted by the
command line, generated from the argument dataclasses (so it cannot drift from the parser)."""
from __future__ import annotations

import dataclasses
import sys

from ..transformers.configuration_utils import LlmMetaConfig
from .hparams import DataArguments, ExportArguments, GeneratingArguments, ModelArguments, TrainingArguments


def _rows(cls):
    for f in dataclasses.fields(cls):
        if f.name.startswith("_"):
            continue
        default = f.default if f.default is not dataclasses.MISSING else (f.default_factory() if f.default_factory is not dataclasses.MISSING else "")
        typ = getattr(f.type, "__name__", str(f.type)).replace("typing.", "")
        yield f.name, typ, repr(default), (f.metadata or {}).get("help", "").replace("|", "\\|")


def render() -> str:
    out = ["# Configuration keys", "",
           "One flat YAML / JSON file (plus `key=value` overrides on the command line) is split over these groups by key name; "
           "unknown keys are rejected.", ""]
    for title, cls in (("Model", ModelArguments), ("Data", DataArguments), ("Generation", GeneratingArguments),
                       ("Export", ExportArguments), ("Training", TrainingArguments)):
        out += [f"## {title} (`{cls.__name__}`)", "", "| key | type | default | meaning |", "|---|---|---|---|"]
        out += [f"| `{n}` | {t} | `{d}` | {h} |" for n, t, d, h in _rows(cls)]
        out.append("")
    out += ["## Model run-time attributes copied from the training arguments onto the model configuration", "",
            "| key | default | meaning |", "|---|---|---|"]
    for group in ("op_fusion_attributes", "hybrid_parallel_attributes", "recompute_attributes", "loss_attributes", "moe_attributes",
                  "mtp_attributes", "fp8_attributes"):
        for entry in getattr(LlmMetaConfig, group, []):
            name, _typ, default, help_ = entry
            out.append(f"| `{name}` | `{default!r}` | {help_.replace('|', chr(92) + '|')} |")
    return "\n".join(out) + "\n"


if __name__ == "__main__":
    sys.stdout.write(render())
