"""``python -m paddleformers_b200.cli.docgen > docs/arguments.md``: reference of every configuration key accepted by the
command line, generated from the argument dataclasses (so it cannot drift from the parser)."""
from __future__ import annotations

import dataclasses
import sys

from ..transformers.configuration_utils import LlmMetaConfig
from .hparams import DataArguments, ExportArguments, GeneratingArguments, ModelArguments, TrainingArguments


REFERENCE_KEYS_SECTION = """## Configuration files written for the reference trainer

Keys that only the reference's `TrainingArguments` knows (about 100 of its 238 fields, and the options inside
`tensor_parallel_config`, `pipeline_parallel_config`, `sharding_parallel_config`, `data_parallel_config`,
`sequence_parallel_config`) are handled by `paddleformers_b200/cli/reference_flags.py` before the arguments are parsed:

* aliases move to this package's field (`evaluation_strategy` -> `eval_strategy`, `sharding_degree` ->
  `sharding_parallel_size`, `use_async_save` -> `async_save`, `unified_checkpoint` -> `save_checkpoint_format: unified`,
  `use_dualpipev` -> `pipeline_schedule: zbv`, `split_backward` -> `pipeline_schedule: zero_bubble`, the overlap switches
  -> `sharding_overlap`, ...);
* switches for behaviour that is built in (`split_param`, `tensor_fusion`, `mp_fused_linear_param_grad_add`,
  `mp_async_allreduce`, `overlap_p2p_comm`, `save_safetensors`, ...) and keys without a meaning in a PyTorch build
  (`fp16_opt_level`, AMP lists, `scale_loss`, platform hooks) are accepted and logged as having no effect;
* keys that ask for something that is not provided (`to_static`, `enable_auto_parallel`, `using_sonic_moe`,
  `forward_backward_overlap_scheduler`, `ckpt_quant_stage`) raise when enabled and name the alternative.

Every YAML under the reference's `tests/config/benchmark/config/pt/` parses this way; anything else that is unknown still
raises `unknown configuration keys` (set `ALLOW_EXTRA_ARGS=1` to ignore)."""


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
    out += ["", REFERENCE_KEYS_SECTION]
    return "\n".join(out) + "\n"


if __name__ == "__main__":
    sys.stdout.write(render())
