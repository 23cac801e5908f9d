"""``paddleformers-b200 {train|export|merge|preprocess|ckpt|env|version|help}``: the user-facing command.

``train cfg.yaml [key=value ...]`` starts one process per visible GPU with ``torch.distributed.run`` (rendezvous on
MASTER_ADDR / 127.0.0.1), optionally under ``numactl`` binding, and kills the whole process tree if any rank fails;
``export`` folds LoRA adapters into a base model and writes an HF directory. Counterparts: paddleformers/cli/cli.py:57
(``main``), :147-177 (launch + tree kill), paddleformers/cli/launcher.py:48-73 (NUMA binding), cli/export/export.py:83.
"""
from __future__ import annotations

import os
import shutil
import signal
import subprocess
import sys
from typing import List, Optional

USAGE = """usage: paddleformers-b200 <command> [args]

commands:
  train  <config.yaml|json> [key=value ...]   run a training stage (SFT | PT | DPO | VL-SFT | VL-PT | VL-DPO | recipes; with or without LoRA)
  export <config.yaml|json> [key=value ...]   merge LoRA adapters into the base model and write an HF checkpoint
  merge  <config.yaml|json> [key=value ...]   merge several checkpoints of one architecture (linear | slerp | ties, with
                                              dare / magprune / trim sparsification of the task vectors)
  preprocess --input F --tokenizer DIR --output-prefix P [...]   tokenise raw text into the .bin / .idx corpus format
  ckpt   inspect|reshard ...                  look into a training checkpoint, or re-cut its optimizer shards
  env                                         versions, GPUs and the state of the compiled extension
  version                                     print the package version
  help                                        this text
"""


def visible_gpus() -> int:
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    if env is not None:
        return len([x for x in env.split(",") if x.strip() != ""])
    try:
        import torch

        return torch.cuda.device_count()
    except Exception:  # noqa: BLE001
        return 0


def build_launch_command(argv: List[str], nproc: int) -> List[str]:
    nnodes = os.environ.get("NNODES", "1")
    node_rank = os.environ.get("NODE_RANK", os.environ.get("RANK", "0")) if int(nnodes) > 1 else "0"
    master_addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    master_port = os.environ.get("MASTER_PORT", "29533")
    cmd = [sys.executable, "-m", "torch.distributed.run", f"--nnodes={nnodes}", f"--node-rank={node_rank}",
           f"--nproc-per-node={nproc}", f"--master-addr={master_addr}", f"--master-port={master_port}"]
    # BIND_TRAINER_NUMA=1: every trainer process pins itself to the NUMA node of its GPU (utils/numa.py); the launcher
    # itself needs no wrapper
    return cmd + ["-m", "paddleformers_b200.cli.train"] + argv


def _kill_tree(proc: subprocess.Popen):
    try:
        os.killpg(proc.pid, signal.SIGTERM)
    except ProcessLookupError:
        pass


def train(argv: List[str]) -> int:
    n = visible_gpus()
    env = dict(os.environ)
    env.setdefault("NVIDIA_TF32_OVERRIDE", "0")
    for k in list(env):
        if k.startswith("PADDLE_"):
            env.pop(k)
    if n <= 1 and int(env.get("NNODES", "1")) == 1:
        from .train import run_tuner

        run_tuner(argv)
        return 0
    proc = subprocess.Popen(build_launch_command(argv, n), env=env, start_new_session=True)
    try:
        rc = proc.wait()
    except KeyboardInterrupt:
        _kill_tree(proc)
        raise
    if rc != 0:
        _kill_tree(proc)
    return rc


def export(argv: List[str]) -> int:
    from ..mergekit.merge import merge_lora_and_export
    from .hparams import get_train_args

    model_args, _, _, export_args, train_args = get_train_args(argv)
    if not (model_args.model_name_or_path and model_args.lora_path):
        raise ValueError("export needs model_name_or_path (base) and lora_path")
    out = export_args.export_dir or os.path.join(train_args.output_dir, "export")
    import torch

    dt = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[export_args.export_dtype]
    merge_lora_and_export(model_args.model_name_or_path, model_args.lora_path, out, dtype=dt)
    print(f"exported merged model to {out}")
    return 0


def merge(argv: List[str]) -> int:
    """``merge cfg.yaml [key=value ...]``: the fields of ``mergekit.MergeConfig`` from a YAML / JSON file and overrides
    (paddleformers/mergekit/merge_model.py, examples/tools/merge.py)."""
    import dataclasses
    import json

    from ..mergekit.merge import MergeConfig, MergeModel

    cfg = {}
    for a in argv:
        if "=" in a and not os.path.exists(a):
            k, v = a.split("=", 1)
            try:
                cfg[k] = json.loads(v)
            except json.JSONDecodeError:
                cfg[k] = v
        elif a.endswith((".yaml", ".yml")):
            import yaml

            cfg.update(yaml.safe_load(open(a)) or {})
        else:
            cfg.update(json.load(open(a)))
    known = {f.name for f in dataclasses.fields(MergeConfig)}
    unknown = sorted(set(cfg) - known)
    if unknown:
        raise ValueError(f"unknown merge options {unknown}; known: {sorted(known)}")
    out = MergeModel(MergeConfig(**cfg)).merge()
    print(f"merged model written to {out}")
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("help", "-h", "--help"):
        print(USAGE)
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "version":
        from .. import __version__

        print(__version__)
        return 0
    if cmd == "train":
        return train(rest)
    if cmd == "export":
        return export(rest)
    if cmd == "merge":
        return merge(rest)
    if cmd == "preprocess":
        from ..data.preprocess import main as preprocess_main

        return preprocess_main(rest) or 0
    if cmd == "ckpt":
        from ..trainer.ckpt_converter import main as ckpt_main

        return ckpt_main(rest)
    if cmd == "env":
        import json

        from ..utils.env_report import collect

        print(json.dumps(collect(), indent=2, default=str))
        return 0
    print(f"unknown command {cmd!r}\n\n{USAGE}", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main())
