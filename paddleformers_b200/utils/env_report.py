"""``python -m paddleformers_b200.utils.env_report``: one screen of facts for bug reports and run logs - library versions,
visible GPUs, NCCL, whether the in-tree extensions are built and load, and the operators they provide."""
from __future__ import annotations

import json
import os
import platform
import sys


def collect() -> dict:
    import torch

    from ..ops import _build

    info = {"python": sys.version.split()[0], "platform": platform.platform(), "torch": torch.__version__,
            "cuda_runtime": torch.version.cuda, "cuda_available": torch.cuda.is_available()}
    try:
        info["nccl"] = ".".join(str(v) for v in torch.cuda.nccl.version())
    except Exception:  # noqa: BLE001
        info["nccl"] = None
    if torch.cuda.is_available():
        info["gpus"] = [{"index": i, "name": torch.cuda.get_device_name(i), "capability": list(torch.cuda.get_device_capability(i)),
                         "memory_gb": round(torch.cuda.get_device_properties(i).total_memory / 2 ** 30, 1),
                         "sms": torch.cuda.get_device_properties(i).multi_processor_count} for i in range(torch.cuda.device_count())]
    info["extension"] = {"path": _build.ext_path(), "built": os.path.exists(_build.ext_path()),
                         "host_library_built": os.path.exists(_build.HOST_LIB)}
    if info["extension"]["built"]:
        try:
            _build.load_extension(required=True)
            info["extension"]["operators"] = sorted({s.name.split("::", 1)[1] for s in torch._C._jit_get_all_schemas()
                                                     if s.name.startswith("pfb200::")})
        except Exception as e:  # noqa: BLE001
            info["extension"]["load_error"] = f"{type(e).__name__}: {e}"
    for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK", "MASTER_ADDR", "NCCL_NVLS_ENABLE", "PFB_FUSED_TP", "PFB_FUSED_EP", "PFB_EP_CAPACITY"):
        if k in os.environ:
            info.setdefault("env", {})[k] = os.environ[k]
    return info


if __name__ == "__main__":
    print(json.dumps(collect(), indent=2))
