"""``TrainingArguments``: every run-time flag of the trainer, and the derivation of the hybrid-parallel degrees.

Mirrors the reference's dataclass (paddleformers/trainer/training_args.py:80) in naming and behaviour where it
matters to users: the parallel degrees (``tensor_model_parallel_size``, ``pipeline_model_parallel_size``,
``expert_model_parallel_size``, ``context_parallel_size``, ``sep_parallel_size``, ``sharding_parallel_size``,
``sharding`` stage), the derived data-parallel degree (:2819-2947), dataset rank / world rules (:3038-3101), batch
size arithmetic, logging / saving / evaluation strategies. Unlike the reference, building the arguments does not
initialise the process groups as a side effect; ``setup_parallel()`` does so explicitly (the Trainer calls it).
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from ..parallel.topology import ParallelDegrees, ParallelState, get_parallel_state, initialize_parallel
from ..transformers.configuration_utils import llmmetaclass
from .trainer_utils import IntervalStrategy, SchedulerType


@dataclass
@llmmetaclass
class TrainingArguments:
    output_dir: str = field(default="./output", metadata={"help": "where checkpoints and logs go"})
    overwrite_output_dir: bool = False
    do_train: bool = True
    do_eval: bool = False
    do_predict: bool = False
    # batch / steps
    per_device_train_batch_size: int = 1
    per_device_eval_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    num_train_epochs: float = 1.0
    max_steps: int = -1
    max_seq_len: int = 2048
    # optimisation
    learning_rate: float = 1e-4
    min_lr: float = 0.0
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    lr_scheduler_type: str = "linear"
    warmup_steps: int = 0
    warmup_ratio: float = 0.0
    decay_steps: Optional[int] = None
    num_cycles: float = 0.5            # cosine: number of waves (0.5 = decay to the minimum once)
    power: float = 1.0                 # polynomial: exponent of the decay
    lr_end: Optional[float] = None     # polynomial: final learning rate (same role as min_lr; used when min_lr is 0)
    optim: str = field(default="adamw", metadata={"help": "adamw | adamw_mini (one second moment per row) | adamw_custom | muon"})
    use_lowprecision_moment: bool = False        # adamw_custom: Adam moments stored in bf16
    tensorwise_offload_optimizer: bool = False   # adamw_custom: Adam moments live in host memory, streamed through the device
    hf_bitexact: bool = False                    # adamw_custom: torch.optim.AdamW / clip_grad_norm_ operation order (one process)
    freeze_training: bool = field(default=False, metadata={"help": "lr = 0 and no updates (debugging aid)"})
    # precision
    bf16: bool = False
    fp16: bool = False
    amp_master_grad: bool = True
    # parallelism
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    context_parallel_size: int = 1
    sep_parallel_size: int = 1
    sharding_parallel_size: int = -1
    sharding: str = field(default="", metadata={"help": "'' | stage1 | stage2 (optimizer-state sharding; stage2 is accepted for "
                                                        "configuration compatibility and runs the stage1 plan: gradients stay in the "
                                                        "full fp32 accumulation buffer that the weight-gradient GEMMs write) | stage3 "
                                                        "(alias fsdp: parameters, gradients and optimizer state sharded per decoder "
                                                        "layer over the data ranks, with per-layer recompute)"})
    sequence_parallel: bool = False
    hybrid_parallel_topo_order: str = "sharding_first"
    pipeline_schedule: str = field(default="1F1B", metadata={"help": "1F1B | interleaved | FThenB | zero_bubble (backward split into input-gradient and deferred weight-gradient parts) | zbv (zero_bubble on a V-shaped placement with two chunks per stage)"})
    sharding_comm_buffer_size_MB: int = 256
    sharding_overlap: bool = True
    # logging / saving / eval
    logging_steps: int = 1
    logging_first_step: bool = True
    save_strategy: str = "steps"
    save_steps: int = 500
    save_total_limit: Optional[int] = None
    save_hf_steps: int = -1
    eval_strategy: str = "no"
    eval_steps: Optional[int] = None
    max_evaluate_steps: int = -1       # > 0: evaluate on at most that many batches
    load_best_model_at_end: bool = False        # reload the checkpoint with the best evaluation metric when training ends
    metric_for_best_model: Optional[str] = None   # default "loss" (looked up as eval_<name>)
    greater_is_better: Optional[bool] = None      # default: False for losses, True otherwise
    report_to: str = "none"            # none | comma-separated: tensorboard, visualdl, jsonl
    logging_dir: Optional[str] = None  # scalar logs (default <output_dir>/runs)
    enable_zero_cost_checkpoint: bool = False   # snapshot the optimizer shard on a side stream, persist in the background
    zcc_save_model_weights: bool = False        # also export HF weights at every save (collective and synchronous)
    nccl_comm_group_config: Optional[str] = None   # JSON file / string: per-group NCCL communicator options
    ema_decay: float = 0.0                      # > 0: keep an exponential moving average of the fp32 master shards
    zcc_save_ema_coef: Optional[float] = None   # with enable_zero_cost_checkpoint: EMA coefficient (same average, saved with the checkpoint)
    zcc_ema_interval: int = 1                   # average every that many optimizer steps
    zcc_ema_loss_threshold: Optional[float] = None   # average only while the last logged loss is below this value
    ema_start_step: int = 0
    enable_timer: bool = False         # per-step read-data / forward-backward / optimizer-step timers in the log record
    log_loss_md5: bool = False         # md5 of the logged loss's fp32 bytes in the log record (also: LOG_LOSS_MD5=1)
    log_memory: bool = False           # device memory high-water marks in the log record
    internal_medicine_monitors: Optional[str] = None   # "all" or a comma list of activations,router,grads,weights
    internal_medicine_monitor_interval: int = 0       # sample the monitors every N steps (0 = off)
    metrics_output_path: Optional[str] = None
    resume_from_checkpoint: Optional[str] = None
    flash_device_path: Optional[str] = None     # fast local device: every checkpoint is mirrored there (verified copy, newest
    #                                             kept) and resume_from_checkpoint=auto looks there first
    save_checkpoint_format: str = field(default="sharded", metadata={"help": "sharded | unified | hf"})
    load_checkpoint_format: str = "sharded"
    async_save: bool = False
    skip_data_intervals: Optional[List[List[int]]] = None
    ignore_data_skip: bool = False
    # data
    dataloader_num_workers: int = 0
    dataloader_drop_last: bool = True
    seed: int = 42
    data_seed: Optional[int] = None
    # misc
    profile: bool = False
    profile_step_start: int = 3
    profile_step_end: int = 5
    skip_profile_timer: bool = True
    profile_nvtx_depth: int = 0         # > 0: inside the profile window, one NVTX range per sub-module down to this depth
    profile_backend: str = "cuda_api"   # cuda_api: cudaProfilerStart/Stop window for an external profiler | torch: torch.profiler trace
    disable_tqdm: bool = True
    device: Optional[str] = None
    pg_timeout_s: int = 0
    distributed_backend: Optional[str] = None
    heartbeat_interval_s: float = 0.0
    release_grads: bool = False
    moe_aux_free_bias_update_rate: float = 0.0
    count_trained_tokens: bool = False
    cuda_graph: bool = field(default=False, metadata={"help": "capture one micro-batch of forward + backward in a CUDA graph "
                                                          "and replay it (static shapes, dense models)"})
    cuda_graph_warmup: int = 2

    def __post_init__(self):
        self.lr_scheduler_type = SchedulerType(self.lr_scheduler_type).value
        if self.lr_end is not None and not self.min_lr:
            self.min_lr = float(self.lr_end)
        # the reference's names for the same two layouts: per-rank shards / layout-independent state
        fmt_alias = {"sharding_io": "sharded", "flex_checkpoint": "unified", "unified_checkpoint": "unified"}
        self.save_checkpoint_format = fmt_alias.get(self.save_checkpoint_format, self.save_checkpoint_format)
        self.load_checkpoint_format = fmt_alias.get(self.load_checkpoint_format, self.load_checkpoint_format)
        self.save_strategy = IntervalStrategy(self.save_strategy).value
        self.eval_strategy = IntervalStrategy(self.eval_strategy).value
        if self.bf16 and self.fp16:
            raise ValueError("choose one of bf16 / fp16")
        if self.device is None:
            if torch.cuda.is_available():
                self.device = f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}"
            else:
                self.device = "cpu"
        self.world_size = int(os.environ.get("WORLD_SIZE", "1"))
        self.process_index = int(os.environ.get("RANK", "0"))
        self._post_init_parallel_degree()
        self._state: Optional[ParallelState] = None

    # ------------------------------------------------------------------ parallel degrees
    def _post_init_parallel_degree(self):
        """dp = world / (tp * pp * sep * cp * sharding); sharding defaults to "everything that is left" when a sharding
        stage is requested (paddleformers/trainer/training_args.py:2819-2947)."""
        world = self.world_size
        tp, pp = max(self.tensor_model_parallel_size, 1), max(self.pipeline_model_parallel_size, 1)
        sep, cp = max(self.sep_parallel_size, 1), max(self.context_parallel_size, 1)
        if sep > 1 and cp > 1:
            raise ValueError("sep_parallel_size and context_parallel_size are mutually exclusive")
        model_par = tp * pp * sep * cp
        if world % model_par != 0:
            raise ValueError(f"world size {world} is not divisible by tp*pp*sep*cp = {model_par}")
        rest = world // model_par
        if self.sharding:
            if self.sharding in ("fsdp", "p_g_os"):
                self.sharding = "stage3"
            if self.sharding not in ("stage1", "stage2", "stage3"):
                raise ValueError("sharding must be '', 'stage1', 'stage2' or 'stage3' (alias fsdp)")
            if self.sharding == "stage2":
                # gradients stay whole per rank: the fp32 main_grad buffers that the weight-gradient GEMMs accumulate into
                # are the gradient store of this design, so stage 2 runs the stage-1 plan (stage 3 shards them per layer)
                import warnings

                warnings.warn("sharding stage2 runs the stage1 plan here (optimizer state sharded, fp32 gradients kept whole "
                              "per rank); use stage3 to shard gradients and parameters too", stacklevel=2)
            if self.sharding == "stage3" and (tp > 1 or pp > 1 or max(self.expert_model_parallel_size, 1) > 1 or sep > 1 or cp > 1):
                raise ValueError("sharding stage3 shards over the data ranks only: tensor / pipeline / expert / context "
                                 "parallel degrees must be 1")
            sharding = rest if self.sharding_parallel_size in (-1, 0) else self.sharding_parallel_size
        else:
            sharding = 1 if self.sharding_parallel_size in (-1, 0) else self.sharding_parallel_size
        if rest % sharding != 0:
            raise ValueError(f"sharding_parallel_size {sharding} must divide {rest}")
        dp = rest // sharding
        ep = max(self.expert_model_parallel_size, 1)
        if (world // pp) % ep != 0:
            raise ValueError(f"expert_model_parallel_size {ep} must divide world/pp = {world // pp}")
        if self.sequence_parallel and tp == 1:
            self.sequence_parallel = False
        self.data_parallel_size = dp
        self.sharding_parallel_size = sharding
        self.moe_sharding_parallel_size = world // (pp * ep)
        self.degrees = ParallelDegrees(dp=dp, sharding=sharding, pp=pp, sep=sep, cp=cp, mp=tp, ep=ep,
                                       order=self.hybrid_parallel_topo_order)

    def setup_parallel(self) -> ParallelState:
        if self._state is None:
            if self.world_size > 1:
                if self.pg_timeout_s:
                    os.environ.setdefault("PFB_PG_TIMEOUT", str(self.pg_timeout_s))
                self._state = initialize_parallel(self.degrees, backend=self.distributed_backend,
                                                   nccl_config=getattr(self, "nccl_comm_group_config", None))
            else:
                from ..parallel.topology import set_parallel_state

                self._state = ParallelState(self.degrees, rank=0, create_groups=False)
                set_parallel_state(self._state)
        return self._state

    # ------------------------------------------------------------------ derived quantities
    @property
    def parallel_state(self) -> ParallelState:
        return self.setup_parallel()

    @property
    def dataset_world_size(self) -> int:
        return self.data_parallel_size * self.sharding_parallel_size

    @property
    def dataset_rank(self) -> int:
        return self.parallel_state.dataset_rank

    @property
    def train_batch_size(self) -> int:
        return self.per_device_train_batch_size

    @property
    def global_batch_size(self) -> int:
        return self.per_device_train_batch_size * self.gradient_accumulation_steps * self.dataset_world_size

    @property
    def should_log(self) -> bool:
        return self.process_index == 0

    @property
    def should_save(self) -> bool:
        return True  # every rank writes its own shard; rank 0 writes the shared files

    def get_warmup_steps(self, num_training_steps: int) -> int:
        return self.warmup_steps if self.warmup_steps > 0 else int(num_training_steps * self.warmup_ratio)

    @property
    def compute_dtype(self) -> torch.dtype:
        return torch.bfloat16 if self.bf16 else (torch.float16 if self.fp16 else torch.float32)

    def to_dict(self) -> Dict[str, Any]:
        out = {}
        for f in dataclasses.fields(self):
            v = getattr(self, f.name)
            out[f.name] = v
        return out

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, default=str)
