"""Training loop.

Same user-facing shape as the reference's ``Trainer`` (paddleformers/trainer/trainer.py:282: ``train`` :1877,
``training_step`` :4458, ``evaluate`` :5409, ``save_model``, callbacks, gradient accumulation, logging of speed
metrics :2984-3170, checkpoint / resume :4730) with a different engine underneath:

* the optimizer is the flat-buffer sharded AdamW of ``parallel.sharding`` (fp32 master weights and main grads,
  optimizer state sharded over the sharding group, fused update kernel);
* nothing on the step path synchronises with the host: the loss stays on the device until a logging step, a
  non-finite gradient norm turns the update into a no-op on the device, and token counts are device scalars;
* inputs are staged through pinned host memory with non-blocking copies.
"""
from __future__ import annotations

import contextlib
import json
import math
import os
import time
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, Dataset, IterableDataset

from ..parallel.sharding import ShardedAdamW
from ..parallel.topology import get_parallel_state
from ..utils.log import logger
from . import checkpoint as ckpt
from .trainer_callback import (CallbackHandler, DefaultFlowCallback, FP8QuantWeightCallback, MetricsDumpCallback,
                               MoECorrectionBiasAdjustCallback, PrinterCallback, ProfilerCallback, TrainerCallback,
                               TrainerControl, TrainerState)
from .trainer_utils import (PREFIX_CHECKPOINT_DIR, EvalPrediction, EvalSampler, LRScheduler, PredictionOutput, TrainerMemoryTracker,
                            get_last_checkpoint, tensor_md5, get_scheduler_lambda, set_random_seed, speed_metrics)
from .training_args import TrainingArguments


class ShardedSampler(torch.utils.data.Sampler):
    """Deterministic (seeded) epoch permutation, sliced by dataset rank; supports skipping consumed samples on
    resume."""

    def __init__(self, n: int, rank: int, world: int, batch: int, seed: int, shuffle: bool = True, drop_last=True):
        self.n, self.rank, self.world, self.batch, self.seed, self.shuffle = n, rank, world, batch, seed, shuffle
        self.epoch = 0
        self.skip_batches = 0
        self.drop_last = drop_last

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def __len__(self):
        per = self.n // (self.world * self.batch)
        return per * self.batch

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        order = torch.randperm(self.n, generator=g).tolist() if self.shuffle else list(range(self.n))
        per_rank_batches = self.n // (self.world * self.batch)
        for b in range(self.skip_batches, per_rank_batches):
            base = (b * self.world + self.rank) * self.batch
            for i in range(self.batch):
                yield order[base + i]
        self.skip_batches = 0


class Trainer:
    def __init__(self, model: torch.nn.Module = None, args: TrainingArguments = None, data_collator: Callable = None,
                 train_dataset: Dataset = None, eval_dataset: Dataset = None, tokenizer=None,
                 callbacks: Optional[List[TrainerCallback]] = None, optimizers: Tuple[Any, Any] = (None, None),
                 compute_metrics: Optional[Callable] = None, criterion: Optional[Callable] = None,
                 preprocess_logits_for_metrics: Optional[Callable] = None):
        self.args = args or TrainingArguments()
        self.ps = self.args.setup_parallel()
        set_random_seed(self.args.seed, self.ps)
        self.model = model
        self.data_collator = data_collator or default_data_collator
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        self.tokenizer = tokenizer
        self.compute_metrics = compute_metrics
        self.preprocess_logits_for_metrics = preprocess_logits_for_metrics
        self.criterion = criterion
        self.optimizer, self.lr_scheduler = optimizers
        self.state = TrainerState(is_world_process_zero=self.args.process_index == 0)
        self.control = TrainerControl()
        self.device = torch.device(self.args.device)
        if self.model is not None and next(self.model.parameters()).device != self.device:
            self.model.to(self.device)
        default_cbs: List[TrainerCallback] = [DefaultFlowCallback(), PrinterCallback()]
        if self.args.profile and getattr(self.args, "profile_backend", "cuda_api") == "torch":
            from ..utils.profiler import TorchProfilerCallback

            default_cbs.append(TorchProfilerCallback(self.args.profile_step_start, self.args.profile_step_end))
        elif self.args.profile:
            default_cbs.append(ProfilerCallback())
        if self.args.metrics_output_path:
            default_cbs.append(MetricsDumpCallback(self.args.metrics_output_path))
        if self.args.moe_aux_free_bias_update_rate > 0:
            default_cbs.append(MoECorrectionBiasAdjustCallback(self.args.moe_aux_free_bias_update_rate))
        if getattr(getattr(model, "config", None), "fp8", None):
            default_cbs.append(FP8QuantWeightCallback())
        from .integrations import callbacks_from_args

        default_cbs.extend(callbacks_from_args(self.args))
        self.callback_handler = CallbackHandler(default_cbs + list(callbacks or []), self.model, self.optimizer, self.lr_scheduler)
        self._tr_loss = None
        self._interval_tokens = None
        self._last_log_time = None
        self._last_log_step = 0
        self.pipeline_engine = None
        self.control = self.callback_handler.on_init_end(self.args, self.state, self.control)

    # ------------------------------------------------------------------ public helpers
    def add_callback(self, cb):
        self.callback_handler.add_callback(cb)

    def remove_callback(self, cb):
        self.callback_handler.remove_callback(cb)

    # ------------------------------------------------------------------ data
    def get_train_dataloader(self) -> DataLoader:
        a = self.args
        ds = self.train_dataset
        if ds is None:
            raise ValueError("Trainer: training requires a train_dataset")
        if isinstance(ds, IterableDataset):
            from ..data.dist_dataloader import IterableDatasetShard

            shard = IterableDatasetShard(ds, a.per_device_train_batch_size, a.dataloader_drop_last, a.dataset_world_size,
                                         self.ps.dataset_rank)
            return DataLoader(shard, batch_size=a.per_device_train_batch_size, collate_fn=self.data_collator,
                              num_workers=a.dataloader_num_workers, pin_memory=self.device.type == "cuda")
        self._sampler = ShardedSampler(len(ds), self.ps.dataset_rank, a.dataset_world_size, a.per_device_train_batch_size,
                                       a.data_seed if a.data_seed is not None else a.seed)
        return DataLoader(ds, batch_size=a.per_device_train_batch_size, sampler=self._sampler, collate_fn=self.data_collator,
                          num_workers=a.dataloader_num_workers, pin_memory=self.device.type == "cuda", drop_last=True)

    def get_eval_dataloader(self, eval_dataset=None) -> DataLoader:
        ds = eval_dataset if eval_dataset is not None else self.eval_dataset
        a = self.args
        sampler = ShardedSampler(len(ds), self.ps.dataset_rank, a.dataset_world_size, a.per_device_eval_batch_size, a.seed,
                                 shuffle=False)
        return DataLoader(ds, batch_size=a.per_device_eval_batch_size, sampler=sampler, collate_fn=self.data_collator,
                          pin_memory=self.device.type == "cuda", drop_last=True)

    def _prepare_inputs(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        out = {}
        for k, v in inputs.items():
            if isinstance(v, torch.Tensor):
                if self.device.type == "cuda" and not v.is_cuda:
                    if not v.is_pinned():
                        v = v.pin_memory()
                    v = v.to(self.device, non_blocking=True)
                out[k] = v
            else:
                out[k] = v
        ps = self.ps
        if ps.degrees.cp > 1:
            from ..parallel.context_parallel import get_batch_on_this_cp_rank

            out = get_batch_on_this_cp_rank(out, ps, getattr(self.args, "cp_balance_mode", None) or "dualchunk_allgather")
        if ps.degrees.sep > 1:
            from ..parallel.context_parallel import split_inputs_sequence_dim

            out = split_inputs_sequence_dim(out, ps)
        return out

    # ------------------------------------------------------------------ optimizer
    def create_optimizer_and_scheduler(self, num_training_steps: int):
        a = self.args
        if self.optimizer is None:
            opt_cls, extra = ShardedAdamW, {}
            name = str(getattr(a, "optim", "adamw")).lower()
            if a.sharding == "stage3":
                from ..parallel.fsdp import FullyShardedOptimizer

                if name not in ("adamw", "adamw_torch", "adamw_fused"):
                    raise ValueError("sharding stage3 is implemented for optim=adamw")
                opt_cls = FullyShardedOptimizer
            elif name == "muon":
                from ..parallel.sharding import ShardedMuon

                opt_cls = ShardedMuon
            elif name == "adamw_mini":
                from ..utils.optimizer import AdamWMini

                opt_cls = AdamWMini
            elif name == "adamw_custom" or a.use_lowprecision_moment or a.tensorwise_offload_optimizer or a.hf_bitexact:
                from ..utils.optimizer import AdamWCustom

                opt_cls = AdamWCustom
                extra = dict(moment_dtype=torch.bfloat16 if a.use_lowprecision_moment else torch.float32,
                             offload_moments=a.tensorwise_offload_optimizer, hf_bitexact=a.hf_bitexact)
            elif name not in ("adamw", "adamw_torch", "adamw_fused"):
                raise ValueError(f"optim={a.optim!r}: expected adamw, adamw_mini, adamw_custom or muon")
            self.optimizer = opt_cls(self.model, lr=a.learning_rate, betas=(a.adam_beta1, a.adam_beta2),
                                          eps=a.adam_epsilon, weight_decay=a.weight_decay, max_grad_norm=a.max_grad_norm,
                                          parallel_state=self.ps, release_grads=a.release_grads, **extra)
        if self.lr_scheduler is None:
            min_ratio = a.min_lr / a.learning_rate if a.learning_rate > 0 else 0.0
            fn = get_scheduler_lambda(a.lr_scheduler_type, a.get_warmup_steps(num_training_steps), num_training_steps,
                                      min_lr_ratio=min_ratio, num_cycles=a.num_cycles, power=a.power, decay_steps=a.decay_steps)
            self.lr_scheduler = LRScheduler(a.learning_rate, fn)
        self.callback_handler.optimizer, self.callback_handler.lr_scheduler = self.optimizer, self.lr_scheduler
        self.zcc = None
        if getattr(a, "enable_zero_cost_checkpoint", False) and isinstance(self.optimizer, ShardedAdamW):
            from .zero_cost_checkpoint import ZeroCostCheckpointManager

            self.zcc = ZeroCostCheckpointManager(self.optimizer, self.model)

    # ------------------------------------------------------------------ one micro step
    def compute_loss(self, model, inputs: Dict[str, Any]):
        if self.criterion is not None:
            labels = inputs.pop("labels")
            outputs = model(**inputs, return_logits=True)
            return self.criterion(outputs.logits, labels), outputs
        outputs = model(**inputs)
        return outputs.loss, outputs

    def autocast_context(self):
        return contextlib.nullcontext()

    def training_step(self, model, inputs: Dict[str, Any]) -> torch.Tensor:
        model.train()
        inputs = self._prepare_inputs(inputs)
        if self.args.cuda_graph and self.device.type == "cuda":
            return self._graphed_training_step(model, inputs)
        loss, outputs = self.compute_loss(model, inputs)
        loss.backward()
        self.optimizer.accumulate_grads()
        nt = getattr(outputs, "num_tokens", None)
        if nt is not None:
            self._interval_tokens = nt if self._interval_tokens is None else self._interval_tokens + nt
        return loss.detach()

    def _graphed_training_step(self, model, inputs: Dict[str, Any]) -> torch.Tensor:
        """One micro-batch of forward + backward as a CUDA graph replay. At tensor-parallel degree 8 a decoder layer
        is a few dozen kernels of 10-100 us each, far less than the host needs to launch them through autograd; the
        graph removes the host from the loop. The first ``cuda_graph_warmup`` calls per input signature run eagerly
        (they create workspaces, scratch buffers and function attributes), the next one captures."""
        from ..ops import functional as F

        tensors = {k: v for k, v in inputs.items() if isinstance(v, torch.Tensor)}
        key = tuple(sorted((k, tuple(v.shape), str(v.dtype)) for k, v in tensors.items()))
        graphs = self.__dict__.setdefault("_graphs", {})
        st = graphs.setdefault(key, {"warm": 0})
        if st["warm"] < self.args.cuda_graph_warmup:
            st["warm"] += 1
            loss, outputs = self.compute_loss(model, inputs)
            loss.backward()
            self.optimizer.accumulate_grads()
            nt = getattr(outputs, "num_tokens", None)
            if nt is not None:
                self._interval_tokens = nt if self._interval_tokens is None else self._interval_tokens + nt
            return loss.detach()
        if "graph" not in st:
            static_in = {k: v.clone() for k, v in tensors.items()}
            others = {k: v for k, v in inputs.items() if not isinstance(v, torch.Tensor)}
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
            g = torch.cuda.CUDAGraph()
            n0 = F.kernel_launch_count()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                loss, outputs = self.compute_loss(model, dict(static_in, **others))
                loss.backward()
                self.optimizer.accumulate_grads()
                static_loss = loss.detach()
                ntok = getattr(outputs, "num_tokens", None)
            st.update(graph=g, inputs=static_in, loss=static_loss, ntok=ntok, launches=F.kernel_launch_count() - n0)
        for k, v in tensors.items():
            st["inputs"][k].copy_(v, non_blocking=True)
        st["graph"].replay()
        F.add_replayed_launches(st["launches"])
        if st["ntok"] is not None:
            self._interval_tokens = st["ntok"].clone() if self._interval_tokens is None else self._interval_tokens + st["ntok"]
        return st["loss"].clone()

    def release_graphs(self) -> None:
        """Drop captured CUDA graphs (call before destroying the process group: graphs that captured collectives keep
        communicator resources alive)."""
        import gc

        self.__dict__.pop("_graphs", None)
        gc.collect()
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def _pipeline_engine(self, model):
        if self.pipeline_engine is None:
            from ..parallel.pipeline import PipelineEngine

            self.pipeline_engine = PipelineEngine(model, self.ps, schedule=self.args.pipeline_schedule,
                                                  num_virtual_stages=self.args.virtual_pipeline_model_parallel_size)
        return self.pipeline_engine

    def training_pipeline_step(self, model, micro_batches: List[Dict[str, Any]]) -> torch.Tensor:
        self._pipeline_engine(model)
        batches = [self._prepare_inputs(mb) for mb in micro_batches]
        loss = self.pipeline_engine.forward_backward(batches)
        self.optimizer.accumulate_grads()
        return loss

    # ------------------------------------------------------------------ train
    def train(self, resume_from_checkpoint: Optional[str] = None):
        a = self.args
        model = self.model
        loader = self.get_train_dataloader()
        accum = a.gradient_accumulation_steps
        try:
            steps_per_epoch = max(len(loader) // accum, 1)
        except TypeError:
            steps_per_epoch = None
        if a.max_steps > 0:
            max_steps = a.max_steps
            epochs = math.ceil(max_steps / steps_per_epoch) if steps_per_epoch else 10 ** 9
        else:
            if steps_per_epoch is None:
                raise ValueError("max_steps is required with an iterable dataset")
            max_steps = int(math.ceil(a.num_train_epochs * steps_per_epoch))
            epochs = int(math.ceil(a.num_train_epochs))
        self.state.max_steps, self.state.num_train_epochs = max_steps, epochs
        self.create_optimizer_and_scheduler(max_steps)
        if hasattr(model, "loss_accumulation_steps"):
            model.loss_accumulation_steps = accum

        resume = resume_from_checkpoint if resume_from_checkpoint is not None else a.resume_from_checkpoint
        if resume is True or resume == "auto":
            if getattr(a, "flash_device_path", None):
                # newest checkpoint that verifies, the fast device first; rank 0 copies it under output_dir if it is not there
                from ..utils.ckpt_mirror import restore_latest

                if a.process_index == 0:
                    restore_latest([a.flash_device_path, a.output_dir], a.output_dir)
                if dist.is_initialized() and dist.get_world_size() > 1:
                    dist.barrier()
            resume = get_last_checkpoint(a.output_dir)
        if resume:
            self._load_from_checkpoint(resume)
            self.state.max_steps, self.state.num_train_epochs = max_steps, epochs
        start_step = self.state.global_step
        if dist.is_initialized() and dist.get_world_size() > 1:
            # all ranks must agree on where they resume (paddleformers/trainer/trainer.py:2348-2356)
            t = torch.tensor([start_step], device=self.device if self.device.type == "cuda" else "cpu")
            lo, hi = t.clone(), t.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            if int(lo) != int(hi):
                raise RuntimeError(f"ranks disagree on the resume step: min {int(lo)} max {int(hi)}")

        flops_per_token = None
        if hasattr(model, "get_hardware_flops_per_token"):
            try:
                flops_per_token = model.get_hardware_flops_per_token(a.max_seq_len)
            except Exception:
                flops_per_token = None
        self._flops_per_token = flops_per_token

        self.control = self.callback_handler.on_train_begin(a, self.state, self.control)
        self._tr_loss = torch.zeros((), dtype=torch.float32, device=self.device)
        self._last_log_time, self._last_log_step = time.time(), start_step
        train_start = time.time()
        use_pp = self.ps.degrees.pp > 1
        start_epoch = start_step // steps_per_epoch if steps_per_epoch else 0
        skip_batches = (start_step % steps_per_epoch) * accum if (steps_per_epoch and not a.ignore_data_skip) else 0
        skip_intervals = [tuple(x) for x in (a.skip_data_intervals or [])]

        for epoch in range(start_epoch, epochs):
            if hasattr(self, "_sampler"):
                self._sampler.set_epoch(epoch)
                self._sampler.skip_batches = skip_batches if epoch == start_epoch else 0
            self.control = self.callback_handler.on_epoch_begin(a, self.state, self.control)
            micro: List[Dict[str, Any]] = []
            skip_left = 0
            for step, inputs in enumerate(loader):
                self.control = self.callback_handler.on_load_data_end(a, self.state, self.control, inputs=inputs)
                if skip_left == 0 and len(micro) == 0 and any(lo <= self.state.global_step + 1 <= hi for lo, hi in skip_intervals):
                    # operator-requested skip of poisonous steps (paddleformers/trainer/trainer.py:2490-2547): the whole
                    # global batch of the step (all of its micro-batches) is read and dropped, then the step counter, the
                    # sample counter and the scheduler advance once
                    skip_left = accum
                if skip_left > 0:
                    skip_left -= 1
                    if skip_left == 0:
                        self.state.global_step += 1
                        self.state.consumed_samples += a.global_batch_size
                        self.lr_scheduler.step()
                        if a.max_steps > 0 and self.state.global_step >= max_steps:
                            self.control.should_training_stop = True
                            break
                    continue
                if len(micro) == 0 and not use_pp:
                    self.control = self.callback_handler.on_step_begin(a, self.state, self.control)
                if use_pp:
                    micro.append(inputs)
                    if len(micro) < accum:
                        continue
                    self.control = self.callback_handler.on_step_begin(a, self.state, self.control)
                    self._tr_loss += self.training_pipeline_step(model, micro)
                    micro = []
                else:
                    self._tr_loss += self.training_step(model, inputs)
                    micro.append(None)
                    if len(micro) < accum:
                        self.control = self.callback_handler.on_substep_end(a, self.state, self.control)
                        continue
                    micro = []
                # ---- optimizer step boundary
                self.control = self.callback_handler.on_optimizer_begin(a, self.state, self.control)
                self.optimizer_step()
                self.control = self.callback_handler.on_optimizer_end(a, self.state, self.control)
                self.state.global_step += 1
                self.state.consumed_samples += a.global_batch_size
                self.state.epoch = epoch + (step + 1) / max(len(loader), 1) if steps_per_epoch else 0
                self.control = self.callback_handler.on_step_end(a, self.state, self.control)
                self._maybe_log_save_evaluate()
                if self.control.should_training_stop or self.control.should_epoch_stop:
                    break
            self.control = self.callback_handler.on_epoch_end(a, self.state, self.control)
            self._maybe_log_save_evaluate(epoch_end=True)
            if self.control.should_training_stop:
                break
        metrics = speed_metrics("train", train_start, num_samples=(self.state.global_step - start_step) * a.global_batch_size,
                                num_steps=self.state.global_step - start_step, seq_length=a.max_seq_len,
                                model_flops_per_token=flops_per_token, world_size=a.world_size)
        if a.load_best_model_at_end and self.state.best_model_checkpoint and \
                os.path.isdir(self.state.best_model_checkpoint):
            ckpt.wait_for_pending_saves()
            logger.info(f"loading the best checkpoint {self.state.best_model_checkpoint} (metric {self.state.best_metric})")
            keep = (self.state.global_step, self.state.best_metric, self.state.best_model_checkpoint, self.state.log_history)
            self._load_from_checkpoint(self.state.best_model_checkpoint)
            self.state.global_step, self.state.best_metric, self.state.best_model_checkpoint, self.state.log_history = keep
        self.control = self.callback_handler.on_train_end(a, self.state, self.control)
        self.log(metrics)
        return metrics

    def optimizer_step(self):
        a = self.args
        if a.freeze_training:
            self.optimizer.zero_grad()
            self.lr_scheduler.step()
            return
        lr = self.lr_scheduler.get_lr()
        if getattr(self, "zcc", None) is not None:
            self.zcc.before_update()
        self._last_grad_norm = self.optimizer.step(lr=lr)
        self.lr_scheduler.step()

    # ------------------------------------------------------------------ log / save / eval
    def _maybe_log_save_evaluate(self, epoch_end: bool = False):
        a = self.args
        if self.control.should_log:
            steps = max(self.state.global_step - self._last_log_step, 1)
            loss = self._tr_loss / steps
            # ranks that saw different samples, or different slices of one sequence (cp / sep), each hold a partial mean
            n_parts = self.ps.size("dp_sharding_cp")
            if dist.is_initialized() and n_parts > 1:
                loss = loss.clone()
                dist.all_reduce(loss, group=self.ps.group("dp_sharding_cp"))
                loss = loss / n_parts
            loss_v = float(loss)   # the only host sync of the training loop, on logging steps
            if self.device.type == "cuda":
                # a bounded device wait that ran out or a failed bounds check leaves a code in the device status word; stop
                # here instead of training on wrong numbers
                from ..ops import functional as F

                F.check_kernel_status()
                # routed pairs dropped because an expert-parallel receive buffer was full are counted, not fatal
                # (PFB_EP_OVERFLOW=error makes them fatal)
                from ..parallel.fused_ep import dropped_pairs

                self._ep_dropped = dropped_pairs() if getattr(self.ps.degrees, "ep", 1) > 1 else 0
                # PFB_DEBUG_CANARY=1: guard words behind every peer-visible buffer must be intact
                from ..parallel.fused_collectives import check_canaries

                n_bad = check_canaries()
                if n_bad:
                    raise RuntimeError(f"{n_bad} peer-memory regions were written past their end (PFB_DEBUG_CANARY guard words)")
            if not math.isfinite(loss_v):
                raise FloatingPointError(f"LOSS_{'NAN' if math.isnan(loss_v) else 'INF'}_ERROR: loss is {loss_v} at "
                                         f"step {self.state.global_step}")
            now = time.time()
            dt = max(now - self._last_log_time, 1e-9)
            logs = {"loss": round(loss_v, 6), "learning_rate": self.lr_scheduler.get_lr(), "global_step": self.state.global_step,
                    "epoch": round(self.state.epoch, 4)}
            if a.log_loss_md5 or os.environ.get("LOG_LOSS_MD5", "0") == "1":
                # digest of the fp32 bit pattern: two runs (or two frameworks) agree bit for bit iff the digests match
                # (paddleformers/trainer/trainer.py:3006-3015)
                logs["loss_md5"] = tensor_md5(loss.detach().float().reshape(1))
            gn = getattr(self, "_last_grad_norm", None)
            if gn is not None:
                logs["global_norm"] = round(float(gn), 6)
            if getattr(self, "_ep_dropped", 0):
                logs["moe_dropped_pairs"] = int(self._ep_dropped)
            sps = steps * a.global_batch_size / dt
            logs["interval_runtime"] = round(dt, 4)
            logs["interval_samples_per_second"] = round(sps, 4)
            logs["interval_steps_per_second"] = round(steps / dt, 4)
            tps = sps * a.max_seq_len / max(a.world_size, 1)
            logs["interval_tokens_per_second_per_device"] = round(tps, 2)
            if self._flops_per_token:
                logs["interval_hardware_tflops_per_device"] = round(tps * self._flops_per_token / 2 ** 40, 3)
            if self._interval_tokens is not None:
                real = float(self._interval_tokens) * a.dataset_world_size / max(a.world_size, 1)
                logs["interval_real_tokens_per_second_per_device"] = round(real / dt, 2)
                self.state.trained_tokens += int(float(self._interval_tokens) * a.dataset_world_size)
                self._interval_tokens = None
            logs.update(TrainerMemoryTracker.snapshot())
            self._tr_loss.zero_()
            self._last_log_time, self._last_log_step = now, self.state.global_step
            self.log(logs)
        if self.control.should_evaluate and self.eval_dataset is not None:
            self._last_eval = (self.state.global_step, self.evaluate())
        if self.control.should_save:
            last = getattr(self, "_last_eval", None)      # evaluation and save of one step may come in separate calls
            self._track_best_checkpoint(last[1] if last and last[0] == self.state.global_step else None)   # before the state is written
            self._save_checkpoint()
            self.control = self.callback_handler.on_save(a, self.state, self.control)
        self.control._new_step()

    def _track_best_checkpoint(self, metrics: Optional[Dict[str, float]]):
        """Remember the checkpoint written at the step with the best evaluation metric (``metric_for_best_model``,
        ``greater_is_better``; paddleformers/trainer/trainer.py best-model bookkeeping of the save path)."""
        a = self.args
        if not metrics or not (a.load_best_model_at_end or a.metric_for_best_model):
            return
        name = a.metric_for_best_model or "loss"
        key = name if name.startswith("eval_") else f"eval_{name}"
        if key not in metrics:
            return
        greater = a.greater_is_better if a.greater_is_better is not None else not key.endswith("loss")
        value = float(metrics[key])
        best = self.state.best_metric
        if best is None or (value > best if greater else value < best):
            self.state.best_metric = value
            self.state.best_model_checkpoint = os.path.join(a.output_dir, f"{PREFIX_CHECKPOINT_DIR}-{self.state.global_step}")

    def log(self, logs: Dict[str, float]):
        for cb in self.callback_handler.callbacks:        # callbacks that add fields (timers, memory) run before the sinks
            aug = getattr(cb, "augment_logs", None)
            if aug is not None:
                aug(self.args, self.state, logs)
        self.state.log_history.append(dict(logs))
        self.control = self.callback_handler.on_log(self.args, self.state, self.control, logs=logs)

    @torch.no_grad()
    def evaluate(self, eval_dataset=None, metric_key_prefix: str = "eval") -> Dict[str, float]:
        """Loss and perplexity over the WHOLE evaluation set (token-weighted, summed over the data ranks), plus whatever
        ``compute_metrics`` returns for the gathered predictions. A dict of datasets is evaluated one by one, each under
        ``<prefix>_<name>`` (paddleformers/trainer/trainer.py ``evaluate`` / ``evaluation_loop``)."""
        ds = eval_dataset if eval_dataset is not None else self.eval_dataset
        if isinstance(ds, dict):
            metrics = {}
            for name, one in ds.items():
                metrics.update(self.evaluate(one, f"{metric_key_prefix}_{name}"))
            return metrics
        start = time.time()
        loss, preds, labels, n_batches = self._evaluation_loop(ds, want_predictions=self.compute_metrics is not None)
        metrics = {f"{metric_key_prefix}_loss": loss, f"{metric_key_prefix}_ppl": math.exp(min(loss, 50.0))}
        if self.compute_metrics is not None:
            extra = self.compute_metrics(EvalPrediction(predictions=preds, label_ids=labels)) or {}
            metrics.update({(k if k.startswith(metric_key_prefix + "_") else f"{metric_key_prefix}_{k}"): float(v) for k, v in extra.items()})
        metrics.update(speed_metrics(metric_key_prefix, start, num_samples=len(ds), num_steps=n_batches))
        self.log(metrics)
        self.control = self.callback_handler.on_evaluate(self.args, self.state, self.control, metrics=metrics)
        return metrics

    @torch.no_grad()
    def _whole_sequences(self, pred, lab, inputs):
        """Under context / segment parallelism every rank predicted a slice of the sequence: gather the slices and put every
        token at its global position (predictions with a sequence dimension only); the labels are the unsliced rows."""
        ps = self.ps
        local = inputs["input_ids"].shape[1]
        for axis in ("cp", "sep"):
            n = getattr(ps.degrees, axis)
            if n == 1 or pred.dim() < 2 or pred.shape[1] != local:
                continue
            parts = [torch.empty_like(pred) for _ in range(n)]
            dist.all_gather(parts, pred.contiguous(), group=ps.group(axis))
            if axis == "sep":
                pred = torch.cat(parts, dim=1)
            else:
                from ..parallel.context_parallel import cp_positions

                mode = getattr(self.args, "cp_balance_mode", None) or "dualchunk_allgather"
                whole = torch.empty((pred.shape[0], local * n) + tuple(pred.shape[2:]), dtype=pred.dtype, device=pred.device)
                for r, part in enumerate(parts):
                    whole[:, cp_positions(local * n, n, r, mode, pred.device)] = part
                pred = whole
            if lab is not None and inputs.get("full_labels") is not None:
                lab = inputs["full_labels"]
        return pred, lab

    @torch.no_grad()
    def _evaluation_loop(self, dataset, want_predictions: bool, with_labels: bool = True):
        """(token-weighted mean loss, predictions, labels, batches per rank). Predictions are the arg-max token ids unless
        ``preprocess_logits_for_metrics(logits, labels)`` says otherwise; rows that only fill up the last batch are left out."""
        model = self.model
        was_training = model.training
        model.eval()
        a = self.args
        sampler = EvalSampler(len(dataset), self.ps.dataset_rank, a.dataset_world_size, a.per_device_eval_batch_size)
        loader = DataLoader(dataset, batch_size=a.per_device_eval_batch_size, sampler=sampler, collate_fn=self.data_collator,
                            pin_memory=self.device.type == "cuda")
        tot = torch.zeros((), dtype=torch.float64, device=self.device)
        cnt = torch.zeros((), dtype=torch.float64, device=self.device)
        saved_accum = getattr(model, "loss_accumulation_steps", 1)
        if hasattr(model, "loss_accumulation_steps"):
            model.loss_accumulation_steps = 1
        rows_p, rows_l, n_batches = [], [], 0
        try:
            for b, inputs in enumerate(loader):
                if 0 < a.max_evaluate_steps <= n_batches:
                    break
                inputs = self._prepare_inputs(inputs)
                pad_rows = sampler.padding_rows(b)
                has_labels = with_labels and inputs.get("labels") is not None
                if not with_labels:
                    inputs.pop("labels", None)
                if pad_rows and has_labels:
                    inputs["labels"] = inputs["labels"].clone()
                    inputs["labels"][pad_rows] = -100
                if self.ps.degrees.pp > 1:
                    if want_predictions or not has_labels:
                        raise NotImplementedError("under pipeline parallelism evaluation reports the loss only: predictions "
                                                  "and compute_metrics need the logits, which the last stage does not keep")
                    loss_sum, n = self._pipeline_engine(model).forward_only([inputs])
                    tot += loss_sum
                    cnt += n
                    n_batches += 1
                    self.control = self.callback_handler.on_prediction_step(a, self.state, self.control)
                    continue
                out = model(**inputs, return_logits=True) if want_predictions else model(**inputs)
                if has_labels and out.loss is not None:
                    n = out.num_tokens.double() if out.num_tokens is not None else torch.ones_like(cnt)
                    loss = out.loss.double()
                    for axis in ("cp", "sep"):
                        # ranks that hold slices of one sequence: each loss is this slice's sum over the mean count of a
                        # slice, so their mean is the loss of the sequence; the counts add up
                        if getattr(self.ps.degrees, axis) > 1:
                            pair = torch.stack([loss, n])
                            dist.all_reduce(pair, group=self.ps.group(axis))
                            loss, n = pair[0] / getattr(self.ps.degrees, axis), pair[1]
                    if len(pad_rows) < a.per_device_eval_batch_size:        # a batch of fill-ins only has no valid token
                        tot += loss * n
                        cnt += n
                if want_predictions:
                    keep = [i for i in range(out.logits.shape[0]) if i not in pad_rows]
                    lab = inputs.get("labels")
                    pre = getattr(self, "preprocess_logits_for_metrics", None)
                    pred = pre(out.logits, lab) if pre is not None else out.logits.argmax(-1)
                    pred, lab = self._whole_sequences(pred, lab, inputs)
                    rows_p += [pred[i].cpu() for i in keep]
                    if lab is not None:
                        rows_l += [lab[i].cpu() for i in keep]
                n_batches += 1
                self.control = self.callback_handler.on_prediction_step(a, self.state, self.control)
        finally:
            if hasattr(model, "loss_accumulation_steps"):
                model.loss_accumulation_steps = saved_accum
            model.train(was_training)
        if dist.is_initialized() and self.ps.size("data") > 1:
            both = torch.stack([tot, cnt])
            dist.all_reduce(both, group=self.ps.group("data"))
            tot, cnt = both[0], both[1]
            if want_predictions:
                gathered = [None] * self.ps.size("data")
                dist.all_gather_object(gathered, (rows_p, rows_l), group=self.ps.group("data"))
                # back to dataset order: global batch by global batch, rank by rank
                per = a.per_device_eval_batch_size
                rows_p, rows_l = [], []
                for gb in range(n_batches):
                    for rp, rl in gathered:
                        rows_p += rp[gb * per:(gb + 1) * per]
                        rows_l += rl[gb * per:(gb + 1) * per]
        loss = float(tot / cnt.clamp(min=1))

        def stack(rows):
            if not rows:
                return None
            if rows[0].dim() == 0:
                return torch.stack(rows).numpy()
            width = max(r.shape[0] for r in rows)
            outp = torch.full((len(rows), width) + tuple(rows[0].shape[1:]), -100, dtype=rows[0].dtype)
            for i, r in enumerate(rows):
                outp[i, :r.shape[0]] = r
            return outp.numpy()

        return loss, stack(rows_p), stack(rows_l), n_batches

    def predict(self, test_dataset, metric_key_prefix: str = "test") -> PredictionOutput:
        """Predictions (and, where the set has labels, loss and ``compute_metrics`` results) for every example of the set."""
        start = time.time()
        has_labels = len(test_dataset) > 0 and "labels" in test_dataset[0]
        loss, preds, labels, n_batches = self._evaluation_loop(test_dataset, want_predictions=True, with_labels=has_labels)
        metrics = {}
        if has_labels:
            metrics[f"{metric_key_prefix}_loss"] = loss
            if self.compute_metrics is not None:
                extra = self.compute_metrics(EvalPrediction(predictions=preds, label_ids=labels)) or {}
                metrics.update({f"{metric_key_prefix}_{k}": float(v) for k, v in extra.items()})
        metrics.update(speed_metrics(metric_key_prefix, start, num_samples=len(test_dataset), num_steps=n_batches))
        return PredictionOutput(predictions=preds, label_ids=labels, metrics=metrics)

    # ------------------------------------------------------------------ checkpointing
    def save_model(self, output_dir: Optional[str] = None):
        """Final export: HF-compatible safetensors + config (+ tokenizer files)."""
        output_dir = output_dir or self.args.output_dir
        self.model.save_pretrained(output_dir)
        if self.tokenizer is not None and self.args.process_index == 0 and hasattr(self.tokenizer, "save_pretrained"):
            self.tokenizer.save_pretrained(output_dir)
        if self.args.process_index == 0:
            with open(os.path.join(output_dir, "training_args.json"), "w") as f:
                f.write(self.args.to_json_string())

    def _save_checkpoint(self):
        out = os.path.join(self.args.output_dir, f"{PREFIX_CHECKPOINT_DIR}-{self.state.global_step}")
        from ..ops import functional as F

        if self.device.type == "cuda":
            F.check_kernel_status()      # never persist a state produced after a kernel reported an error
        ckpt.save_checkpoint(self, out)  # rotation happens inside, once the new checkpoint is complete
        if self.args.save_hf_steps > 0 and self.state.global_step % self.args.save_hf_steps == 0:
            self.save_model(os.path.join(self.args.output_dir, f"hf_checkpoint-{self.state.global_step}"))

    def _load_from_checkpoint(self, path: str):
        ckpt.load_checkpoint(self, path)


def default_data_collator(features: List[Dict[str, Any]]) -> Dict[str, torch.Tensor]:
    out = {}
    for k in features[0]:
        vals = [f[k] for f in features]
        if isinstance(vals[0], torch.Tensor):
            out[k] = torch.stack(vals)
        else:
            out[k] = torch.as_tensor(vals)
    return out
