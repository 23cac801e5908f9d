"""Configuration keys of the reference trainer that have no field of their own here.

A YAML written for the reference (paddleformers/trainer/training_args.py, 238 fields) should start a run here without
being edited. Every reference key that is not a field of this package's argument classes is listed below with what
happens to it:

* ``alias``    the value moves to this package's field (optionally through a converter);
* ``builtin``  the behaviour the flag switches on is how this package always works (for example gradients accumulate in
               fp32 ``main_grad`` buffers inside the GEMM epilogue, parameters and gradients live in flat buffers, the
               tensor-parallel collectives are fused into the GEMM kernels): the key is accepted and ignored;
* ``noop``     the key configures something that does not exist in a PyTorch build (static graph, Paddle AMP lists,
               platform hooks): accepted and ignored;
* ``reject``   the key asks for behaviour that is not provided: a truthy value raises, naming what to use instead.

The grouped option strings (``tensor_parallel_config: "enable_mp_async_allreduce ..."`` and the pipeline / sharding /
data / sequence-parallel ones, paddleformers/trainer/training_args.py:1593-1760) are split into their options, and each
option is looked up in the same table with its ``enable_`` prefix removed.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Tuple

from ..utils.log import logger


def _unified(v) -> Tuple[str, Any]:
    return "save_checkpoint_format", "unified" if _truthy(v) else "sharded"


def _truthy(v) -> bool:
    if isinstance(v, str):
        return v.lower() in ("1", "true", "yes", "on")
    return bool(v)


# name -> (kind, payload). alias payload: target field name or a callable value -> (field, value)
REFERENCE_FLAGS: Dict[str, Tuple[str, Any]] = {
    # ---- aliases
    "evaluation_strategy": ("alias", "eval_strategy"),
    "sharding_degree": ("alias", "sharding_parallel_size"),
    "use_async_save": ("alias", "async_save"),
    "use_flex_async_save": ("alias", "async_save"),
    "unified_checkpoint": ("alias", _unified),
    "moe_router_bias_update_rate": ("alias", "moe_aux_free_bias_update_rate"),
    "no_cuda": ("alias", lambda v: ("device", "cpu" if _truthy(v) else None)),
    "use_dualpipev": ("alias", lambda v: ("pipeline_schedule", "zbv" if _truthy(v) else None)),
    "split_backward": ("alias", lambda v: ("pipeline_schedule", "zero_bubble" if _truthy(v) else None)),
    "best_unbalanced_scheduler": ("noop", "a variant of 1F1B warm-up; pick the schedule with pipeline_schedule"),
    "timer": ("alias", "enable_timer"),
    "dataloader_shuffle": ("noop", "the samplers shuffle with `seed` / `data_seed`; set ignore_data_skip for resume behaviour"),
    "deterministic_mode": ("alias", lambda v: ("_env:PFB_ATTN_DETERMINISTIC", "1" if _truthy(v) else None)),
    "sd_release_grads": ("alias", "release_grads"),
    "pp_release_grads": ("alias", "release_grads"),
    "stage1_overlap": ("alias", "sharding_overlap"),
    "overlap": ("alias", "sharding_overlap"),
    "stage2_overlap": ("alias", "sharding_overlap"),
    "sd_sharding_comm_overlap": ("alias", "sharding_overlap"),
    "sd_shardingv1_comm_overlap": ("alias", "sharding_overlap"),
    "pp_sharding_comm_overlap": ("alias", "sharding_overlap"),
    "dp_comm_overlap": ("alias", "sharding_overlap"),
    # ---- how this package always works
    "split_param": ("builtin", "optimizer state and master weights are split by flat-buffer slice (the V2 layout)"),
    "stage1_tensor_fusion": ("builtin", "parameters and gradients live in flat buffers"),
    "tensor_fusion": ("builtin", "parameters and gradients live in flat buffers"),
    "flatten_param_grads": ("builtin", "parameters and gradients live in flat buffers"),
    "fuse_optimizer_states": ("builtin", "master weights and both moments are flat shards updated by one kernel"),
    "stage1_allgather_overlap": ("builtin", "the AdamW kernel stores its bf16 output into every peer's parameter buffer"),
    "stage1_broadcast_overlap": ("builtin", "the AdamW kernel stores its bf16 output into every peer's parameter buffer"),
    "stage1_reduce_avg": ("builtin", "the reduce kernel applies the 1/world scale while it sums"),
    "dp_allreduce_avg_in_gradinent_scale": ("builtin", "the reduce kernel applies the 1/world scale while it sums"),
    "sp_allreduce_avg_in_gradinent_scale": ("builtin", "sequence-parallel parameter gradients are summed once per step"),
    "gradient_sync_after_accumulate": ("builtin", "gradients are reduced once per optimizer step, after accumulation"),
    "mp_fused_linear_param_grad_add": ("builtin", "weight-gradient GEMMs accumulate into fp32 main_grad in their epilogue"),
    "mp_async_allreduce": ("builtin", "tensor-parallel collectives are fused into the GEMM kernels"),
    "tp_async_allreduce": ("builtin", "tensor-parallel collectives are fused into the GEMM kernels"),
    "sp_async_reduce_scatter": ("builtin", "tensor-parallel collectives are fused into the GEMM kernels"),
    "mp_skip_c_identity": ("builtin", "no identity collective is launched"),
    "fuse_sequence_parallel_allreduce": ("builtin", "sequence-parallel parameter gradients travel in one packed all-reduce"),
    "replace_with_c_embedding": ("builtin", "the vocabulary-parallel embedding is the only embedding under tensor parallelism"),
    "replace_with_parallel_cross_entropy": ("builtin", "the vocabulary-parallel fused head + loss is the default"),
    "overlap_p2p_comm": ("builtin", "activations and gradients travel on two communicators with their own streams"),
    "batch_p2p_comm": ("builtin", "activations and gradients travel on two communicators with their own streams"),
    "non_batch_p2p_comm": ("builtin", "activations and gradients travel on two communicators with their own streams"),
    "send_recv_overlap": ("builtin", "activations and gradients travel on two communicators with their own streams"),
    "pp_delay_scale_loss": ("builtin", "the 1/accumulation factor is folded into the loss kernel's gradient"),
    "partial_send_recv": ("builtin", "stages exchange the sequence-parallel slice"),
    "variable_seq_lengths": ("builtin", "packed rows carry their document bounds; no padding to a fixed length"),
    "save_safetensors": ("builtin", "weights are written as Hugging Face safetensors"),
    "convert_from_hf": ("builtin", "checkpoints are read and written in the Hugging Face layout"),
    "load_from_hf": ("builtin", "checkpoints are read and written in the Hugging Face layout"),
    "resume_from_huggingface_ckpt": ("noop", "pass the Hugging Face directory as model_name_or_path"),
    "save_rng_states": ("builtin", "every checkpoint holds the random-number state of each rank"),
    "save_sharded_model": ("builtin", "optimizer state is saved as per-rank shards (save_checkpoint_format: sharded)"),
    "load_sharded_model": ("builtin", "optimizer state is loaded from per-rank shards, re-cut when the layout changed"),
    "use_expert_parallel": ("builtin", "expert parallelism follows expert_model_parallel_size"),
    "hybrid_parallel_expert_grad_scale": ("builtin", "expert gradients are scaled by their own reduction domain"),
    "distributed_dataloader": ("builtin", "one rank per data-parallel group reads and the batch is broadcast"),
    "lazy_data_processing": ("builtin", "datasets tokenise on access"),
    "amp_master_grad": ("builtin", "gradients accumulate in fp32"),
    "tp_sync_param": ("noop", "replicated parameters are initialised from one seed and updated identically"),
    "pp_sync_param": ("noop", "replicated parameters are initialised from one seed and updated identically"),
    "tp_sync_moment": ("noop", "replicated parameters are initialised from one seed and updated identically"),
    "pp_sync_moment": ("noop", "replicated parameters are initialised from one seed and updated identically"),
    "sync_grad": ("noop", "replicated gradients are identical after the sequence-parallel sync"),
    "clear_every_step_cache": ("noop", "the pipeline engine keeps no per-step cache"),
    "p2p_cache_shape": ("noop", "stage-to-stage shapes are static per run"),
    "auto_parallel_sync_shared_params": ("builtin", "tied embeddings on the first and last stage are summed every step"),
    # ---- nothing to configure in a PyTorch build
    "to_static": ("reject", "there is no tracing compiler on the training path; CUDA graphs (cuda_graph: true) remove launch overhead"),
    "enable_auto_parallel": ("reject", "use stage: auto-parallel, which plans over the hand-written strategies"),
    "use_intermediate_api": ("reject", "use stage: auto-parallel"),
    "auto_parallel_resume_form_hybrid_parallel": ("noop", "checkpoints are layout independent (save_checkpoint_format: unified)"),
    "fp16_opt_level": ("noop", "bf16 autocast is not used: kernels take bf16 operands and accumulate in fp32"),
    "amp_custom_black_list": ("noop", "no autocast lists: precision is fixed per kernel"),
    "amp_custom_white_list": ("noop", "no autocast lists: precision is fixed per kernel"),
    "bf16_full_eval": ("noop", "evaluation runs in the model's dtype"),
    "fp16_full_eval": ("noop", "evaluation runs in the model's dtype"),
    "scale_loss": ("noop", "bf16 needs no loss scaling"),
    "local_rank": ("noop", "read from the launcher's environment"),
    "log_on_each_node": ("noop", "rank 0 logs"),
    "save_on_each_node": ("noop", "every rank writes its own shard"),
    "logging_strategy": ("noop", "logging is by steps (logging_steps)"),
    "past_index": ("noop", ""), "run_name": ("noop", ""), "remove_unused_columns": ("noop", ""), "label_names": ("noop", ""),
    "skip_memory_metrics": ("noop", "log_memory switches memory figures on"),
    "ddp_find_unused_parameters": ("noop", "gradients are reduced from flat buffers, unused parameters contribute zeros"),
    "wandb_api_key": ("noop", "report_to supports tensorboard and jsonl"), "wandb_http_proxy": ("noop", ""),
    "pdc_download_ckpt": ("noop", "platform hook"), "pdc_download_timeout": ("noop", "platform hook"),
    "output_signal_dir": ("noop", "completion markers are written next to the checkpoint"),
    "ordered_save_group_size": ("noop", ""), "optim_shard_num": ("noop", ""), "pre_alloc_memory": ("noop", ""),
    "use_cache": ("noop", "training never keeps a key/value cache"),
    "load_via_cpu": ("noop", "safetensors are read through host memory already"),
    "zcc_workers_num": ("noop", "one writer thread per rank"),
    "zcc_pipeline_hooks_capacity_usage": ("noop", "the snapshot is three large copies on a side stream"),
    "fa_version": ("noop", "one attention implementation: the tcgen05 kernels"),
    "offload_queue": ("noop", ""), "reorder_pipeline_priority": ("noop", ""),
    "using_sonic_moe": ("reject", "not provided; the grouped tcgen05 expert GEMMs are used"),
    "forward_backward_overlap_scheduler": ("reject", "not provided; pipeline_schedule: zero_bubble or zbv shorten the bubble"),
    "ckpt_quant_stage": ("reject", "checkpoint quantisation of optimizer state is not provided"),
    "muon_use_symmetric_gemm": ("noop", ""),
}

GROUPED_OPTION_KEYS = ("tensor_parallel_config", "pipeline_parallel_config", "sharding_parallel_config", "data_parallel_config",
                       "sequence_parallel_config", "unified_checkpoint_config")


def translate(cfg: Dict[str, Any], known: set) -> Dict[str, Any]:
    """Returns ``cfg`` with reference-only keys translated; raises on rejected ones. ``known``: this package's fields."""
    out = dict(cfg)
    notes: List[str] = []

    def apply(key: str, value, origin: str):
        kind, payload = REFERENCE_FLAGS[key]
        if kind == "alias":
            field, val = payload(value) if callable(payload) else (payload, value)
            if val is None:
                return
            if field.startswith("_env:"):
                import os

                os.environ[field[5:]] = str(val)
            elif field not in out:
                out[field] = val
            notes.append(f"{origin} -> {field}={val}")
        elif kind == "reject":
            if _truthy(value):
                raise ValueError(f"configuration key {origin}: {payload}")
        else:
            notes.append(f"{origin}: accepted, no effect ({payload})" if payload else f"{origin}: accepted, no effect")

    for key in list(out):
        if key in known:
            continue
        if key in GROUPED_OPTION_KEYS:
            for opt in str(out.pop(key) or "").split():
                name = opt[len("enable_"):] if opt.startswith("enable_") else opt
                if name in REFERENCE_FLAGS:
                    apply(name, True, f"{key}:{opt}")
                elif name in known:
                    out.setdefault(name, True)
                else:
                    notes.append(f"{key}:{opt}: unknown option, ignored")
        elif key in REFERENCE_FLAGS:
            apply(key, out.pop(key), key)
    if isinstance(out.get("recompute_modules"), dict):
        # the reference's refined recompute: {operation: layers that recompute it}, applied on top of per-layer recompute
        out.setdefault("refined_recompute", out.pop("recompute_modules"))
        if not out.get("recompute_granularity"):
            out["recompute_granularity"] = "full"
        notes.append("recompute_modules (per-operation counts) -> refined_recompute with recompute_granularity=full")
    if notes:
        logger.info("reference configuration keys: " + "; ".join(notes))
    return out
