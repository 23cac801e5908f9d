"""Stage router and workflows: ``stage`` in {SFT, PT, DPO} -> build config, model, tokenizer, datasets, collator,
trainer; train; export the final HF checkpoint.

Counterparts: paddleformers/cli/train/tuner.py:33-68 (router), paddleformers/cli/train/sft/workflow.py:196
(``run_sft``) and paddleformers/cli/train/dpo/workflow.py:65 (``run_dpo``).
"""
from __future__ import annotations

import functools
import os
from typing import Optional

import torch

from ..transformers.auto import AutoConfig, AutoModelForCausalLM, AutoTokenizer
from ..transformers.configuration_utils import LlmMetaConfig
from ..utils.log import logger
from .hparams import get_train_args


def _build_model(model_args, train_args, dtype):
    if model_args.model_name_or_path and os.path.isdir(model_args.model_name_or_path) or (model_args.model_name_or_path and not model_args.from_scratch and not model_args.model_type):
        config = AutoConfig.from_pretrained(model_args.model_name_or_path, **(model_args.config_overrides or {}))
    else:
        from ..models.configuration import CONFIG_MAPPING, named_config

        over = model_args.config_overrides or {}
        try:
            config = named_config(model_args.model_type, **over)
        except KeyError:
            config = CONFIG_MAPPING[model_args.model_type](**over)
    LlmMetaConfig.set_llm_config(config, train_args)
    config.dtype = str(dtype).replace("torch.", "")
    device = torch.device(train_args.device)
    # under pipeline parallelism every rank builds (and loads) only the layers of its own stage
    auto_cls = AutoModelForCausalLM
    if train_args.pipeline_model_parallel_size > 1:
        from ..transformers.auto import AutoModelForCausalLMPipe as auto_cls
    if model_args.from_scratch or not model_args.model_name_or_path:
        model = auto_cls.from_config(config, dtype=dtype, device=device)
    else:
        model = auto_cls.from_pretrained(model_args.model_name_or_path, config=config, dtype=dtype, device=device)
    if getattr(config, "fp8", None):
        # block-scaled fp8 forward / input-gradient GEMMs for the dense projections (experts switch on config.fp8 themselves);
        # the vocabulary head and the routers stay in bf16 / fp32
        from ..quantization.fp8 import convert_linears_to_fp8

        n = convert_linears_to_fp8(model)
        logger.info(f"fp8 ({config.fp8}): {n} dense linear layers run block-scaled e4m3 GEMMs")
    if train_args.weight_quantize_algo:
        from ..quantization.weight_only import quantize_model

        n = quantize_model(model, train_args.weight_quantize_algo)
        logger.info(f"quantised {n} linear layers to {train_args.weight_quantize_algo}")
    if model_args.lora:
        from ..peft.lora import LoRAConfig, LoRAModel

        if model_args.lora_path:
            model = LoRAModel.from_pretrained(model, model_args.lora_path)
        else:
            cfg = LoRAConfig(r=model_args.lora_rank, lora_alpha=model_args.lora_alpha, lora_dropout=model_args.lora_dropout,
                             rslora=model_args.rslora, lora_plus_scale=model_args.lora_plus_scale)
            if model_args.lora_target_modules:
                cfg.target_modules = model_args.lora_target_modules
            model = LoRAModel(model, cfg)
        logger.info(model.print_trainable_parameters())
    return model, config


def _tokenizer(model_args):
    if model_args.model_name_or_path:
        try:
            return AutoTokenizer.from_pretrained(model_args.model_name_or_path)
        except Exception as e:  # noqa: BLE001
            logger.warning(f"no tokenizer loaded from {model_args.model_name_or_path}: {e}")
    return None


def run_sft(model_args, data_args, gen_args, train_args, pretrain: bool = False):
    from ..datasets.collate import collate_fn
    from ..datasets.sft_dataset import create_dataset
    from ..trainer.sft_trainer import SFTTrainer

    train_args.setup_parallel()
    dtype = train_args.compute_dtype
    model, config = _build_model(model_args, train_args, dtype)
    tokenizer = _tokenizer(model_args)
    if pretrain and data_args.input_dir:
        from ..data.indexed_dataset import build_train_valid_test_datasets
        from ..trainer.trainer import default_data_collator

        prefix = data_args.input_dir.split()
        n_train = max(train_args.max_steps, 1) * train_args.global_batch_size
        train_ds, eval_ds, _ = build_train_valid_test_datasets(prefix, data_args.split, train_args.max_seq_len,
                                                               [n_train, max(n_train // 100, 1), 0], seed=train_args.seed,
                                                               eos_token_id=getattr(tokenizer, "eos_token_id", None),
                                                               build_masks=model_args.use_attn_mask_startend_row_indices)
        collator = default_data_collator
    else:
        if tokenizer is None:
            raise ValueError("SFT needs a tokenizer (model_name_or_path with tokenizer files)")
        packing = data_args.packing_strategy if data_args.packing else "truncate"
        train_ds = create_dataset(data_args.train_dataset_path, tokenizer, train_args.max_seq_len, data_args.train_dataset_prob,
                                  template=data_args.template, packing=packing, mix_strategy=data_args.mix_strategy,
                                  streaming=data_args.streaming, train_on_prompt=data_args.train_on_prompt or pretrain,
                                  seed=train_args.seed)
        eval_ds = None
        if data_args.eval_dataset_path:
            eval_ds = create_dataset(data_args.eval_dataset_path, tokenizer, train_args.max_seq_len, data_args.eval_dataset_prob,
                                     template=data_args.template, packing=packing)
        collator = functools.partial(collate_fn, tokenizer=tokenizer, training_args=train_args,
                                     max_seq_len=None if data_args.padding_free else train_args.max_seq_len,
                                     padding_free=data_args.padding_free,
                                     use_attn_mask_startend_row_indices=model_args.use_attn_mask_startend_row_indices,
                                     use_global_causal_attn=model_args.use_global_causal_attn)
    trainer = SFTTrainer(model=model, args=train_args, data_collator=collator, train_dataset=train_ds, eval_dataset=eval_ds,
                         tokenizer=tokenizer)
    if model_args.lora and getattr(model_args, "loraga", False) and not model_args.lora_path and not train_args.resume_from_checkpoint:
        import itertools

        from ..peft.lora_ga import lora_ga_init

        ps = train_args.parallel_state
        batches = (trainer._prepare_inputs(b) for b in itertools.islice(iter(trainer.get_train_dataloader()), model_args.loraga_init_iters))
        lora_ga_init(model, batches, model_args.loraga_stable_gamma,
                     dp_group=ps.group("data") if ps.size("data") > 1 else None)
        logger.info(f"LoRA-GA: adapters initialised from {model_args.loraga_init_iters} batches of full-weight gradients")
    metrics = None
    if train_args.do_train:
        metrics = trainer.train(resume_from_checkpoint=train_args.resume_from_checkpoint)
        tokens = train_args.max_seq_len * train_args.global_batch_size * trainer.state.global_step
        rt = metrics.get("train_runtime", 0) or 1e-9
        logger.info(f"Total_Tokens_per_second_per_gpu: {tokens / rt / max(train_args.world_size, 1):.2f}")
        trainer.save_model(train_args.output_dir)
    if train_args.do_eval and eval_ds is not None:
        trainer.evaluate()
    return trainer, metrics


def run_dpo(model_args, data_args, gen_args, train_args):
    from ..datasets.collate import dpo_collate_fn
    from ..datasets.dpo_dataset import create_dpo_dataset
    from ..trainer.dpo_trainer import DPOTrainer

    train_args.setup_parallel()
    dtype = train_args.compute_dtype
    model, config = _build_model(model_args, train_args, dtype)
    tokenizer = _tokenizer(model_args)
    if tokenizer is None:
        raise ValueError("DPO needs a tokenizer")
    ref = None
    if not model_args.lora and train_args.dpo_loss_type not in ("or", "simpo"):
        ref_path = train_args.ref_model_name_or_path or model_args.model_name_or_path
        ref = AutoModelForCausalLM.from_pretrained(ref_path, dtype=dtype, device=torch.device(train_args.device))
    ds = create_dpo_dataset(data_args.train_dataset_path, tokenizer, train_args.max_seq_len, data_args.template)
    collator = functools.partial(dpo_collate_fn, tokenizer=tokenizer, training_args=train_args, max_seq_len=train_args.max_seq_len)
    trainer = DPOTrainer(model=model, args=train_args, data_collator=collator, train_dataset=ds, tokenizer=tokenizer, ref_model=ref,
                         dpo_beta=train_args.dpo_beta, dpo_loss_type=train_args.dpo_loss_type,
                         dpo_label_smoothing=train_args.dpo_label_smoothing, sft_loss_ratio=train_args.sft_loss_ratio)
    metrics = trainer.train(resume_from_checkpoint=train_args.resume_from_checkpoint)
    trainer.save_model(train_args.output_dir)
    return trainer, metrics


def run_tuner(argv: Optional[list] = None):
    from ..utils.numa import maybe_bind_trainer

    maybe_bind_trainer()       # BIND_TRAINER_NUMA=1: CPUs and memory of the NUMA node next to this rank's GPU
    model_args, data_args, gen_args, export_args, train_args = get_train_args(argv)
    stage = model_args.stage.upper()
    if stage == "VL-SFT":
        return run_vl_sft(model_args, data_args, gen_args, train_args)
    if stage == "SFT":
        return run_sft(model_args, data_args, gen_args, train_args)
    if stage == "VL-PT":
        return run_vl_sft(model_args, data_args, gen_args, train_args, pretrain=True)
    if stage == "VL-DPO":
        return run_vl_dpo(model_args, data_args, gen_args, train_args)
    if stage in ("PT", "CPT"):
        return run_sft(model_args, data_args, gen_args, train_args, pretrain=True)
    if stage == "DPO":
        return run_dpo(model_args, data_args, gen_args, train_args)
    if stage in ("AUTO-PARALLEL", "AUTO_PARALLEL"):
        return run_auto_parallel(model_args, data_args, gen_args, train_args)
    if stage in RECIPES:
        return run_recipe_pretrain(stage, model_args, data_args, gen_args, train_args)
    raise ValueError(f"unknown stage {model_args.stage!r}; expected SFT | PT | DPO | VL-SFT | VL-PT | VL-DPO | auto-parallel | "
                     f"{' | '.join(sorted(RECIPES)).lower()}")


# Pre-training recipes: what the reference ships as separate, hand-tuned workflows for one model family each
# (paddleformers/cli/train/deepseek_v3_pretrain/workflow.py:340, paddleformers/cli/train/ernie_pretrain/workflow.py) is here the
# ordinary pre-training workflow with that recipe's switches turned on; every switch the user set explicitly wins.
RECIPES = {
    # MLA + fp8 linears and experts + peer-memory expert exchange + aux-loss-free balancing + overlapped pipeline schedule
    "DSV3_PRETRAIN": dict(fp8="e4m3", moe_token_dispatcher_type="fused", moe_aux_free_bias_update_rate=0.001,
                          recompute_granularity="selective", recompute_modules=["attn"], _pp_schedule="zero_bubble",
                          _model_types=("deepseek_v3", "deepseek_v2", "kimi_k2", "deepseek-v3-4l")),
    # sequence-parallel linears with the all-gather / reduce-scatter fused into the GEMMs + fp8 experts
    "ERNIE_PRETRAIN": dict(fp8="e4m3", moe_token_dispatcher_type="fused", _sequence_parallel=True,
                           _model_types=("ernie4_5", "ernie4_5_moe")),
}
RECIPES["DEEPSEEK_V3_PRETRAIN"] = RECIPES["DSV3_PRETRAIN"]


def apply_recipe(stage: str, model_args, train_args) -> dict:
    """Turns on the recipe's switches that are still at their defaults; returns what was changed."""
    import dataclasses

    recipe = RECIPES[stage.upper()]
    defaults = {f.name: (f.default if f.default is not dataclasses.MISSING else None) for f in dataclasses.fields(train_args)}
    changed = {}

    def put(name, value):
        if name in defaults and getattr(train_args, name) == defaults[name] and value != defaults[name]:
            setattr(train_args, name, value)
            changed[name] = value

    for k, v in recipe.items():
        if not k.startswith("_"):
            put(k, v)
    if recipe.get("_pp_schedule") and train_args.pipeline_model_parallel_size > 1:
        put("pipeline_schedule", recipe["_pp_schedule"])
    if train_args.tensor_model_parallel_size > 1:
        put("sequence_parallel", True)
    mt = (model_args.model_type or "").lower()
    if mt and not model_args.model_name_or_path and mt not in recipe["_model_types"]:
        logger.warning(f"stage {stage}: model_type {mt!r} is not one of {recipe['_model_types']}; the recipe's switches still apply")
    return changed


def run_recipe_pretrain(stage, model_args, data_args, gen_args, train_args):
    changed = apply_recipe(stage, model_args, train_args)
    logger.info(f"stage {stage}: recipe switches {changed}")
    return run_sft(model_args, data_args, gen_args, train_args, pretrain=True)


def _vl_model_and_processor(model_args, data_args, train_args):
    """(model, tokenizer, image processor, placeholder token names) of a vision-language stage."""
    from ..transformers.auto import AutoModelForConditionalGeneration
    from ..transformers.image_processing import Qwen2VLImageProcessor

    train_args.setup_parallel()
    dtype = train_args.compute_dtype
    model = AutoModelForConditionalGeneration.from_pretrained(model_args.model_name_or_path, dtype=dtype,
                                                              device=torch.device(train_args.device))
    tokenizer = _tokenizer(model_args)
    if tokenizer is None:
        raise ValueError("vision-language stages need a tokenizer (model_name_or_path with tokenizer files)")
    vc = model.config.vision_config
    if not isinstance(vc, dict) or "spatial_merge_size" not in vc:    # fixed image size, a fixed number of tokens per image
        from ..transformers.image_processing import SiglipImageProcessor

        size = vc["image_size"] if isinstance(vc, dict) else vc.image_size
        proc = SiglipImageProcessor(image_size=size, tokens_per_image=model.config.num_image_tokens)
        start, end = getattr(model.config, "boi_token_index", None), getattr(model.config, "eoi_token_index", None)
        names = dict(image_token=tokenizer.convert_ids_to_tokens(model.config.image_token_id),
                     vision_start_token=None if start is None else tokenizer.convert_ids_to_tokens(start),
                     vision_end_token=None if end is None else tokenizer.convert_ids_to_tokens(end),
                     emit_token_types=model.config.model_type in ("paligemma", "paligemma2"))      # prompt two-way, answer causal
    else:
        proc_kw = dict(patch_size=vc["patch_size"], merge_size=vc["spatial_merge_size"], temporal_patch_size=vc.get("temporal_patch_size", 1))
        if model.config.model_type == "paddleocr_vl":   # single-frame patches in raster order, pixels in [-1, 1]
            proc_kw.update(raster_order=True, image_mean=(0.5, 0.5, 0.5), image_std=(0.5, 0.5, 0.5))
        for k in ("min_pixels", "max_pixels"):
            if getattr(data_args, k, None):
                proc_kw[k] = getattr(data_args, k)
        if model.config.model_type in ("ernie4_5_vl_moe", "ernie4_5_moe_vl"):      # single-frame patches; frames are paired later
            proc_kw.update(temporal_patch_size=1)
        if model.config.model_type == "qwen3_vl":       # this generation normalises pixels to [-1, 1]
            proc_kw.update(image_mean=(0.5, 0.5, 0.5), image_std=(0.5, 0.5, 0.5))
        proc = Qwen2VLImageProcessor(**proc_kw)
        names = dict(image_token=tokenizer.convert_ids_to_tokens(model.config.image_token_id),
                     vision_start_token=tokenizer.convert_ids_to_tokens(model.config.vision_start_token_id),
                     vision_end_token=tokenizer.convert_ids_to_tokens(model.config.vision_end_token_id))
    return model, tokenizer, proc, names


def run_vl_sft(model_args, data_args, gen_args, train_args, pretrain: bool = False):
    """Supervised fine-tuning of a vision-language model on conversations with images, or (``pretrain``, stage VL-PT)
    next-token training on ``{"text": "... <image> ...", "images": [...]}`` records where every text token is a target
    (paddleformers/cli/train/tuner.py:33-68 routes VL-SFT / VL-PT to the same workflow with multimodal data plugins)."""
    import functools as ft

    from ..datasets.mm_dataset import MMSFTDataset
    from ..models.vision_language import mm_collate_fn
    from ..trainer.trainer import Trainer

    model, tokenizer, proc, names = _vl_model_and_processor(model_args, data_args, train_args)
    train_ds = MMSFTDataset(data_args.train_dataset_path, tokenizer, proc, data_args.template, train_args.max_seq_len,
                            pretrain=pretrain, **names)
    pad = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else 0
    trainer = Trainer(model=model, args=train_args, train_dataset=train_ds, data_collator=ft.partial(mm_collate_fn, pad_token_id=pad),
                      tokenizer=tokenizer)
    metrics = trainer.train(resume_from_checkpoint=train_args.resume_from_checkpoint)
    trainer.save_model(train_args.output_dir)
    return trainer, metrics


def run_vl_dpo(model_args, data_args, gen_args, train_args):
    """Preference optimisation of a vision-language model: prompt (with images) + chosen and + rejected as two rows, a frozen
    copy of the starting model as the reference (none for the reference-free losses)
    (paddleformers/cli/train/dpo/workflow.py:65 with the multimodal plugins)."""
    import functools as ft

    from ..datasets.mm_dataset import MMDPODataset, mm_dpo_collate_fn
    from ..trainer.dpo_trainer import DPOTrainer
    from ..transformers.auto import AutoModelForConditionalGeneration

    model, tokenizer, proc, names = _vl_model_and_processor(model_args, data_args, train_args)
    ref = None
    if train_args.dpo_loss_type not in ("or", "simpo"):
        ref = AutoModelForConditionalGeneration.from_pretrained(train_args.ref_model_name_or_path or model_args.model_name_or_path,
                                                                dtype=train_args.compute_dtype, device=torch.device(train_args.device))
    ds = MMDPODataset(data_args.train_dataset_path, tokenizer, proc, data_args.template, train_args.max_seq_len, **names)
    pad = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else 0
    trainer = DPOTrainer(model=model, args=train_args, data_collator=ft.partial(mm_dpo_collate_fn, pad_token_id=pad), train_dataset=ds,
                         tokenizer=tokenizer, ref_model=ref, dpo_beta=train_args.dpo_beta, dpo_loss_type=train_args.dpo_loss_type,
                         dpo_label_smoothing=train_args.dpo_label_smoothing, sft_loss_ratio=train_args.sft_loss_ratio)
    metrics = trainer.train(resume_from_checkpoint=train_args.resume_from_checkpoint)
    trainer.save_model(train_args.output_dir)
    return trainer, metrics


def run_auto_parallel(model_args, data_args, gen_args, train_args):
    """Pre-training with the parallel degrees chosen by ``parallel.auto_plan`` for this job's GPU count (the role of
    the reference's auto-parallel stage, paddleformers/cli/train/auto_parallel/workflow.py): any degree the user left
    at 1 is overwritten by the plan, then the PT workflow runs unchanged."""
    import os

    from ..models.configuration import CONFIG_MAPPING, named_config
    from ..parallel.auto_plan import plan_parallelism

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if model_args.model_name_or_path and not model_args.from_scratch:
        config = AutoConfig.from_pretrained(model_args.model_name_or_path)
    else:
        try:
            config = named_config(model_args.model_type)
        except KeyError:
            config = CONFIG_MAPPING[model_args.model_type]()
    plan = plan_parallelism(config, world, train_args.max_seq_len, train_args.per_device_train_batch_size,
                            recompute=getattr(train_args, "recompute_granularity", None) == "full")
    logger.info(f"auto-parallel plan for {world} GPU(s): {plan.reason}")
    for k, v in plan.training_args().items():
        if hasattr(train_args, k) and getattr(train_args, k) in (1, "", False, None):
            setattr(train_args, k, v)
    return run_sft(model_args, data_args, gen_args, train_args, pretrain=True)


if __name__ == "__main__":
    run_tuner()
