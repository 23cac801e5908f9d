"""Hybrid-parallel logic on CPU ranks (gloo): every strategy must reproduce the single-process losses."""
import os

import pytest
import torch

from dist_utils import run_distributed


def _tiny_cfg(moe=False, **kw):
    from paddleformers_b200.models.configuration import named_config

    if moe == "gemma4":          # dense + routed feed-forward sum, two head geometries, per-layer inputs
        from paddleformers_b200.transformers.auto import AutoConfig

        base = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=16, global_head_dim=32, sliding_window=8, vocab_size_per_layer_input=128,
                    hidden_size_per_layer_input=8, enable_moe_block=True, num_experts=4, top_k_experts=2, moe_intermediate_size=32,
                    attention_k_eq_v=True, num_global_key_value_heads=2)
        base.update(kw)
        return AutoConfig.for_model("gemma4_text", **base)
    if isinstance(moe, str) and moe.startswith("fam:"):       # any family of the registry at tiny size
        from paddleformers_b200.transformers.auto import AutoConfig

        base = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=16, max_position_embeddings=128)
        extra = {"mixtral": dict(num_local_experts=4, num_experts_per_tok=2),
                 "qwen2_moe": dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=48),
                 "ernie4_5_moe": dict(moe_num_experts=4, moe_k=2, moe_intermediate_size=32, moe_num_shared_experts=1, moe_layer_start_index=1),
                 "gpt_oss": dict(num_local_experts=4, num_experts_per_tok=2, sliding_window=8),
                 "gemma3_text": dict(sliding_window=8, query_pre_attn_scalar=16)}.get(moe[4:].replace("+noaux", ""), {})
        base.update(extra)
        base.update(kw)
        if moe.endswith("+noaux"):
            base["router_aux_loss_coef"] = 0.0
            return AutoConfig.for_model(moe[4:-6], **base)
        return AutoConfig.for_model(moe[4:], **base)
    if moe == "mla":             # latent attention + sigmoid group-limited router + shared expert + one MTP layer
        from paddleformers_b200.transformers.auto import AutoConfig

        base = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=4, n_routed_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, n_shared_experts=1,
                    first_k_dense_replace=1, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                    n_group=2, topk_group=1, num_nextn_predict_layers=1, max_position_embeddings=128)
        base.update(kw)
        return AutoConfig.for_model("deepseek_v3", **base)
    if moe == "tied":            # dense, the head shares the embedding table
        kw = dict(kw, tie_word_embeddings=True)
        moe = False
    if moe:
        base = dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                    num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, vocab_size=128, router_aux_loss_coef=0.0)
        base.update(kw)
        return named_config("qwen3-30b-a3b", **base)
    base = dict(num_hidden_layers=2, hidden_size=64, intermediate_size=96, num_attention_heads=4, num_key_value_heads=2,
                head_dim=16, vocab_size=128)
    base.update(kw)
    return named_config("tiny-llama", **base)


def _data(n, S=32, vocab=128):
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, vocab, (n, S + 1), generator=g)
    labels = ids[:, 1:].clone()
    labels[:, :3] = -100                  # prompt positions without a label
    labels[::2, 17] = -100
    return [{"input_ids": ids[i, :-1], "labels": labels[i]} for i in range(n)]


class _DS(torch.utils.data.Dataset):
    def __init__(self, items):
        self.items = items

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]


def _train(rank, world, moe, targs, steps, full_state):
    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.models.modeling import DecoderForCausalLM, MODEL_MAPPING
    from paddleformers_b200.transformers.model_utils import param_shard_spec
    from paddleformers_b200.transformers.conversion_utils import ShardSpec

    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=1, max_steps=steps,
                             learning_rate=1e-2, lr_scheduler_type="constant", logging_steps=1, save_strategy="no",
                             max_seq_len=32, max_grad_norm=1.0, seed=3, device="cpu", **targs)
    ps = args.setup_parallel()
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig

    cfg = _tiny_cfg(moe)
    LlmMetaConfig.set_llm_config(cfg, args)
    model = MODEL_MAPPING[cfg.model_type](cfg)
    # load the same full weights on every configuration, cut for this rank
    with torch.no_grad():
        for name, p in model.named_parameters():
            spec = param_shard_spec(p)
            p.copy_(spec.shard(full_state[name], ps.coord["mp"], ps.degrees.mp, ps.rank_in("ep"), ps.degrees.ep))
    ds = _DS(_data(8 * steps))
    tr = Trainer(model=model, args=args, train_dataset=ds)
    tr._sampler_shuffle = False
    tr.train()
    # the gradient norm of the first step rides along as a fourth number: it reacts to a wrong or missing gradient
    # reduction long before the losses of a few steps do
    return [h["loss"] for h in tr.state.log_history if "loss" in h] + [tr.state.log_history[0]["global_norm"]]


def _reference(moe, steps, accum):
    from paddleformers_b200.models.modeling import MODEL_MAPPING

    torch.manual_seed(5)
    cfg = _tiny_cfg(moe)
    model = MODEL_MAPPING[cfg.model_type](cfg)
    full = {k: v.detach().clone() for k, v in model.named_parameters()}
    return full


_REF_CACHE = {}


def _single_process_run(worker, kind, single, steps, full):
    """The single-process trajectory of a model kind is the same for every strategy that is compared with it: run it once."""
    key = (worker.__name__, kind, tuple(sorted(single.items())), steps)
    if key not in _REF_CACHE:
        _REF_CACHE[key] = run_distributed(worker, 1, kind, single, steps, full)[0]
    return _REF_CACHE[key]


@pytest.mark.parametrize("name,world,moe,targs", [
    ("tp2_sp", 2, False, dict(tensor_model_parallel_size=2, sequence_parallel=True, gradient_accumulation_steps=2)),
    ("tp2", 2, False, dict(tensor_model_parallel_size=2, gradient_accumulation_steps=2)),
    ("tp2_sp_filtered_loss", 2, False, dict(tensor_model_parallel_size=2, sequence_parallel=True, gradient_accumulation_steps=2,
                                            use_filtered_label_loss=True)),
    ("tp2_sp_refined_recompute", 2, False, dict(tensor_model_parallel_size=2, sequence_parallel=True, gradient_accumulation_steps=2,
                                                recompute_granularity="full",
                                                refined_recompute={"flash_attn": 0, "attention_column_ln": 0, "mlp_row_ln": 1})),
    ("sharding2", 2, False, dict(sharding="stage1", gradient_accumulation_steps=1)),
    ("sharding2_custom_adamw", 2, False, dict(sharding="stage1", gradient_accumulation_steps=1, optim="adamw_custom",
                                              tensorwise_offload_optimizer=True)),
    ("dp2", 2, False, dict(gradient_accumulation_steps=1)),
    ("stage3_fsdp2", 2, False, dict(sharding="stage3", gradient_accumulation_steps=1)),
    ("ep2", 2, True, dict(expert_model_parallel_size=2, sharding="stage1", gradient_accumulation_steps=1, moe_token_dispatcher_type="alltoall")),
    ("gemma4_ep2", 2, "gemma4", dict(expert_model_parallel_size=2, sharding="stage1", gradient_accumulation_steps=1,
                                     moe_token_dispatcher_type="alltoall")),
    ("tp2_qk_norm_moe", 2, True, dict(tensor_model_parallel_size=2, gradient_accumulation_steps=2, moe_token_dispatcher_type="alltoall")),
    ("tp2_sp_qk_norm_moe", 2, True, dict(tensor_model_parallel_size=2, sequence_parallel=True, gradient_accumulation_steps=2,
                                         moe_token_dispatcher_type="alltoall")),
    ("tp2_sp_ep2_moe", 4, True, dict(tensor_model_parallel_size=2, sequence_parallel=True, expert_model_parallel_size=2, sharding="stage1",
                                     gradient_accumulation_steps=1, moe_token_dispatcher_type="alltoall")),
    ("tp2_ep2_moe", 4, True, dict(tensor_model_parallel_size=2, expert_model_parallel_size=2, sharding="stage1",
                                  gradient_accumulation_steps=1, moe_token_dispatcher_type="alltoall")),
    ("ep2_cp2_moe", 4, True, dict(expert_model_parallel_size=2, context_parallel_size=2, sharding="stage1", gradient_accumulation_steps=1,
                                  moe_token_dispatcher_type="alltoall")),
    ("ep2_sep2_moe", 4, True, dict(expert_model_parallel_size=2, sep_parallel_size=2, sharding="stage1", gradient_accumulation_steps=1,
                                   moe_token_dispatcher_type="alltoall")),
    ("tp2_cp2", 4, False, dict(tensor_model_parallel_size=2, context_parallel_size=2, gradient_accumulation_steps=2)),
    # latent attention (shared rotary key read by every rank's heads), multi-token prediction (weighted term, look-ahead across
    # slices), sigmoid group-limited router with shared expert
    ("mla_mtp_tp2", 2, "mla", dict(tensor_model_parallel_size=2, gradient_accumulation_steps=2, moe_token_dispatcher_type="alltoall")),
    ("mla_mtp_tp2_sp", 2, "mla", dict(tensor_model_parallel_size=2, sequence_parallel=True, gradient_accumulation_steps=2,
                                      moe_token_dispatcher_type="alltoall")),
    ("mla_mtp_cp2", 2, "mla", dict(context_parallel_size=2, gradient_accumulation_steps=2, moe_token_dispatcher_type="alltoall")),
    ("mla_mtp_ep2", 2, "mla", dict(expert_model_parallel_size=2, sharding="stage1", gradient_accumulation_steps=1,
                                   moe_token_dispatcher_type="alltoall")),
    ("gemma4_tp2", 2, "gemma4", dict(tensor_model_parallel_size=2, gradient_accumulation_steps=2, moe_token_dispatcher_type="alltoall")),
    ("cp2", 2, False, dict(context_parallel_size=2, gradient_accumulation_steps=2)),
    ("cp2_contiguous", 2, False, dict(context_parallel_size=2, cp_balance_mode="contiguous_allgather", gradient_accumulation_steps=2)),
    ("cp2_ring", 2, False, dict(context_parallel_size=2, context_parallel_algo="ring", gradient_accumulation_steps=2)),
    ("sep2", 2, False, dict(sep_parallel_size=2, gradient_accumulation_steps=2)),
])
def test_parallel_matches_single_process(name, world, moe, targs):
    steps = 3
    full = _reference(moe, steps, 2)
    single = dict(gradient_accumulation_steps=2)
    if moe:
        single["moe_token_dispatcher_type"] = "alltoall"
    ref = _single_process_run(_train, moe, single, steps, full)
    got = run_distributed(_train, world, moe, targs, steps, full)
    for r in range(world):
        assert len(got[r]) == steps + 1
        for a, b in zip(ref, got[r]):
            assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (name, ref, got[r])


def _train_pp(rank, world, moe, targs, steps, full_state):
    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.parallel.pipeline import build_pipeline_model
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig
    from paddleformers_b200.transformers.model_utils import param_shard_spec

    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=1, max_steps=steps,
                             learning_rate=1e-2, lr_scheduler_type="constant", logging_steps=1, save_strategy="no",
                             max_seq_len=32, max_grad_norm=1.0, seed=3, device="cpu", **targs)
    ps = args.setup_parallel()
    cfg = _tiny_cfg(moe, num_hidden_layers=4)
    LlmMetaConfig.set_llm_config(cfg, args)
    model = build_pipeline_model(cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            g = model.global_param_name(name)
            spec = param_shard_spec(p)
            p.copy_(spec.shard(full_state[g], ps.coord["mp"], ps.degrees.mp, ps.rank_in("ep"), ps.degrees.ep))
    tr = Trainer(model=model, args=args, train_dataset=_DS(_data(8 * steps)))
    tr.train()
    return [h["loss"] for h in tr.state.log_history if "loss" in h] + [tr.state.log_history[0]["global_norm"]]


def _train_single4(rank, world, moe, targs, steps, full_state):
    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.models.modeling import MODEL_MAPPING

    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=1, max_steps=steps,
                             learning_rate=1e-2, lr_scheduler_type="constant", logging_steps=1, save_strategy="no",
                             max_seq_len=32, max_grad_norm=1.0, seed=3, device="cpu", **targs)
    args.setup_parallel()
    cfg = _tiny_cfg(moe, num_hidden_layers=4)
    model = MODEL_MAPPING[cfg.model_type](cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            p.copy_(full_state[name])
    tr = Trainer(model=model, args=args, train_dataset=_DS(_data(8 * steps)))
    tr.train()
    return [h["loss"] for h in tr.state.log_history if "loss" in h] + [tr.state.log_history[0]["global_norm"]]


@pytest.mark.parametrize("name,targs", [
    ("pp2_1f1b", dict(pipeline_model_parallel_size=2, gradient_accumulation_steps=4)),
    ("pp2_interleaved", dict(pipeline_model_parallel_size=2, virtual_pipeline_model_parallel_size=2, gradient_accumulation_steps=4,
                             pipeline_schedule="interleaved")),
    ("pp2_zero_bubble", dict(pipeline_model_parallel_size=2, gradient_accumulation_steps=4, pipeline_schedule="zero_bubble")),
    ("pp2_zbv", dict(pipeline_model_parallel_size=2, gradient_accumulation_steps=4, pipeline_schedule="zbv")),
    ("pp2_1f1b_refined_recompute", dict(pipeline_model_parallel_size=2, gradient_accumulation_steps=4, recompute_granularity="full",
                                        refined_recompute={"flash_attn": 0, "mlp_column_ln": 2})),
    ("pp2_zero_bubble_refined_recompute", dict(pipeline_model_parallel_size=2, gradient_accumulation_steps=4,
                                               pipeline_schedule="zero_bubble", recompute_granularity="full",
                                               refined_recompute={"attention_row_ln": 0, "mlp_row_ln": 0})),
])
def test_pipeline_matches_single_process(name, targs):
    _pipeline_case(name, 2, False, targs, 4)


@pytest.mark.parametrize("name,world,kind,targs,single_accum", [
    # stages hand over token slices under sequence parallelism; the last stage gathers them for the loss
    ("pp2_tp2_sp", 4, False, dict(pipeline_model_parallel_size=2, tensor_model_parallel_size=2, sequence_parallel=True,
                                  gradient_accumulation_steps=4), 4),
    # a head tied to the input embedding: the gradients of both copies are summed, the norm counts them once
    ("pp2_tied", 2, "tied", dict(pipeline_model_parallel_size=2, gradient_accumulation_steps=4), 4),
    ("pp2_tied_zbv", 2, "tied", dict(pipeline_model_parallel_size=2, gradient_accumulation_steps=4, pipeline_schedule="zbv"), 4),
    # ... and to a vocabulary-parallel embedding: the last stage holds a vocabulary shard
    ("pp2_tp2_tied", 4, "tied", dict(pipeline_model_parallel_size=2, tensor_model_parallel_size=2, gradient_accumulation_steps=4), 4),
    ("pp2_tp2_sp_tied", 4, "tied", dict(pipeline_model_parallel_size=2, tensor_model_parallel_size=2, sequence_parallel=True,
                                        gradient_accumulation_steps=4), 4),
    # experts sharded inside every stage
    ("pp2_ep2_moe", 4, True, dict(pipeline_model_parallel_size=2, expert_model_parallel_size=2, sharding="stage1",
                                  gradient_accumulation_steps=2, moe_token_dispatcher_type="alltoall"), 4),
    ("pp2_ep2_moe_zero_bubble", 4, True, dict(pipeline_model_parallel_size=2, expert_model_parallel_size=2, sharding="stage1",
                                              gradient_accumulation_steps=2, pipeline_schedule="zero_bubble",
                                              moe_token_dispatcher_type="alltoall"), 4),
    # stages hold slices of one sequence: global positions and the labelled-token count of the whole sequence reach the stages
    ("pp2_cp2", 4, False, dict(pipeline_model_parallel_size=2, context_parallel_size=2, gradient_accumulation_steps=4), 4),
    ("pp2_sep2", 4, False, dict(pipeline_model_parallel_size=2, sep_parallel_size=2, gradient_accumulation_steps=4), 4),
    # multi-token prediction on the last stage: its embedding copy is a vocabulary shard like the first stage's table
    ("pp2_tp2_mla_mtp", 4, "mla", dict(pipeline_model_parallel_size=2, tensor_model_parallel_size=2, gradient_accumulation_steps=4,
                                       moe_token_dispatcher_type="alltoall"), 4),
])
def test_pipeline_with_tensor_and_expert_parallelism(name, world, kind, targs, single_accum):
    _pipeline_case(name, world, kind, targs, single_accum)


def _pipeline_case(name, world, kind, targs, single_accum):
    from paddleformers_b200.models.modeling import MODEL_MAPPING

    steps = 2
    torch.manual_seed(5)
    cfg = _tiny_cfg(kind, num_hidden_layers=4)
    full = {k: v.detach().clone() for k, v in MODEL_MAPPING[cfg.model_type](cfg).named_parameters()}
    single = dict(gradient_accumulation_steps=single_accum)
    if kind is True or kind == "mla":
        single["moe_token_dispatcher_type"] = "alltoall"
    ref = _single_process_run(_train_single4, kind, single, steps, full)
    got = run_distributed(_train_pp, world, kind, targs, steps, full)
    for r in range(world):
        for a, b in zip(ref, got[r]):
            assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (name, ref, got[r])


def _cp_attention_worker(rank, world, mode):
    """Blocked all-gather attention with document bounds on a cp-sharded sequence against full attention."""
    from paddleformers_b200.ops import functional as F
    from paddleformers_b200.parallel.context_parallel import cp_attention, cp_positions
    from paddleformers_b200.parallel.topology import ParallelDegrees, initialize_parallel

    ps = initialize_parallel(ParallelDegrees(cp=world), backend="gloo")
    g = torch.Generator().manual_seed(21)
    B, S, Hq, Hkv, D = 2, 32, 4, 2, 8
    q, k, v = (torch.randn(B, S, h, D, generator=g) for h in (Hq, Hkv, Hkv))
    # two packed documents per row: keys of the first document are invisible to rows >= 12 (row 0) / 20 (row 1)
    kend = torch.full((B, S), S, dtype=torch.int32)
    kend[0, :12], kend[1, :20] = 12, 20
    ref = F.attention_reference(q, k, v, True, kend)
    idx = cp_positions(S, world, ps.coord["cp"], mode, q.device)
    ql, kl, vl = (t.index_select(1, idx).requires_grad_(True) for t in (q, k, v))
    out = cp_attention(ql, kl, vl, idx, S, mode, ps.group("cp"), None, kend, block=8)
    err = (out - ref.index_select(1, idx)).abs().max().item()
    out.sum().backward()          # the gathered K/V gradients flow back through the reduce-scatter
    return err, float(kl.grad.abs().sum())


@pytest.mark.parametrize("mode", ["dualchunk_allgather", "contiguous_allgather"])
def test_cp_attention_blocked_with_document_mask(mode):
    res = run_distributed(_cp_attention_worker, 2, mode)
    for err, gsum in res:
        assert err < 1e-5 and gsum > 0


@pytest.mark.parametrize("P,M", [(2, 4), (4, 8), (8, 16), (8, 32)])
def test_zero_bubble_schedule_shortens_the_pipeline(P, M):
    """Timed simulation with unit costs (F = B = W = 1, fused backward = 2): splitting the backward pass removes the
    weight-gradient share of the bubble at unchanged activation memory."""
    from paddleformers_b200.parallel.pipeline import make_schedule, simulate

    base = simulate([make_schedule("1F1B", s, P, M) for s in range(P)], P, 1)
    zb = simulate([make_schedule("zero_bubble", s, P, M) for s in range(P)], P, 1)
    assert base["makespan"] == 3 * M + 3 * (P - 1)
    assert zb["makespan"] == 3 * M + 2 * (P - 1)
    assert zb["peak_live"] == base["peak_live"] == list(range(P, 0, -1))
    assert zb["bubble_fraction"] < base["bubble_fraction"]


@pytest.mark.parametrize("P,M", [(2, 4), (4, 8), (8, 16), (8, 32)])
def test_v_placement_schedule_is_valid_and_nearly_bubble_free(P, M):
    from paddleformers_b200.parallel.pipeline import (make_schedule, partition_layers, simulate, stage_of_virtual,
                                                      virtual_stage)

    # placement: down the stages with chunk 0, back up with chunk 1; first and last part of the model on stage 0
    order = [stage_of_virtual(v, P, True) for v in range(2 * P)]
    assert order[0] == (0, 0) and order[P - 1] == (P - 1, 0) and order[P] == (P - 1, 1) and order[-1] == (0, 1)
    assert all(virtual_stage(s, c, P, True) == v for v, (s, c) in enumerate(order))
    parts = partition_layers(4 * P, P, 2, v_shape=True)
    assert parts[0][0] == range(0, 2) and parts[0][1] == range(4 * P - 2, 4 * P) and parts[P - 1][0].stop == parts[P - 1][1].start
    sch = [make_schedule("zbv", s, P, M, 2) for s in range(P)]
    for s in range(P):                       # every chunk of every micro-batch runs F, B and W exactly once
        assert sorted((a.kind, a.chunk, a.mb) for a in sch[s]) == sorted((k, c, m) for k in "FBW" for c in (0, 1) for m in range(M))
    unit = {"F": 1.0, "B": 1.0, "W": 1.0}    # one half-size chunk = one unit per pass
    r = simulate(sch, P, 2, unit, v_shape=True)
    one = simulate([make_schedule("1f1b", s, P, M, 1) for s in range(P)], P, 1, {"F": 2.0, "B": 4.0})
    zb = simulate([make_schedule("zero_bubble", s, P, M, 1) for s in range(P)], P, 1, {"F": 2.0, "B": 2.0, "W": 2.0})
    assert r["makespan"] < zb["makespan"] < one["makespan"]
    assert r["bubble_fraction"] < 0.6 * one["bubble_fraction"]
    assert max(r["peak_live"]) <= 2 * P + 1       # half-size chunks: about the activation memory of 1F1B's first stage


def test_nccl_group_config_parsing_and_options():
    import torch.distributed as dist

    from paddleformers_b200.parallel.nccl_config import group_options, load_nccl_config, make_pg_options

    cfg = load_nccl_config('{"default": {"cga_cluster_size": 2}, "mp": {"high_priority": true, "max_ctas": 16}}')
    assert group_options(cfg, "mp") == {"cga_cluster_size": 2, "high_priority": True, "max_ctas": 16}
    assert group_options(cfg, "pp") == {"cga_cluster_size": 2}
    assert make_pg_options(cfg, "mp", "gloo") is None and make_pg_options({}, "mp", "nccl") is None
    if hasattr(dist, "ProcessGroupNCCL"):
        o = make_pg_options(cfg, "mp", "nccl")
        assert o.is_high_priority_stream and o.config.max_ctas == 16 and o.config.cga_cluster_size == 2
    with pytest.raises(ValueError, match="unknown option"):
        load_nccl_config({"mp": {"ctas": 3}})
    with pytest.raises(ValueError, match="unknown group"):
        load_nccl_config({"tp": {"max_ctas": 3}})


def _train_and_save(rank, world, targs, steps, full_state, out_dir, resume):
    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.models.modeling import MODEL_MAPPING
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig
    from paddleformers_b200.transformers.model_utils import param_shard_spec

    args = TrainingArguments(output_dir=out_dir, per_device_train_batch_size=1, max_steps=steps, learning_rate=1e-2,
                             lr_scheduler_type="constant", logging_steps=1, save_steps=2, max_seq_len=32, max_grad_norm=1.0,
                             seed=3, device="cpu", **targs)
    ps = args.setup_parallel()
    cfg = _tiny_cfg(False)
    LlmMetaConfig.set_llm_config(cfg, args)
    model = MODEL_MAPPING[cfg.model_type](cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            p.copy_(param_shard_spec(p).shard(full_state[name], ps.coord["mp"], ps.degrees.mp, ps.rank_in("ep"), ps.degrees.ep))
    tr = Trainer(model=model, args=args, train_dataset=_DS(_data(8 * 4)))
    tr._sampler_shuffle = False
    tr.train(resume_from_checkpoint="auto" if resume else None)
    return [h["loss"] for h in tr.state.log_history if "loss" in h]


def test_resume_with_a_different_sharding_degree(tmp_path):
    """Optimizer shards written by 2 sharding ranks are re-cut for 1 rank; the run continues like an uninterrupted one."""
    full = _reference(False, 4, 2)
    ref = run_distributed(_train_and_save, 1, dict(gradient_accumulation_steps=2), 4, full, str(tmp_path / "ref"), False)[0]
    run_distributed(_train_and_save, 2, dict(sharding="stage1", gradient_accumulation_steps=1), 2, full, str(tmp_path / "run"), False)
    got = run_distributed(_train_and_save, 1, dict(gradient_accumulation_steps=2), 4, full, str(tmp_path / "run"), True)[0]
    assert len(got) >= 2
    for a, b in zip(ref[2:], got[-2:]):
        assert abs(a - b) < 3e-4 * max(1.0, abs(a)), (ref, got)


def test_stage3_checkpoint_resumes_on_the_same_and_on_another_number_of_ranks(tmp_path):
    """Parameters, gradients and optimizer state sharded per layer over 2 ranks: the exported weights are whole, and the run
    resumes from its per-unit slices on 2 ranks and (re-cut) on 1 rank like an uninterrupted single-process run."""
    from paddleformers_b200.transformers.auto import AutoModelForCausalLM

    full = _reference(False, 4, 2)
    ref = run_distributed(_train_and_save, 1, dict(gradient_accumulation_steps=2), 4, full, str(tmp_path / "ref"), False)[0]
    s3 = dict(sharding="stage3", gradient_accumulation_steps=1)
    run_distributed(_train_and_save, 2, s3, 2, full, str(tmp_path / "run"), False)
    # the checkpoint's Hugging Face weights equal those of the single-process run at the same step
    a = AutoModelForCausalLM.from_pretrained(str(tmp_path / "run" / "checkpoint-2"), dtype=torch.float32)
    b = AutoModelForCausalLM.from_pretrained(str(tmp_path / "ref" / "checkpoint-2"), dtype=torch.float32)
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        torch.testing.assert_close(p, q, rtol=1e-4, atol=1e-5, msg=n)
    import shutil

    shutil.copytree(str(tmp_path / "run"), str(tmp_path / "run1"))
    got2 = run_distributed(_train_and_save, 2, s3, 4, full, str(tmp_path / "run"), True)[0]
    got1 = run_distributed(_train_and_save, 1, dict(sharding="stage3", gradient_accumulation_steps=2), 4, full, str(tmp_path / "run1"), True)[0]
    for got in (got2, got1):
        assert len(got) >= 2
        for x, y in zip(ref[2:], got[-2:]):
            assert abs(x - y) < 3e-4 * max(1.0, abs(x)), (ref, got)


def test_offline_resharding_tool_prepares_a_checkpoint_for_more_ranks(tmp_path):
    """A checkpoint written by one process is re-cut offline for 2 sharding ranks; they find their own shard files and continue
    like the uninterrupted run."""
    from paddleformers_b200.trainer import ckpt_converter as cc

    full = _reference(False, 4, 2)
    ref = run_distributed(_train_and_save, 1, dict(gradient_accumulation_steps=2), 4, full, str(tmp_path / "ref"), False)[0]
    run_distributed(_train_and_save, 1, dict(gradient_accumulation_steps=2), 2, full, str(tmp_path / "one"), False)
    src = str(tmp_path / "one" / "checkpoint-2")
    info = cc.inspect(src)
    assert info["complete"] and info["global_step"] == 2 and all(d["shard_size"] == 1 for d in info["optimizer_domains"].values())
    dst = tmp_path / "two" / "checkpoint-2"
    files = cc.reshard(src, str(dst), 2)
    assert len(files) == 2 * len(info["optimizer_domains"]) and all("of002" in f for f in files)
    after = cc.inspect(str(dst))
    assert after["complete"] and all(d["shard_size"] == 2 and d["files"] == 2 for d in after["optimizer_domains"].values())
    assert cc.main(["inspect", str(dst)]) == 0
    got = run_distributed(_train_and_save, 2, dict(sharding="stage1", gradient_accumulation_steps=1), 4, full, str(tmp_path / "two"), True)[0]
    for a, b in zip(ref[2:], got[-2:]):
        assert abs(a - b) < 3e-4 * max(1.0, abs(a)), (ref, got)


@pytest.mark.parametrize("extra", [dict(), dict(enable_zero_cost_checkpoint=True)], ids=["sharded", "zcc"])
def test_sharded_checkpoint_resumes_under_tensor_parallelism(tmp_path, extra):
    """Two tensor-parallel ranks share the sharding coordinate 0: each must get back its OWN master weights and
    moments (the shard files carry the tensor / pipeline / expert coordinate), so the resumed run continues like the
    uninterrupted one."""
    full = _reference(False, 4, 2)
    tp2 = dict(tensor_model_parallel_size=2, sequence_parallel=True, gradient_accumulation_steps=2, **extra)
    ref = run_distributed(_train_and_save, 2, dict(tp2), 4, full, str(tmp_path / "ref"), False)
    run_distributed(_train_and_save, 2, dict(tp2), 2, full, str(tmp_path / "run"), False)
    files = os.listdir(str(tmp_path / "run" / "checkpoint-2" / "optimizer"))
    assert any("_m00p00e00_" in f for f in files) and any("_m01p00e00_" in f for f in files), files
    got = run_distributed(_train_and_save, 2, dict(tp2), 4, full, str(tmp_path / "run"), True)
    for r in range(2):
        assert len(got[r]) >= 2
        for a, b in zip(ref[r][2:], got[r][-2:]):
            assert abs(a - b) < 3e-4 * max(1.0, abs(a)), (ref[r], got[r])


def test_tensor_parallel_checkpoint_loads_in_one_process(tmp_path):
    """Weights saved by 2 tensor-parallel ranks form one Hugging Face checkpoint that a single process loads."""
    from paddleformers_b200.transformers.auto import AutoModelForCausalLM

    full = _reference(False, 2, 2)
    run_distributed(_train_and_save, 2, dict(tensor_model_parallel_size=2, sequence_parallel=True, gradient_accumulation_steps=2),
                    2, full, str(tmp_path / "tp"), False)
    ref_losses = run_distributed(_train_and_save, 1, dict(gradient_accumulation_steps=2), 2, full, str(tmp_path / "one"), False)[0]
    a = AutoModelForCausalLM.from_pretrained(str(tmp_path / "tp" / "checkpoint-2"), dtype=torch.float32)
    b = AutoModelForCausalLM.from_pretrained(str(tmp_path / "one" / "checkpoint-2"), dtype=torch.float32)
    assert len(ref_losses) == 2
    for (n1, p1), (n2, p2) in zip(a.state_dict().items(), b.state_dict().items()):
        assert n1 == n2
        torch.testing.assert_close(p1, p2, rtol=2e-3, atol=2e-4)


def test_unified_checkpoint_resumes_under_a_different_tensor_parallel_degree(tmp_path):
    """Optimizer state written under parameter names by 2 tensor-parallel ranks restores a 1-rank run that continues
    like an uninterrupted one (and the other way round: 1 rank -> 2 tensor-parallel ranks)."""
    full = _reference(False, 4, 2)
    single = dict(gradient_accumulation_steps=2, save_checkpoint_format="unified")
    tp2 = dict(tensor_model_parallel_size=2, sequence_parallel=True, gradient_accumulation_steps=2, save_checkpoint_format="unified")
    ref = run_distributed(_train_and_save, 1, dict(gradient_accumulation_steps=2), 4, full, str(tmp_path / "ref"), False)[0]
    run_distributed(_train_and_save, 2, tp2, 2, full, str(tmp_path / "a"), False)
    got = run_distributed(_train_and_save, 1, single, 4, full, str(tmp_path / "a"), True)[0]
    for a, b in zip(ref[2:], got[-2:]):
        assert abs(a - b) < 3e-4 * max(1.0, abs(a)), (ref, got)
    run_distributed(_train_and_save, 1, single, 2, full, str(tmp_path / "b"), False)
    got2 = run_distributed(_train_and_save, 2, tp2, 4, full, str(tmp_path / "b"), True)
    for r in range(2):
        for a, b in zip(ref[2:], got2[r][-2:]):
            assert abs(a - b) < 3e-4 * max(1.0, abs(a)), (ref, got2[r])


def _global_aux_worker(rank, world):
    """Balance loss from the expert loads and mean probabilities of all data ranks (``global_aux_loss``)."""
    from paddleformers_b200.models.configuration import Qwen3MoeConfig
    from paddleformers_b200.nn.moe import TopkRouter
    from paddleformers_b200.parallel.topology import ParallelDegrees, initialize_parallel

    initialize_parallel(ParallelDegrees(sharding=world), backend="gloo")
    cfg = Qwen3MoeConfig(hidden_size=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=16, intermediate_size=16,
                         num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2, vocab_size=64, router_aux_loss_coef=0.01)
    cfg.global_aux_loss = True
    torch.manual_seed(3)
    gate = TopkRouter(cfg)
    torch.nn.init.normal_(gate.weight, std=0.5)
    gate.train()
    x_all = torch.randn(world * 24, 32, generator=torch.Generator().manual_seed(9))
    _, _, aux = gate(x_all[rank * 24:(rank + 1) * 24])
    aux.backward()
    return float(aux), gate.weight.grad.clone()


def test_global_aux_loss_uses_the_statistics_of_all_data_ranks():
    from paddleformers_b200.models.configuration import Qwen3MoeConfig
    from paddleformers_b200.nn.moe import TopkRouter

    res = run_distributed(_global_aux_worker, 2)
    cfg = Qwen3MoeConfig(hidden_size=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=16, intermediate_size=16,
                         num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2, vocab_size=64, router_aux_loss_coef=0.01)
    torch.manual_seed(3)
    gate = TopkRouter(cfg)
    torch.nn.init.normal_(gate.weight, std=0.5)
    gate.train()
    x_all = torch.randn(48, 32, generator=torch.Generator().manual_seed(9))
    _, _, aux = gate(x_all)
    aux.backward()
    for a, _ in res:
        assert abs(a - float(aux)) < 1e-6                              # every rank reports the loss of the whole batch
    # each rank differentiates through its own probabilities only: the ranks' gradients add up to the whole-batch gradient
    torch.testing.assert_close(res[0][1] + res[1][1], gate.weight.grad, rtol=1e-4, atol=1e-7)


@pytest.mark.parametrize("name,P,M,V", [("1F1B", 4, 8, 1), ("interleaved", 2, 8, 2), ("zero_bubble", 4, 8, 1), ("FThenB", 2, 6, 1),
                                        ("zbv", 2, 8, 2)])
def test_expert_exchange_buffer_slots_follow_the_pipeline_schedule(name, P, M, V):
    """Every micro-batch holds one buffer slot from its first forward to its last backward chunk on a stage; slots are
    reused, so their number is the schedule's maximum of micro-batches in flight (P - stage for 1F1B, all of them for FThenB)."""
    from paddleformers_b200.parallel.fused_ep import SlotAllocator
    from paddleformers_b200.parallel.pipeline import make_schedule

    for stage in range(P):
        alloc = SlotAllocator(V)
        live, peak = set(), 0
        for a in make_schedule(name, stage, P, M, V):
            if a.kind == "W":
                continue
            slot = alloc.acquire(a.mb)
            # no two micro-batches in flight share a slot
            assert all(alloc.slot_of[m] != slot for m in live if m != a.mb)
            live.add(a.mb)
            peak = max(peak, len(live))
            if a.kind == "B":
                alloc.backward_done(a.mb)
                if a.mb not in alloc.slot_of:
                    live.discard(a.mb)
        assert not alloc.slot_of and alloc.high_water == peak
        if name == "1F1B":
            assert alloc.high_water == P - stage
        if name == "FThenB":
            assert alloc.high_water == M


def _modality_moe_worker(rank, world, full):
    """Text / vision expert groups under expert parallelism: both groups' exchanges run on every rank, also on a rank
    whose batch has no vision rows."""
    from paddleformers_b200.models.ernie4_5_vl import Ernie4_5VLTextConfig
    from paddleformers_b200.nn.moe import ModalityMoELayer
    from paddleformers_b200.parallel.topology import ParallelDegrees, initialize_parallel
    from paddleformers_b200.transformers.model_utils import param_shard_spec

    ps = initialize_parallel(ParallelDegrees(sharding=world, ep=world), backend="gloo") if world > 1 else \
        initialize_parallel(ParallelDegrees(), backend="gloo")
    cfg = Ernie4_5VLTextConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=2,
                               moe_intermediate_size=[16, 8], moe_k=2, moe_num_experts=4, moe_num_shared_experts=1,
                               router_aux_loss_coef=0.0, mlp_layer_types=["sparse"])
    cfg.moe_token_dispatcher_type = "alltoall"
    layer = ModalityMoELayer(cfg, dtype=torch.float32)
    with torch.no_grad():
        for name, p in layer.named_parameters():
            p.copy_(param_shard_spec(p).shard(full[name], 0, 1, ps.rank_in("ep"), ps.degrees.ep))
        for name, b in layer.named_buffers():
            if name in full:
                b.copy_(full[name])
    outs = []
    for r in (range(2) if world == 1 else [rank]):        # the single process plays both ranks' batches
        g = torch.Generator().manual_seed(100 + r)
        x = torch.randn(12, 32, generator=g, requires_grad=True)
        vis = torch.zeros(12, dtype=torch.bool)
        if r == 0:
            vis[3:9] = True                                # rank 1 holds text only
        layer.vision_rows = vis
        y = layer(x)
        y.square().sum().backward()
        outs.append((y.detach(), x.grad.clone()))
    return outs


def test_modality_isolated_experts_under_expert_parallelism():
    from paddleformers_b200.models.ernie4_5_vl import Ernie4_5VLTextConfig
    from paddleformers_b200.nn.moe import ModalityMoELayer

    torch.manual_seed(2)
    cfg = Ernie4_5VLTextConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=2,
                               moe_intermediate_size=[16, 8], moe_k=2, moe_num_experts=4, moe_num_shared_experts=1,
                               router_aux_loss_coef=0.0, mlp_layer_types=["sparse"])
    layer = ModalityMoELayer(cfg, dtype=torch.float32)
    full = {}
    for name, p in layer.named_parameters():
        full[name] = torch.randn_like(p) * 0.2
    full["text_moe.gate.e_score_correction_bias"] = torch.randn(4) * 0.1
    full["vision_moe.gate.e_score_correction_bias"] = torch.randn(4) * 0.1
    ref = run_distributed(_modality_moe_worker, 1, full)[0]
    got = run_distributed(_modality_moe_worker, 2, full)
    for r in range(2):
        y, gx = got[r][0]
        assert (y - ref[r][0]).abs().max() < 1e-5 and (gx - ref[r][1]).abs().max() < 1e-5


def _qk_norm_weights_worker(rank, world, full):
    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.models.configuration import named_config
    from paddleformers_b200.models.modeling import MODEL_MAPPING
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig
    from paddleformers_b200.transformers.model_utils import param_shard_spec

    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=2, max_steps=2, learning_rate=5e-2,
                             lr_scheduler_type="constant", logging_steps=1, save_strategy="no", max_seq_len=32, seed=3, device="cpu",
                             tensor_model_parallel_size=world, max_grad_norm=0.0)
    ps = args.setup_parallel()
    cfg = named_config("qwen3-30b-a3b", num_hidden_layers=1, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                       num_experts=0, intermediate_size=96, vocab_size=128)
    LlmMetaConfig.set_llm_config(cfg, args)
    model = MODEL_MAPPING[cfg.model_type](cfg)
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.copy_(param_shard_spec(p).shard(full[n], ps.coord["mp"], ps.degrees.mp, 0, 1))
    tr = Trainer(model=model, args=args, train_dataset=_DS(_data(8)))
    tr._sampler_shuffle = False
    tr.train()
    return {n: p.detach().clone() for n, p in model.named_parameters() if "q_norm" in n or "k_norm" in n}


def test_per_head_norm_weights_get_the_gradient_of_all_heads_under_tensor_parallelism():
    """One norm weight vector serves all heads, every tensor-parallel rank holds some of the heads: the partial gradients are
    summed over the group, so the replicas stay equal and follow the single-process trajectory."""
    from paddleformers_b200.models.configuration import named_config
    from paddleformers_b200.models.modeling import MODEL_MAPPING

    torch.manual_seed(0)
    cfg = named_config("qwen3-30b-a3b", num_hidden_layers=1, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                       num_experts=0, intermediate_size=96, vocab_size=128)
    full = {k: v.detach().clone() for k, v in MODEL_MAPPING[cfg.model_type](cfg).named_parameters()}
    ref = run_distributed(_qk_norm_weights_worker, 1, full)[0]
    got = run_distributed(_qk_norm_weights_worker, 2, full)
    for n in ref:
        assert (ref[n] - 1.0).abs().max() > 1e-3                                 # the weights moved
        assert torch.equal(got[0][n], got[1][n]), n
        assert (got[0][n] - ref[n]).abs().max() < 2e-3 * (ref[n] - 1.0).abs().max() + 1e-6, n


def _train_and_save_pp(rank, world, kind, targs, steps, full_state, out_dir, resume):
    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.parallel.pipeline import build_pipeline_model
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig
    from paddleformers_b200.transformers.model_utils import param_shard_spec

    args = TrainingArguments(output_dir=out_dir, per_device_train_batch_size=1, max_steps=steps, learning_rate=1e-2,
                             lr_scheduler_type="constant", logging_steps=1, save_steps=2, max_seq_len=32, max_grad_norm=1.0,
                             seed=3, device="cpu", **targs)
    ps = args.setup_parallel()
    cfg = _tiny_cfg(kind, num_hidden_layers=4)
    LlmMetaConfig.set_llm_config(cfg, args)
    model = build_pipeline_model(cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            g = model.global_param_name(name)
            p.copy_(param_shard_spec(p).shard(full_state[g], ps.coord["mp"], ps.degrees.mp, ps.rank_in("ep"), ps.degrees.ep))
    tr = Trainer(model=model, args=args, train_dataset=_DS(_data(8 * 4)))
    tr._sampler_shuffle = False
    tr.train(resume_from_checkpoint="auto" if resume else None)
    return [h["loss"] for h in tr.state.log_history if "loss" in h]


@pytest.mark.parametrize("name,world,kind,targs", [
    ("pp2_tied", 2, "tied", dict(pipeline_model_parallel_size=2, gradient_accumulation_steps=4)),
    ("pp2_ep2", 4, True, dict(pipeline_model_parallel_size=2, expert_model_parallel_size=2, sharding="stage1",
                              gradient_accumulation_steps=2, moe_token_dispatcher_type="alltoall")),
])
def test_checkpoint_resumes_under_pipeline_parallelism(tmp_path, name, world, kind, targs):
    """Stages save and reload their own layers, optimizer shards and (tied head) shared tensors: the resumed run continues like
    the uninterrupted one."""
    from paddleformers_b200.models.modeling import MODEL_MAPPING

    torch.manual_seed(5)
    cfg = _tiny_cfg(kind, num_hidden_layers=4)
    full = {k: v.detach().clone() for k, v in MODEL_MAPPING[cfg.model_type](cfg).named_parameters()}
    ref = run_distributed(_train_and_save_pp, world, kind, dict(targs), 4, full, str(tmp_path / "ref"), False)[0]
    run_distributed(_train_and_save_pp, world, kind, dict(targs), 2, full, str(tmp_path / "run"), False)
    got = run_distributed(_train_and_save_pp, world, kind, dict(targs), 4, full, str(tmp_path / "run"), True)[0]
    assert len(got) >= 2
    for a, b in zip(ref[2:], got[-2:]):
        assert abs(a - b) < 3e-4 * max(1.0, abs(a)), (name, ref, got)


def _lora_tp_worker(rank, world, full, sp):
    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.models.modeling import MODEL_MAPPING
    from paddleformers_b200.peft.lora import LoRAConfig, LoRAModel
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig
    from paddleformers_b200.transformers.model_utils import param_shard_spec

    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=2, max_steps=3, learning_rate=1e-2,
                             lr_scheduler_type="constant", logging_steps=1, save_strategy="no", max_seq_len=32, seed=3, device="cpu",
                             tensor_model_parallel_size=world, sequence_parallel=sp and world > 1, max_grad_norm=1.0)
    ps = args.setup_parallel()
    cfg = _tiny_cfg(False)
    LlmMetaConfig.set_llm_config(cfg, args)
    model = LoRAModel(MODEL_MAPPING[cfg.model_type](cfg), LoRAConfig(r=4, lora_alpha=8))
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.copy_(param_shard_spec(p).shard(full[n], ps.coord["mp"], ps.degrees.mp, 0, 1))
    tr = Trainer(model=model, args=args, train_dataset=_DS(_data(8)))
    tr._sampler_shuffle = False
    tr.train()
    return [h["loss"] for h in tr.state.log_history if "loss" in h] + [tr.state.log_history[0]["global_norm"]]


def test_lora_adapters_under_tensor_parallelism():
    """The adapter factor that is whole on every rank (A beside a column-parallel layer, B beside a row-parallel one) gets its
    gradient summed over the tensor-parallel group; losses and the gradient norm follow the single-process run."""
    from paddleformers_b200.models.modeling import MODEL_MAPPING
    from paddleformers_b200.peft.lora import LoRAConfig, LoRAModel

    torch.manual_seed(5)
    cfg = _tiny_cfg(False)
    m = LoRAModel(MODEL_MAPPING[cfg.model_type](cfg), LoRAConfig(r=4, lora_alpha=8))
    full = {k: (v.detach().clone() if "lora_B" not in k else torch.randn_like(v) * 0.05) for k, v in m.named_parameters()}
    ref = run_distributed(_lora_tp_worker, 1, full, False)[0]
    got = run_distributed(_lora_tp_worker, 2, full, True)
    for r in range(2):
        for a, b in zip(ref, got[r]):
            assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (ref, got[r])


def test_balance_loss_weighs_the_same_under_sequence_parallelism():
    """Every tensor-parallel rank adds the balance term of its own token slice and the router gradients are summed over the
    ranks: the terms count 1 / tp each. The statistics are per slice, so the run is close to the single-process one, not equal;
    without the factor the gradient norm of this model (large balance coefficient) doubles."""
    kind = "fam:gpt_oss"
    full = _reference(kind, 3, 2)
    single = dict(gradient_accumulation_steps=2, moe_token_dispatcher_type="alltoall")
    ref = _single_process_run(_train, kind, single, 3, full)
    got = run_distributed(_train, 2, kind, dict(tensor_model_parallel_size=2, sequence_parallel=True, gradient_accumulation_steps=2,
                                                moe_token_dispatcher_type="alltoall"), 3, full)[0]
    assert abs(got[-1] - ref[-1]) < 0.02 * ref[-1], (ref, got)          # first-step gradient norm
    assert abs(got[0] - ref[0]) < 1e-4 * ref[0]
    # and exactly equal without the balance term
    kind = "fam:mixtral+noaux"
    full = _reference(kind, 3, 2)
    ref = _single_process_run(_train, kind, single, 3, full)
    got = run_distributed(_train, 2, kind, dict(tensor_model_parallel_size=2, sequence_parallel=True, gradient_accumulation_steps=2,
                                                moe_token_dispatcher_type="alltoall"), 3, full)[0]
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (ref, got)


class _PreferencePairs(torch.utils.data.Dataset):
    def __len__(self):
        return 16

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(i)
        return {"prompt_ids": torch.randint(10, 60, (6,), generator=g).tolist(), "chosen_ids": [7, 7, 7, 1],
                "rejected_ids": [9, 9, 9, 1]}


def _dpo_tp_worker(rank, world, full, kind, targs):
    from paddleformers_b200 import TrainingArguments
    from paddleformers_b200.datasets.collate import dpo_collate_fn
    from paddleformers_b200.models.modeling import MODEL_MAPPING
    from paddleformers_b200.trainer.dpo_trainer import DPOTrainer
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig
    from paddleformers_b200.transformers.model_utils import param_shard_spec

    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=2, max_steps=3, learning_rate=5e-3,
                             lr_scheduler_type="constant", logging_steps=1, save_strategy="no", max_seq_len=32, seed=3,
                             device="cpu", **targs)
    ps = args.setup_parallel()
    cfg = _tiny_cfg(kind)
    LlmMetaConfig.set_llm_config(cfg, args)

    def build():
        m = MODEL_MAPPING[cfg.model_type](cfg)
        with torch.no_grad():
            for n, p in m.named_parameters():
                p.copy_(param_shard_spec(p).shard(full[n], ps.coord["mp"], ps.degrees.mp, 0, 1))
        return m

    tr = DPOTrainer(model=build(), ref_model=build(), args=args, train_dataset=_PreferencePairs(),
                    data_collator=lambda b: dpo_collate_fn(b, max_seq_len=32), dpo_beta=0.5)
    tr._sampler_shuffle = False
    tr.train()
    return [h["loss"] for h in tr.state.log_history if "loss" in h] + [tr.state.log_history[0]["global_norm"]]


@pytest.mark.parametrize("kind", [False, "tied"])
def test_preference_training_under_tensor_parallelism(kind):
    """(Also context and segment parallelism.) DPO reads the full logits: under tensor parallelism the vocabulary shards are concatenated by an operation whose
    backward pass keeps this rank's shard, and the hidden states' gradient is summed over the shards (reduce-scattered under
    sequence parallelism). Losses and the first gradient norm follow the single-process run, also with a tied
    vocabulary-parallel embedding as the head."""
    from paddleformers_b200.models.modeling import MODEL_MAPPING

    torch.manual_seed(5)
    cfg = _tiny_cfg(kind)
    full = {k: v.detach().clone() for k, v in MODEL_MAPPING[cfg.model_type](cfg).named_parameters()}
    ref = run_distributed(_dpo_tp_worker, 1, full, kind, {})[0]
    cases = [dict(tensor_model_parallel_size=2), dict(tensor_model_parallel_size=2, sequence_parallel=True)]
    if kind is False:
        # ranks that hold slices of one sequence add up their parts of every response's log-probability
        cases += [dict(context_parallel_size=2), dict(sep_parallel_size=2)]
    for targs in cases:
        got = run_distributed(_dpo_tp_worker, 2, full, kind, targs)
        for r in range(2):
            for a, b in zip(ref, got[r]):
                assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (targs, ref, got[r])


def _packed_data(n, S=32, vocab=128):
    """Two documents per row: positions restart, keys of the first document end at its last row."""
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, vocab, (n, S + 1), generator=g)
    out = []
    for i in range(n):
        cut = 9 + (i * 5) % 14
        lab = ids[i, 1:].clone()
        lab[:2], lab[cut - 1], lab[cut:cut + 2] = -100, -100, -100
        out.append({"input_ids": ids[i, :-1], "labels": lab, "position_ids": torch.cat([torch.arange(cut), torch.arange(S - cut)]),
                    "attn_mask_startend_row_indices": torch.cat([torch.full((cut,), cut), torch.full((S - cut,), S)]).to(torch.int32)})
    return out


def _train_packed(rank, world, kind, targs, steps, full, pipeline):
    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.models.modeling import MODEL_MAPPING
    from paddleformers_b200.parallel.pipeline import build_pipeline_model
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig
    from paddleformers_b200.transformers.model_utils import param_shard_spec

    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=1, max_steps=steps, learning_rate=1e-2,
                             lr_scheduler_type="constant", logging_steps=1, save_strategy="no", max_seq_len=32, max_grad_norm=1.0,
                             seed=3, device="cpu", **targs)
    ps = args.setup_parallel()
    cfg = _tiny_cfg(kind, num_hidden_layers=4)
    LlmMetaConfig.set_llm_config(cfg, args)
    model = build_pipeline_model(cfg) if pipeline else MODEL_MAPPING[cfg.model_type](cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            g = model.global_param_name(name) if pipeline else name
            p.copy_(param_shard_spec(p).shard(full[g], ps.coord["mp"], ps.degrees.mp, ps.rank_in("ep"), ps.degrees.ep))
    tr = Trainer(model=model, args=args, train_dataset=_DS(_packed_data(8 * steps)))
    tr._sampler_shuffle = False
    tr.train()
    return [h["loss"] for h in tr.state.log_history if "loss" in h] + [tr.state.log_history[0]["global_norm"]]


def test_packed_documents_under_pipeline_and_context_parallelism():
    """Rows that pack two documents (restarting positions, per-key visibility bounds) train the same on 2 stages x 2 sequence
    slices as in one process: the bounds of the whole row and the global positions reach every stage."""
    from paddleformers_b200.models.modeling import MODEL_MAPPING

    torch.manual_seed(5)
    cfg = _tiny_cfg(False, num_hidden_layers=4)
    full = {k: v.detach().clone() for k, v in MODEL_MAPPING[cfg.model_type](cfg).named_parameters()}
    ref = run_distributed(_train_packed, 1, False, dict(gradient_accumulation_steps=4), 2, full, False)[0]
    got = run_distributed(_train_packed, 4, False, dict(pipeline_model_parallel_size=2, context_parallel_size=2,
                                                        gradient_accumulation_steps=4), 2, full, True)
    for r in range(4):
        for a, b in zip(ref, got[r]):
            assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (ref, got[r])


def _classifier_worker(rank, world, targs, full, token_level):
    from paddleformers_b200 import TrainingArguments
    from paddleformers_b200.models.classification import DecoderForSequenceClassification, DecoderForTokenClassification
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig
    from paddleformers_b200.transformers.model_utils import param_shard_spec

    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=1, max_steps=1, save_strategy="no",
                             max_seq_len=32, seed=3, device="cpu", **targs)
    ps = args.setup_parallel()
    cfg = _tiny_cfg(False)
    cfg.num_labels = 3
    LlmMetaConfig.set_llm_config(cfg, args)
    model = (DecoderForTokenClassification if token_level else DecoderForSequenceClassification)(cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            p.copy_(param_shard_spec(p).shard(full[name], ps.coord["mp"], ps.degrees.mp, 0, 1))
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(1, 120, (2, 16), generator=g)
    labels = torch.randint(0, 3, (2, 16), generator=g) if token_level else torch.tensor([2, 0])
    out = model(ids, labels=labels)
    out.loss.backward()
    square = 0.0
    for name, p in model.named_parameters():
        grad = p.grad if p.grad is not None else getattr(p, "main_grad", None)
        if grad is None:
            continue
        grad = grad.double().clone()
        if getattr(p, "sequence_parallel", False) and world > 1:         # partial per rank: what the optimizer sums
            torch.distributed.all_reduce(grad)
        v = grad.pow(2).sum()
        if tuple(p.shape) != tuple(full[name].shape) and world > 1:      # a shard: the norm adds the ranks' parts
            torch.distributed.all_reduce(v)
        square += float(v)
    return [float(out.loss), square ** 0.5]


@pytest.mark.parametrize("token_level", [False, True])
def test_classification_heads_under_tensor_and_sequence_parallelism(token_level):
    """Sequence (last kept token) and token classification on a tensor-parallel decoder: under sequence parallelism the token
    slices are gathered before the head; loss and the norm of all gradients equal the single-process values."""
    from paddleformers_b200.models.classification import DecoderForSequenceClassification, DecoderForTokenClassification

    torch.manual_seed(5)
    cfg = _tiny_cfg(False)
    cfg.num_labels = 3
    cls = DecoderForTokenClassification if token_level else DecoderForSequenceClassification
    full = {k: v.detach().clone() for k, v in cls(cfg).named_parameters()}
    ref = run_distributed(_classifier_worker, 1, {}, full, token_level)[0]
    for targs in (dict(tensor_model_parallel_size=2), dict(tensor_model_parallel_size=2, sequence_parallel=True)):
        for got in run_distributed(_classifier_worker, 2, targs, full, token_level):
            assert abs(got[0] - ref[0]) < 1e-5 and abs(got[1] - ref[1]) < 1e-4 * ref[1], (targs, ref, got)


def _tiny_vl_cfg():
    from paddleformers_b200.models.vision_language import Qwen2VLConfig
    return Qwen2VLConfig(text_config=dict(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2,
                                         num_key_value_heads=2, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}),
                        vision_config=dict(depth=1, embed_dim=16, hidden_size=32, mlp_ratio=2, num_heads=2, patch_size=4), image_token_id=60)
def _vl_worker(rank, world, targs, full):
    import numpy as np

    from paddleformers_b200 import TrainingArguments
    from paddleformers_b200.models.vision_language import Qwen2VLForConditionalGeneration
    from paddleformers_b200.models.vision_language import mm_collate_fn
    from paddleformers_b200.transformers.image_processing import Qwen2VLImageProcessor
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig
    from paddleformers_b200.transformers.model_utils import param_shard_spec
    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=1, max_steps=1, save_strategy="no", max_seq_len=32, seed=3, device="cpu", **targs)
    ps = args.setup_parallel()
    cfg = _tiny_vl_cfg()
    LlmMetaConfig.set_llm_config(cfg.text_config, args)
    model = Qwen2VLForConditionalGeneration(cfg, dtype=torch.float32)
    with torch.no_grad():
        for name, p in model.named_parameters():
            p.copy_(param_shard_spec(p).shard(full[name], ps.coord["mp"], ps.degrees.mp, 0, 1))
    rng = np.random.default_rng(0)
    proc = Qwen2VLImageProcessor(patch_size=4, min_pixels=64, max_pixels=1024)
    out = proc([rng.integers(0, 255, (24, 32, 3), dtype=np.uint8)])
    n = proc.num_image_tokens(out["image_grid_thw"][0])
    ids = [1, 2] + [60] * n + [3, 4, 5, 6]
    ids = ids + [7] * (-len(ids) % 2)
    labels = [-100] * (2 + n) + [4, 5, 6, -100] + [-100] * (len(ids) - n - 6)
    batch = mm_collate_fn([{"input_ids": ids, "labels": labels, **out}])
    o = model(**batch)
    o.loss.backward()
    sq = 0.0
    for name, p in model.named_parameters():
        g = p.grad if p.grad is not None else getattr(p, "main_grad", None)
        if g is None: continue
        g = g.double().clone()
        if getattr(p, "sequence_parallel", False) and world > 1: torch.distributed.all_reduce(g)
        v = g.pow(2).sum()
        if tuple(p.shape) != tuple(full[name].shape) and world > 1: torch.distributed.all_reduce(v)
        sq += float(v)
    vis = model.visual.patch_embed.weight
    gv = vis.grad if vis.grad is not None else vis.main_grad
    return [float(o.loss), sq ** 0.5, float(gv.double().norm())]


def test_vision_language_model_under_tensor_and_sequence_parallelism():
    """Qwen2-VL on a tensor-parallel decoder: the image features are written over the placeholder rows of the whole-sequence
    embeddings, then every rank cuts its token slice; loss, the norm of all gradients and the vision tower's gradient equal the
    single-process values."""
    from paddleformers_b200.models.vision_language import Qwen2VLForConditionalGeneration

    torch.manual_seed(5)
    full = {k: v.detach().clone() for k, v in Qwen2VLForConditionalGeneration(_tiny_vl_cfg(), dtype=torch.float32).named_parameters()}
    ref = run_distributed(_vl_worker, 1, {}, full)[0]
    for targs in (dict(tensor_model_parallel_size=2), dict(tensor_model_parallel_size=2, sequence_parallel=True)):
        for got in run_distributed(_vl_worker, 2, targs, full):
            for a, b in zip(ref, got):
                assert abs(a - b) < 1e-4 * max(1.0, abs(a)), (targs, ref, got)
