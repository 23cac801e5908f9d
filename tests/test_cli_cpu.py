"""Command line: argument parsing, unknown-key errors, a full PT run from a YAML config, launch command."""
import json
import os

import numpy as np
import pytest
import torch


def test_parse_overrides_and_unknown_keys(tmp_path):
    from paddleformers_b200.cli.hparams import get_train_args

    cfg = tmp_path / "c.yaml"
    cfg.write_text("stage: SFT\nmodel_type: tiny-llama\nlearning_rate: 1.0e-3\nlora: true\ncompute_type: float32\n"
                   "tensor_model_parallel_size: 1\noutput_dir: %s\n" % tmp_path)
    m, d, g, e, t = get_train_args([str(cfg), "lora_rank=4", "max_steps=3", "packing=false"])
    assert m.lora and m.lora_rank == 4 and t.max_steps == 3 and t.learning_rate == 1e-3 and d.packing is False
    assert t.bf16 is False and t.data_parallel_size == 1
    with pytest.raises(ValueError, match="unknown configuration keys"):
        get_train_args([str(cfg), "not_a_flag=1"])


@pytest.mark.parametrize("stage", ["PT", "auto-parallel"])
def test_pretrain_stage_end_to_end_from_yaml(tmp_path, stage):
    from paddleformers_b200.cli.cli import main
    from paddleformers_b200.data.indexed_dataset import MMapIndexedDatasetBuilder

    prefix = str(tmp_path / "corpus")
    b = MMapIndexedDatasetBuilder(prefix, dtype=np.uint16)
    rng = np.random.RandomState(0)
    for _ in range(64):
        b.add_document(rng.randint(2, 120, size=rng.randint(20, 60)))
    b.finalize()
    out = tmp_path / "out"
    cfg = tmp_path / "pt.json"
    cfg.write_text(json.dumps({
        "stage": stage, "model_type": "tiny-llama", "from_scratch": True, "compute_type": "float32", "device": "cpu",
        "config_overrides": {"vocab_size": 128, "hidden_size": 32, "intermediate_size": 48, "num_attention_heads": 2,
                             "num_key_value_heads": 1, "head_dim": 16},
        "input_dir": prefix, "split": "9,1,0", "max_seq_len": 32, "max_steps": 4, "per_device_train_batch_size": 2,
        "learning_rate": 1e-3, "logging_steps": 1, "save_strategy": "no", "output_dir": str(out)}))
    env = os.environ.pop("CUDA_VISIBLE_DEVICES", None)
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    try:
        assert main(["train", str(cfg)]) == 0
    finally:
        if env is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = env
    assert os.path.exists(out / "model.safetensors") and os.path.exists(out / "config.json")


def test_launch_command_uses_loopback_rendezvous(monkeypatch):
    from paddleformers_b200.cli.cli import build_launch_command

    monkeypatch.delenv("MASTER_ADDR", raising=False)
    cmd = build_launch_command(["cfg.yaml", "a=1"], 8)
    assert "--nproc-per-node=8" in cmd and "--master-addr=127.0.0.1" in cmd and cmd[-2:] == ["cfg.yaml", "a=1"]


def _tiny_tokenizer_dir(tmp_path):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    words = ["<pad>", "<s>", "</s>", "<unk>", "Human:", "Assistant:", "System:"] + [f"w{i}" for i in range(60)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", bos_token="<s>", eos_token="</s>", unk_token="<unk>")
    d = tmp_path / "tok"
    fast.save_pretrained(str(d))
    return str(d), len(words)


def test_sft_lora_stage_then_export_merges_adapters(tmp_path):
    """SFT stage with LoRA from a jsonl of conversations, then the export command merges the adapters into a
    Hugging Face directory that loads as a plain model."""
    from paddleformers_b200.cli.cli import main
    from paddleformers_b200.transformers.auto import AutoModelForCausalLM

    tok_dir, vocab = _tiny_tokenizer_dir(tmp_path)
    data = tmp_path / "sft.jsonl"
    rng = np.random.RandomState(0)
    with open(data, "w") as f:
        for _ in range(32):
            q = " ".join(f"w{i}" for i in rng.randint(0, 60, size=5))
            a = " ".join(f"w{i}" for i in rng.randint(0, 60, size=4))
            f.write(json.dumps({"messages": [{"role": "user", "content": q}, {"role": "assistant", "content": a}]}) + "\n")
    # a base model directory that also holds the tokenizer
    base_dir = tmp_path / "base"
    from paddleformers_b200.models.configuration import named_config

    cfg = named_config("tiny-llama", vocab_size=vocab, hidden_size=32, intermediate_size=48, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=16)
    AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).save_pretrained(str(base_dir))
    for fn in os.listdir(tok_dir):
        with open(os.path.join(tok_dir, fn), "rb") as src, open(base_dir / fn, "wb") as dst:
            dst.write(src.read())
    out = tmp_path / "lora_out"
    cfg_file = tmp_path / "sft.json"
    cfg_file.write_text(json.dumps({
        "stage": "SFT", "model_name_or_path": str(base_dir), "compute_type": "float32", "device": "cpu", "lora": True,
        "lora_rank": 4, "loraga": True, "loraga_init_iters": 2, "train_dataset_path": str(data), "template": "default", "max_seq_len": 32, "max_steps": 3,
        "per_device_train_batch_size": 2, "learning_rate": 1e-3, "logging_steps": 1, "save_strategy": "no", "output_dir": str(out)}))
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    try:
        assert main(["train", str(cfg_file)]) == 0
        merged = tmp_path / "merged"
        exp_file = tmp_path / "export.json"
        exp_file.write_text(json.dumps({"model_name_or_path": str(base_dir), "lora_path": str(out), "output_dir": str(merged),
                                        "compute_type": "float32", "device": "cpu"}))
        assert main(["export", str(exp_file)]) == 0
    finally:
        if env is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = env
    final = merged / "export"                  # the export command writes into <output_dir>/export, like the reference's
    model = AutoModelForCausalLM.from_pretrained(str(final), dtype=torch.float32)
    assert not any("lora_" in n for n, _ in model.named_parameters())
    assert os.path.exists(final / "tokenizer.json")


def test_vl_sft_stage_trains_on_images(tmp_path):
    """VL-SFT stage: conversations with <image> markers and image files, a Qwen2-VL directory with tokenizer files."""
    from PIL import Image
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from paddleformers_b200.cli.cli import main
    from paddleformers_b200.models.vision_language import Qwen2VLConfig, Qwen2VLForConditionalGeneration
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    words = ["<pad>", "<s>", "</s>", "<unk>", "Human:", "Assistant:", "System:", "<image>", "<|image_pad|>", "<|vision_start|>",
             "<|vision_end|>"] + [f"w{i}" for i in range(40)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", bos_token="<s>", eos_token="</s>", unk_token="<unk>")
    base = tmp_path / "base"
    cfg = Qwen2VLConfig(text_config=dict(vocab_size=len(words), hidden_size=32, intermediate_size=48, num_hidden_layers=1,
                                         num_attention_heads=2, num_key_value_heads=1, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}),
                        vision_config=dict(depth=1, embed_dim=16, hidden_size=32, mlp_ratio=2, num_heads=2, patch_size=4),
                        image_token_id=words.index("<|image_pad|>"), vision_start_token_id=words.index("<|vision_start|>"),
                        vision_end_token_id=words.index("<|vision_end|>"))
    torch.manual_seed(0)
    Qwen2VLForConditionalGeneration(cfg, dtype=torch.float32).save_pretrained(str(base))
    fast.save_pretrained(str(base))
    rng = np.random.RandomState(0)
    data = tmp_path / "vl.jsonl"
    with open(data, "w") as f:
        for i in range(8):
            img = tmp_path / f"img{i}.png"
            Image.fromarray((rng.rand(20 + 4 * (i % 3), 24, 3) * 255).astype("uint8")).save(img)
            f.write(json.dumps({"images": [str(img)], "messages": [{"role": "user", "content": "<image> w1 w2"},
                                                                     {"role": "assistant", "content": f"w{3 + i % 5} w9"}]}) + "\n")
    out = tmp_path / "out"
    cfg_file = tmp_path / "vl.json"
    cfg_file.write_text(json.dumps({
        "stage": "VL-SFT", "model_name_or_path": str(base), "compute_type": "float32", "device": "cpu", "train_dataset_path": str(data),
        "template": "default", "max_seq_len": 64, "max_steps": 4, "per_device_train_batch_size": 1, "learning_rate": 5e-3,
        "logging_steps": 1, "save_strategy": "no", "output_dir": str(out), "min_pixels": 256, "max_pixels": 4096}))
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    try:
        assert main(["train", str(cfg_file)]) == 0
    finally:
        if env is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = env
    model = AutoModelForConditionalGeneration.from_pretrained(str(out), dtype=torch.float32)
    assert model.visual.patch_embed.weight.shape == (16, 3 * 2 * 4 * 4) and os.path.exists(out / "tokenizer.json")


def test_vl_pt_and_vl_dpo_stages(tmp_path):
    """VL-PT: image-text records where every text token is a target. VL-DPO: preference pairs that share a prompt with an image;
    the policy moves away from the frozen reference and the logged reward margin becomes positive."""
    from PIL import Image
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from paddleformers_b200.cli.cli import main
    from paddleformers_b200.datasets.mm_dataset import MMDPODataset, MMSFTDataset, mm_dpo_collate_fn
    from paddleformers_b200.models.vision_language import Qwen2VLConfig, Qwen2VLForConditionalGeneration
    from paddleformers_b200.transformers.image_processing import Qwen2VLImageProcessor

    words = ["<pad>", "<s>", "</s>", "<unk>", "Human:", "Assistant:", "System:", "<image>", "<|image_pad|>", "<|vision_start|>",
             "<|vision_end|>"] + [f"w{i}" for i in range(40)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", bos_token="<s>", eos_token="</s>", unk_token="<unk>")
    base = tmp_path / "base"
    cfg = Qwen2VLConfig(text_config=dict(vocab_size=len(words), hidden_size=32, intermediate_size=48, num_hidden_layers=1,
                                         num_attention_heads=2, num_key_value_heads=1, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}),
                        vision_config=dict(depth=1, embed_dim=16, hidden_size=32, mlp_ratio=2, num_heads=2, patch_size=4),
                        image_token_id=words.index("<|image_pad|>"), vision_start_token_id=words.index("<|vision_start|>"),
                        vision_end_token_id=words.index("<|vision_end|>"))
    torch.manual_seed(0)
    Qwen2VLForConditionalGeneration(cfg, dtype=torch.float32).save_pretrained(str(base))
    fast.save_pretrained(str(base))
    rng = np.random.RandomState(0)
    pt, dpo = tmp_path / "pt.jsonl", tmp_path / "dpo.jsonl"
    with open(pt, "w") as f, open(dpo, "w") as g:
        for i in range(8):
            img = tmp_path / f"img{i}.png"
            Image.fromarray((rng.rand(16 + 8 * (i % 2), 24, 3) * 255).astype("uint8")).save(img)
            f.write(json.dumps({"images": [str(img)], "text": f"w1 <image> w{2 + i % 5} w7 w8"}) + "\n")
            g.write(json.dumps({"images": [str(img)], "messages": [{"role": "user", "content": "<image> w1 w2"}],
                                "chosen": "w5 w6 w7", "rejected": "w30 w31"}) + "\n")
    proc = Qwen2VLImageProcessor(patch_size=4, merge_size=2, temporal_patch_size=2, min_pixels=256, max_pixels=4096)
    names = dict(image_token="<|image_pad|>", vision_start_token="<|vision_start|>", vision_end_token="<|vision_end|>")
    item = MMSFTDataset(str(pt), fast, proc, "default", 64, pretrain=True, **names)[0]
    n_img = int((item["input_ids"] == words.index("<|image_pad|>")).sum())
    assert n_img == proc.num_image_tokens(item["image_grid_thw"][0].tolist())
    assert int((item["labels"] != -100).sum()) == 4            # w2 w7 w8 </s> after the image run; never an image token
    pair = MMDPODataset(str(dpo), fast, proc, "default", 64, **names)[1]
    assert len(pair["input_ids"]) == 2 and [int((x != -100).sum()) for x in pair["labels"]] == [4, 3]     # response + end token
    batch = mm_dpo_collate_fn([pair, pair])
    assert batch["input_ids"].shape[0] == 4 and batch["image_grid_thw"].shape[0] == 4 and int(batch["preference_pairs"]) == 2
    common = {"model_name_or_path": str(base), "compute_type": "float32", "device": "cpu", "template": "default", "max_seq_len": 64,
              "per_device_train_batch_size": 2, "logging_steps": 1, "save_strategy": "no", "min_pixels": 256, "max_pixels": 4096}
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    try:
        f1 = tmp_path / "pt.json"
        f1.write_text(json.dumps(dict(common, stage="VL-PT", train_dataset_path=str(pt), max_steps=3, learning_rate=5e-3,
                                      output_dir=str(tmp_path / "out_pt"))))
        assert main(["train", str(f1)]) == 0
        f2 = tmp_path / "dpo.json"
        f2.write_text(json.dumps(dict(common, stage="VL-DPO", train_dataset_path=str(dpo), max_steps=6, learning_rate=2e-2,
                                      output_dir=str(tmp_path / "out_dpo"), dpo_beta=0.5, logging_dir=str(tmp_path / "logs"))))
        from paddleformers_b200.cli.train import run_tuner

        trainer, _ = run_tuner([str(f2)])
    finally:
        if env is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = env
    assert os.path.exists(tmp_path / "out_pt" / "model.safetensors") and os.path.exists(tmp_path / "out_dpo" / "model.safetensors")
    assert trainer.ref_model is not None and trainer.last_metrics["rewards/margins"] > 0 and trainer.last_metrics["rewards/accuracies"] == 1.0


def test_example_configs_parse(monkeypatch):
    """Every file under examples/config is accepted by the argument parser (no unknown keys, right types, parallel
    degrees that divide a 64-GPU job)."""
    import glob

    monkeypatch.setenv("WORLD_SIZE", "64")
    monkeypatch.setenv("RANK", "0")

    from paddleformers_b200.cli.hparams import read_args

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "config")
    files = sorted(glob.glob(os.path.join(root, "*.yaml")))
    assert len(files) >= 8
    for f in files:
        flat = read_args([f])
        if os.path.basename(f).startswith("merge"):
            from paddleformers_b200.mergekit.merge import MergeConfig

            assert set(flat) <= {x.name for x in __import__("dataclasses").fields(MergeConfig)}, f
            continue
        if "export" in os.path.basename(f):
            from paddleformers_b200.cli.hparams import ExportArguments

            known = {x.name for x in __import__("dataclasses").fields(ExportArguments)} | {"model_name_or_path", "compute_type", "device"}
            assert set(flat) <= known | {"lora_path", "output_dir"}, (f, set(flat) - known)
            continue
        from paddleformers_b200.cli.hparams import parse_dict

        model_args, data_args, gen_args, export_args, train_args = parse_dict(dict(flat, device="cpu"))
        assert model_args.stage and train_args.output_dir, f


def test_preprocess_tool_writes_a_corpus_that_gpt_dataset_reads(tmp_path):
    from paddleformers_b200.data.indexed_dataset import GPTDataset, MMapIndexedDataset
    from paddleformers_b200.data.preprocess import main as preprocess_main

    tok_dir, vocab = _tiny_tokenizer_dir(tmp_path)
    src = tmp_path / "corpus.jsonl"
    rng = np.random.RandomState(0)
    docs = [" ".join(f"w{i}" for i in rng.randint(0, 60, size=rng.randint(5, 30))) for _ in range(40)]
    with open(src, "w") as f:
        for d in docs:
            f.write(json.dumps({"text": d}) + "\n")
    prefix = str(tmp_path / "out" / "corpus")
    assert preprocess_main(["--input", str(src), "--tokenizer", tok_dir, "--output-prefix", prefix, "--append-eos"]) == 0
    ds = MMapIndexedDataset(prefix)
    assert len(ds) == 40 and ds.dtype == np.uint16
    first = ds[0]
    assert first[-1] == 2 and len(first) == len(docs[0].split()) + 1             # eos appended
    g = GPTDataset(ds, None, num_samples=10, seq_length=16, seed=1)
    item = g[0]
    assert item["input_ids"].shape == (16,) and torch.equal(item["input_ids"][1:], item["labels"][:-1])


def test_fp8_flag_converts_dense_linears_in_the_workflow(tmp_path):
    from paddleformers_b200.cli.hparams import parse_dict
    from paddleformers_b200.cli.train import _build_model
    from paddleformers_b200.quantization.fp8 import FP8Linear

    flat = {"stage": "PT", "model_type": "tiny-llama", "from_scratch": True, "compute_type": "float32", "device": "cpu", "fp8": "e4m3",
            "config_overrides": {"vocab_size": 128, "hidden_size": 128, "intermediate_size": 256, "num_attention_heads": 2,
                                 "num_key_value_heads": 1, "head_dim": 64}, "output_dir": str(tmp_path)}
    model_args, _, _, _, train_args = parse_dict(flat)
    train_args.setup_parallel()
    model, cfg = _build_model(model_args, train_args, torch.float32)
    layer = model.model.layers["0"]
    assert isinstance(layer.self_attn.qkv_proj, FP8Linear) and isinstance(layer.mlp.down_proj, FP8Linear)
    assert not isinstance(model.lm_head, FP8Linear)
    ids = torch.randint(0, 128, (2, 16))
    out = model(ids, labels=torch.roll(ids, -1, 1))
    out.loss.backward()
    assert torch.isfinite(out.loss) and layer.self_attn.qkv_proj.weight.grad is not None


def test_recipe_stages_turn_on_their_switches_and_train(tmp_path):
    from paddleformers_b200.cli.cli import main
    from paddleformers_b200.cli.hparams import parse_dict
    from paddleformers_b200.cli.train import apply_recipe
    from paddleformers_b200.data.indexed_dataset import MMapIndexedDatasetBuilder

    base = {"model_type": "deepseek_v3", "from_scratch": True, "compute_type": "float32", "device": "cpu", "output_dir": str(tmp_path)}
    margs, _, _, _, targs = parse_dict(dict(base, stage="dsv3_pretrain"))
    changed = apply_recipe("dsv3_pretrain", margs, targs)
    assert targs.fp8 == "e4m3" and targs.moe_token_dispatcher_type == "fused" and targs.moe_aux_free_bias_update_rate == 0.001
    assert targs.recompute_granularity == "selective" and "pipeline_schedule" not in changed      # one pipeline stage
    # what the user set explicitly stays
    margs, _, _, _, targs = parse_dict(dict(base, stage="ernie_pretrain", moe_token_dispatcher_type="alltoall"))
    apply_recipe("ernie_pretrain", margs, targs)
    assert targs.moe_token_dispatcher_type == "alltoall" and targs.fp8 == "e4m3"

    prefix = str(tmp_path / "corpus")
    b = MMapIndexedDatasetBuilder(prefix, dtype=np.uint16)
    rng = np.random.RandomState(0)
    for _ in range(64):
        b.add_document(rng.randint(2, 120, size=rng.randint(20, 60)))
    b.finalize()
    out = tmp_path / "out"
    cfg = tmp_path / "dsv3.json"
    cfg.write_text(json.dumps(dict(base, stage="dsv3_pretrain", output_dir=str(out), input_dir=prefix, split="9,1,0", max_seq_len=32,
                                   max_steps=3, per_device_train_batch_size=2, learning_rate=1e-3, logging_steps=1, save_strategy="no",
                                   config_overrides={"vocab_size": 128, "hidden_size": 128, "intermediate_size": 256,
                                                     "moe_intermediate_size": 128, "num_hidden_layers": 2, "first_k_dense_replace": 1,
                                                     "num_attention_heads": 2, "n_routed_experts": 4, "num_experts_per_tok": 2,
                                                     "n_group": 1, "topk_group": 1, "q_lora_rank": 32, "kv_lora_rank": 32,
                                                     "qk_nope_head_dim": 16, "qk_rope_head_dim": 16, "v_head_dim": 16,
                                                     "num_nextn_predict_layers": 1})))
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    try:
        assert main(["train", str(cfg)]) == 0
    finally:
        if env is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = env
    assert os.path.exists(out / "model.safetensors")
    saved = json.loads((out / "config.json").read_text())
    assert saved["model_type"] == "deepseek_v3"


@pytest.mark.parametrize("family", ["gemma3", "paligemma"])
def test_vl_sft_stage_trains_the_siglip_families(tmp_path, family):
    """VL-SFT on fixed-size-image families: Gemma 3 (begin / end-of-image tokens around a fixed run of placeholders, two-way attention
    inside each image) and PaliGemma (placeholders only, token types mark the two-way prompt)."""
    from PIL import Image
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from paddleformers_b200.cli.cli import main
    from paddleformers_b200.datasets.mm_dataset import MMSFTDataset
    from paddleformers_b200.models.paligemma import Gemma3Config, PaliGemmaConfig
    from paddleformers_b200.models.vision_language import mm_collate_fn
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration
    from paddleformers_b200.transformers.image_processing import SiglipImageProcessor

    words = ["<pad>", "<s>", "</s>", "<unk>", "Human:", "Assistant:", "System:", "<image>", "<image_soft_token>", "<start_of_image>",
             "<end_of_image>"] + [f"w{i}" for i in range(40)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", bos_token="<s>", eos_token="</s>", unk_token="<unk>")
    vision = dict(hidden_size=16, intermediate_size=32, num_hidden_layers=1, num_attention_heads=2, image_size=16, patch_size=4)
    text = dict(vocab_size=len(words), hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                head_dim=16)
    if family == "gemma3":
        cfg = Gemma3Config(text_config=dict(text, sliding_window=8, query_pre_attn_scalar=16), vision_config=vision, mm_tokens_per_image=4,
                           image_token_index=words.index("<image_soft_token>"), boi_token_index=words.index("<start_of_image>"),
                           eoi_token_index=words.index("<end_of_image>"))
    else:
        cfg = PaliGemmaConfig(text_config=dict(text, model_type="gemma"), vision_config=vision, image_token_index=words.index("<image>"),
                              projection_dim=32)
    base = tmp_path / "base"
    torch.manual_seed(0)
    AutoModelForConditionalGeneration.from_config(cfg, dtype=torch.float32).save_pretrained(str(base))
    fast.save_pretrained(str(base))
    rng = np.random.RandomState(0)
    data = tmp_path / "vl.jsonl"
    with open(data, "w") as f:
        for i in range(8):
            img = tmp_path / f"img{i}.png"
            Image.fromarray((rng.rand(20 + 4 * (i % 3), 24, 3) * 255).astype("uint8")).save(img)
            f.write(json.dumps({"images": [str(img)], "messages": [{"role": "user", "content": "<image> w1 w2"},
                                                                     {"role": "assistant", "content": f"w{3 + i % 5} w9"}]}) + "\n")
    proc = SiglipImageProcessor(image_size=16, tokens_per_image=cfg.num_image_tokens)
    ds = MMSFTDataset(str(data), fast, proc, "default", 64, image_token=words[cfg.image_token_id],
                      vision_start_token="<start_of_image>" if family == "gemma3" else None,
                      vision_end_token="<end_of_image>" if family == "gemma3" else None, emit_token_types=family == "paligemma")
    batch = mm_collate_fn([ds[0], ds[1]])
    assert batch["pixel_values"].shape == (2, 3, 16, 16) and "image_grid_thw" not in batch
    assert int((batch["input_ids"] == cfg.image_token_id).sum()) == 2 * cfg.num_image_tokens
    if family == "paligemma":
        assert batch["token_type_ids"].shape == batch["input_ids"].shape and int(batch["token_type_ids"][0, 0]) == 0
        answered = batch["labels"][0] != -100
        assert bool((batch["token_type_ids"][0][answered.roll(1, 0)][1:] == 1).all())     # answer tokens are fed back causally
    out = tmp_path / "out"
    cfg_file = tmp_path / "vl.json"
    cfg_file.write_text(json.dumps({
        "stage": "VL-SFT", "model_name_or_path": str(base), "compute_type": "float32", "device": "cpu", "train_dataset_path": str(data),
        "template": "default", "max_seq_len": 64, "max_steps": 4, "per_device_train_batch_size": 2, "learning_rate": 5e-3,
        "logging_steps": 1, "save_strategy": "no", "output_dir": str(out)}))
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    try:
        assert main(["train", str(cfg_file)]) == 0
    finally:
        if env is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = env
    model = AutoModelForConditionalGeneration.from_pretrained(str(out), dtype=torch.float32)
    assert model.config.model_type == family and os.path.exists(out / "tokenizer.json")


def test_vl_sft_stage_trains_paddleocr_vl(tmp_path):
    """Variable-resolution tower fed with raster-order single-frame patches from the image processor."""
    from PIL import Image
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from paddleformers_b200.cli.cli import main
    from paddleformers_b200.models.paddleocr_vl import PaddleOCRVLConfig
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    words = ["<pad>", "<s>", "</s>", "<unk>", "Human:", "Assistant:", "System:", "<image>", "<|image_pad|>", "<|vision_start|>",
             "<|vision_end|>"] + [f"w{i}" for i in range(40)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", bos_token="<s>", eos_token="</s>", unk_token="<unk>")
    cfg = PaddleOCRVLConfig(
        text_config=dict(vocab_size=len(words), hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=2,
                         num_key_value_heads=1, head_dim=16, rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [4, 2, 2]}),
        vision_config=dict(hidden_size=16, intermediate_size=32, num_hidden_layers=1, num_attention_heads=2, image_size=16, patch_size=4),
        image_token_id=words.index("<|image_pad|>"), vision_start_token_id=words.index("<|vision_start|>"),
        vision_end_token_id=words.index("<|vision_end|>"))
    base = tmp_path / "base"
    torch.manual_seed(0)
    AutoModelForConditionalGeneration.from_config(cfg, dtype=torch.float32).save_pretrained(str(base))
    fast.save_pretrained(str(base))
    rng = np.random.RandomState(0)
    data = tmp_path / "vl.jsonl"
    with open(data, "w") as f:
        for i in range(6):
            img = tmp_path / f"img{i}.png"
            Image.fromarray((rng.rand(20 + 4 * (i % 3), 24, 3) * 255).astype("uint8")).save(img)
            f.write(json.dumps({"images": [str(img)], "messages": [{"role": "user", "content": "<image> w1 w2"},
                                                                     {"role": "assistant", "content": f"w{3 + i % 5} w9"}]}) + "\n")
    out = tmp_path / "out"
    cfg_file = tmp_path / "vl.json"
    cfg_file.write_text(json.dumps({
        "stage": "VL-SFT", "model_name_or_path": str(base), "compute_type": "float32", "device": "cpu", "train_dataset_path": str(data),
        "template": "default", "max_seq_len": 64, "max_steps": 3, "per_device_train_batch_size": 2, "learning_rate": 5e-3,
        "logging_steps": 1, "save_strategy": "no", "output_dir": str(out), "min_pixels": 256, "max_pixels": 1024}))
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    try:
        assert main(["train", str(cfg_file)]) == 0
    finally:
        if env is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = env
    assert AutoModelForConditionalGeneration.from_pretrained(str(out), dtype=torch.float32).config.model_type == "paddleocr_vl"


def test_reference_only_configuration_keys_are_translated_accepted_or_refused():
    """A YAML written for the reference trainer starts a run here: aliases move to this package's fields, switches for
    behaviour that is built in are accepted, and keys that ask for something that is not provided raise with a pointer."""
    from paddleformers_b200.cli.hparams import parse_dict

    base = dict(model_name_or_path="tiny", output_dir="/tmp/x", stage="PT")
    args = parse_dict(dict(base, sharding_degree=1, evaluation_strategy="steps", use_async_save=True, unified_checkpoint=True,
                           split_param=True, amp_master_grad=True, tensor_parallel_config="enable_mp_async_allreduce enable_sp_async_reduce_scatter",
                           pipeline_parallel_config="enable_split_backward enable_overlap_p2p_comm", sharding_parallel_config="enable_stage1_overlap split_param",
                           scale_loss=32768, to_static=False))
    ta = args[-1]
    assert ta.sharding_parallel_size == 1 and ta.eval_strategy == "steps" and ta.async_save is True
    assert ta.save_checkpoint_format == "unified" and ta.pipeline_schedule == "zero_bubble" and ta.sharding_overlap is True
    with pytest.raises(ValueError, match="tracing compiler"):
        parse_dict(dict(base, to_static=True))
    with pytest.raises(ValueError, match="unknown configuration keys"):
        parse_dict(dict(base, definitely_not_a_flag=1))


def test_numa_binding_reads_the_gpu_node_from_sysfs(tmp_path, monkeypatch):
    """BIND_TRAINER_NUMA: PCI address -> numa_node -> cpulist -> sched_setaffinity, against a fake sysfs tree."""
    import os

    from paddleformers_b200.utils import numa

    assert numa.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    pci, node = tmp_path / "pci", tmp_path / "node"
    (pci / "0000:1b:00.0").mkdir(parents=True)
    (pci / "0000:1b:00.0" / "numa_node").write_text("1\n")
    (pci / "0000:9a:00.0").mkdir(parents=True)
    (pci / "0000:9a:00.0" / "numa_node").write_text("-1\n")
    allowed = sorted(os.sched_getaffinity(0))
    (node / "node1").mkdir(parents=True)
    (node / "node1" / "cpulist").write_text(f"{allowed[0]}-{allowed[0]},4000-4003\n")
    assert numa.numa_node_of_pci("0000:1b:00.0", str(pci)) == 1 and numa.numa_node_of_pci("0000:9a:00.0", str(pci)) is None
    assert numa.cpus_of_node(1, str(node))[0] == allowed[0]
    monkeypatch.setattr(numa, "gpu_pci_address", lambda i: "0000:1b:00.0" if i == 0 else ("0000:9a:00.0" if i == 1 else None))
    try:
        res = numa.bind_to_gpu_node(0, str(pci), str(node), set_memory=False)
        assert res["node"] == 1 and res["cpus"] == 1 and sorted(os.sched_getaffinity(0)) == [allowed[0]]
    finally:
        os.sched_setaffinity(0, allowed)
    assert numa.bind_to_gpu_node(1, str(pci), str(node))["node"] is None          # the platform hides the node: no-op
    assert numa.bind_to_gpu_node(2, str(pci), str(node))["reason"].startswith("no PCI")
    monkeypatch.delenv("BIND_TRAINER_NUMA", raising=False)
    assert numa.maybe_bind_trainer() is None


def test_per_operation_recompute_counts_become_refined_recompute():
    from paddleformers_b200.cli.reference_flags import translate

    out = translate({"recompute_modules": {"flash_attn": 0, "mlp_row_ln": 2}}, {"recompute_modules", "recompute_granularity", "refined_recompute"})
    assert out == {"refined_recompute": {"flash_attn": 0, "mlp_row_ln": 2}, "recompute_granularity": "full"}
    keep = translate({"recompute_modules": ["attn"], "recompute_granularity": "selective"}, {"recompute_modules", "recompute_granularity"})
    assert keep["recompute_modules"] == ["attn"]


def test_merge_preprocess_ckpt_and_env_commands(tmp_path, capsys):
    """``merge``: two checkpoints averaged into several output files with an index that loads back; unknown options refused.
    ``env`` prints the report; ``preprocess`` and ``ckpt`` reach their tools."""
    from paddleformers_b200.cli.cli import main
    from paddleformers_b200.models.configuration import named_config
    from paddleformers_b200.models.modeling import MODEL_MAPPING
    from paddleformers_b200.transformers.auto import AutoModelForCausalLM

    cfg = named_config("tiny-llama", num_hidden_layers=2, hidden_size=32, intermediate_size=48, num_attention_heads=2,
                       num_key_value_heads=2, head_dim=16, vocab_size=64)
    models = []
    for i in range(2):
        torch.manual_seed(i)
        m = MODEL_MAPPING[cfg.model_type](cfg)
        m.save_pretrained(str(tmp_path / f"m{i}"))
        models.append(m)
    spec = tmp_path / "merge.json"
    spec.write_text(json.dumps({"merge_method": "linear", "model_path_list": [str(tmp_path / "m0"), str(tmp_path / "m1")],
                                "weight_list": [0.25, 0.75], "output_path": str(tmp_path / "merged")}))
    assert main(["merge", str(spec), "max_shard_size_gb=0.00001"]) == 0          # ~10 KB per file: several files + index
    files = sorted(os.listdir(tmp_path / "merged"))
    assert "model.safetensors.index.json" in files and sum(f.endswith(".safetensors") for f in files) > 1
    merged = AutoModelForCausalLM.from_pretrained(str(tmp_path / "merged"), dtype=torch.float32)
    a, b = (dict(m.named_parameters()) for m in models)
    for n, p in merged.named_parameters():
        assert torch.allclose(p, 0.25 * a[n] + 0.75 * b[n], atol=1e-6), n
    with pytest.raises(ValueError, match="unknown merge options"):
        main(["merge", str(spec), "blend=1"])
    capsys.readouterr()
    assert main(["env"]) == 0
    assert "torch" in capsys.readouterr().out
    with pytest.raises(SystemExit):
        main(["preprocess", "--help"])


def test_vl_sft_stage_trains_ernie4_5_vl(tmp_path):
    """ERNIE-4.5-VL through the VL-SFT stage: single-frame patches in merge-block order, image markers routed to the vision
    experts, the published checkpoint layout written at the end."""
    from PIL import Image
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from paddleformers_b200.cli.train import run_tuner
    from paddleformers_b200.models.ernie4_5_vl import Ernie4_5VLConfig
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    words = ["<pad>", "<s>", "</s>", "<unk>", "Human:", "Assistant:", "System:", "<image>", "<|IMAGE_PLACEHOLDER|>", "<|IMAGE_START|>",
             "<|IMAGE_END|>", "<|VIDEO_PLACEHOLDER|>"] + [f"w{i}" for i in range(40)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", bos_token="<s>", eos_token="</s>", unk_token="<unk>")
    cfg = Ernie4_5VLConfig(
        text_config=dict(vocab_size=len(words), hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2,
                         num_key_value_heads=1, moe_intermediate_size=[16, 8], moe_k=2, moe_num_experts=4, moe_num_shared_experts=1,
                         mlp_layer_types=["dense", "sparse"], rope_parameters={"rope_theta": 10000.0, "mrope_section": [3, 3, 2]}),
        vision_config=dict(depth=1, hidden_size=16, num_heads=2, intermediate_size=32, patch_size=4, spatial_merge_size=2),
        image_token_id=words.index("<|IMAGE_PLACEHOLDER|>"), video_token_id=words.index("<|VIDEO_PLACEHOLDER|>"),
        image_start_token_id=words.index("<|IMAGE_START|>"), image_end_token_id=words.index("<|IMAGE_END|>"),
        video_start_token_id=None, video_end_token_id=None)
    base = tmp_path / "base"
    torch.manual_seed(0)
    AutoModelForConditionalGeneration.from_config(cfg, dtype=torch.float32).save_pretrained(str(base))
    fast.save_pretrained(str(base))
    rng = np.random.RandomState(0)
    data = tmp_path / "vl.jsonl"
    with open(data, "w") as f:
        for i in range(6):
            img = tmp_path / f"img{i}.png"
            Image.fromarray((rng.rand(16 + 8 * (i % 2), 24, 3) * 255).astype("uint8")).save(img)
            f.write(json.dumps({"images": [str(img)], "messages": [{"role": "user", "content": "<image> w1 w2"},
                                                                     {"role": "assistant", "content": f"w{3 + i % 5} w9"}]}) + "\n")
    out = tmp_path / "out"
    cfg_file = tmp_path / "vl.json"
    cfg_file.write_text(json.dumps({
        "stage": "VL-SFT", "model_name_or_path": str(base), "compute_type": "float32", "device": "cpu", "train_dataset_path": str(data),
        "template": "default", "max_seq_len": 64, "max_steps": 4, "per_device_train_batch_size": 2, "learning_rate": 5e-3,
        "logging_steps": 1, "save_strategy": "no", "output_dir": str(out), "min_pixels": 256, "max_pixels": 1024}))
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    try:
        trainer, _ = run_tuner([str(cfg_file)])
    finally:
        if env is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = env
    losses = [h["loss"] for h in trainer.state.log_history if "loss" in h]
    assert len(losses) == 4 and losses[-1] < losses[0]
    batch = next(iter(trainer.get_train_dataloader()))
    assert batch["pixel_values"].shape[1] == 3 * 4 * 4 and int(trainer.model.vision_rows(batch["input_ids"]).sum()) > 0
    from safetensors import safe_open

    with safe_open(str(out / "model.safetensors"), "pt") as f:
        keys = set(f.keys())
    assert "model.layers.1.mlp.gate.weight_1" in keys and "model.layers.1.mlp.experts.7.down_proj.weight" in keys
    assert "model.vision_model.patch_embed.proj.weight" in keys and "model.resampler_model.spatial_linear.0.weight" in keys
    again = AutoModelForConditionalGeneration.from_pretrained(str(out), dtype=torch.float32)
    assert again.config.model_type == "ernie4_5_vl_moe" and os.path.exists(out / "tokenizer.json")
