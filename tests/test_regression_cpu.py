"""Loss replay: tiny truncated versions of real architectures train for a few steps through the ``train`` command on a fixed
corpus and must reproduce stored per-step losses and the token ids generated afterwards
(the reference's main correctness gate: tests/integration_test/check_loss.py:22-120 and scripts/regression/test_models.py compare
with stored values in the same way). ``UPDATE_GROUND_TRUTH=1 python -m pytest tests/test_regression_cpu.py`` rewrites the
stored values after an intended numerical change."""
import json
import os

import pytest
import torch

from paddleformers_b200.models.configuration import named_config
from paddleformers_b200.transformers.auto import AutoConfig, AutoModelForCausalLM

TRUTH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures", "regression_ground_truth.json")

CASES = {
    # name: (family, configuration overrides, extra training options)
    "llama_pt": ("llama", dict(), dict()),
    "llama_pt_accum_recompute": ("llama", dict(), dict(gradient_accumulation_steps=2, recompute_granularity="full",
                                                        refined_recompute={"flash_attn": 0})),
    "qwen3_moe_pt": ("qwen3_moe", dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, router_aux_loss_coef=1e-3), dict()),
    "glm4_moe_pt": ("glm4_moe", dict(n_routed_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, n_shared_experts=1,
                                     first_k_dense_replace=1, partial_rotary_factor=0.5, use_qk_norm=True), dict()),
    "deepseek_v3_mtp_pt": ("deepseek_v3", dict(n_routed_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, n_shared_experts=1,
                                               first_k_dense_replace=1, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16,
                                               qk_rope_head_dim=8, v_head_dim=16, n_group=2, topk_group=1, num_nextn_predict_layers=1),
                           dict()),
    "gemma4_moe_pt": ("gemma4_text", dict(head_dim=16, global_head_dim=32, sliding_window=8, vocab_size_per_layer_input=96,
                                          hidden_size_per_layer_input=8, enable_moe_block=True, num_experts=4, top_k_experts=2,
                                          moe_intermediate_size=32, attention_k_eq_v=True, num_global_key_value_heads=1,
                                          layer_types=["sliding_attention", "full_attention", "full_attention"]), dict()),
}
BASE = dict(vocab_size=96, hidden_size=48, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
            max_position_embeddings=128)


def _corpus(path):
    """A fixed pre-training corpus in the mmap format: 64 documents of a noisy counting language."""
    from paddleformers_b200.data.indexed_dataset import MMapIndexedDatasetBuilder

    import numpy as np

    g = torch.Generator().manual_seed(1234)
    b = MMapIndexedDatasetBuilder(path, dtype=np.uint16)
    for _ in range(64):
        start = int(torch.randint(2, 40, (1,), generator=g))
        n = int(torch.randint(20, 60, (1,), generator=g))
        doc = [(start + 3 * i) % 90 + 2 for i in range(n)]
        for j in torch.randint(0, n, (3,), generator=g).tolist():
            doc[j] = int(torch.randint(2, 92, (1,), generator=g))
        b.add_document(doc + [1])
    b.finalize()


def _run(name, tmp_path):
    from paddleformers_b200.cli.train import run_tuner
    from paddleformers_b200.generation.utils import GenerationConfig

    family, over, extra = CASES[name]
    torch.manual_seed(7)
    cfg = AutoConfig.for_model(family, **{**BASE, **over})
    base = tmp_path / "base"
    AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).save_pretrained(str(base))
    _corpus(str(tmp_path / "corpus"))
    spec = dict(stage="PT", model_name_or_path=str(base), compute_type="float32", device="cpu", input_dir=f"1.0 {tmp_path / 'corpus'}",
                dataset_type="pretrain", max_seq_len=32, max_steps=6, per_device_train_batch_size=2, learning_rate=2e-3,
                lr_scheduler_type="constant", logging_steps=1, save_strategy="no", output_dir=str(tmp_path / "out"), seed=11, **extra)
    f = tmp_path / "cfg.json"
    f.write_text(json.dumps(spec))
    trainer, _ = run_tuner([str(f)])
    losses = [round(h["loss"], 6) for h in trainer.state.log_history if "loss" in h]
    model = trainer.model.eval()
    prompt = torch.tensor([[5, 8, 11, 14, 17, 20]])
    ids = model.generate(prompt, GenerationConfig(max_new_tokens=8, eos_token_id=-1))[0, prompt.shape[1]:].tolist()
    return {"losses": losses, "generated": ids}, model, prompt


@pytest.mark.parametrize("name", sorted(CASES))
def test_loss_replay_and_generated_tokens(name, tmp_path):
    got, model, prompt = _run(name, tmp_path)
    truth = json.load(open(TRUTH)) if os.path.exists(TRUTH) else {}
    if os.environ.get("UPDATE_GROUND_TRUTH") == "1":
        truth[name] = got
        with open(TRUTH, "w") as f:
            json.dump(truth, f, indent=1, sort_keys=True)
        return
    assert name in truth, f"no stored values for {name}: run with UPDATE_GROUND_TRUTH=1"
    want = truth[name]
    assert len(got["losses"]) == len(want["losses"]) == 6
    for a, b in zip(got["losses"], want["losses"]):
        assert abs(a - b) <= 1e-4 * max(1.0, abs(b)), (name, got["losses"], want["losses"])
    assert got["losses"][-1] < got["losses"][0]
    if got["generated"] != want["generated"]:
        # greedy decoding may break a numerical tie differently on another machine: the stored continuation must still be
        # (within rounding) the arg-max at every step when it is fed back
        full = torch.cat([prompt, torch.tensor([want["generated"]])], dim=1)
        with torch.no_grad():
            logits = model(full[:, :-1], return_logits=True).logits[0, prompt.shape[1] - 1:].float()
        chosen = logits.gather(1, torch.tensor(want["generated"])[:, None])[:, 0]
        assert (logits.max(-1).values - chosen).max() < 1e-3, (name, got["generated"], want["generated"])
