

def test_gradient_accumulation_reaches_the_wrapped_model():
    """The trainer sets the number of accumulation steps on the model it is given; through the adapter wrapper it must arrive
    at the wrapped model, which divides its loss by it (otherwise loss and gradients grow with the number of micro-batches)."""
    import torch

    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.models.configuration import LlamaConfig
    from paddleformers_b200.models.modeling import MODEL_MAPPING
    from paddleformers_b200.peft.lora import LoRAConfig, LoRAModel

    class Rows(torch.utils.data.Dataset):
        def __len__(self):
            return 8

        def __getitem__(self, i):
            g = torch.Generator().manual_seed(i)
            ids = torch.randint(0, 64, (17,), generator=g)
            return {"input_ids": ids[:-1], "labels": ids[1:].clone()}

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=2,
                      num_key_value_heads=2, dtype="float32")
    model = LoRAModel(MODEL_MAPPING[cfg.model_type](cfg), LoRAConfig(r=2, lora_alpha=4))
    model.loss_accumulation_steps = 4
    assert model.model.loss_accumulation_steps == 4 and model.loss_accumulation_steps == 4
    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=1, gradient_accumulation_steps=4, max_steps=1,
                             learning_rate=1e-3, logging_steps=1, save_strategy="no", max_seq_len=16, device="cpu")
    args.setup_parallel()
    tr = Trainer(model=model, args=args, train_dataset=Rows())
    tr.train()
    loss = [h["loss"] for h in tr.state.log_history if "loss" in h][0]
    assert 3.0 < loss < 5.5, loss            # about ln(64) = 4.16 for a fresh model, not four times that
