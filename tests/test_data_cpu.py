"""Data pipeline: templates, packing, collators and their mask semantics, mmap datasets."""
import json
import os

import numpy as np
import pytest
import torch

from paddleformers_b200.datasets.collate import (calc_padding_size, collate_fn, dpo_collate_fn,
                                                 gen_attn_mask_startend_row_indices, gen_self_attn_mask)
from paddleformers_b200.datasets.sft_dataset import (IGNORE_INDEX, Sequence, create_dataset, encode_example, pack_sequences)
from paddleformers_b200.datasets.template import get_template
from paddleformers_b200.ops.functional import dense_mask_from_kend


class _Tok:
    """Whitespace tokenizer with a growing vocabulary (enough for dataflow tests)."""

    eos_token, eos_token_id, pad_token_id = "</s>", 1, 0

    def __init__(self):
        self.vocab = {"<pad>": 0, "</s>": 1}

    def encode(self, text, add_special_tokens=False):
        out = []
        for w in text.replace("</s>", " </s> ").split():
            out.append(self.vocab.setdefault(w, len(self.vocab)))
        return out


def _seq(n, start=0):
    return Sequence(list(range(start, start + n)), list(range(start + 1, start + n + 1)), list(range(n)))


def test_row_indices_match_dense_mask_and_reference_semantics():
    kend = gen_attn_mask_startend_row_indices([3, 2], 7)
    assert kend.tolist() == [3, 3, 3, 5, 5, 5, 6]  # documents end at 3 and 5, pad keys mask themselves
    dense = gen_self_attn_mask([3, 2], 7)[0]
    ref = dense_mask_from_kend(torch.from_numpy(kend)[None], 7, True, "cpu")[0].numpy()
    assert (dense == ref).all()
    assert dense[4, 3] and not dense[4, 2] and not dense[5, 3] and not dense[6, 6]
    assert gen_attn_mask_startend_row_indices([3, 2], 7, use_global_causal_attn=True).tolist() == [5, 5, 5, 5, 5, 5, 6]


def test_packing_strategies():
    seqs = [_seq(n) for n in (5, 3, 6, 2, 4)]
    greedy = list(pack_sequences(seqs, 8, "greedy"))
    assert [[len(s) for s in b] for b in greedy] == [[5, 3], [6, 2], [4]]
    bins = list(pack_sequences(seqs, 8, "binpacking"))
    assert all(sum(len(s) for s in b) <= 8 for b in bins) and len(bins) == 3
    assert sorted(len(s) for b in bins for s in b) == [2, 3, 4, 5, 6]
    assert len(list(pack_sequences(seqs, 8, "truncate"))) == 5


def test_collate_padding_free_and_padded():
    class A:
        context_parallel_size, tensor_model_parallel_size, sequence_parallel, fp8 = 2, 2, True, None

    assert calc_padding_size(13, A) == 16
    batch = [[_seq(3), _seq(2, 10)], [_seq(4, 20)]]
    out = collate_fn(batch, _Tok(), None, max_seq_len=6)
    assert out["input_ids"].shape == (2, 6) and out["labels"][0, 5] == IGNORE_INDEX
    assert out["attn_mask_startend_row_indices"][0].tolist() == [3, 3, 3, 5, 5, 5]
    assert out["position_ids"][0].tolist() == [0, 1, 2, 0, 1, 0]
    flat = collate_fn(batch, _Tok(), None, padding_free=True)
    assert flat["input_ids"].shape == (1, 9)
    assert flat["attn_mask_startend_row_indices"][0].tolist() == [3, 3, 3, 5, 5, 9, 9, 9, 9]


def test_template_masks_prompt_and_dataset_roundtrip(tmp_path):
    tok = _Tok()
    ex = {"messages": [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi there"},
                       {"role": "assistant", "content": "hello friend"}]}
    s = encode_example(ex, tok, get_template("default"), 64)
    trained = [l for l in s.labels if l != IGNORE_INDEX]
    assert trained == tok.encode("hello friend </s>")
    # tool call rendering
    pairs = get_template("qwen").render_turns(
        [{"role": "user", "content": "weather?"}, {"role": "assistant", "content": "", "tool_calls": [{"name": "get", "arguments": {"c": 1}}]},
         {"role": "tool", "content": "sunny"}, {"role": "assistant", "content": "It is sunny"}], tools=[{"name": "get"}])
    assert "<tool_call>" in pairs[0][1] and "<tool_response>" in pairs[1][0] and "# Tools" in pairs[0][0]
    p = tmp_path / "a.jsonl"
    with open(p, "w") as f:
        for i in range(10):
            f.write(json.dumps({"src": [f"question {i}"], "tgt": [f"answer {i} " * (i + 1)]}) + "\n")
    ds = create_dataset(str(p), tok, 32, template="default", packing="greedy")
    assert len(ds) >= 2 and all(sum(len(s) for s in sample) <= 32 for sample in ds.samples)
    mixed = create_dataset(f"{p},{p}", tok, 32, dataset_prob="0.5,0.5", template="default", mix_strategy="interleave", streaming=True)
    assert sum(len(sample) for sample in mixed) == 20


def test_dpo_collate_layout():
    out = dpo_collate_fn([{"prompt_ids": [5, 6, 7], "chosen_ids": [8, 9], "rejected_ids": [10, 11, 12]}], max_seq_len=12)
    assert out["input_ids"][0, :11].tolist() == [5, 6, 7, 8, 9, 5, 6, 7, 10, 11, 12]
    assert out["response_indexs"][0].tolist() == [0, 2, 4, 7, 10]
    assert out["chosen_labels"][0, 2:4].tolist() == [8, 9] and out["rejected_labels"][0, 7:10].tolist() == [10, 11, 12]
    assert out["attn_mask_startend_row_indices"][0, :11].tolist() == [5] * 5 + [11] * 6


def test_mmap_dataset_and_gpt_samples(tmp_path):
    from paddleformers_b200.data.indexed_dataset import (BlendableDataset, GPTDataset, MMapIndexedDataset,
                                                         MMapIndexedDatasetBuilder, build_train_valid_test_datasets)

    prefix = str(tmp_path / "corpus")
    b = MMapIndexedDatasetBuilder(prefix, dtype=np.uint16)
    docs = [np.arange(10 * i, 10 * i + 7 + i) for i in range(12)]
    for d in docs:
        b.add_document(d)
    b.finalize()
    ds = MMapIndexedDataset(prefix)
    assert len(ds) == 12 and (ds[3] == docs[3]).all() and (ds.get(3, 2, 3) == docs[3][2:5]).all()
    g = GPTDataset(ds, None, num_samples=8, seq_length=16, seed=1, shuffle=False)
    stream = np.concatenate(docs)
    item = g[2]
    assert item["input_ids"].tolist() == stream[32:48].tolist() and item["labels"].tolist() == stream[33:49].tolist()
    g2 = GPTDataset(ds, None, num_samples=8, seq_length=16, seed=1, shuffle=True)
    g3 = GPTDataset(ds, None, num_samples=8, seq_length=16, seed=1, shuffle=True)
    assert all(torch.equal(g2[i]["input_ids"], g3[i]["input_ids"]) for i in range(len(g2)))
    blend = BlendableDataset([g, g2], [0.75, 0.25], 16)
    assert (blend.dataset_index == 0).sum() == 12
    tr, va, te = build_train_valid_test_datasets([prefix], "8,2,2", 16, [4, 1, 1], seed=3)
    assert tr is not None and len(tr) >= 4 and va is not None


def test_native_index_helpers_match_numpy():
    """The compiled index builders and the numpy fallbacks produce identical indices."""
    import numpy as np

    from paddleformers_b200.data import indexed_dataset as idx

    if idx._host() is None:
        pytest.skip("no C++ compiler available")
    rng = np.random.RandomState(0)
    sizes = rng.randint(1, 50, size=200).astype(np.int32)
    order = rng.permutation(np.tile(np.arange(200), 3)).astype(np.int64)
    for seq, ns in ((16, 10), (7, 10_000), (128, 50)):
        a = idx.build_sample_index(sizes, order, seq, ns, use_native=True)
        b = idx.build_sample_index(sizes, order, seq, ns, use_native=False)
        assert a.shape == b.shape and (a == b).all()
    ds = [list(range(10)), list(range(20)), list(range(5))]
    x = idx.BlendableDataset(ds, [0.5, 0.3, 0.2], 1000, use_native=True)
    y = idx.BlendableDataset(ds, [0.5, 0.3, 0.2], 1000, use_native=False)
    assert (x.dataset_index == y.dataset_index).all() and (x.sample_index == y.sample_index).all()
    share = np.bincount(x.dataset_index, minlength=3) / 1000
    assert np.allclose(share, [0.5, 0.3, 0.2], atol=2e-3)
    # document bounds of a packed sample: documents end after every eos (token 0 here)
    import ctypes

    ids = np.array([5, 3, 0, 7, 7, 7, 0, 0, 2, 9], dtype=np.int64)
    kend, pos = np.empty(10, dtype=np.int32), np.empty(10, dtype=np.int64)
    idx._host().pfb_build_doc_bounds(idx._ptr(ids, ctypes.c_int64), 10, 0, idx._ptr(kend, ctypes.c_int32), idx._ptr(pos, ctypes.c_int64))
    assert kend.tolist() == [3, 3, 3, 7, 7, 7, 7, 8, 10, 10] and pos.tolist() == [0, 1, 2, 0, 1, 2, 3, 0, 0, 1]


def test_every_template_renders_a_multi_turn_conversation():
    from paddleformers_b200.datasets.template import TEMPLATES

    msgs = [{"role": "system", "content": "SYS"}, {"role": "user", "content": "Q1"}, {"role": "assistant", "content": "A1"},
            {"role": "user", "content": "Q2"}, {"role": "assistant", "content": "A2"}]
    assert len(TEMPLATES) >= 45
    for name, t in TEMPLATES.items():
        pairs = t.render_turns(msgs)
        assert len(pairs) == 2, name
        text = "".join(p + r for p, r in pairs)
        for piece in ("Q1", "A1", "Q2", "A2"):
            assert piece in text, (name, piece)
        assert text.index("Q1") < text.index("A1") < text.index("Q2") < text.index("A2"), name
        if name != "empty":
            assert "SYS" in pairs[0][0], name


def _stream_worker(rank, world):
    import torch
    import torch.distributed as dist

    from paddleformers_b200.data.dist_dataloader import StreamDistDataLoader

    class Stream(torch.utils.data.IterableDataset):
        reads = 0

        def __iter__(self):
            for i in range(11):            # 11 samples, batch 2, 2 ranks: two global batches, the rest is dropped
                Stream.reads += 1
                yield {"input_ids": torch.full((4,), i)}

    def collate(items):
        return {"input_ids": torch.stack([x["input_ids"] for x in items])}

    ds = Stream() if rank == 0 else None
    loader = StreamDistDataLoader(ds, batch_size=2, collate_fn=collate, stream_group=dist.group.WORLD)
    got = [b["input_ids"][:, 0].tolist() for b in loader]
    return got, (Stream.reads if rank == 0 else 0)


def test_stream_loader_reads_on_one_rank_and_scatters():
    from dist_utils import run_distributed

    res = run_distributed(_stream_worker, 2)
    assert res[0][0] == [[0, 1], [4, 5]] and res[1][0] == [[2, 3], [6, 7]]
    assert res[0][1] >= 8 and res[1][1] == 0
    # one process: plain batching of the stream
    import torch

    from paddleformers_b200.data.dist_dataloader import StreamDistDataLoader

    out = list(StreamDistDataLoader(iter(range(5)) and list(range(5)), batch_size=2, collate_fn=lambda x: torch.tensor(x)))
    assert [o.tolist() for o in out] == [[0, 1], [2, 3]]


def test_rl_prompt_dataset_left_pads_and_batch_container_operations(tmp_path):
    import json

    import numpy as np
    import pytest
    import torch

    from paddleformers_b200.datasets.rl_dataset import DataProto, RLHFDataset, left_padding, rl_collate_fn

    class Tok:
        chat_template = None
        pad_token_id = 0

        def __call__(self, text, add_special_tokens=True):
            return {"input_ids": ([1] if add_special_tokens else []) + [2 + (ord(c) % 50) for c in text]}

    path = tmp_path / "prompts.jsonl"
    path.write_text("\n".join(json.dumps({"src": s, "tgt": t}) for s, t in
                              [("hi", "a"), ("what is 2+2", "4"), ("x" * 40, "long"), ("bye now", "ok")]))
    ds = RLHFDataset(str(path), Tok(), max_prompt_len=16, requires_label=True, response_key="tgt")
    assert len(ds) == 3                                              # the 40-character prompt is dropped, not cut
    batch = rl_collate_fn([ds[i] for i in range(3)], pad_token_id=0, requires_label=True)
    ids, mask = batch["input_ids"], batch["attention_mask"]
    assert ids.shape == (3, 12) and ids[0, :9].eq(0).all() and ids[0, 9] == 1 and mask[0].tolist() == [0] * 9 + [1] * 3
    assert batch["position_ids"][0].tolist() == [0] * 9 + [0, 1, 2] and batch["position_ids"][1].tolist() == list(range(12))
    assert batch["label_ids"].shape[0] == 3
    assert left_padding([torch.tensor([1, 2, 3])], 0, 2).tolist() == [[2, 3]]

    dp = DataProto.from_dict({"input_ids": ids, "attention_mask": mask}, {"uid": ["a", "b", "c"]}, {"temperature": 0.7})
    assert len(dp) == 3 and dp[1]["uid"] == "b"
    padded, pad = dp.pad_to_divisor(2)
    assert len(padded) == 4 and pad == 1 and padded[3]["uid"] == "a"
    parts = padded.chunk(2)
    assert [len(p) for p in parts] == [2, 2] and parts[1].non_tensor_batch["uid"].tolist() == ["c", "a"]
    back = DataProto.concat(parts).unpad(pad)
    assert torch.equal(back.batch["input_ids"], ids) and back.non_tensor_batch["uid"].tolist() == ["a", "b", "c"]
    rep = dp.repeat(2, interleave=True)
    assert rep.non_tensor_batch["uid"].tolist() == ["a", "a", "b", "b", "c", "c"] and torch.equal(rep.batch["input_ids"][1], ids[0])
    assert dp.repeat(2, interleave=False).non_tensor_batch["uid"].tolist() == ["a", "b", "c", "a", "b", "c"]
    sel = dp.select(batch_keys=["input_ids"])
    assert set(sel.batch) == {"input_ids"} and "uid" in sel.non_tensor_batch
    scores = DataProto.from_dict({"reward": torch.tensor([1.0, 0.0, 0.5])})
    dp.union(scores)
    assert "reward" in dp.batch
    with pytest.raises(ValueError):
        dp.union(DataProto.from_dict({"reward": torch.zeros(3)}))
    popped = dp.pop(batch_keys=["reward"])
    assert "reward" not in dp.batch and popped.batch["reward"].tolist() == [1.0, 0.0, 0.5]
    dp.reorder(torch.tensor([2, 0, 1]))
    assert dp.non_tensor_batch["uid"].tolist() == ["c", "a", "b"] and torch.equal(dp.batch["input_ids"][1], ids[0])
    seen = [m.non_tensor_batch["uid"].tolist() for m in dp.select().pad_to_divisor(1)[0].make_iterator(1, epochs=2, seed=0)]
    assert len(seen) == 6 and sorted(x[0] for x in seen[:3]) == ["a", "b", "c"]
    with pytest.raises(ValueError):
        DataProto.from_dict({"a": torch.zeros(2)}, {"b": np.zeros(3)})


def test_image_processor_raster_order_matches_plain_patch_cutting():
    """Towers that merge patches after the encoder read them row by row: the processor's raster layout equals cutting the
    normalised image into P x P tiles in reading order, and holds the same patches as the merge-block layout."""
    import numpy as np
    import torch

    from paddleformers_b200.transformers.image_processing import Qwen2VLImageProcessor

    rng = np.random.RandomState(0)
    img = (rng.rand(40, 56, 3) * 255).astype("uint8")
    kw = dict(patch_size=4, merge_size=2, temporal_patch_size=1, min_pixels=64, max_pixels=4096, image_mean=(0.5,) * 3, image_std=(0.5,) * 3)
    raster = Qwen2VLImageProcessor(raster_order=True, **kw)([img])
    blocks = Qwen2VLImageProcessor(**kw)([img])
    t, gh, gw = raster["image_grid_thw"][0].tolist()
    assert raster["pixel_values"].shape == (gh * gw, 3 * 4 * 4) and torch.equal(raster["image_grid_thw"], blocks["image_grid_thw"])
    tiles = raster["pixel_values"].view(gh, gw, 3, 4, 4)
    full = tiles.permute(2, 0, 3, 1, 4).reshape(3, gh * 4, gw * 4)                 # stitch the tiles back into the image
    again = full.view(3, gh, 4, gw, 4).permute(1, 3, 0, 2, 4).reshape(gh * gw, -1)
    assert torch.equal(again, raster["pixel_values"])
    reordered = blocks["pixel_values"].view(gh // 2, gw // 2, 2, 2, -1).permute(0, 2, 1, 3, 4).reshape(gh * gw, -1)
    assert torch.equal(reordered, raster["pixel_values"])


def test_model_files_resolve_from_the_cache_of_the_selected_hub(tmp_path, monkeypatch):
    """DOWNLOAD_SOURCE picks whose cache is searched first; flat <org>/<name> layouts (ModelScope, AI Studio) and the
    Hugging Face snapshot layout both resolve; nothing is downloaded."""
    from paddleformers_b200.utils.download import resolve_dir, resolve_file_path

    ms = tmp_path / "ms"
    (ms / "hub" / "org" / "tiny").mkdir(parents=True)
    (ms / "hub" / "org" / "tiny" / "config.json").write_text("{\"from\": \"modelscope\"}")
    hf = tmp_path / "hf"
    snap = hf / "hub" / "models--org--tiny" / "snapshots" / "abc"
    snap.mkdir(parents=True)
    (snap / "config.json").write_text("{\"from\": \"huggingface\"}")
    monkeypatch.setenv("MODELSCOPE_CACHE", str(ms))
    monkeypatch.setenv("HF_HOME", str(hf))
    monkeypatch.setenv("HF_HUB_OFFLINE", "1")
    monkeypatch.setenv("DOWNLOAD_SOURCE", "modelscope")
    assert "modelscope" in open(resolve_file_path("org/tiny", "config.json")).read()
    monkeypatch.setenv("DOWNLOAD_SOURCE", "huggingface")
    assert "huggingface" in open(resolve_file_path("org/tiny", "config.json")).read()
    assert resolve_dir("org/tiny") == str(snap)
    with pytest.raises(FileNotFoundError):
        resolve_file_path("org/absent", "config.json")


def test_phi4_processors_match_hugging_face_and_feed_the_model():
    """Dynamic-HD image tiling (grid choice, white padding, global view, patch masks, placeholder count) and the Kaldi-style
    log-mel front end (pre-emphasis, Hamming window, mel-space triangles) against ``transformers``; the combined processor
    expands the prompt so that the model finds one placeholder per feature row."""
    import numpy as np
    from transformers.models.phi4_multimodal.feature_extraction_phi4_multimodal import Phi4MultimodalFeatureExtractor
    from transformers.models.phi4_multimodal.image_processing_phi4_multimodal import Phi4MultimodalImageProcessor

    from paddleformers_b200.models.phi4_multimodal import Phi4MultimodalConfig, Phi4MultimodalForCausalLM, Phi4MultimodalProcessor
    from paddleformers_b200.transformers.audio_processing import KaldiFbankFeatureExtractor
    from paddleformers_b200.transformers.image_processing import DynamicHDImageProcessor

    rng = np.random.default_rng(0)
    imgs = [rng.integers(0, 255, (300, 700, 3), dtype=np.uint8), rng.integers(0, 255, (900, 500, 3), dtype=np.uint8)]
    want = Phi4MultimodalImageProcessor()(images=[torch.from_numpy(i).permute(2, 0, 1) for i in imgs], return_tensors="pt")
    got = DynamicHDImageProcessor()(imgs)
    for k in ("image_pixel_values", "image_attention_mask", "image_sizes"):
        assert want[k].shape == got[k].shape and (want[k].float() - got[k].float()).abs().max() < 1e-5, k
    assert want["num_img_tokens"].tolist() == got["num_img_tokens"] == [735, 1617]
    assert DynamicHDImageProcessor(dynamic_hd=4).grid(2000, 3100) == (2, 1)             # more tiles than allowed: closest aspect ratio
    a, b = rng.standard_normal(16000).astype(np.float32) * 0.1, rng.standard_normal(9000).astype(np.float32) * 0.1
    w = Phi4MultimodalFeatureExtractor()([a, b], sampling_rate=16000, return_tensors="pt")
    g = KaldiFbankFeatureExtractor()([a, b], sampling_rate=16000)
    n_b = int(g["audio_attention_mask"][1].sum())
    assert w["audio_embed_sizes"].tolist() == g["audio_embed_sizes"].tolist() == [13, 7] and n_b == int(w["audio_attention_mask"][1].sum())
    assert (w["audio_input_features"][0] - g["audio_input_features"][0]).abs().max() < 1e-4
    assert (w["audio_input_features"][1, :n_b] - g["audio_input_features"][1, :n_b]).abs().max() < 1e-4
    with pytest.raises(ValueError, match="16000"):
        KaldiFbankFeatureExtractor()(a, sampling_rate=8000)

    class Tok:                                     # whitespace tokenizer that knows the two tags
        vocab = {"<|image|>": 290, "<|audio|>": 291}

        def encode(self, text, add_special_tokens=False):
            import re

            return [self.vocab.get(t, 5 + len(t) % 50) for t in re.findall(r"<\|image\|>|<\|audio\|>|\S+", text)]

    cfg = Phi4MultimodalConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=1, num_attention_heads=4,
                               num_key_value_heads=2, max_position_embeddings=4096,
                               vision_config=dict(hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2,
                                                  image_size=56, patch_size=14, crop_size=56, image_token_id=290),
                               audio_config=dict(hidden_size=32, intermediate_size=48, num_blocks=1, num_attention_heads=2,
                                                 ext_pw_out_channel=32, depthwise_separable_out_channel=32, input_size=80,
                                                 nemo_conv_channels=8, nemo_final_size=10, time_reduction=8, bias_max_distance=20,
                                                 audio_token_id=291))
    torch.manual_seed(0)
    model = Phi4MultimodalForCausalLM(cfg, dtype=torch.float32).eval()
    proc = Phi4MultimodalProcessor(Tok(), image_processor=DynamicHDImageProcessor(crop=56, patch_size=14, dynamic_hd=4))
    batch = proc("look <|image|> and listen <|audio|> then answer", images=[imgs[0][:60, :130]], audio=[a], sampling_rate=16000)
    # 60 x 130 pixels cover 2 x 3 tiles of 56, more than 4: the 1 x 2 grid is chosen; every tile pools to 2 x 2 rows
    assert int((batch["input_ids"] == 290).sum()) == (2 * 4 + 2) + 1 + (2 * 2 + 2) == 17
    assert int((batch["input_ids"] == 291).sum()) == 13
    with torch.no_grad():
        out = model(**batch)
    assert out.logits.shape[:2] == batch["input_ids"].shape and torch.isfinite(out.logits).all()
    with pytest.raises(ValueError, match="tags"):
        proc("no tags here", images=[imgs[0]])


def test_molmo_multi_crop_processor_is_geometrically_consistent_and_feeds_the_model():
    """Every ``<im_patch>`` token is claimed by exactly one pooled cell of one crop; the cell and the token describe the same
    2 x 2 patches of the canvas; crops overlap by the margins; the overview comes first; masks give the visible fraction of a
    patch; the model adds feature rows at the claimed positions only."""
    import numpy as np

    from paddleformers_b200.models.molmo import MolmoConfig, MolmoForCausalLM, MolmoProcessor
    from paddleformers_b200.transformers.image_processing import MolmoImageProcessor

    proc = MolmoImageProcessor()
    rng = np.random.default_rng(0)
    img = rng.integers(0, 255, (500, 900, 3), dtype=np.uint8)
    PATCH, COL, START, END = 3, 4, 1, 2
    images, masks, tokens, idx = proc.preprocess_one(img, PATCH, COL, START, END)
    rows, cols = proc.select_tiling(500 - 112, 900 - 112, 224)
    assert (rows, cols) == (2, 4) and images.shape == (1 + 8, 576, 588) and masks.shape == (9, 576) and idx.shape == (9, 144)
    valid = idx[idx >= 0]
    assert len(valid) == int((tokens == PATCH).sum()) == len(set(valid.tolist())) and (tokens[valid] == PATCH).all()
    assert tokens[0] == START and tokens[12 * 13 + 1] == END and (idx[0] == np.flatnonzero(tokens == PATCH)[:144]).all()
    # geometry: crop (i, j) starts 16 patches after its neighbour; cell (a, b) of it covers canvas patches (16 i + 2 a, 16 j + 2 b);
    # the token at row R, column C of the pooled canvas grid covers canvas patches (2 R, 2 C)
    Wp = (cols * 16 + 8 + 1) // 2
    base = (1 + 12 * 13 + 1) + 1
    for c in range(rows * cols):
        i, j = divmod(c, cols)
        for cell in np.flatnonzero(idx[1 + c] >= 0):
            a, b = divmod(int(cell), 12)
            R, C = divmod(int(idx[1 + c, cell]) - base, Wp + 1)
            assert (16 * i + 2 * a, 16 * j + 2 * b) == (2 * R, 2 * C)
    # neighbouring crops share 8 patch columns; the picture is centred with black (normalised zero) bars and masks say so
    left, right = images[1].reshape(24, 24, 588), images[2].reshape(24, 24, 588)
    assert np.allclose(left[:, 16:], right[:, :8])
    assert masks[-1].min() == masks[-1].max() == -1 and 0 <= masks[:-1].min() and masks[:-1].max() == 1
    _, m2, _, _ = proc.preprocess_one(rng.integers(0, 255, (333, 900, 3), dtype=np.uint8), PATCH, COL, START, END)
    assert (m2[:-1] == 0).any() and ((m2[:-1] > 0) & (m2[:-1] < 1)).any() and (m2[:-1] == 1).any()    # bars, their edge, the picture
    # a small image that fits one crop: one crop whose whole 12 x 12 grid is used
    _, _, t1, i1 = proc.preprocess_one(rng.integers(0, 255, (200, 300, 3), dtype=np.uint8), PATCH, COL, START, END)
    assert i1.shape == (2, 144) and (i1 >= 0).all() and int((t1 == PATCH).sum()) == 288

    class Tok:
        bos_token_id, eos_token_id = 0, 0
        vocab = {"<im_start>": 91, "<im_end>": 92, "<im_patch>": 93, "<im_col>": 94}

        def encode(self, text, add_special_tokens=False):
            import re

            return [self.vocab.get(t, 5 + len(t) % 50) for t in re.findall(r"<im_\w+>|\S+", text)]

    small = MolmoImageProcessor(max_crops=4, overlap_margins=(2, 2), base_image_input_size=(56, 56), image_token_length_w=2,
                                image_token_length_h=2, image_patch_size=14)
    mp = MolmoProcessor(Tok(), small)
    batch = mp("what is this", images=[rng.integers(0, 255, (60, 100, 3), dtype=np.uint8)])
    cfg = MolmoConfig(vocab_size=90, embedding_size=96, hidden_size=32, intermediate_size=96, num_hidden_layers=1, num_attention_heads=2,
                      additional_vocab_size=8, max_position_embeddings=256,
                      vision_backbone=dict(image_default_input_size=(56, 56), image_patch_size=14, image_emb_dim=16, image_num_heads=2,
                                           image_num_key_value_heads=2, image_num_layers=2, image_head_dim=8, image_mlp_dim=24,
                                           image_num_pos=17), vit_layers=(-1, -2))
    torch.manual_seed(0)
    model = MolmoForCausalLM(cfg, dtype=torch.float32).eval()
    ids = batch["input_ids"]
    assert ids[0, 0] == 0 and ids[0, 1] == 91
    with torch.no_grad():
        with_img = model(**batch).logits
        without = model(ids).logits
    touched = (with_img - without).abs().amax(-1)[0] > 0
    first = int(batch["image_input_idx"][batch["image_input_idx"] >= 0].min())
    assert not touched[:first].any() and touched[first]                                   # causal: nothing before the first feature row moves
    assert set(batch["image_input_idx"][batch["image_input_idx"] >= 0].tolist()) == set(torch.nonzero(ids[0] == 93)[:, 0].tolist())


def test_qwen3_omni_processor_expands_and_interleaves_like_hugging_face():
    """Audio-encoder row counts, longest-padding mel features with their frame mask, and the expanded prompt (plain tags, and a
    clip's audio rows merged into its video rows by time stamp) against ``transformers``; the whole call on a toy tokenizer."""
    import types

    import numpy as np
    from transformers import WhisperFeatureExtractor as HFExtractor
    from transformers.models.qwen3_omni_moe import processing_qwen3_omni_moe as hf

    from paddleformers_b200.transformers.audio_processing import LogMelFeatureExtractor
    from paddleformers_b200.transformers.omni_processing import Qwen3OmniProcessor, audio_encoder_output_lengths, interleave_by_time

    rng = np.random.default_rng(0)
    clips = [rng.standard_normal(16000 * 3 + 77).astype(np.float32), rng.standard_normal(9000).astype(np.float32)]
    want = HFExtractor(feature_size=128)(clips, sampling_rate=16000, padding=True, truncation=False, return_attention_mask=True,
                                         return_tensors="pt")
    got = LogMelFeatureExtractor(feature_size=128)(clips, sampling_rate=16000, padding="longest", truncation=False,
                                                   return_attention_mask=True)
    assert (want["input_features"] - got["input_features"]).abs().max() < 1e-5
    assert want["attention_mask"].tolist() == got["attention_mask"].tolist()
    n = np.arange(1, 3000)
    assert (hf._get_feat_extract_output_lengths(torch.tensor(n)).numpy() == audio_encoder_output_lengths(n)).all()
    assert interleave_by_time(np.array([0.0, 0.0, 2.5]), 4) == [True, True, False, False, False, True, False]

    tok = _Tok()
    tok.encode = lambda text, add_special_tokens=False: [tok.vocab.setdefault(w, len(tok.vocab)) for w in
                                                         text.replace("<|", " <|").replace("|>", "|> ").split()]
    proc = Qwen3OmniProcessor(tok)
    stand_in = types.SimpleNamespace(image_processor=proc.image_processor, video_processor=proc.video_processor,
                                     **{k: getattr(proc, k) for k in ("audio_token", "image_token", "video_token", "vision_bos_token",
                                                                      "vision_eos_token", "audio_bos_token", "audio_eos_token")})
    text = ("a <|audio_pad|> b <|vision_start|><|image_pad|><|vision_end|> c <|vision_start|><|video_pad|><|vision_end|> "
            "d <|audio_pad|>")
    for in_video, lengths in ((False, [7, 3]), (True, [7, 41, 3])):
        ref = hf.Qwen3OmniMoeProcessor.replace_multimodal_special_tokens(
            stand_in, [text], iter(torch.tensor(lengths)), iter([torch.tensor([1, 4, 6])]), iter([torch.tensor([3, 4, 4])]),
            iter([2.0]), in_video, 13.0, 2.0)[0]
        assert proc.expand_tags(text, lengths, [[1, 4, 6]], [[3, 4, 4]], [2.0], in_video) == ref
    with pytest.raises(ValueError):
        proc.expand_tags(text, [7], [[1, 4, 6]], [[3, 4, 4]], [2.0])                    # a tag without an input
    with pytest.raises(ValueError):
        proc.expand_tags("a <|audio_pad|>", [7, 3], [], [], [])                           # an input without a tag

    image = rng.integers(0, 255, (90, 120, 3), dtype=np.uint8)
    video = rng.integers(0, 255, (4, 64, 64, 3), dtype=np.uint8)
    out = proc([text, "e <|audio_pad|>"], images=[image], videos=[video], audio=[clips[0], clips[1], clips[1]], sampling_rate=16000)
    ids = out["input_ids"]
    count = lambda tag: int((ids == tok.vocab[tag]).sum())
    rows = audio_encoder_output_lengths(out["feature_attention_mask"].sum(-1).numpy())
    assert count("<|audio_pad|>") == int(rows.sum())
    assert count("<|image_pad|>") == int(out["image_grid_thw"].prod(-1).sum()) // 4 == out["pixel_values"].shape[0] // 4
    assert count("<|video_pad|>") == int(out["video_grid_thw"].prod(-1).sum()) // 4
    assert out["video_second_per_grid"].tolist() == [2.0]
    assert ids.shape == out["attention_mask"].shape and out["attention_mask"][1, 0] == 0 and out["attention_mask"][0].all()


def test_tool_declarations_render_as_the_typescript_like_text():
    """Stored text for a tool list that exercises every schema form: constraints, defaults, enums with null, arrays with and
    without item comments, nested objects with additional properties, anyOf, type unions, ``$defs`` references and a
    reference to the root."""
    import json
    import os

    from paddleformers_b200.transformers.tool_declaration import function_to_typescript, sort_keys_deep, tools_to_typescript

    with open(os.path.join(os.path.dirname(__file__), "fixtures", "tool_declaration_golden.json")) as f:
        golden = json.load(f)
    assert tools_to_typescript(golden["tools"]) == golden["text"]
    assert tools_to_typescript([]) == "" and tools_to_typescript([{"type": "_plugin"}]) == ""
    assert function_to_typescript({"name": "f", "parameters": {"type": "object", "properties": {"a": True, "b": False}}}) == \
        "type f = (_: {\n  a?: any,\n  b?: null\n}) => any;"
    with pytest.raises(ValueError):
        function_to_typescript({"name": "f", "parameters": {"type": "object", "properties": {"a": {"enum": [1], "type": "string"}}}})
    with pytest.raises(ValueError):
        function_to_typescript({"name": "f", "parameters": {"type": "object", "properties": {"a": {"$ref": "#/$defs/Nope"}}}})
    assert list(sort_keys_deep({"b": [{"d": 1, "c": 2}], "a": 0})) == ["a", "b"]


def test_kimi_processor_round_trip(tmp_path):
    """Native-resolution geometry (the reference's own expectation for a 400 x 30 image), patch order, video chunking with
    time-stamped prompts, the tiktoken tokenizer on a small rank file (special tokens in the text, save / load), the chat
    template with the tool block, and the joined processor through ``AutoProcessor``."""
    import base64

    import numpy as np

    from paddleformers_b200.transformers.auto import AutoProcessor
    from paddleformers_b200.transformers.kimi_processing import (KimiProcessor, KimiVisionProcessor, TikTokenTokenizer,
                                                                 native_resolution_geometry, timestamp_text)

    assert native_resolution_geometry(400, 30, 14, 2, 16384, 512) == {
        "num_tokens": 30, "new_width": 400, "new_height": 30, "pad_width": 20, "pad_height": 26, "sampled_nframes": 1}
    g = native_resolution_geometry(4000, 3000, 14, 2, 1024, 512)                 # shrunk to the patch budget
    assert (g["new_width"] // 14) * (g["new_height"] // 14) <= 1024 and g["new_width"] * 3 // 4 in (g["new_height"], g["new_height"] + 1)
    assert native_resolution_geometry(20000, 100, 14, 2, 16384, 64)["new_width"] == 64 * 14       # side limit
    assert timestamp_text(3723.25) == "01:02:03.250" and timestamp_text(75.5, "mm:ss") == "01:15"

    vp = KimiVisionProcessor()
    rng = np.random.default_rng(0)
    img = rng.integers(0, 255, (30, 400, 3), dtype=np.uint8)
    out = vp([{"type": "image", "image": img}])
    assert out["pixel_values"].shape == (120, 3, 14, 14) and out["grid_thws"].tolist() == [[1, 4, 30]]
    # no resize for this size: patch (row 1, column 2) is that block of the normalised image; the padding normalises to -1
    want = torch.from_numpy(img[14:28, 28:42]).permute(2, 0, 1).float() / 255.0 * 2 - 1
    assert torch.allclose(out["pixel_values"][30 + 2], want, atol=1e-6)
    assert (out["pixel_values"][3 * 30] == -1).all()

    video = rng.integers(0, 255, (40, 56, 84, 3), dtype=np.uint8)
    chunks = vp.split_video_chunks(video, fps=10.0)                          # 4 s at 2 frames / s -> 8 frames -> 2 chunks
    assert [c["video_chunk"].shape[0] for c in chunks] == [4, 4]
    assert chunks[1]["prompt"].startswith("00:00:02.200<|media_begin|>video") and vp.media_tokens(chunks[0]) == 2 * 3

    toks = [bytes([i]) for i in range(256)] + [b"he", b"ll", b"hell", b"hello", b" w", b"or", b" wor"]
    with open(tmp_path / "tiktoken.model", "wb") as f:
        f.write(b"\n".join(base64.b64encode(t) + b" " + str(i).encode() for i, t in enumerate(toks)))
    n = len(toks)
    template = ("{% if tools_ts_str %}{{ tools_ts_str }}{% endif %}{% for m in messages %}<|im_user|>{% for p in m['content'] %}"
                "{% if p['type'] == 'text' %}{{ p['text'] }}{% elif p['type'] == 'image' %}<|media_pad|>{% else %}"
                "<|kimi_k25_video_placeholder|>{% endif %}{% endfor %}<|im_end|>{% endfor %}")
    tok = TikTokenTokenizer(str(tmp_path / "tiktoken.model"), {n: "[BOS]", n + 1: "[EOS]", n + 2: "<|im_end|>", n + 3: "<|media_pad|>",
                                                              n + 4: "<|im_user|>"}, pad_token="[EOS]", chat_template=template)
    ids = tok.encode("hello world<|im_end|>")
    assert ids == [259, 262, ord("l"), ord("d"), n + 2] and tok.decode(ids) == "hello world<|im_end|>"
    assert tok.decode(ids, skip_special_tokens=True) == "hello world" and tok.vocab_size == n + 256
    assert tok.encode("<|im_end|>", allow_special_tokens=False) != [n + 2]
    assert tok.special_tokens[f"<|reserved_token_{n + 200}|>"] == n + 200
    assert list(TikTokenTokenizer._bounded_runs("a" * 7 + "  b", 3)) == ["aaa", "aaa", "a  b"]      # no run longer than 3
    tools = [{"type": "function", "function": {"name": "now", "description": "Current time"}}]
    text = tok.apply_chat_template([{"role": "user", "content": [{"type": "text", "text": "hello"}]}], tools=tools)
    assert text.startswith("# Tools\n\n## functions\nnamespace functions {\n// Current time\ntype now = (_: {}) => any;\n}\n<|im_user|>hello")

    KimiProcessor(vp, tok).save_pretrained(str(tmp_path))
    proc = AutoProcessor.from_pretrained(str(tmp_path))
    assert isinstance(proc, KimiProcessor) and proc.tokenizer.get_vocab() == tok.get_vocab()
    out = proc(messages=[{"role": "user", "content": [{"type": "image", "image_url": img},
                                                      {"type": "video", "video_url": video, "fps": 10.0}, {"type": "text", "text": "hello"}]}])
    assert list(out) == proc.model_input_names and out["grid_thws"].tolist() == [[1, 4, 30], [4, 4, 6], [4, 4, 6]]
    assert out["pixel_values"].shape[0] == 120 + 2 * 96 and int((out["input_ids"] == n + 3).sum()) == 3          # one pad per item
    assert "00:00:02.200<|media_begin|>" in proc.decode(out["input_ids"][0])
    again = proc(text="<|media_pad|>hello", medias=[{"type": "image", "image": img}])
    assert again["pixel_values"].shape[0] == 120
    with pytest.raises(ValueError):
        proc(text="hello")
    with pytest.raises(ValueError):
        proc()
