"""Generation: cache vs. no-cache consistency, beams, logits processors, stopping criteria, streamers."""
import torch

from paddleformers_b200.generation.logits_process import (EosTokenCriteria, ForcedEOSTokenLogitsProcessor, LogitsProcessorList,
                                                           MaxLengthCriteria, MinLengthLogitsProcessor,
                                                           NoRepeatNGramLogitsProcessor, RepetitionPenaltyLogitsProcessor,
                                                           StoppingCriteriaList, StopSequenceCriteria,
                                                           SuppressTokensLogitsProcessor, TextIteratorStreamer, TopKLogitsWarper,
                                                           TopPLogitsWarper)
from paddleformers_b200.generation.utils import GenerationConfig, generate
from paddleformers_b200.models.configuration import named_config
from paddleformers_b200.transformers.auto import AutoModelForCausalLM


def _model():
    torch.manual_seed(0)
    cfg = named_config("tiny-llama", vocab_size=64, hidden_size=32, intermediate_size=64, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=16)
    return AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).eval()


def test_greedy_matches_full_recompute_and_beams_run():
    m = _model()
    ids = torch.randint(0, 64, (2, 5))
    out = generate(m, ids, GenerationConfig(max_new_tokens=6))
    assert out.shape == (2, 11)
    # greedy decoding with the cache equals argmax of a full forward over the generated prefix
    full = m(out[:, :-1], return_logits=True).logits
    assert torch.equal(full[:, 4:].argmax(-1), out[:, 5:])
    beams = generate(m, ids, GenerationConfig(max_new_tokens=4, num_beams=3))
    assert beams.shape[0] == 2 and beams.shape[1] <= 9


def test_processors():
    ids = torch.tensor([[1, 2, 3, 1, 2]])
    scores = torch.zeros(1, 8)
    assert NoRepeatNGramLogitsProcessor(3)(ids, scores)[0, 3] == float("-inf")          # "1 2 3" would repeat
    assert NoRepeatNGramLogitsProcessor(3)(ids, scores)[0, 4] == 0
    assert MinLengthLogitsProcessor(10, 7)(ids, scores)[0, 7] == float("-inf")
    assert MinLengthLogitsProcessor(3, 7)(ids, scores)[0, 7] == 0
    s = torch.tensor([[2.0, -2.0, 0.5, 0, 0, 0, 0, 0]])
    r = RepetitionPenaltyLogitsProcessor(2.0)(torch.tensor([[0, 1]]), s)
    assert r[0, 0] == 1.0 and r[0, 1] == -4.0 and r[0, 2] == 0.5
    assert (TopKLogitsWarper(2)(ids, torch.arange(8.0)[None]) > float("-inf")).sum() == 2
    p = TopPLogitsWarper(0.5)(ids, torch.log(torch.tensor([[0.6, 0.3, 0.05, 0.05]])))
    assert (p > float("-inf")).sum() == 1
    f = ForcedEOSTokenLogitsProcessor(6, 7)(ids, scores)
    assert f[0, 7] == 0 and f[0, 0] == float("-inf")
    assert SuppressTokensLogitsProcessor([1, 2])(ids, scores)[0, 1] == float("-inf")
    crit = StoppingCriteriaList([MaxLengthCriteria(5), EosTokenCriteria(9), StopSequenceCriteria([[1, 2]])])
    assert bool(crit(ids)[0]) and not bool(StoppingCriteriaList([StopSequenceCriteria([[3, 2]])])(ids)[0])


def test_generate_with_processors_criteria_and_streamer():
    m = _model()
    ids = torch.randint(0, 64, (1, 4))
    banned = list(range(0, 32))
    out = generate(m, ids, GenerationConfig(max_new_tokens=8), logits_processor=LogitsProcessorList([SuppressTokensLogitsProcessor(banned)]),
                   stopping_criteria=StoppingCriteriaList([MaxLengthCriteria(8)]))
    assert out.shape[1] == 8 and (out[0, 4:] >= 32).all()

    class Tok:
        def decode(self, ids, **kw):
            return " ".join(str(i) for i in ids) + " "

    st = TextIteratorStreamer(Tok())
    generate(m, ids, GenerationConfig(max_new_tokens=3), streamer=st)
    text = "".join(st)
    assert len(text.split()) == 3


def _seq_logprob(m, seq, L0):
    lp = torch.log_softmax(m(seq[:, :-1], return_logits=True).logits.float(), -1)
    return lp[:, L0 - 1:].gather(-1, seq[:, L0:, None]).squeeze(-1).sum(-1)


def test_beam_search_beats_greedy_and_groups_diversify():
    import pytest

    m = _model()
    ids = torch.randint(0, 64, (2, 5))
    n = 5
    greedy = generate(m, ids, GenerationConfig(max_new_tokens=n))
    beams = generate(m, ids, GenerationConfig(max_new_tokens=n, num_beams=4, length_penalty=0.0))
    assert beams.shape == greedy.shape
    assert (_seq_logprob(m, beams, 5) >= _seq_logprob(m, greedy, 5) - 1e-5).all()
    # several hypotheses per input, best first
    many = generate(m, ids, GenerationConfig(max_new_tokens=n, num_beams=4, num_return_sequences=3, length_penalty=0.0))
    assert many.shape == (6, 10) and torch.equal(many[0], beams[0]) and torch.equal(many[3], beams[1])
    lp = _seq_logprob(m, many, 5).view(2, 3)
    assert (lp[:, :-1] >= lp[:, 1:] - 1e-5).all()
    # diverse beam search: a large penalty forces every group onto its own first token
    div = generate(m, ids, GenerationConfig(max_new_tokens=n, num_beams=4, num_beam_groups=4, diversity_penalty=100.0,
                                            num_return_sequences=4, length_penalty=0.0))
    first = div[:, 5].view(2, 4)
    assert all(len(set(row.tolist())) == 4 for row in first)
    # plain beams of the same width share first tokens more often than not on a peaked model; at the least they are legal
    with pytest.raises(ValueError):
        generate(m, ids, GenerationConfig(max_new_tokens=2, num_beams=4, num_beam_groups=3, diversity_penalty=1.0))
    with pytest.raises(ValueError):
        generate(m, ids, GenerationConfig(max_new_tokens=2, num_beams=4, num_beam_groups=2))
