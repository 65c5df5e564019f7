"""The generation loop's decisions, with a scripted backend in place of the GPU."""
import pytest

import longbow_quarrel_b200  # noqa: F401
from longbow_quarrel_b200.engine.generate import generate


class Scripted:
    """Each sequence's next token is a function of its history; slots are counted."""

    def __init__(self, rule, n_slots=3):
        self.rule, self.free, self.live = rule, list(range(n_slots)), {}
        self.calls, self.max_live = [], 0

    def start(self):
        h = self.free.pop(0)
        self.live[h] = []
        self.max_live = max(self.max_live, len(self.live))
        return h

    def finish(self, h):
        assert h in self.live, "a sequence was ended twice"
        del self.live[h]
        self.free.append(h)

    def run(self, entries, requests, steps, histories):
        self.calls.append(([len(t) for _, t in entries], list(requests), list(steps)))
        out = []
        for (h, toks), hist in zip(entries, histories):
            assert h in self.live
            self.live[h] += toks
            assert self.live[h] == hist, "the history must be the prompt followed by the generated tokens"
            out.append(self.rule(self.live[h]))
        return out


def test_unequal_prompts_stop_tokens_and_early_finishers():
    rule = lambda h: 99 if len(h) >= 6 else len(h)        # noqa: E731   stop once a sequence has 6 tokens
    be = Scripted(rule)
    prompts = [[1, 2, 3, 4, 5], [7], [1, 2, 3]]
    out, stats = generate(be, prompts, max_new_tokens=10, stop_ids=[99], batch_size=3)
    assert out == [[5], [1, 2, 3, 4, 5], [3, 4, 5]]
    assert stats.finish_reasons == ["stop", "stop", "stop"]
    # one prefill step with unequal lengths, then only the live sequences go on
    assert be.calls[0] == ([5, 1, 3], [0, 1, 2], [0, 0, 0])
    assert be.calls[1] == ([1, 1, 1], [0, 1, 2], [1, 1, 1])
    assert be.calls[2][1] == [1, 2] and be.calls[-1][1] == [1]
    assert be.live == {} and sorted(be.free) == [0, 1, 2]


def test_first_sampled_token_can_stop_a_sequence():
    be = Scripted(lambda h: 99)
    out, stats = generate(be, [[1, 2], [3]], 5, stop_ids=[99], batch_size=2)
    assert out == [[], []] and len(be.calls) == 1 and stats.generated_tokens == 2
    out, _ = generate(Scripted(lambda h: 99), [[1, 2]], 5, stop_ids=[99], include_stop=True, batch_size=1)
    assert out == [[99]]


def test_length_limit_counts_the_token_of_the_prefill():
    be = Scripted(lambda h: 5)
    out, stats = generate(be, [[1], [2, 3]], max_new_tokens=4, batch_size=2)
    assert out == [[5, 5, 5, 5], [5, 5, 5, 5]]
    assert len(be.calls) == 4          # P + N - 1 forward passes, as in the reference
    assert stats.finish_reasons == ["length", "length"] and stats.decode_steps == 3
    out, _ = generate(Scripted(lambda h: 5), [[1]], max_new_tokens=0)
    assert out == [[]]


def test_context_limit_ends_a_sequence():
    be = Scripted(lambda h: 5)
    out, stats = generate(be, [[1, 2, 3]], max_new_tokens=100, batch_size=1, max_context=6)
    assert out == [[5, 5, 5]] and stats.finish_reasons == ["context"]
    with pytest.raises(ValueError, match="context limit"):
        generate(be, [[1] * 7], 1, max_context=6)


def test_batches_follow_one_another_and_reuse_slots():
    be = Scripted(lambda h: 99 if len(h) >= 4 else 1, n_slots=2)
    prompts = [[1], [1, 2, 3], [4, 5], [6], [7, 8, 9]]
    out, stats = generate(be, prompts, 10, stop_ids=[99], batch_size=2)
    assert stats.batches == 3 and be.max_live == 2
    assert [len(o) for o in out] == [3, 1, 2, 3, 1]
    firsts = [c for c in be.calls if c[2][0] == 0]
    assert [c[1] for c in firsts] == [[0, 1], [2, 3], [4]]


def test_callback_and_errors():
    seen = []
    generate(Scripted(lambda h: len(h)), [[1], [1, 2]], 2, callback=lambda i, t: seen.append((i, t)), batch_size=2)
    assert seen == [(0, 1), (1, 2), (0, 2), (1, 3)]
    with pytest.raises(ValueError, match="empty"):
        generate(Scripted(lambda h: 1), [[1], []], 2)
    be = Scripted(lambda h: 1 / 0)
    with pytest.raises(ZeroDivisionError):
        generate(be, [[1]], 2)
    assert be.live == {}                 # slots go back even when a step fails
