"""Each request alone and whole, against the plain implementation."""
import numpy as np
import pytest

from helpers import TINY, TOL, make_model_folder, plain_logits, random_tokens, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_sequence_matches_plain(tmp_path, name, dtype):
    from longbow_quarrel_b200.engine import Engine
    folder = make_model_folder(tmp_path, name, seed=3)
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=512)
    vocab = TINY[name]["vocab_size"]
    for n, seed in ((1, 1), (7, 2), (100, 3)):
        tokens = random_tokens(n, vocab, seed)
        slot = eng.new_sequence()
        got = eng.step([(slot, tokens)], want=[list(range(n))]).cpu().numpy()
        eng.end_sequence(slot)
        ref = plain_logits(folder, tokens)
        assert rel_err(got, ref) < TOL[dtype], (name, dtype, n)
    assert eng.cache.pages_in_use() == 0
