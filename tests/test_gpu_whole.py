"""Each request alone and whole, against the plain implementation."""
import numpy as np
import pytest

from helpers import TINY, TOL, assert_rows_close, make_model_folder, plain_logits, random_tokens, rel_err, tolerance

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole_sequence_matches_plain(tmp_path, name, dtype):
    from longbow_quarrel_b200.engine import Engine
    folder = make_model_folder(tmp_path, name, seed=3)
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=512)
    vocab = TINY[name]["vocab_size"]
    for n, seed in ((1, 1), (7, 2), (100, 3)) + (((300, 4),) if name in "DE" else ()):
        tokens = random_tokens(n, vocab, seed)
        slot = eng.new_sequence()
        got = eng.step([(slot, tokens)], want=[list(range(n))]).cpu().numpy()
        eng.end_sequence(slot)
        ref = plain_logits(folder, tokens)
        assert_rows_close(got, ref, tolerance(dtype, folder, tokens), (name, dtype, n))
    assert eng.cache.pages_in_use() == 0


UNUSUAL = {
    # a width that is no multiple of 8: the bfloat16 products take the plain kernel
    "width 100": dict(hidden_size=100, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
                      intermediate_size=150, vocab_size=333, rms_norm_eps=1e-6),
    # a head size between the templates of the tensor-core attention kernels
    "head 96": dict(hidden_size=192, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=96,
                    intermediate_size=344, vocab_size=1001),
    # heads * head_dim != hidden and a head of 8, below every tensor-core tile
    "head 8": dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=8,
                   intermediate_size=88, vocab_size=200),
    # an even head size that is no multiple of 8: rotation pairs that no 16-byte access covers
    "head 26": dict(hidden_size=104, num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=1, head_dim=26,
                    intermediate_size=120, vocab_size=300, tie_word_embeddings=True),
    # three heads to a kv head (as the 3B shape has): the tensor-core prompt attention takes one head per block,
    # where an even group shares a block between two heads
    "group of 3, head 128": dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=1,
                                 head_dim=128, intermediate_size=352, vocab_size=640),
    "group of 3, head 64": dict(hidden_size=192, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2,
                                head_dim=64, intermediate_size=264, vocab_size=512, sliding_window=100),
    # a head size above 128: the plain attention kernel
    "head 160": dict(hidden_size=320, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, head_dim=160,
                     intermediate_size=520, vocab_size=777, tie_word_embeddings=True),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", sorted(UNUSUAL))
def test_sizes_that_the_fast_kernels_do_not_take(tmp_path, case, dtype):
    """Whole and with the last tokens one by one: every size the configuration allows gives the right
    result, through whichever kernel takes it (also sizes that take another variant of a fast kernel)."""
    from longbow_quarrel_b200.engine import Engine
    overrides = {"max_position_embeddings": 512, **UNUSUAL[case]}
    folder = make_model_folder(tmp_path, "A", seed=4, overrides=overrides)
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=512)
    tokens = random_tokens(150, UNUSUAL[case]["vocab_size"], 5)
    ref = plain_logits(folder, tokens)
    slot = eng.new_sequence()
    whole = eng.step([(slot, tokens)], want=[list(range(150))]).cpu().numpy()
    eng.end_sequence(slot)
    slot = eng.new_sequence()
    eng.step([(slot, tokens[:118])], want=[[]])
    tail = np.stack([eng.step([(slot, [t])]).cpu().numpy()[0] for t in tokens[118:]])
    eng.end_sequence(slot)
    tol = tolerance(dtype, folder, tokens)
    assert_rows_close(whole, ref, tol, (case, dtype, "whole"))
    assert_rows_close(tail, ref[118:], tol, (case, dtype, "one by one"))


def test_weights_stored_in_32_bit_stay_32_bit(tmp_path):
    """A checkpoint stored in float32 is read as float32: the 32-bit path then agrees with the
    plain implementation on weights that bfloat16 could not hold."""
    import torch
    from longbow_quarrel_b200.engine import Engine
    folder = make_model_folder(tmp_path, "A", seed=4, dtype=torch.float32)
    eng = Engine.from_pretrained(folder, dtype="float32", max_tokens=256)
    assert eng.model.embedding.table.dtype == torch.float32
    assert eng.model.blocks[0].mixer.w_qkv.tensor.dtype == torch.float32
    tokens = random_tokens(50, 256, 8)
    slot = eng.new_sequence()
    got = eng.step([(slot, tokens)], want=[list(range(50))]).cpu().numpy()
    assert rel_err(got, plain_logits(folder, tokens)) < TOL["float32"]
    # the bfloat16 engine takes the same folder: 32-bit weights go through the plain product, and it says so
    from longbow_quarrel_b200.kernels import ops
    with pytest.warns(UserWarning, match="stored in 32-bit.*convert_weights"):
        eng16 = Engine.from_pretrained(folder, dtype="bfloat16", max_tokens=256)
    assert eng16.model.blocks[0].mixer.w_qkv.tensor.dtype == torch.float32
    slot = eng16.new_sequence()
    before = ops.launches_by_name()
    got = eng16.step([(slot, tokens)], want=[list(range(50))]).cpu().numpy()
    assert rel_err(got, plain_logits(folder, tokens)) < TOL["bfloat16"]
    assert "gemm_tc" not in ops.launches_since(before) and ops.launches_since(before)["linear"] > 0
    # asked to, the loader rounds the matrices to bfloat16 (norm gains stay in 32-bit): the tensor-core kernels run
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        conv = Engine.from_pretrained(folder, dtype="bfloat16", max_tokens=256, convert_weights=True)
    assert conv.model.blocks[0].mixer.w_qkv.tensor.dtype == torch.bfloat16
    assert conv.model.blocks[0].norm1.gain.dtype == torch.float32
    slot = conv.new_sequence()
    before = ops.launches_by_name()
    got = conv.step([(slot, tokens)], want=[list(range(50))]).cpu().numpy()
    assert rel_err(got, plain_logits(folder, tokens)) < TOL["bfloat16"]
    assert ops.launches_since(before).get("gemm_tc", 0) > 0 and "linear" not in ops.launches_since(before)


def test_step_errors_are_raised_before_anything_runs(tmp_path):
    from longbow_quarrel_b200.cache import CacheError
    from longbow_quarrel_b200.engine import Engine, StepError
    folder = make_model_folder(tmp_path, "A", seed=5)
    eng = Engine.from_pretrained(folder, dtype="float32", max_tokens=128)
    slot = eng.new_sequence()
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([(slot, [1, 256])])
    with pytest.raises(StepError, match="no tokens"):
        eng.step([(slot, [])])
    with pytest.raises(StepError, match="twice"):
        eng.step([(slot, [1]), (slot, [2])])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([(slot, [1, 2])], want=[[2]])
    with pytest.raises(CacheError, match="context limit|cache is full"):
        eng.step([(slot, [1] * 129)])
    assert eng.cache.length(slot) == 0
    eng.step([(slot, [1, 2, 3])])
    assert eng.cache.length(slot) == 3
