"""The plain implementation checked against closed forms and simple restatements."""
import math

import numpy as np
import torch

import plain_llama as pl


def test_rms_norm_closed_form():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    out = pl.rms_norm(x, torch.tensor([1.0, 2.0], dtype=torch.float64), 0.0)
    rms = math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[3 / rms, 8 / rms]], dtype=torch.float64))


def test_rope_is_identity_at_position_zero_and_rotates_pairs():
    x = torch.randn(1, 2, 8, dtype=torch.float64)
    f = pl.rope_frequencies(8, 10000.0, None)
    assert torch.equal(pl.rope(x, [0], f), x)
    y = pl.rope(x, [3], f)
    for i in range(4):                    # element i pairs with i + 4
        a = 3 * f[i]
        assert math.isclose(float(y[0, 0, i]), float(x[0, 0, i]) * math.cos(a) - float(x[0, 0, i + 4]) * math.sin(a))
        assert math.isclose(float(y[0, 0, i + 4]), float(x[0, 0, i]) * math.sin(a) + float(x[0, 0, i + 4]) * math.cos(a))
    # the score of a rotated pair depends on the distance only
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    s1 = (pl.rope(q, [10], f) * pl.rope(k, [7], f)).sum()
    s2 = (pl.rope(q, [103], f) * pl.rope(k, [100], f)).sum()
    assert math.isclose(float(s1), float(s2), rel_tol=1e-9)


def test_llama3_scaling_hits_all_three_branches():
    sc = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=64)
    base = pl.rope_frequencies(32, 500000.0, None)
    f = pl.rope_frequencies(32, 500000.0, sc)
    kept = [i for i in range(16) if f[i] == base[i]]
    divided = [i for i in range(16) if math.isclose(f[i], base[i] / 8.0)]
    blended = [i for i in range(16) if i not in kept and i not in divided]
    assert kept == [0, 1] and blended == [2] and divided == list(range(3, 16))
    assert base[2] / 8.0 < f[2] < base[2]


def test_attention_with_equal_inputs_returns_the_value():
    """All keys and values equal: the output is that value at every position
    (the closed-form case of internal/device/attention_test.go:10-55)."""
    T, H, Hkv, hd = 9, 4, 2, 8
    q = torch.full((T, H, hd), 0.1, dtype=torch.float64)
    k = torch.full((T, Hkv, hd), 0.1, dtype=torch.float64)
    v = torch.full((T, Hkv, hd), 0.1, dtype=torch.float64)
    assert torch.allclose(pl.attention(q, k, v, hd ** -0.5), torch.full((T, H, hd), 0.1, dtype=torch.float64))


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    T, H, Hkv, hd = 7, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, dtype=torch.float64) for n in (H, Hkv, Hkv))
    out = pl.attention(q, k, v, 0.3)
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 9.0, 9.0                         # later keys do not reach earlier rows
    assert torch.equal(pl.attention(q, k2, v2, 0.3)[:5], out[:5])
    assert torch.equal(out[0], v[0].repeat_interleave(2, dim=0))      # first row sees only itself; heads 0,1 -> kv 0
    w = pl.attention(q, k, v, 0.3, window=3)
    row = 6
    s = (k[4:7, 1] @ q[row, 3]) * 0.3                  # head 3 reads kv head 1, keys 4..6
    assert torch.allclose(w[row, 3], torch.softmax(s, 0) @ v[4:7, 1])


def test_swiglu_and_linear():
    g, u = torch.tensor([0.0, 2.0], dtype=torch.float64), torch.tensor([3.0, 5.0], dtype=torch.float64)
    assert torch.allclose(pl.swiglu(g, u), torch.tensor([0.0, 5.0 * 2.0 / (1 + math.exp(-2.0))], dtype=torch.float64))
    x, w = torch.randn(3, 4, dtype=torch.float64), torch.randn(5, 4, dtype=torch.float64)
    assert torch.allclose(pl.linear(x, w), torch.einsum("tk,nk->tn", x, w))


def test_forward_prefix_property(tmp_path):
    """Logits at a position do not depend on later tokens."""
    from helpers import TINY, make_model_folder, random_tokens
    folder = make_model_folder(tmp_path, "C", seed=9)
    cfg, w = pl.load_folder(folder)
    toks = random_tokens(60, TINY["C"]["vocab_size"], 1)
    full = pl.forward(cfg, w, toks)
    part = pl.forward(cfg, w, toks[:45])
    assert torch.allclose(full[:45], part, atol=1e-12)
    assert pl.layer_window(cfg, 0) == 40 and pl.layer_window(cfg, 1) is None


def test_sampler_rules():
    logits = np.log(np.array([0.5, 0.2, 0.2, 0.1]))
    assert pl.sample_reference(logits, 0.0, 0, 1.0, 0.3) == 0
    kept, probs = pl.kept_set(logits, 1.0, 2, 1.0)
    assert kept == [0, 1]                         # ties at the cut-off go to the lower index
    kept, probs = pl.kept_set(logits, 1.0, 0, 0.75)
    assert kept == [0, 1, 2] and math.isclose(sum(probs), 1.0)
    assert pl.sample_reference(logits, 1.0, 0, 1.0, 0.69) == 1
    assert pl.sample_reference(logits, 1.0, 0, 1.0, 0.95) == 3
    pen = pl.repetition_penalty([2.0, -2.0, 1.0], [0, 1, 0], 2.0)
    assert list(pen) == [1.0, -4.0, 1.0]
