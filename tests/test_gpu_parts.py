"""Each part alone against the plain implementation's function for it, and a toy
mixer with state of its own that is registered from here."""
import numpy as np
import pytest
import torch

import plain_llama as pl
from helpers import TOL, rel_err

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _runtime(dtype, max_context=256):
    from longbow_quarrel_b200.parts.base import Runtime
    return Runtime(DEV, dtype, max_context)


def _ctx(entries, past, part=None):
    from longbow_quarrel_b200.engine.step import make_context, pack_step
    flat, info = pack_step(entries, None, past, part.step_needs() if part is not None else None)
    return make_context(torch.from_numpy(flat).to(DEV), info, [s for s, _ in entries])


def _rand(shape, seed, std=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from longbow_quarrel_b200.parts.norm import RMSNorm
    part = RMSNorm(_runtime(dtype), size=88, eps=3e-4, name="g")
    assert part.weights()["g"].shape == (88,)
    gain = 1 + 0.1 * _rand((88,), 1)
    part.load({"g": gain.to(torch.bfloat16).to(DEV)})          # gains stored in bfloat16 are read as such
    x = _rand((5, 88), 2, 2.0)
    ref = pl.rms_norm(x.double(), gain.to(torch.bfloat16).double(), 3e-4)
    out = part.forward(x.to(DEV))
    assert out.dtype == dtype
    assert rel_err(out.float().cpu().numpy(), ref.numpy()) < (1e-6 if dtype == torch.float32 else 2e-2)


def test_rope_part_tables():
    from longbow_quarrel_b200.config import RopeScaling
    from longbow_quarrel_b200.parts.rope import Rope, rope_frequencies
    sc = RopeScaling("llama3", 8.0, 1.0, 4.0, 64)
    f = rope_frequencies(32, 500000.0, sc).numpy()
    ref = pl.rope_frequencies(32, 500000.0, dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                                 high_freq_factor=4.0, original_max_position_embeddings=64))
    assert np.allclose(f, ref, rtol=1e-14)
    part = Rope(_runtime(torch.float32, 200), head_dim=32, theta=500000.0, scaling=sc)
    cos, sin = part.tables()
    assert cos.shape == (200, 16) and cos.dtype == torch.float32
    ang = np.arange(200)[:, None] * ref[None]
    assert np.abs(cos.cpu().numpy() - np.cos(ang)).max() < 1e-7 and np.abs(sin.cpu().numpy() - np.sin(ang)).max() < 1e-7
    assert Rope(part.runtime, 32, 500000.0, sc).tables()[0] is cos        # equal parts share one table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part(dtype, window):
    """Two sequences of unequal length in one step, then one more token each."""
    from longbow_quarrel_b200.cache import Cache
    from longbow_quarrel_b200.parts.attention import Attention
    from longbow_quarrel_b200.parts.spec import PartSpec
    D, H, Hkv, hd = 72, 6, 2, 16
    rt = _runtime(dtype)
    part = Attention(rt, hidden_size=D, n_heads=H, n_kv_heads=Hkv, head_dim=hd, scale=0.31, window=window,
                     position=PartSpec("rope", {"head_dim": hd, "theta": 10000.0, "scaling": None}))
    w = {n: _rand(s.shape, i, 0.15, torch.bfloat16) for i, (n, s) in enumerate(part.weights().items())}
    part.load({n: t.to(DEV) for n, t in w.items()})
    cache = Cache({0: part.cache_need()}, 1024, 256, dtype, DEV)
    lens = [37, 70]
    xs = [_rand((n + 1, D), 10 + i, 1.0, torch.bfloat16).float() for i, n in enumerate(lens)]

    def plain(x):
        T = x.shape[0]
        x = x.double()
        q = pl.linear(x, w["q_proj.weight"].double()).reshape(T, H, hd)
        k = pl.linear(x, w["k_proj.weight"].double()).reshape(T, Hkv, hd)
        v = pl.linear(x, w["v_proj.weight"].double()).reshape(T, Hkv, hd)
        f = pl.rope_frequencies(hd, 10000.0, None)
        a = pl.attention(pl.rope(q, np.arange(T), f), pl.rope(k, np.arange(T), f), v, 0.31, window)
        return pl.linear(a.reshape(T, H * hd), w["o_proj.weight"].double())

    refs = [plain(x) for x in xs]
    slots = [cache.alloc_slot() for _ in lens]
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    # the prompts together
    for s, n in zip(slots, lens):
        cache.reserve(s, n)
    cache.upload()
    ctx = _ctx([(s, [0] * n) for s, n in zip(slots, lens)], [0, 0], part)
    h = torch.cat([x[:n] for x, n in zip(xs, lens)]).to(dtype).to(DEV)
    resid = torch.zeros((sum(lens), D), dtype=torch.float32, device=DEV)
    part.forward(h, ctx, cache.view(0), resid)
    for s, n in zip(slots, lens):
        cache.commit(s, n)
    got = resid.cpu().numpy()
    assert rel_err(got[:lens[0]], refs[0][:lens[0]].numpy()) < tol
    assert rel_err(got[lens[0]:], refs[1][:lens[1]].numpy()) < tol
    # one more token each, added onto a residual that is not zero
    for s in slots:
        cache.reserve(s, 1)
    cache.upload()
    ctx = _ctx([(s, [0]) for s in slots], lens, part)
    h = torch.stack([x[n] for x, n in zip(xs, lens)]).to(dtype).to(DEV)
    resid = torch.ones((2, D), dtype=torch.float32, device=DEV)
    part.forward(h, ctx, cache.view(0), resid)
    got = resid.cpu().numpy() - 1.0
    for i in range(2):
        assert rel_err(got[i], refs[i][lens[i]].numpy()) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,F", [(3, 176), (70, 44)])
def test_feed_forward_part(dtype, T, F):
    from longbow_quarrel_b200.parts.mlp import GatedMLP
    D = 56
    part = GatedMLP(_runtime(dtype), hidden_size=D, intermediate_size=F)
    w = {n: _rand(s.shape, i, 0.2, torch.bfloat16) for i, (n, s) in enumerate(part.weights().items())}
    part.load({n: t.to(DEV) for n, t in w.items()})
    x = _rand((T, D), 7, 1.0, torch.bfloat16).float()
    ref = pl.linear(pl.swiglu(pl.linear(x.double(), w["gate_proj.weight"].double()),
                              pl.linear(x.double(), w["up_proj.weight"].double())), w["down_proj.weight"].double())
    resid = torch.full((T, D), 2.0, dtype=torch.float32, device=DEV)
    part.forward(x.to(dtype).to(DEV), None, resid)
    assert rel_err(resid.cpu().numpy() - 2.0, ref.numpy()) < (2e-5 if dtype == torch.float32 else 3e-2)


def test_embedding_and_head_parts():
    from longbow_quarrel_b200.parts.embedding import LinearHead, TokenEmbedding
    rt = _runtime(torch.float32)
    emb = TokenEmbedding(rt, vocab_size=50, hidden_size=24, name="E")
    table = _rand((50, 24), 1, 1.0, torch.bfloat16)
    emb.load({"E": table.to(DEV)})
    toks = torch.tensor([3, 49, 0], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(toks).cpu(), table[[3, 49, 0]].float())
    tied = LinearHead(rt, vocab_size=50, hidden_size=24, name="H", tied_to="E", tied=True)
    assert tied.weights() == {}
    tied.load({"E": table.to(DEV)})
    h = _rand((4, 24), 2)
    assert rel_err(tied.forward(h.to(DEV)).cpu().numpy(), (h.double() @ table.double().T).numpy()) < 1e-5
    own = LinearHead(rt, vocab_size=50, hidden_size=24, name="H", tied_to="E")
    assert own.weights()["H"].fallback == "E"


# ------------------------------------------------------------------ a toy mixer with state of its own
def test_a_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """A mixer that keeps a running sum of its inputs per sequence (fixed-size state, no
    keys or values) is defined here, registered, put into a two-layer model beside an
    attention layer, and stepped in every way of cutting -- no framework file changes."""
    from dataclasses import dataclass

    from longbow_quarrel_b200.config import register_architecture
    from longbow_quarrel_b200.engine import Engine
    from longbow_quarrel_b200.parts import (LayerSpec, Mixer, ModelSpec, PartSpec, ScheduleEntry, StateNeed,
                                            register_part)
    from longbow_quarrel_b200.weights import WeightSpec

    @register_part("mixer", "toy_running_sum")
    class RunningSum(Mixer):
        """out_t = (state + sum of inputs up to t) * mix / (position + 1); state carries over."""

        def __init__(self, runtime, hidden_size):
            self.runtime, self.D, self.mix = runtime, hidden_size, None

        def weights(self):
            return {"mix": WeightSpec((self.D,), init="gain")}

        def load(self, tensors):
            self.mix = tensors["mix"].float()

        def cache_need(self):
            return StateNeed((self.D,), torch.float32)

        def forward(self, h, ctx, state, residual, writes_cache=True):
            h = h.float()
            row = 0
            for b, n in enumerate(ctx.h_new):
                slot = ctx.h_slots[b]
                run = state[slot] + torch.cumsum(h[row:row + n], dim=0)
                pos = torch.arange(ctx.h_past[b], ctx.h_past[b] + n, device=h.device, dtype=torch.float32)
                residual[row:row + n] += run * self.mix / (pos[:, None] + 1.0)
                state[slot] = run[-1]
                row += n

    @dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int
        vocab_size: int
        architectures: tuple = ("ToyStateLM",)

    def describe(cfg):
        norm = lambda name: PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": 1e-5, "name": name})  # noqa: E731
        ffn = PartSpec("gated_mlp", {"hidden_size": cfg.hidden_size, "intermediate_size": 48})
        attn = PartSpec("attention", {"hidden_size": cfg.hidden_size, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16,
                                      "scale": 0.25, "position": PartSpec("rope", {"head_dim": 16, "theta": 1e4})})
        layer = lambda prefix, mixer: LayerSpec(prefix, dict(mixer=mixer, ffn=ffn, norm1=norm("n1"), norm2=norm("n2")))  # noqa: E731
        layers = (layer("l0.", PartSpec("toy_running_sum", {"hidden_size": cfg.hidden_size})), layer("l1.", attn))
        return ModelSpec(name="ToyStateLM", hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
                         embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size,
                                                                "hidden_size": cfg.hidden_size, "name": "emb"}),
                         layers=layers, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1)),
                         final_norm=norm("fn"),
                         head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                                       "name": "head", "tied_to": "emb", "tied": True}),
                         max_positions=256)

    register_architecture("ToyStateLM", lambda d: ToyConfig(d["hidden_size"], d["vocab_size"]), describe)
    eng = Engine.from_config({"architectures": ["ToyStateLM"], "hidden_size": 32, "vocab_size": 100}, seed=3,
                             dtype="float32", max_tokens=1024, gain_std=0.1)
    assert len(eng.cache.state_groups) == 1 and len(eng.cache.kv_groups) == 1
    assert not eng.model.graph_safe and not eng.stepper.use_graphs     # the toy reads host lists
    toks = [[5, 9, 33, 2, 71, 8, 40], [11, 3, 6]]
    s = [eng.new_sequence() for _ in toks]
    whole = eng.step([(s[0], toks[0]), (s[1], toks[1])], want=[list(range(7)), list(range(3))]).cpu().numpy()
    for slot in s:
        eng.end_sequence(slot)
    # the same tokens cut differently, in slots that are used again: state must start from zero and carry over
    s = [eng.new_sequence() for _ in toks]
    first = eng.step([(s[0], toks[0][:4]), (s[1], toks[1][:1])], want=[[0, 1, 2, 3], [0]]).cpu().numpy()
    rest = [eng.step([(s[0], [toks[0][4 + i]])] + ([(s[1], [toks[1][1 + i]])] if i < 2 else [])).cpu().numpy()
            for i in range(3)]
    assert np.allclose(first[:4], whole[:4], atol=1e-5) and np.allclose(first[4], whole[7], atol=1e-5)
    for i in range(3):
        assert np.allclose(rest[i][0], whole[4 + i], atol=1e-5)
        if i < 2:
            assert np.allclose(rest[i][1], whole[8 + i], atol=1e-5)
    assert not np.allclose(whole[1], whole[0])


# ------------------------------------------------------------------ other kinds of parts, defined here
def test_a_routed_feed_forward_and_a_learned_position_encoding_from_a_test():
    """A feed-forward that routes each token to one of three small experts (router in 32-bit) and a
    position encoding with a tensor of its own that shifts q and k in place (no cos/sin tables, so the
    attention takes its unfused path) are defined here, registered and put into a model whose two
    layers differ; whole prompts, token-by-token decoding and a batch agree with each other and with
    the same computation spelled out with the plain functions."""
    from dataclasses import dataclass

    from longbow_quarrel_b200.config import register_architecture
    from longbow_quarrel_b200.engine import Engine
    from longbow_quarrel_b200.parts import (FeedForward, LayerSpec, ModelSpec, PartSpec, PositionEncoding,
                                            ScheduleEntry, register_part)
    from longbow_quarrel_b200.weights import WeightSpec

    D, H, Hkv, hd, F, V, E, P = 48, 3, 1, 16, 40, 90, 3, 64

    @register_part("ffn", "toy_routed")
    class Routed(FeedForward):
        """y = gate-free expert e(x) = relu(x We1^T) We2^T for the one expert with the largest router logit."""

        def __init__(self, runtime, hidden_size, inner, experts):
            self.runtime, self.D, self.F, self.E = runtime, hidden_size, inner, experts

        def weights(self):
            out = {"router": WeightSpec((self.E, self.D))}
            for e in range(self.E):
                out[f"e{e}.w1"] = WeightSpec((self.F, self.D))
                out[f"e{e}.w2"] = WeightSpec((self.D, self.F))
            return out

        def load(self, tensors):
            self.t = {k: v.float() for k, v in tensors.items()}

        def forward(self, h, ctx, residual):
            x = h.float()
            choice = (x @ self.t["router"].T).argmax(dim=-1)
            for e in range(self.E):
                rows = (choice == e).nonzero().squeeze(1)
                if rows.numel():
                    y = torch.relu(x[rows] @ self.t[f"e{e}.w1"].T) @ self.t[f"e{e}.w2"].T
                    residual.index_add_(0, rows, y)

    @register_part("position", "toy_learned_shift")
    class LearnedShift(PositionEncoding):
        """q and k of position p get table[p] added (one vector per position, shared by the heads)."""

        def __init__(self, runtime, head_dim, positions):
            self.runtime, self.hd, self.P, self.table = runtime, head_dim, positions, None

        def weights(self):
            return {"pos_table": WeightSpec((self.P, self.hd))}

        def load(self, tensors):
            self.table = tensors["pos_table"]

        def apply(self, q, k, positions):
            shift = self.table[positions.long()].to(q.dtype).unsqueeze(1)
            q += shift
            if k is not None:
                k += shift

    @dataclass(frozen=True)
    class Cfg:
        architectures: tuple = ("ToyRoutedLM",)

    def describe(cfg):
        norm = lambda name: PartSpec("rms_norm", {"size": D, "eps": 1e-5, "name": name})  # noqa: E731
        attn = lambda position: PartSpec("attention", {"hidden_size": D, "n_heads": H, "n_kv_heads": Hkv,  # noqa: E731
                                                       "head_dim": hd, "scale": hd ** -0.5, "position": position})
        layers = (LayerSpec("l0.", dict(mixer=attn(PartSpec("toy_learned_shift", {"head_dim": hd, "positions": P})),
                                        ffn=PartSpec("toy_routed", {"hidden_size": D, "inner": F, "experts": E}),
                                        norm1=norm("n1"), norm2=norm("n2"))),
                  LayerSpec("l1.", dict(mixer=attn(PartSpec("rope", {"head_dim": hd, "theta": 1e4})),
                                        ffn=PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": 64}),
                                        norm1=norm("n1"), norm2=norm("n2"))))
        return ModelSpec(name="ToyRoutedLM", hidden_size=D, vocab_size=V,
                         embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": D, "name": "emb"}),
                         layers=layers, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1)), final_norm=norm("fn"),
                         head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": D, "name": "head",
                                                       "tied_to": "emb", "tied": True}),
                         max_positions=P)

    register_architecture("ToyRoutedLM", lambda d: Cfg(), describe)
    eng = Engine.from_config({"architectures": ["ToyRoutedLM"]}, seed=9, dtype="float32", max_tokens=512, gain_std=0.1)
    table = eng.model.weight_table()
    assert "l0.pos_table" in table and "l0.router" in table and "l0.e2.w2" in table and "l1.gate_proj.weight" in table
    toks = [[int(t) for t in np.random.default_rng(i).integers(0, V, n)] for i, n in enumerate((23, 9))]

    # the same computation with the plain functions
    b0, b1 = eng.model.blocks
    dd = lambda t: t.double().cpu()  # noqa: E731
    emb = dd(eng.model.embedding.table)

    def plain(tokens):
        T = len(tokens)
        pos = np.arange(T)
        x = emb[tokens]
        for blk in (b0, b1):
            m = blk.mixer
            w = dd(m.w_qkv.tensor)
            n = pl.rms_norm(x, dd(blk.norm1.gain), 1e-5)
            q = pl.linear(n, w[:H * hd]).reshape(T, H, hd)
            k = pl.linear(n, w[H * hd:(H + Hkv) * hd]).reshape(T, Hkv, hd)
            v = pl.linear(n, w[(H + Hkv) * hd:]).reshape(T, Hkv, hd)
            if blk is b0:
                shift = dd(m.position.table)[pos][:, None, :]
                q, k = q + shift, k + shift
            else:
                f = pl.rope_frequencies(hd, 1e4, None)
                q, k = pl.rope(q, pos, f), pl.rope(k, pos, f)
            x = x + pl.linear(pl.attention(q, k, v, hd ** -0.5, None).reshape(T, H * hd), dd(m.w_o.tensor))
            n = pl.rms_norm(x, dd(blk.norm2.gain), 1e-5)
            if blk is b0:
                t = {kk: dd(vv) for kk, vv in blk.ffn.t.items()}
                choice = (n @ t["router"].T).argmax(-1)
                y = torch.zeros_like(x)
                for r in range(T):
                    e = int(choice[r])
                    y[r] = torch.relu(n[r] @ t[f"e{e}.w1"].T) @ t[f"e{e}.w2"].T
                x = x + y
                assert len(set(choice.tolist())) > 1          # the router does route
            else:
                gu = dd(blk.ffn.w_gu.tensor)
                Fi = gu.shape[0] // 2
                x = x + pl.linear(pl.swiglu(pl.linear(n, gu[:Fi]), pl.linear(n, gu[Fi:])), dd(blk.ffn.w_down.tensor))
        return pl.linear(pl.rms_norm(x, dd(eng.model.final_norm.gain), 1e-5), emb).numpy()

    want = [plain(t) for t in toks]
    s = [eng.new_sequence() for _ in toks]
    whole = eng.step([(s[0], toks[0]), (s[1], toks[1])], want=[list(range(23)), list(range(9))]).cpu().numpy()
    assert rel_err(whole[:23], want[0]) < 1e-4 and rel_err(whole[23:], want[1]) < 1e-4
    for slot in s:
        eng.end_sequence(slot)
    # prompts cut short, the rest token by token, the shorter request ending earlier
    s = [eng.new_sequence() for _ in toks]
    eng.step([(s[0], toks[0][:15]), (s[1], toks[1][:4])], want=[[], []])
    for i in range(8):
        entries = [(s[0], [toks[0][15 + i]])] + ([(s[1], [toks[1][4 + i]])] if i < 5 else [])
        out = eng.step(entries).cpu().numpy()
        assert rel_err(out[0], want[0][15 + i]) < 1e-4
        if i < 5:
            assert rel_err(out[1], want[1][4 + i]) < 1e-4


# ------------------------------------------------------------------ the order of layers is data
def test_a_layer_run_twice_and_a_layer_that_reads_anothers_cache():
    """Schedule: layer 0 (cache entry 0), layer 1 reading entry 0 without keys and values of its
    own, then layer 0 once more (cache entry 1).  Compared with the same computation spelled out
    with the plain functions, whole and token by token."""
    from dataclasses import dataclass

    from longbow_quarrel_b200.config import register_architecture
    from longbow_quarrel_b200.engine import Engine
    from longbow_quarrel_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    D, H, Hkv, hd, F, V = 64, 4, 2, 16, 96, 120

    @dataclass(frozen=True)
    class Cfg:
        architectures: tuple = ("ToyScheduleLM",)

    def describe(cfg):
        norm = lambda name: PartSpec("rms_norm", {"size": D, "eps": 1e-5, "name": name})  # noqa: E731
        rope = PartSpec("rope", {"head_dim": hd, "theta": 1e4})
        attn = lambda own: PartSpec("attention", {"hidden_size": D, "n_heads": H, "n_kv_heads": Hkv, "head_dim": hd,  # noqa: E731
                                                  "scale": hd ** -0.5, "position": rope, "own_kv": own})
        ffn = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": F})
        layers = (LayerSpec("a.", dict(mixer=attn(True), ffn=ffn, norm1=norm("n1"), norm2=norm("n2"))),
                  LayerSpec("b.", dict(mixer=attn(False), ffn=ffn, norm1=norm("n1"), norm2=norm("n2"))))
        return ModelSpec(name="ToyScheduleLM", hidden_size=D, vocab_size=V,
                         embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": D, "name": "emb"}),
                         layers=layers,
                         schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 0, writes_cache=False), ScheduleEntry(0, 1)),
                         final_norm=norm("fn"),
                         head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": D, "name": "head",
                                                       "tied_to": "emb", "tied": True}),
                         max_positions=256)

    register_architecture("ToyScheduleLM", lambda d: Cfg(), describe)
    tokens = [int(t) for t in np.random.default_rng(3).integers(0, V, 45)]
    for dtype, tol in (("float32", 1e-4), ("bfloat16", 6e-2)):
        eng = Engine.from_config({"architectures": ["ToyScheduleLM"]}, seed=5, dtype=dtype, max_tokens=512,
                                 gain_std=0.1)
        assert "b.k_proj.weight" not in eng.model.weight_table() and "b.q_proj.weight" in eng.model.weight_table()
        assert sorted(eng.model.cache_needs()) == [0, 1]
        # the same weights for the plain computation
        W = {}
        for blk in eng.model.blocks:
            m = blk.mixer
            wq = m.w_qkv.tensor.double().cpu()
            W[blk.prefix + "q"] = wq[:H * hd]
            if m.own_kv:
                W[blk.prefix + "k"], W[blk.prefix + "v"] = wq[H * hd:(H + Hkv) * hd], wq[(H + Hkv) * hd:]
            W[blk.prefix + "o"] = m.w_o.tensor.double().cpu()
            gu = blk.ffn.w_gu.tensor.double().cpu()
            if blk.ffn.block:
                gu = gu.reshape(F // 8, 2, 8, D)
                W[blk.prefix + "g"], W[blk.prefix + "u"] = gu[:, 0].reshape(F, D), gu[:, 1].reshape(F, D)
            else:
                W[blk.prefix + "g"], W[blk.prefix + "u"] = gu[:F], gu[F:]
            W[blk.prefix + "d"] = blk.ffn.w_down.tensor.double().cpu()
            W[blk.prefix + "n1"], W[blk.prefix + "n2"] = blk.norm1.gain.double().cpu(), blk.norm2.gain.double().cpu()
        emb = eng.model.embedding.table.double().cpu()
        fn = eng.model.final_norm.gain.double().cpu()
        T = len(tokens)
        f = pl.rope_frequencies(hd, 1e4, None)
        pos = np.arange(T)

        def block(p, x, shared_kv=None):
            n = pl.rms_norm(x, W[p + "n1"], 1e-5)
            q = pl.rope(pl.linear(n, W[p + "q"]).reshape(T, H, hd), pos, f)
            if shared_kv is None:
                k = pl.rope(pl.linear(n, W[p + "k"]).reshape(T, Hkv, hd), pos, f)
                v = pl.linear(n, W[p + "v"]).reshape(T, Hkv, hd)
            else:
                k, v = shared_kv
            x = x + pl.linear(pl.attention(q, k, v, hd ** -0.5).reshape(T, H * hd), W[p + "o"])
            n = pl.rms_norm(x, W[p + "n2"], 1e-5)
            x = x + pl.linear(pl.swiglu(pl.linear(n, W[p + "g"]), pl.linear(n, W[p + "u"])), W[p + "d"])
            return x, (k, v)

        x = pl.embedding(emb, tokens)
        x, kv0 = block("a.", x)
        x, _ = block("b.", x, shared_kv=kv0)
        x, _ = block("a.", x)
        ref = pl.linear(pl.rms_norm(x, fn, 1e-5), emb).numpy()

        slot = eng.new_sequence()
        whole = eng.step([(slot, tokens)], want=[list(range(T))]).cpu().numpy()
        eng.end_sequence(slot)
        assert rel_err(whole, ref) < tol, dtype
        slot = eng.new_sequence()
        head = eng.step([(slot, tokens[:20])], want=[[19]]).cpu().numpy()
        assert rel_err(head[0], ref[19]) < tol
        for i in range(20, T):
            got = eng.step([(slot, [tokens[i]])]).cpu().numpy()[0]
            assert rel_err(got, ref[i]) < tol, (dtype, i)
        eng.end_sequence(slot)


# ------------------------------------------------------------------ storage, step integers and arrangement of a test's own
def test_a_mixer_with_storage_of_its_own_a_step_array_and_a_block_with_a_third_norm():
    """Three things that only registrations add, each defined here and none in the framework:
    a mixer whose keys and values have different widths, with a cache need and a cache group of its own
    (dense rows per slot, no pages); a per-step integer array of its own, packed by the step function and
    found in `ctx.extra`; and an arrangement with a third norm (the feed-forward's output is normed before
    it joins the residual stream).  Whole prompts, cut prompts and single tokens agree with the same
    computation in float64, in slots that are used again."""
    from dataclasses import dataclass

    from longbow_quarrel_b200.cache import CacheError, CacheGroup
    from longbow_quarrel_b200.config import register_architecture
    from longbow_quarrel_b200.engine import Engine
    from longbow_quarrel_b200.parts import (CacheNeed, LayerSpec, Mixer, ModelSpec, Part, PartSpec, ScheduleEntry,
                                            make_part, register_part)
    from longbow_quarrel_b200.weights import WeightSpec

    D, DK, DV, V, F = 40, 12, 28, 70, 56

    class DenseRows(CacheGroup):
        """keys [entry, slot, position, dk] and values [entry, slot, position, dv]: a row per position."""

        def __init__(self, entries, dk, dv, sizing):
            self.entries, self.index = list(entries), {e: i for i, e in enumerate(entries)}
            self.limit = sizing.max_context
            self.k = torch.full((len(entries), sizing.max_slots, self.limit, dk), float("nan"), device=sizing.device)
            self.v = torch.full((len(entries), sizing.max_slots, self.limit, dv), float("nan"), device=sizing.device)
            self.started, self.released = [], []

        def start(self, slot):
            self.started.append(slot)

        def reserve(self, slot, old_len, new_len):
            if new_len > self.limit:
                raise CacheError("toy rows are full")

        def release(self, slot):
            self.released.append(slot)
            self.k[:, slot] = float("nan")           # what a sequence leaves must never be read again
            self.v[:, slot] = float("nan")

        def view(self, entry):
            return self.k[self.index[entry]], self.v[self.index[entry]]

        def nbytes(self):
            return 4 * (self.k.numel() + self.v.numel())

    @dataclass(frozen=True)
    class RowsNeed(CacheNeed):
        dk: int
        dv: int

        def make_group(self, entries, sizing):
            return DenseRows(entries, self.dk, self.dv, sizing)

    @register_part("mixer", "toy_wide_values")
    class WideValues(Mixer):
        """One head; scores over keys of width dk, values of width dv; causal."""

        def __init__(self, runtime, hidden_size, dk, dv):
            self.D, self.dk, self.dv = hidden_size, dk, dv

        def weights(self):
            return {"wq": WeightSpec((self.dk, self.D)), "wk": WeightSpec((self.dk, self.D)),
                    "wv": WeightSpec((self.dv, self.D)), "wo": WeightSpec((self.D, self.dv))}

        def load(self, tensors):
            self.t = {k: v.float() for k, v in tensors.items()}

        def cache_need(self):
            return RowsNeed(self.dk, self.dv)

        def step_needs(self):
            # For every sequence of the step: its first row in the packed batch and its rows, as [2, B].
            return {"toy_row_ranges": lambda step: np.asarray([step.cu[:-1], step.new], dtype=np.int32)}

        def forward(self, h, ctx, rows, residual, writes_cache=True):
            keys, values = rows
            ranges = ctx.extra["toy_row_ranges"].view(2, -1).cpu().tolist()      # the part's own step integers
            assert ranges[1] == ctx.h_new
            x = h.float()
            for b, (first, n) in enumerate(zip(*ranges)):
                slot, past = ctx.h_slots[b], ctx.h_past[b]
                xs = x[first:first + n]
                keys[slot, past:past + n] = xs @ self.t["wk"].T
                values[slot, past:past + n] = xs @ self.t["wv"].T
                s = (xs @ self.t["wq"].T) @ keys[slot, :past + n].T / self.dk ** 0.5
                pos = torch.arange(past, past + n, device=x.device)[:, None]
                s = s.masked_fill(torch.arange(past + n, device=x.device)[None, :] > pos, float("-inf"))
                residual[first:first + n] += torch.softmax(s, dim=-1) @ values[slot, :past + n] @ self.t["wo"].T

    @register_part("block", "toy_sandwich")
    class Sandwich(Part):
        """x += mixer(norm1(x)); x += norm3(ffn(norm2(x))): the place `norm3` is this arrangement's own."""

        def __init__(self, runtime, layer):
            self.prefix = layer.prefix
            self.norm1, self.norm2, self.norm3 = (make_part("norm", layer.part(p), runtime) for p in ("norm1", "norm2", "norm3"))
            self.mixer = make_part("mixer", layer.part("mixer"), runtime)
            self.ffn = make_part("ffn", layer.part("ffn"), runtime)

        def parts(self):
            return (self.norm1, self.mixer, self.norm2, self.ffn, self.norm3)

        def weights(self):
            return {name: spec for part in self.parts() for name, spec in part.weights().items()}

        def load(self, tensors):
            for part in self.parts():
                part.load({n: tensors[n] for n in part.weights()})

        def cache_need(self):
            return self.mixer.cache_need()

        def step_needs(self):
            return self.mixer.step_needs()

        def forward(self, x, ctx, cache_view, writes_cache=True):
            self.mixer.forward(self.norm1.forward(x), ctx, cache_view, x, writes_cache)
            branch = torch.zeros_like(x)
            self.ffn.forward(self.norm2.forward(x), ctx, branch)
            x += self.norm3.forward(branch).float()

    @dataclass(frozen=True)
    class Cfg:
        architectures: tuple = ("ToySandwichLM",)

    def describe(cfg):
        norm = lambda name: PartSpec("rms_norm", {"size": D, "eps": 1e-5, "name": name})  # noqa: E731
        layers = tuple(LayerSpec(f"l{i}.", arrangement="toy_sandwich", parts=dict(
            mixer=PartSpec("toy_wide_values", {"hidden_size": D, "dk": DK, "dv": DV}),
            ffn=PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": F}),
            norm1=norm("n1"), norm2=norm("n2"), norm3=norm("n3"))) for i in range(2))
        return ModelSpec(name="ToySandwichLM", hidden_size=D, vocab_size=V,
                         embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": D, "name": "emb"}),
                         layers=layers, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1)), final_norm=norm("fn"),
                         head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": D, "name": "head",
                                                       "tied_to": "emb", "tied": True}),
                         max_positions=128)

    register_architecture("ToySandwichLM", lambda d: Cfg(), describe)
    eng = Engine.from_config({"architectures": ["ToySandwichLM"]}, seed=5, dtype="float32", max_tokens=512,
                             std=0.3, gain_std=0.1, weight_dtype=torch.float32)
    group = eng.cache.groups[0]
    assert isinstance(group, DenseRows) and group.entries == [0, 1] and eng.cache.kv_groups == []
    assert list(eng.stepper.needs) == ["toy_row_ranges"] and not eng.stepper.use_graphs

    # the same computation, whole sequences in float64
    w = {}
    for prefix, part in eng.model._named_parts():
        for owner in (part.parts() if hasattr(part, "parts") else (part,)):
            for key, value in vars(owner).items():
                if key == "t":
                    w.update({prefix + k: v.double().cpu() for k, v in value.items()})
    blocks = eng.model.blocks
    emb = eng.model.embedding.table.double().cpu()

    def rms(x, gain):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * gain.double().cpu()

    def reference(tokens):
        x = emb[torch.tensor(tokens)]
        T = len(tokens)
        for i, blk in enumerate(blocks):
            p = f"l{i}."
            n = rms(x, blk.norm1.gain)
            q, k, v = n @ w[p + "wq"].T, n @ w[p + "wk"].T, n @ w[p + "wv"].T
            s = (q @ k.T / DK ** 0.5).masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            x = x + torch.softmax(s, -1) @ v @ w[p + "wo"].T
            n = rms(x, blk.norm2.gain)
            gu = n @ blk.ffn.w_gu.tensor.double().cpu().T
            g, u = gu[:, :F], gu[:, F:]
            y = (u * (g / (1 + torch.exp(-g)))) @ blk.ffn.w_down.tensor.double().cpu().T
            x = x + rms(y, blk.norm3.gain)
        return (rms(x, eng.model.final_norm.gain) @ emb.T).numpy()

    rng = np.random.default_rng(9)
    seqs = [rng.integers(0, V, n).tolist() for n in (23, 1, 9)]
    refs = [reference(t) for t in seqs]
    for round_ in range(2):                                  # the second round runs in slots that were used before
        slots = [eng.new_sequence() for _ in seqs]
        cut = [10, 1, 4]
        got = eng.step([(s, t[:c]) for s, t, c in zip(slots, seqs, cut)], want=[list(range(c)) for c in cut]).cpu().numpy()
        row = 0
        for r, c in zip(refs, cut):
            assert rel_err(got[row:row + c], r[:c]) < TOL["float32"]
            row += c
        done = list(cut)
        # a continuation of several tokens beside single tokens, then single tokens until each sequence ends
        live = [b for b in range(3) if done[b] < len(seqs[b])]
        step_new = {0: 5, 2: 1}
        while live:
            entries = [(slots[b], seqs[b][done[b]:done[b] + step_new.get(b, 1)]) for b in live]
            got = eng.step(entries, want=[list(range(len(t))) for _, t in entries]).cpu().numpy()
            row = 0
            for b, (_, t) in zip(live, entries):
                r = refs[b][done[b]:done[b] + len(t)]
                assert rel_err(got[row:row + len(t)], r) < TOL["float32"], (round_, b, done[b])
                row += len(t)
                done[b] += len(t)
            step_new = {}
            live = [b for b in live if done[b] < len(seqs[b])]
        for s in slots:
            eng.end_sequence(s)
    assert group.started == group.released and len(group.started) == 6
    assert torch.isnan(group.k).all()                        # nothing of an ended sequence is left readable
