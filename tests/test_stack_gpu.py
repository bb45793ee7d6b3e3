"""Layer-stack models (Matulorn design) on the GPU against the plain numpy restatement in tests/stack_oracle.py: every
mixer alone, whole prompts against token-by-token decoding, portions down to two tokens, contexts that are cleared and used
again, window edges and far keys with sharpened attention, the soft-max sink, long decoding through the replayed graph,
odd sizes (vector and scalar load paths, grouped key heads, one norm group, partial rotation, no YaRN), bfloat16, and greedy
generation through the bridge's job loop. Small random models written to a temporary folder; float32 is the sharp
comparison."""
import copy
import ctypes as C
import os

import numpy as np
import pytest

import stack_oracle as so
from booster_b200 import _lib, engine

pytestmark = pytest.mark.gpu

TOL32 = 2e-4


def err(got, want):
    """root mean square of the difference with its mean taken off, over the root mean square of the expected row; worst row"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float((np.sqrt((d * d).mean(-1)) / (np.sqrt((w * w).mean(-1)) + 1e-30)).max())


def mingru(width=40, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def latent(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, window=7, scaling=True, dims=None, mlp=None, scale=0.3):
    rot = {"base": 10000.0, "dims": dims if dims is not None else rot_dim}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "fast": 32.0, "slow": 1.0, "original": 16}
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if window:
        mx["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def delta(heads=4, kv_heads=2, dim=8, vdim=6, conv=3, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def ff(n=56, limit=1.5):
    return {"ff": n, "kind": "dense", "limit": limit}


def config(layers, width=48, vocab=61, groups=3, eps=1e-5):
    return {"architecture": "Matulorn", "layers": layers, "norm": {"eps": eps, "groups": groups}, "vocab": vocab, "width": width}


class Pair:
    """the same random model in the framework and in the oracle"""

    def __init__(self, tmp_path, cfg, seed=0, dtype="float32", n_ctx=512, edit=None):
        self.cfg = cfg
        self.w = so.random_model(cfg, seed)
        if edit:
            edit(self.w)
        d = so.write_model(str(tmp_path / f"m{seed}_{dtype}_{abs(hash(str(cfg))) % 10**8}"), cfg, self.w)
        self.oracle = so.Oracle(cfg, {k: np.asarray(v, np.float64) for k, v in self.w.items()})
        self.model = engine.Model(d, dtype=dtype)
        self.ctx = engine.Context(self.model, n_ctx)
        self.dir = d

    def close(self):
        self.ctx.close()
        self.model.close()

    def tokens(self, n, seed=1):
        return np.random.default_rng(seed).integers(0, self.cfg["vocab"], size=n).tolist()

    def expected(self, toks):
        self.oracle.reset()
        return self.oracle.forward(toks)

    def run(self, toks, cuts=None, ctx=None):
        """logits of every position, the token stream cut into steps of the given sizes (None: one step)"""
        ctx = ctx or self.ctx
        ctx.kv_clear()
        out, pos = [], 0
        cuts = list(cuts) if cuts else [len(toks)]
        i = 0
        while pos < len(toks):
            n = min(cuts[i % len(cuts)], len(toks) - pos)
            out.append(ctx.decode_rows(toks[pos:pos + n], pos, list(range(n))))
            pos += n
            i += 1
        return np.concatenate(out)


@pytest.mark.parametrize("layer", [mingru(), mingru(mlp=ff()), latent(), latent(window=0, mlp=ff()), delta(), delta(heads=3, kv_heads=3, dim=5, vdim=7, conv=4)],
                         ids=["mingru", "mingru+ff", "latent", "latent-unmasked+ff", "delta-grouped", "delta-odd"])
def test_each_mixer_alone_with_layer_taps(tmp_path, layer):
    p = Pair(tmp_path, config([layer]))
    toks = p.tokens(23)
    p.oracle.reset()
    lay = []
    want = p.oracle.forward(toks, lay)
    p.ctx.set_taps(True)
    got = p.ctx.decode_rows(toks, 0, list(range(len(toks))))
    taps = p.ctx.layer_taps(len(toks))
    p.ctx.set_taps(False)
    assert np.abs(taps[0] - lay[0]).max() < 1e-4 * max(1.0, np.abs(lay[0]).max())
    assert err(got, want) < TOL32
    p.close()


FULL = [mingru(), latent(mlp=ff()), delta(), mingru(width=24, mlp=ff(40, 0.75)), latent(heads=2, dim=12, rot_dim=8, vdim=4, kv_rank=16, window=5, dims=4),
        delta(heads=2, kv_heads=1, dim=16, vdim=8, conv=2, mlp=ff(32, 2.0))]


def test_whole_prompt_token_by_token_and_portions_agree(tmp_path):
    p = Pair(tmp_path, config(FULL))
    toks = p.tokens(75)
    want = p.expected(toks)
    whole = p.run(toks)
    assert err(whole, want) < TOL32
    single = p.run(toks, [1])                         # every token through the replayed one-token graph
    assert err(single, want) < TOL32
    for cuts in ([2], [3, 2, 7, 1, 5], [37, 2, 2, 30], [6, 1, 1, 11]):
        assert err(p.run(toks, cuts), want) < TOL32, cuts
    assert err(single, whole) < TOL32
    p.close()


def test_only_wanted_rows_are_returned_in_order(tmp_path):
    p = Pair(tmp_path, config(FULL[:3]))
    toks = p.tokens(19)
    want = p.expected(toks)
    p.ctx.kv_clear()
    a = p.ctx.decode_rows(toks[:11], 0, [0, 4, 10])
    b = p.ctx.decode_rows(toks[11:], 11, [])
    c = p.ctx.decode(toks[:1], 19)                    # b200_decode: the last row
    assert a.shape == (3, p.cfg["vocab"]) and b.shape[0] == 0 and c.shape == (p.cfg["vocab"],)
    assert err(a, want[[0, 4, 10]]) < TOL32
    with pytest.raises(_lib.B200Error):               # recurrent state cannot rewind: a step must continue the sequence
        p.ctx.decode_rows(toks[:2], 3, [0])
    with pytest.raises(_lib.B200Error):
        p.ctx.decode_rows([p.cfg["vocab"]], 20, [0])
    p.close()


def test_cleared_context_is_as_good_as_new(tmp_path):
    p = Pair(tmp_path, config(FULL))
    a, b = p.tokens(40, seed=3), p.tokens(29, seed=4)
    fresh = engine.Context(p.model, 512)
    ref_b = p.run(b, [5, 1, 1, 9], ctx=fresh)
    p.run(a, [7, 1])                                  # fills cache rows, recurrent state and convolution history
    again = p.run(b, [5, 1, 1, 9])                    # run() clears first: the same context, used again
    assert np.array_equal(again, ref_b)
    assert err(again, p.expected(b)) < TOL32
    # several contexts of one model do not disturb each other
    p.ctx.kv_clear(); fresh.kv_clear()
    x1 = p.ctx.decode_rows(a[:9], 0, [8]); y1 = fresh.decode_rows(b[:9], 0, [8])
    x2 = p.ctx.decode_rows(a[9:10], 9, [0]); y2 = fresh.decode_rows(b[9:10], 9, [0])
    assert err(np.concatenate([x1, x2]), p.expected(a[:10])[[8, 9]]) < TOL32
    assert err(np.concatenate([y1, y2]), p.expected(b[:10])[[8, 9]]) < TOL32
    fresh.close()
    p.close()


def sharpen(w):
    """make the soft-max peaky, so that one key more or less in the window moves the logits visibly"""
    for k in list(w):
        if k.endswith("mix.q"):
            w[k] = so.round_bf16(w[k] * 6.0)


@pytest.mark.parametrize("window", [1, 2, 9, 33])
def test_window_edges_in_prompts_and_in_decoding(tmp_path, window):
    cfg = config([latent(window=window, heads=2, kv_rank=12), mingru(width=16)], width=32, groups=2)
    p = Pair(tmp_path, cfg, seed=window, edit=sharpen)
    toks = p.tokens(3 * window + 20, seed=window)
    want = p.expected(toks)
    # the oracle itself tells windows apart by far more than the tolerance: a window one token off would show
    for off in (-1, 1):
        c2 = copy.deepcopy(cfg)
        if window + off >= 1:
            c2["layers"][0]["mixer"]["mask"]["size"] = window + off
            o2 = so.Oracle(c2, p.oracle.w)
            assert err(o2.forward(toks)[window + 1:], want[window + 1:]) > 50 * TOL32
    assert err(p.run(toks), want) < TOL32
    assert err(p.run(toks, [window + 1, 1]), want) < TOL32            # the window passes over decoded tokens
    assert err(p.run(toks, [max(window - 1, 1), 2, 1]), want) < TOL32 # portions that start and end inside a window
    p.close()


def test_far_keys_and_first_tokens_without_a_mask(tmp_path):
    cfg = config([latent(window=0, heads=2, kv_rank=12, scale=1.0), delta(heads=2, kv_heads=2, dim=8, vdim=8, conv=4)], width=32, groups=4)
    p = Pair(tmp_path, cfg, seed=5, edit=sharpen, n_ctx=400)
    toks = p.tokens(330, seed=9)
    want = p.expected(toks)
    got = p.run(toks, [300, 1])
    assert err(got, want) < TOL32
    assert err(got[:4], want[:4]) < TOL32             # the first tokens of a sequence: empty history, zero state
    assert err(p.run(toks[:40], [1]), want[:40]) < TOL32
    p.close()


def test_sink_counts_once_in_the_denominator(tmp_path):
    cfg = config([latent(window=6)])

    def big_sink(w):
        w["l0.mix.sink"] = so.round_bf16(np.array([2.5, -1.0, 0.75], np.float32))
    p = Pair(tmp_path, cfg, seed=7, edit=big_sink)
    toks = p.tokens(20)
    want = p.expected(toks)
    no_sink = dict(p.oracle.w); no_sink["l0.mix.sink"] = np.full(3, -1e30)
    assert err(so.Oracle(cfg, no_sink).forward(toks), want) > 50 * TOL32
    assert err(p.run(toks, [9, 1]), want) < TOL32
    p.close()


def test_long_decoding_through_the_graph(tmp_path):
    p = Pair(tmp_path, config(FULL[:3] + [delta(heads=2, kv_heads=2, dim=40, vdim=33, conv=3)]))
    toks = p.tokens(260, seed=11)
    want = p.expected(toks)
    got = p.run(toks, [4, 1])
    assert err(got, want) < 2 * TOL32
    assert err(got[-1:], want[-1:]) < 2 * TOL32
    p.close()


@pytest.mark.parametrize("width,groups,vocab", [(36, 1, 50), (40, 5, 77), (64, 8, 130)], ids=["scalar-loads", "five-groups", "vector-loads"])
def test_other_sizes(tmp_path, width, groups, vocab):
    layers = [delta(heads=6, kv_heads=2, dim=9, vdim=5, conv=1, mlp=ff(20, 0.5)), latent(heads=1, dim=6, rot_dim=6, vdim=3, kv_rank=9, window=4, scaling=False, dims=2),
              mingru(width=7), latent(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=32, window=50, dims=8), delta(heads=1, kv_heads=1, dim=64, vdim=40, conv=5)]
    p = Pair(tmp_path, config(layers, width=width, vocab=vocab, groups=groups, eps=1e-6), seed=width)
    toks = p.tokens(70, seed=width)
    want = p.expected(toks)
    assert err(p.run(toks), want) < TOL32
    assert err(p.run(toks, [13, 2, 1]), want) < TOL32
    p.close()


def random_config(rng):
    """a random arrangement of the three mixers with random sizes: nothing may rest on one model's values"""
    pick = lambda values: int(rng.choice(values))
    groups = pick([1, 2, 3, 4, 5, 8])
    layers = []
    for _ in range(pick([2, 3, 4, 5])):
        mlp = ff(pick([24, 64, 100, 136]), float(rng.choice([0.5, 1.0, 7.0]))) if rng.random() < 0.5 else None
        kind = pick([0, 1, 2])
        if kind == 0:
            layers.append(mingru(pick([8, 24, 56, 130]), mlp))
        elif kind == 1:
            rot_dim = pick([2, 4, 8, 16, 32])
            L = latent(heads=pick([1, 2, 3, 5, 6, 12]), dim=pick([4, 8, 24, 64]), rot_dim=rot_dim, vdim=pick([4, 16, 40, 64]), kv_rank=pick([8, 24, 64, 96, 192]),
                       window=pick([0, 1, 3, 17, 64, 100, 300]), scaling=bool(rng.random() < 0.7), dims=rot_dim if rng.random() < 0.6 else pick([d for d in (2, 4, 8, 16) if d <= rot_dim]),
                       mlp=mlp, scale=float(rng.choice([0.1, 0.2, 0.35])))
            if "scaling" in L["mixer"]["rot"]:
                L["mixer"]["rot"]["scaling"] = {"factor": float(rng.choice([2.0, 8.0, 40.0])), "fast": float(rng.choice([32.0, 16.0])), "slow": float(rng.choice([1.0, 2.0])),
                                                "original": pick([16, 64, 4096])}
                L["mixer"]["rot"]["base"] = float(rng.choice([10000.0, 500000.0]))
            layers.append(L)
        else:
            kv = pick([1, 2, 3])
            layers.append(delta(heads=kv * pick([1, 2, 4]), kv_heads=kv, dim=pick([4, 16, 32, 128]), vdim=pick([4, 8, 48, 128]), conv=pick([1, 2, 3, 5]), mlp=mlp))
    return config(layers, width=groups * pick([8, 12, 24, 40, 72]), vocab=pick([37, 100, 257, 513]), groups=groups, eps=float(rng.choice([1e-6, 1e-5])))


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(tmp_path, seed):
    rng = np.random.default_rng(500 + seed)
    cfg = random_config(rng)
    n = int(rng.choice([70, 150, 330]))
    p = Pair(tmp_path, cfg, seed=seed, n_ctx=n + 4)
    toks = p.tokens(n, seed=seed)
    want = p.expected(toks)
    assert err(p.run(toks), want) < 2 * TOL32, cfg
    assert err(p.run(toks, [n - 20] + [1] * 20), want) < 2 * TOL32, cfg
    assert err(p.run(toks, [2, 67, 3, 129, 1, 5]), want) < 2 * TOL32, cfg
    p.close()


def test_large_heads_and_ranks(tmp_path):
    """more heads than one attention block takes, a latent wider than one sweep of the weighted sum, a row that is no whole number
    of 16-byte chunks, and a delta-rule key size that takes the widest recurrence kernel"""
    layers = [latent(heads=20, dim=16, rot_dim=32, vdim=24, kv_rank=640, window=70), latent(heads=7, dim=20, rot_dim=6, vdim=10, kv_rank=37, window=129, dims=6),
              delta(heads=2, kv_heads=1, dim=192, vdim=80, conv=2)]
    p = Pair(tmp_path, config(layers, width=128, vocab=90, groups=2), seed=2, n_ctx=208)
    toks = p.tokens(200, seed=8)
    want = p.expected(toks)
    assert err(p.run(toks), want) < TOL32
    assert err(p.run(toks, [170] + [1] * 30), want) < TOL32
    assert err(p.run(toks, [2, 67, 3]), want) < TOL32
    p.close()


def test_a_step_longer_than_one_pass(tmp_path):
    """a 700-token step runs as two passes of the layers: the window, the convolution's inputs and the recurrent state cross the pass's edge"""
    layers = [latent(heads=3, dim=8, rot_dim=4, vdim=8, kv_rank=16, window=40), delta(heads=2, kv_heads=1, dim=8, vdim=8, conv=4), mingru(24, ff(40)),
              latent(heads=2, dim=8, rot_dim=8, vdim=4, kv_rank=24, window=0)]
    p = Pair(tmp_path, config(layers), n_ctx=704)
    toks = p.tokens(700, seed=5)
    want = p.expected(toks)
    assert err(p.run(toks), want) < 2 * TOL32
    assert err(p.run(toks, [509, 2, 3, 186]), want) < 2 * TOL32
    p.close()


def row_errs(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / (np.sqrt((w * w).mean(-1)) + 1e-30)


def test_bfloat16_prompt_kernels_and_decode(tmp_path):
    cfg = config(FULL, width=64, groups=4, vocab=96)
    p = Pair(tmp_path, cfg, dtype="bfloat16")
    toks = p.tokens(150, seed=2)
    want = p.expected(toks)
    # token by token: mat-vec kernels with float32 activations on the stored bfloat16 weights — nothing is rounded that the
    # oracle does not round, so this path is as sharp as float32
    assert err(p.run(toks[:60], [1]), want[:60]) < TOL32
    assert err(p.run(toks[:60], [3, 4, 2]), want[:60]) < TOL32         # portions of up to 4 tokens take the same kernels
    # longer portions: tensor-core products round the activation operand to bfloat16 (2^-9 relative per product input)
    for cuts in (None, [140, 1], [5, 17, 33]):
        e = row_errs(p.run(toks, cuts), want)
        assert np.median(e) < 3e-2 and e.max() < 0.25, (cuts, float(np.median(e)), float(e.max()))
    p.close()


def test_greedy_generation_through_the_bridge(tmp_path, monkeypatch):
    """initContext / doInference on a folder model: decimal-id prompt, standard chain at temperature 0 (arg-max on the device),
    prompt through the prompt kernels, generation through the one-token graph — the ids the oracle generates greedily"""
    monkeypatch.setenv("BOOSTER_B200_DTYPE", "float32")
    p = Pair(tmp_path, config(FULL[:4]))
    prompt, n_gen = p.tokens(21, seed=6), 10
    p.oracle.reset()
    lg = p.oracle.forward(prompt)[-1]
    ids = []
    for _ in range(n_gen):
        ids.append(int(np.argmax(lg)))
        srt = np.sort(lg)
        assert srt[-1] - srt[-2] > 1e-3               # no near-tie: float32 must pick the same id
        lg = p.oracle.forward([ids[-1]])[-1]
    L = _lib.lib()
    L.init(b"", b"")
    ctx = L.initContext(5, p.dir.encode(), 1, 0, 100, 0, 0, 0, 64, n_gen, 0, 0.0, 0.0, 0.0, 1, 1.0, 1.0, 1.0, 0, 0, 200, 1.0, 1.0, 1.0, 42, b"")
    assert ctx, _lib.last_error()
    n = L.doInference(5, ctx, b"stack-job", b"", " ".join(map(str, prompt)).encode())
    out = [int(x) for x in L.status(b"stack-job").decode().split()]
    assert out[:len(prompt)] == prompt and out[len(prompt):] == ids
    assert n == len(prompt) + n_gen - 1 and L.getPromptTokenCount(b"stack-job") == len(prompt)
    # the device-resident loop of the token-level interface gives the same ids
    p.ctx.kv_clear()
    first = int(np.argmax(p.ctx.decode(prompt, 0)))
    dev = p.ctx.generate_greedy(first, len(prompt), n_gen - 1).tolist()
    assert [first] + dev == ids
    # the burst left cache, state and position where a host-driven step continues them
    after = p.ctx.decode([ids[-1]], len(prompt) + n_gen - 1)
    assert err(after[None], lg[None]) < TOL32
    assert p.ctx.L.b200_kernel_launches(p.ctx.h) > 0
    p.close()


def test_bad_models_fail_loudly(tmp_path):
    cfg = config([mingru()])
    w = so.random_model(cfg)
    d = so.write_model(str(tmp_path / "ok"), cfg, w)
    bad = dict(cfg); bad["architecture"] = "Nonesuch"
    with pytest.raises(_lib.B200Error, match="unsupported architecture"):
        engine.Model(so.write_model(str(tmp_path / "arch"), bad, w))
    w2 = dict(w); del w2["l0.mix.o"]
    with pytest.raises(_lib.B200Error, match="missing tensor"):
        engine.Model(so.write_model(str(tmp_path / "missing"), cfg, w2))
    w3 = dict(w); w3["l0.mix.z.b"] = w["l0.mix.z.b"][:-1]
    with pytest.raises(_lib.B200Error, match="shape"):
        engine.Model(so.write_model(str(tmp_path / "shape"), cfg, w3))
    c3 = copy.deepcopy(cfg); c3["layers"][0]["type"] = "lstm"
    with pytest.raises(_lib.B200Error, match="unknown mixer"):
        engine.Model(so.write_model(str(tmp_path / "mixer"), c3, w))
    with pytest.raises(_lib.B200Error, match="dtype"):
        engine.Model(d, dtype="float16")
    m = engine.Model(d)                               # bfloat16 by default
    assert m.n_vocab == cfg["vocab"] and m.n_embd == cfg["width"] and m.n_layer == 1
    c = engine.Context(m, 16)
    with pytest.raises(_lib.B200Error, match="exceeds the context"):
        c.decode_rows([1] * 17, 0, [16])
    with pytest.raises(_lib.B200Error, match="not available"):
        c.kv_seq_rm(0, 1)
    c.close(); m.close()


@pytest.mark.parametrize("dtype,T,N,K,glu", [
    ("bfloat16", 1, 70, 48, False), ("bfloat16", 4, 66, 36, True),            # mat-vec: vector and scalar loads
    ("bfloat16", 37, 100, 64, False), ("bfloat16", 21, 64, 40, True),         # mma.sync
    ("bfloat16", 200, 300, 136, False), ("bfloat16", 130, 512, 64, True),     # tcgen05 + TMEM: ragged and whole tiles
    ("bfloat16", 513, 258, 1032, False),                                      # more K steps than pipeline stages, several token tiles
    ("bfloat16", 70, 130, 35, False),                                         # odd K: CUDA cores
    ("float32", 50, 70, 33, True), ("float32", 3, 9, 7, False)], ids=str)
def test_products_pick_their_kernel_and_agree_with_numpy(dtype, T, N, K, glu):
    rng = np.random.default_rng(T * 1000 + N)
    x = rng.standard_normal((T, K)).astype(np.float32)
    w = so.round_bf16(rng.standard_normal((N, K)).astype(np.float32) / np.sqrt(K))
    b = so.round_bf16(rng.standard_normal(N).astype(np.float32))
    limit = 0.8
    y = np.zeros((T, N // 2 if glu else N), np.float32)
    f32p = C.POINTER(C.c_float)
    L = _lib.lib()
    rc = L.b200_stack_linear(0, 0 if dtype == "bfloat16" else 1, T, N, K, x.ctypes.data_as(f32p), w.ctypes.data_as(f32p), b.ctypes.data_as(f32p),
                             int(glu), limit, y.ctypes.data_as(f32p))
    assert rc == 0, _lib.last_error()
    # the tensor-core paths round the activations to bfloat16; everything else keeps them in float32
    tensor = dtype == "bfloat16" and T > 4 and K % 8 == 0
    xe = so.round_bf16(x) if tensor else x
    ref = xe.astype(np.float64) @ w.astype(np.float64).T + b
    if glu:
        g, u = np.minimum(ref[:, 0::2], limit), np.clip(ref[:, 1::2], -limit, limit)
        ref = g * so.sigmoid(1.702 * g) * (u + 1.0)
    assert np.abs(y - ref).max() < 2e-5 * max(1.0, np.abs(ref).max()) * np.sqrt(K)
