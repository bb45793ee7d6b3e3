"""The Dopilorn design on the GPU against the plain numpy restatement in tests/dopilorn_oracle.py: every mechanism alone
(with and without a feed-forward, with the residual stream after the layer), the repeated span with a state per pass, whole
prompts against token-by-token decoding and portions down to two tokens, contexts that are cleared and used again, several
live contexts stepping in turn, window edges and far keys with sharpened attention in prompts and in decoding, the first
tokens of a sequence, long decoding through the replayed graph, odd sizes (scalar and vector load paths, grouped and
ungrouped key heads, head sizes that differ between queries and values, one tap, many passes), bfloat16, and greedy
generation through the bridge's job loop. Small random models in a temporary folder; float32 is the sharp comparison."""
import copy

import numpy as np
import pytest

import dopilorn_oracle as do
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


def ff(n=56):
    return {"ff": n, "kind": "dense"}


def gdelta(heads=3, dim=8, mlp=None, decay_rank=5):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": decay_rank}, "mlp": mlp}


def attn(heads=4, kv_heads=2, dim=6, vdim=10, conv=3, window=7, diff=0.4, scale=0.4, mlp=None):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale, "mask": {"size": window}}
    if conv:
        mx["conv"] = conv
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def latent(heads=3, dim=8, vdim=12, q_rank=10, kv_rank=20, scale=0.35, mlp=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}, "mlp": mlp}


def config(layers, width=48, vocab=61, eps=1e-5, taps=2, loop=None, cap=20.0):
    cfg = {"architecture": "Dopilorn", "canon": {"taps": taps}, "layers": layers, "logit_softcap": cap, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


class Pair:
    """the same random model in the framework and in the oracle"""

    def __init__(self, tmp_path, cfg, seed=0, dtype="float32", n_ctx=512, edit=None):
        self.cfg = cfg
        self.w = do.random_model(cfg, seed)
        if edit:
            edit(self.w)
        self.dir = do.write_model(str(tmp_path / f"d{seed}_{dtype}_{abs(hash(str(cfg))) % 10**8}"), cfg, self.w)
        self.model = engine.Model(self.dir, dtype=dtype)
        self.ctx = engine.Context(self.model, n_ctx)

    def close(self):
        self.ctx.close()
        self.model.close()

    def tokens(self, n, seed=1):
        return np.random.default_rng(seed).integers(0, self.cfg["vocab"], size=n).tolist()

    def expected(self, toks, residuals=None, cfg=None, w=None):
        return do.forward(cfg or self.cfg, w or self.w, toks, residuals)

    def run(self, toks, cuts=None, ctx=None):
        """logits of every position, the token stream cut into steps of the given sizes (None: one step)"""
        ctx = ctx or self.ctx
        ctx.kv_clear()
        out, pos, i = [], 0, 0
        cuts = list(cuts) if cuts else [len(toks)]
        while pos < len(toks):
            n = min(cuts[i % len(cuts)], len(toks) - pos)
            out.append(ctx.decode_rows(toks[pos:pos + n], pos, list(range(n))))
            pos += n
            i += 1
        return np.concatenate(out)


@pytest.mark.parametrize("layer", [gdelta(), gdelta(heads=2, dim=5, mlp=ff()), attn(), attn(heads=3, kv_heads=3, dim=5, vdim=7, conv=0, mlp=ff(40)),
                                   latent(), latent(heads=1, dim=6, vdim=3, q_rank=7, kv_rank=9, mlp=ff(30))],
                         ids=["gdelta", "gdelta-odd+ff", "attention-grouped", "attention-no-conv+ff", "latent", "latent-one-head+ff"])
def test_each_mixer_alone_with_the_residual_after_the_layer(tmp_path, layer):
    p = Pair(tmp_path, config([layer]))
    toks = p.tokens(23)
    res = []
    want = p.expected(toks, res)
    p.ctx.set_taps(True)
    got = p.ctx.decode_rows(toks, 0, list(range(len(toks))))
    taps = p.ctx.layer_taps(len(toks))
    p.ctx.set_taps(False)
    assert taps.shape[0] == 1 and np.abs(taps[0] - res[0]).max() < 1e-4 * max(1.0, np.abs(res[0]).max())
    assert err(got, want) < TOL32
    assert err(p.run(toks, [1]), want) < TOL32
    p.close()


def test_input_convolution_norm_weights_cap_and_activation_matter(tmp_path):
    """the oracle without one of the small mechanisms is far from the framework: none of them is a no-op in these models"""
    cfg = config([gdelta(mlp=ff())], taps=3, cap=4.0)
    p = Pair(tmp_path, cfg)
    toks = p.tokens(17)
    got = p.run(toks)
    assert err(got, p.expected(toks)) < TOL32
    for key in ("l0.canon1", "l0.canon2", "l0.norm1", "l0.norm2", "final.norm", "l0.mlp.act"):
        w2 = dict(p.w); w2[key] = np.zeros_like(p.w[key])
        assert err(got, p.expected(toks, w=w2)) > 50 * TOL32, key
    c2 = dict(cfg); c2["logit_softcap"] = 2000.0
    assert err(got, p.expected(toks, cfg=c2)) > 50 * TOL32
    p.close()


FULL = [gdelta(mlp=ff(40)), latent(mlp=ff()), attn(mlp=ff()), gdelta(heads=2, dim=16), attn(heads=2, kv_heads=1, dim=8, vdim=16, conv=2, window=11, mlp=ff(32)),
        latent(heads=2, dim=12, vdim=4, q_rank=6, kv_rank=16)]


@pytest.mark.parametrize("loop", [None, (1, 4, 2), (0, 6, 3), (2, 3, 1), (3, 6, 2)], ids=str)
def test_whole_prompt_token_by_token_and_portions_agree(tmp_path, loop):
    p = Pair(tmp_path, config(FULL, loop=loop, taps=3))
    toks = p.tokens(75)
    res = []
    want = p.expected(toks, res)
    p.ctx.set_taps(True)
    p.ctx.kv_clear()
    p.ctx.decode_rows(toks, 0, [])
    taps = p.ctx.layer_taps(len(toks))
    p.ctx.set_taps(False)
    assert taps.shape[0] == len(res) == len(do.run_order(p.cfg))          # a repeated layer counts each time
    for a, b in zip(taps, res):
        assert np.abs(a - b).max() < 1e-4 * max(1.0, np.abs(b).max())
    whole = p.run(toks)
    assert err(whole, want) < TOL32
    single = p.run(toks, [1])                         # every token through the replayed one-token graph
    assert err(single, want) < TOL32
    for cuts in ([2], [3, 2, 7, 1, 5], [37, 2, 2, 30], [6, 1, 1, 11]):
        assert err(p.run(toks, cuts), want) < TOL32, cuts
    p.close()


def test_each_pass_of_the_repeated_span_has_its_own_state(tmp_path):
    """an oracle that lets the passes share nothing by construction; the framework agrees in prompts and in decoding, and a
    wrong pass order (the step vectors swapped) is far away"""
    cfg = config([attn(window=5), gdelta(), latent()], loop=(0, 3, 3))
    p = Pair(tmp_path, cfg, seed=3)
    toks = p.tokens(40, seed=2)
    want = p.expected(toks)
    w2 = dict(p.w); w2["loop.step"] = p.w["loop.step"][::-1].copy()
    assert err(p.expected(toks, w=w2), want) > 50 * TOL32
    assert err(p.run(toks, [25, 1]), want) < TOL32
    assert err(p.run(toks, [1]), want) < TOL32
    p.close()


def test_cleared_context_is_as_good_as_new_and_contexts_do_not_meet(tmp_path):
    p = Pair(tmp_path, config(FULL, loop=(1, 4, 2)))
    a, b = p.tokens(40, seed=3), p.tokens(29, seed=4)
    fresh = engine.Context(p.model, 512)
    ref_b = p.run(b, [5, 1, 1, 9], ctx=fresh)
    p.run(a, [7, 1])                                  # fills cache rows, recurrent state and both kinds of convolution history
    again = p.run(b, [5, 1, 1, 9])                    # run() clears first: the same context, used again
    assert np.array_equal(again, ref_b)
    assert err(again, p.expected(b)) < TOL32
    # two live sequences of unequal length stepping in turn, each as if alone
    p.ctx.kv_clear(); fresh.kv_clear()
    ga, gb, pa, pb = [], [], 0, 0
    for na, nb in ((9, 3), (1, 1), (4, 13), (1, 2), (25, 10)):
        ga.append(p.ctx.decode_rows(a[pa:pa + na], pa, list(range(na)))); pa += na
        gb.append(fresh.decode_rows(b[pb:pb + nb], pb, list(range(nb)))); pb += nb
    assert err(np.concatenate(ga), p.expected(a)) < TOL32
    assert err(np.concatenate(gb), p.expected(b)) < TOL32
    fresh.close()
    p.close()


def sharpen(names, gain=6.0):
    def edit(w):
        for k in list(w):
            if any(k.endswith(n) for n in names):
                w[k] = so.round_bf16(w[k] * gain)
    return edit


@pytest.mark.parametrize("window", [1, 2, 9, 33, 64])
def test_window_edges_in_prompts_and_in_decoding(tmp_path, window):
    cfg = config([attn(heads=2, kv_heads=1, dim=8, vdim=8, window=window, scale=1.0), gdelta(heads=2, dim=4)], width=32)
    p = Pair(tmp_path, cfg, seed=window, edit=sharpen(["mix.q"]))
    toks = p.tokens(3 * window + 20, seed=window)
    want = p.expected(toks)
    # the oracle itself tells windows apart by far more than the tolerance: a window one token off would show
    for off in (-1, 1):
        if window + off >= 1:
            c2 = copy.deepcopy(cfg)
            c2["layers"][0]["mixer"]["mask"]["size"] = window + off
            assert err(p.expected(toks, cfg=c2)[window + 1:], want[window + 1:]) > 50 * TOL32
    assert err(p.run(toks), want) < TOL32
    assert err(p.run(toks, [window + 1, 1]), want) < TOL32              # the window passes over decoded tokens
    assert err(p.run(toks, [max(window - 1, 1), 2, 1]), want) < TOL32   # portions that start and end inside a window
    assert err(p.run(toks, [3, 5, 2, 31]), want) < TOL32
    p.close()


def test_one_changed_token_just_inside_and_just_outside_the_window(tmp_path):
    """a model whose only path between positions is the window (no convolutions, no recurrence) with peaky soft-max rows: one
    token is changed; the last query that still sees it moves visibly, the first query past the window must not move at all"""
    window = 12
    cfg = config([attn(heads=2, kv_heads=2, dim=8, vdim=8, conv=0, window=window, scale=1.0)], width=32, taps=1, vocab=40)

    def edit(w):
        sharpen(["mix.q"], 4.0)(w)
        w["l0.canon1"][:] = 0.0
    p = Pair(tmp_path, cfg, seed=1, edit=edit)
    toks = [t if t != 7 else 8 for t in p.tokens(60, seed=3)]
    at = 20
    toks[at] = 7
    want = p.expected(toks)
    plain = list(toks); plain[at] = 9
    base = p.expected(plain)
    last_in, first_out = at + window - 1, at + window
    assert err(want[last_in:last_in + 1], base[last_in:last_in + 1]) > 100 * TOL32         # still seen
    assert err(want[first_out:], base[first_out:]) < 1e-9                                  # gone for good (no other path in this model)
    for cuts in (None, [at + 3, 1], [last_in, 1], [first_out, 1], [at + 1, 2]):
        got = p.run(toks, cuts)
        assert err(got, want) < TOL32, cuts
        assert err(got[first_out:], base[first_out:]) < TOL32, cuts
    p.close()


def test_far_keys_and_first_tokens(tmp_path):
    """latent attention has no window: a sharpened query finds keys hundreds of positions back, in a prompt and in decoding"""
    cfg = config([latent(heads=2, kv_rank=12, scale=1.0), gdelta(heads=2, dim=8)], width=32)
    p = Pair(tmp_path, cfg, seed=5, edit=sharpen(["mix.uq"]), n_ctx=400)
    toks = p.tokens(330, seed=9)
    want = p.expected(toks)
    # the attention layer alone, without the first 250 positions: the late logits are somewhere else, far keys carry weight
    alone = config([cfg["layers"][0]], width=32)
    assert err(p.expected(toks[250:], cfg=alone)[60:], p.expected(toks, cfg=alone)[310:]) > 50 * TOL32
    got = p.run(toks, [300, 1])
    assert err(got, want) < TOL32
    assert err(got[:4], want[:4]) < TOL32             # the first tokens of a sequence: empty histories, zero state, one key
    assert err(p.run(toks[:40], [1]), want[:40]) < TOL32
    assert err(p.run(toks, [2, 129, 3, 64]), want) < TOL32
    p.close()


def test_long_decoding_through_the_graph(tmp_path):
    p = Pair(tmp_path, config(FULL[:3] + [gdelta(heads=2, dim=40)], loop=(1, 3, 2)))
    toks = p.tokens(300, seed=11)
    want = p.expected(toks)
    got = p.run(toks, [4, 1])
    assert err(got, want) < 2 * TOL32
    assert err(got[-1:], want[-1:]) < 2 * TOL32
    p.close()


@pytest.mark.parametrize("width,vocab,taps", [(36, 50, 1), (40, 77, 4), (64, 130, 2), (37, 53, 3)], ids=["scalar-loads-one-tap", "four-taps", "vector-loads", "odd-width"])
def test_other_sizes(tmp_path, width, vocab, taps):
    layers = [attn(heads=6, kv_heads=2, dim=9, vdim=5, conv=1, window=4, diff=0.1, mlp=ff(20)), latent(heads=1, dim=6, vdim=3, q_rank=5, kv_rank=9),
              gdelta(heads=1, dim=64, decay_rank=3), attn(heads=4, kv_heads=4, dim=16, vdim=40, conv=5, window=50, diff=0.8),
              latent(heads=5, dim=16, vdim=16, q_rank=32, kv_rank=32, mlp=ff(24)), gdelta(heads=5, dim=3, mlp=ff(64))]
    p = Pair(tmp_path, config(layers, width=width, vocab=vocab, eps=1e-6, taps=taps, loop=(3, 5, 2), cap=7.5), seed=width)
    toks = p.tokens(70, seed=width)
    want = p.expected(toks)
    assert err(p.run(toks), want) < TOL32
    assert err(p.run(toks, [13, 2, 1]), want) < TOL32
    p.close()


def random_config(rng):
    """a random arrangement of the three mixers with random sizes: nothing may rest on one model's values"""
    pick = lambda values: int(rng.choice(values))
    layers = []
    for _ in range(pick([2, 3, 4, 5])):
        mlp = ff(pick([24, 64, 100, 136])) if rng.random() < 0.6 else None
        kind = pick([0, 1, 2])
        if kind == 0:
            layers.append(gdelta(heads=pick([1, 2, 3, 6]), dim=pick([4, 16, 32, 48, 128]), mlp=mlp, decay_rank=pick([1, 4, 16])))
        elif kind == 1:
            layers.append(latent(heads=pick([1, 2, 3, 5, 6, 12]), dim=pick([4, 8, 24, 64]), vdim=pick([4, 16, 40, 64]), q_rank=pick([4, 12, 31, 96]),
                                 kv_rank=pick([8, 24, 64, 96, 192]), mlp=mlp, scale=float(rng.choice([0.1, 0.2, 0.35]))))
        else:
            kv = pick([1, 2, 3])
            layers.append(attn(heads=kv * pick([1, 2, 4]), kv_heads=kv, dim=pick([4, 16, 32, 128]), vdim=pick([4, 8, 48, 128, 200]), conv=pick([0, 1, 2, 3, 5]),
                               window=pick([1, 3, 17, 32, 33, 100, 300]), diff=float(rng.choice([0.2, 0.5, 0.8])), scale=float(rng.choice([0.1, 0.3])), mlp=mlp))
    n = len(layers)
    loop = None
    if rng.random() < 0.7:
        start = pick(range(n))
        loop = (start, pick(range(start + 1, n + 1)), pick([1, 2, 3]))
    return config(layers, width=pick([24, 36, 64, 100, 136]), vocab=pick([37, 100, 257, 513]), eps=float(rng.choice([1e-6, 1e-5])), taps=pick([1, 2, 3, 4]),
                  loop=loop, cap=float(rng.choice([5.0, 30.0])))


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(tmp_path, seed):
    rng = np.random.default_rng(700 + seed)
    cfg = random_config(rng)
    n = int(rng.choice([70, 150, 330]))
    p = Pair(tmp_path, cfg, seed=seed, n_ctx=n + 4)
    toks = p.tokens(n, seed=seed)
    want = p.expected(toks)
    assert err(p.run(toks), want) < 2 * TOL32, cfg
    assert err(p.run(toks, [n - 20] + [1] * 20), want) < 2 * TOL32, cfg
    assert err(p.run(toks, [2, 67, 3, 129, 1, 5]), want) < 2 * TOL32, cfg
    p.close()


def test_a_step_longer_than_one_pass(tmp_path):
    """a 700-token step runs as two passes of the layers: window, convolution inputs and recurrent state cross the pass's edge"""
    layers = [attn(heads=2, kv_heads=1, dim=8, vdim=8, conv=4, window=40), gdelta(heads=2, dim=8, mlp=ff(40)), latent(heads=2, dim=8, vdim=4, q_rank=8, kv_rank=24)]
    p = Pair(tmp_path, config(layers, loop=(0, 2, 2), taps=3), n_ctx=704)
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
    cfg = config(FULL, width=64, vocab=96, loop=(2, 5, 2))
    p = Pair(tmp_path, cfg, dtype="bfloat16")
    toks = p.tokens(150, seed=2)
    want = p.expected(toks)
    # token by token: mat-vec kernels with float32 activations on the stored bfloat16 weights: as sharp as float32
    assert err(p.run(toks[:60], [1]), want[:60]) < TOL32
    assert err(p.run(toks[:60], [3, 4, 2]), want[:60]) < TOL32
    # longer portions: tensor-core products round the activation operand to bfloat16
    for cuts in (None, [140, 1], [5, 17, 33]):
        e = row_errs(p.run(toks, cuts), want)
        assert np.median(e) < 3e-2 and e.max() < 0.25, (cuts, float(np.median(e)), float(e.max()))
    p.close()


def test_greedy_generation_through_the_bridge(tmp_path, monkeypatch):
    """initContext / doInference on a folder model: decimal-id prompt, standard chain at temperature 0 (arg-max on the device),
    prompt through the prompt kernels, generation through the one-token graph: the ids the oracle generates greedily"""
    monkeypatch.setenv("BOOSTER_B200_DTYPE", "float32")
    p = Pair(tmp_path, config(FULL[:4], loop=(1, 3, 2)))
    prompt, n_gen = p.tokens(21, seed=6), 10
    seq, ids = list(prompt), []
    for _ in range(n_gen):
        lg = p.expected(seq)[-1]
        srt = np.sort(lg)
        assert srt[-1] - srt[-2] > 1e-3               # no near-tie: float32 must pick the same id
        ids.append(int(np.argmax(lg)))
        seq.append(ids[-1])
    L = _lib.lib()
    L.init(b"", b"")
    ctx = L.initContext(6, p.dir.encode(), 1, 0, 100, 0, 0, 0, 64, n_gen, 0, 0.0, 0.0, 0.0, 1, 1.0, 1.0, 1.0, 0, 0, 200, 1.0, 1.0, 1.0, 42, b"")
    assert ctx, _lib.last_error()
    n = L.doInference(6, ctx, b"dopilorn-job", b"", " ".join(map(str, prompt)).encode())
    out = [int(x) for x in L.status(b"dopilorn-job").decode().split()]
    assert out[:len(prompt)] == prompt and out[len(prompt):] == ids
    assert n == len(prompt) + n_gen - 1 and L.getPromptTokenCount(b"dopilorn-job") == len(prompt)
    # the device-resident loop of the token-level interface gives the same ids
    p.ctx.kv_clear()
    first = int(np.argmax(p.ctx.decode(prompt, 0)))
    dev = p.ctx.generate_greedy(first, len(prompt), n_gen - 1).tolist()
    assert [first] + dev == ids
    after = p.ctx.decode([ids[-1]], len(prompt) + n_gen - 1)
    assert err(after[None], p.expected(seq)[-1][None]) < TOL32
    assert p.ctx.L.b200_kernel_launches(p.ctx.h) > 0
    p.close()


def test_bad_models_fail_loudly(tmp_path):
    cfg = config([gdelta(), attn()])
    w = do.random_model(cfg)
    c2 = copy.deepcopy(cfg); c2["layers"][0]["type"] = "mingru"
    with pytest.raises(_lib.B200Error, match="not part of the Dopilorn design"):
        engine.Model(do.write_model(str(tmp_path / "mixer"), c2, w))
    w2 = dict(w); del w2["l1.mix.k.conv"]
    with pytest.raises(_lib.B200Error, match="missing tensor"):
        engine.Model(do.write_model(str(tmp_path / "missing"), cfg, w2))
    c3 = copy.deepcopy(cfg); c3["loop"] = {"start": 1, "stop": 3, "times": 2}
    with pytest.raises(_lib.B200Error, match="loop"):
        engine.Model(do.write_model(str(tmp_path / "loop"), c3, w))
    c4 = copy.deepcopy(cfg); c4["layers"][1]["mixer"]["kv_heads"] = 3
    with pytest.raises(_lib.B200Error, match="multiple of kv_heads"):
        engine.Model(do.write_model(str(tmp_path / "heads"), c4, w))
