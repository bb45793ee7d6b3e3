"""The numpy restatement of the Dopilorn design checked against itself on the CPU: properties that follow from the equations
(causality, the window's exact reach, the recurrence against its one-step closed form, the order of layer runs) hold for the
oracle the GPU tests compare with."""
import copy

import numpy as np

import dopilorn_oracle as do


def cfg_of(layers, **kw):
    c = {"architecture": "Dopilorn", "canon": {"taps": 3}, "layers": layers, "logit_softcap": 10.0, "norm": {"eps": 1e-5}, "vocab": 41, "width": 24}
    c.update(kw)
    return c


GD = {"type": "general_delta", "mixer": {"heads": 2, "dim": 6, "decay_rank": 3}, "mlp": {"ff": 20, "kind": "dense"}}
AT = {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "conv": 2, "diff": 0.3, "scale": 0.5, "mask": {"size": 5}}, "mlp": None}
LA = {"type": "latent_attention", "mixer": {"heads": 2, "dim": 4, "vdim": 6, "q_rank": 5, "kv_rank": 7, "scale": 0.5}, "mlp": {"ff": 16, "kind": "dense"}}


def test_run_order_repeats_the_span_and_marks_each_pass():
    c = cfg_of([GD, AT, LA, GD], loop={"start": 1, "stop": 3, "times": 3})
    assert do.run_order(c) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert do.run_order(cfg_of([GD, AT])) == [(0, None), (1, None)]
    assert do.run_order(cfg_of([GD, AT], loop={"start": 0, "stop": 2, "times": 1})) == [(0, 0), (1, None)]


def test_later_tokens_do_not_reach_back_and_residuals_are_reported_per_run():
    c = cfg_of([LA, GD, AT], loop={"start": 0, "stop": 2, "times": 2})
    W = do.random_model(c, 1)
    toks = np.random.default_rng(0).integers(0, 41, size=30).tolist()
    res = []
    full = do.forward(c, W, toks, res)
    assert len(res) == 5 and res[0].shape == (30, 24)
    other = toks[:20] + [(t + 1) % 41 for t in toks[20:]]
    assert np.allclose(do.forward(c, W, other)[:20], full[:20], atol=1e-12)
    assert np.abs(full).max() <= 10.0


def test_the_window_reaches_exactly_its_size():
    c = cfg_of([AT], canon={"taps": 1})
    W = do.random_model(c, 2)
    W["l0.canon1"][:] = 0
    W["l0.mix.q.conv"][:, 0] = 0; W["l0.mix.k.conv"][:, 0] = 0; W["l0.mix.v.conv"][:, 0] = 0      # only the current token's tap
    toks = np.random.default_rng(1).integers(0, 41, size=20).tolist()
    a = do.forward(c, W, toks)
    b = do.forward(c, W, toks[:7] + [(toks[7] + 3) % 41] + toks[8:])
    moved = np.abs(a - b).max(axis=1) > 1e-9
    assert moved[7:12].all() and not moved[:7].any() and not moved[12:].any()      # positions 7 .. 7 + 5 - 1


def test_the_recurrence_after_one_token_is_the_outer_product_read_by_r():
    c = cfg_of([dict(GD, mlp=None)])
    W = {k: np.asarray(v, np.float64) for k, v in do.random_model(c, 3).items()}
    u = np.random.default_rng(2).standard_normal((1, 24))
    M = do.sub(W, "l0.mix.")
    r, k, v = (u @ M["r"].T).reshape(2, 6), (u @ M["k"].T).reshape(2, 6), (u @ M["v"].T).reshape(2, 6)
    o = np.stack([(r[h] @ k[h]) * v[h] for h in range(2)])                 # S_1 = k v^T from a zero state
    want = (do.unit_rms(o, 1e-5).reshape(1, 12) * M["norm"] * do.sigm(u @ M["g"].T)) @ M["o"].T
    assert np.allclose(do.mix_general_delta(u, M, c["layers"][0]["mixer"], 1e-5), want, atol=1e-12)


def test_poly_act_and_fir_by_hand():
    z = np.array([[1.0, -2.0, 3.0]])
    n = lambda x: x / np.sqrt(np.mean(x * x) + 0.5)
    assert np.allclose(do.poly_act(z, (2.0, -1.0, 0.5, 0.25), 0.5), 2 * n(z) - n(z ** 2) + 0.5 * n(z ** 3) + 0.25)
    x = np.arange(8.0).reshape(4, 2)
    c = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = do.causal_fir(x, c)
    assert np.allclose(y[:, 1], x[:, 1])
    assert np.allclose(y[:, 0], [0.0, 200.0, 420.0, 642.0])


def test_lambda_and_the_subtraction_matter():
    c = cfg_of([AT])
    W = do.random_model(c, 4)
    toks = list(range(12))
    base = do.forward(c, W, toks)
    c2 = copy.deepcopy(c); c2["layers"][0]["mixer"]["diff"] = 0.6
    assert np.abs(do.forward(c2, W, toks) - base).max() > 1e-3
    W2 = dict(W); W2["l0.mix.lq1"] = W["l0.mix.lq1"] + 1.0
    assert np.abs(do.forward(c, W2, toks) - base).max() > 1e-3
