"""Plain, slow restatement of the Dopilorn design in numpy float64: one function per mechanism, written from the equations
and not from the kernels; recurrences walk token by token. Test infrastructure only: nothing here is shared with the CUDA
path (the safetensors writer of stack_oracle.py, also test infrastructure, is reused for the model files).

Notation: a mechanism gets the whole sequence h [T, width] and returns [T, width]; matrices are stored [out, in], so a
projection is h @ M.T; positions count from 0.

Design in short. Every layer: x <- x + mix(u1) + ff(u2), u_i = h_i + causal_fir(h_i, c_i), h_i = x / rms(x) * (1 + g_i).
Mixers: general_delta (matrix state with per-channel decay and removal along the unit key), attention (two soft-max maps per
head over a sliding window, subtracted), latent_attention (keys and values expanded from a cached latent, queries through a
latent of their own, gated heads). A span of layers may run several times; each time x is first re-mixed with the embedding.
"""
from __future__ import annotations

import numpy as np

import stack_oracle as so

F = np.float64
DECAY_RATE = float(np.exp(-0.5))


def sigm(x):
    return 1.0 / (1.0 + np.exp(-x))


def unit_rms(x, eps):
    """x over the root of (mean square + eps), along the last axis"""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def causal_fir(x, c):
    """y[t] = sum_j c[:, j] x[t - (n - 1) + j] with n taps per channel (the last tap is the current token); x[<0] = 0"""
    n = c.shape[1]
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(n):
            s = t - (n - 1) + j
            if s >= 0:
                y[t] += c[:, j] * x[s]
    return y


def poly_act(z, coef, eps):
    """coef = (a, b, c, e): a n(z) + b n(z^2) + c n(z^3) + e, n = unit_rms over a token's row"""
    a, b, c, e = coef
    return a * unit_rms(z, eps) + b * unit_rms(z ** 2, eps) + c * unit_rms(z ** 3, eps) + e


def feed_forward(u, W, eps):
    return poly_act(u @ W["up"].T, W["act"], eps) @ W["down"].T


def mix_general_delta(u, W, mx, eps):
    T = u.shape[0]
    H, D = mx["heads"], mx["dim"]
    r = (u @ W["r"].T).reshape(T, H, D)
    k = (u @ W["k"].T).reshape(T, H, D)
    v = (u @ W["v"].T).reshape(T, H, D)
    decay = np.exp(-DECAY_RATE * sigm(np.tanh(u @ W["w1"].T) @ W["w2"].T + W["w0"])).reshape(T, H, D)
    take = sigm(u @ W["a"].T + W["a.b"]).reshape(T, H, D)
    out = np.zeros((T, H, D))
    for h in range(H):
        S = np.zeros((D, D))                                  # [key channel, value channel]
        for t in range(T):
            kk = k[t, h]
            n = kk / np.sqrt(np.sum(kk * kk) + 1e-6)
            seen = n @ S                                      # what the old state returns for the unit key
            S = decay[t, h][:, None] * S - np.outer(take[t, h] * n, seen) + np.outer(kk, v[t, h])
            out[t, h] = r[t, h] @ S
    out = unit_rms(out, eps).reshape(T, H * D) * W["norm"] * sigm(u @ W["g"].T)
    return out @ W["o"].T


def soft_rows(s, allowed):
    s = np.where(allowed, s, -np.inf)
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def mix_diff_attention(u, W, mx, eps):
    T = u.shape[0]
    H, G, D, V = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
    q, k, v = u @ W["q"].T + W["q.b"], u @ W["k"].T + W["k.b"], u @ W["v"].T + W["v.b"]
    if mx.get("conv"):
        q, k, v = causal_fir(q, W["q.conv"]), causal_fir(k, W["k.conv"]), causal_fir(v, W["v.conv"])
    q, k, v = q.reshape(T, H, 2, D), k.reshape(T, G, 2, D), v.reshape(T, G, V)
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    allowed = (j <= i)
    if mx.get("mask"):
        allowed &= (i - j < mx["mask"]["size"])
    lam = np.exp(np.sum(W["lq1"] * W["lk1"])) - np.exp(np.sum(W["lq2"] * W["lk2"])) + mx["diff"]
    out = np.zeros((T, H, V))
    for h in range(H):
        g = h // (H // G)
        a = [soft_rows(q[:, h, m] @ k[:, g, m].T * mx["scale"], allowed) @ v[:, g] for m in (0, 1)]
        out[:, h] = unit_rms(a[0] - lam * a[1], eps) * (1.0 - mx["diff"])
    return out.reshape(T, H * V) @ W["o"].T


def mix_latent_attention(u, W, mx, eps):
    T = u.shape[0]
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    q = (unit_rms(u @ W["dq"].T, eps) * W["dq.norm"]) @ W["uq"].T
    lat = unit_rms(u @ W["dkv"].T, eps) * W["dkv.norm"]           # all a position leaves behind
    q, k, v = q.reshape(T, H, D), (lat @ W["uk"].T).reshape(T, H, D), (lat @ W["uv"].T).reshape(T, H, V)
    allowed = np.tril(np.ones((T, T), bool))
    gate = sigm(u @ W["g"].T)                                     # [T, H]
    out = np.zeros((T, H, V))
    for h in range(H):
        out[:, h] = (soft_rows(q[:, h] @ k[:, h].T * mx["scale"], allowed) @ v[:, h]) * gate[:, h:h + 1]
    return out.reshape(T, H * V) @ W["o"].T


MIXERS = {"general_delta": mix_general_delta, "attention": mix_diff_attention, "latent_attention": mix_latent_attention}


def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def block(x, W, cfg, i):
    L, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    xn = unit_rms(x, eps)
    h1 = xn * (1.0 + W[p + "norm1"])
    if cfg.get("canon"):
        h1 = h1 + causal_fir(h1, W[p + "canon1"])
    y = MIXERS[L["type"]](h1, sub(W, p + "mix."), L["mixer"], eps)
    if L.get("mlp"):
        h2 = xn * (1.0 + W[p + "norm2"])
        if cfg.get("canon"):
            h2 = h2 + causal_fir(h2, W[p + "canon2"])
        y = y + feed_forward(h2, sub(W, p + "mlp."), eps)
    return x + y


def run_order(cfg):
    """[(layer, pass or None)]: pass t is set on the run that opens the t-th repetition of the repeated span"""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp or lp["stop"] <= lp["start"]:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        order += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return order + [(i, None) for i in range(lp["stop"], n)]


def forward(cfg, W, tokens, residuals=None):
    """logits [T, vocab] of one sequence from its start; residuals (a list) receives x after every layer run"""
    W = {k: np.asarray(v, F) for k, v in W.items()}
    x0 = W["embed"][np.asarray(tokens)]
    x = x0
    for i, t in run_order(cfg):
        if t is not None:
            x = np.concatenate([x, x0], axis=1) @ W["loop.in"].T + W["loop.step"][t]
        x = block(x, W, cfg, i)
        if residuals is not None:
            residuals.append(x.copy())
    z = (unit_rms(x, cfg["norm"]["eps"]) * (1.0 + W["final.norm"])) @ W["head"].T
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(z / cap) if cap else z


# ---------------------------------------------------------------------------------------------------------------
# random models
# ---------------------------------------------------------------------------------------------------------------
def tensor_shapes(cfg):
    E, V = cfg["width"], cfg["vocab"]
    t = {"embed": [V, E], "final.norm": [E], "head": [V, E]}
    lp = cfg.get("loop")
    if lp and lp["stop"] > lp["start"]:
        t["loop.in"] = [E, 2 * E]
        t["loop.step"] = [lp["times"], E]
    ct = cfg["canon"]["taps"] if cfg.get("canon") else 0
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        t[p + "norm1"] = [E]
        if ct:
            t[p + "canon1"] = [E, ct]
        if L["type"] == "general_delta":
            n = mx["heads"] * mx["dim"]
            r = mx.get("decay_rank", 8)                          # read from the tensor's shape by the loader; not a config key
            for k in "rkvga":
                t[p + "mix." + k] = [n, E]
            t.update({p + "mix.a.b": [n], p + "mix.w1": [r, E], p + "mix.w2": [n, r], p + "mix.w0": [n], p + "mix.norm": [n], p + "mix.o": [E, n]})
        elif L["type"] == "attention":
            H, G, D, Vd = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
            for k, n in (("q", H * 2 * D), ("k", G * 2 * D), ("v", G * Vd)):
                t[p + "mix." + k] = [n, E]
                t[p + "mix." + k + ".b"] = [n]
                if mx.get("conv"):
                    t[p + "mix." + k + ".conv"] = [n, mx["conv"]]
            for k in ("lq1", "lk1", "lq2", "lk2"):
                t[p + "mix." + k] = [D]
            t[p + "mix.o"] = [E, H * Vd]
        elif L["type"] == "latent_attention":
            H, D, Vd, qr, kr = mx["heads"], mx["dim"], mx["vdim"], mx["q_rank"], mx["kv_rank"]
            t.update({p + "mix.dq": [qr, E], p + "mix.dq.norm": [qr], p + "mix.uq": [H * D, qr], p + "mix.dkv": [kr, E], p + "mix.dkv.norm": [kr],
                      p + "mix.uk": [H * D, kr], p + "mix.uv": [H * Vd, kr], p + "mix.g": [H, E], p + "mix.o": [E, H * Vd]})
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            t.update({p + "norm2": [E], p + "mlp.up": [ff, E], p + "mlp.down": [E, ff], p + "mlp.act": [4]})
            if ct:
                t[p + "canon2"] = [E, ct]
    return t


def random_model(cfg, seed=0):
    """weights that bfloat16 holds exactly, sized so that every mechanism matters in the logits"""
    rng = np.random.default_rng(seed)
    W = {}
    for name, shp in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[1] if name[0] == "l" and name[1].isdigit() else name
        if leaf in ("norm1", "norm2") or name == "final.norm" or leaf.endswith("canon1") or leaf.endswith("canon2") or leaf.endswith(".conv"):
            x = 0.4 * rng.standard_normal(shp)
        elif leaf == "mlp.act":
            x = np.array([0.8, 0.5, 0.3, 0.1]) + 0.1 * rng.standard_normal(4)
        elif leaf in ("mix.norm", "mix.dq.norm", "mix.dkv.norm"):
            x = 1.0 + 0.3 * rng.standard_normal(shp)
        elif leaf in ("mix.lq1", "mix.lk1", "mix.lq2", "mix.lk2"):
            x = 0.3 * rng.standard_normal(shp)
        elif len(shp) == 1 or name == "loop.step":
            x = 0.5 * rng.standard_normal(shp)
        elif name == "embed":
            x = rng.standard_normal(shp)
        elif name == "loop.in":
            x = rng.standard_normal(shp) / np.sqrt(shp[1] / 2)
        else:
            gain = 2.0 if leaf in ("mix.a", "mix.w2", "mix.g", "mix.k", "mix.q") else 1.0
            x = gain * rng.standard_normal(shp) / np.sqrt(shp[1])
        W[name] = so.round_bf16(np.asarray(x, np.float32))
    return W


def write_model(d, cfg, W):
    return so.write_model(d, cfg, W)
