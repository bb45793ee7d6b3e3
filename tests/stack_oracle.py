"""Plain, slow restatement of the layer-stack models (Matulorn design) in numpy float64: one function per mechanism,
token by token where a mechanism is a recurrence. Test infrastructure only: it shares no code with the CUDA path and is
written from the equations, not from the kernels.

Notation: h = a mixer's input [T, width]; W @ x with W stored [out, in]; positions count from 0 in each sequence.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

F = np.float64


# ---------------------------------------------------------------------------------------------------------------
# weights: safetensors (8-byte length, JSON header, raw data), bfloat16 / float32 / int32
# ---------------------------------------------------------------------------------------------------------------
def bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def round_bf16(x: np.ndarray) -> np.ndarray:
    return bf16_to_f32(f32_to_bf16_bits(x))


def load_safetensors(path: str) -> dict:
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        head = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, d in head.items():
        if name == "__metadata__":
            continue
        a, b = d["data_offsets"]
        buf = np.frombuffer(data[a:b], dtype={"BF16": np.uint16, "F32": np.float32, "I32": np.int32}[d["dtype"]])
        if d["dtype"] == "BF16":
            buf = bf16_to_f32(buf)
        out[name] = buf.reshape(d["shape"]).astype(F if d["dtype"] != "I32" else np.int64)
    return out


def save_safetensors(path: str, tensors: dict) -> None:
    """tensors: name -> float array (stored as bfloat16)"""
    head, blobs, off = {}, [], 0
    for name, a in tensors.items():
        b = f32_to_bf16_bits(np.asarray(a, dtype=np.float32)).tobytes()
        head[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(head).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


# ---------------------------------------------------------------------------------------------------------------
# mechanisms
# ---------------------------------------------------------------------------------------------------------------
def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return np.logaddexp(0.0, x)


def group_rms_norm(x, w, groups, eps):
    """x [.., n] in `groups` equal consecutive parts, each over its own root mean square; then times w"""
    shp = x.shape
    p = x.reshape(shp[:-1] + (groups, shp[-1] // groups))
    p = p / np.sqrt(np.mean(p * p, axis=-1, keepdims=True) + eps)
    return p.reshape(shp) * w


def min_gru(h, W, state):
    """state [width] carried across calls (updated in place). Returns [T, out]"""
    z = sigmoid(h @ W["z"].T + W["z.b"])
    u = h @ W["x"].T + W["x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    gate = silu(h @ W["g"].T)
    out = np.zeros((h.shape[0], W["o"].shape[0]), F)
    for t in range(h.shape[0]):
        state[:] = (1.0 - z[t]) * state + z[t] * cand[t]
        out[t] = W["o"] @ (state * gate[t])
    return out


def yarn_tables(cfg_rot, n_pos):
    """(cos, sin) [n_pos, dims/2] with YaRN-scaled frequencies and magnitude"""
    dims, base = int(cfg_rot["dims"]), float(cfg_rot["base"])
    i = np.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = cfg_rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def dim_of(t):
            return dims * math.log(orig / (2 * math.pi * t)) / (2 * math.log(base))
        lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    a = np.arange(n_pos, dtype=F)[:, None] * f[None, :]
    return np.cos(a) * mag, np.sin(a) * mag


def rotate_half(x, cos, sin, dims):
    """x [.., n >= dims]: pair (i, i + dims/2) for i < dims/2, the rest unchanged; cos/sin [dims/2] of the position"""
    y = x.copy()
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    y[..., :dims // 2] = u * cos - v * sin
    y[..., dims // 2:dims] = v * cos + u * sin
    return y


def latent_attention(h, W, mx, eps, cache, pos0):
    """cache: dict with lists 'c' (latents) and 'kr' (rotated shared key parts) of all earlier positions of the sequence"""
    H, D, R, V, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    T = h.shape[0]
    rot = mx["rot"]
    dims = int(rot["dims"])
    cos, sin = yarn_tables(rot, pos0 + T)
    window = mx.get("mask", {}).get("size") if mx.get("mask") else None
    q = (h @ W["q"].T).reshape(T, H, D + R)
    dkv = h @ W["dkv"].T
    out = np.zeros((T, H * V), F)
    for t in range(T):
        p = pos0 + t
        c = dkv[t, :rank]
        c = c / np.sqrt(np.mean(c * c) + eps) * W["dkv.norm"]
        cache["c"].append(c)
        cache["kr"].append(rotate_half(dkv[t, rank:], cos[p], sin[p], dims))
        j0 = 0 if window is None else max(0, p - window + 1)
        C = np.stack(cache["c"][j0:p + 1])                 # [n, rank]
        KR = np.stack(cache["kr"][j0:p + 1])               # [n, R]
        for hh in range(H):
            qu = q[t, hh, :D]
            qr = rotate_half(q[t, hh, D:], cos[p], sin[p], dims)
            ku = C @ W["uk"][hh * D:(hh + 1) * D].T        # [n, D]
            vv = C @ W["uv"][hh * V:(hh + 1) * V].T        # [n, V]
            s = (ku @ qu + KR @ qr) * mx["scale"]
            sink = W["sink"][hh]
            m = max(s.max(), sink)
            e = np.exp(s - m)
            den = e.sum() + math.exp(sink - m)
            out[t, hh * V:(hh + 1) * V] = (e / den) @ vv
    return out @ W["o"].T


def short_conv(x, w, hist):
    """x [T, C], w [C, taps] (last column = the current token), hist [taps - 1, C] = the inputs before x (updated)"""
    taps = w.shape[1]
    full = np.concatenate([hist, x], axis=0)
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        y[t] = np.einsum("kc,ck->c", full[t:t + taps], w)
    if taps > 1:
        hist[:] = full[-(taps - 1):]
    return y


def gated_delta(h, W, mx, eps, st):
    """st: dict with 'S' [heads, dim, vdim] and conv histories 'q', 'k', 'v' ([taps - 1, channels])"""
    H, KH, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = silu(short_conv(h @ W["q"].T, W["q.conv"], st["q"])).reshape(T, KH, D)
    k = silu(short_conv(h @ W["k"].T, W["k.conv"], st["k"])).reshape(T, KH, D)
    v = silu(short_conv(h @ W["v"].T, W["v.conv"], st["v"])).reshape(T, H, V)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W["b"].T)
    g = np.exp(-np.exp(W["A_log"]) * softplus(h @ W["a"].T + W["dt_bias"]))
    gate = silu(h @ W["g"].T).reshape(T, H, V)
    o = np.zeros((T, H, V), F)
    rep = H // KH
    for t in range(T):
        for hh in range(H):
            kk, qq = k[t, hh // rep], q[t, hh // rep]
            S = st["S"][hh]
            S *= g[t, hh]
            u = beta[t, hh] * (v[t, hh] - S.T @ kk)
            S += np.outer(kk, u)
            o[t, hh] = S.T @ qq
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps) * W["norm"] * gate
    return o.reshape(T, H * V) @ W["o"].T


def dense_ff(h, W, mlp):
    lim = mlp["limit"]
    g = np.minimum(h @ W["gate"].T + W["gate.b"], lim)
    u = np.clip(h @ W["up"].T + W["up.b"], -lim, lim)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W["down"].T + W["down.b"]


# ---------------------------------------------------------------------------------------------------------------
# the model: state per sequence, any cut of the token stream into calls
# ---------------------------------------------------------------------------------------------------------------
class Oracle:
    def __init__(self, cfg: dict, tensors: dict):
        self.cfg, self.w = cfg, tensors
        self.reset()

    @classmethod
    def from_dir(cls, d):
        with open(os.path.join(d, "config.json")) as f:
            cfg = json.load(f)
        return cls(cfg, load_safetensors(os.path.join(d, "model.safetensors")))

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def reset(self):
        self.pos, self.state = 0, []
        for L in self.cfg["layers"]:
            mx = L["mixer"]
            if L["type"] == "mingru":
                self.state.append(np.zeros(mx["width"], F))
            elif L["type"] == "latent_attention":
                self.state.append({"c": [], "kr": []})
            elif L["type"] == "delta":
                t = mx["conv"] - 1
                self.state.append({"S": np.zeros((mx["heads"], mx["dim"], mx["vdim"]), F),
                                   "q": np.zeros((t, mx["kv_heads"] * mx["dim"]), F), "k": np.zeros((t, mx["kv_heads"] * mx["dim"]), F),
                                   "v": np.zeros((t, mx["heads"] * mx["vdim"]), F)})
            else:
                raise ValueError(L["type"])

    def forward(self, tokens, layers_out=None):
        """the next tokens of the sequence -> logits [T, vocab]"""
        cfg = self.cfg
        G, eps = cfg["norm"]["groups"], cfg["norm"]["eps"]
        x = self.w["embed"][np.asarray(tokens)]
        for i, L in enumerate(cfg["layers"]):
            p = f"l{i}."
            W = self.sub(p + "mix.")
            hin = group_rms_norm(x, self.w[p + "norm1"], G, eps)
            if L["type"] == "mingru":
                y = min_gru(hin, W, self.state[i])
            elif L["type"] == "latent_attention":
                y = latent_attention(hin, W, L["mixer"], eps, self.state[i], self.pos)
            else:
                y = gated_delta(hin, W, L["mixer"], eps, self.state[i])
            x = x + group_rms_norm(y, self.w[p + "norm1b"], G, eps)
            if L.get("mlp"):
                y = dense_ff(group_rms_norm(x, self.w[p + "norm2"], G, eps), self.sub(p + "mlp."), L["mlp"])
                x = x + group_rms_norm(y, self.w[p + "norm2b"], G, eps)
            if layers_out is not None:
                layers_out.append(x.copy())
        self.pos += len(tokens)
        return group_rms_norm(x, self.w["final.norm"], G, eps) @ self.w["head"].T


# ---------------------------------------------------------------------------------------------------------------
# random models for the tests
# ---------------------------------------------------------------------------------------------------------------
def random_model(cfg: dict, seed: int = 0, scale: float = 1.0) -> dict:
    """random bfloat16-representable weights for a configuration (names and shapes as the loader expects them)"""
    rng = np.random.default_rng(seed)
    E, V = cfg["width"], cfg["vocab"]
    t = {}

    def mat(o, i, s=1.0):
        return round_bf16((rng.standard_normal((o, i)) * s * scale / math.sqrt(i)).astype(np.float32))

    def vec(n, mean=0.0, s=0.5):
        return round_bf16((mean + s * rng.standard_normal(n)).astype(np.float32))
    t["embed"] = round_bf16(rng.standard_normal((V, E)).astype(np.float32))
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        t[p + "norm1"], t[p + "norm1b"] = vec(E, 1.0, 0.2), vec(E, 1.0, 0.2)
        if L["type"] == "mingru":
            w = mx["width"]
            t[p + "mix.z"], t[p + "mix.z.b"] = mat(w, E, 2.0), vec(w)
            t[p + "mix.x"], t[p + "mix.x.b"] = mat(w, E, 2.0), vec(w)
            t[p + "mix.g"], t[p + "mix.o"] = mat(w, E, 2.0), mat(E, w)
        elif L["type"] == "latent_attention":
            H, D, R, Vd, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
            t[p + "mix.q"] = mat(H * (D + R), E, 2.0)
            t[p + "mix.dkv"] = mat(rank + R, E, 2.0)
            t[p + "mix.dkv.norm"] = vec(rank, 1.0, 0.2)
            t[p + "mix.uk"], t[p + "mix.uv"] = mat(H * D, rank, 2.0), mat(H * Vd, rank, 2.0)
            t[p + "mix.sink"] = vec(H, 0.0, 1.0)
            t[p + "mix.o"] = mat(E, H * Vd)
        else:
            H, KH, D, Vd, taps = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["conv"]
            for nm, ch in (("q", KH * D), ("k", KH * D), ("v", H * Vd)):
                t[p + "mix." + nm] = mat(ch, E, 2.0)
                t[p + "mix." + nm + ".conv"] = round_bf16((rng.standard_normal((ch, taps)) * 0.6).astype(np.float32))
            t[p + "mix.b"], t[p + "mix.a"] = mat(H, E, 2.0), mat(H, E, 2.0)
            t[p + "mix.A_log"], t[p + "mix.dt_bias"] = vec(H, -1.0, 0.7), vec(H, 0.0, 1.0)
            t[p + "mix.norm"] = vec(Vd, 1.0, 0.2)
            t[p + "mix.g"], t[p + "mix.o"] = mat(H * Vd, E, 2.0), mat(E, H * Vd)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            t[p + "norm2"], t[p + "norm2b"] = vec(E, 1.0, 0.2), vec(E, 1.0, 0.2)
            t[p + "mlp.gate"], t[p + "mlp.gate.b"] = mat(ff, E, 2.0), vec(ff)
            t[p + "mlp.up"], t[p + "mlp.up.b"] = mat(ff, E, 2.0), vec(ff)
            t[p + "mlp.down"], t[p + "mlp.down.b"] = mat(E, ff), vec(E)
    t["final.norm"] = vec(E, 1.0, 0.2)
    t["head"] = mat(V, E)
    return t


def write_model(d: str, cfg: dict, tensors: dict) -> str:
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d
