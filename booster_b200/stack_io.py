"""Synthetic models of the layer-stack family (config.json + model.safetensors) for benchmarks and smoke runs: random
bfloat16 weights of the right shapes, the counterpart of gguf_io.synth_llama for the GGUF path. Pure host code."""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List

import numpy as np


def matulorn_config(width: int, n_layer: int, ff: int, heads: int, vocab: int = 32000, head_dim: int = 128, rot_dim: int = 64,
                    kv_rank: int = 512, window: int = 1024, groups: int = 8, pattern=("mingru", "latent_attention", "delta", "latent_attention")) -> dict:
    """a configuration whose layers resemble a real model's: mixers in `pattern` order, a feed-forward on every layer"""
    layers = []
    for i in range(n_layer):
        kind = pattern[i % len(pattern)]
        if kind == "mingru":
            mx = {"width": width}
        elif kind == "latent_attention":
            mx = {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "kv_rank": kv_rank, "scale": (head_dim + rot_dim) ** -0.5,
                  "mask": {"size": window},
                  "rot": {"base": 500000.0, "dims": rot_dim, "scaling": {"factor": 8.0, "fast": 32.0, "slow": 1.0, "original": 4096}}}
        else:
            mx = {"heads": heads, "kv_heads": max(1, heads // 2), "dim": head_dim, "vdim": head_dim, "conv": 4}
        layers.append({"type": kind, "mixer": mx, "mlp": {"ff": ff, "kind": "dense", "limit": 7.0}})
    return {"architecture": "Matulorn", "layers": layers, "norm": {"eps": 1e-6, "groups": groups}, "vocab": vocab, "width": width}


def tensor_shapes(cfg: dict) -> Dict[str, List[int]]:
    E, V = cfg["width"], cfg["vocab"]
    t = {"embed": [V, E]}
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        t[p + "norm1"] = [E]; t[p + "norm1b"] = [E]
        if L["type"] == "mingru":
            w = mx["width"]
            t.update({p + "mix.z": [w, E], p + "mix.z.b": [w], p + "mix.x": [w, E], p + "mix.x.b": [w], p + "mix.g": [w, E], p + "mix.o": [E, w]})
        elif L["type"] == "latent_attention":
            H, D, R, Vd, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
            t.update({p + "mix.q": [H * (D + R), E], p + "mix.dkv": [rank + R, E], p + "mix.dkv.norm": [rank], p + "mix.uk": [H * D, rank],
                      p + "mix.uv": [H * Vd, rank], p + "mix.sink": [H], p + "mix.o": [E, H * Vd]})
        elif L["type"] == "delta":
            H, KH, D, Vd, taps = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["conv"]
            t.update({p + "mix.q": [KH * D, E], p + "mix.q.conv": [KH * D, taps], p + "mix.k": [KH * D, E], p + "mix.k.conv": [KH * D, taps],
                      p + "mix.v": [H * Vd, E], p + "mix.v.conv": [H * Vd, taps], p + "mix.b": [H, E], p + "mix.A_log": [H], p + "mix.norm": [Vd],
                      p + "mix.a": [H, E], p + "mix.dt_bias": [H], p + "mix.g": [H * Vd, E], p + "mix.o": [E, H * Vd]})
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            t.update({p + "norm2": [E], p + "norm2b": [E], p + "mlp.gate": [ff, E], p + "mlp.gate.b": [ff], p + "mlp.up": [ff, E],
                      p + "mlp.up.b": [ff], p + "mlp.down": [E, ff], p + "mlp.down.b": [E]})
    t["final.norm"] = [E]
    t["head"] = [V, E]
    return t


def synth_stack(d: str, cfg: dict, seed: int = 1234) -> str:
    """write config.json + model.safetensors with random bfloat16 weights: matrices ~ N(0, 1/fan_in), norm weights ~ 1"""
    os.makedirs(d, exist_ok=True)
    shapes = tensor_shapes(cfg)
    head, off = {}, 0
    for name, shp in shapes.items():
        n = int(np.prod(shp)) * 2
        head[name] = {"dtype": "BF16", "shape": shp, "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(head).encode()
    hj += b" " * (-len(hj) % 8)
    rng = np.random.default_rng(seed)
    tmp = os.path.join(d, f"model.safetensors.tmp{os.getpid()}")
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for name, shp in shapes.items():
            n = int(np.prod(shp))
            if len(shp) == 2 and not name.endswith(".conv"):
                x = rng.standard_normal(n, dtype=np.float32) * (1.0 / math.sqrt(shp[1]))
            elif "norm" in name:
                x = 1.0 + 0.1 * rng.standard_normal(n, dtype=np.float32)
            elif name.endswith("A_log"):
                x = -1.0 + 0.5 * rng.standard_normal(n, dtype=np.float32)
            else:
                x = 0.3 * rng.standard_normal(n, dtype=np.float32)
            f.write((x.view(np.uint32) >> 16).astype(np.uint16).tobytes())        # truncation to bfloat16: random data
    os.replace(tmp, os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return d


def n_params(cfg: dict) -> int:
    return sum(int(np.prod(s)) for s in tensor_shapes(cfg).values())
