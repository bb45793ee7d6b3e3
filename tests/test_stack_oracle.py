"""The numpy restatement of the layer-stack models is itself consistent (CPU only): any cut of a token stream gives the
same logits, a cleared state equals a new one, the safetensors writer and reader round-trip, and — without a CUDA device —
loading a folder model fails loudly like every other compute entry point."""
import numpy as np

import stack_oracle as so
from booster_b200 import _lib


def small_cfg():
    layers = [
        {"type": "mingru", "mixer": {"width": 10}, "mlp": None},
        {"type": "latent_attention", "mlp": {"ff": 14, "kind": "dense", "limit": 1.25},
         "mixer": {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 8, "scale": 0.4, "mask": {"size": 4},
                   "rot": {"base": 1000.0, "dims": 4, "scaling": {"factor": 2.0, "fast": 16.0, "slow": 1.0, "original": 8}}}},
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 4, "vdim": 3, "conv": 3}, "mlp": None},
    ]
    return {"architecture": "Matulorn", "layers": layers, "norm": {"eps": 1e-5, "groups": 2}, "vocab": 23, "width": 12}


def test_oracle_is_invariant_to_the_cut_and_to_reuse():
    cfg = small_cfg()
    o = so.Oracle(cfg, {k: np.asarray(v, np.float64) for k, v in so.random_model(cfg, 3).items()})
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], size=17).tolist()
    whole = o.forward(toks)
    for cuts in ([1], [2], [5, 1, 3]):
        o.reset()
        out, pos, i = [], 0, 0
        while pos < len(toks):
            n = min(cuts[i % len(cuts)], len(toks) - pos)
            out.append(o.forward(toks[pos:pos + n]))
            pos += n; i += 1
        assert np.allclose(np.concatenate(out), whole, rtol=1e-10, atol=1e-10)
    # the window really hides older keys: changing a token outside every window of the attention layer still changes the
    # recurrent layers, so compare an attention-only model
    c2 = dict(cfg); c2["layers"] = [cfg["layers"][1]]
    o2 = so.Oracle(c2, {k: np.asarray(v, np.float64) for k, v in so.random_model(c2, 4).items()})
    a = o2.forward(toks)
    o2.reset()
    t2 = list(toks); t2[2] = (t2[2] + 1) % cfg["vocab"]
    b = o2.forward(t2)
    assert np.allclose(a[6:], b[6:]) and not np.allclose(a[5], b[5])       # position 5 still sees key 2 (window 4), position 6 does not


def test_safetensors_round_trip(tmp_path):
    cfg = small_cfg()
    w = so.random_model(cfg, 1)
    d = so.write_model(str(tmp_path / "m"), cfg, w)
    back = so.load_safetensors(d + "/model.safetensors")
    assert set(back) == set(w)
    for k in w:
        assert np.array_equal(back[k], np.asarray(w[k], np.float64)), k


def test_folder_model_needs_a_gpu(tmp_path):
    L = _lib.lib()
    if L.b200_device_count() > 0:
        return
    cfg = small_cfg()
    d = so.write_model(str(tmp_path / "m"), cfg, so.random_model(cfg, 1))
    assert not L.b200_model_load_dtype(d.encode(), 0, 0, -1, b"float32")
    assert b"no CUDA device" in L.b200_last_error()
    assert L.b200_stack_time_linear(0, 0, 1, 8, 8, 1) < 0
