"""Small Nufasun configurations for the tests and a writer of model folders whose weights make every mechanism
count: queries and keys whose norm weights are large enough for peaked attention, a lambda of order one, decays that
let the recurrent state live for hundreds of tokens, convolutions with weight on every tap, gate and up values on both
sides of the feed-forward's limit. The sizes differ from layer to layer and avoid coincidences (key size != value
size, kv_heads != 1, rotated part smaller than the key, windows that are no multiple of the page size, ...).
"""
import json
import math
import os

import numpy as np
import torch


def _attn(heads, kv, dim, vdim, window, rot_dims, base=10000.0, scale=None, softcap=30.0, diff=0.2):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "diff": diff, "softcap": softcap,
         "scale": scale if scale is not None else dim ** -0.5, "rot": {"base": base, "dims": rot_dims}}
    if window is not None:
        d["mask"] = {"size": window}
    return d


def _delta(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _layer(kind, mixer, ff=None, limit=1.0):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def _model(vocab, width, eps, layers, loop=None, scale=1.0, cap=0.0):
    d = {"architecture": "Nufasun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
         "logit_softcap": cap, "layers": layers}
    if loop is not None:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


# one mechanism each between embedding and head
ONLY_ATTENTION = _model(200, 64, 1e-5, [_layer("attention", _attn(6, 2, 16, 24, 11, 8))])
ONLY_DELTA = _model(200, 64, 1e-5, [_layer("delta", _delta(6, 3, 12, 20, 3))])
ONLY_MLP = _model(200, 64, 1e-6, [_layer("attention", _attn(2, 1, 8, 8, 5, 8), ff=96, limit=0.7)], scale=3.0, cap=9.0)
# a loop over the whole model, three passes, a single layer: the stream additions alone matter
ONLY_LOOP = _model(150, 48, 1e-5, [_layer("delta", _delta(2, 1, 8, 8, 2), ff=40)], loop=(0, 1, 3), scale=2.0)

# all of it, every layer different; the loop runs layers 1..3 twice and starts inside the model
MIXED_A = _model(331, 96, 1e-5, [
    _layer("delta", _delta(4, 2, 24, 16, 4), ff=160, limit=1.5),
    _layer("attention", _attn(4, 2, 32, 16, 21, 32, base=50000.0, softcap=20.0), ff=None),
    _layer("delta", _delta(3, 3, 16, 32, 2), ff=64),
    _layer("attention", _attn(3, 3, 16, 32, 9, 4, scale=0.3, diff=0.35), ff=128, limit=0.5),
    _layer("attention", _attn(6, 1, 8, 16, None, 8, softcap=0.0), ff=72),
], loop=(1, 4, 2), scale=5.0, cap=12.0)
# sizes in multiples of 16 (what tensor-core kernels take), more heads, wider, loop from the first layer, three passes
MIXED_B = _model(500, 256, 2e-6, [
    _layer("attention", _attn(8, 2, 64, 32, 70, 32, base=250.0), ff=384),
    _layer("delta", _delta(8, 2, 32, 64, 4), ff=384, limit=2.0),
    _layer("attention", _attn(4, 1, 48, 80, 33, 48, softcap=40.0, diff=0.1), ff=128),
    _layer("delta", _delta(4, 4, 64, 32, 3), ff=None),
], loop=(0, 2, 3), scale=8.0, cap=20.0)
# sizes that are multiples of nothing useful, no loop, no cap
ODD = _model(97, 70, 3e-5, [
    _layer("attention", _attn(3, 1, 10, 14, 7, 6, base=77.0), ff=50),
    _layer("delta", _delta(6, 3, 5, 9, 3), ff=None),
    _layer("attention", _attn(5, 5, 20, 12, 13, 20), ff=46, limit=3.0),
    _layer("delta", _delta(2, 1, 7, 11, 5), ff=18),
], scale=1.0)
CONFIGS = {"odd": ODD, "attention": ONLY_ATTENTION, "delta": ONLY_DELTA, "mlp": ONLY_MLP, "loop": ONLY_LOOP,
           "mixed_a": MIXED_A, "mixed_b": MIXED_B}
PAGE_SIZE = {"odd": 4, "attention": 8, "delta": 16, "mlp": 4, "loop": 16, "mixed_a": 8, "mixed_b": 16}


def _tensors(cfg, seed):
    """{name: float32 array}, from a numpy generator; rounded to bfloat16 when written."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    out = {}

    def lin(name, n_out, n_in, gain=1.0):
        out[name] = (rng.standard_normal((n_out, n_in)) * gain / math.sqrt(n_in)).astype(np.float32)

    def vec(name, n, mean=0.0, std=1.0):
        out[name] = (mean + std * rng.standard_normal(n)).astype(np.float32)

    out["embed"] = (rng.standard_normal((cfg["vocab"], W)) / cfg["embedding"]["scale"]).astype(np.float32)
    if cfg.get("loop"):
        out["loop.step"] = (0.5 * rng.standard_normal((cfg["loop"]["times"], W))).astype(np.float32)
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        vec(p + "norm1", W, 1.0, 0.1)
        vec(p + "norm1b", W, 1.0, 0.2)
        H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        if layer["type"] == "attention":
            lin(p + "mix.q", H * 2 * dk, W); lin(p + "mix.k", G * 2 * dk, W); lin(p + "mix.v", G * dv, W)
            # normed queries and keys have entries of order (norm weight); scores of standard deviation about 2.5
            g = (2.5 / (mx["scale"] * math.sqrt(dk))) ** 0.5
            vec(p + "mix.q.norm", dk, g, 0.2 * g); vec(p + "mix.k.norm", dk, g, 0.2 * g)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                vec(p + "mix." + n, dk, 0.0, 0.25)
            lin(p + "mix.g", H, W, 2.0)
            lin(p + "mix.o", W, H * dv)
        else:
            K = mx["conv"]
            lin(p + "mix.q", G * dk, W); lin(p + "mix.k", G * dk, W); lin(p + "mix.v", H * dv, W)
            for n, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out[p + f"mix.{n}.conv"] = (rng.standard_normal((c, K)) * 0.6).astype(np.float32)
            lin(p + "mix.b", H, W, 2.0)
            lin(p + "mix.a", H, W)
            out[p + "mix.dt_bias"] = rng.uniform(-5.0, -1.0, H).astype(np.float32)     # decays of 0.97 to 0.999 a token
            out[p + "mix.A_log"] = np.log(rng.uniform(0.3, 4.0, H)).astype(np.float32)
            vec(p + "mix.norm", dv, 1.0, 0.1)
            lin(p + "mix.g", H * dv, W, 2.0)
            lin(p + "mix.o", W, H * dv)
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            vec(p + "norm2", W, 1.0, 0.1)
            vec(p + "norm2b", W, 1.0, 0.2)
            lim = layer["mlp"]["limit"]
            lin(p + "mlp.gate", F, W, 1.2 * lim); lin(p + "mlp.up", F, W, 1.2 * lim); lin(p + "mlp.down", W, F)
            vec(p + "mlp.gate.b", F, 0.0, 0.3 * lim); vec(p + "mlp.up.b", F, 0.0, 0.3 * lim); vec(p + "mlp.down.b", W, 0.0, 0.3)
    vec("final.norm", W, 1.0, 0.1)
    lin("head", cfg["vocab"], W, 3.0)
    return out


def write_folder(folder, cfg, seed, change=None):
    """A model folder with the weights above in bfloat16. ``change(tensors)`` may edit the float32 arrays first (a test
    that builds a key which stands out, say)."""
    from llm_steadyinfer_b200.weights import write_safetensors
    os.makedirs(folder, exist_ok=True)
    arrays = _tensors(cfg, seed)
    if change is not None:
        change(arrays)
    tensors = {n: torch.from_numpy(a).to(torch.bfloat16) for n, a in arrays.items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1)
    return folder
