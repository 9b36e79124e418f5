"""Small Mivorax configurations for the tests and a writer of model folders whose weights make every mechanism
count: queries and keys large enough for peaked attention, bias tables and sinks of order one, step sizes that let
the recurrent state live for hundreds of tokens, convolutions with weight on every tap. The sizes differ from
layer to layer and avoid coincidences (key size != value size, groups != norm groups, more than one key/value
head, rotated part larger than what is rotated, ...).
"""
import json
import math
import os

import numpy as np
import torch


def _attn(heads, kv, dim, vdim, bias_max, buckets, scale=None):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "bias_max": bias_max, "bias_buckets": buckets,
            "scale": scale if scale is not None else dim ** -0.5}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, base=10000.0, dims=None, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "rot": {"base": base, "dims": rot_dim if dims is None else dims},
            "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _layer(kind, mixer, ff=None, weights_of=None):
    d = {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def _model(vocab, width, eps, bigram, layers):
    d = {"architecture": "Mivorax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if bigram is not None:
        d["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return d


# one mixer each: the mechanism alone between embedding and head
ONLY_ATTENTION = _model(200, 64, 1e-5, None, [_layer("attention", _attn(6, 2, 16, 24, 40.0, 12), ff=None)])
ONLY_LATENT = _model(200, 64, 1e-5, None, [_layer("latent_attention", _latent(3, 24, 16, 40, 48, 56, dims=8), ff=None)])
ONLY_SSM = _model(200, 64, 1e-5, None, [_layer("mamba2", _ssm(6, 8, 20, 3, 3, 1), ff=None)])
ONLY_PAIR_MLP = _model(200, 64, 1e-6, (97, 31, 7), [_layer("attention", _attn(2, 1, 8, 8, 9.0, 6), ff=96)])

# all of it, every layer different; layer 5 runs layer 1's weights, layer 6 layer 2's
MIXED_A = _model(331, 96, 1e-5, (211, 13, 101), [
    _layer("mamba2", _ssm(4, 24, 16, 2, 4, 4), ff=160),
    _layer("attention", _attn(4, 2, 32, 16, 100.0, 16), ff=None),
    _layer("latent_attention", _latent(2, 32, 32, 24, 40, 96, base=50000.0), ff=128),
    _layer("attention", _attn(3, 3, 16, 32, 17.5, 10, scale=0.3), ff=64),
    _layer("mamba2", _ssm(3, 32, 8, 1, 2, 3), ff=None),
    _layer("attention", _attn(4, 2, 32, 16, 100.0, 16), ff=None, weights_of=1),
    _layer("latent_attention", _latent(2, 32, 32, 24, 40, 96, base=50000.0), ff=128, weights_of=2),
])
# the layout the bf16 tensor-core kernels take (sizes in multiples of 16), more heads, wider
MIXED_B = _model(500, 256, 2e-6, (509, 3, 1000003), [
    _layer("latent_attention", _latent(8, 64, 32, 64, 96, 128, base=250.0), ff=384),
    _layer("attention", _attn(8, 2, 64, 32, 300.0, 32), ff=384),
    _layer("mamba2", _ssm(8, 32, 64, 2, 4, 2), ff=None),
    _layer("mamba2", _ssm(8, 32, 64, 2, 4, 2), ff=None, weights_of=2),
    _layer("attention", _attn(4, 1, 48, 80, 64.0, 8), ff=128),
])
# sizes that are multiples of nothing useful: every kernel's general route (no 16-byte rows, no tensor-core tiles)
ODD = _model(97, 70, 3e-5, (89, 5, 3), [
    _layer("latent_attention", _latent(3, 12, 10, 14, 26, 36, base=77.0, dims=6), ff=50),
    _layer("mamba2", _ssm(6, 5, 10, 3, 3, 2), ff=None),
    _layer("attention", _attn(5, 5, 20, 12, 33.0, 14), ff=46),
    _layer("mamba2", _ssm(2, 9, 7, 1, 5, 3), ff=18),
    _layer("attention", _attn(6, 2, 7, 9, 21.5, 6), ff=None),
])
CONFIGS = {"odd": ODD, "attention": ONLY_ATTENTION, "latent": ONLY_LATENT, "ssm": ONLY_SSM, "pair_mlp": ONLY_PAIR_MLP,
           "mixed_a": MIXED_A, "mixed_b": MIXED_B}
PAGE_SIZE = {"odd": 4, "attention": 8, "latent": 16, "ssm": 16, "pair_mlp": 4, "mixed_a": 8, "mixed_b": 16}


def _tensors(cfg, seed):
    """{name: float32 array}, from a numpy generator; rounded to bfloat16 when written."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    out = {}

    def lin(name, n_out, n_in, gain=1.0):
        out[name] = (rng.standard_normal((n_out, n_in)) * gain / math.sqrt(n_in)).astype(np.float32)

    def vec(name, n, mean=0.0, std=1.0):
        out[name] = (mean + std * rng.standard_normal(n)).astype(np.float32)

    out["embed"] = rng.standard_normal((cfg["vocab"], W)).astype(np.float32)
    big = cfg.get("embedding", {}).get("bigram")
    if big:
        out["bigram"] = rng.standard_normal((big["buckets"] + 1, W)).astype(np.float32)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, mx = f"l{i}.", layer["mixer"]
        vec(p + "norm1", W, 1.0, 0.1)
        if layer["type"] == "attention":
            H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            g = (2.0 / (mx["scale"] * math.sqrt(dk))) ** 0.5           # scores of standard deviation about 2
            lin(p + "mix.q", H * dk, W, g); lin(p + "mix.k", G * dk, W, g); lin(p + "mix.v", G * dv, W)
            lin(p + "mix.o", W, H * dv)
            out[p + "mix.rel"] = (1.5 * rng.standard_normal((mx["bias_buckets"], H))).astype(np.float32)
        elif layer["type"] == "latent_attention":
            H, dk, dr, dv, rq, rk = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["q_rank"], mx["kv_rank"]
            g = (2.0 / (mx["scale"] * math.sqrt(dk + dr))) ** 0.5
            lin(p + "mix.dq", rq, W); vec(p + "mix.dq.norm", rq, 1.0, 0.1)
            lin(p + "mix.uq", H * (dk + dr), rq, g)
            lin(p + "mix.dkv", rk + dr, W, 1.0); vec(p + "mix.dkv.norm", rk, 1.0, 0.1)
            out[p + "mix.dkv"][rk:] *= g                               # the shared rotated key part, unnormed
            lin(p + "mix.uk", H * dk, rk, g); lin(p + "mix.uv", H * dv, rk)
            vec(p + "mix.sink", H, 0.0, 2.0)
            lin(p + "mix.o", W, H * dv)
        else:
            h, P, N, G, K = mx["heads"], mx["vdim"], mx["state"], mx["groups"], mx["conv"]
            inner, C = h * P, h * P + 2 * G * N
            lin(p + "mix.in", 2 * inner + 2 * G * N + h, W)
            out[p + "mix.conv"] = (rng.standard_normal((C, K)) * 0.6).astype(np.float32)
            vec(p + "mix.conv.b", C, 0.0, 0.2)
            out[p + "mix.dt_bias"] = rng.uniform(-5.0, -1.0, h).astype(np.float32)     # steps of 0.007 to 0.3
            out[p + "mix.A_log"] = np.log(rng.uniform(0.3, 4.0, h)).astype(np.float32)
            vec(p + "mix.D", h, 1.0, 0.5)
            vec(p + "mix.norm", inner, 1.0, 0.1)
            lin(p + "mix.o", W, inner)
        if layer.get("mlp") is not None:
            vec(p + "norm2", W, 1.0, 0.1)
            lin(p + "mlp.up", layer["mlp"]["ff"], W); lin(p + "mlp.down", W, layer["mlp"]["ff"])
    vec("final.norm", W, 1.0, 0.1)
    lin("head", cfg["vocab"], W)
    return out


def write_folder(folder, cfg, seed, drop_bias_buckets=False):
    """A model folder with the weights above in bfloat16. ``drop_bias_buckets``: config.json is written without the
    bias tables' row counts, as a checkpoint from elsewhere comes (the tensor's shape then says it)."""
    from llm_steadyinfer_b200.weights import write_safetensors
    os.makedirs(folder, exist_ok=True)
    tensors = {n: torch.from_numpy(a).to(torch.bfloat16) for n, a in _tensors(cfg, seed).items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
    cfg = json.loads(json.dumps(cfg))
    if drop_bias_buckets:
        for layer in cfg["layers"]:
            layer["mixer"].pop("bias_buckets", None)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1)
    return folder
