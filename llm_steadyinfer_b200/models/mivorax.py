"""Mivorax: a decoder whose layers are listed one by one in config.json, each with one of three mixers (attention
with a learned bias by distance, latent attention with a softmax sink, a state-space mixer) and a dense
feed-forward or none; a layer may run with another layer's weights and a cache or state of its own; the
embedding adds a hashed embedding of the (previous, current) token pair.

config.json:
    architecture  "Mivorax"
    vocab, width  sizes of the embedding and of the residual stream
    norm.eps      of every RMS norm
    embedding.bigram {buckets, mul_prev, mul_cur}   the pair table (absent: the plain embedding)
    layers[i]     {type, mixer{...}, mlp{kind: "dense", ff} | null, weights_of: j (optional)}
      type "attention":        mixer {heads, kv_heads, dim, vdim, scale, bias_max [, bias_buckets]}
      type "latent_attention": mixer {heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot{base, dims}}
      type "mamba2":           mixer {heads, vdim, state, groups, conv, norm_groups}
Tensors: embed, bigram, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.up, l<i>.mlp.down, final.norm, head; a layer
with ``weights_of`` has none. The bias table's row count is the tensor's (``bias_buckets``, which this package
writes into the configurations of its random models, only fixes it ahead of a checkpoint).

Everything is expressed with registered parts: the model below is a ``ModelSpec`` and nothing else.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.base import (ConfigError, EmbedderSpec, FeedForwardSpec, LayerSpec, MixerSpec, ModelConfig, ModelSpec,
                           NormSpec, read_key, register_architecture)

MIXER_KEYS = {
    "attention": (("heads", int), ("kv_heads", int), ("dim", int), ("vdim", int), ("scale", float), ("bias_max", float)),
    "latent_attention": (("heads", int), ("dim", int), ("rot_dim", int), ("vdim", int), ("q_rank", int),
                         ("kv_rank", int), ("scale", float)),
    "mamba2": (("heads", int), ("vdim", int), ("state", int), ("groups", int), ("conv", int), ("norm_groups", int)),
}


def _sub(d: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = d.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


@dataclass(frozen=True)
class MivoraxConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    bigram: Optional[Tuple[int, int, int]]          # buckets, mul_prev, mul_cur
    layers: Tuple[Dict[str, Any], ...]              # as in config.json, checked

    architecture = "Mivorax"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MivoraxConfig":
        vocab = read_key(d, "vocab", int, positive=True)
        width = read_key(d, "width", int, positive=True)
        eps = read_key(_sub(d, "norm", ""), "eps", float, positive=True)
        bigram = None
        emb = _sub(d, "embedding", "", optional=True)
        if emb is not None and emb.get("bigram") is not None:
            b = _sub(emb, "bigram", "embedding.")
            bigram = (read_key(b, "buckets", int, positive=True), read_key(b, "mul_prev", int), read_key(b, "mul_cur", int))
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers: List[Dict[str, Any]] = []
        for i, ent in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(ent, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = read_key(ent, "type", str)
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where}type {kind!r} is not one of {sorted(MIXER_KEYS)}")
            mx = _sub(ent, "mixer", where)
            for key, typ in MIXER_KEYS[kind]:
                try:
                    read_key(mx, key, typ, positive=True)
                except ConfigError as e:
                    raise ConfigError(str(e).replace("key ", f"key {where}mixer.", 1)) from None
            if kind == "latent_attention":
                rot = _sub(mx, "rot", where + "mixer.")
                read_key(rot, "base", float, positive=True)
                if read_key(rot, "dims", int) > mx["rot_dim"] or rot["dims"] % 2 or rot["dims"] < 0:
                    raise ConfigError(f"config.json: {where}mixer.rot.dims must be even and at most rot_dim")
            if kind == "attention":
                if mx["heads"] % mx["kv_heads"]:
                    raise ConfigError(f"config.json: {where}mixer.heads is not a multiple of kv_heads")
                if mx.get("bias_buckets") is not None:
                    read_key(mx, "bias_buckets", int, positive=True)
            if kind == "mamba2" and (mx["heads"] % mx["groups"] or (mx["heads"] * mx["vdim"]) % mx["norm_groups"]):
                raise ConfigError(f"config.json: {where}mixer: heads must be a multiple of groups and heads * vdim "
                                  f"of norm_groups")
            mlp = ent.get("mlp")
            if mlp is not None:
                mlp = _sub(ent, "mlp", where)
                if read_key(mlp, "kind", str) != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp['kind']!r} is not supported (supported: 'dense')")
                read_key(mlp, "ff", int, positive=True)
            src = ent.get("weights_of")
            if src is not None:
                if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < len(raw) or src == i:
                    raise ConfigError(f"config.json: {where}weights_of must name another layer")
            layers.append(copy.deepcopy(ent))
        for i, ent in enumerate(layers):
            src = ent.get("weights_of")
            if src is None:
                continue
            if layers[src].get("weights_of") is not None:
                raise ConfigError(f"config.json: layers[{i}].weights_of names layer {src}, which has no weights of its own")
            same = all(layers[src].get(k) == ent.get(k) for k in ("type", "mixer", "mlp"))
            if not same:
                raise ConfigError(f"config.json: layers[{i}] runs with the weights of layer {src} but differs from it")
        return cls(vocab=vocab, width=width, eps=eps, bigram=bigram, layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.bigram is not None:
            d["embedding"] = {"bigram": {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}}
        return d

    def eos_token_ids(self) -> List[int]:
        return []

    # ---- the model as data ---------------------------------------------------------------------
    def _mixer(self, kind: str, mx: Dict[str, Any]) -> MixerSpec:
        if kind == "attention":
            return MixerSpec("attention", {
                "hidden_size": self.width, "num_heads": mx["heads"], "num_kv_heads": mx["kv_heads"],
                "head_dim": mx["dim"], "value_dim": mx["vdim"], "scale": float(mx["scale"]), "window": None,
                "distance_bias": {"max_distance": float(mx["bias_max"]), "buckets": mx.get("bias_buckets"), "name": "rel"},
                "names": {"q": "q", "k": "k", "v": "v", "o": "o"}})
        if kind == "latent_attention":
            return MixerSpec("latent_attention", {
                "hidden_size": self.width, "num_heads": mx["heads"], "head_dim": mx["dim"], "rot_dim": mx["rot_dim"],
                "value_dim": mx["vdim"], "q_rank": mx["q_rank"], "kv_rank": mx["kv_rank"], "scale": float(mx["scale"]),
                "rot_base": float(mx["rot"]["base"]), "rot_dims": mx["rot"]["dims"], "eps": self.eps, "sink": True})
        return MixerSpec("state_space", {
            "hidden_size": self.width, "num_heads": mx["heads"], "head_dim": mx["vdim"], "state_size": mx["state"],
            "groups": mx["groups"], "conv_taps": mx["conv"], "norm_groups": mx["norm_groups"], "eps": self.eps})

    def model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", {"size": self.width, "eps": self.eps, "weight_name": ""})
        specs: List[LayerSpec] = []
        place: Dict[int, int] = {}                    # config layer -> index among the layers that own weights
        for i, ent in enumerate(self.layers):
            if ent.get("weights_of") is not None:
                continue
            place[i] = len(specs)
            mlp = ent.get("mlp")
            ffn = None if mlp is None else FeedForwardSpec("dense_mlp", {
                "hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "relu2",
                "up_name": "up", "down_name": "down"})
            specs.append(LayerSpec(
                mixer=self._mixer(ent["type"], ent["mixer"]), feed_forward=ffn, mixer_norm=norm,
                feed_forward_norm=None if ffn is None else norm, weight_prefix=f"l{i}.", mixer_prefix="mix.",
                feed_forward_prefix="mlp.", mixer_norm_name="norm1", feed_forward_norm_name="norm2"))
        order = [place[ent["weights_of"] if ent.get("weights_of") is not None else i] for i, ent in enumerate(self.layers)]
        embedder = None
        if self.bigram is not None:
            embedder = EmbedderSpec("table_pair", {"buckets": self.bigram[0], "mul_prev": self.bigram[1],
                                                   "mul_cur": self.bigram[2], "pair_name": "bigram"})
        return ModelSpec(hidden_size=self.width, vocab_size=self.vocab, layers=specs, order=order, final_norm=norm,
                         tie_word_embeddings=False, embed_name="embed", final_norm_name="final.norm",
                         lm_head_name="head", max_position=0, embedder=embedder)


register_architecture(MivoraxConfig.architecture, MivoraxConfig)
