"""Nufasun: a decoder whose config.json lists its layers one by one, each with a differential-attention mixer
(sliding window, query/key norm, partial rotation in neighbouring pairs, a soft limit on the scores, a gate per head)
or a gated-delta-rule mixer (short convolutions, a matrix state per head), a norm before and behind each sublayer, and
a gated feed-forward with limits and biases. A span of the layers may run several times in a row with the same
weights and a cache or state of its own per pass.

config.json:
    architecture    "Nufasun"
    vocab, width    sizes of the embedding and of the residual stream
    norm.eps        of every RMS norm
    embedding.scale the embedding's rows are multiplied by it
    logit_softcap   logits <- cap * tanh(logits / cap)   (absent or 0: none)
    layers[i]       {type, mixer{...}, mlp{kind: "dense", ff, limit} | null}
      type "attention": mixer {heads, kv_heads, dim, vdim, scale, softcap, diff, mask{size}, rot{base, dims}}
      type "delta":     mixer {heads, kv_heads, dim, vdim, conv}
    loop            {start, stop, times}: layers start .. stop-1 run ``times`` times before the rest follow. Before each
                    pass but the first the embedding's output joins the stream again; before every pass row t of
                    ``loop.step`` ([times, width]) does (absent: every layer once, no such tensor).
Tensors: embed, loop.step, l<i>.norm1, l<i>.norm1b, l<i>.norm2, l<i>.norm2b, l<i>.mix.*, l<i>.mlp.{gate,up,down}[.b],
final.norm, head.

Everything is expressed with registered parts: the model below is a ``ModelSpec`` and nothing else.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.base import (ConfigError, EmbedderSpec, FeedForwardSpec, LayerSpec, MixerSpec, ModelConfig, ModelSpec,
                           NormSpec, PositionSpec, StreamAddSpec, read_key, register_architecture)

MIXER_KEYS = {
    "attention": (("heads", int), ("kv_heads", int), ("dim", int), ("vdim", int), ("scale", float)),
    "delta": (("heads", int), ("kv_heads", int), ("dim", int), ("vdim", int), ("conv", int)),
}


def _sub(d: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = d.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


def _keyed(fn, where: str):
    try:
        return fn()
    except ConfigError as e:
        raise ConfigError(str(e).replace("key ", f"key {where}", 1)) from None


@dataclass(frozen=True)
class NufasunConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_softcap: float
    loop: Optional[Tuple[int, int, int]]            # start, stop, times
    layers: Tuple[Dict[str, Any], ...]              # as in config.json, checked

    architecture = "Nufasun"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "NufasunConfig":
        vocab = read_key(d, "vocab", int, positive=True)
        width = read_key(d, "width", int, positive=True)
        eps = _keyed(lambda: read_key(_sub(d, "norm", ""), "eps", float, positive=True), "norm.")
        emb = _sub(d, "embedding", "", optional=True)
        scale = 1.0 if emb is None else _keyed(lambda: read_key(emb, "scale", float, 1.0), "embedding.")
        cap = read_key(d, "logit_softcap", float, 0.0)
        if cap < 0:
            raise ConfigError(f"config.json: key 'logit_softcap' must not be negative, found {cap!r}")
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
                _keyed(lambda: read_key(mx, key, typ, positive=True), where + "mixer.")
            if mx["heads"] % mx["kv_heads"]:
                raise ConfigError(f"config.json: {where}mixer.heads is not a multiple of kv_heads")
            if kind == "attention":
                _keyed(lambda: read_key(mx, "softcap", float, 0.0), where + "mixer.")
                _keyed(lambda: read_key(mx, "diff", float), where + "mixer.")
                mask = _sub(mx, "mask", where + "mixer.", optional=True)
                if mask is not None:
                    _keyed(lambda: read_key(mask, "size", int, positive=True), where + "mixer.mask.")
                rot = _sub(mx, "rot", where + "mixer.", optional=True)
                if rot is not None:
                    _keyed(lambda: read_key(rot, "base", float, positive=True), where + "mixer.rot.")
                    dims = _keyed(lambda: read_key(rot, "dims", int), where + "mixer.rot.")
                    if dims < 0 or dims % 2 or dims > mx["dim"]:
                        raise ConfigError(f"config.json: {where}mixer.rot.dims must be even and at most dim")
            mlp = ent.get("mlp")
            if mlp is not None:
                mlp = _sub(ent, "mlp", where)
                if _keyed(lambda: read_key(mlp, "kind", str), where + "mlp.") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp['kind']!r} is not supported (supported: 'dense')")
                _keyed(lambda: read_key(mlp, "ff", int, positive=True), where + "mlp.")
                _keyed(lambda: read_key(mlp, "limit", float, positive=True), where + "mlp.")
            layers.append(copy.deepcopy(ent))
        loop = None
        lp = _sub(d, "loop", "", optional=True)
        if lp is not None:
            a = _keyed(lambda: read_key(lp, "start", int), "loop.")
            b = _keyed(lambda: read_key(lp, "stop", int), "loop.")
            times = _keyed(lambda: read_key(lp, "times", int, positive=True), "loop.")
            if not 0 <= a < b <= len(layers):
                raise ConfigError(f"config.json: loop.start and loop.stop must name a span of the {len(layers)} layers")
            loop = (a, b, times)
        return cls(vocab=vocab, width=width, eps=eps, embedding_scale=scale, logit_softcap=cap, loop=loop,
                   layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
                             "logit_softcap": self.logit_softcap, "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d

    def eos_token_ids(self) -> List[int]:
        return []

    # ---- the model as data ---------------------------------------------------------------------
    def _mixer(self, kind: str, mx: Dict[str, Any]) -> MixerSpec:
        if kind == "attention":
            rot = mx.get("rot")
            position = None
            if rot is not None and rot["dims"] > 0:
                position = PositionSpec("rotary", {"head_dim": mx["dim"], "rot_dim": rot["dims"], "theta": float(rot["base"])})
            mask = mx.get("mask")
            return MixerSpec("diff_attention", {
                "hidden_size": self.width, "num_heads": mx["heads"], "num_kv_heads": mx["kv_heads"], "head_dim": mx["dim"],
                "value_dim": mx["vdim"], "scale": float(mx["scale"]), "softcap": float(mx.get("softcap") or 0.0),
                "window": None if mask is None else mask["size"], "diff": float(mx["diff"]), "eps": self.eps,
                "gate": True, "rot_interleaved": True}, position)
        return MixerSpec("gated_delta", {
            "hidden_size": self.width, "num_heads": mx["heads"], "num_kv_heads": mx["kv_heads"], "head_dim": mx["dim"],
            "value_dim": mx["vdim"], "conv_taps": mx["conv"], "eps": self.eps})

    def run_order(self) -> List[Tuple[int, Optional[int]]]:
        """(layer, pass number if it is the first layer of a pass, else None) in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop
        order: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(a)]
        for t in range(times):
            order += [(i, t if i == a else None) for i in range(a, b)]
        return order + [(i, None) for i in range(b, n)]

    def model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", {"size": self.width, "eps": self.eps, "weight_name": ""})
        specs: List[LayerSpec] = []
        for i, ent in enumerate(self.layers):
            mlp = ent.get("mlp")
            ffn = None if mlp is None else FeedForwardSpec("gated_mlp_limited", {
                "hidden_size": self.width, "intermediate_size": mlp["ff"], "limit": float(mlp["limit"]), "alpha": 1.702,
                "names": {"gate": "gate", "up": "up", "down": "down"}, "bias_suffix": ".b"})
            specs.append(LayerSpec(
                mixer=self._mixer(ent["type"], ent["mixer"]), feed_forward=ffn, mixer_norm=norm,
                feed_forward_norm=None if ffn is None else norm, weight_prefix=f"l{i}.", arrangement="sandwich",
                mixer_prefix="mix.", feed_forward_prefix="mlp.", mixer_norm_name="norm1", feed_forward_norm_name="norm2",
                mixer_post_norm=norm, feed_forward_post_norm=None if ffn is None else norm,
                mixer_post_norm_name="norm1b", feed_forward_post_norm_name="norm2b"))
        run = self.run_order()
        adds = tuple(StreamAddSpec(place=o, embedding=t > 0, vector_name="loop.step", row=t)
                     for o, (_, t) in enumerate(run) if t is not None)
        return ModelSpec(hidden_size=self.width, vocab_size=self.vocab, layers=specs, order=[i for i, _ in run],
                         final_norm=norm, tie_word_embeddings=False, embed_name="embed", final_norm_name="final.norm",
                         lm_head_name="head", max_position=0,
                         embedder=EmbedderSpec("table", {"scale": self.embedding_scale}),
                         stream_adds=adds,
                         stream_vector_shapes={"loop.step": (self.loop[2], self.width)} if self.loop is not None else None,
                         logit_softcap=self.logit_softcap)


register_architecture(NufasunConfig.architecture, NufasunConfig)
