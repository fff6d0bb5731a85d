"""Typed configuration of Fobatar: a decoder whose layers put a weighted RMS norm in front of every sublayer
and another on its output, scale what they add to the stream by one constant, attend either inside chunks
(with short convolutions on q, k and v and a zero sink) or over a cached low-rank latent, choose their
experts by the token's id, and may run a stretch of layers several times over.

``config.json`` keys: ``architecture`` ("Fobatar"), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``residual_mult``, ``loop`` (``start``, ``stop``, ``times``: layers start .. stop-1 run ``times`` times in a
row with the same weights, every pass with a cache of its own, and every pass but the first begins by
adding the embedding's output to the stream; absent: every layer once) and ``layers``, a list whose entries
give ``type`` ("attention" | "latent_attention"), ``mixer`` (its sizes and constants) and ``mlp`` (a
feed-forward, or null).

* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``conv`` (taps of the convolutions
  on q, k, v; absent: none), ``mask.size`` (the chunk length; absent: every earlier key), ``rot`` (``base``,
  ``dims``, ``scaling`` = ``factor``, ``original``, ``fast``, ``slow``; absent: no rotation).  Its q/k norm
  goes over the whole projection, its softmax has a sink of score 0, its output gate is one number per head.
* ``latent_attention``: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``rot`` (as above;
  the turned part is the ``rot_dim`` part).  Plain softmax, a gate per head.
* ``mlp``: ``{"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}, "shared": {"ff",
  "limit"} or absent}``: the experts of a token are a row of an integer table indexed by its id.

Tensor names: ``embed``, ``final.norm``; layer i: ``l<i>.norm1``, ``norm1b``, ``norm2``, ``norm2b``;
``mix.{q,k,v,q.norm,k.norm,q.conv,k.conv,v.conv,g,o}`` for attention; ``mix.{q,dkv,dkv.norm,uk,uv,g,o}`` for
latent attention; ``mlp.table``, ``mlp.e<j>.{gate,up,down}``, ``mlp.shared.{gate,up,down}``.  The head is
the embedding table.  The file states no context limit: the engine's page pool is the only one.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .lfm2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

UNBOUNDED_POSITIONS = 1 << 24
NAME = "Fobatar"


def _need(mapping: Any, keys, where: str) -> None:
    if not isinstance(mapping, Mapping):
        raise ConfigError(f"{NAME} config.json: {where} must be an object")
    missing = [key for key in keys if mapping.get(key) is None]
    if missing:
        raise ConfigError(f"{NAME} config.json: {where} is missing " + ", ".join(missing))


def _positive(mapping: Mapping[str, Any], keys, where: str) -> None:
    for key in keys:
        if not float(mapping[key]) > 0:
            raise ConfigError(f"{NAME} config.json: {where}: {key} must be positive")


def _check_rot(rot, where: str, dims_at_most: int) -> None:
    _need(rot, ("base", "dims"), where)
    if int(rot["dims"]) % 2 or not 0 <= int(rot["dims"]) <= dims_at_most:
        raise ConfigError(f"{NAME} config.json: {where}: dims must be even and at most {dims_at_most}")
    if rot.get("scaling") is not None:
        _need(rot["scaling"], ("factor", "original", "fast", "slow"), f"{where}.scaling")
        _positive(rot["scaling"], ("factor", "original", "fast", "slow"), f"{where}.scaling")


def _rope(rot, dims: int) -> PartSpec:
    if rot is None or dims <= 0:
        return PartSpec("no_position")
    params = {"theta": float(rot["base"]), "rotary_dim": dims, "pairing": "interleaved"}
    if rot.get("scaling") is not None:
        params["scaling"] = {key: float(rot["scaling"][key]) for key in ("factor", "original", "fast", "slow")}
    return PartSpec("rope", params)


@dataclass(frozen=True)
class FobatarConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    layers: Tuple[Mapping[str, Any], ...]          # as config.json gives them, checked
    loop: Optional[Tuple[int, int, int]] = None    # (start, stop, times)
    architectures: Tuple[str, ...] = (NAME,)
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------------ reading / writing
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "FobatarConfig":
        _need(raw, ("vocab", "width", "norm", "layers"), "the top level")
        _need(raw["norm"], ("eps",), "'norm'")
        _positive(raw, ("vocab", "width"), "the top level")
        if not isinstance(raw["layers"], (list, tuple)) or not raw["layers"]:
            raise ConfigError(f"{NAME} config.json: 'layers' must be a list with at least one layer")
        layers = []
        for index, layer in enumerate(raw["layers"]):
            where = f"layer {index}"
            _need(layer, ("type", "mixer"), where)
            layer = copy.deepcopy(dict(layer))
            mixer = layer["mixer"]
            if layer["type"] == "attention":
                _need(mixer, ("heads", "kv_heads", "dim", "vdim", "scale"), f"{where}'s mixer")
                _positive(mixer, ("heads", "kv_heads", "dim", "vdim"), f"{where}'s mixer")
                if int(mixer["heads"]) % int(mixer["kv_heads"]):
                    raise ConfigError(f"{NAME} config.json: {where}: heads must be a multiple of kv_heads")
                if mixer.get("rot") is not None:
                    _check_rot(mixer["rot"], f"{where}'s mixer.rot", int(mixer["dim"]))
                if mixer.get("mask") is not None:
                    _need(mixer["mask"], ("size",), f"{where}'s mixer.mask")
                    _positive(mixer["mask"], ("size",), f"{where}'s mixer.mask")
                if int(mixer.get("conv") or 0) < 0:
                    raise ConfigError(f"{NAME} config.json: {where}: conv must not be negative")
            elif layer["type"] == "latent_attention":
                _need(mixer, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"), f"{where}'s mixer")
                _positive(mixer, ("heads", "dim", "vdim", "kv_rank"), f"{where}'s mixer")
                if int(mixer["rot_dim"]) < 0 or int(mixer["rot_dim"]) % 2:
                    raise ConfigError(f"{NAME} config.json: {where}: rot_dim must be even and not negative")
                _check_rot(mixer["rot"], f"{where}'s mixer.rot", max(int(mixer["rot_dim"]), int(mixer["rot"]["dims"])))
            else:
                raise ConfigError(f"{NAME} config.json: {where} has the unknown type {layer['type']!r} "
                                  "(known: attention, latent_attention)")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind",), f"{where}'s mlp")
                if mlp["kind"] != "moe":
                    raise ConfigError(f"{NAME} config.json: {where} has the unknown feed-forward "
                                      f"{mlp['kind']!r} (known: moe)")
                _need(mlp, ("expert", "router"), f"{where}'s mlp")
                _need(mlp["expert"], ("ff", "limit"), f"{where}'s mlp.expert")
                _need(mlp["router"], ("experts", "top"), f"{where}'s mlp.router")
                _positive(mlp["expert"], ("ff", "limit"), f"{where}'s mlp.expert")
                _positive(mlp["router"], ("experts", "top"), f"{where}'s mlp.router")
                if int(mlp["router"]["top"]) > int(mlp["router"]["experts"]):
                    raise ConfigError(f"{NAME} config.json: {where}: top exceeds the number of experts")
                if mlp.get("shared") is not None:
                    _need(mlp["shared"], ("ff", "limit"), f"{where}'s mlp.shared")
                    _positive(mlp["shared"], ("ff", "limit"), f"{where}'s mlp.shared")
            layers.append(layer)
        loop = raw.get("loop")
        if loop is not None:
            _need(loop, ("start", "stop", "times"), "'loop'")
            start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            if not 0 <= start <= stop <= len(layers) or times < 1:
                raise ConfigError(f"{NAME} config.json: 'loop' must have 0 <= start <= stop <= {len(layers)} and "
                                  "times >= 1")
            loop = (start, stop, times)
        embedding = raw.get("embedding") or {}
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers", "loop", "embedding",
                 "residual_mult"}
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   embedding_scale=float(embedding["scale"]) if embedding.get("scale") is not None else 1.0,
                   residual_mult=float(raw["residual_mult"]) if raw.get("residual_mult") is not None else 1.0,
                   layers=tuple(layers), loop=loop, extra={k: v for k, v in raw.items() if k not in known})

    def to_dict(self) -> dict:
        out = {"architecture": self.architectures[0], "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
               "residual_mult": self.residual_mult, "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        out.update(self.extra)
        return out

    # ------------------------------------------------------------------ the model in parts
    def runs(self):
        """(layer index, adds the embedding's output first) for every execution, in order."""
        n = len(self.layers)
        if self.loop is None or self.loop[1] <= self.loop[0]:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        runs = [(i, False) for i in range(start)]
        for again in range(times):
            runs += [(i, again > 0 and i == start) for i in range(start, stop)]
        return runs + [(i, False) for i in range(stop, n)]

    def _attention(self, m, prefix: str) -> PartSpec:
        rot = m.get("rot")
        tensors = {"q": prefix + "q", "k": prefix + "k", "v": prefix + "v", "o": prefix + "o",
                   "q_norm": prefix + "q.norm", "k_norm": prefix + "k.norm", "g": prefix + "g",
                   "q_conv": prefix + "q.conv", "k_conv": prefix + "k.conv", "v_conv": prefix + "v.conv"}
        return PartSpec(
            "gqa_attention",
            {"hidden_size": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
             "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "scale": float(m["scale"]),
             "qk_norm_eps": self.norm_eps, "qk_norm": "whole",
             "position": _rope(rot, int(rot["dims"]) if rot is not None else 0),
             "chunk": int((m.get("mask") or {}).get("size") or 0), "sink": "zero", "gate": "head",
             "conv": int(m.get("conv") or 0)},
            tensors)

    def _latent(self, m, prefix: str) -> PartSpec:
        return PartSpec(
            "latent_attention",
            {"hidden_size": self.width, "num_heads": int(m["heads"]), "dim": int(m["dim"]),
             "rot_dim": int(m["rot_dim"]), "vdim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]),
             "scale": float(m["scale"]), "eps": self.norm_eps, "sink": False, "gate": "head",
             "position": _rope(m["rot"], int(m["rot_dim"]))},
            {"q": prefix + "q", "dkv": prefix + "dkv", "dkv_norm": prefix + "dkv.norm", "uk": prefix + "uk",
             "uv": prefix + "uv", "o": prefix + "o", "g": prefix + "g"})

    def _experts(self, mlp, prefix: str) -> PartSpec:
        E = int(mlp["router"]["experts"])
        shared = mlp.get("shared")
        params = {"hidden_size": self.width, "vocab_size": self.vocab, "ffn_dim": int(mlp["expert"]["ff"]),
                  "experts": E, "top": int(mlp["router"]["top"]), "activation": "swish_clamped",
                  "limit": float(mlp["expert"]["limit"])}
        tensors = {"table": prefix + "table"}
        for j in range(E):
            for role in ("gate", "up", "down"):
                tensors[f"{role}{j}"] = f"{prefix}e{j}.{role}"
        if shared is not None:
            params.update(shared_ffn_dim=int(shared["ff"]), shared_limit=float(shared["limit"]))
            for role in ("gate", "up", "down"):
                tensors[f"shared_{role}"] = f"{prefix}shared.{role}"
        return PartSpec("table_experts", params, tensors)

    def model_spec(self) -> ModelSpec:
        W, eps, mult = self.width, self.norm_eps, self.residual_mult

        def norm(name: str, gain: float = 1.0) -> PartSpec:
            params = {"size": W, "eps": eps}
            if gain != 1.0:
                params["gain"] = gain
            return PartSpec("rmsnorm", params, {"weight": name})

        layers = []
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}."
            m = layer["mixer"]
            mixer = (self._attention if layer["type"] == "attention" else self._latent)(m, prefix + "mix.")
            # the constant that scales what a sublayer adds rides on the norm behind the sublayer
            parts = {"mixer_norm": norm(prefix + "norm1"), "mixer": mixer,
                     "mixer_out_norm": norm(prefix + "norm1b", mult)}
            if layer.get("mlp") is not None:
                parts["ffn_norm"] = norm(prefix + "norm2")
                parts["feed_forward"] = self._experts(layer["mlp"], prefix + "mlp.")
                parts["ffn_out_norm"] = norm(prefix + "norm2b", mult)
            layers.append(LayerSpec("sandwich_residual", parts=parts))
        spec = ModelSpec(
            architecture=self.architectures[0], hidden_size=W, vocab_size=self.vocab,
            max_positions=UNBOUNDED_POSITIONS, embedding_tensor="embed", final_norm=norm("final.norm"),
            head_tensor=None, layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i, add_embedding=again) for i, again in self.runs()),
            embedding_scale=self.embedding_scale)
        spec.validate()
        return spec
