"""Typed configuration of Gukosun: a decoder whose layers run mixer and feed-forward side by side on one
norm's output, scale each result per channel, and add a token-indexed side input behind them.

``config.json`` keys: ``architecture`` ("Gukosun"), ``vocab``, ``width``, ``norm.eps``, ``logit_scale``
(1 when absent), ``token_side.dim`` (absent or 0: no side input) and ``layers``, a list whose entries
give ``type`` ("attention" | "parallel"), ``mixer`` (its sizes and constants) and ``mlp`` (a feed-forward,
or null).

* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (a sliding window;
  absent: every earlier key), ``v_mix`` (true: the layer takes part in the mixing of values between
  layers; the first such layer is the source), optionally ``rot`` and ``softcap``.  Its q/k norm is per
  head, its output gate per channel.
* ``parallel``: ``left`` -- ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``softcap``, ``rot``
  (``base``, ``dims``, ``scaling`` = ``factor``, ``low``, ``high``, ``original``), optionally ``mask.size``;
  its q/k norm goes over the whole projection, its output gate is one number per head -- and ``right`` --
  ``heads``, ``dim``, ``vdim``, ``decay`` (one number per head).
* ``mlp``: ``{"kind": "dense", "ff": F}`` (the square of relu between the two products).

Tensor names: ``embed``, ``head``, ``final.norm``, ``side.embed``; layer i: ``l<i>.norm1``, ``ls1``, ``ls2``,
``side.{gate,proj,norm}``, ``mlp.{up,down}``; ``mix.{q,k,v,q.norm,k.norm,vmix,sink,g,o}`` for attention;
``mix.left.{q,k,v,q.norm,k.norm,sink,g,o,out}`` and ``mix.right.{q,k,v,g,norm,o,out}`` for the pair.
The file states no context limit: the engine's page pool is the only one.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping, Tuple

from .lfm2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

UNBOUNDED_POSITIONS = 1 << 24
VALUE_MIX_KEY = "values of the first mixing layer"


def _need(mapping: Any, keys, where: str) -> None:
    if not isinstance(mapping, Mapping):
        raise ConfigError(f"Gukosun config.json: {where} must be an object")
    missing = [key for key in keys if mapping.get(key) is None]
    if missing:
        raise ConfigError(f"Gukosun config.json: {where} is missing " + ", ".join(missing))


def _positive(mapping: Mapping[str, Any], keys, where: str) -> None:
    for key in keys:
        if int(mapping[key]) <= 0:
            raise ConfigError(f"Gukosun config.json: {where}: {key} must be positive")


def _check_softmax_attention(mixer, where: str) -> None:
    _need(mixer, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
    _positive(mixer, ("heads", "kv_heads", "dim", "vdim"), where)
    if int(mixer["heads"]) % int(mixer["kv_heads"]):
        raise ConfigError(f"Gukosun config.json: {where}: heads must be a multiple of kv_heads")
    rot = mixer.get("rot")
    if rot is not None:
        _need(rot, ("base", "dims"), f"{where}.rot")
        if int(rot["dims"]) % 2 or not 0 <= int(rot["dims"]) <= int(mixer["dim"]):
            raise ConfigError(f"Gukosun config.json: {where}: rot.dims must be even and at most dim")
        if rot.get("scaling") is not None:
            _need(rot["scaling"], ("factor", "low", "high", "original"), f"{where}.rot.scaling")
    mask = mixer.get("mask")
    if mask is not None:
        _need(mask, ("size",), f"{where}.mask")
        _positive(mask, ("size",), f"{where}.mask")
    if float(mixer.get("softcap") or 0.0) < 0:
        raise ConfigError(f"Gukosun config.json: {where}: softcap must not be negative")


@dataclass(frozen=True)
class GukosunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]          # as config.json gives them, checked
    logit_scale: float = 1.0
    side_dim: int = 0
    architectures: Tuple[str, ...] = ("Gukosun",)
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------------ reading / writing
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "GukosunConfig":
        _need(raw, ("vocab", "width", "norm", "layers"), "the top level")
        _need(raw["norm"], ("eps",), "'norm'")
        _positive(raw, ("vocab", "width"), "the top level")
        if not isinstance(raw["layers"], (list, tuple)) or not raw["layers"]:
            raise ConfigError("Gukosun config.json: 'layers' must be a list with at least one layer")
        layers = []
        mixed_values = None
        for index, layer in enumerate(raw["layers"]):
            where = f"layer {index}"
            _need(layer, ("type", "mixer"), where)
            layer = copy.deepcopy(dict(layer))
            mixer = layer["mixer"]
            if layer["type"] == "attention":
                _check_softmax_attention(mixer, f"{where}'s mixer")
                if mixer.get("v_mix"):
                    shape = (int(mixer["kv_heads"]), int(mixer["vdim"]), int(mixer["dim"]))
                    if mixed_values is None:
                        mixed_values = shape
                    elif shape != mixed_values:
                        raise ConfigError(f"Gukosun config.json: {where} mixes values of {shape[0]} heads of "
                                          f"{shape[1]} (keys of {shape[2]}), the first such layer has "
                                          f"{mixed_values[0]} of {mixed_values[1]} (keys of {mixed_values[2]})")
            elif layer["type"] == "parallel":
                _need(mixer, ("left", "right"), f"{where}'s mixer")
                _check_softmax_attention(mixer["left"], f"{where}'s mixer.left")
                right = mixer["right"]
                _need(right, ("heads", "dim", "vdim", "decay"), f"{where}'s mixer.right")
                _positive(right, ("heads", "dim", "vdim"), f"{where}'s mixer.right")
                if len(right["decay"]) != int(right["heads"]):
                    raise ConfigError(f"Gukosun config.json: {where}: one decay per head of the right mixer")
            else:
                raise ConfigError(f"Gukosun config.json: {where} has the unknown type {layer['type']!r} "
                                  "(known: attention, parallel)")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind",), f"{where}'s mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"Gukosun config.json: {where} has the unknown feed-forward "
                                      f"{mlp['kind']!r} (known: dense)")
                _need(mlp, ("ff",), f"{where}'s mlp")
                _positive(mlp, ("ff",), f"{where}'s mlp")
            layers.append(layer)
        side = raw.get("token_side") or {}
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers", "logit_scale", "token_side"}
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   layers=tuple(layers),
                   logit_scale=float(raw["logit_scale"]) if raw.get("logit_scale") is not None else 1.0,
                   side_dim=int(side.get("dim") or 0),
                   extra={k: v for k, v in raw.items() if k not in known})

    def to_dict(self) -> dict:
        out = {"architecture": self.architectures[0], "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
               "layers": copy.deepcopy(list(self.layers))}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        out.update(self.extra)
        return out

    # ------------------------------------------------------------------ the model in parts
    def _softmax_attention(self, m, prefix: str, *, qk_norm: str, gate: str, value_mix) -> PartSpec:
        rot = m.get("rot")
        if rot is not None and int(rot["dims"]) > 0:
            params = {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]), "pairing": "interleaved"}
            if rot.get("scaling") is not None:
                params["scaling"] = {key: float(rot["scaling"][key]) for key in ("factor", "low", "high", "original")}
            position = PartSpec("rope", params)
        else:
            position = PartSpec("no_position")
        tensors = {"q": prefix + "q", "k": prefix + "k", "v": prefix + "v", "o": prefix + "o",
                   "q_norm": prefix + "q.norm", "k_norm": prefix + "k.norm", "sink": prefix + "sink",
                   "g": prefix + "g"}
        if value_mix == "mixed":
            tensors["vmix"] = prefix + "vmix"
        return PartSpec(
            "gqa_attention",
            {"hidden_size": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
             "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "scale": float(m["scale"]),
             "qk_norm_eps": self.norm_eps, "qk_norm": qk_norm, "position": position,
             "window": int((m.get("mask") or {}).get("size") or 0), "sink": True,
             "softcap": float(m.get("softcap") or 0.0), "gate": gate, "value_mix": value_mix,
             "value_mix_key": VALUE_MIX_KEY},
            tensors)

    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": W, "eps": eps}, {"weight": name})

        layers, unused = [], []
        source_seen = False
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}."
            m = layer["mixer"]
            if layer["type"] == "attention":
                role = None
                if m.get("v_mix"):
                    role = "mixed" if source_seen else "source"
                    source_seen = True
                if role != "mixed":
                    unused.append(prefix + "mix.vmix")          # (the source's and a non-mixing layer's are not read)
                mixer = self._softmax_attention(m, prefix + "mix.", qk_norm="head", gate="element", value_mix=role)
            else:
                left = self._softmax_attention(m["left"], prefix + "mix.left.", qk_norm="whole", gate="head",
                                               value_mix=None)
                r = m["right"]
                rp = prefix + "mix.right."
                right = PartSpec(
                    "decayed_linear_attention",
                    {"hidden_size": W, "num_heads": int(r["heads"]), "dim": int(r["dim"]), "vdim": int(r["vdim"]),
                     "decay": tuple(float(x) for x in r["decay"]), "eps": eps},
                    {"q": rp + "q", "k": rp + "k", "v": rp + "v", "g": rp + "g", "norm": rp + "norm", "o": rp + "o"})
                mixer = PartSpec("mixer_pair", {"hidden_size": W, "eps": eps, "left": left, "right": right},
                                 {"left_out": prefix + "mix.left.out", "right_out": prefix + "mix.right.out"})
            parts = {"norm": norm(prefix + "norm1"), "mixer": mixer,
                     "mixer_scale": PartSpec("channel_scale", {"size": W}, {"weight": prefix + "ls1"})}
            mlp = layer.get("mlp")
            if mlp is None:
                unused += [prefix + "ls2"]
            else:
                parts["feed_forward"] = PartSpec(
                    "dense_mlp", {"hidden_size": W, "ffn_dim": int(mlp["ff"]), "activation": "relu_squared"},
                    {"up": prefix + "mlp.up", "down": prefix + "mlp.down"})
                parts["ffn_scale"] = PartSpec("channel_scale", {"size": W}, {"weight": prefix + "ls2"})
            if self.side_dim:
                parts["side"] = PartSpec(
                    "token_side_input",
                    {"hidden_size": W, "vocab_size": self.vocab, "dim": self.side_dim, "index": index,
                     "count": len(self.layers), "eps": eps},
                    {"table": "side.embed", "gate": prefix + "side.gate", "proj": prefix + "side.proj",
                     "norm": prefix + "side.norm"})
            else:
                unused += [prefix + "side.gate", prefix + "side.proj", prefix + "side.norm"]
            layers.append(LayerSpec("parallel_residual", parts=parts))
        if not self.side_dim:
            unused.append("side.embed")
        spec = ModelSpec(
            architecture=self.architectures[0], hidden_size=W, vocab_size=self.vocab,
            max_positions=UNBOUNDED_POSITIONS, embedding_tensor="embed", final_norm=norm("final.norm"),
            head_tensor="head", layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(len(self.layers))),
            logit_scale=self.logit_scale, unused_tensors=tuple(unused))
        spec.validate()
        return spec
