"""Typed configuration of the Tepavik decoder: a stack of layers that each name their own mixer.

``config.json`` carries ``architecture: "Tepavik"``, ``vocab``, ``width``, ``norm.eps`` and
``layers``, a list with one entry per layer: ``type`` (``attention``, ``lightning`` or
``mamba2``), ``mixer`` (that mixer's sizes and constants) and ``mlp`` (``{"kind": "dense", "ff":
n}``, or null for a layer without a feed-forward).  Every layer is pre-norm with RMS norms whose
stored weight lies around zero (the weight is one plus it).

``attention``: grouped-query softmax attention without a position encoding; queries and keys are
divided by their root mean square per head; scores are multiplied by ``scale`` and capped with
``softcap * tanh(score / softcap)``; ``mask.size`` makes the mask chunked (a token sees the earlier
tokens of its own block of that many positions).  ``kv_from: j`` marks a layer without key/value
projections that reads the pages of layer j.  ``lightning``: linear attention with a decay per
head.  ``mamba2``: a state-space layer.  Checkpoint names are ``embed``, ``l<i>.norm1``,
``l<i>.mix.<name>``, ``l<i>.norm2``, ``l<i>.mlp.up|down``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_ATTENTION_NAMES = {
    "q_proj.weight": "q", "q_proj.bias": "q.b", "k_proj.weight": "k", "k_proj.bias": "k.b",
    "v_proj.weight": "v", "v_proj.bias": "v.b", "o_proj.weight": "o",
}
_LIGHTNING_NAMES = {
    "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g", "o_proj.weight": "o",
    "norm.weight": "norm",
}
_MAMBA2_NAMES = {
    "in_proj.weight": "in", "conv.weight": "conv", "conv.bias": "conv.b", "norm.weight": "norm", "o_proj.weight": "o",
}
_MLP_NAMES = {"up_proj.weight": "up", "down_proj.weight": "down"}


def _positive(where: str, value: Any) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"{where} must be a positive integer, got {value!r}")
    return value


@dataclasses.dataclass(frozen=True)
class TepavikConfig(ModelConfig):
    architecture: ClassVar[str] = "Tepavik"

    vocab: int
    width: int
    layers: list
    norm: dict

    def validate(self) -> None:
        _positive("vocab", self.vocab)
        _positive("width", self.width)
        if not isinstance(self.norm, dict) or not (float(self.norm.get("eps", 0)) > 0):
            raise ConfigError(f"norm.eps must be positive, got {self.norm!r}")
        if not isinstance(self.layers, (list, tuple)) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            kind = layer.get("type")
            mixer = layer.get("mixer")
            if kind not in ("attention", "lightning", "mamba2"):
                raise ConfigError(f"{where}.type must be attention, lightning or mamba2, got {kind!r}")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            required = {
                "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
                "lightning": ("heads", "dim", "vdim", "decay"),
                "mamba2": ("heads", "vdim", "state", "groups", "conv"),
            }[kind]
            missing = [key for key in required if key not in mixer]
            if missing:
                raise ConfigError(f"{where}.mixer lacks {', '.join(missing)}")
            for key in required:
                if key not in ("scale", "decay"):
                    _positive(f"{where}.mixer.{key}", mixer[key])
            if kind == "attention":
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"{where}: {mixer['heads']} heads are not a multiple of {mixer['kv_heads']} kv_heads")
                source = mixer.get("kv_from")
                if source is not None:
                    if not isinstance(source, int) or not 0 <= source < index:
                        raise ConfigError(f"{where}.mixer.kv_from must name an earlier layer, got {source!r}")
                    other = self.layers[source]
                    if other.get("type") != "attention" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}.mixer.kv_from names layer {source}, which has no keys of its own")
                mask = mixer.get("mask")
                if mask is not None:
                    _positive(f"{where}.mixer.mask.size", mask.get("size"))
            elif kind == "lightning":
                decay = mixer["decay"]
                if not isinstance(decay, (list, tuple)) or len(decay) != mixer["heads"]:
                    raise ConfigError(f"{where}.mixer.decay must list one decay per head")
            else:
                if mixer["heads"] % mixer["groups"]:
                    raise ConfigError(f"{where}: {mixer['heads']} heads are not a multiple of {mixer['groups']} groups")
                parts = mixer.get("norm_groups", 1)
                if (mixer["heads"] * mixer["vdim"]) % _positive(f"{where}.mixer.norm_groups", parts):
                    raise ConfigError(f"{where}: the inner width cannot be normalised in {parts} equal parts")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp.kind must be 'dense', got {mlp.get('kind')!r}")
                _positive(f"{where}.mlp.ff", mlp.get("ff"))

    def to_dict(self) -> dict[str, Any]:
        data = {"architecture": self.architecture}
        data.update(dataclasses.asdict(self))
        return data

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    # The part-by-part description --------------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "offset": 1.0, "tensor_names": {"weight": ""}}, name)

    def _mixer(self, kind: str, m: dict, prefix: str) -> PartSpec:
        if kind == "attention":
            shared = m.get("kv_from") is not None
            return PartSpec(
                "attention",
                {
                    "hidden_size": self.width,
                    "num_heads": m["heads"],
                    "num_kv_heads": m["kv_heads"],
                    "head_size": m["dim"],
                    "value_head_size": m["vdim"],
                    "qkv_bias": True,
                    "out_bias": False,
                    "scale": float(m["scale"]),
                    "window": None,
                    "chunk": (m.get("mask") or {}).get("size"),
                    "softcap": m.get("softcap"),
                    "qk_unit_eps": self.eps,
                    "shared_kv": shared,
                    "position": PartSpec("none", {}),
                    "tensor_names": _ATTENTION_NAMES,
                },
                prefix,
            )
        if kind == "lightning":
            return PartSpec(
                "lightning",
                {
                    "hidden_size": self.width,
                    "num_heads": m["heads"],
                    "head_size": m["dim"],
                    "value_head_size": m["vdim"],
                    "decay": tuple(float(d) for d in m["decay"]),
                    "eps": self.eps,
                    "tensor_names": _LIGHTNING_NAMES,
                },
                prefix,
            )
        return PartSpec(
            "mamba2",
            {
                "hidden_size": self.width,
                "num_heads": m["heads"],
                "value_head_size": m["vdim"],
                "state_size": m["state"],
                "num_groups": m["groups"],
                "conv_taps": m["conv"],
                "norm_groups": m.get("norm_groups", 1),
                "eps": self.eps,
                "tensor_names": _MAMBA2_NAMES,
            },
            prefix,
        )

    def model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}."
            parts = {
                "mixer_norm": self._norm(prefix + "norm1"),
                "mixer": self._mixer(layer["type"], layer["mixer"], prefix + "mix."),
            }
            mlp = layer.get("mlp")
            if mlp is not None:
                parts["feed_forward_norm"] = self._norm(prefix + "norm2")
                parts["feed_forward"] = PartSpec(
                    "dense_mlp",
                    {"hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "relu2",
                     "tensor_names": _MLP_NAMES},
                    prefix + "mlp.",
                )
            layers.append(LayerSpec("prenorm" if mlp is not None else "prenorm_mixer", parts))
            source = layer["mixer"].get("kv_from") if layer["type"] == "attention" else None
            schedule.append(ScheduleEntry(index, source))
        return ModelSpec(
            hidden_size=self.width,
            vocab_size=self.vocab,
            embedding=PartSpec(
                "embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "tensor_names": {"weight": "embed"}}, ""
            ),
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=PartSpec(
                "linear_head",
                {"vocab_size": self.vocab, "hidden_size": self.width, "tied_to": None, "tensor_names": {"weight": "head"}},
                "",
            ),
        )
