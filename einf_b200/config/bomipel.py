"""Typed configuration of the Bomipel decoder: parallel layers with routed feed-forwards.

``config.json`` carries ``architecture: "Bomipel"``, ``vocab``, ``width``, ``norm.eps``,
``logit_softcap`` (optional) and ``layers``, a list with one entry per layer: ``type``
(``attention`` or ``latent_attention``), ``mixer`` (that mixer's sizes and constants) and ``mlp``
(``{"kind": "moe", "expert": {"ff": n}, "router": {"experts": E, "top": k}}``, or null for a layer
without a feed-forward).

A layer is parallel: one RMS norm (plain weight) feeds both the mixer and the feed-forward, and the
sum of their outputs is added to the residual stream.  The output matrix is the embedding table;
logits pass ``cap * tanh(logits / cap)``.

``attention``: grouped-query softmax attention; rotary positions on the first ``rot.dims``
dimensions of each head with neighbouring dimensions paired (2i, 2i + 1), frequencies
``rot.base^(-2i/dims)`` optionally rescaled by wavelength (``rot.scaling``: ``factor``, ``low``,
``high``, ``original``); ``mask.size`` keys of sliding window plus the first ``mask.keep_first``
positions of the sequence; ``v_mix``: every such layer after the first blends its values with the
first such layer's, ``(1 - l) v + l v_first`` with the stored scalar ``vmix``.

``latent_attention``: queries through a normed latent of ``q_rank``; keys and values from one
normed latent of ``kv_rank`` per token plus one rotated key part of ``rot_dim`` shared by all heads
(dimension i paired with i + rot_dim / 2); causal.

Checkpoint names are ``embed``, ``l<i>.norm1``, ``l<i>.mix.<name>``, ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.gate|up|down``, ``final.norm``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Optional

from .base import ConfigError, ModelConfig
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_ATTENTION_NAMES = {
    "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o", "value_mix": "vmix",
}
_LATENT_NAMES = {
    "q_down.weight": "dq", "q_norm.weight": "dq.norm", "q_up.weight": "uq", "kv_down.weight": "dkv",
    "kv_norm.weight": "dkv.norm", "k_up.weight": "uk", "v_up.weight": "uv", "o_proj.weight": "o",
}


def _positive(where: str, value: Any) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"{where} must be a positive integer, got {value!r}")
    return value


def _rotation(where: str, rot: Any, most: int) -> None:
    if not isinstance(rot, dict) or "base" not in rot or "dims" not in rot:
        raise ConfigError(f"{where}.rot must give base and dims")
    dims = _positive(f"{where}.rot.dims", rot["dims"])
    if dims % 2 or dims > most:
        raise ConfigError(f"{where}.rot.dims must be even and at most {most}, got {dims}")
    if not float(rot["base"]) > 0:
        raise ConfigError(f"{where}.rot.base must be positive")
    scaling = rot.get("scaling")
    if scaling is not None:
        missing = [key for key in ("factor", "low", "high", "original") if key not in scaling]
        if missing:
            raise ConfigError(f"{where}.rot.scaling lacks {', '.join(missing)}")
        if float(scaling["high"]) == float(scaling["low"]):
            raise ConfigError(f"{where}.rot.scaling: low and high must differ")


@dataclasses.dataclass(frozen=True)
class BomipelConfig(ModelConfig):
    architecture: ClassVar[str] = "Bomipel"

    vocab: int
    width: int
    layers: list
    norm: dict
    logit_softcap: Optional[float] = None

    def validate(self) -> None:
        _positive("vocab", self.vocab)
        _positive("width", self.width)
        if not isinstance(self.norm, dict) or not (float(self.norm.get("eps", 0)) > 0):
            raise ConfigError(f"norm.eps must be positive, got {self.norm!r}")
        if self.logit_softcap is not None and not float(self.logit_softcap) > 0:
            raise ConfigError(f"logit_softcap must be positive, got {self.logit_softcap!r}")
        if not isinstance(self.layers, (list, tuple)) or not self.layers:
            raise ConfigError("layers must be a non-empty list")
        mixed_values = None
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            kind, mixer = layer.get("type"), layer.get("mixer")
            if kind not in ("attention", "latent_attention"):
                raise ConfigError(f"{where}.type must be attention or latent_attention, got {kind!r}")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            required = {
                "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
                "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot"),
            }[kind]
            missing = [key for key in required if key not in mixer]
            if missing:
                raise ConfigError(f"{where}.mixer lacks {', '.join(missing)}")
            for key in required:
                if key not in ("scale", "rot"):
                    _positive(f"{where}.mixer.{key}", mixer[key])
            if kind == "attention":
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"{where}: {mixer['heads']} heads are not a multiple of {mixer['kv_heads']} kv_heads")
                if mixer.get("rot") is not None:
                    _rotation(f"{where}.mixer", mixer["rot"], mixer["dim"])
                mask = mixer.get("mask")
                if mask is not None:
                    _positive(f"{where}.mixer.mask.size", mask.get("size"))
                    keep = mask.get("keep_first", 0)
                    if not isinstance(keep, int) or keep < 0:
                        raise ConfigError(f"{where}.mixer.mask.keep_first must be a count, got {keep!r}")
                if mixer.get("v_mix"):
                    shape = (mixer["kv_heads"], mixer["vdim"])
                    if mixed_values is None:
                        mixed_values = shape
                    elif shape != mixed_values:
                        raise ConfigError(
                            f"{where}: values of {shape} (kv_heads, vdim) cannot be mixed with the first "
                            f"value-mixing layer's {mixed_values}"
                        )
            else:
                _rotation(f"{where}.mixer", mixer["rot"], mixer["rot_dim"])
                if mixer["rot"]["dims"] != mixer["rot_dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims must equal rot_dim")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "moe":
                    raise ConfigError(f"{where}.mlp.kind must be 'moe', got {mlp.get('kind')!r}")
                _positive(f"{where}.mlp.expert.ff", (mlp.get("expert") or {}).get("ff"))
                router = mlp.get("router") or {}
                experts = _positive(f"{where}.mlp.router.experts", router.get("experts"))
                top = _positive(f"{where}.mlp.router.top", router.get("top"))
                if top > experts:
                    raise ConfigError(f"{where}.mlp.router: top {top} exceeds {experts} experts")

    def to_dict(self) -> dict[str, Any]:
        data = {"architecture": self.architecture}
        data.update(dataclasses.asdict(self))
        return data

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def init_std(self) -> float:
        # random matrices that keep activations of order one, so that scores spread
        return float(self.width) ** -0.5

    # The part-by-part description --------------------------------------
    def _norm(self, name: str, size: Optional[int] = None) -> PartSpec:
        return PartSpec("rmsnorm", {"size": size or self.width, "eps": self.eps, "tensor_names": {"weight": ""}}, name)

    @staticmethod
    def _rope(rot: Optional[dict], layout: str) -> PartSpec:
        if rot is None:
            return PartSpec("none", {})
        scaling = rot.get("scaling")
        return PartSpec("rope", {
            "rotary_dim": int(rot["dims"]), "theta": float(rot["base"]), "layout": layout,
            "scaling": None if scaling is None else {k: float(scaling[k]) for k in ("factor", "low", "high", "original")},
        })

    def _mixer(self, kind: str, m: dict, prefix: str, value_mix: Optional[str]) -> PartSpec:
        if kind == "attention":
            mask = m.get("mask") or {}
            return PartSpec(
                "attention",
                {
                    "hidden_size": self.width,
                    "num_heads": m["heads"],
                    "num_kv_heads": m["kv_heads"],
                    "head_size": m["dim"],
                    "value_head_size": m["vdim"],
                    "qkv_bias": False,
                    "out_bias": False,
                    "scale": float(m["scale"]),
                    "window": mask.get("size"),
                    "keep_first": int(mask.get("keep_first", 0)) if mask.get("size") else 0,
                    "value_mix": value_mix,
                    "position": self._rope(m.get("rot"), "interleaved"),
                    "tensor_names": _ATTENTION_NAMES,
                },
                prefix,
            )
        return PartSpec(
            "latent_attention",
            {
                "hidden_size": self.width,
                "num_heads": m["heads"],
                "head_size": m["dim"],
                "rotary_size": m["rot_dim"],
                "value_head_size": m["vdim"],
                "kv_rank": m["kv_rank"],
                "q_rank": m["q_rank"],
                "scale": float(m["scale"]),
                "eps": self.eps,
                "position": self._rope(m["rot"], "halves"),
                "tensor_names": _LATENT_NAMES,
            },
            prefix,
        )

    def model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        mixing_seen = False
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}."
            value_mix = None
            if layer["type"] == "attention" and layer["mixer"].get("v_mix"):
                value_mix = "blend" if mixing_seen else "source"
                mixing_seen = True
            parts = {
                "mixer_norm": self._norm(prefix + "norm1"),
                "mixer": self._mixer(layer["type"], layer["mixer"], prefix + "mix.", value_mix),
            }
            mlp = layer.get("mlp")
            if mlp is not None:
                experts = int(mlp["router"]["experts"])
                names = {"router.weight": "router"}
                for e in range(experts):
                    for local, stored in (("gate_proj", "gate"), ("up_proj", "up"), ("down_proj", "down")):
                        names[f"experts.{e}.{local}.weight"] = f"e{e}.{stored}"
                parts["feed_forward"] = PartSpec(
                    "routed_mlp",
                    {
                        "hidden_size": self.width,
                        "intermediate_size": int(mlp["expert"]["ff"]),
                        "num_experts": experts,
                        "top_k": int(mlp["router"]["top"]),
                        "score": "sigmoid",
                        "renormalise": False,
                        "weight_on": "input",
                        "tensor_names": names,
                    },
                    prefix + "mlp.",
                )
            layers.append(LayerSpec("parallel" if mlp is not None else "prenorm_mixer", parts))
            schedule.append(ScheduleEntry(index))
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
                {"vocab_size": self.vocab, "hidden_size": self.width, "tied_to": "embed",
                 "softcap": None if self.logit_softcap is None else float(self.logit_softcap),
                 "tensor_names": {"weight": "head"}},
                "",
            ),
        )
