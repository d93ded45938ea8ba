"""Configuration of the Goguvik decoder, read from the keys of its own ``config.json``.

The design: an embedding that is also the output head; layers of differential attention (two softmax
maps per head over shared values, grouped key/value heads, no rotation, a query temperature that grows
with the logarithm of the position, a sigmoid output gate, biased projections) and a dense gated
feed-forward with tanh-approximated gelu; Dynamic Tanh wherever another decoder norms; several residual
streams joined to the sublayers by hyper-connections; layers that attend over the keys and values an
earlier layer cached instead of projecting their own.

``config.json`` gives ``architecture``, ``vocab``, ``width``, ``streams``, ``norm.eps`` and a list
``layers``; each layer has ``type`` (the mixer, ``"attention"``), ``mixer`` (``heads``, ``kv_heads``,
``dim``, ``vdim``, ``scale``, ``diff``, optional ``q_temp`` = ``{coef, every}``, optional ``kv_from``)
and ``mlp`` (``{kind: "dense", ff}`` or null).  Every size and constant is read from there; a key
this design does not know is an error, never ignored.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

from .qwen3 import ConfigError
from .spec import (
    DifferentialAttentionSpec,
    DynamicTanhSpec,
    GatedFeedForwardSpec,
    HyperConnectionSpec,
    ModelSpec,
    QueryTemperatureSpec,
    ScheduleEntry,
    hyper_layer,
)

_TOP = {"architecture", "architectures", "layers", "norm", "streams", "vocab", "width", "torch_dtype", "dtype"}
_MIXER = {"heads", "kv_heads", "dim", "vdim", "scale", "diff", "q_temp", "kv_from"}
_MLP = {"kind", "ff"}


def _positive(where: str, value) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json has {where}={value!r}: a positive integer is needed")
    return value


def _unknown(where: str, raw: dict, known) -> None:
    extra = sorted(k for k in raw if k not in known)
    if extra:
        raise ConfigError(f"config.json has key(s) {', '.join(extra)} in {where} that this design does not define")


@dataclass(frozen=True)
class GoguvikConfig:
    vocab: int
    width: int
    streams: int
    norm_eps: float
    layers: tuple          # the layer dicts as config.json gives them (validated)
    torch_dtype: str = "bfloat16"

    architecture = "Goguvik"

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, raw: dict) -> "GoguvikConfig":
        missing = [k for k in ("layers", "norm", "streams", "vocab", "width") if k not in raw]
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))
        _unknown("the model", raw, _TOP)
        if not isinstance(raw["norm"], dict) or "eps" not in raw["norm"]:
            raise ConfigError("config.json lacks required key(s): norm.eps")
        _unknown("norm", raw["norm"], {"eps"})
        eps = float(raw["norm"]["eps"])
        if not eps >= 0.0:
            raise ConfigError(f"norm.eps={eps} must not be negative")
        layers = raw["layers"]
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json has no layers")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"{where} is not an object")
            _unknown(where, layer, {"type", "mixer", "mlp"})
            if layer.get("type") != "attention":
                raise ConfigError(f"{where}.type={layer.get('type')!r}: this design's mixer is 'attention'")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where} lacks required key(s): mixer")
            _unknown(where + ".mixer", mixer, _MIXER)
            lacking = [k for k in ("heads", "kv_heads", "dim", "vdim", "scale", "diff") if k not in mixer]
            if lacking:
                raise ConfigError(f"{where}.mixer lacks required key(s): " + ", ".join(lacking))
            heads = _positive(where + ".mixer.heads", mixer["heads"])
            kv_heads = _positive(where + ".mixer.kv_heads", mixer["kv_heads"])
            _positive(where + ".mixer.dim", mixer["dim"])
            _positive(where + ".mixer.vdim", mixer["vdim"])
            if heads % kv_heads:
                raise ConfigError(f"{where}.mixer: heads={heads} must be a multiple of kv_heads={kv_heads}")
            temp = mixer.get("q_temp")
            if temp is not None:
                if not isinstance(temp, dict) or "coef" not in temp or "every" not in temp:
                    raise ConfigError(f"{where}.mixer.q_temp needs coef and every")
                _unknown(where + ".mixer.q_temp", temp, {"coef", "every"})
                _positive(where + ".mixer.q_temp.every", temp["every"])
            source = mixer.get("kv_from")
            if source is not None:
                if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
                    raise ConfigError(f"{where}.mixer.kv_from={source!r} must name an earlier layer")
                other = checked[source]["mixer"]
                if "kv_from" in other and other["kv_from"] is not None:
                    raise ConfigError(f"{where}.mixer.kv_from={source}: that layer has no keys and values of its own")
                for key in ("kv_heads", "dim", "vdim"):
                    if other[key] != mixer[key]:
                        raise ConfigError(f"{where}.mixer.kv_from={source}: {key} differs ({mixer[key]} vs {other[key]})")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"{where}.mlp is neither an object nor null")
                _unknown(where + ".mlp", mlp, _MLP)
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp.kind={mlp.get('kind')!r}: this design's feed-forward is 'dense'")
                _positive(where + ".mlp.ff", mlp.get("ff"))
            checked.append(copy.deepcopy(layer))
        return cls(
            vocab=_positive("vocab", raw["vocab"]),
            width=_positive("width", raw["width"]),
            streams=_positive("streams", raw["streams"]),
            norm_eps=eps,
            layers=tuple(checked),
            torch_dtype=str(raw.get("torch_dtype", raw.get("dtype", "bfloat16"))),
        )

    # ------------------------------------------------------------------ writing

    def to_dict(self) -> dict:
        return {
            "architecture": self.architecture,
            "layers": copy.deepcopy(list(self.layers)),
            "norm": {"eps": self.norm_eps},
            "streams": self.streams,
            "vocab": self.vocab,
            "width": self.width,
            "torch_dtype": self.torch_dtype,
        }

    # ------------------------------------------------------------------ meaning

    def to_model_spec(self) -> ModelSpec:
        norm = DynamicTanhSpec(size=self.width)
        connection = HyperConnectionSpec(streams=self.streams)
        layers, schedule, ignored = [], [], []
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            prefix = f"l{i}."
            source = m.get("kv_from")
            temp = m.get("q_temp")
            mixer = DifferentialAttentionSpec(
                hidden_size=self.width,
                num_heads=int(m["heads"]),
                num_kv_heads=int(m["kv_heads"]),
                head_dim=int(m["dim"]),
                value_dim=int(m["vdim"]),
                scale=float(m["scale"]),
                lambda_init=float(m["diff"]),
                norm_eps=self.norm_eps,
                q_temperature=QueryTemperatureSpec(float(temp["coef"]), int(temp["every"])) if temp else None,
                bias=True,
                gated=True,
                own_kv=source is None,
            )
            names = {
                "norm1.weight": prefix + "norm1", "norm1.alpha": prefix + "norm1.alpha", "norm1.bias": prefix + "norm1.b",
                "mixer.q": prefix + "mix.q", "mixer.q_bias": prefix + "mix.q.b",
                "mixer.g": prefix + "mix.g",
                "mixer.o": prefix + "mix.o", "mixer.o_bias": prefix + "mix.o.b",
                "mixer.lq1": prefix + "mix.lq1", "mixer.lk1": prefix + "mix.lk1",
                "mixer.lq2": prefix + "mix.lq2", "mixer.lk2": prefix + "mix.lk2",
                "connection1.in": prefix + "hc1.in", "connection1.out": prefix + "hc1.out",
                "connection1.mix": prefix + "hc1.mix",
            }
            if source is None:
                names.update({"mixer.k": prefix + "mix.k", "mixer.k_bias": prefix + "mix.k.b",
                              "mixer.v": prefix + "mix.v", "mixer.v_bias": prefix + "mix.v.b"})
            mlp = layer.get("mlp")
            second = {
                "norm2.weight": prefix + "norm2", "norm2.alpha": prefix + "norm2.alpha", "norm2.bias": prefix + "norm2.b",
                "connection2.in": prefix + "hc2.in", "connection2.out": prefix + "hc2.out",
                "connection2.mix": prefix + "hc2.mix",
            }
            if mlp is not None:
                ff = GatedFeedForwardSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]),
                                          activation="gelu_tanh")
                names.update(second)
                names.update({"feed_forward.gate": prefix + "mlp.gate", "feed_forward.up": prefix + "mlp.up",
                              "feed_forward.down": prefix + "mlp.down"})
                layers.append(hyper_layer(mixer, ff, norm, norm, connection, names))
            else:
                # a layer without a feed-forward has no second sublayer; should a checkpoint carry the
                # second norm and connection all the same, nothing reads them
                ignored.extend(second.values())
                layers.append(hyper_layer(mixer, None, norm, None, connection, names))
            schedule.append(ScheduleEntry(layer=i, cache=i if source is None else int(source),
                                          writes_cache=source is None))
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=self.width,
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=norm,
            tie_embeddings=True,
            embed_name="embed",
            final_norm_name="final.norm",
            lm_head_name="lm_head",
            streams=self.streams,
            final_norm_names={"weight": "final.norm", "alpha": "final.norm.alpha", "bias": "final.norm.b"},
            ignored_tensors=tuple(ignored),
        )
