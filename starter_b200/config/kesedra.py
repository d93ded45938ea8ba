"""Configuration of the Kesedra decoder, read from the keys of its own ``config.json``.

The design: an embedding times a constant; layers with a norm in front of and behind each sublayer
around a residual stream that is a 32-bit sum, the norms' gains stored around zero; per layer one of
two mixers (``wkv``: a linear recurrence with a matrix state per head and a decay that depends on the
token; ``latent_attention``: attention over a cached low-rank latent with a rotated key part shared by
all heads and a sliding window, which may read the latent another layer cached) and one of two
feed-forwards (``dense``: squared relu with biases; ``moe``: routed clamped gated experts) or none; a
final norm and an output head of its own.

``config.json`` gives ``architecture``, ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and a
list ``layers``; a layer has ``type``, ``mixer`` and ``mlp``:

* ``wkv``: ``mixer = {heads, dim}``.  The rank of the decay's two small matrices is the one size that
  config.json leaves to the checkpoint (the shape of ``l<i>.mix.w1``); ``load_model`` reads it from
  there.  A model made without a checkpoint (random weights) states it as ``mixer.decay_rank``.
* ``latent_attention``: ``mixer = {heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask{size},
  rot{base, dims}, kv_from?}``.
* ``mlp``: null, ``{kind: "dense", ff}`` or ``{kind: "moe", expert{ff, limit}, router{experts, top}}``.

Every size and constant is read from there; a key this design does not know is an error.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, replace

from .qwen3 import ConfigError
from .spec import (
    BiasedFeedForwardSpec,
    InterleavedRopeSpec,
    LatentAttentionSpec,
    ModelSpec,
    NormSpec,
    RoutedExpertsSpec,
    ScheduleEntry,
    WkvSpec,
    sandwich_layer,
)

_TOP = {"architecture", "architectures", "embedding", "layers", "norm", "vocab", "width", "torch_dtype", "dtype"}
_WKV = {"heads", "dim", "decay_rank"}
_LATENT = {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "mask", "rot", "kv_from"}
_SHARED = ("kv_rank", "rot_dim", "rot")       # what a layer and the layer whose latent it reads must agree on
_SHIFTS = ("r", "k", "v", "g", "w")


def _positive(where: str, value) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json has {where}={value!r}: a positive integer is needed")
    return value


def _number(where: str, value) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json has {where}={value!r}: a number is needed")
    return float(value)


def _unknown(where: str, raw: dict, known) -> None:
    extra = sorted(k for k in raw if k not in known)
    if extra:
        raise ConfigError(f"config.json has key(s) {', '.join(extra)} in {where} that this design does not define")


def _lacking(where: str, raw, keys) -> None:
    if not isinstance(raw, dict):
        raise ConfigError(f"{where} is not an object")
    missing = [k for k in keys if k not in raw]
    if missing:
        raise ConfigError(f"{where} lacks required key(s): " + ", ".join(missing))


def _check_mlp(where: str, mlp) -> None:
    if mlp is None:
        return
    _lacking(where, mlp, ("kind",))
    if mlp["kind"] == "dense":
        _unknown(where, mlp, {"kind", "ff"})
        _positive(where + ".ff", mlp.get("ff"))
    elif mlp["kind"] == "moe":
        _unknown(where, mlp, {"kind", "expert", "router"})
        _lacking(where + ".expert", mlp.get("expert"), ("ff", "limit"))
        _unknown(where + ".expert", mlp["expert"], {"ff", "limit"})
        _lacking(where + ".router", mlp.get("router"), ("experts", "top"))
        _unknown(where + ".router", mlp["router"], {"experts", "top"})
        _positive(where + ".expert.ff", mlp["expert"]["ff"])
        if not _number(where + ".expert.limit", mlp["expert"]["limit"]) > 0.0:
            raise ConfigError(f"{where}.expert.limit must be positive")
        experts = _positive(where + ".router.experts", mlp["router"]["experts"])
        top = _positive(where + ".router.top", mlp["router"]["top"])
        if top > experts:
            raise ConfigError(f"{where}.router: top={top} of experts={experts}")
    else:
        raise ConfigError(f"{where}.kind={mlp['kind']!r}: this design's feed-forwards are 'dense' and 'moe'")


@dataclass(frozen=True)
class KesedraConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple          # the layer dicts as config.json gives them (validated)
    torch_dtype: str = "bfloat16"

    architecture = "Kesedra"

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, raw: dict) -> "KesedraConfig":
        _lacking("config.json", raw, ("embedding", "layers", "norm", "vocab", "width"))
        _unknown("the model", raw, _TOP)
        _lacking("norm", raw["norm"], ("eps",))
        _unknown("norm", raw["norm"], {"eps"})
        _lacking("embedding", raw["embedding"], ("scale",))
        _unknown("embedding", raw["embedding"], {"scale"})
        eps = _number("norm.eps", raw["norm"]["eps"])
        if not eps >= 0.0:
            raise ConfigError(f"norm.eps={eps} must not be negative")
        layers = raw["layers"]
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json has no layers")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            _lacking(where, layer, ("type", "mixer"))
            _unknown(where, layer, {"type", "mixer", "mlp"})
            mixer = layer["mixer"]
            if layer["type"] == "wkv":
                _lacking(where + ".mixer", mixer, ("heads", "dim"))
                _unknown(where + ".mixer", mixer, _WKV)
                _positive(where + ".mixer.heads", mixer["heads"])
                _positive(where + ".mixer.dim", mixer["dim"])
                if mixer.get("decay_rank") is not None:
                    _positive(where + ".mixer.decay_rank", mixer["decay_rank"])
            elif layer["type"] == "latent_attention":
                _lacking(where + ".mixer", mixer, ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale",
                                                   "mask", "rot"))
                _unknown(where + ".mixer", mixer, _LATENT)
                for key in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
                    _positive(f"{where}.mixer.{key}", mixer[key])
                _number(where + ".mixer.scale", mixer["scale"])
                _lacking(where + ".mixer.mask", mixer["mask"], ("size",))
                _unknown(where + ".mixer.mask", mixer["mask"], {"size"})
                _positive(where + ".mixer.mask.size", mixer["mask"]["size"])
                _lacking(where + ".mixer.rot", mixer["rot"], ("base", "dims"))
                _unknown(where + ".mixer.rot", mixer["rot"], {"base", "dims"})
                dims = _positive(where + ".mixer.rot.dims", mixer["rot"]["dims"])
                if not _number(where + ".mixer.rot.base", mixer["rot"]["base"]) > 0.0:
                    raise ConfigError(f"{where}.mixer.rot.base must be positive")
                if dims % 2 or dims > mixer["rot_dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims={dims} must be even and at most rot_dim="
                                      f"{mixer['rot_dim']}")
                source = mixer.get("kv_from")
                if source is not None:
                    if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
                        raise ConfigError(f"{where}.mixer.kv_from={source!r} must name an earlier layer")
                    other = checked[source]
                    if other["type"] != "latent_attention" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}.mixer.kv_from={source}: that layer caches no latent of its own")
                    for key in _SHARED:
                        if other["mixer"][key] != mixer[key]:
                            raise ConfigError(f"{where}.mixer.kv_from={source}: {key} differs "
                                              f"({mixer[key]} vs {other['mixer'][key]})")
            else:
                raise ConfigError(f"{where}.type={layer['type']!r}: this design's mixers are 'wkv' and "
                                  "'latent_attention'")
            _check_mlp(where + ".mlp", layer.get("mlp"))
            checked.append(copy.deepcopy(dict(layer)))
        return cls(
            vocab=_positive("vocab", raw["vocab"]),
            width=_positive("width", raw["width"]),
            embedding_scale=_number("embedding.scale", raw["embedding"]["scale"]),
            norm_eps=eps,
            layers=tuple(checked),
            torch_dtype=str(raw.get("torch_dtype", raw.get("dtype", "bfloat16"))),
        )

    def with_tensor_shapes(self, shapes: dict) -> "KesedraConfig":
        """The same configuration with the sizes that only the checkpoint gives filled in from
        ``shapes`` (tensor name -> shape): the rank of every recurrent layer's decay matrices."""
        layers = []
        for i, layer in enumerate(self.layers):
            layer = copy.deepcopy(layer)
            name = f"l{i}.mix.w1"
            if layer["type"] == "wkv" and name in shapes and len(shapes[name]) == 2:
                rank = int(shapes[name][0])
                stated = layer["mixer"].get("decay_rank")
                if stated is not None and stated != rank:
                    raise ConfigError(f"layers[{i}].mixer.decay_rank={stated}, but {name} has {rank} rows")
                layer["mixer"]["decay_rank"] = rank
            layers.append(layer)
        return replace(self, layers=tuple(layers))

    # ------------------------------------------------------------------ writing

    def to_dict(self) -> dict:
        return {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": copy.deepcopy(list(self.layers)),
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
            "torch_dtype": self.torch_dtype,
        }

    # ------------------------------------------------------------------ meaning

    def _mixer(self, i: int, m: dict, kind: str, prefix: str):
        if kind == "wkv":
            if m.get("decay_rank") is None:
                raise ConfigError(f"layers[{i}]: the rank of the decay matrices is given neither by a checkpoint "
                                  f"({prefix}w1) nor by mixer.decay_rank")
            spec = WkvSpec(hidden_size=self.width, num_heads=int(m["heads"]), head_dim=int(m["dim"]),
                           decay_rank=int(m["decay_rank"]), norm_eps=self.norm_eps)
            names = {f"mixer.{n}": prefix + n for n in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")}
            names.update({f"mixer.mu_{s}": f"{prefix}mu.{s}" for s in _SHIFTS})
            return spec, names
        own = m.get("kv_from") is None
        spec = LatentAttentionSpec(
            hidden_size=self.width, num_heads=int(m["heads"]), head_dim=int(m["dim"]), rot_dim=int(m["rot_dim"]),
            value_dim=int(m["vdim"]), q_rank=int(m["q_rank"]), kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
            norm_eps=self.norm_eps,
            position=InterleavedRopeSpec(dims=int(m["rot"]["dims"]), base=float(m["rot"]["base"])),
            window=int(m["mask"]["size"]), own_kv=own)
        names = {"mixer.dq": prefix + "dq", "mixer.dq_norm": prefix + "dq.norm", "mixer.uq": prefix + "uq",
                 "mixer.uk": prefix + "uk", "mixer.uv": prefix + "uv", "mixer.o": prefix + "o"}
        if own:
            names.update({"mixer.dkv": prefix + "dkv", "mixer.dkv_norm": prefix + "dkv.norm"})
        return spec, names

    def _feed_forward(self, mlp: dict, prefix: str):
        if mlp["kind"] == "dense":
            spec = BiasedFeedForwardSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]), activation="relu2")
            return spec, {"feed_forward.up": prefix + "up", "feed_forward.up_bias": prefix + "up.b",
                          "feed_forward.down": prefix + "down", "feed_forward.down_bias": prefix + "down.b"}
        experts = int(mlp["router"]["experts"])
        spec = RoutedExpertsSpec(hidden_size=self.width, intermediate_size=int(mlp["expert"]["ff"]), experts=experts,
                                 top=int(mlp["router"]["top"]), limit=float(mlp["expert"]["limit"]))
        names = {"feed_forward.router": prefix + "router", "feed_forward.router_bias": prefix + "router.b"}
        for e in range(experts):
            for part in ("gate", "up", "down"):
                names[f"feed_forward.e{e}_{part}"] = f"{prefix}e{e}.{part}"
        return spec, names

    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec(size=self.width, eps=self.norm_eps, unit_offset=True)
        layers, schedule, ignored = [], [], []
        for i, layer in enumerate(self.layers):
            prefix = f"l{i}."
            mixer, names = self._mixer(i, layer["mixer"], layer["type"], prefix + "mix.")
            names.update({"norm1.weight": prefix + "norm1", "norm1b.weight": prefix + "norm1b"})
            second = {"norm2.weight": prefix + "norm2", "norm2b.weight": prefix + "norm2b"}
            mlp = layer.get("mlp")
            if mlp is not None:
                ff, ff_names = self._feed_forward(mlp, prefix + "mlp.")
                names.update(second)
                names.update(ff_names)
                layers.append(sandwich_layer(mixer, ff, norm, names))
            else:
                # nothing reads the second pair of norms of a layer without a feed-forward, should a
                # checkpoint carry them all the same
                ignored.extend(second.values())
                layers.append(sandwich_layer(mixer, None, norm, names))
            source = layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None
            schedule.append(ScheduleEntry(layer=i, cache=i if source is None else int(source),
                                          writes_cache=source is None))
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=self.width,
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=norm,
            tie_embeddings=False,
            embed_name="embed",
            final_norm_name="final.norm",
            lm_head_name="head",
            ignored_tensors=tuple(ignored),
            embedding_scale=self.embedding_scale,
        )
