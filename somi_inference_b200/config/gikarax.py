"""Typed configuration of the Gikarax architecture: a decoder whose layers add a mixer and a
feed-forward that both read the output of one layer norm (a weight, no bias), with three kinds of
mixer: latent attention without positions and with a sigmoid gate per output element; sliding-
window attention with an RMS norm per query/key head, rotation of a head's halves with banded
frequency scaling, capped scores, a sink in the softmax's denominator and a sigmoid gate per head;
and a causal attention (biases, rotation with ramped frequency scaling) side by side with a gated
linear attention whose decay per key channel is sigmoid(.)^(1/tau), each normalised over the model
width before they are averaged.  Feed-forwards are mixtures of experts without gates (erf gelu)
whose router keeps the largest logits and weighs them by the softmax over the kept.  A block of
layers may run several times in a row with the same weights; each run keeps its own cache and
state, and in front of every pass the stream is re-mixed with the embedding's output by a product
of its own.

config.json gives `architecture`, `vocab`, `width`, `norm.eps`, optionally `loop` = {start, stop,
times}, and `layers`: per layer `type` ("latent_attention", "attention" or "parallel"), `mixer`
(its sizes) and `mlp` (null or {"kind": "moe", "expert": {ff}, "router": {experts, top}}).
latent_attention: heads, dim, vdim, q_rank, kv_rank, scale.  attention: heads, kv_heads, dim, vdim,
scale, softcap | absent, mask: {size} | absent, rot: {dims, base, scaling: {factor, low, high,
original} | absent} | absent.  parallel: `left` = {heads, kv_heads, dim, vdim, scale, rot: {dims,
base, scaling: {factor, original, fast, slow} | absent} | absent} and `right` = {heads, dim, vdim,
tau}.  The rank of the decay's narrow projection is read from the tensors' shapes.

Tensor names: `embed`, `loop.in`, `final.norm`, `head`; per layer `l<i>.`: `norm1`;
latent_attention `mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o}`; attention `mix.{q, k, v,
q.norm, k.norm, g, o}`; parallel `mix.left.{q,k,v,o}` with `.b`, `mix.left.out`,
`mix.right.{q, k, v, g, o, norm, a1, a2, a2.b, out}`; `mlp.router`, `mlp.e<j>.{up,down}`.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Mapping

from .qwen2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunSpec

ARCHITECTURE = "Gikarax"
DEFAULT_MAX_POSITIONS = 1 << 20   # positions are computed, not learned: a bound for tables only
DEFAULT_DECAY_RANK = 16           # where no weight file says: rank of the decay's narrow pair
MIXER_TYPES = ("latent_attention", "attention", "parallel")


def _int(d: Any, key: str, where: str, least: int = 1) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, int) or isinstance(v, bool) or v < least:
        raise ConfigError(f"config.json: {where}{key} must be an integer >= {least}, got {v!r}")
    return v


def _number(d: Any, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, (int, float)) or isinstance(v, bool):
        raise ConfigError(f"config.json: {where}{key} must be a number, got {v!r}")
    return float(v)


def _rotation(m: dict, where: str, dim: int, scaling_keys: tuple[str, ...]) -> dict[str, Any] | None:
    rot = m.get("rot")
    if rot is None:
        return None
    w = where + "rot."
    out: dict[str, Any] = {"dims": _int(rot, "dims", w, 0), "base": _number(rot, "base", w)}
    if out["dims"] % 2 or out["dims"] > dim:
        raise ConfigError(f"config.json: {w}dims must be even and at most dim")
    if not out["base"] > 0.0:
        raise ConfigError(f"config.json: {w}base must be positive")
    if rot.get("scaling") is not None:
        out["scaling"] = {k: _number(rot["scaling"], k, w + "scaling.") for k in scaling_keys}
    return out


@dataclass(frozen=True)
class GikaraxLayerConfig:
    type: str                    # one of MIXER_TYPES
    mixer: dict[str, Any]        # the mixer's sizes, as the file gives them (validated)
    mlp: dict[str, Any] | None   # None: the layer has no feed-forward


@dataclass(frozen=True)
class GikaraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[GikaraxLayerConfig, ...]
    loop: tuple[int, int, int] | None = None      # (start, stop, times)
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: int | None = None

    architecture = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    # ---------------------------------------------------------------- reading
    @staticmethod
    def _grouped(m: Any, w: str) -> dict[str, Any]:
        out: dict[str, Any] = {k: _int(m, k, w) for k in ("heads", "kv_heads", "dim", "vdim")}
        out["scale"] = _number(m, "scale", w)
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"config.json: {w}heads must be a multiple of kv_heads")
        return out

    @classmethod
    def _mixer(cls, kind: str, m: Any, where: str) -> dict[str, Any]:
        if not isinstance(m, dict):
            raise ConfigError(f"config.json: {where}mixer must be an object")
        w = where + "mixer."
        if kind == "latent_attention":
            out: dict[str, Any] = {k: _int(m, k, w) for k in ("heads", "dim", "vdim", "q_rank", "kv_rank")}
            out["scale"] = _number(m, "scale", w)
            return out
        if kind == "attention":
            out = cls._grouped(m, w)
            if m.get("softcap") is not None:
                out["softcap"] = _number(m, "softcap", w)
                if not out["softcap"] > 0.0:
                    raise ConfigError(f"config.json: {w}softcap must be positive")
            if m.get("mask") is not None:
                out["mask"] = {"size": _int(m["mask"], "size", w + "mask.")}
            rot = _rotation(m, w, out["dim"], ("factor", "low", "high", "original"))
            if rot is not None:
                out["rot"] = rot
            return out
        left, right = m.get("left"), m.get("right")
        if not isinstance(left, dict) or not isinstance(right, dict):
            raise ConfigError(f"config.json: {w}left and {w}right must be objects")
        lo = cls._grouped(left, w + "left.")
        rot = _rotation(left, w + "left.", lo["dim"], ("factor", "original", "fast", "slow"))
        if rot is not None:
            lo["rot"] = rot
        ro: dict[str, Any] = {k: _int(right, k, w + "right.") for k in ("heads", "dim", "vdim")}
        ro["tau"] = _number(right, "tau", w + "right.")
        if not ro["tau"] > 0.0:
            raise ConfigError(f"config.json: {w}right.tau must be positive")
        if "decay_rank" in right:                      # not in a model's file; kept by to_dict
            ro["decay_rank"] = _int(right, "decay_rank", w + "right.")
        return {"left": lo, "right": ro}

    @staticmethod
    def _mlp(mlp: Any, where: str) -> dict[str, Any] | None:
        if mlp is None:
            return None
        w = where + "mlp."
        if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
            raise ConfigError(f"config.json: {where}mlp must be null or of kind 'moe'")
        r = mlp.get("router")
        router = {"experts": _int(r, "experts", w + "router."), "top": _int(r, "top", w + "router.")}
        if router["top"] > router["experts"]:
            raise ConfigError(f"config.json: {w}router.top exceeds the number of experts")
        return {"kind": "moe", "expert": {"ff": _int(mlp.get("expert"), "ff", w + "expert.")},
                "router": router}

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "GikaraxConfig":
        missing = [k for k in ("vocab", "width", "norm", "layers") if k not in d]
        if missing:
            raise ConfigError("config.json lacks: " + ", ".join(missing))
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, raw in enumerate(d["layers"]):
            where = f"layers[{i}]."
            if not isinstance(raw, dict) or "type" not in raw or "mixer" not in raw:
                raise ConfigError(f"config.json: {where[:-1]} needs 'type' and 'mixer'")
            if raw["type"] not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}type {raw['type']!r} is not a mixer of this "
                                  f"architecture (known: {', '.join(MIXER_TYPES)})")
            layers.append(GikaraxLayerConfig(raw["type"], cls._mixer(raw["type"], raw["mixer"], where),
                                             cls._mlp(raw.get("mlp"), where)))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = (_int(lp, "start", "loop.", 0), _int(lp, "stop", "loop.", 0), _int(lp, "times", "loop."))
        cfg = cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                  norm_eps=_number(d["norm"], "eps", "norm."), layers=tuple(layers), loop=loop,
                  max_positions=int(d.get("max_positions", DEFAULT_MAX_POSITIONS)),
                  eos_token_id=d.get("eos_token_id"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "GikaraxConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": json.loads(json.dumps(l.mixer)),
                        "mlp": None if l.mlp is None else json.loads(json.dumps(l.mlp))}
                       for l in self.layers]}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    # ------------------------------------------------------------- validation
    def validate(self) -> None:
        if not self.norm_eps > 0.0:
            raise ConfigError("norm.eps must be positive")
        if self.max_positions <= 0:
            raise ConfigError("max_positions must be positive")
        if self.loop is not None:
            start, stop, _ = self.loop
            if not 0 <= start <= stop <= len(self.layers):
                raise ConfigError(f"loop {start}..{stop} does not lie within the {len(self.layers)} layers")

    # ------------------------------------------------------------ model spec
    def runs(self) -> list[tuple[int, bool]]:
        """(layer, whether a pass of the loop opens in front of it) for every run: layers before
        the loop once, the looped layers `times` times in a row, then the rest.  Every pass, the
        first too, opens with the re-mix of the stream with the embedding's output."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        out = [(i, False) for i in range(start)]
        for _ in range(times):
            out += [(i, i == start) for i in range(start, stop)]
        return out + [(i, False) for i in range(stop, n)]

    def with_shapes(self, shapes: Mapping[str, tuple[int, ...]]) -> "GikaraxConfig":
        """This config with the sizes that only the weight file states (the rank of the decay's
        narrow pair of projections) read from the tensors' shapes."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            name = f"l{i}.mix.right.a1"
            if layer.type == "parallel" and name in shapes:
                m = {"left": m["left"], "right": {**m["right"], "decay_rank": int(shapes[name][0])}}
            layers.append(GikaraxLayerConfig(layer.type, m, layer.mlp))
        return GikaraxConfig(self.vocab, self.width, self.norm_eps, tuple(layers), self.loop,
                             self.max_positions, self.eos_token_id)

    @staticmethod
    def _rotary(rot: dict[str, Any] | None, kind: str) -> dict[str, Any] | None:
        if rot is None:
            return None
        out: dict[str, Any] = {"dims": rot["dims"], "base": rot["base"]}
        if rot.get("scaling") is not None:
            out["scaling"] = {"kind": kind, **rot["scaling"]}
        return out

    def to_model_spec(self) -> ModelSpec:
        D, eps = self.width, self.norm_eps

        def norm(name: str) -> PartSpec:
            return PartSpec("layernorm", {"size": D, "eps": eps, "names": {"weight": name}})

        layers = []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}", layer.mixer
            if layer.type == "latent_attention":
                mixer = PartSpec("latent_attention", {
                    "hidden_size": D, "heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
                    "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps,
                    "window": None, "sink": False, "own_latent": True, "gate": True,
                    "names": {"q_down": f"{p}.mix.dq", "q_norm": f"{p}.mix.dq.norm",
                              "q_up": f"{p}.mix.uq", "kv_down": f"{p}.mix.dkv",
                              "kv_norm": f"{p}.mix.dkv.norm", "k_up": f"{p}.mix.uk",
                              "v_up": f"{p}.mix.uv", "gate": f"{p}.mix.g", "out": f"{p}.mix.o"}})
            elif layer.type == "attention":
                mask = m.get("mask")
                mixer = PartSpec("normed_attention", {
                    "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                    "key_dim": m["dim"], "value_dim": m["vdim"], "scale": m["scale"],
                    "qkv_bias": False, "head_norm": True, "eps": eps,
                    "rotary": self._rotary(m.get("rot"), "bands"),
                    "mask": None if mask is None else {"kind": "window", "size": mask["size"]},
                    "softcap": m.get("softcap"), "sink": "zero", "head_gate": True,
                    "names": {"q_weight": f"{p}.mix.q", "k_weight": f"{p}.mix.k",
                              "v_weight": f"{p}.mix.v", "q_norm": f"{p}.mix.q.norm",
                              "k_norm": f"{p}.mix.k.norm", "gate_weight": f"{p}.mix.g",
                              "o_weight": f"{p}.mix.o"}})
            else:
                lo, ro = m["left"], m["right"]
                lp, rp = f"{p}.mix.left", f"{p}.mix.right"
                names = {"o_weight": f"{lp}.o", "o_bias": f"{lp}.o.b"}
                for part in ("q", "k", "v"):
                    names.update({f"{part}_weight": f"{lp}.{part}", f"{part}_bias": f"{lp}.{part}.b"})
                left = PartSpec("normed_attention", {
                    "hidden_size": D, "num_heads": lo["heads"], "num_kv_heads": lo["kv_heads"],
                    "key_dim": lo["dim"], "value_dim": lo["vdim"], "scale": lo["scale"],
                    "qkv_bias": True, "o_bias": True, "head_norm": False, "eps": eps,
                    "rotary": self._rotary(lo.get("rot"), "ramp"), "mask": None, "names": names})
                right = PartSpec("gated_linear_attention", {
                    "hidden_size": D, "heads": ro["heads"], "key_dim": ro["dim"],
                    "value_dim": ro["vdim"], "tau": ro["tau"], "eps": eps,
                    "q_scale": ro["dim"] ** -0.5,
                    "decay_rank": ro.get("decay_rank", DEFAULT_DECAY_RANK),
                    "names": {"q_weight": f"{rp}.q", "k_weight": f"{rp}.k", "v_weight": f"{rp}.v",
                              "gate_weight": f"{rp}.g", "decay_down": f"{rp}.a1",
                              "decay_up": f"{rp}.a2", "decay_bias": f"{rp}.a2.b",
                              "norm": f"{rp}.norm", "o_weight": f"{rp}.o"}})
                mixer = PartSpec("side_by_side", {
                    "hidden_size": D, "eps": eps, "left": left, "right": right,
                    "names": {"left_norm": f"{lp}.out", "right_norm": f"{rp}.out"}})
            ff, mlp = None, layer.mlp
            if mlp is not None:
                E = mlp["router"]["experts"]
                ff = PartSpec("routed_moe", {
                    "hidden_size": D, "experts": E, "top": mlp["router"]["top"],
                    "weights": "softmax_chosen", "activation": "gelu",
                    "expert_ff": mlp["expert"]["ff"],
                    "names": {"router": f"{p}.mlp.router",
                              "up": [f"{p}.mlp.e{e}.up" for e in range(E)],
                              "down": [f"{p}.mlp.e{e}.down" for e in range(E)]}})
            layers.append(LayerSpec(prefix=p, mixer=mixer, feed_forward=ff,
                                    norms={"shared": norm(f"{p}.norm1")}, arrangement="shared_norm"))
        stream_parts = {}
        if self.loop is not None:
            stream_parts["loop_in"] = PartSpec("embedding_remix", {"hidden_size": D,
                                                                   "names": {"weight": "loop.in"}})
        spec = ModelSpec(
            architecture=ARCHITECTURE, hidden_size=D, vocab_size=self.vocab,
            max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D,
                                                   "scale": 1.0, "names": {"weight": "embed"}}),
            layers=tuple(layers),
            # every run of a looped layer keeps a cache and a state of its own
            schedule=tuple(RunSpec(i, remix="loop_in" if opens else None) for i, opens in self.runs()),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": D, "tied": False,
                                      "names": {"weight": "head", "tied_to": "embed"}}),
            stream_parts=stream_parts)
        spec.validate()
        return spec
