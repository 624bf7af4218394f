"""Typed configuration of the Poselorn architecture: a decoder whose layers add a mixer and a
feed-forward that read the same stream (each through an RMS norm of its own, each scaled per
channel, their sum times one factor), with two kinds of mixer: a gated delta rule with a decay
per key channel, and a sliding-window softmax attention (biases, RMS norm per query/key head,
rotation of a head's halves) side by side with a linear attention of constant decays, each
normalised over the model width before they are averaged.  Feed-forwards are dense (squared relu,
biases) or a routed mixture of experts (softmax router, a correction for the choice only, groups
of experts, identity experts).  A block of layers may run several times in a row with the same
weights; each run keeps its own cache and state, and the embedding's output is added to the
stream again in front of every repetition.

config.json gives `architecture`, `vocab`, `width`, `norm.eps`, `embedding.scale`,
`residual_mult`, optionally `loop` = {start, stop, times}, and `layers`: per layer `type`
("channel_delta" or "parallel"), `mixer` (its sizes) and `mlp` (null, {"kind": "dense", "ff"} or
{"kind": "moe", "expert": {ff}, "router": {experts, top, identity, groups: {count, keep}}}).
channel_delta: `heads`, `kv_heads`, `dim`, `vdim`, `conv` (taps).  parallel: `left` = {heads,
kv_heads, dim, vdim, scale, rot: {dims, base} | absent, mask: {size} | absent} and `right` =
{heads, dim, vdim, decay: [one per head]}.  The ranks of the narrow projections and the number of
router outputs are read from the tensors' shapes.

Tensor names: `embed`, `final.norm`, `head`; per layer `l<i>.`: `norm1`, `norm2`, `ls1`, `ls2`;
channel_delta `mix.{q,k,v}` with `.conv`, `mix.{b, A_log, a1, a2, dt_bias, g1, g2, norm, o}`;
parallel `mix.left.{q,k,v}` with `.b`, `mix.left.{q.norm, k.norm, o, out}`,
`mix.right.{q, k, v, g, o, norm, out}`; `mlp.{up,down}` with `.b` (dense) or `mlp.router`,
`mlp.correction`, `mlp.e<j>.{gate,up,down}`.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Mapping

from .qwen2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunSpec

ARCHITECTURE = "Poselorn"
UNIT_VECTOR_EPS = 1e-6            # fixed by the design: q, k / sqrt(sum of squares + this)
DEFAULT_MAX_POSITIONS = 1 << 20   # positions are computed, not learned: a bound for tables only
DEFAULT_NARROW_RANK = 16          # where no weight file says: rank of the decay and gate pairs


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


@dataclass(frozen=True)
class PoselornLayerConfig:
    type: str                    # "channel_delta" | "parallel"
    mixer: dict[str, Any]        # the mixer's sizes, as the file gives them (validated)
    mlp: dict[str, Any] | None   # None: the layer has no feed-forward


@dataclass(frozen=True)
class PoselornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    layers: tuple[PoselornLayerConfig, ...]
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
    def _mixer(kind: str, m: Any, where: str) -> dict[str, Any]:
        if not isinstance(m, dict):
            raise ConfigError(f"config.json: {where}mixer must be an object")
        w = where + "mixer."
        if kind == "channel_delta":
            out: dict[str, Any] = {k: _int(m, k, w) for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
            if out["heads"] % out["kv_heads"]:
                raise ConfigError(f"config.json: {w}heads must be a multiple of kv_heads")
            for k in ("decay_rank", "gate_rank"):      # not in a model's file; kept by to_dict
                if k in m:
                    out[k] = _int(m, k, w)
            return out
        left, right = m.get("left"), m.get("right")
        if not isinstance(left, dict) or not isinstance(right, dict):
            raise ConfigError(f"config.json: {w}left and {w}right must be objects")
        lw, rw = w + "left.", w + "right."
        lo: dict[str, Any] = {k: _int(left, k, lw) for k in ("heads", "kv_heads", "dim", "vdim")}
        lo["scale"] = _number(left, "scale", lw)
        if lo["heads"] % lo["kv_heads"]:
            raise ConfigError(f"config.json: {lw}heads must be a multiple of kv_heads")
        if left.get("rot") is not None:
            lo["rot"] = {"dims": _int(left["rot"], "dims", lw + "rot.", 0),
                         "base": _number(left["rot"], "base", lw + "rot.")}
            if lo["rot"]["dims"] % 2 or lo["rot"]["dims"] > lo["dim"]:
                raise ConfigError(f"config.json: {lw}rot.dims must be even and at most dim")
        if left.get("mask") is not None:
            lo["mask"] = {"size": _int(left["mask"], "size", lw + "mask.")}
        ro: dict[str, Any] = {k: _int(right, k, rw) for k in ("heads", "dim", "vdim")}
        decay = right.get("decay")
        if (not isinstance(decay, list) or len(decay) != ro["heads"]
                or not all(isinstance(v, (int, float)) and not isinstance(v, bool) for v in decay)):
            raise ConfigError(f"config.json: {rw}decay must list one number per head")
        ro["decay"] = [float(v) for v in decay]
        return {"left": lo, "right": ro}

    @staticmethod
    def _mlp(mlp: Any, where: str) -> dict[str, Any] | None:
        if mlp is None:
            return None
        w = where + "mlp."
        if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
            raise ConfigError(f"config.json: {where}mlp must be null or of kind 'dense' or 'moe'")
        if mlp["kind"] == "dense":
            return {"kind": "dense", "ff": _int(mlp, "ff", w)}
        r = mlp.get("router")
        router: dict[str, Any] = {"experts": _int(r, "experts", w + "router."),
                                  "top": _int(r, "top", w + "router."),
                                  "identity": _int(r, "identity", w + "router.", 0) if "identity" in r else 0}
        outputs = router["experts"] + router["identity"]
        if router["top"] > outputs:
            raise ConfigError(f"config.json: {w}router.top exceeds the router's outputs")
        if r.get("groups") is not None:
            g = {"count": _int(r["groups"], "count", w + "router.groups."),
                 "keep": _int(r["groups"], "keep", w + "router.groups.")}
            if outputs % g["count"] or g["keep"] > g["count"]:
                raise ConfigError(f"config.json: {w}router.groups must cut {outputs} outputs into "
                                  "equal groups and keep no more than there are")
            if router["top"] > g["keep"] * (outputs // g["count"]):
                raise ConfigError(f"config.json: {w}router.top exceeds what the kept groups hold")
            router["groups"] = g
        return {"kind": "moe", "expert": {"ff": _int(mlp.get("expert"), "ff", w + "expert.")},
                "router": router}

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "PoselornConfig":
        missing = [k for k in ("vocab", "width", "norm", "embedding", "residual_mult", "layers")
                   if k not in d]
        if missing:
            raise ConfigError("config.json lacks: " + ", ".join(missing))
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, raw in enumerate(d["layers"]):
            where = f"layers[{i}]."
            if not isinstance(raw, dict) or "type" not in raw or "mixer" not in raw:
                raise ConfigError(f"config.json: {where[:-1]} needs 'type' and 'mixer'")
            if raw["type"] not in ("channel_delta", "parallel"):
                raise ConfigError(f"config.json: {where}type {raw['type']!r} is not a mixer of this "
                                  "architecture (known: 'channel_delta', 'parallel')")
            layers.append(PoselornLayerConfig(raw["type"], cls._mixer(raw["type"], raw["mixer"], where),
                                              cls._mlp(raw.get("mlp"), where)))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = (_int(lp, "start", "loop.", 0), _int(lp, "stop", "loop.", 0), _int(lp, "times", "loop."))
        cfg = cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                  norm_eps=_number(d["norm"], "eps", "norm."),
                  embedding_scale=_number(d["embedding"], "scale", "embedding."),
                  residual_mult=_number(d, "residual_mult", ""),
                  layers=tuple(layers), loop=loop,
                  max_positions=int(d.get("max_positions", DEFAULT_MAX_POSITIONS)),
                  eos_token_id=d.get("eos_token_id"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "PoselornConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
            "residual_mult": self.residual_mult,
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
        """(layer, whether the embedding's output is added in front of it) for every run: layers
        before the loop once, the looped layers `times` times in a row, then the rest."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        out = [(i, False) for i in range(start)]
        for turn in range(times):
            out += [(i, turn > 0 and i == start) for i in range(start, stop)]
        return out + [(i, False) for i in range(stop, n)]

    def with_shapes(self, shapes: Mapping[str, tuple[int, ...]]) -> "PoselornConfig":
        """This config with the sizes that only the weight file states (the ranks of the narrow
        decay and gate projections) read from the tensors' shapes."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "channel_delta":
                m = dict(m)
                for key, name in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                    if name in shapes:
                        m[key] = int(shapes[name][0])
            layers.append(PoselornLayerConfig(layer.type, m, layer.mlp))
        return PoselornConfig(self.vocab, self.width, self.norm_eps, self.embedding_scale,
                              self.residual_mult, tuple(layers), self.loop, self.max_positions,
                              self.eos_token_id)

    def to_model_spec(self) -> ModelSpec:
        D, eps = self.width, self.norm_eps

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": D, "eps": eps, "names": {"weight": name}})

        layers = []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}", layer.mixer
            if layer.type == "channel_delta":
                names = {"beta_weight": f"{p}.mix.b", "a_log": f"{p}.mix.A_log",
                         "decay_down": f"{p}.mix.a1", "decay_up": f"{p}.mix.a2",
                         "dt_bias": f"{p}.mix.dt_bias", "gate_down": f"{p}.mix.g1",
                         "gate_up": f"{p}.mix.g2", "norm": f"{p}.mix.norm", "o_weight": f"{p}.mix.o"}
                for part in ("q", "k", "v"):
                    names.update({f"{part}_weight": f"{p}.mix.{part}", f"{part}_taps": f"{p}.mix.{part}.conv"})
                mixer = PartSpec("delta_rule", {
                    "hidden_size": D, "heads": m["heads"], "qk_heads": m["kv_heads"],
                    "key_dim": m["dim"], "value_dim": m["vdim"], "taps": m["conv"], "eps": eps,
                    "unit_eps": UNIT_VECTOR_EPS, "q_scale": m["dim"] ** -0.5,
                    "decay_rank": m.get("decay_rank", DEFAULT_NARROW_RANK),
                    "gate_rank": m.get("gate_rank", DEFAULT_NARROW_RANK), "names": names})
            else:
                lo, ro = m["left"], m["right"]
                lp, rp = f"{p}.mix.left", f"{p}.mix.right"
                names = {"o_weight": f"{lp}.o", "q_norm": f"{lp}.q.norm", "k_norm": f"{lp}.k.norm"}
                for part in ("q", "k", "v"):
                    names.update({f"{part}_weight": f"{lp}.{part}", f"{part}_bias": f"{lp}.{part}.b"})
                mask = lo.get("mask")
                left = PartSpec("normed_attention", {
                    "hidden_size": D, "num_heads": lo["heads"], "num_kv_heads": lo["kv_heads"],
                    "key_dim": lo["dim"], "value_dim": lo["vdim"], "scale": lo["scale"],
                    "qkv_bias": True, "head_norm": True, "eps": eps, "rotary": lo.get("rot"),
                    "mask": None if mask is None else {"kind": "window", "size": mask["size"]},
                    "names": names})
                right = PartSpec("decay_sum", {
                    "hidden_size": D, "heads": ro["heads"], "key_dim": ro["dim"],
                    "value_dim": ro["vdim"], "decay": list(ro["decay"]), "eps": eps,
                    "names": {"q_weight": f"{rp}.q", "k_weight": f"{rp}.k", "v_weight": f"{rp}.v",
                              "gate_weight": f"{rp}.g", "norm": f"{rp}.norm", "o_weight": f"{rp}.o"}})
                mixer = PartSpec("side_by_side", {
                    "hidden_size": D, "eps": eps, "left": left, "right": right,
                    "names": {"left_norm": f"{lp}.out", "right_norm": f"{rp}.out"}})
            norms = {"mixer": norm(f"{p}.norm1")}
            extras = {"mixer_scale": PartSpec("channel_scale", {"size": D, "names": {"weight": f"{p}.ls1"}}),
                      "branch_factor": PartSpec("constant", {"value": self.residual_mult})}
            ff, mlp = None, layer.mlp
            if mlp is not None:
                norms["feed_forward"] = norm(f"{p}.norm2")
                extras["feed_forward_scale"] = PartSpec(
                    "channel_scale", {"size": D, "names": {"weight": f"{p}.ls2"}})
                if mlp["kind"] == "dense":
                    ff = PartSpec("dense_ff", {
                        "hidden_size": D, "intermediate_size": mlp["ff"], "activation": "relu2",
                        "bias": True,
                        "names": {"up": f"{p}.mlp.up", "down": f"{p}.mlp.down",
                                  "up_bias": f"{p}.mlp.up.b", "down_bias": f"{p}.mlp.down.b"}})
                else:
                    r = mlp["router"]
                    E = r["experts"]
                    ff = PartSpec("routed_moe", {
                        "hidden_size": D, "experts": E, "identity": r.get("identity", 0),
                        "top": r["top"], "groups": r.get("groups"), "correction": True,
                        "expert_ff": mlp["expert"]["ff"],
                        "names": {"router": f"{p}.mlp.router", "correction": f"{p}.mlp.correction",
                                  "gate": [f"{p}.mlp.e{e}.gate" for e in range(E)],
                                  "up": [f"{p}.mlp.e{e}.up" for e in range(E)],
                                  "down": [f"{p}.mlp.e{e}.down" for e in range(E)]}})
            layers.append(LayerSpec(prefix=p, mixer=mixer, feed_forward=ff, norms=norms,
                                    arrangement="parallel_branches", extras=extras))
        spec = ModelSpec(
            architecture=ARCHITECTURE, hidden_size=D, vocab_size=self.vocab,
            max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D,
                                                   "scale": self.embedding_scale,
                                                   "names": {"weight": "embed"}}),
            layers=tuple(layers),
            # every run of a looped layer keeps a cache and a state of its own
            schedule=tuple(RunSpec(i, add_embedding=again) for i, again in self.runs()),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": D, "tied": False,
                                      "names": {"weight": "head", "tied_to": "embed"}}))
        spec.validate()
        return spec
