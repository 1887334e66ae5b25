"""Typed configuration of the Rogosun design and its model spec.

A Rogosun model is a decoder whose layers norm a sublayer's OUTPUT, x <- x + norm1(mixer(x)), then
x <- x + norm2(ff(x)), and differ in their mixers: ``gla`` (gated linear attention: a matrix-valued state
per head with a decay per key channel) or ``parallel`` (two mixers side by side on the same input: ``left``,
grouped-query attention with query/key norm, rotation of part of the head with linearly scaled positions, a
softmax with a sink, and the raw keys as values; ``right``, a gated delta rule behind short convolutions; the
result is left_scale * left + right_scale * right).  The feed-forward of a layer is dense (the square of relu,
no gate), a mixture of gated experts with a sigmoid router over groups of experts and a shared expert, or
absent.  config.json gives every size and every constant that may differ between models; the ranks of the
low-rank pairs are read from the tensors' shapes; the tensor names (``l<i>.norm1``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``embed``, ``head``, ``final.norm``) are fixed.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Optional

from .luvavik import _positive
from .qwen3 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Rogosun"
DEFAULT_MAX_POSITIONS = 1 << 17       # the design has no position limit; the engine needs one for its tables

_GLA_KEYS = ("heads", "dim", "vdim", "tau")
_LEFT_KEYS = ("heads", "kv_heads", "dim", "scale", "rot")
_RIGHT_KEYS = ("heads", "kv_heads", "dim", "vdim", "conv")


@dataclass(frozen=True)
class RogosunConfig:
    vocab_size: int
    hidden_size: int
    layers: tuple[dict, ...]               # as in config.json: type, mixer, mlp
    norm_eps: float
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: tuple[int, ...] = field(default_factory=tuple)
    model_type: str = "rogosun"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "RogosunConfig":
        for k in ("vocab", "width", "layers", "norm"):
            if k not in d:
                raise ConfigError(f"config.json lacks required key {k!r}")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: `layers` must be a list with at least one layer")
        if "eps" not in d["norm"]:
            raise ConfigError("config.json: norm lacks 'eps'")
        eos = d.get("eos_token_id", ())
        if isinstance(eos, int):
            eos = (eos,)
        cfg = cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]),
                  layers=tuple(copy.deepcopy(layer) for layer in d["layers"]), norm_eps=float(d["norm"]["eps"]),
                  max_position_embeddings=int(d.get("max_position_embeddings", DEFAULT_MAX_POSITIONS)),
                  eos_token_id=tuple(int(t) for t in (eos or ())))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0:
            raise ConfigError("vocab and width must be positive")
        if not self.norm_eps >= 0.0:
            raise ConfigError(f"norm.eps must be >= 0, got {self.norm_eps}")
        for i, layer in enumerate(self.layers):
            kind, mixer = layer.get("type"), layer.get("mixer")
            if kind not in ("gla", "parallel"):
                raise ConfigError(f"config.json: layer {i} has the unknown mixer type {kind!r}; known: gla, parallel")
            if not isinstance(mixer, dict):
                raise ConfigError(f"config.json: layer {i} lacks its mixer's sizes")
            where = f"layers[{i}].mixer"
            if kind == "gla":
                _positive(where, mixer, _GLA_KEYS)
            else:
                for side, keys in (("left", _LEFT_KEYS), ("right", _RIGHT_KEYS)):
                    if not isinstance(mixer.get(side), dict):
                        raise ConfigError(f"config.json: {where} lacks {side!r}")
                    _positive(f"{where}.{side}", mixer[side], keys)
                    if mixer[side]["heads"] % mixer[side]["kv_heads"]:
                        raise ConfigError(f"config.json: {where}.{side}: {mixer[side]['heads']} heads do not divide into "
                                          f"{mixer[side]['kv_heads']} kv heads")
                for k in ("left_scale", "right_scale"):
                    if k not in mixer:
                        raise ConfigError(f"config.json: {where} lacks {k!r}")
                left = mixer["left"]
                if "vdim" in left and left["vdim"] != left["dim"]:
                    raise ConfigError(f"config.json: {where}.left: the values are the keys, so vdim must equal dim")
                rot = left["rot"]
                _positive(f"{where}.left.rot", rot, ("base", "dims"))
                if rot["dims"] % 2 or rot["dims"] > left["dim"]:
                    raise ConfigError(f"config.json: {where}.left.rot.dims {rot['dims']} must be even and at most dim")
                if rot.get("scaling") is not None:
                    _positive(f"{where}.left.rot.scaling", rot["scaling"], ("factor",))
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") == "dense":
                _positive(f"layers[{i}].mlp", mlp, ("ff",))
            elif mlp.get("kind") == "moe":
                _positive(f"layers[{i}].mlp.expert", mlp.get("expert") or {}, ("ff",))
                router = mlp.get("router") or {}
                _positive(f"layers[{i}].mlp.router", router, ("experts", "top"))
                groups = router.get("groups")
                if groups is not None:
                    _positive(f"layers[{i}].mlp.router.groups", groups, ("count", "keep"))
                    if router["experts"] % groups["count"] or groups["keep"] > groups["count"]:
                        raise ConfigError(f"config.json: layer {i}: {router['experts']} experts do not form {groups['count']} "
                                          f"groups of which {groups['keep']} are kept")
                count, keep = (groups["count"], groups["keep"]) if groups is not None else (1, 1)
                if router["top"] > keep * (router["experts"] // count):
                    raise ConfigError(f"config.json: layer {i}: more experts chosen than the kept groups hold")
                if mlp.get("shared") is not None:
                    _positive(f"layers[{i}].mlp.shared", mlp["shared"], ("ff",))
            else:
                raise ConfigError(f"config.json: layer {i} has the unknown feed-forward kind {mlp.get('kind')!r}")

    def describe(self) -> list[str]:
        """Lines for the command line's model inspection."""
        lines = [f"hidden_size: {self.hidden_size}", f"vocab_size: {self.vocab_size}", f"num_layers: {len(self.layers)}",
                 f"norm_eps: {self.norm_eps:e}"]
        flat = lambda m: ", ".join(f"{k}={v}" for k, v in sorted(m.items()) if not isinstance(v, dict))
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            if layer["type"] == "gla":
                mixer = flat(m)
            else:
                mixer = (f"left {m['left_scale']} x attention ({flat(m['left'])}, rot {flat(m['left']['rot'])}); "
                         f"right {m['right_scale']} x delta rule ({flat(m['right'])})")
            mlp = layer.get("mlp")
            if mlp is None:
                ff = "none"
            elif mlp["kind"] == "dense":
                ff = f"dense ff={mlp['ff']}"
            else:
                r = mlp["router"]
                g = r.get("groups") or {"count": 1, "keep": 1}
                ff = (f"moe experts={r['experts']} top={r['top']} groups={g['count']} keep={g['keep']} ff={mlp['expert']['ff']}"
                      + (f" shared ff={mlp['shared']['ff']}" if mlp.get("shared") else ""))
            lines.append(f"layer {i}: {layer['type']} ({mixer}); feed-forward: {ff}")
        return lines

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                             "layers": [copy.deepcopy(layer) for layer in self.layers], "norm": {"eps": self.norm_eps}}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d


# ---------------------------------------------------------------------- the family
def _gla_spec(cfg: RogosunConfig, m: dict) -> PartSpec:
    # `rank` is not a key of the design (the tensors give it); the random-weights mode takes it as the size to draw
    return PartSpec("gated_linear_attention", {
        "hidden_size": cfg.hidden_size, "num_heads": int(m["heads"]), "dim": int(m["dim"]), "vdim": int(m["vdim"]),
        "tau": float(m["tau"]), "norm_eps": cfg.norm_eps, "decay_rank": int(m.get("rank", 16))})


def _parallel_spec(cfg: RogosunConfig, m: dict) -> PartSpec:
    left, right = m["left"], m["right"]
    rot = left["rot"]
    scaling = rot.get("scaling") or {}
    position = PartSpec("rope", {"head_dim": int(rot["dims"]), "theta": float(rot["base"]),
                                 "scaling_factor": float(scaling.get("factor", 1.0)),
                                 "max_positions": cfg.max_position_embeddings})
    attention = PartSpec("gqa_attention", {
        "hidden_size": cfg.hidden_size, "num_heads": int(left["heads"]), "num_kv_heads": int(left["kv_heads"]),
        "head_dim": int(left["dim"]), "qk_norm_eps": cfg.norm_eps, "window": None, "position": position,
        "scale": float(left["scale"]), "sink": 1.0, "values": "keys",
        "names": {"q": "q", "k": "k", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}})
    delta = PartSpec("gated_delta_rule", {
        "hidden_size": cfg.hidden_size, "num_heads": int(right["heads"]), "num_kv_heads": int(right["kv_heads"]),
        "dim": int(right["dim"]), "vdim": int(right["vdim"]), "conv_taps": int(right["conv"]), "norm_eps": cfg.norm_eps,
        "decay_rank": int(right.get("rank", 16)), "gate_rank": int(right.get("gate_rank", right.get("rank", 16)))})
    return PartSpec("parallel_mixer", {"left": attention, "right": delta, "left_scale": float(m["left_scale"]),
                                       "right_scale": float(m["right_scale"]), "left_name": "left.", "right_name": "right."})


def _ffn_spec(cfg: RogosunConfig, layer: dict) -> Optional[PartSpec]:
    mlp = layer.get("mlp")
    if mlp is None:
        return None
    H = cfg.hidden_size
    if mlp["kind"] == "dense":
        return PartSpec("plain_mlp", {"hidden_size": H, "intermediate_size": int(mlp["ff"]), "activation": "relu2",
                                      "names": ("up", "down")})
    router = mlp["router"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    shared = None
    if mlp.get("shared") is not None:
        shared = PartSpec("swiglu_mlp", {"hidden_size": H, "intermediate_size": int(mlp["shared"]["ff"]),
                                         "activation": "silu", "names": ("gate", "up", "down")})
    return PartSpec("routed_experts", {
        "hidden_size": H, "intermediate_size": int(mlp["expert"]["ff"]), "experts": int(router["experts"]),
        "top": int(router["top"]), "renormalize": False, "correction": False, "activation": "silu_gated",
        "score": "sigmoid", "groups": int(groups["count"]), "groups_kept": int(groups["keep"]),
        "weight_scale": float(router.get("scale", 1.0)), "expert_names": "e{}.", "shared": shared, "shared_name": "shared."})


def rogosun_model_spec(cfg: RogosunConfig) -> ModelSpec:
    H = cfg.hidden_size
    norm = lambda tensor: PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "tensor": tensor})
    layers = []
    for i, layer in enumerate(cfg.layers):
        mixer = _gla_spec(cfg, layer["mixer"]) if layer["type"] == "gla" else _parallel_spec(cfg, layer["mixer"])
        ffn = _ffn_spec(cfg, layer)
        block = PartSpec("outnorm_block", {
            "mixer": mixer, "mixer_norm": norm("norm1"), "mixer_name": "mix.", "feed_forward": ffn,
            "ffn_norm": norm("norm2") if ffn is not None else None, "ffn_name": "mlp.", "mixer_norm_name": "",
            "ffn_norm_name": "", "verbatim_names": True})
        layers.append(LayerSpec(block=block, prefix=f"l{i}."))
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=cfg.vocab_size, hidden_size=H, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": H, "name": "embed", "suffix": ""}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "tensor": "norm", "prefix": "final."}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": H, "name": "head", "suffix": "", "tied_to": None}),
        eos_token_ids=cfg.eos_token_id)
