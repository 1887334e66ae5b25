"""Typed configuration of the Luvavik design and its model spec.

A Luvavik model is a pre-norm decoder whose layers differ: each entry of ``layers`` names its
mixer (``rglru``: a recurrent block with a real-gated linear recurrent unit; ``latent_attention``:
attention over a cached latent) with the mixer's sizes, and its feed-forward (dense and gated, a
mixture of experts, or none).  ``loop`` runs a span of layers several times in a row with the same
weights, every pass with caches and states of its own, and adds a per-pass vector to the residual
stream before each pass.  Both residual updates of a layer are multiplied by ``residual_mult``; the
logits by ``logit_scale``.  config.json gives every size and every constant that may differ between
models; the tensor names (``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``embed``, ``head``,
``final.norm``, ``loop.step``) are fixed.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Optional

from .qwen3 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Luvavik"
DEFAULT_MAX_POSITIONS = 1 << 17       # the design has no position limit; the engine needs one for its tables

_MIXER_KEYS = {
    "rglru": ("width", "blocks", "conv"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"),
}


def _positive(where: str, d: dict, keys) -> None:
    for k in keys:
        if k not in d:
            raise ConfigError(f"config.json: {where} lacks {k!r}")
        if isinstance(d[k], (int, float)) and not isinstance(d[k], bool) and not d[k] > 0:
            raise ConfigError(f"config.json: {where}.{k} must be positive, got {d[k]!r}")


@dataclass(frozen=True)
class LuvavikConfig:
    vocab_size: int
    hidden_size: int
    layers: tuple[dict, ...]               # as in config.json: type, mixer, mlp
    norm_eps: float
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    loop: Optional[dict] = None            # start, stop, times
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: tuple[int, ...] = field(default_factory=tuple)
    model_type: str = "luvavik"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "LuvavikConfig":
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
        loop = d.get("loop")
        cfg = cls(
            vocab_size=int(d["vocab"]), hidden_size=int(d["width"]),
            layers=tuple(copy.deepcopy(layer) for layer in d["layers"]),
            norm_eps=float(d["norm"]["eps"]), residual_mult=float(d.get("residual_mult", 1.0)),
            logit_scale=float(d.get("logit_scale", 1.0)),
            loop=None if not loop else {k: int(loop[k]) for k in ("start", "stop", "times") if k in loop},
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
            kind = layer.get("type")
            if kind not in _MIXER_KEYS:
                raise ConfigError(f"config.json: layer {i} has the unknown mixer type {kind!r}; known: {', '.join(_MIXER_KEYS)}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"config.json: layer {i} lacks its mixer's sizes")
            _positive(f"layers[{i}].mixer", mixer, _MIXER_KEYS[kind])
            if kind == "rglru" and mixer["width"] % mixer["blocks"]:
                raise ConfigError(f"config.json: layer {i}: width {mixer['width']} does not divide into {mixer['blocks']} blocks")
            if kind == "latent_attention":
                rot = mixer["rot"]
                _positive(f"layers[{i}].mixer.rot", rot, ("base", "dims"))
                if rot["dims"] % 2 or rot["dims"] > mixer["rot_dim"]:
                    raise ConfigError(f"config.json: layer {i}: rot.dims {rot['dims']} must be even and at most rot_dim")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") == "dense":
                _positive(f"layers[{i}].mlp", mlp, ("ff",))
            elif mlp.get("kind") == "moe":
                _positive(f"layers[{i}].mlp.expert", mlp.get("expert") or {}, ("ff",))
                router = mlp.get("router") or {}
                _positive(f"layers[{i}].mlp.router", router, ("experts", "top"))
                if router["top"] > router["experts"] + int(router.get("identity", 0)):
                    raise ConfigError(f"config.json: layer {i}: more experts chosen than there are")
            else:
                raise ConfigError(f"config.json: layer {i} has the unknown feed-forward kind {mlp.get('kind')!r}")
        if self.loop is not None:
            for k in ("start", "stop", "times"):
                if k not in self.loop:
                    raise ConfigError(f"config.json: loop lacks {k!r}")
            if not (0 <= self.loop["start"] < self.loop["stop"] <= len(self.layers)) or self.loop["times"] < 1:
                raise ConfigError(f"config.json: loop {self.loop} does not fit {len(self.layers)} layers")

    def describe(self) -> list[str]:
        """Lines for the command line's model inspection."""
        lines = [f"hidden_size: {self.hidden_size}", f"vocab_size: {self.vocab_size}", f"num_layers: {len(self.layers)}",
                 f"norm_eps: {self.norm_eps:e}", f"residual_mult: {self.residual_mult}", f"logit_scale: {self.logit_scale}"]
        if self.loop is not None:
            lines.append(f"loop: layers {self.loop['start']}..{self.loop['stop'] - 1} run {self.loop['times']} times")
        for i, layer in enumerate(self.layers):
            mixer = ", ".join(f"{k}={v}" for k, v in sorted(layer["mixer"].items()) if not isinstance(v, dict))
            mlp = layer.get("mlp")
            if mlp is None:
                ff = "none"
            elif mlp["kind"] == "dense":
                ff = f"dense ff={mlp['ff']}"
            else:
                r = mlp["router"]
                ff = f"moe experts={r['experts']} top={r['top']} identity={r.get('identity', 0)} ff={mlp['expert']['ff']}"
            lines.append(f"layer {i}: {layer['type']} ({mixer}); feed-forward: {ff}")
        return lines

    def to_dict(self) -> dict:
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
            "layers": [copy.deepcopy(layer) for layer in self.layers], "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult, "logit_scale": self.logit_scale,
        }
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d


# ---------------------------------------------------------------------- the family
def _mixer_spec(cfg: LuvavikConfig, layer: dict) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "rglru":
        return PartSpec("rglru", {"hidden_size": cfg.hidden_size, "width": int(m["width"]), "blocks": int(m["blocks"]),
                                  "conv_taps": int(m["conv"]), "decay_scale": 8.0})
    rot = m["rot"]
    position = PartSpec("rope", {"head_dim": int(rot["dims"]), "theta": float(rot["base"]),
                                 "max_positions": cfg.max_position_embeddings})
    return PartSpec("latent_attention", {
        "hidden_size": cfg.hidden_size, "num_heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
        "vdim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]), "scale": float(m["scale"]), "norm_eps": cfg.norm_eps,
        "output_gate": True, "window": None, "position": position})


def _ffn_spec(cfg: LuvavikConfig, layer: dict) -> Optional[PartSpec]:
    mlp = layer.get("mlp")
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("swiglu_mlp", {"hidden_size": cfg.hidden_size, "intermediate_size": int(mlp["ff"]),
                                       "activation": "gelu_tanh", "names": ("gate", "up", "down")})
    router = mlp["router"]
    return PartSpec("routed_experts", {
        "hidden_size": cfg.hidden_size, "intermediate_size": int(mlp["expert"]["ff"]), "experts": int(router["experts"]),
        "identity_experts": int(router.get("identity", 0)), "top": int(router["top"]), "renormalize": False,
        "correction": True, "activation": "relu2", "score": "softmax", "expert_names": "e{}."})


def luvavik_model_spec(cfg: LuvavikConfig) -> ModelSpec:
    H = cfg.hidden_size
    norm = lambda tensor: PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "tensor": tensor})
    layers = []
    for i, layer in enumerate(cfg.layers):
        ffn = _ffn_spec(cfg, layer)
        block = PartSpec("prenorm_block", {
            "mixer": _mixer_spec(cfg, layer), "mixer_norm": norm("norm1"), "mixer_name": "mix.",
            "feed_forward": ffn, "ffn_norm": norm("norm2") if ffn is not None else None, "ffn_name": "mlp.",
            "mixer_norm_name": "", "ffn_norm_name": "", "verbatim_names": True, "residual_scale": cfg.residual_mult})
        layers.append(LayerSpec(block=block, prefix=f"l{i}."))
    n = len(layers)
    tables = ()
    if cfg.loop is None:
        schedule = tuple(ScheduleEntry(i) for i in range(n))
    else:
        start, stop, times = cfg.loop["start"], cfg.loop["stop"], cfg.loop["times"]
        schedule = [ScheduleEntry(i) for i in range(start)]
        for t in range(times):      # every pass has caches of its own (no cache name: one per entry)
            schedule += [ScheduleEntry(i, pre_add=("loop.step", t) if i == start else None) for i in range(start, stop)]
        schedule += [ScheduleEntry(i) for i in range(stop, n)]
        schedule = tuple(schedule)
        tables = (("loop.step", (times, H)),)
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=cfg.vocab_size, hidden_size=H, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": H, "name": "embed", "suffix": ""}),
        layers=tuple(layers), schedule=schedule,
        final_norm=PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "tensor": "norm", "prefix": "final."}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": H, "name": "head", "suffix": "",
                                  "tied_to": None, "scale": cfg.logit_scale}),
        eos_token_ids=cfg.eos_token_id, tables=tables)
