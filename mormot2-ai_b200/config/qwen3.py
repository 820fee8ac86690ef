"""The typed configuration of the Qwen3 dense decoder, read from its own config.json keys.

Keys, required keys, refusals and bounds follow the reference's
``TQwen3Model.LoadConfig`` (``model.qwen3.pas:216-313``), its window rules
(``model.qwen3.pas:327-403``) and ``TDecoderModel.CheckConfig`` (``decoder.pas:1588-1608``).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Any, Dict, Tuple

from ..errors import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, Run

# model.qwen3.pas:216-220; head_dim is required too for Qwen3 (no hidden/heads fallback,
# model.qwen3.pas:245-246)
REQUIRED_KEYS = (
    "vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
    "num_key_value_heads", "intermediate_size", "max_position_embeddings",
    "rms_norm_eps", "hidden_act", "head_dim",
)


def _integer(doc: Dict[str, Any], key: str, source: str) -> int:
    value = doc[key]
    if isinstance(value, bool) or not isinstance(value, int):
        if isinstance(value, float) and value == int(value):
            return int(value)
        raise ConfigError(f"{source}: \"{key}\" is {value!r}, not an integer")
    return value


def _number(value: Any, key: str, source: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{source}: \"{key}\" is {value!r}, not a number")
    return float(value)


@dataclass(frozen=True)
class Qwen3Config:
    """Hyper-parameters of a Qwen3 dense model (``TDecoderConfig``, ``decoder.pas:158-225``).

    ``layer_windows[i]`` is the sliding window of layer ``i`` (0: every earlier key).
    """
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    layer_windows: Tuple[int, ...] = ()

    ARCHITECTURE = "Qwen3ForCausalLM"
    MODEL_TYPE = "qwen3"

    def __post_init__(self):
        if not self.layer_windows and 0 < self.num_hidden_layers <= 1024:
            object.__setattr__(self, "layer_windows", (0,) * self.num_hidden_layers)

    # ------------------------------------------------------------------ derived sizes
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_file(cls, path: str) -> "Qwen3Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        try:
            with open(path, "r", encoding="utf-8") as f:
                doc = json.load(f)
        except (OSError, ValueError) as e:
            raise ConfigError(f"cannot read {path}: {e}") from None
        return cls.from_dict(doc, path)

    @classmethod
    def from_dict(cls, doc: Dict[str, Any], source: str = "config") -> "Qwen3Config":
        if not isinstance(doc, dict):
            raise ConfigError(f"{source} is no JSON object")
        # decoder.pas:1498-1500
        if doc.get("model_type") != cls.MODEL_TYPE:
            raise ConfigError(
                f"{source}: model_type \"{doc.get('model_type')}\" is not {cls.MODEL_TYPE}")
        for key in REQUIRED_KEYS:
            if key not in doc:
                raise ConfigError(f"{source} has no \"{key}\"")
        if doc["hidden_act"] != "silu":
            raise ConfigError(f"{source}: hidden_act \"{doc['hidden_act']}\" not supported")
        if doc.get("attention_bias") or doc.get("mlp_bias"):
            raise ConfigError(f"{source}: attention_bias or mlp_bias not supported")
        # rope_theta at the top level or in rope_parameters; plain RoPE only
        # (model.qwen3.pas:251-269)
        rope = doc.get("rope_parameters")
        if isinstance(rope, dict):
            if rope.get("rope_type") not in (None, "", "default"):
                raise ConfigError(f"{source}: rope_type \"{rope.get('rope_type')}\" not supported")
            theta = rope.get("rope_theta", 0)
        else:
            theta = doc.get("rope_theta", 0)
        scaling = doc.get("rope_scaling")
        if isinstance(scaling, dict) and len(scaling) > 0:
            raise ConfigError(f"{source}: rope_scaling not supported")
        layers = _integer(doc, "num_hidden_layers", source)
        if not 0 < layers <= 1024:
            raise ConfigError(f"{source} has an invalid or unsupported shape: {layers} layers")
        cfg = cls(
            vocab_size=_integer(doc, "vocab_size", source),
            hidden_size=_integer(doc, "hidden_size", source),
            num_hidden_layers=layers,
            num_attention_heads=_integer(doc, "num_attention_heads", source),
            num_key_value_heads=_integer(doc, "num_key_value_heads", source),
            head_dim=_integer(doc, "head_dim", source),
            intermediate_size=_integer(doc, "intermediate_size", source),
            max_position_embeddings=_integer(doc, "max_position_embeddings", source),
            rms_norm_eps=_number(doc["rms_norm_eps"], "rms_norm_eps", source),
            rope_theta=_number(theta, "rope_theta", source),
            tie_word_embeddings=bool(doc.get("tie_word_embeddings", False)),
            layer_windows=cls._windows(doc, layers, source),
        )
        cfg.check(source)
        return cfg

    @staticmethod
    def _windows(doc: Dict[str, Any], layers: int, source: str) -> Tuple[int, ...]:
        """The window of every layer (``model.qwen3.pas:327-403``): none unless
        ``use_sliding_window``; then ``layer_types``, else the layers from
        ``max_window_layers`` (default 28) on; ``sliding_window`` defaults to 4096."""
        window = 0
        if doc.get("use_sliding_window"):
            if "sliding_window" not in doc:
                window = 4096
            elif doc["sliding_window"] is not None:
                w = doc["sliding_window"]
                if isinstance(w, bool) or not isinstance(w, int) or not 0 < w <= 1 << 24:
                    raise ConfigError(f"{source}: a sliding_window of {w!r}")
                window = w
        windows = [0] * layers
        types = doc.get("layer_types")
        if isinstance(types, list):
            if len(types) != layers:
                raise ConfigError(f"{source}: {len(types)} layer types for {layers} layers")
            for i, t in enumerate(types):
                if t == "sliding_attention":
                    if window <= 0:
                        raise ConfigError(f"{source}: layer {i} slides without a sliding window")
                    windows[i] = window
                elif t != "full_attention":
                    raise ConfigError(f"{source}: layer type \"{t}\" not supported")
            return tuple(windows)
        if window == 0:
            return tuple(windows)
        first = doc.get("max_window_layers", 28)
        if isinstance(first, bool) or not isinstance(first, int):
            raise ConfigError(f"{source}: max_window_layers is {first!r}")
        for i in range(max(first, 0), layers):
            windows[i] = window
        return tuple(windows)

    def check(self, source: str = "config") -> None:
        """Bounds of every value on its own (``decoder.pas:1596-1608``)."""
        c = self
        ok = (
            0 < c.vocab_size <= 1 << 22 and 0 < c.hidden_size <= 1 << 16
            and 0 < c.num_hidden_layers <= 1024
            and 0 < c.num_attention_heads <= 1 << 12
            and 0 < c.num_key_value_heads <= c.num_attention_heads
            and c.num_attention_heads % c.num_key_value_heads == 0
            and 0 < c.head_dim <= 1024 and c.head_dim % 2 == 0
            and c.num_attention_heads * c.head_dim <= 1 << 16
            and 0 < c.intermediate_size <= 1 << 18
            and 0 < c.max_position_embeddings <= 1 << 24
            and 0 < c.rms_norm_eps <= 1 and math.isfinite(c.rms_norm_eps)
            and 1 < c.rope_theta <= 1e12
        )
        if not ok:
            raise ConfigError(f"{source} has an invalid or unsupported shape: {self}")
        if len(c.layer_windows) not in (0, c.num_hidden_layers):
            raise ConfigError(
                f"{source}: {len(c.layer_windows)} layer kinds for {c.num_hidden_layers} layers")
        for i, w in enumerate(c.layer_windows):
            if not 0 <= w <= 1 << 24:
                raise ConfigError(f"{source} has a window of {w} in layer {i}")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        """The config.json of this configuration (what the random-weights mode writes)."""
        doc: Dict[str, Any] = {
            "architectures": [self.ARCHITECTURE],
            "model_type": self.MODEL_TYPE,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "hidden_act": "silu",
        }
        windows = self.windows()
        if any(windows):
            doc["use_sliding_window"] = True
            doc["sliding_window"] = max(windows)
            doc["layer_types"] = [
                "sliding_attention" if w else "full_attention" for w in windows]
        else:
            doc["use_sliding_window"] = False
        return doc

    def windows(self) -> Tuple[int, ...]:
        return self.layer_windows

    # ------------------------------------------------------------------ the model as data
    def to_model_spec(self) -> ModelSpec:
        """Layers from parts: GQA attention with per-head q/k RMSNorm and rotate-half RoPE,
        SwiGLU, RMSNorm, in a pre-norm residual block; tensor names are Hugging Face's
        (``model.qwen3.pas:544-604``, ``:628-630``)."""
        c = self
        layers = []
        schedule = []
        for i, window in enumerate(c.windows()):
            norm = lambda name: PartSpec("rmsnorm", {
                "name": name, "size": c.hidden_size, "eps": c.rms_norm_eps})
            layers.append(LayerSpec(
                block=PartSpec("prenorm_residual"),
                mixer=PartSpec("gqa_attention", {
                    "hidden_size": c.hidden_size,
                    "heads": c.num_attention_heads,
                    "kv_heads": c.num_key_value_heads,
                    "head_dim": c.head_dim,
                    "head_norm_eps": c.rms_norm_eps,   # q_norm/k_norm: same eps (decoder.pas:2662-2668)
                    "position": "rope",
                    "window": window,
                    "scale": 1.0 / math.sqrt(c.head_dim),  # backend.cpu.pas:1377-1380
                    "names": {
                        "q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight",
                        "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight",
                        "q_norm": "self_attn.q_norm.weight",
                        "k_norm": "self_attn.k_norm.weight"},
                }),
                feed_forward=PartSpec("swiglu", {
                    "hidden_size": c.hidden_size,
                    "intermediate_size": c.intermediate_size,
                    "names": {"gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight",
                              "down": "mlp.down_proj.weight"},
                }),
                norms={"mixer": norm("input_layernorm.weight"),
                       "feed_forward": norm("post_attention_layernorm.weight")},
                prefix=f"model.layers.{i}.",
            ))
            schedule.append(Run(layer=i, cache_line=i, writes_cache=True))
        return ModelSpec(
            architecture=c.ARCHITECTURE,
            vocab_size=c.vocab_size,
            hidden_size=c.hidden_size,
            max_positions=c.max_position_embeddings,
            embedding=PartSpec("token_embedding", {
                "name": "model.embed_tokens.weight", "vocab_size": c.vocab_size,
                "hidden_size": c.hidden_size}),
            positions={"rope": PartSpec("rope_half", {
                "theta": c.rope_theta, "rot_dim": c.head_dim})},
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=PartSpec("rmsnorm", {
                "name": "model.norm.weight", "size": c.hidden_size, "eps": c.rms_norm_eps}),
            head=PartSpec("lm_head", {
                "name": "lm_head.weight", "tied": c.tie_word_embeddings,
                "tied_to": "model.embed_tokens.weight",
                "vocab_size": c.vocab_size, "hidden_size": c.hidden_size}),
        )
