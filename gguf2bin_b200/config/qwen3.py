"""Qwen3 dense: the typed configuration read from ``config.json`` and its
translation into a ``ModelSpec``.

Defaults follow the reference's ``read_cfg`` (src/l4_gbin.c:67-81): kv heads default
to the head count, head_dim to hidden/heads, eps to 1e-6, rope theta to 1e6 for this
architecture.  The reference implements no bias, no rope scaling and no sliding
window for it (include/g2b.h:19-23 has no bias role; src/l3_math.c:84-102 has no
scaling), so a configuration that asks for one is refused instead of ignored.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .specs import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Qwen3ForCausalLM"


def _as_int(d: Mapping[str, Any], key: str, default=None) -> int:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: missing required key {key!r}")
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json: {key!r} must be an integer, got {v!r}")
    return int(v)


def _as_float(d: Mapping[str, Any], key: str, default: float) -> float:
    v = d.get(key, default)
    if v is None:
        return float(default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {key!r} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    eos_token_ids: tuple = ()

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "Qwen3Config":
        nh = _as_int(d, "num_attention_heads")
        hidden = _as_int(d, "hidden_size")
        head_dim = d.get("head_dim")
        if head_dim is None:
            if nh <= 0 or hidden % nh:
                raise ConfigError("config.json: head_dim absent and hidden_size is not a "
                                  "multiple of num_attention_heads")
            head_dim = hidden // nh
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        cfg = Qwen3Config(
            hidden_size=hidden,
            intermediate_size=_as_int(d, "intermediate_size"),
            num_hidden_layers=_as_int(d, "num_hidden_layers"),
            num_attention_heads=nh,
            num_key_value_heads=_as_int(d, "num_key_value_heads", nh),
            head_dim=_as_int({"head_dim": head_dim}, "head_dim"),
            vocab_size=_as_int(d, "vocab_size"),
            max_position_embeddings=_as_int(d, "max_position_embeddings", 2048),
            rms_norm_eps=_as_float(d, "rms_norm_eps", 1e-6),
            rope_theta=_as_float(d, "rope_theta", 1e6),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            eos_token_ids=eos_ids,
        )
        cfg._check(d)
        return cfg

    def _check(self, d: Mapping[str, Any]) -> None:
        for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"config.json: {key} must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads ({self.num_attention_heads}) is not a multiple "
                f"of num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim ({self.head_dim}) must be even for the "
                              "half-split rotation")
        if not (self.rms_norm_eps > 0) or not (self.rope_theta > 0):
            raise ConfigError("config.json: rms_norm_eps and rope_theta must be positive")
        # options the reference has no code for: refuse, never ignore
        if d.get("attention_bias"):
            raise ConfigError("config.json: attention_bias=true is not supported (the reference's "
                              "Qwen3 path has no bias tensors)")
        if d.get("mlp_bias"):
            raise ConfigError("config.json: mlp_bias=true is not supported")
        if d.get("rope_scaling") not in (None, {}):
            rs = d.get("rope_scaling")
            if not (isinstance(rs, Mapping) and rs.get("rope_type", rs.get("type")) == "default"):
                raise ConfigError(f"config.json: rope_scaling={rs!r} is not supported (plain "
                                  "rotary positions only)")
        if d.get("use_sliding_window"):
            raise ConfigError("config.json: use_sliding_window=true is not supported for "
                              f"{ARCHITECTURE} (full attention only)")
        lt = d.get("layer_types")
        if lt is not None and any(t != "full_attention" for t in lt):
            raise ConfigError("config.json: layer_types other than 'full_attention' are not "
                              f"supported for {ARCHITECTURE}")
        if d.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"config.json: hidden_act={d.get('hidden_act')!r} is not supported "
                              "(SiLU-gated feed-forward only)")

    # ------------------------------------------------------------------
    def to_dict(self) -> dict:
        """A config.json dict that reads back to this configuration."""
        d = dict(
            architectures=[ARCHITECTURE], model_type="qwen3",
            hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
            num_hidden_layers=self.num_hidden_layers,
            num_attention_heads=self.num_attention_heads,
            num_key_value_heads=self.num_key_value_heads, head_dim=self.head_dim,
            vocab_size=self.vocab_size, max_position_embeddings=self.max_position_embeddings,
            rms_norm_eps=self.rms_norm_eps, rope_theta=self.rope_theta,
            tie_word_embeddings=self.tie_word_embeddings, hidden_act="silu",
            attention_bias=False, rope_scaling=None, use_sliding_window=False,
        )
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        return d

    def to_model_spec(self, source: Mapping[str, Any] | None = None) -> ModelSpec:
        """Pre-norm blocks of (grouped-query attention with per-head RMSNorm on Q and K
        and half-split rotary positions) and (SiLU-gated feed-forward), as in
        src/l5_model.c:493-598; final RMSNorm and an lm_head that is the embedding
        matrix when tied (src/l5_model.c:600-605)."""
        norm = PartSpec.make("rmsnorm", eps=self.rms_norm_eps)
        position = PartSpec.make("rope_neox", theta=self.rope_theta, rotary_dim=self.head_dim)
        mixer = PartSpec.make(
            "gqa_attention", n_heads=self.num_attention_heads,
            n_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
            qk_norm=PartSpec.make("rmsnorm", eps=self.rms_norm_eps), position=position,
            window=0, scale=None,
            names=(("q", "self_attn.q_proj.weight"), ("k", "self_attn.k_proj.weight"),
                   ("v", "self_attn.v_proj.weight"), ("o", "self_attn.o_proj.weight"),
                   ("q_norm", "self_attn.q_norm.weight"), ("k_norm", "self_attn.k_norm.weight")))
        ffn = PartSpec.make(
            "swiglu", intermediate_size=self.intermediate_size,
            names=(("gate", "mlp.gate_proj.weight"), ("up", "mlp.up_proj.weight"),
                   ("down", "mlp.down_proj.weight")))
        block = PartSpec.make("prenorm", names=(("mixer_norm", "input_layernorm.weight"),
                                                ("ffn_norm", "post_attention_layernorm.weight")))
        layers = tuple(LayerSpec(block=block, mixer=mixer, feed_forward=ffn, norm=norm,
                                 prefix=f"model.layers.{i}.")
                       for i in range(self.num_hidden_layers))
        spec = ModelSpec(
            architecture=ARCHITECTURE, hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings, layers=layers,
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            embedding=PartSpec.make("token_embedding", name="model.embed_tokens.weight"),
            final_norm=PartSpec.make("rmsnorm", eps=self.rms_norm_eps, name="model.norm.weight"),
            head=PartSpec.make("lm_head", tied=self.tie_word_embeddings, name="lm_head.weight"),
            stop_token_ids=self.eos_token_ids, source=dict(source or self.to_dict()))
        spec.validate()
        return spec
