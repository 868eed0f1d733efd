"""The Qwen2 dense decoder (`Qwen2ForCausalLM`, model_type "qwen2"): its configuration, read from
the keys of its own config.json, and its description as a list of parts.

What the reference reads and how it derives sizes is in qwen_infer.c:19357-19493; the tensor names
are the checkpoint's own (qwen_infer.c:263-287, :19627-19669).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterable, Optional, Tuple

from ..config.reader import ConfigError, ConfigFields
from ..config.registry import Architecture, register_architecture
from ..parts.spec import (AttentionSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec, Stage,
                          SwiGLUSpec)


@dataclass(frozen=True)
class RopeScaling:
    """config.json's `rope_scaling` object of rope_type "llama3", the only one the reference's
    safetensors loader accepts (qwen_infer.c:19383-19428)."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    qkv_bias: bool
    max_position_embeddings: Optional[int]
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    rope_scaling: Optional[RopeScaling]
    eos_token_ids: Tuple[int, ...]
    bos_token_id: Optional[int]

    architecture = "Qwen2ForCausalLM"
    model_type = "qwen2"

    @classmethod
    def from_fields(cls, f: ConfigFields, tensor_names: Optional[Iterable[str]] = None) -> "Qwen2Config":
        """Required without default, as in the reference (qwen_infer.c:19431-19437):
        num_hidden_layers, hidden_size, intermediate_size, num_attention_heads,
        num_key_value_heads, rope_theta, rms_norm_eps.  vocab_size is required here too, since a
        configuration must stand without a weight file (the reference takes it from the embedding's
        shape and cross-checks the key, :19446-19455; the loader's shape check does that here).

        Whether q/k/v carry a bias is a fact of the tensor list in the reference (:19457-19460);
        with `tensor_names` given it is decided the same way, else by the key `attention_bias`,
        else it is on, as every Qwen2 checkpoint has it."""
        names = set(tensor_names) if tensor_names is not None else None
        nl = f.integer("num_hidden_layers", required=True)
        d = f.integer("hidden_size", required=True)
        im = f.integer("intermediate_size", required=True)
        nh = f.integer("num_attention_heads", required=True)
        nkv = f.integer("num_key_value_heads", required=True)
        theta = f.number("rope_theta", required=True)
        eps = f.number("rms_norm_eps", required=True)
        vocab = f.integer("vocab_size", required=True)

        if nh <= 0 or nkv <= 0 or nh % nkv != 0:
            raise ConfigError(f"{f.origin}: num_attention_heads={nh} not a positive multiple of "
                              f"num_key_value_heads={nkv}")
        hd = f.integer("head_dim")
        if hd is None:
            if d <= 0 or d % nh != 0:
                raise ConfigError(f"{f.origin}: hidden_size={d} not evenly divisible by "
                                  f"num_attention_heads={nh} (cannot derive head_dim)")
            hd = d // nh
        if hd <= 0 or hd % 2 != 0:
            raise ConfigError(f"{f.origin}: head_dim={hd} must be positive and even")
        for key, v in (("num_hidden_layers", nl), ("hidden_size", d), ("intermediate_size", im),
                       ("vocab_size", vocab)):
            if v <= 0:
                raise ConfigError(f"{f.origin}: {key}={v} must be positive")
        if not (theta > 0.0) or not (eps >= 0.0):
            raise ConfigError(f"{f.origin}: rope_theta={theta} must be positive and rms_norm_eps={eps} not negative")

        act = f.string("hidden_act")
        if act is not None and act != "silu":
            raise ConfigError(f"{f.origin}: hidden_act='{act}' is not supported (the feed-forward is "
                              "SwiGLU with SiLU, qwen_infer.c:727-733)")

        bias_key = f.boolean("attention_bias")
        if names is not None:
            qkv_bias = "model.layers.0.self_attn.q_proj.bias" in names
            if bias_key is not None and bias_key != qkv_bias:
                raise ConfigError(f"{f.origin}: attention_bias={bias_key} disagrees with the tensor list "
                                  f"(q_proj.bias {'present' if qkv_bias else 'absent'})")
        else:
            qkv_bias = True if bias_key is None else bias_key

        tie = f.boolean("tie_word_embeddings")
        if names is not None:
            # with a tensor list, presence decides, as in the reference, which never reads the key: the head
            # is lm_head.weight when that tensor exists, else the embedding table (qwen_infer.c:318-319)
            has_head = "lm_head.weight" in names
            if tie is False and not has_head:
                raise ConfigError(f"{f.origin}: tie_word_embeddings=false but the tensor list has no lm_head.weight")
            tie = not has_head
        elif tie is None:
            tie = False

        usw = bool(f.boolean("use_sliding_window", default=False))
        sw = f.integer("sliding_window")
        mwl = f.integer("max_window_layers", default=0)
        if usw and (sw is None or sw <= 0):
            raise ConfigError(f"{f.origin}: use_sliding_window=true needs a positive sliding_window")

        rs = None
        rs_fields = f.mapping("rope_scaling")
        if rs_fields is not None:
            rope_type = rs_fields.string("rope_type") or rs_fields.string("type")
            if rope_type is None:
                raise ConfigError(f"{f.origin} rope_scaling missing 'rope_type'")
            if rope_type != "llama3":
                raise ConfigError(f"{f.origin} rope_scaling.rope_type='{rope_type}' -- only 'llama3' is implemented")
            rs = RopeScaling(
                factor=rs_fields.number("factor", required=True),
                low_freq_factor=rs_fields.number("low_freq_factor", required=True),
                high_freq_factor=rs_fields.number("high_freq_factor", required=True),
                original_max_position_embeddings=rs_fields.integer("original_max_position_embeddings", required=True))
            if rs.high_freq_factor == rs.low_freq_factor:
                raise ConfigError(f"{f.origin} rope_scaling has high_freq_factor==low_freq_factor")
            if rs.factor <= 0 or rs.original_max_position_embeddings <= 0:
                raise ConfigError(f"{f.origin} rope_scaling has non-positive factor or original_max_position_embeddings")

        return cls(vocab_size=vocab, hidden_size=d, intermediate_size=im, num_hidden_layers=nl,
                   num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, rope_theta=theta,
                   rms_norm_eps=eps, tie_word_embeddings=bool(tie), qkv_bias=qkv_bias,
                   max_position_embeddings=f.integer("max_position_embeddings"),
                   use_sliding_window=usw, sliding_window=sw, max_window_layers=mwl, rope_scaling=rs,
                   eos_token_ids=tuple(f.integer_or_list("eos_token_id")),
                   bos_token_id=f.integer("bos_token_id"))

    def layer_window(self, layer: int) -> Optional[int]:
        """With use_sliding_window, layers from max_window_layers on see the last sliding_window
        positions; the others see all.  (The reference runs full attention always.)"""
        if self.use_sliding_window and self.sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    def to_json_dict(self) -> dict:
        """The configuration as config.json keys (what the random-weights mode writes)."""
        out = {
            "architectures": [self.architecture], "model_type": self.model_type,
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "hidden_act": "silu", "rope_theta": self.rope_theta, "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings, "attention_bias": self.qkv_bias,
            "use_sliding_window": self.use_sliding_window, "max_window_layers": self.max_window_layers,
        }
        if self.max_position_embeddings is not None:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.sliding_window is not None:
            out["sliding_window"] = self.sliding_window
        if self.rope_scaling is not None:
            r = self.rope_scaling
            out["rope_scaling"] = {"rope_type": "llama3", "factor": r.factor,
                                   "low_freq_factor": r.low_freq_factor,
                                   "high_freq_factor": r.high_freq_factor,
                                   "original_max_position_embeddings": r.original_max_position_embeddings}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out


def llama3_frequency_scale(theta: float, rot: int, r: RopeScaling) -> Tuple[float, ...]:
    """Per-frequency ratio of rope_type "llama3" (rope_llama3_scale.h:18-28): wavelengths above
    orig/low_freq_factor are divided by `factor`, those below orig/high_freq_factor are kept, and
    the band between is blended.  The reference computes the ratio in 32-bit, operation by operation;
    so does this (with `powf` as the correctly rounded power), and the ratios come out bit for bit."""
    import numpy as np
    f = np.float32
    theta32, factor, low, high = f(theta), f(r.factor), f(r.low_freq_factor), f(r.high_freq_factor)
    orig = f(r.original_max_position_embeddings)
    out = []
    low_wl = orig / low
    high_wl = orig / high
    for i in range(rot // 2):
        exponent = -(f(2.0) * f(i)) / f(rot)
        inv = f(np.float64(theta32) ** np.float64(exponent))
        wl = (f(2.0) * f(math.pi)) / inv
        if wl > low_wl:
            out.append(float(f(1.0) / factor))
        elif wl < high_wl:
            out.append(1.0)
        else:
            smooth = (orig / wl - low) / (high - low)
            out.append(float((f(1.0) - smooth) / factor + smooth))
    return tuple(out)


def build_spec(cfg: Qwen2Config) -> ModelSpec:
    """Every layer: RMSNorm, grouped-query attention with q/k/v bias and split-half RoPE over the
    whole head, residual add, RMSNorm, SwiGLU, residual add (qwen_infer.c:1447-1577); then the
    final RMSNorm and the head, which is the embedding table when tied (:1585-1599)."""
    scale = None
    if cfg.rope_scaling is not None:
        scale = llama3_frequency_scale(cfg.rope_theta, cfg.head_dim, cfg.rope_scaling)
    position = PositionSpec(kind="rope", rotary_dim=cfg.head_dim, theta=cfg.rope_theta,
                            pairing="split_half", freq_scale=scale)
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        names = {
            "mixer_norm.weight": p + "input_layernorm.weight",
            "feed_forward_norm.weight": p + "post_attention_layernorm.weight",
            "mixer.q_proj.weight": p + "self_attn.q_proj.weight",
            "mixer.k_proj.weight": p + "self_attn.k_proj.weight",
            "mixer.v_proj.weight": p + "self_attn.v_proj.weight",
            "mixer.o_proj.weight": p + "self_attn.o_proj.weight",
            "mixer.q_proj.bias": p + "self_attn.q_proj.bias",
            "mixer.k_proj.bias": p + "self_attn.k_proj.bias",
            "mixer.v_proj.bias": p + "self_attn.v_proj.bias",
            "mixer.o_proj.bias": p + "self_attn.o_proj.bias",
            "feed_forward.gate_proj.weight": p + "mlp.gate_proj.weight",
            "feed_forward.up_proj.weight": p + "mlp.up_proj.weight",
            "feed_forward.down_proj.weight": p + "mlp.down_proj.weight",
        }
        layers.append(LayerSpec(
            mixer=AttentionSpec(hidden=cfg.hidden_size, n_heads=cfg.num_attention_heads,
                                n_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                                qkv_bias=cfg.qkv_bias, position=position, out_bias=False,
                                window=cfg.layer_window(i)),
            feed_forward=SwiGLUSpec(hidden=cfg.hidden_size, intermediate=cfg.intermediate_size),
            mixer_norm=NormSpec(size=cfg.hidden_size, eps=cfg.rms_norm_eps),
            feed_forward_norm=NormSpec(size=cfg.hidden_size, eps=cfg.rms_norm_eps),
            names=names))
    return ModelSpec(
        vocab=cfg.vocab_size, hidden=cfg.hidden_size, layers=layers,
        order=[Stage(layer=i) for i in range(cfg.num_hidden_layers)],
        final_norm=NormSpec(size=cfg.hidden_size, eps=cfg.rms_norm_eps),
        embed_name="model.embed_tokens.weight", final_norm_name="model.norm.weight",
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        max_positions=cfg.max_position_embeddings, eos_ids=cfg.eos_token_ids)


ARCHITECTURE = register_architecture(Architecture(
    name=Qwen2Config.architecture, model_type=Qwen2Config.model_type,
    config_class=Qwen2Config, build_spec=build_spec))
