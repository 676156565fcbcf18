"""The dense Qwen3 decoder's configuration, read from its own config.json keys.

Keys, defaults and refusals follow what the reference's config inspector reads for ``model_type: "qwen3"``
(evidence/pipeline/onboarding/Starlings.Roost.Onboarding/ConfigInspector.cs:217-257 for the sizes, :266-318
for the layer kinds, :519-553 for the rotation, :679-731 for the activation and quantisation) and what its
Qwen3-shaped model definition binds (src/Starlings.Roost.Models.Tiny/RoostTiny.cs:14-57).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

from .reader import ConfigError, ConfigReader
from .spec import (AttentionSpec, BlockSpec, GatedMlpSpec, ModelSpec, NormSpec, PositionSpec, RunEntry)

ARCHITECTURE = "Qwen3ForCausalLM"
MODEL_TYPE = "qwen3"
_DTYPES = ("bfloat16", "float16", "float32")


@dataclass
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int | None
    tie_word_embeddings: bool | None          # None: decided by whether the checkpoint has lm_head.weight
    torch_dtype: str
    layer_windows: tuple                       # per layer: None (every key) or the window in keys
    sliding_window: int | None = None
    eos_token_ids: tuple = ()
    warnings: list = field(default_factory=list)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_reader(cls, c: ConfigReader) -> "Qwen3Config":
        warnings: list[str] = []
        model_type = c.opt_str("model_type")
        if model_type is not None and model_type != MODEL_TYPE:
            raise ConfigError(f"{c.source}: key 'model_type' is '{model_type}'; this reader serves '{MODEL_TYPE}'")
        hidden = c.positive_int("hidden_size")
        layers = c.positive_int("num_hidden_layers")
        heads = c.positive_int("num_attention_heads")
        kv_heads = c.positive_int("num_key_value_heads", default=heads)
        head_dim = c.opt_int("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"{c.source}: key 'head_dim' is absent and hidden_size {hidden} is not a multiple of num_attention_heads {heads}")
            head_dim = hidden // heads
        if head_dim <= 0:
            raise ConfigError(f"{c.source}: key 'head_dim' is {head_dim}; it must be positive")
        if heads % kv_heads:
            raise ConfigError(f"{c.source}: num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        vocab = c.positive_int("vocab_size")
        inter = c.positive_int("intermediate_size")

        act = c.opt_str("hidden_act")
        if act not in (None, "silu", "swish"):
            raise ConfigError(f"{c.source}: key 'hidden_act' is '{act}'; the dense Qwen3 feed-forward is gated with silu")
        if c.opt_bool("attention_bias"):
            raise ConfigError(f"{c.source}: key 'attention_bias' is true; Qwen3's projections have no bias and none is loaded")
        if (c.opt_int("num_experts") or 0) > 0 or (c.opt_int("num_local_experts") or 0) > 0:
            raise ConfigError(f"{c.source}: key 'num_experts' is set; that is the mixture-of-experts model, another architecture")
        if c.has("quantization_config"):
            raise ConfigError(f"{c.source}: key 'quantization_config' is set; quantised weights are not served")

        eps = c.opt_float("rms_norm_eps")
        if eps is None:
            eps = 1e-6
            warnings.append("rms_norm_eps is absent: 1e-6 is used, the value the reference's Qwen3 definition binds")
        if eps <= 0:
            raise ConfigError(f"{c.source}: key 'rms_norm_eps' is {eps}; it must be positive")

        theta = c.opt_float("rope_theta")
        for key in ("rope_scaling", "rope_parameters"):
            sub = c.opt_object(key)
            if sub is None:
                continue
            kind = sub.opt_str("rope_type") or sub.opt_str("type")
            if kind not in (None, "default"):
                raise ConfigError(f"{c.source}: {key} has rope_type '{kind}'; only the unscaled rotation is built")
            t = sub.opt_float("rope_theta")
            if t is not None:
                theta = t
        if theta is None:
            theta = 10000.0
            warnings.append("rope_theta is absent: 10000 is assumed")
        if theta <= 0:
            raise ConfigError(f"{c.source}: key 'rope_theta' is {theta}; it must be positive")
        prf = c.opt_float("partial_rotary_factor")
        if prf is not None and prf != 1.0:
            raise ConfigError(f"{c.source}: key 'partial_rotary_factor' is {prf}; Qwen3 rotates the whole head")
        if head_dim % 2:
            raise ConfigError(f"{c.source}: head_dim {head_dim} is odd; the rotation pairs element i with i + head_dim/2")

        max_pos = c.opt_int("max_position_embeddings")
        if max_pos is not None and max_pos <= 0:
            raise ConfigError(f"{c.source}: key 'max_position_embeddings' is {max_pos}; it must be positive")

        dtype = c.opt_str("dtype") or c.opt_str("torch_dtype")
        if dtype is None:
            dtype = "bfloat16"
            warnings.append("dtype and torch_dtype are absent: weights are assumed bfloat16")
        if dtype not in _DTYPES:
            raise ConfigError(f"{c.source}: key 'torch_dtype' is '{dtype}'; expected one of {', '.join(_DTYPES)}")

        # layer kinds
        window = c.opt_int("sliding_window")
        types = c.opt_strs("layer_types")
        use_sliding = c.opt_bool("use_sliding_window")
        max_window_layers = c.opt_int("max_window_layers")
        windows: list[int | None] = [None] * layers
        if types is not None:
            if len(types) != layers:
                raise ConfigError(f"{c.source}: key 'layer_types' has {len(types)} entries for {layers} layers")
            for i, t in enumerate(types):
                if t == "full_attention":
                    continue
                if t == "sliding_attention":
                    if window is None:
                        raise ConfigError(f"{c.source}: layer_types[{i}] is 'sliding_attention' but key 'sliding_window' is absent")
                    windows[i] = window
                else:
                    raise ConfigError(f"{c.source}: layer_types[{i}] is '{t}'; the dense Qwen3 decoder has full_attention and sliding_attention layers only")
        elif window is not None and use_sliding:
            first = layers if max_window_layers is None else max_window_layers
            for i in range(layers):
                if i >= first:
                    windows[i] = window
        if window is not None and window <= 0 and any(w is not None for w in windows):
            raise ConfigError(f"{c.source}: key 'sliding_window' is {window}; it must be positive")

        eos = tuple(c.opt_ints("eos_token_id") or ())
        return cls(vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                   num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter, rms_norm_eps=eps,
                   rope_theta=theta, max_position_embeddings=max_pos, tie_word_embeddings=c.opt_bool("tie_word_embeddings"),
                   torch_dtype=dtype, layer_windows=tuple(windows), sliding_window=window, eos_token_ids=eos,
                   warnings=warnings)

    @classmethod
    def from_dict(cls, values: dict, source: str = "config") -> "Qwen3Config":
        return cls.from_reader(ConfigReader(values, source))

    # ------------------------------------------------------------------ writing (random-weights mode)
    def to_dict(self) -> dict:
        d = {
            "architectures": [ARCHITECTURE],
            "model_type": MODEL_TYPE,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "attention_bias": False,
            "tie_word_embeddings": bool(self.tie_word_embeddings),
            "torch_dtype": self.torch_dtype,
        }
        if self.max_position_embeddings is not None:
            d["max_position_embeddings"] = self.max_position_embeddings
        if any(w is not None for w in self.layer_windows):
            d["sliding_window"] = self.sliding_window
            d["layer_types"] = ["full_attention" if w is None else "sliding_attention" for w in self.layer_windows]
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d

    # ------------------------------------------------------------------ the reference's weight slots
    def reference_slots(self, tied: bool | None = None) -> list:
        """(slot name, slot shape, checkpoint tensors that hold the slot's rows in order) for every weight, with the
        slot names and shapes of the reference's own Qwen3-shaped model definition
        (src/Starlings.Roost.Models.Tiny/RoostTiny.cs:26-38): ``embed``, per layer ``l{i}.input_norm``, ``q_proj``,
        ``k_proj``, ``v_proj``, ``q_norm``, ``k_norm``, ``o_proj``, ``post_norm``, ``gate_up`` (one slot of 2 x
        intermediate rows: gate_proj then up_proj), ``down``, then ``final_norm`` and ``lm_head``. The reference's seeded
        generator draws a slot's values from the slot's name, so the names are part of the weights."""
        tie = self.tie_word_embeddings if tied is None else tied
        H, d, I = self.hidden_size, self.head_dim, self.intermediate_size
        Q, KV = self.num_attention_heads * d, self.num_key_value_heads * d
        slots = [("embed", (self.vocab_size, H), ("model.embed_tokens.weight",))]
        for i in range(self.num_hidden_layers):
            p, a = f"model.layers.{i}.", f"model.layers.{i}.self_attn."
            slots += [
                (f"l{i}.input_norm", (H,), (p + "input_layernorm.weight",)),
                (f"l{i}.q_proj", (Q, H), (a + "q_proj.weight",)),
                (f"l{i}.k_proj", (KV, H), (a + "k_proj.weight",)),
                (f"l{i}.v_proj", (KV, H), (a + "v_proj.weight",)),
                (f"l{i}.q_norm", (d,), (a + "q_norm.weight",)),
                (f"l{i}.k_norm", (d,), (a + "k_norm.weight",)),
                (f"l{i}.o_proj", (H, Q), (a + "o_proj.weight",)),
                (f"l{i}.post_norm", (H,), (p + "post_attention_layernorm.weight",)),
                (f"l{i}.gate_up", (2 * I, H), (p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight")),
                (f"l{i}.down", (H, I), (p + "mlp.down_proj.weight",)),
            ]
        slots.append(("final_norm", (H,), ("model.norm.weight",)))
        if not tie:
            slots.append(("lm_head", (self.vocab_size, H), ("lm_head.weight",)))
        return slots

    # ------------------------------------------------------------------ the model as parts
    def to_spec(self, tied: bool | None = None) -> ModelSpec:
        """Blocks, run order and checkpoint names. ``tied`` overrides ``tie_word_embeddings`` when the
        config leaves it open (the loader looks for lm_head.weight)."""
        tie = self.tie_word_embeddings if tied is None else tied
        if tie is None:
            tie = True  # the reference's inspector default when the key is absent (ConfigInspector.cs:255)
        H, d = self.hidden_size, self.head_dim
        norm = NormSpec(size=H, eps=self.rms_norm_eps)
        head_norm = NormSpec(size=d, eps=self.rms_norm_eps)
        rope = PositionSpec(kind="rope_neox", rotary_dim=d, theta=self.rope_theta,
                            max_positions=self.max_position_embeddings or 0)
        ff = GatedMlpSpec(hidden=H, intermediate=self.intermediate_size, activation="silu")
        blocks = []
        names: dict = {
            "embed": {"table": ("model.embed_tokens.weight",)},
            "final_norm": {"weight": ("model.norm.weight",)},
        }
        if not tie:
            names["lm_head"] = {"weight": ("lm_head.weight",)}
        for i, w in enumerate(self.layer_windows):
            mixer = AttentionSpec(hidden=H, num_heads=self.num_attention_heads, num_kv_heads=self.num_key_value_heads,
                                  head_dim=d, scale=1.0 / math.sqrt(d), window=w, qk_norm=head_norm, position=rope)
            blocks.append(BlockSpec(mixer=mixer, feed_forward=ff, input_norm=norm, post_mixer_norm=norm))
            p = f"model.layers.{i}."
            a = p + "self_attn."
            names[f"blocks.{i}.input_norm"] = {"weight": (p + "input_layernorm.weight",)}
            names[f"blocks.{i}.post_mixer_norm"] = {"weight": (p + "post_attention_layernorm.weight",)}
            names[f"blocks.{i}.mixer"] = {
                "qkv": (a + "q_proj.weight", a + "k_proj.weight", a + "v_proj.weight"),
                "out": (a + "o_proj.weight",),
                "q_norm": (a + "q_norm.weight",),
                "k_norm": (a + "k_norm.weight",),
            }
            names[f"blocks.{i}.feed_forward"] = {
                "gate_up": (p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"),
                "down": (p + "mlp.down_proj.weight",),
            }
        return ModelSpec(architecture=ARCHITECTURE, hidden=H, vocab=self.vocab_size, blocks=tuple(blocks),
                         schedule=tuple(RunEntry(block=i) for i in range(len(blocks))), final_norm=norm,
                         tie_embeddings=tie, max_positions=self.max_position_embeddings or 0,
                         stop_token_ids=tuple(self.eos_token_ids), stored_dtype=self.torch_dtype, weight_names=names)
