"""Architecture description shared by the trainer model, the rollout decoder, the checkpoint converters and the
FLOPs counter.  ``MODEL_ARCH`` names follow gpatch_v4/core/constants.py:24-72; ``from_hf_config`` reads the fields
of a HuggingFace ``config.json`` so real checkpoints and the random-init benchmark shapes use one path."""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Tuple, Any, Dict, List, Optional


@dataclass
class ModelConfig:
    arch: str = "llama"
    num_layers: int = 2
    hidden_size: int = 256
    num_attention_heads: int = 4
    num_kv_heads: int = 2
    head_dim: Optional[int] = None
    ffn_hidden_size: int = 688
    vocab_size: int = 1024
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rotary_percent: float = 1.0
    rope_interleaved: bool = False
    max_position_embeddings: int = 131072
    qkv_bias: bool = False
    qk_layernorm: bool = False
    tie_word_embeddings: bool = False
    attention_dropout: float = 0.0
    # sliding window + sinks (gpt_oss / long-context recipes): window applies to layers where pattern[i % len] == 1
    sliding_window: int = 0
    sliding_window_pattern: List[int] = field(default_factory=list)
    attention_sinks: bool = False
    # MoE
    num_experts: int = 0
    moe_top_k: int = 0
    moe_ffn_hidden_size: int = 0
    moe_shared_expert_ffn: int = 0
    moe_shared_expert_gate: bool = False   # qwen2_moe: the shared expert's output is scaled by sigmoid(x . g)
    moe_router_type: str = "softmax"  # softmax | sigmoid_group
    moe_n_group: int = 1
    moe_topk_group: int = 1
    moe_norm_topk_prob: bool = True
    moe_routed_scaling_factor: float = 1.0
    moe_aux_loss_coef: float = 0.0
    moe_z_loss_coef: float = 0.0
    moe_router_bias: bool = False
    first_k_dense: int = 0
    moe_layer_freq: int = 1
    # MLA (DeepSeek-V3)
    use_mla: bool = False
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # vision tower stub for VLM families (patch embedding + merger feeding the decoder)
    vision: Dict[str, Any] = field(default_factory=dict)
    # multi-axis rotary position ids (vision-language decoders): frequencies per (temporal, height, width) axis,
    # summing to rotary_dim / 2; interleaved assignment (Qwen3-VL) or consecutive chunks (Qwen2-VL)
    mrope_sections: Optional[Tuple[int, int, int]] = None
    mrope_interleaved: bool = True
    dtype: str = "bfloat16"
    init_std: float = 0.02
    # multi-token prediction: extra depth-k blocks behind the trunk that predict token t + k + 1 from the hidden state
    # at t and the embedding of token t + k; trained with a scaled cross-entropy beside the main objective
    mtp_num_layers: int = 0
    mtp_loss_scaling_factor: float = 0.1
    fp8_base_weights: bool = False  # frozen e4m3 base with 128x128 block scales

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.num_kv_heads is None:
            self.num_kv_heads = self.num_attention_heads
        if self.num_attention_heads % self.num_kv_heads:
            raise ValueError("num_attention_heads must be a multiple of num_kv_heads")
        if self.num_experts and not self.moe_top_k:
            raise ValueError("MoE models need moe_top_k")
        if self.num_experts and not self.moe_ffn_hidden_size:
            self.moe_ffn_hidden_size = self.ffn_hidden_size

    # ---- derived
    @property
    def is_moe(self):
        return self.num_experts > 0

    def layer_is_moe(self, i: int) -> bool:
        return self.is_moe and i >= self.first_k_dense and (i % self.moe_layer_freq == 0)

    def layer_window(self, i: int) -> int:
        if not self.sliding_window:
            return 0
        if not self.sliding_window_pattern:
            return self.sliding_window
        return self.sliding_window if self.sliding_window_pattern[i % len(self.sliding_window_pattern)] else 0

    @property
    def rotary_dim(self):
        if self.use_mla:
            return self.qk_rope_head_dim
        return int(self.head_dim * self.rotary_percent)

    @property
    def qk_head_dim(self):
        return self.qk_nope_head_dim + self.qk_rope_head_dim if self.use_mla else self.head_dim

    def num_parameters(self, include_embedding=True) -> int:
        h, L = self.hidden_size, self.num_layers
        if self.use_mla:
            attn = (h * self.q_lora_rank + self.q_lora_rank * self.num_attention_heads * self.qk_head_dim
                    if self.q_lora_rank else h * self.num_attention_heads * self.qk_head_dim)
            attn += h * (self.kv_lora_rank + self.qk_rope_head_dim)
            attn += self.kv_lora_rank * self.num_attention_heads * (self.qk_nope_head_dim + self.v_head_dim)
            attn += self.num_attention_heads * self.v_head_dim * h
        else:
            attn = h * (self.num_attention_heads + 2 * self.num_kv_heads) * self.head_dim
            attn += self.num_attention_heads * self.head_dim * h
        total = 0
        for i in range(L):
            total += attn + 2 * h
            if self.layer_is_moe(i):
                total += self.num_experts * 3 * h * self.moe_ffn_hidden_size + h * self.num_experts
                total += 3 * h * self.moe_shared_expert_ffn
            else:
                total += 3 * h * self.ffn_hidden_size
        total += h
        if include_embedding:
            total += self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        return total

    def active_parameters(self) -> int:
        if not self.is_moe:
            return self.num_parameters()
        dense = ModelConfig(**{f.name: getattr(self, f.name) for f in fields(self)})
        total = self.num_parameters()
        for i in range(self.num_layers):
            if self.layer_is_moe(i):
                total -= (self.num_experts - self.moe_top_k) * 3 * self.hidden_size * self.moe_ffn_hidden_size
        del dense
        return total

    def to_dict(self):
        return {f.name: getattr(self, f.name) for f in fields(self)}


MODEL_ARCH = ("llama", "llama4", "qwen2", "qwen2_5_vl", "qwen3", "qwen3_moe", "qwen3_vl", "qwen3_vl_moe", "qwen2_moe",
              "qwen2_vl", "deepseek_v3", "mistral", "gemma3_text", "seed_oss", "gpt_oss")

PRESETS: Dict[str, Dict[str, Any]] = {
    # BASELINE config 1: tiny Llama-style decoder
    "tiny_llama": dict(arch="llama", num_layers=2, hidden_size=256, num_attention_heads=4, num_kv_heads=2,
                       ffn_hidden_size=688, vocab_size=1024, rms_norm_eps=1e-6, rope_theta=10000.0),
    "qwen2.5-7b": dict(arch="qwen2", num_layers=28, hidden_size=3584, num_attention_heads=28, num_kv_heads=4,
                       ffn_hidden_size=18944, vocab_size=152064, rms_norm_eps=1e-6, rope_theta=1e6, qkv_bias=True),
    "qwen2.5-1.5b": dict(arch="qwen2", num_layers=28, hidden_size=1536, num_attention_heads=12, num_kv_heads=2,
                         ffn_hidden_size=8960, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6, qkv_bias=True,
                         tie_word_embeddings=True),
    "qwen3-30b-a3b": dict(arch="qwen3_moe", num_layers=48, hidden_size=2048, num_attention_heads=32, num_kv_heads=4,
                          head_dim=128, ffn_hidden_size=6144, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6,
                          qk_layernorm=True, num_experts=128, moe_top_k=8, moe_ffn_hidden_size=768,
                          moe_router_type="softmax", moe_norm_topk_prob=True, moe_aux_loss_coef=1e-3),
    "llama3-8b-swa": dict(arch="llama", num_layers=32, hidden_size=4096, num_attention_heads=32, num_kv_heads=8,
                          ffn_hidden_size=14336, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=5e5,
                          sliding_window=4096, sliding_window_pattern=[0, 1], attention_sinks=True),
    "deepseek-v3-12l": dict(arch="deepseek_v3", num_layers=12, hidden_size=7168, num_attention_heads=128,
                            num_kv_heads=128, ffn_hidden_size=18432, vocab_size=129280, rms_norm_eps=1e-6,
                            rope_theta=10000.0, use_mla=True, q_lora_rank=1536, kv_lora_rank=512,
                            qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, head_dim=192,
                            num_experts=256, moe_top_k=8, moe_ffn_hidden_size=2048, moe_shared_expert_ffn=2048,
                            moe_router_type="sigmoid_group", moe_n_group=8, moe_topk_group=4, first_k_dense=1,
                            moe_routed_scaling_factor=2.5, moe_router_bias=True, rope_interleaved=True),
}


def get_preset(name: str, **overrides) -> ModelConfig:
    d = dict(PRESETS[name])
    d.update(overrides)
    return ModelConfig(**d)


def from_hf_config(hf: Dict[str, Any]) -> ModelConfig:
    """Maps a HuggingFace config dict (llama / qwen2 / qwen3 / qwen3_moe / deepseek_v3 / mistral / gpt_oss)."""
    mt = hf.get("model_type", "llama")
    kw: Dict[str, Any] = dict(
        arch={"qwen2": "qwen2", "qwen3": "qwen3", "qwen3_moe": "qwen3_moe", "deepseek_v3": "deepseek_v3",
              "mistral": "mistral", "gpt_oss": "gpt_oss", "seed_oss": "seed_oss"}.get(mt, "llama"),
        num_layers=hf["num_hidden_layers"], hidden_size=hf["hidden_size"],
        num_attention_heads=hf["num_attention_heads"],
        num_kv_heads=hf.get("num_key_value_heads", hf["num_attention_heads"]),
        head_dim=hf.get("head_dim"), ffn_hidden_size=hf.get("intermediate_size", 0), vocab_size=hf["vocab_size"],
        rms_norm_eps=hf.get("rms_norm_eps", 1e-6), rope_theta=hf.get("rope_theta", 10000.0),
        tie_word_embeddings=hf.get("tie_word_embeddings", False),
        max_position_embeddings=hf.get("max_position_embeddings", 131072),
    )
    if mt == "qwen2" or hf.get("attention_bias"):   # seed_oss and other llama-style configs with biased projections
        kw["qkv_bias"] = True
    if mt in ("qwen3", "qwen3_moe"):
        kw["qk_layernorm"] = True
    if hf.get("sliding_window") and hf.get("use_sliding_window", mt in ("mistral", "gpt_oss")):
        kw["sliding_window"] = hf["sliding_window"]
    if mt == "gpt_oss":
        kw["attention_sinks"] = True
        kw["sliding_window_pattern"] = [1, 0]
    if mt == "qwen3_moe":
        kw.update(num_experts=hf["num_experts"], moe_top_k=hf["num_experts_per_tok"],
                  moe_ffn_hidden_size=hf["moe_intermediate_size"], moe_norm_topk_prob=hf.get("norm_topk_prob", True),
                  moe_aux_loss_coef=hf.get("router_aux_loss_coef", 0.0))
    if mt == "qwen2_moe":
        kw.update(arch="qwen2_moe", qkv_bias=True, num_experts=hf["num_experts"], moe_top_k=hf["num_experts_per_tok"],
                  moe_ffn_hidden_size=hf["moe_intermediate_size"],
                  moe_shared_expert_ffn=hf.get("shared_expert_intermediate_size", 0),
                  moe_shared_expert_gate=bool(hf.get("shared_expert_intermediate_size", 0)),
                  moe_norm_topk_prob=hf.get("norm_topk_prob", False),
                  moe_aux_loss_coef=hf.get("router_aux_loss_coef", 0.0))
    if mt == "deepseek_v3":
        kw.update(use_mla=True, q_lora_rank=hf.get("q_lora_rank") or 0, kv_lora_rank=hf["kv_lora_rank"],
                  qk_nope_head_dim=hf["qk_nope_head_dim"], qk_rope_head_dim=hf["qk_rope_head_dim"],
                  v_head_dim=hf["v_head_dim"], head_dim=hf["qk_nope_head_dim"] + hf["qk_rope_head_dim"],
                  num_experts=hf["n_routed_experts"], moe_top_k=hf["num_experts_per_tok"],
                  moe_ffn_hidden_size=hf["moe_intermediate_size"],
                  moe_shared_expert_ffn=hf["moe_intermediate_size"] * hf.get("n_shared_experts", 0),
                  moe_router_type="sigmoid_group", moe_n_group=hf.get("n_group", 1),
                  moe_topk_group=hf.get("topk_group", 1), first_k_dense=hf.get("first_k_dense_replace", 0),
                  moe_routed_scaling_factor=hf.get("routed_scaling_factor", 1.0), moe_router_bias=True,
                  rope_interleaved=True)
    return ModelConfig(**{k: v for k, v in kw.items() if v is not None or k == "head_dim"})


def build_model_config(arch_or_preset: str, overrides: Optional[Dict[str, Any]] = None) -> ModelConfig:
    overrides = dict(overrides or {})
    if arch_or_preset in PRESETS:
        return get_preset(arch_or_preset, **overrides)
    if "hf_config" in overrides:
        return from_hf_config(overrides.pop("hf_config"))
    overrides.setdefault("arch", arch_or_preset)
    return ModelConfig(**overrides)
