"""Config dataclasses.  Section and field names follow the reference's YAML surface
(gpatch_v4/configs/config.py:113-772, training_config.py, ppo_config.py, policy_config.py, dist_config.py,
infer_engine_config.py, checkpoint_config.py, optimizer_config.py, lora_config.py) so its recipes carry over;
cross-field validation lives in ``__post_init__``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, MappingMixin


# ------------------------------------------------------------------------------------------------ leaves
@dataclass
class DistConfig(MappingMixin):
    num_gpus_per_node: int = 8
    nnodes: int = -1
    num_cpu_nodes: int = 0
    torch_dist_timeout_minutes: int = 30
    use_tp_pp_dp_mapping: bool = False
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: int = 1
    context_parallel_size: int = 1
    dynamic_context_parallel: bool = False
    max_seqlen_per_dp_cp_rank: Optional[int] = None
    max_seqlen_per_dp_cp_rank_fwd_only: Optional[int] = None
    min_dynamic_context_parallel_size: int = 1
    dynamic_cp_scheduler_type: str = "default"
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    num_layers_in_first_pipeline_stage: Optional[int] = None
    num_layers_in_last_pipeline_stage: Optional[int] = None
    virtual_pipeline_model_parallel_size: Optional[int] = None
    sequence_parallel: bool = True
    custom_device_mesh: Optional[Dict[str, Any]] = None
    fsdp2_forward_prefetch: int = 1
    fsdp2_backward_prefetch: int = 1

    def __post_init__(self):
        for n in ("tensor_model_parallel_size", "pipeline_model_parallel_size", "context_parallel_size",
                  "expert_model_parallel_size", "expert_tensor_parallel_size"):
            if getattr(self, n) < 1:
                raise ConfigError(f"dist_config.{n} must be >= 1")
        if self.tensor_model_parallel_size == 1:
            self.sequence_parallel = False
        if self.dynamic_context_parallel and self.max_seqlen_per_dp_cp_rank is None:
            raise ConfigError("dynamic_context_parallel needs max_seqlen_per_dp_cp_rank")

    @property
    def model_parallel_size(self):
        return (self.tensor_model_parallel_size * self.pipeline_model_parallel_size * self.context_parallel_size)


@dataclass
class LoRAConfig(MappingMixin):
    rank: int = 0
    alpha: float = 32
    type: str = "canonical_lora"
    dropout: float = 0.0
    target_modules: List[str] = field(default_factory=lambda: ["linear_qkv", "linear_proj", "linear_fc1",
                                                               "linear_fc2"])
    exclude_modules: List[str] = field(default_factory=list)
    lora_A_init_method: str = "xavier"
    lora_B_init_method: str = "zero"
    dtype: Optional[str] = None
    check_lora_all_coverage: bool = False
    verify_weight_consistency: bool = True
    share_expert_adapters: bool = True

    def __post_init__(self):
        if self.type not in ("lora", "canonical_lora"):
            raise ConfigError(f"lora.type must be lora|canonical_lora, got {self.type}")

    @property
    def enabled(self):
        return self.rank > 0


@dataclass
class ClientConfig(MappingMixin):
    rpc_type: str = "local"
    rpc_timeout: int = 60
    update_weight_max_size_mb: int = 512
    update_weight_use_bucketed_ipc: bool = True
    split_generate_repeat_n: bool = False


@dataclass
class OptimizerConfig(MappingMixin):
    lr: float = 1e-5
    min_lr: float = 0.0
    lr_warmup_steps: int = 0
    lr_warmup_step_frac: Optional[float] = None
    lr_warmup_init: float = 0.0
    lr_decay_steps: Optional[int] = None
    lr_decay_style: str = "linear"
    lr_wsd_decay_steps: Optional[int] = None
    lr_wsd_decay_style: str = "exponential"
    weight_decay: float = 0.01
    optimizer_type: str = "adam"
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-8
    max_grad_norm: float = 1.0
    use_distributed_optimizer: bool = True
    grad_reduce_in_fp32: bool = True
    overlap_grad_reduce: bool = False
    overlap_param_gather: bool = False
    bucket_size: Optional[int] = None
    override_optimizer_config: Dict[str, Any] = field(default_factory=dict)
    muon_momentum: float = 0.95
    muon_ns_steps: int = 5
    muon_scale_mode: str = "spectral"
    per_module_lr: Dict[str, float] = field(default_factory=dict)

    def __post_init__(self):
        if self.lr_decay_style not in ("constant", "linear", "cosine", "inverse-square-root", "WSD"):
            raise ConfigError(f"unknown lr_decay_style {self.lr_decay_style}")
        if self.optimizer_type not in ("adam", "sgd", "muon"):
            raise ConfigError(f"unknown optimizer_type {self.optimizer_type}")


@dataclass
class CheckpointConfig(MappingMixin):
    load_ckpt_path: Optional[str] = None
    save_ckpt_path: Optional[str] = None
    no_load_optim: bool = False
    no_save_optim: bool = False
    no_load_rng: bool = False
    ref_load_ckpt_path: Optional[str] = None
    save_total_limit: Optional[int] = None
    save_retain_interval: Optional[int] = None
    use_dist_checkpointing: bool = True
    async_save: bool = False
    convert_mcore_to_hf_online: bool = False
    convert_mcore_to_hf_offline: bool = False
    export_hf_save_path: Optional[str] = None
    strict_export: bool = True
    skip_save_mcore_model: bool = False
    save_merged_lora_weights: bool = True


@dataclass
class ProfileConfig(MappingMixin):
    enable: bool = False
    profile_start_step: int = 2
    profile_end_step: int = 3
    export_dir: Optional[str] = None
    export_ranks: List[int] = field(default_factory=lambda: [0])
    gzip: bool = False
    with_stack: bool = False
    record_shapes: bool = False
    profile_memory: bool = False
    use_nsys: bool = False
    comm_summary: bool = True

    def __post_init__(self):
        if self.enable and self.profile_end_step < self.profile_start_step:
            raise ConfigError("profile_end_step must be >= profile_start_step")


@dataclass
class ReportConfig(MappingMixin):
    report_to: List[str] = field(default_factory=list)  # "wandb", "tensorboard", "jsonl"
    project: str = "gcore_b200"
    run_name: Optional[str] = None
    log_dir: str = "./logs"
    log_interval: int = 1
    use_verl_metric_names: bool = False
    debug_log_shards: bool = False      # one DEBUG log file per process under <task dir>/debug
    redirect_engine_log: bool = False   # stdout / stderr of the rollout phase go to <task dir>/infer_engine_log
    profile: ProfileConfig = field(default_factory=ProfileConfig)


@dataclass
class DebugConfig(MappingMixin):
    debug_update_weight: bool = False
    replay_rollout_path: Optional[str] = None
    dump_rollout_path: Optional[str] = None
    check_rollout_batches: bool = True
    check_a2a_legality: bool = False
    trace_python_calls: bool = False
    trace_roots: List[str] = field(default_factory=list)
    ppo_padding_check: bool = False
    fault_injection: Dict[str, Any] = field(default_factory=dict)  # host-side only: {"raise_at_step": n, ...}


@dataclass
class DataConfig(MappingMixin):
    py_path: Optional[str] = None
    fn_name: Optional[str] = None
    train_data_path: Optional[str] = None
    eval_data_path: Optional[str] = None
    prompt_key: str = "prompt"
    label_key: str = "answer"
    max_prompt_length: int = 1024
    num_workers: int = 0
    shuffle: bool = True
    seed: int = 42
    synthetic: Dict[str, Any] = field(default_factory=dict)
    extra: Dict[str, Any] = field(default_factory=dict)
    _allow_extra = True


@dataclass
class RewardModelInfo(MappingMixin):
    name: str = "rule"
    py_path: Optional[str] = None
    fn_name: Optional[str] = None
    reward_weight: float = 1.0
    hf_model_path: Optional[str] = None
    gen_reward_repeat_n: int = 1


@dataclass
class RewardConfig(MappingMixin):
    reward_type: str = "rule_only"  # rule_only | rm_only | mix
    reward_model_info: List[RewardModelInfo] = field(default_factory=list)
    rule_py_path: Optional[str] = None
    rule_fn_name: Optional[str] = None
    external_url: Optional[str] = None
    external_timeout: int = 600
    stream: bool = False

    def __post_init__(self):
        if self.reward_type not in ("rule_only", "rm_only", "mix"):
            raise ConfigError(f"reward_type must be rule_only|rm_only|mix, got {self.reward_type}")


@dataclass
class InferEngineConfig(MappingMixin):
    dist_config: DistConfig = field(default_factory=DistConfig)
    dp_size: int = 1
    dtype: str = "bfloat16"
    gpu_memory_utilization: float = 0.7
    max_running_requests: Optional[int] = None
    max_model_len: Optional[int] = None
    kv_block_size: int = 16
    num_kv_blocks: Optional[int] = None
    max_prefill_tokens: int = 16384
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    min_p: float = 0.0
    generate_max_tokens: int = 128
    generate_params: Dict[str, Any] = field(default_factory=dict)
    eval_generate_params: Dict[str, Any] = field(default_factory=dict)
    seed: int = 42
    engine_seed: int = 42
    repetition_penalty: float = 1.0
    load_format: str = "auto"
    enable_weights_cpu_backup: bool = False
    disable_cuda_graph: bool = False
    attention_backend: str = "native"
    return_routed_experts: bool = False
    fp8_weights: bool = False
    watchdog_timeout: int = 600
    model_override_args: Dict[str, Any] = field(default_factory=dict)
    override_infer_engine_config: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if self.dist_config.pipeline_model_parallel_size != 1:
            raise ConfigError("rollout engines run with pipeline_model_parallel_size == 1")
        if not 0 < self.gpu_memory_utilization <= 1:
            raise ConfigError("gpu_memory_utilization must be in (0, 1]")


@dataclass
class ModelInfo(MappingMixin):
    name: str = "policy"
    hf_model_path: Optional[str] = None
    model_arch: Optional[str] = None
    gen_rollout_py_path: Optional[str] = None
    gen_rollout_fn_name: Optional[str] = None


@dataclass
class SamplerConfig(MappingMixin):
    backend: str = "native"
    model_info: List[ModelInfo] = field(default_factory=lambda: [ModelInfo()])
    infer_engine_configs: List[InferEngineConfig] = field(default_factory=lambda: [InferEngineConfig()])

    def __post_init__(self):
        if self.backend not in ("native", "eager", "sglang", "vllm"):
            raise ConfigError(f"unknown sampler backend {self.backend}")
        if self.backend in ("sglang", "vllm"):
            # the external engines of the reference are replaced by the built-in decoder
            self.backend = "native"


@dataclass
class PolicyConfig(MappingMixin):
    dist_config: DistConfig = field(default_factory=DistConfig)
    model_arch: str = "qwen2"
    model_config: Dict[str, Any] = field(default_factory=dict)  # explicit architecture (random init) or overrides
    hf_model_path: Optional[str] = None
    hf_tokenizer_path: Optional[str] = None
    ref_hf_model_path: Optional[str] = None
    attn_implementation: str = "native"
    ep_backend: str = "fused"
    fp8: bool = False
    fp8_qat: bool = False
    fp4_qat: bool = False
    rollout_gen_type: str = "base"
    rollout_gen_py_path: Optional[str] = None
    rollout_gen_cls: Optional[str] = None
    forward_only_mbs: int = 1
    dynamic_mbs_target_seqlen: Optional[int] = None
    dynamic_mbs_limit: Optional[int] = None
    dynamic_mbs_target_seqlen_fwd_only: Optional[int] = None  # token budget of forward-only micro-batches
    ppo_pack_seq: bool = True
    without_ref: bool = False
    without_optim: bool = False
    balance_dp_seqlen: bool = False
    smart_pad_infer: bool = False
    smart_pad_train: bool = False
    wrap_with_ddp: bool = True
    recompute: str = "full"  # none | full (per-layer activation recompute)
    recompute_num_layers: Optional[int] = None  # with "full": only the first N layers are recomputed (None = all)
    override_ddp_config: Dict[str, Any] = field(default_factory=dict)
    override_transformer_config: Dict[str, Any] = field(default_factory=dict)
    freeze_patterns: List[str] = field(default_factory=list)
    unfreeze_patterns: List[str] = field(default_factory=list)
    lora: LoRAConfig = field(default_factory=LoRAConfig)
    offload_process_group: bool = False
    manual_clear_memory: bool = False
    export_weights_buffer_max_size_mb: int = 2048
    share_rollout_weights: bool = True  # colocated trainer and decoder read the same bf16 parameter storage
    offload_ref_model: bool = False  # frozen reference policy in pinned host memory except during its forward pass
    release_rollout_weights: bool = False  # separate copy only: free it after each rollout, rebuild it at each resync
    ce_token_compaction: bool = True    # vocabulary projection / log-probs only at positions inside the loss mask
    # vision-language policy: fields of ``models.vlm.VisionConfig`` (empty = text-only) and the placeholder token id
    vision_config: Dict[str, Any] = field(default_factory=dict)
    image_token_id: Optional[int] = None
    # Qwen3-VL family (model_config.mrope_sections set): video_token_id, deepstack_layers, temporal_patch
    vision_options: Dict[str, Any] = field(default_factory=dict)
    sampler_client: ClientConfig = field(default_factory=ClientConfig)
    bt_rm_client: ClientConfig = field(default_factory=ClientConfig)
    gen_rm_client: ClientConfig = field(default_factory=ClientConfig)


@dataclass
class PpoConfig(MappingMixin):
    advantage_type: str = "grpo"
    loss_func: str = "grpo"
    use_legacy_loss: bool = False
    loss_func_py_path: Optional[str] = None
    loss_func_fn_name: Optional[str] = None
    advantage_py_path: Optional[str] = None
    advantage_fn_name: Optional[str] = None
    post_advantage_py_path: Optional[str] = None
    post_advantage_fn_name: Optional[str] = None
    ppo_initial_policy_kl_penalty: float = 0.0
    ppo_discount_factor: float = 1.0
    ppo_gae_lambda: float = 0.95
    ppo_entropy_bonus: float = 0.0
    use_adaptive_entropy: bool = False
    entropy_target: float = 0.2
    entropy_coef_delta: float = 0.005
    entropy_coef_min: float = 0.0
    entropy_coef_max: float = 1.0
    feature_store_enable: bool = False
    ppo_ratio_eps: float = 0.2
    ppo_clip_ratio_low: Optional[float] = None
    ppo_clip_ratio_high: Optional[float] = None
    ppo_dual_clip_ratio_c: Optional[float] = None
    grpo_advantage_epsilon: float = 1e-8
    ppo_logps_ratio_clamp: Optional[float] = None
    ppo_clamp_kl_val: Optional[float] = None
    ppo_value_clip: Optional[float] = None
    advantage_clip: bool = False
    advantage_clip_low: float = -10.0
    advantage_clip_high: float = 10.0
    whiten_advantages: bool = False
    grpo_kl_loss_beta: float = 1e-3
    kl_estimator: str = "k3"
    norm_adv_by_std_in_grpo: bool = True
    per_token_loss: bool = True
    # train-vs-rollout mismatch correction (truncate | clip | mask | icepop | kpop | none)
    offpolicy_correction: str = "none"
    offpolicy_correction_level: str = "token"  # token | sequence | geometric
    offpolicy_correction_upper: float = 2.0
    offpolicy_correction_lower: Optional[float] = None
    offpolicy_correction_veto: Optional[float] = None
    critic_model_warmup_steps: int = 0
    mask_negative_samples: bool = False
    gdpo_reward_weights: Dict[str, float] = field(default_factory=dict)
    skip_prev_logps: bool = False
    use_original_logprob: bool = False
    feature_store_enable: bool = False
    sapo_tau_pos: float = 1.0
    sapo_tau_neg: float = 1.05
    # entropy regularisation on the clipped surrogate: clip-cov | kl-cov | None (loss_func clip_cov / kl_cov select
    # the same losses directly)
    entropy_regularization_type: Optional[str] = None
    clip_cov_ratio: float = 2e-4
    clip_cov_ub: float = 5.0
    clip_cov_lb: float = 1.0
    kl_cov_ratio: float = 2e-4
    kl_cov_coef: float = 0.1
    # steer: token weights in [steer_token_weight_min, 1] from the estimated entropy change, on top of a base loss
    steer_token_weight_min: float = 0.8
    steer_policy_method: str = "grpo"
    # fipo: advantages weighted by exp(discounted future log-ratio), gamma = 2^(-1/decay_rate)
    fipo_decay_rate: float = 32.0
    fipo_chunk_size: int = 512
    fipo_clip_ratio: float = 0.2
    fipo_clip_high_only: bool = False
    fipo_safety_thresh: float = 3.0
    # vespo: phi(W) = W^c1 * exp(c2 * (1 - W)), separate shapes for sequences with positive / negative advantage
    vespo_c1_pos: float = 1.0
    vespo_c2_pos: float = 1.0
    vespo_c1_neg: float = 1.0
    vespo_c2_neg: float = 1.0

    # the spellings of gpatch_v4/configs/ppo_config.py for the fields this package names differently
    _aliases = {
        "ppo_entropy_regularization_type": "entropy_regularization_type",
        "ppo_clip_cov_ratio": "clip_cov_ratio", "ppo_clip_cov_ub": "clip_cov_ub", "ppo_clip_cov_lb": "clip_cov_lb",
        "ppo_kl_cov_ratio": "kl_cov_ratio", "ppo_kl_cov_coef": "kl_cov_coef",
        "off_policy_correction_mode": "offpolicy_correction", "off_policy_correction_level": "offpolicy_correction_level",
        "off_policy_correction_upper_bound": "offpolicy_correction_upper",
        "off_policy_correction_lower_bound": "offpolicy_correction_lower",
        "off_policy_correction_veto_threshold": "offpolicy_correction_veto",
        "custom_advantage_py_path": "advantage_py_path", "custom_advantage_py_name": "advantage_fn_name",
        "custom_post_advantage_py_name": "post_advantage_fn_name", "loss_func_py_name": "loss_func_fn_name",
        "advantage_clip_lower_bound": "advantage_clip_low", "advantage_clip_upper_bound": "advantage_clip_high",
    }

    def __post_init__(self):
        if self.loss_func == "steer":
            if self.skip_prev_logps:
                raise ConfigError("loss_func=steer needs the previous log-probs (skip_prev_logps=false)")
            if not 0.0 < self.steer_token_weight_min <= 1.0:
                raise ConfigError("steer_token_weight_min must be in (0, 1]")
            if self.steer_policy_method not in ("grpo", "cispo", "gspo", "sapo"):
                raise ConfigError(f"steer_policy_method must be grpo|cispo|gspo|sapo, got {self.steer_policy_method}")
        if self.entropy_regularization_type not in (None, "clip-cov", "kl-cov"):
            raise ConfigError(f"entropy_regularization_type must be clip-cov|kl-cov, got "
                              f"{self.entropy_regularization_type}")
        if self.entropy_regularization_type and self.loss_func != "grpo":
            raise ConfigError("entropy_regularization_type applies to loss_func=grpo")
        if self.advantage_type not in ("grpo", "gdpo", "gdpo_sample_bn", "group_gdpo", "group_gdpo_sample_bn", "ppo",
                                       "reinforce", "on_policy_distill", "g_opd", "identity", "custom"):
            raise ConfigError(f"unknown advantage_type {self.advantage_type}")
        if self.loss_func == "gspo" and self.per_token_loss:
            # sequence-level ratios are aggregated per sequence (gpatch_v4/configs/config.py:273-276)
            raise ConfigError("loss_func=gspo requires per_token_loss=false")
        if self.offpolicy_correction not in ("none", "truncate", "clip", "mask", "icepop", "kpop"):
            raise ConfigError(f"unknown offpolicy_correction {self.offpolicy_correction}")

    @property
    def clip_low(self):
        return self.ppo_clip_ratio_low if self.ppo_clip_ratio_low is not None else self.ppo_ratio_eps

    @property
    def clip_high(self):
        return self.ppo_clip_ratio_high if self.ppo_clip_ratio_high is not None else self.ppo_ratio_eps


@dataclass
class DynamicSamplingConfig(MappingMixin):
    enable: bool = False
    oversampling_ratio: float = 1.2
    ema_decay: float = 0.9
    max_refill_times: int = 3
    filter_py_path: Optional[str] = None
    filter_fn_name: Optional[str] = None
    epoch_mode: bool = False


@dataclass
class TrainingConfig(MappingMixin):
    training_backend: str = "native"  # native (fused sm_100a kernels) | nccl_eager (library baseline) | fsdp2 (ZeRO-3)
    train_gbs: int = 8
    train_mbs: int = 1
    gradient_accumulation_steps: Optional[int] = None
    exit_step: Optional[int] = None
    seed: int = 42
    seq_length: int = 2048
    total_training_step: Optional[int] = None
    num_train_epoches: int = 1
    apply_deterministic_mode: bool = False
    save_interval: int = 100
    eval_interval: Optional[int] = None
    pad_to_mulitiple_of: int = 128
    auto_load_from_save_ckpt: bool = True
    allow_tf32: bool = True
    max_train_step_waiting_time: float = 3600.0
    max_restart_attempts: int = 0
    node_replacer_cls: Optional[str] = None
    attention_backend: str = "auto"
    moe_token_dispatcher_type: str = "alltoall"
    moe_router_load_balancing_type: str = "none"
    moe_balance_loss_coef: float = 0.0
    moe_router_replay: bool = False
    offload_process_group: bool = False
    use_dynamic_mbs: bool = False
    ppo_dump_metrics_interval: Optional[int] = None
    calc_mfu_freq: int = 1
    use_linear_ce: bool = True
    linear_ce_backend: str = "separate"
    ce_compaction: bool = False
    # supervised objective: cross_entropy | square_averaging_cross_entropy (a token of a sample with N answer tokens
    # weighs 1 / sqrt(N), normalised by the global sum of sqrt(N))
    loss_func: str = "cross_entropy"
    cross_entropy_loss_fusion: bool = True
    per_token_loss: bool = True
    # RL / distillation: also train the multi-token-prediction blocks (model_config.mtp_num_layers) with a next-token
    # cross-entropy on the sampled responses; the trunk receives no gradient from it
    online_mtp_sft: bool = False
    sort_batched: bool = False
    manual_gc: bool = False
    manual_gc_interval: int = 1
    # parameter groups kept out of training (on top of policy.freeze_patterns); the vision ones apply to
    # vision-language policies
    freeze_moe_router: bool = False
    freeze_moe_shared_experts: bool = False
    freeze_llm: bool = False
    freeze_vit: bool = False
    freeze_projector: bool = False
    # selection bias of sigmoid routers (loss-free load balancing): frozen by default; when released it moves by
    # update_speed per step towards the mean expert load (sign update, or the log-ratio update)
    freeze_router_correction_bias: bool = True
    router_correction_bias_update_speed: float = 1e-3
    router_correction_bias_use_abs_update: bool = True
    # held-out evaluation inside the RL loop: also once before the first step; its own samples per prompt
    eval_before_train: bool = False
    eval_sampling_repeat_n: Optional[int] = None
    # RL-only
    total_ppo_step: Optional[int] = None
    ppo_step_per_epoch: Optional[int] = None
    dynamic_sampling: DynamicSamplingConfig = field(default_factory=DynamicSamplingConfig)
    rollout_gbs: int = 8
    rollout_mbs: int = 1
    sampling_repeat_n: int = 8
    sampling_keep_n: Optional[int] = None
    sampling_keeping_strategy: str = "all"
    filter_sampling_py_path: Optional[str] = None
    filter_sampling_fn_name: Optional[str] = None
    filter_sampling_stage: str = "pre"
    metrics_report: List[str] = field(default_factory=list)
    ppo_max_epochs_2: int = 1
    use_bt_rm_reward: bool = False
    use_gen_rm_reward: bool = False
    use_external_reward: bool = False
    stream_external_reward: bool = False
    early_swap_model: bool = False
    async_rollout: bool = False
    single_controller: bool = False
    dynamic_batch_train: bool = False
    rollout_max_staleness: int = 0
    rollout_over_dispatch_ratio: float = 1.0
    rollout_reuse_unused_prompts: bool = False
    num_agent_loop_workers: int = 4
    load_aware_sampler_routing: bool = False
    rb_multiplier: int = 1
    custom_actors: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if self.training_backend in ("mcore", "mlite"):
            self.training_backend = "native"   # the Megatron-style ZeRO-1 / TP / PP / CP / EP engine of this package
        if self.training_backend not in ("native", "nccl_eager", "fsdp2"):
            raise ConfigError(f"unknown training_backend {self.training_backend}")
        if self.loss_func not in ("cross_entropy", "square_averaging_cross_entropy"):
            raise ConfigError(f"training.loss_func must be cross_entropy|square_averaging_cross_entropy, "
                              f"got {self.loss_func}")
        if self.sampling_keep_n is None:
            self.sampling_keep_n = self.sampling_repeat_n
        if self.sampling_keep_n > self.sampling_repeat_n:
            raise ConfigError("sampling_keep_n cannot exceed sampling_repeat_n")
        if self.filter_sampling_stage not in ("pre", "post"):
            raise ConfigError("filter_sampling_stage must be pre|post")
        if self.rollout_max_staleness < 0:
            raise ConfigError("rollout_max_staleness must be >= 0")


@dataclass
class MonitorConfig(MappingMixin):
    heartbeat_interval: float = 30.0
    heartbeat_dir: Optional[str] = None
    enable_training_plt: bool = False


@dataclass
class CriticConfig(PolicyConfig):
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)


# ------------------------------------------------------------------------------------------------ top level
@dataclass
class BaseTopConfig(MappingMixin):
    data: DataConfig = field(default_factory=DataConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    policy: PolicyConfig = field(default_factory=PolicyConfig)
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    report: ReportConfig = field(default_factory=ReportConfig)
    monitor: MonitorConfig = field(default_factory=MonitorConfig)
    debug: DebugConfig = field(default_factory=DebugConfig)
    task: Dict[str, Any] = field(default_factory=dict)

    def world_size_required(self) -> int:
        d = self.policy.dist_config
        return d.tensor_model_parallel_size * d.pipeline_model_parallel_size * d.context_parallel_size


@dataclass
class FinetuneConfig(BaseTopConfig):
    def __post_init__(self):
        d = self.policy.dist_config
        if d.dynamic_context_parallel and not self.training.per_token_loss:
            # per-sequence means cannot be rebuilt after per-sequence CP re-sharding
            raise ConfigError("dynamic context parallel requires training.per_token_loss=true")


@dataclass
class PretrainConfig(FinetuneConfig):
    pass


@dataclass
class RlConfig(BaseTopConfig):
    placement_type: str = "colocate"
    # disaggregated placement: ranks [0, disaggregated_train_gpus) train, the others run rollout engines
    # (default: half of the job each)
    disaggregated_train_gpus: Optional[int] = None
    critic: Optional[CriticConfig] = None
    teacher: Optional[PolicyConfig] = None  # frozen teacher for on-policy distillation (advantage_type on_policy_distill)
    sampler: SamplerConfig = field(default_factory=SamplerConfig)
    gen_rm: Optional[SamplerConfig] = None
    bt_rm: RewardConfig = field(default_factory=RewardConfig)
    external_reward: Optional[RewardConfig] = None
    ppo: PpoConfig = field(default_factory=PpoConfig)

    def __post_init__(self):
        if self.placement_type not in ("colocate", "disaggregated", "partial_colocated"):
            raise ConfigError(f"unknown placement_type {self.placement_type}")
        t = self.training
        if (t.rollout_gbs * t.sampling_keep_n) % max(t.train_gbs, 1) and t.train_gbs > 0:
            raise ConfigError("rollout_gbs * sampling_keep_n must be a multiple of train_gbs")
        if self.ppo.advantage_type == "ppo" and self.critic is None:
            raise ConfigError("advantage_type=ppo needs a `critic:` section")
        if self.ppo.advantage_type in ("on_policy_distill", "g_opd") and self.teacher is None:
            raise ConfigError(f"advantage_type={self.ppo.advantage_type} needs a `teacher:` section")
        if t.rollout_max_staleness > 0 and not (t.async_rollout or t.single_controller):
            raise ConfigError("rollout_max_staleness > 0 needs async_rollout or single_controller")
        if t.use_gen_rm_reward and self.gen_rm is None:
            raise ConfigError("use_gen_rm_reward needs a `gen_rm:` section")
        if self.policy.dist_config.dynamic_context_parallel and not self.ppo.per_token_loss:
            raise ConfigError("dynamic context parallel requires ppo.per_token_loss=true")

    def require_critic_model(self) -> bool:
        return self.ppo.advantage_type == "ppo"


@dataclass
class DpoConfig(RlConfig):
    """``train_lm_dpo``: the sections of the RL configuration plus the preference-loss options at the top level."""
    dpo_beta: float = 0.1
    dpo_loss_type: str = "sigmoid"
    dpo_label_smoothing: float = 0.0
    dpo_sft_loss_coef: float = 0.0      # weight of the cross-entropy term on the chosen responses
    reference_free: bool = False

    _aliases = {"dpo_ftx_gamma": "dpo_sft_loss_coef"}

    def __post_init__(self):
        sup = getattr(super(), "__post_init__", None)
        if sup is not None:
            sup()
        if self.dpo_loss_type != "sigmoid":
            raise ConfigError(f"dpo_loss_type must be sigmoid, got {self.dpo_loss_type}")


@dataclass
class RewardTrainConfig(RlConfig):
    """``train_lm_reward_model``: ``rm_margin`` is subtracted from the chosen - rejected score gap."""
    rm_loss: str = "bt"  # Bradley-Terry pairwise
    rm_margin: float = 0.0

    def __post_init__(self):
        super().__post_init__() if hasattr(super(), "__post_init__") else None
        if self.rm_loss != "bt":
            raise ConfigError(f"rm_loss must be bt (Bradley-Terry), got {self.rm_loss}")


@dataclass
class DistillConfig(RlConfig):
    distill_type: str = "on_policy"  # on_policy | off_policy
    distill_topk: int = 0
    distill_loss: str = "reverse_kl"
    teacher: Optional[PolicyConfig] = None
    distill_alpha: float = 1.0


@dataclass
class EvaluateConfig(BaseTopConfig):
    sampler: SamplerConfig = field(default_factory=SamplerConfig)
    eval_repeat_n: int = 1


@dataclass
class InferenceConfig(EvaluateConfig):
    output_path: Optional[str] = None


# ---------------------------------------------------------------------------------------------------- image generation
@dataclass
class T2iModelConfig(MappingMixin):
    """Architecture of the diffusion transformer, its text encoder and its latent autoencoder (random init unless
    ``state_dict_path`` is given); fields of ``models.dit.DiTConfig`` under ``transformer``."""
    pipeline: str = "flux"   # flux | qwen_image_edit | flux_kontext | bagel
    transformer: Dict[str, Any] = field(default_factory=dict)
    text_layers: int = 2
    text_max_length: int = 32
    latent_channels: int = 16
    vae_factor: int = 8
    vae_base_channels: int = 16
    state_dict_path: Optional[str] = None
    freeze_text_encoder: bool = True
    freeze_vae: bool = True
    # bagel: width / depth of the unified decoder
    lm_hidden_size: int = 128
    lm_layers: int = 2
    lm_heads: int = 4
    lm_vocab_size: int = 258


@dataclass
class T2iTrainingConfig(MappingMixin):
    """Names follow the reference's text-to-image training section (gpatch_v4/configs/config.py ``T2i*`` and the use
    sites in extended_pipeline/pipeline_flux.py:232-535)."""
    seed: int = 42
    height: int = 64
    width: int = 64
    sampling_steps: int = 8
    shift: float = 3.0
    eta: float = 0.3
    guidance_scale: float = 3.5
    timestep_fraction: float = 0.5          # share of a trajectory's steps the update trains on
    rollout_gbs: int = 4                    # prompts per rollout, whole job
    rollout_mbs: int = 1
    rollout_model_mbs: Optional[int] = None
    sampling_repeat_n: int = 4
    same_noise_for_same_prompt: bool = False
    train_gbs_wo_timestep: int = 16         # trajectories per optimizer step, whole job
    train_mbs: int = 1
    train_gas_wo_timestep: int = 1
    total_ppo_step: int = 2
    total_training_step: int = 2
    gradient_accumulation_steps: int = 1
    train_method: str = "dpo"               # preference trainer: dpo | sft
    use_torch_autocast: bool = False
    use_bf16: bool = True
    gradient_checkpointing: bool = False
    ema_decay: float = 0.0
    save_interval: int = 0
    eval_interval: int = 0
    noise_scheme: str = "logit_normal"
    ce_loss_weight: float = 1.0             # bagel: weight of the text cross-entropy against the flow loss
    mse_loss_weight: float = 1.0

    def __post_init__(self):
        if not 0 < self.timestep_fraction <= 1:
            raise ConfigError("timestep_fraction must be in (0, 1]")
        if self.train_method not in ("dpo", "sft"):
            raise ConfigError("train_method must be dpo | sft")


@dataclass
class T2iPpoConfig(MappingMixin):
    ppo_ratio_eps: float = 1e-4
    ppo_clip_ratio_low: Optional[float] = None
    ppo_clip_ratio_high: Optional[float] = None
    adv_clip_min: float = -5.0
    adv_clip_max: float = 5.0
    grpo_advantage_epsilon: float = 1e-8
    reward_weights: Dict[str, float] = field(default_factory=dict)


@dataclass
class T2iDpoSection(MappingMixin):
    beta_dpo: float = 5000.0


@dataclass
class T2iConfig(MappingMixin):
    model: T2iModelConfig = field(default_factory=T2iModelConfig)
    training: T2iTrainingConfig = field(default_factory=T2iTrainingConfig)
    ppo: T2iPpoConfig = field(default_factory=T2iPpoConfig)
    dpo: T2iDpoSection = field(default_factory=T2iDpoSection)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    data: DataConfig = field(default_factory=DataConfig)
    bt_rm: RewardConfig = field(default_factory=RewardConfig)
    report: ReportConfig = field(default_factory=ReportConfig)
    debug: DebugConfig = field(default_factory=DebugConfig)
    task: Dict[str, Any] = field(default_factory=dict)
