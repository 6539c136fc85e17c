"""Typed configuration.

Field names follow the Megatron/Primus knob vocabulary that the reference's run
notes quote (``notes/2026-04/2026-04-19_gptoss_01_mlperf_best_e2e_run.md:60-110``,
``notes/2026-04/2026-04-28_gptoss_27_mlperf_legal_baseline.md:165-177``) so a
user of those launch scripts recognises every knob.

Design rules, each one a pitfall recorded by the reference:

* Booleans are parsed strictly: the *string* ``"false"`` is False, anything that
  is not a recognised boolean literal is an error
  (``notes/2026-04/2026-04-24_gptoss_20_truthy_flag_fix.md``: env substitution
  produced a truthy ``"false"``).
* One resolution order: dataclass defaults < preset < YAML file < ``key=value``
  command line overrides.  Nothing else (no env var, no runtime ``setattr``)
  may change a value (``notes/2026-04/2026-04-25_gptoss_22_*:20-44``).
* The resolved config is dumped next to the run so what ran is what is written
  (``notes/mlperf-llama/*meeting_summary_en.md:35,49-57``).
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field, fields, is_dataclass
from pathlib import Path
from typing import Any, get_type_hints

_TRUE = {"true", "1", "yes", "on"}
_FALSE = {"false", "0", "no", "off"}


class ConfigError(ValueError):
    pass


def parse_bool(v: Any) -> bool:
    """Strict boolean parse; rejects anything that is not a boolean literal."""
    if isinstance(v, bool):
        return v
    if isinstance(v, int) and v in (0, 1):
        return bool(v)
    if isinstance(v, str):
        s = v.strip().lower()
        if s in _TRUE:
            return True
        if s in _FALSE:
            return False
    raise ConfigError(f"not a boolean literal: {v!r}")


@dataclass
class ModelConfig:
    name: str = "simplemoe-tiny"
    num_layers: int = 2
    hidden_size: int = 256
    num_attention_heads: int = 4
    num_query_groups: int = 4            # KV heads (GQA)
    kv_channels: int = 64                # head_dim
    vocab_size: int = 1024
    seq_length: int = 128
    rotary_base: float = 10000.0
    norm_epsilon: float = 1e-6
    init_method_std: float = 0.02
    tie_embeddings: bool = False
    # attention flavour: "gqa" (multi/grouped query) or "mla" (DeepSeek latent attention)
    attention_type: str = "gqa"
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    sliding_window: int = 0              # 0 = full causal; >0 on alternate layers (GPT-OSS style)
    # low-rank adapters (LoRA fine-tuning): > 0 freezes every other parameter and trains rank-r updates of the
    # attention projections ("attn") or of the attention and dense feed-forward projections ("attn+mlp")
    lora_rank: int = 0
    lora_alpha: float = 32.0
    lora_targets: str = "attn"
    # dense FFN (used by the first `first_k_dense` layers and by non-MoE models)
    ffn_hidden_size: int = 1024
    first_k_dense: int = 0
    # MoE
    num_experts: int = 8
    moe_router_topk: int = 2
    moe_ffn_hidden_size: int = 512
    moe_shared_expert_intermediate_size: int = 0
    moe_router_score_function: str = "softmax"   # softmax | sigmoid
    moe_router_load_balancing_type: str = "aux_loss"  # aux_loss | bias | none
    moe_aux_loss_coeff: float = 0.0
    moe_router_bias_update_rate: float = 1e-3
    moe_router_dtype: str = "fp32"
    moe_router_topk_scaling_factor: float = 1.0
    moe_norm_topk_prob: bool = True
    moe_token_dispatcher_type: str = "fused"     # fused (peer-memory kernels) | alltoall (NCCL baseline)
    moe_grouped_gemm: bool = True
    moe_permute_fusion: bool = True
    moe_pad_expert_rows_to: int = 128    # expert segments start on tile boundaries
    moe_router_force_load_balancing: bool = False  # benchmarking aid: route by fixed random logits
    moe_capacity_factor: float = 0.0     # fused dispatcher buffers: 0 = dropless worst case, >0 = x balanced load
    moe_expert_relocation_interval: int = 0   # > 0: every that many steps, re-place experts on ranks by measured load; -1: automatic (every 50 steps plus once at step 3 where the layout supports it: ep > 1, ep == dp, cp == tp == 1; off elsewhere)
    moe_expert_relocation_first_step: int = 0    # > 0: also decide once at this step (early skew of a fresh router)
    moe_expert_relocation_min_gain: float = 0.05  # relative drop of max/mean rank load that justifies moving experts
    moe_combine_push: bool = True        # expert GEMM epilogues push result rows to the token owners (fused combine)
    moe_expert_ordered_dispatch: bool = True   # rows travel expert by expert with one arrival flag per (source, expert); the expert GEMM waits per expert inside the kernel
    moe_scatter_bulk_store: bool = False  # expert-ordered bf16 scatter sends rows with cp.async.bulk stores out of shared memory instead of per-lane 16-byte stores
    moe_scatter_overlap: bool = False    # ep > 1: the remote half of a dispatch scatter runs on a side stream beside the expert GEMM that consumes the rows
    moe_keep_dispatched_factor: float = 0.0  # selective recompute keeps the dispatched rows instead of re-dispatching: >0 = fixed copy of x balanced load (one host wait per step at the start of backward; a layer whose rows did not fit the copy on some rank is dispatched again on every rank), <0 = exactly the rows in use (one host read per layer), 0 = off


@dataclass
class ParallelConfig:
    tensor_model_parallel_size: int = 1
    sequence_parallel: bool = False      # with tp > 1: residual stream, norms and MoE blocks hold 1/tp of every sequence; all-gather / reduce-scatter around the split matrices instead of all-reduces
    tp_fused_gemm_reduce_scatter: bool = True   # sequence_parallel on GPUs: row-split GEMMs push their tiles to the rows' owners over peer memory (GEMM + reduce-scatter in one exchange) instead of GEMM then NCCL reduce-scatter
    expert_tensor_parallel_size: int = 1   # 1: MoE blocks take 1/tp of the tokens per tensor-parallel rank; tp: every rank routes all tokens and holds 1/tp of each local expert's feed-forward columns
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    context_parallel_size: int = 1
    fsdp: bool = True                    # shard params/grads/optimizer state over the data axis
    use_distributed_optimizer: bool = True
    overlap_grad_reduce: bool = True
    overlap_param_gather: bool = True
    grad_reduce_in_bf16: bool = True
    ddp_bucket_size: int = 40_000_000    # elements
    ddp_average_in_collective: bool = True
    num_distributed_optimizer_instances: int = 1
    fsdp_fused_collectives: bool = True  # peer-memory all-gather / reduce-scatter kernels instead of NCCL
    fsdp_nvls_reduce: bool = False       # peer reduce-scatter sums through the switch (multimem.ld_reduce on the workspaces' multicast address) instead of one peer load per rank
    fsdp_prefetch: bool = False          # gather the next unit's parameters on a side stream while this one computes
    fsdp_gather_in_gemm: bool = True     # forward: a decoder layer's dense matrices are all-gathered inside the first GEMM that multiplies one of them (peer collectives only)


@dataclass
class PrecisionConfig:
    params_dtype: str = "fp32"           # fp32 | bf16
    fp8: bool = False                    # fp8 (e4m3) forward of the expert GEMMs, bf16 backward
    fp8_dgrad: bool = False              # with fp8: input gradients of the expert GEMMs in e4m3 as well (row-scaled, transposed weight copy cached per optimizer step); weight gradients stay bf16
    fp8_recipe: str = "rowwise"          # rowwise (per token row / per output channel, full fp8 rate) | tensorwise (one scale per tensor, same kernel) | blockwise (1x128 act, 128x128 weight)
    num_layers_at_start_in_bf16: int = 0
    num_layers_at_end_in_bf16: int = 0
    master_weights: bool = True          # fp32 master copy when params are bf16
    optimizer_state_dtype: str = "fp32"  # fp32 | bf16 | fp8 (block scaled 8-bit moments)
    recompute_granularity: str = "none"  # none | selective | full


@dataclass
class TrainConfig:
    micro_batch_size: int = 4
    global_batch_size: int = 8
    train_iters: int = 20
    seed: int = 0
    lr: float = 3e-4
    min_lr: float = 0.0
    lr_warmup_iters: int = 0
    lr_decay_iters: int = 0
    lr_decay_style: str = "constant"     # constant | cosine | linear | wsd (flat, then linear over the last lr_wsd_decay_iters)
    lr_wsd_decay_iters: int = 0
    weight_decay: float = 0.1
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8
    clip_grad: float = 1.0
    deferred_loss_read: bool = False     # fit(): read a step's loss and gradient norm (pinned buffer) after the next step has been launched, so the device never idles between steps; steps that evaluate, save or may leave are read at once; log lines appear one step late
    optimizer_in_backward: bool = False  # apply AdamW per layer during backward (no grad buffer kept)
    optimizer_background_piece: int = 33554432   # elements per launch of a side-stream AdamW update (multiple of 512; 0 = one launch): bounds how long a compute-stream kernel with large blocks waits for room on the SMs
    eval_interval: int = 0
    eval_iters: int = 0
    log_interval: int = 1
    check_for_nan_in_loss_and_grad: bool = True
    data: str = "synthetic"              # "synthetic" (uniform-random token ids) or the path of a token file
    eval_data: str = ""                  # token file for evaluation ("" = held-out steps of `data`)
    eval_target_loss: float = 0.0        # > 0: training stops when the evaluation loss reaches it
    device: str = "auto"                 # auto | cpu | cuda
    use_cuda_kernels: str = "auto"       # auto | true | false : hand written sm_100a ops vs PyTorch oracle path
    dense_gemm_kernels: bool = True      # dense projections and the vocabulary GEMMs on the hand-written tcgen05 GEMM (false: library GEMM, the comparison path)
    hang_timeout_s: float = 300.0
    heartbeat: bool = True               # ranks publish per-step heartbeats; a peer stuck for hang_timeout_s is reported
    fault_injection: str = ""            # host-side test faults, e.g. "delay:rank=1,step=3,seconds=5;nan:rank=0,step=4"
    mllog: bool = False
    metrics_file: str = ""               # rank 0 appends one JSON line per logged step (loss, step time, tokens/s, memory, MoE load)
    manual_gc: bool = False              # turn the cyclic garbage collector off and collect every `manual_gc_interval` steps on every rank at once (a collection on one rank otherwise stalls all: `summary/training-1024g*:41-101`)
    manual_gc_interval: int = 50
    exit_duration_in_mins: float = 0.0   # > 0: stop (after saving) once the job has run this long; decided on rank 0, applied by all
    exit_signal_handler: bool = False    # SIGTERM on any rank: all ranks finish the step, save a checkpoint and leave (preemption)


@dataclass
class CheckpointConfig:
    save: str = ""
    load: str = ""
    save_interval: int = 0
    disable_last_saving: bool = False
    keep_last: int = 2
    async_save: bool = False             # copy the state to host memory, write it in the background, publish it at a later step boundary


@dataclass
class ProfileConfig:
    profile: bool = False
    profile_step_start: int = 16
    profile_step_end: int = 18
    profile_ranks: list = field(default_factory=lambda: [0])
    torch_profiler_with_stack: bool = False
    torch_profiler_record_shapes: bool = False
    trace_dir: str = "traces"
    snapshot_path: str = ""              # write the tuner Snapshot JSON here at run end


@dataclass
class Config:
    model: ModelConfig = field(default_factory=ModelConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    precision: PrecisionConfig = field(default_factory=PrecisionConfig)
    train: TrainConfig = field(default_factory=TrainConfig)
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    profile: ProfileConfig = field(default_factory=ProfileConfig)

    # ---- construction -------------------------------------------------
    @staticmethod
    def from_dict(d: dict) -> "Config":
        cfg = Config()
        cfg.update(d)
        return cfg

    @staticmethod
    def load(path: str | Path | None = None, overrides: list[str] | None = None,
             preset: str | None = None) -> "Config":
        from .models.presets import PRESETS
        cfg = Config()
        if preset:
            if preset not in PRESETS:
                raise ConfigError(f"unknown preset {preset!r}; have {sorted(PRESETS)}")
            cfg.update(PRESETS[preset])
        if path:
            import yaml
            text = Path(path).read_text()
            data = yaml.safe_load(text) or {}
            if "preset" in data:
                p = data.pop("preset")
                if p not in PRESETS:
                    raise ConfigError(f"unknown preset {p!r}")
                cfg.update(PRESETS[p])
            cfg.update(data)
        for ov in overrides or []:
            if "=" not in ov:
                raise ConfigError(f"override must be key=value, got {ov!r}")
            k, v = ov.split("=", 1)
            cfg.set(k.strip(), v.strip())
        cfg.validate()
        return cfg

    def update(self, d: dict) -> None:
        for k, v in d.items():
            if is_dataclass(getattr(self, k, None)) and isinstance(v, dict):
                for kk, vv in v.items():
                    self.set(f"{k}.{kk}", vv)
            else:
                self.set(k, v)

    def _find(self, key: str):
        """Resolve ``section.name`` or a bare leaf name that is unique across sections."""
        if "." in key:
            sec, name = key.split(".", 1)
            if not hasattr(self, sec):
                raise ConfigError(f"unknown config section {sec!r}")
            obj = getattr(self, sec)
            if not any(f.name == name for f in fields(obj)):
                raise ConfigError(f"unknown config key {key!r}")
            return obj, name
        hits = [(getattr(self, s.name), key) for s in fields(self)
                if any(f.name == key for f in fields(getattr(self, s.name)))]
        if not hits:
            raise ConfigError(f"unknown config key {key!r}")
        if len(hits) > 1:
            raise ConfigError(f"ambiguous config key {key!r}; qualify it with a section")
        return hits[0]

    def set(self, key: str, value: Any) -> None:
        obj, name = self._find(key)
        hint = get_type_hints(type(obj))[name]
        setattr(obj, name, _coerce(value, hint, key))

    def get(self, key: str) -> Any:
        obj, name = self._find(key)
        return getattr(obj, name)

    # ---- output ---------------------------------------------------------
    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    def dump(self, path: str | Path) -> None:
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        Path(path).write_text(json.dumps(self.to_dict(), indent=2, sort_keys=True))

    # ---- legality (the tuner's constraint rules use the same function) ---
    def validate(self, world_size: int | None = None) -> None:
        from .pilot.constraints import check_config
        problems = [p for p in check_config(self, world_size) if p["severity"] == "error"]
        if problems:
            raise ConfigError("; ".join(p["message"] for p in problems))


def _coerce(value: Any, hint: Any, key: str) -> Any:
    if hint is bool:
        return parse_bool(value)
    if hint is int:
        if isinstance(value, bool):
            raise ConfigError(f"{key}: expected int, got bool")
        if isinstance(value, str):
            try:
                return int(value.replace("_", ""))
            except ValueError:
                raise ConfigError(f"{key}: expected int, got {value!r}") from None
        if isinstance(value, float) and value != int(value):
            raise ConfigError(f"{key}: expected int, got {value}")
        return int(value)
    if hint is float:
        if isinstance(value, bool):
            raise ConfigError(f"{key}: expected float, got bool")
        try:
            return float(value)
        except (TypeError, ValueError):
            raise ConfigError(f"{key}: expected float, got {value!r}") from None
    if hint is str:
        if value is None:
            return ""
        return str(value)
    if hint is list or getattr(hint, "__origin__", None) is list:
        if isinstance(value, str):
            value = json.loads(value) if value.startswith("[") else [int(x) for x in value.split(",") if x]
        return list(value)
    return value
