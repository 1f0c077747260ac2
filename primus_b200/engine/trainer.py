"""The training engine: model + buffers + optimizer + schedule + data, and the per-step loop.

One :class:`Trainer` per process (one process per GPU).  A step is

    zero grads -> forward/backward over the micro-batches (pipeline schedule when PP > 1)
    -> finalize grads (DP reduce-scatter / all-reduce, SP norm-weight all-reduce, tied-embedding
       all-reduce) -> clip + AdamW on the local shards -> parameter all-gather -> LR step,

which is the loop the reference delegates to ``megatron.training.pretrain``
(primus/backends/megatron/megatron_pretrain_trainer.py:254-260; grads finalisation
primus/backends/megatron/core/distributed/finalize_model_grad.py:23-74).  The log line carries the
reference's throughput fields — elapsed ms per iteration, TFLOP/s/GPU and tokens/s/GPU with the
windowed harmonic mean (primus/backends/megatron/patches/training_log/print_rank_last_patches.py:435-548).
"""
from __future__ import annotations

import gc
import math
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch
import torch.distributed as dist

from ..models.config import TransformerConfig
from ..models.gpt import build_model
from ..ops import gemm as _gemm_ops
from ..parallel import state as ps
from ..parallel.distributed import DistributedOptimizer, ParamGradBuffer
from . import schedules
from .data import BatchStager, MicroBatchSampler, MockGPTDataset


@dataclass
class TrainConfig:
    """Trainer-level options (names follow primus/configs/modules/megatron/trainer_base.yaml)."""
    micro_batch_size: int = 1
    global_batch_size: int = 8
    seq_length: int = 512
    train_iters: int = 10
    lr: float = 3e-4
    min_lr: float = 0.0
    lr_decay_style: str = "cosine"
    lr_warmup_iters: int = 0
    lr_warmup_fraction: Optional[float] = None    # warm-up as a share of the decay length (instead of lr_warmup_iters)
    lr_warmup_init: float = 0.0                   # learning rate the warm-up starts from
    lr_decay_iters: Optional[int] = None
    lr_wsd_decay_style: str = "exponential"       # shape of the final anneal of lr_decay_style WSD
    lr_wsd_decay_iters: Optional[int] = None      # length of that anneal
    start_weight_decay: Optional[float] = None    # weight-decay schedule: from here ...
    end_weight_decay: Optional[float] = None      # ... to here ...
    weight_decay_incr_style: str = "constant"     # ... constant | linear | cosine over the decay length
    weight_decay: float = 0.1
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8
    clip_grad: float = 1.0
    use_distributed_optimizer: bool = True
    optimizer: str = "adam"          # adam | sgd | muon (sgd / muon need use_distributed_optimizer = false)
    sgd_momentum: float = 0.9
    muon_momentum: float = 0.95
    muon_use_nesterov: bool = True
    muon_num_ns_steps: int = 5
    overlap_grad_reduce: bool = False
    overlap_param_gather: bool = False
    grad_reduce_in_bf16: bool = False    # bf16 on the wire for the data-parallel gradient reduction (fp32 accumulation)
    # trace analysis and artifacts (role of the reference's TraceLens / MLflow upload switches)
    generate_tracelens_report: bool = False        # write a kernel-category report of this rank's profiler traces
    mlflow_upload_tracelens_report: bool = False   # also hand the reports to the artifact sinks (implies generation)
    mlflow_upload_traces: bool = False             # hand the raw trace files to the artifact sinks
    mlflow_tracelens_ranks: Optional[list] = None  # ranks that write a report (None: every profiled rank)
    mlflow_tracelens_output_format: str = "md"     # md | csv | tsv | jsonl
    num_seq_splits: int = 1              # sequence chunks per micro-batch that travel through the pipeline separately
    enable_optimizer_post_validation: bool = False        # pipeline parallel: update first, validate the global norm later
    enable_exact_optimizer_post_validation: bool = True   # restore from a snapshot (exact) instead of inverting the update
    enable_odc: bool = False             # on-demand communication: gradient pushes / parameter pulls, one meeting per step
    odc_grad_spike_threshold: float = 1000.0
    ddp_bucket_size: Optional[int] = None
    seed: int = 1234
    data_seed: int = 1234
    mock_data: bool = True
    mock_data_period: int = 0          # > 0: learnable periodic sequences instead of uniform-random tokens
    eod_token: Optional[int] = None    # indexed corpora: id of the end-of-document token
    eod_mask_loss: bool = False        # ... no loss on it
    reset_position_ids: bool = False   # ... positions restart after it
    mock_data_kind: str = ""           # "markov": learnable first-order Markov chain (smooth loss curve)
    data_path: Optional[str] = None
    log_interval: int = 1
    log_avg_skip_iterations: int = 2
    log_avg_reset_interval: int = 50
    check_for_nan_in_loss_and_grad: bool = True
    calculate_per_token_loss: bool = False
    save: Optional[str] = None
    load: Optional[str] = None
    save_interval: Optional[int] = None
    ckpt_format: str = "torch_dist"          # torch_dist (torch.distributed.checkpoint files) | torch (pickle per rank)
    auto_detect_ckpt_format: bool = False
    async_save: bool = False                 # file writing on a side thread; the step loop continues after the D2H copy
    ckpt_fully_parallel_save: bool = True    # replicated tensors are written by different data-parallel ranks
    ckpt_fully_parallel_load: bool = False   # ... and read by one of them each, then broadcast
    dist_ckpt_strictness: str = "assume_ok_unexpected"
    finetune: bool = False                   # load weights only; iteration, optimizer and RNG start fresh
    no_load_optim: bool = False
    no_save_optim: bool = False
    no_load_rng: bool = False
    no_save_rng: bool = False
    exit_interval: Optional[int] = None
    exit_duration_in_mins: Optional[float] = None
    exit_signal_handler: bool = False
    dump_pp_data: bool = False         # per-node pipeline timeline (one JSON per pipeline rank and iteration; it
    pp_dump_dir: Optional[str] = None  # synchronises after every node, so the timed iterations are slower)
    pp_warmup: bool = False            # throw-away fwd + bwd on every pipeline stage at once before the first iteration
    timing_log_level: int = 0          # 0: no step timers; 1: forward-backward / optimizer ...; 2: + batch staging
    timing_log_option: str = "minmax"  # max | minmax | all (how the per-rank times are reported)
    log_timers_to_tensorboard: bool = False   # also hand the step timers (max over ranks, ms) to the metric sinks
    torch_profiler_record_shapes: bool = True
    torch_profiler_with_stack: bool = False
    torch_profiler_use_gzip: bool = False     # write <trace>.json.gz
    mlflow_run_name: Optional[str] = None     # run name for the MLflow / W&B sinks (default: exp_name)
    use_torch_fsdp2: bool = False      # shard parameters / gradients / optimizer state over the data-parallel ranks
    data_parallel_replicate_degree: int = 1   # with use_torch_fsdp2: HSDP, shard inside world / degree ranks, replicate across
    use_precision_aware_optimizer: bool = False   # Adam moments in exp_avg_dtype / exp_avg_sq_dtype ("fp32" | "bf16")
    exp_avg_dtype: str = "fp32"
    exp_avg_sq_dtype: str = "fp32"
    main_params_dtype: str = "fp32"
    main_grads_dtype: str = "fp32"
    inprocess_restart: bool = False    # reload the newest checkpoint and continue after a failure all ranks agree on
    inprocess_max_restarts: int = 3
    check_for_spiky_loss: bool = False
    check_for_large_grads: bool = False
    rerun_mode: str = "disabled"
    error_injection_rate: float = 0.0
    error_injection_type: str = "transient_error"
    log_straggler: bool = False
    eval_interval: Optional[int] = None
    split: Optional[str] = None           # "99,1,0": train / validation / test shares of the samples of ``data_path``
    valid_data_path: Optional[str] = None
    eval_iters: int = 0
    pipeline_schedule: str = "1f1b"  # 1f1b | interleaved | zerobubble | zbv | v-half | v-min
    # cost-driven re-planning of the B / W-split schedules: node times (and, on GPUs, activation bytes) are measured in
    # iterations [start, end) and the table for the following iterations is built from them (end <= start: off)
    zero_bubble_pipeline_timers_start_iter: int = 0
    zero_bubble_pipeline_timers_end_iter: int = 0
    zero_bubble_adaptive_memory_limit_percentile: float = 85.0   # share of device memory the plan may fill
    zero_bubble_max_pending_backward: object = "auto"   # int: activation budget per rank in forwards instead of adaptive
    pipeline_model_parallel_layout: Optional[str] = None
    decoder_pipeline_manual_split_list: Optional[list] = None
    # uneven splits without a layout string: sizes of the first / last stage (the others share the rest evenly), or the
    # embedding / output layer counted as one layer of their stage
    decoder_first_pipeline_num_layers: Optional[int] = None
    decoder_last_pipeline_num_layers: Optional[int] = None
    account_for_embedding_in_pipeline_split: bool = False
    account_for_loss_in_pipeline_split: bool = False
    manual_gc: bool = True
    fused_dp_optimizer: bool = False  # P2P reduce-scatter + AdamW kernel over symmetric memory
    num_workers: int = 0                         # data loading threads (0: the training thread loads its own batches)
    use_tp_pp_dp_mapping: bool = False           # rank order tensor, context, pipeline, data (default: ..., data, pipeline)
    log_throughput: bool = True                  # TFLOP/s/GPU and tokens/s/GPU in the per-iteration log line
    train_samples: Optional[int] = None          # alternative to train_iters: stop after this many samples
    # costs for the cost-driven zero-bubble tables, given instead of measured (a number, or one per virtual stage)
    pp_cost_f: object = None
    pp_cost_b: object = None
    pp_cost_w: object = None
    pp_max_mem: object = None                    # activation limit per pipeline rank, in chunk-forwards
    debug_scheduler_table: bool = False          # print the schedule table when it is built
    decoupled_lr: Optional[float] = None         # own learning rate (and decoupled_min_lr) for the embeddings and the output layer
    decoupled_min_lr: Optional[float] = None
    head_lr_mult: float = 1.0                    # learning-rate multiplier of the output layer
    rampup_batch_size: Optional[list] = None     # [start, increment, samples]: the global batch grows during the first samples
    ckpt_step: Optional[int] = None              # load the checkpoint of this iteration instead of the newest
    exit_on_missing_checkpoint: bool = False     # ``load`` is set but holds no checkpoint: stop instead of starting fresh
    pretrained_checkpoint: Optional[str] = None  # weights to start from when ``load`` holds nothing (iteration 0, no optimizer state)
    override_opt_param_scheduler: bool = False   # after a load keep this run's LR / WD schedule (what happens by default)
    use_checkpoint_opt_param_scheduler: bool = False   # after a load continue with the schedule stored in the checkpoint
    save_retain_interval: Optional[int] = None   # keep only the checkpoints of multiples of this (and the newest)
    iterations_to_skip: Optional[list] = None    # iterations whose batch is read but not trained on
    skip_train: bool = False                     # no training: load, evaluate if asked, leave
    log_params_norm: bool = False                # L2 norm of the parameters in the log line and the metrics
    log_num_zeros_in_grad: bool = False          # number of exactly-zero gradient entries
    manual_gc_interval: int = 0                  # with manual_gc: collect every N iterations (0: never during training)
    check_weight_hash_across_dp_replicas_interval: Optional[int] = None   # compare the replicas' parameters every N steps
    wandb_exp_name: Optional[str] = None
    wandb_entity: Optional[str] = None
    wandb_save_dir: Optional[str] = None
    # checkpoint format conversion: load as usual, write in ``ckpt_convert_format`` (torch | torch_dist) under
    # ``ckpt_convert_save`` and leave without training
    ckpt_convert_format: Optional[str] = None
    ckpt_convert_save: Optional[str] = None
    # MLPerf-style structured log (engine/mlperf_logging.py); training ends when the validation loss reaches the target
    mlperf_mode: bool = False
    mlperf_benchmark: str = "llm_pretraining"
    mlperf_target_eval_loss: Optional[float] = None
    mlperf_submission_org: str = "primus_b200"
    mlperf_submission_platform: str = "B200"
    mlperf_log_path: Optional[str] = None
    pretrained_hf_path: Optional[str] = None     # directory of Hugging Face weights to start from (when no checkpoint is loaded)
    export_hf_path: Optional[str] = None         # write the trained weights in Hugging Face layout after the last step
    sft_grad_sanitize: bool = False   # zero non-finite gradient entries instead of skipping / failing the step
    # MXFP4 weight de-oscillation (parallel/weight_deosc.py): over windows of ``period`` steps, elements whose quantised
    # value travelled ``ratio`` times further than their master value are snapped onto their current code
    weight_deosc: bool = False
    weight_deosc_period: int = 200
    weight_deosc_ratio: float = 4.0
    weight_deosc_start_step: int = 0
    weight_deosc_log_freq: int = 0
    # frequent throw-away checkpoints next to the persistent ones: only the newest is kept, and a resume takes whichever
    # of the two kinds is newer.  type: "global" (under <save>/non_persistent or non_persistent_global_ckpt_dir), "local"
    # (a node-local directory: single-node jobs) or "in_memory" (a directory in /dev/shm: survives a process restart on
    # the node, not a node loss)
    non_persistent_ckpt_type: Optional[str] = None
    non_persistent_save_interval: Optional[int] = None
    non_persistent_global_ckpt_dir: Optional[str] = None
    non_persistent_local_ckpt_dir: Optional[str] = None
    # with fused_dp_optimizer: the updated parameter shards are pulled by the copy engines on a side stream (one
    # cudaMemcpyAsync per peer and bucket, no SM time) instead of being stored to the peers by the AdamW kernel; also
    # switched on by ENABLE_SDMA_ALLGATHER=1, the reference's switch for its copy-engine parameter all-gather
    param_gather_copy_engine: bool = False
    profile: bool = False
    profile_step_start: int = 3
    profile_step_end: int = 4
    profile_ranks: Optional[list] = None
    disable_profiler_activity_cpu: bool = False
    record_memory_history: bool = False
    memory_snapshot_path: Optional[str] = None
    nvtx_ranges: bool = False
    tensorboard_dir: Optional[str] = None     # also the directory of metrics.jsonl and profiler traces
    disable_tensorboard: bool = True
    wandb_project: Optional[str] = None
    mlflow_experiment_name: Optional[str] = None
    exp_name: str = "exp"

    @classmethod
    def from_dict(cls, d: dict) -> "TrainConfig":
        import dataclasses

        names = {f.name for f in dataclasses.fields(cls)}
        kw = {k: v for k, v in d.items() if k in names}
        if "pipeline_schedule" not in d and d.get("pp_algorithm"):
            kw["pipeline_schedule"] = d["pp_algorithm"]
        if "pipeline_schedule" not in d and not d.get("pp_algorithm") and d.get("enable_zero_bubble"):
            # the reference's switches: enable_zero_bubble (+ zero_bubble_v_schedule, ..._mem_setup zb | half | min)
            v = {"zb": "zbv", "half": "v-half", "min": "v-min"}[str(d.get("zero_bubble_v_schedule_mem_setup", "zb"))]
            kw["pipeline_schedule"] = v if d.get("zero_bubble_v_schedule") else "zerobubble"
        if d.get("tp_comm_overlap"):
            from ..parallel import fused_tp

            fused_tp.ENABLED = True
            fused_tp.ENABLED_RS = bool(d.get("tp_comm_overlap_rs", False))
        gbs = int(kw.get("global_batch_size", cls.global_batch_size))
        if d.get("train_samples"):      # sample-based run length (Megatron's train_samples): whole global batches
            kw["train_iters"] = int(d["train_samples"]) // gbs
        for samples, iters in (("lr_warmup_samples", "lr_warmup_iters"), ("lr_decay_samples", "lr_decay_iters")):
            if d.get(samples):          # sample-based schedule lengths
                kw[iters] = int(d[samples]) // gbs
        return cls(**kw)


def _open_corpus(data_path, seq_length: int, seed: int, tc):
    """Token corpus for pre-training: a Megatron indexed dataset (``<prefix>.idx`` + ``<prefix>.bin``, or a
    ``weight prefix ...`` blend) when the index file exists, else the flat token file of ``primus data tokenize``."""
    import os

    from .data import IndexedTokenDataset

    parts = data_path.split() if isinstance(data_path, str) else list(data_path)
    first = parts[1] if len(parts) > 1 else parts[0]
    if os.path.exists(first + ".idx"):
        from .indexed_dataset import build_gpt_dataset

        return build_gpt_dataset(parts, seq_length, seed, eod_token=getattr(tc, "eod_token", None),
                                 eod_mask_loss=bool(getattr(tc, "eod_mask_loss", False)),
                                 reset_position_ids=bool(getattr(tc, "reset_position_ids", False)))
    return IndexedTokenDataset(parts[0], seq_length)


class SplitView:
    """Samples ``[lo, hi)`` of a dataset, repeated when a run reads past the end."""

    def __init__(self, dataset, lo: int, hi: int):
        assert hi > lo, "an empty share of the data: check the split weights"
        self.dataset, self.lo, self.n = dataset, lo, hi - lo

    def __len__(self):
        return self.n

    def __getitem__(self, i: int):
        return self.dataset[self.lo + i % self.n]


def split_view(dataset, split: str, which: int):
    """Share ``which`` (0 train, 1 validation, 2 test) of a dataset cut by the weights ``split`` ("99,1,0": the first
    99 % of the samples for training, the next 1 % for validation), as Megatron's ``--split`` cuts its sample index."""
    w = [float(x) for x in str(split).replace("/", ",").split(",")]
    w += [0.0] * (3 - len(w))
    total, n = sum(w), len(dataset)
    edges = [0]
    for x in w:
        edges.append(edges[-1] + x / total)
    lo, hi = int(round(edges[which] * n)), int(round(edges[which + 1] * n))
    return SplitView(dataset, lo, hi)


class ThroughputMeter:
    """tokens/s/GPU = seq * global_batch / elapsed_s / world; running figure = harmonic mean over a
    window that skips the first iterations and is reset periodically."""

    def __init__(self, skip: int = 2, reset_interval: int = 50):
        self.skip, self.reset_interval = skip, reset_interval
        self.seen = 0
        self.inv_sum = 0.0
        self.n = 0

    def update(self, tokens_per_s_gpu: float) -> float:
        self.seen += 1
        if self.seen <= self.skip:
            return tokens_per_s_gpu
        if self.reset_interval and self.n >= self.reset_interval:
            self.inv_sum, self.n = 0.0, 0
        self.inv_sum += 1.0 / max(tokens_per_s_gpu, 1e-9)
        self.n += 1
        return self.n / self.inv_sum


def init_parallel_state(model_cfg, train_cfg):
    """Process groups for the configured parallel sizes (``use_tp_pp_dp_mapping``: pipeline stages on neighbouring ranks,
    data-parallel replicas far apart, instead of the other way round)."""
    return ps.initialize_model_parallel(
        tp=model_cfg.tensor_model_parallel_size, pp=model_cfg.pipeline_model_parallel_size,
        cp=model_cfg.context_parallel_size, ep=model_cfg.expert_model_parallel_size,
        etp=model_cfg.expert_tensor_parallel_size or 1, virtual_pp=model_cfg.virtual_pipeline_model_parallel_size,
        hierarchical_cp_sizes=model_cfg.hierarchical_context_parallel_sizes if model_cfg.cp_comm_type == "a2a+p2p" else None,
        tp_pp_dp_mapping=bool(getattr(train_cfg, "use_tp_pp_dp_mapping", False)))


class Trainer:
    def __init__(self, model_cfg: TransformerConfig, train_cfg: TrainConfig, device: Optional[str] = None,
                 log_fn: Callable[[str], None] = print):
        self.mcfg, self.tcfg = model_cfg, train_cfg
        self.log = log_fn
        self.num_seq_splits = max(1, int(train_cfg.num_seq_splits or 1))
        if self.num_seq_splits > 1:
            # sequence chunks travel through the pipeline as separate units; attention keeps the earlier chunks' K / V
            S = self.num_seq_splits
            unit = 128 * S if str(device or "cuda").startswith("cuda") else S
            assert train_cfg.seq_length % unit == 0, f"num_seq_splits = {S}: seq_length must be a multiple of {unit}"
            bad = [n for n, on in (("context parallelism", model_cfg.context_parallel_size > 1),
                                   ("multi-latent attention", model_cfg.multi_latent_attention),
                                   ("Mamba / delta-net / convolution mixers", model_cfg.model_type == "mamba" or bool(model_cfg.lfm_layer_types)),
                                   ("activation recompute", bool(model_cfg.recompute_granularity)),
                                   ("multi-token prediction", bool(model_cfg.mtp_num_layers)),
                                   ("virtual pipeline stages", bool(model_cfg.virtual_pipeline_model_parallel_size)),
                                   ("FSDP2", bool(train_cfg.use_torch_fsdp2))) if on]
            if bad:
                raise NotImplementedError(f"num_seq_splits > 1 is not built together with: {', '.join(bad)}")
        st = ps.get_state()
        if not st.initialized:
            st = init_parallel_state(model_cfg, train_cfg)
        self.st = st
        if device is None:
            device = f"cuda:{torch.cuda.current_device()}" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        from ..ops import gemm as _gemm

        # fp8 recipe of the linear-layer GEMMs (attention, the LM head and the router stay in bf16)
        if model_cfg.fp8 and model_cfg.fp8_recipe not in _gemm.FP8_RECIPES:
            raise NotImplementedError(f"fp8_recipe {model_cfg.fp8_recipe!r}: choose one of {_gemm.FP8_RECIPES}")
        if model_cfg.fp4 and model_cfg.fp4_recipe not in _gemm.FP4_RECIPES:
            raise NotImplementedError(f"fp4_recipe {model_cfg.fp4_recipe!r}: choose one of {_gemm.FP4_RECIPES}")
        if model_cfg.fp4 and model_cfg.fp8:
            raise ValueError("set either fp8 or fp4, not both")
        recipe = model_cfg.fp4_recipe if model_cfg.fp4 else (model_cfg.fp8_recipe if model_cfg.fp8 else None)
        _gemm.set_fp8_recipe(recipe, model_cfg.fp8_amax_history_len, model_cfg.fp8_amax_compute_algo,
                             model_cfg.fp8_margin)
        self.is_cuda = self.device.type == "cuda"
        model_cfg.seq_length = train_cfg.seq_length
        if model_cfg.num_experts and st.tp > 1 and st.ep > 1 and not train_cfg.use_distributed_optimizer:
            raise NotImplementedError("MoE with tensor and expert parallelism needs use_distributed_optimizer (the "
                                      "gradient norm of replicated expert shards is only assembled for sharded state)")
        if model_cfg.attention_dropout > 0.0:
            raise NotImplementedError("attention_dropout > 0: the attention kernels have no dropout path "
                                      "(hidden_dropout is built)")
        from ..parallel import random as _prandom

        if model_cfg.hidden_dropout > 0.0:
            # named random streams: replicated activations share a stream over the tensor-parallel group, shards do not
            _prandom.model_parallel_manual_seed(train_cfg.seed, self.device, st.tp_rank, st.pp_rank, st.ep_rank)
        else:
            _prandom.get_rng_tracker().reset()
        # ---------------------------------------------------------------- model chunks
        from ..parallel import pipeline_schedules as pps

        algo = train_cfg.pipeline_schedule.lower().replace("_", "-")
        v_family = algo in ("zbv", "zbv-formatted", "zbv-greedy", "v-half", "v-min")
        vpp = model_cfg.virtual_pipeline_model_parallel_size if st.pp > 1 else None
        self.pp_chunks = 1 if st.pp == 1 else (2 if v_family else (vpp or 1))
        self.pp_placement = "v" if (v_family and st.pp > 1) else "interleaved"
        n_stages = st.pp * self.pp_chunks
        self.loss_pp_rank = pps.rank_of_stage(n_stages - 1, st.pp, self.pp_placement)[0] if st.pp > 1 else 0
        self.model_chunks = []
        from ..parallel.pipeline_layout import uneven_split

        manual_split = train_cfg.decoder_pipeline_manual_split_list or uneven_split(
            model_cfg.num_layers, n_stages, train_cfg.decoder_first_pipeline_num_layers,
            train_cfg.decoder_last_pipeline_num_layers, train_cfg.account_for_embedding_in_pipeline_split,
            train_cfg.account_for_loss_in_pipeline_split)
        for c in range(self.pp_chunks):
            sid = pps.stage_of(st.pp_rank, c, st.pp, self.pp_placement) if st.pp > 1 else 0
            m = build_model(model_cfg, self.device, sid, n_stages, seed=train_cfg.seed,
                            layout=getattr(train_cfg, "pipeline_model_parallel_layout", None),
                            manual_split=manual_split)
            self.model_chunks.append(m)
        self.model = self.model_chunks[0]
        self._init_embedding_replica()
        # ---------------------------------------------------------------- buffers + optimizer
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.is_cuda else None
        self.fsdp = bool(train_cfg.use_torch_fsdp2) and st.world_size > 1
        if self.fsdp:
            self._init_fsdp2()
        else:
            self._init_buffers_and_optimizer()
        self._init_schedule_and_data()

    def _init_fsdp2(self):
        from . import fsdp

        model_cfg, train_cfg, st = self.mcfg, self.tcfg, self.st
        assert st.tp == st.pp == st.cp == st.ep == 1, "use_torch_fsdp2: data parallelism only (tp = pp = cp = ep = 1)"
        assert not (model_cfg.fp8 and model_cfg.fp8_recipe), "use_torch_fsdp2 runs in bf16 (no MXFP8 recipe)"
        assert train_cfg.optimizer.lower() in ("adam", "adamw"), "use_torch_fsdp2 uses AdamW"
        fsdp.shard_model(self.model, self.device, model_cfg.torch_dtype, int(train_cfg.data_parallel_replicate_degree or 1))
        self.buffers = []
        self.optimizer = fsdp.FSDP2Optimizer(self.model, train_cfg.lr, (train_cfg.adam_beta1, train_cfg.adam_beta2),
                                             train_cfg.adam_eps, train_cfg.weight_decay, train_cfg.clip_grad,
                                             train_cfg.check_for_nan_in_loss_and_grad)

    # ------------------------------------------------------------------ word embeddings shared by first and last stage
    def _init_embedding_replica(self):
        """A tied output head or multi-token prediction under pipeline parallelism: the last stage holds a replica of the
        first stage's word embeddings (``models/gpt.py``).  The replica gets a gradient buffer of its own and the first
        stage's initial values."""
        params = [p for m in self.model_chunks for p in m.parameters()]
        self._emb_primary = [p for p in params if getattr(p, "embedding_primary", False)]
        self._emb_replica = [p for p in params if getattr(p, "embedding_replica", False)]
        if not (self._emb_primary or self._emb_replica):
            return
        if self._emb_primary and self._emb_replica:
            raise NotImplementedError("first and last pipeline stage on the same rank (V-shaped placement) with a tied "
                                      "output head or multi-token prediction is not built")
        assert self.st.embedding_group is not None, "the embedding group exists for pipeline_model_parallel_size > 1"
        for p in self._emb_replica:
            p.main_grad = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
        self._sync_embedding_replica()

    def _sync_embedding_replica(self):
        """First stage -> last stage: current word-embedding weights."""
        for p in self._emb_primary + self._emb_replica:
            dist.broadcast(p.data, src=self.st.pp_ranks[0], group=self.st.embedding_group)

    def _reduce_embedding_replica_grads(self):
        """Last stage -> first stage: the replica's gradient joins the primary's before the data-parallel reduction."""
        for p in self._emb_primary + self._emb_replica:
            dist.all_reduce(p.main_grad, group=self.st.embedding_group)
        for p in self._emb_replica:
            p.main_grad.zero_()

    def _init_buffers_and_optimizer(self):
        model_cfg, train_cfg, st = self.mcfg, self.tcfg, self.st
        dense, expert = [], []
        for m in self.model_chunks:
            for p in m.parameters():
                if getattr(p, "embedding_replica", False):
                    continue        # follows the first stage's copy; not an optimizer parameter
                (expert if getattr(p, "is_expert", False) else dense).append(p)
        if self._emb_primary and train_cfg.overlap_grad_reduce:
            # the replica's gradient must be added before the bucket of the embedding is reduced
            train_cfg.overlap_grad_reduce = False
            self.log("overlap_grad_reduce is off on this run: the word embeddings are shared between the first and the "
                     "last pipeline stage")
        self.buffers = []
        if dense:
            self.buffers.append(ParamGradBuffer(
                dense, st.dp_cp_group if st.cp > 1 else st.dp_group, st.dp * st.cp, st.dp_rank * st.cp + st.cp_rank,
                train_cfg.ddp_bucket_size, torch.float32, train_cfg.use_distributed_optimizer,
                train_cfg.overlap_grad_reduce, True, self.comm_stream,
                symmetric=(train_cfg.fused_dp_optimizer or train_cfg.enable_odc) and train_cfg.use_distributed_optimizer,
                grad_reduce_in_bf16=train_cfg.grad_reduce_in_bf16 and not train_cfg.enable_odc,
                odc=train_cfg.enable_odc))
        if expert:
            self.buffers.append(ParamGradBuffer(
                expert, st.edp_group, st.edp, st.edp_rank, train_cfg.ddp_bucket_size, torch.float32,
                train_cfg.use_distributed_optimizer, train_cfg.overlap_grad_reduce, True, self.comm_stream,
                extra_grad_scale=float(st.edp) / float(st.dp * st.cp),
                grad_reduce_in_bf16=train_cfg.grad_reduce_in_bf16))
        if train_cfg.param_gather_copy_engine or os.environ.get("ENABLE_SDMA_ALLGATHER", "0") == "1":
            for buf in self.buffers:
                buf.copy_engine_gather = buf.symmetric and buf.odc is None
            if not any(buf.copy_engine_gather for buf in self.buffers):
                self.log("param_gather_copy_engine needs fused_dp_optimizer with more than one data-parallel rank on "
                         "GPUs: the parameter all-gather stays on its default path")
        norm_groups = [st.mp_group] if (st.tp > 1 or st.pp > 1) else []
        from ..parallel import matrix_optimizers

        extra = {}
        if train_cfg.optimizer.lower() in ("adam", "adamw") and train_cfg.use_precision_aware_optimizer:
            dts = {train_cfg.exp_avg_dtype, train_cfg.exp_avg_sq_dtype}
            assert len(dts) == 1 and dts <= {"fp32", "bf16"}, "exp_avg_dtype and exp_avg_sq_dtype: both fp32 or both bf16"
            assert train_cfg.main_params_dtype == "fp32" and train_cfg.main_grads_dtype == "fp32", \
                "the master weights and the main gradients stay fp32"
            if dts == {"bf16"}:
                assert not train_cfg.fused_dp_optimizer, "the fused data-parallel optimizer keeps fp32 moments"
                extra = dict(state_dtype=torch.bfloat16)
        if train_cfg.optimizer.lower() == "sgd":
            extra = dict(sgd_momentum=train_cfg.sgd_momentum)
        elif train_cfg.optimizer.lower() == "muon":
            extra = dict(muon_momentum=train_cfg.muon_momentum, muon_use_nesterov=train_cfg.muon_use_nesterov,
                         muon_num_ns_steps=train_cfg.muon_num_ns_steps)
        # learning-rate groups: 1 = embeddings and output layer under ``decoupled_lr``, 2 = the output layer under
        # ``head_lr_mult`` (Megatron's switches of the same names); the optimizer reads the ``lr_group`` attribute
        self._lr_groups = set()
        if train_cfg.decoupled_lr is not None or train_cfg.head_lr_mult != 1.0:
            for m in self.model_chunks:
                for name, p in m.named_parameters():
                    head = name.startswith("output_layer.")
                    emb = name.startswith("embedding.")
                    if head and train_cfg.head_lr_mult != 1.0:
                        p.lr_group = 2
                    elif (head or emb) and train_cfg.decoupled_lr is not None:
                        p.lr_group = 1
                    if getattr(p, "lr_group", 0):
                        self._lr_groups.add(p.lr_group)
            if train_cfg.decoupled_lr is not None:
                self._lr_groups.add(1)
        self.optimizer = matrix_optimizers.build(
            train_cfg.optimizer, self.buffers, **extra, lr=train_cfg.lr, betas=(train_cfg.adam_beta1, train_cfg.adam_beta2), eps=train_cfg.adam_eps,
            weight_decay=train_cfg.weight_decay, clip_grad=train_cfg.clip_grad, norm_groups=norm_groups,
            check_for_nan=train_cfg.check_for_nan_in_loss_and_grad, tp_size=st.tp,
            expert_norm_group=st.ep_group if (st.ep > 1 and not train_cfg.use_distributed_optimizer) else None)
        if train_cfg.enable_optimizer_post_validation:
            self.optimizer.post_validation = True
            self.optimizer.post_validation_exact = bool(train_cfg.enable_exact_optimizer_post_validation)
        if train_cfg.enable_odc:
            self.optimizer.grad_spike_threshold = float(train_cfg.odc_grad_spike_threshold or 0.0)
        if train_cfg.sft_grad_sanitize:
            assert not train_cfg.fused_dp_optimizer, "sft_grad_sanitize works on the NCCL optimizer path"
            self.optimizer.sanitize_grads = True
        if train_cfg.weight_deosc:
            self._install_weight_deosc()
        self._install_param_gather_waits()

    def _install_weight_deosc(self):
        from ..parallel.weight_deosc import WeightDeOsc, WeightDeOscConfig

        tc = self.tcfg
        if not self.mcfg.fp4:
            self.log("[weight de-osc] weight_deosc is set but fp4 is not: nothing is quantised to 4 bits, not installed")
            return
        if not hasattr(self.optimizer, "state") or not hasattr(self.optimizer, "deosc"):
            self.log(f"[weight de-osc] the {tc.optimizer} optimizer keeps no flat fp32 master shards: not installed")
            return
        cfg = WeightDeOscConfig(True, int(tc.weight_deosc_period), float(tc.weight_deosc_ratio),
                                int(tc.weight_deosc_start_step), int(tc.weight_deosc_log_freq))
        self.optimizer.deosc = WeightDeOsc(cfg, log=self.log)
        self.log(f"[weight de-osc] on: period {cfg.period}, ratio {cfg.ratio_threshold}, from step {cfg.start_step}")

    # ------------------------------------------------------------------ overlap_param_gather
    def _install_param_gather_waits(self):
        """``overlap_param_gather``: after an optimizer step the bucket all-gathers run asynchronously; every transformer
        layer waits, right before its forward, for the buckets that hold its parameters, and the model waits for the
        embedding buckets at its start and for the final norm / output layer buckets before the head."""
        tc = self.tcfg
        active = tc.overlap_param_gather and tc.use_distributed_optimizer and not self._emb_primary and \
            not self._emb_replica and any(b.dp_size > 1 and (not b.symmetric or b.copy_engine_gather) for b in self.buffers)
        self.optimizer.overlap_param_gather = bool(active)
        if tc.overlap_param_gather and not active and any(b.dp_size > 1 for b in self.buffers):
            self.log("overlap_param_gather is off on this run (it needs the distributed optimizer on the NCCL or the "
                     "copy-engine path and word embeddings that are not shared between pipeline stages)")
        if not active:
            return

        def waiter(params):
            todo = [(buf, b) for buf in self.buffers for b in buf.buckets_of(params)]

            def wait(*_a):
                for buf, b in todo:
                    buf.wait_bucket_params(b)
            return wait

        for m in self.model_chunks:
            layer_params = set()
            for layer in m.decoder.layers.values():
                ps_ = list(layer.parameters())
                layer_params.update(ps_)
                layer.register_forward_pre_hook(waiter(ps_))
            head = [p for n, p in m.named_parameters() if p not in layer_params and not n.startswith("embedding.")]
            emb = [p for n, p in m.named_parameters() if n.startswith("embedding.")]
            m._param_waiters = {"embedding": waiter(emb), "head": waiter(head + emb)}

    def finish_param_sync(self):
        for buf in self.buffers:
            buf.finish_param_sync()

    def _init_schedule_and_data(self):
        model_cfg, train_cfg, st = self.mcfg, self.tcfg, self.st
        decay_iters = train_cfg.lr_decay_iters or train_cfg.train_iters
        warmup = train_cfg.lr_warmup_iters
        if train_cfg.lr_warmup_fraction is not None:
            assert not warmup, "give lr_warmup_iters or lr_warmup_fraction, not both"
            warmup = int(train_cfg.lr_warmup_fraction * decay_iters)
        start_wd = train_cfg.weight_decay if train_cfg.start_weight_decay is None else train_cfg.start_weight_decay
        end_wd = train_cfg.weight_decay if train_cfg.end_weight_decay is None else train_cfg.end_weight_decay
        if train_cfg.weight_decay_incr_style == "constant":
            assert start_wd == end_wd, "a constant weight decay with different start and end values"
        self.scheduler = schedules.LRScheduler(
            max_lr=train_cfg.lr, min_lr=train_cfg.min_lr, warmup_iters=warmup, warmup_init=train_cfg.lr_warmup_init,
            decay_iters=decay_iters, decay_style=train_cfg.lr_decay_style,
            wsd_decay_iters=int(train_cfg.lr_wsd_decay_iters or 0), wsd_decay_style=train_cfg.lr_wsd_decay_style,
            start_wd=start_wd, end_wd=end_wd, wd_incr_style=train_cfg.weight_decay_incr_style)
        self._decoupled_scheduler = None
        if train_cfg.decoupled_lr is not None:      # the same shape, between the decoupled maximum and minimum
            import dataclasses as _dc

            self._decoupled_scheduler = _dc.replace(
                self.scheduler, max_lr=train_cfg.decoupled_lr,
                min_lr=train_cfg.min_lr if train_cfg.decoupled_min_lr is None else train_cfg.decoupled_min_lr)
        # ---------------------------------------------------------------- data
        self.num_microbatches = schedules.num_microbatches(train_cfg.global_batch_size, train_cfg.micro_batch_size, st.dp)
        if train_cfg.mock_data or not train_cfg.data_path:
            if train_cfg.mock_data_kind == "markov":
                from .data import MarkovGPTDataset

                ds = MarkovGPTDataset(model_cfg.vocab_size, train_cfg.seq_length, train_cfg.data_seed)
            elif train_cfg.mock_data_period:
                from .data import PatternGPTDataset

                ds = PatternGPTDataset(model_cfg.vocab_size, train_cfg.seq_length, train_cfg.data_seed,
                                       train_cfg.mock_data_period)
            else:
                ds = MockGPTDataset(model_cfg.vocab_size, train_cfg.seq_length, train_cfg.data_seed)
        else:
            ds = _open_corpus(train_cfg.data_path, train_cfg.seq_length, train_cfg.data_seed, train_cfg)
            if train_cfg.split and not train_cfg.valid_data_path:
                ds = split_view(ds, train_cfg.split, 0)            # the training share of the samples
        self.sampler = MicroBatchSampler(train_cfg.global_batch_size, train_cfg.micro_batch_size, st.dp, st.dp_rank,
                                         rampup=train_cfg.rampup_batch_size)
        self.stager = BatchStager(ds, self.sampler, self.device, num_workers=train_cfg.num_workers)
        if train_cfg.reset_position_ids:
            self.use_position_ids = True
        self.iteration = 0
        self.meter = ThroughputMeter(train_cfg.log_avg_skip_iterations, train_cfg.log_avg_reset_interval)
        self.flops_per_token = schedules.model_flops_per_token(model_cfg, train_cfg.seq_length)
        self.loss_accum = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.last_metrics: dict = {}
        self._gc_disabled = False
        from .timers import Timers

        self.timers = Timers(train_cfg.timing_log_level, train_cfg.timing_log_option, self.is_cuda)

    # ------------------------------------------------------------------ one micro-batch
    def _loss_weights(self, batch: dict) -> torch.Tensor:
        mask = batch["loss_mask"]
        if "_lb_mini_norm" in batch:     # variable micro-batch counts: normalise by the whole mini-batch's token count
            return mask * batch["_lb_mini_norm"]
        if self.tcfg.calculate_per_token_loss:
            return mask / float(self.num_microbatches)  # normalised later by the global token count
        if "_mask_total" in batch:
            # context parallel: normalise by the whole sequence's token count; gradients are later averaged over
            # dp x cp, so every rank's share is scaled back by cp
            return mask * (float(self.st.cp) / batch["_mask_total"].clamp(min=1.0) / float(self.num_microbatches))
        denom = mask.sum().clamp(min=1.0)
        return mask / denom / float(self.num_microbatches)

    def _cp_shard(self, mb: dict) -> dict:
        """The slice of a micro-batch this context-parallel rank works on, with global position ids.  All-to-all
        scheme: ``seq / cp`` consecutive tokens of every sequence (attention itself runs on whole sequences, so no
        balancing is needed).  All-gather scheme: the zig-zag chunks ``rank`` and ``2 cp - 1 - rank`` of ``2 cp``, so
        that every rank has the same amount of causal attention work."""
        st = self.st
        if st.cp == 1:
            return mb
        b, S = mb["tokens"].shape
        dev = mb["tokens"].device
        if getattr(self.mcfg, "cp_comm_type", "a2a") == "a2a+p2p":
            # zig-zag over the ring (2 x p2p super-chunks), consecutive parts inside an all-to-all group
            a, P = st.cp_a2a, st.cp_p2p
            assert a * P == st.cp, "a2a+p2p context parallelism needs hierarchical_context_parallel_sizes"
            assert S % (2 * st.cp) == 0, "sequence length must divide by 2 x the context-parallel size"
            C, part = S // (2 * P), S // (2 * st.cp)
            if self.is_cuda:
                assert C % 128 == 0, "ring context parallelism needs seq / (2 p2p) to be a multiple of 128"
            i, j = divmod(st.cp_rank, a)
            pos = torch.cat([torch.arange(sc * C + j * part, sc * C + (j + 1) * part, device=dev)
                             for sc in (i, 2 * P - 1 - i)])
            out = {k: v.index_select(1, pos).contiguous() for k, v in mb.items()
                   if torch.is_tensor(v) and v.dim() == 2 and v.shape[1] == S}
            if "position_ids" not in mb:
                out["position_ids"] = pos.repeat(b, 1)
        elif getattr(self.mcfg, "cp_comm_type", "a2a") in ("allgather", "p2p"):
            assert S % (2 * st.cp) == 0, "sequence length must divide by 2 x the context-parallel size"
            c = S // (2 * st.cp)
            if self.is_cuda:
                assert c % 128 == 0, "all-gather context parallelism needs seq / (2 cp) to be a multiple of 128"
            pos = torch.cat([torch.arange(j * c, (j + 1) * c, device=dev) for j in (st.cp_rank, 2 * st.cp - 1 - st.cp_rank)])
            out = {k: v.index_select(1, pos).contiguous() for k, v in mb.items()
                   if torch.is_tensor(v) and v.dim() == 2 and v.shape[1] == S}
            if "position_ids" not in mb:
                out["position_ids"] = pos.repeat(b, 1)
        else:
            assert S % st.cp == 0, "sequence length must divide by the context-parallel size"
            Sl = S // st.cp
            lo = st.cp_rank * Sl
            out = {k: v[:, lo:lo + Sl].contiguous() for k, v in mb.items()
                   if torch.is_tensor(v) and v.dim() == 2 and v.shape[1] == S}
            if "position_ids" not in out:
                out["position_ids"] = torch.arange(lo, lo + Sl, device=dev).repeat(b, 1)
        out["_mask_total"] = mb["loss_mask"].sum()
        return out

    def _seq_chunk(self, mb: dict, split: int) -> dict:
        """Chunk ``split`` of ``num_seq_splits`` of a micro-batch along the sequence, with global position ids and the
        whole micro-batch's loss-mask total (the loss normalisation must not depend on the chunking)."""
        S = self.num_seq_splits
        b, L = mb["tokens"].shape
        c = L // S
        sl = slice(split * c, (split + 1) * c)
        out = {k: mb[k][:, sl].contiguous() for k in ("tokens", "labels", "loss_mask")}
        pos = mb.get("position_ids")
        out["position_ids"] = pos[:, sl].contiguous() if pos is not None else \
            torch.arange(split * c, (split + 1) * c, device=mb["tokens"].device).expand(b, c).contiguous()
        for k in ("_lb_mini_norm", "_mask_total"):
            if k in mb:
                out[k] = mb[k]
        if "_mask_total" not in out and "_lb_mini_norm" not in out:
            out["_mask_total"] = mb["loss_mask"].sum()
        return out

    def _forward_backward_seq_splits(self, micro_batches: list[dict]) -> torch.Tensor:
        """No pipeline, ``num_seq_splits`` > 1: every micro-batch is forwarded chunk by chunk and its chunks' backward
        passes run in reverse order (the activation footprint of the loss head and the MLPs is that of one chunk)."""
        from ..ops import layers as _layers

        model, S = self.model, self.num_seq_splits
        total = self.loss_accum
        total.zero_()
        n = len(micro_batches)
        try:
            for i, mb in enumerate(micro_batches):
                for buf in self.buffers:
                    buf.is_last_microbatch = False
                losses = []
                for q in range(S):
                    ch = self._seq_chunk(mb, q)
                    _layers.SEQ_SPLIT.begin((i, 0), q, S)
                    losses.append(model(ch["tokens"], ch["labels"], loss_weights=self._loss_weights(ch), unit_upstream=True,
                                        position_ids=ch["position_ids"]))
                for q in reversed(range(S)):
                    for buf in self.buffers:       # the bucket reductions start with the very last backward pass only
                        buf.is_last_microbatch = (i == n - 1 and q == 0)
                    _layers.SEQ_SPLIT.begin((i, 0), q, S)
                    losses[q].backward()
                    total += losses[q].detach()
                _layers.SEQ_SPLIT.drop((i, 0))
        finally:
            _layers.SEQ_SPLIT.clear()
            for buf in self.buffers:
                buf.is_last_microbatch = True
        return total

    def forward_backward_no_pipelining(self, micro_batches: list[dict]) -> torch.Tensor:
        if self.num_seq_splits > 1:
            return self._forward_backward_seq_splits(micro_batches)
        model = self.model
        total = self.loss_accum
        total.zero_()
        n = len(micro_batches)
        for i, mb in enumerate(micro_batches):
            last = i == n - 1
            for buf in self.buffers:
                buf.is_last_microbatch = last
            if self.fsdp:      # gradients are reduce-scattered once, with the last micro-batch
                model.set_requires_gradient_sync(last)
            w = self._loss_weights(mb)
            loss = model(mb["tokens"], mb["labels"], loss_weights=w, unit_upstream=True,
                         position_ids=mb.get("position_ids") if (getattr(self, "use_position_ids", False)
                                                                 or self.st.cp > 1) else None,
                         cu_seqlens=mb.get("host_cu_seqlens"))
            loss.backward()
            total += loss.detach()
        return total

    # ------------------------------------------------------------------ grads
    def finalize_grads(self):
        st = self.st
        for m in self.model_chunks:
            for p in m.parameters():
                if p.grad is not None:  # gradients that came through plain autograd
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                    p.grad = None
        if self._emb_primary or self._emb_replica:
            self._reduce_embedding_replica_grads()
        for buf in self.buffers:
            buf.finish_grad_sync()
        # sequence-parallel: norm weights saw only this rank's token shard
        if st.tp > 1 and self.mcfg.sequence_parallel:
            grads = [p.main_grad for m in self.model_chunks for p in m.parameters()
                     if getattr(p, "sequence_parallel", False)]
            if grads and not self.tcfg.use_distributed_optimizer:
                flat = torch.cat([g.reshape(-1) for g in grads])
                dist.all_reduce(flat, group=st.tp_group)
                o = 0
                for g in grads:
                    g.copy_(flat[o:o + g.numel()].view_as(g))
                    o += g.numel()

    def _pre_sync_sp_norm_grads(self):
        """With the distributed optimizer the norm-weight all-reduce over TP must precede the DP
        reduce-scatter (afterwards each rank only holds a shard)."""
        st = self.st
        if st.tp > 1 and self.mcfg.sequence_parallel and self.tcfg.use_distributed_optimizer:
            grads = [p.main_grad for m in self.model_chunks for p in m.parameters()
                     if getattr(p, "sequence_parallel", False)]
            if grads:
                flat = torch.cat([g.reshape(-1) for g in grads])
                dist.all_reduce(flat, group=st.tp_group)
                o = 0
                for g in grads:
                    g.copy_(flat[o:o + g.numel()].view_as(g))
                    o += g.numel()

    # ------------------------------------------------------------------ step
    def train_step(self) -> torch.Tensor:
        """One optimizer step. Returns the (device) mean loss of this rank's micro-batches."""
        timers = self.timers
        with timers("batch-generator", 2):
            micro_batches = self.stager.next_step()
            if self.tcfg.rampup_batch_size:     # the global batch is still growing: this step's number of micro-batches
                self.num_microbatches = len(micro_batches)
                self.current_global_batch = len(micro_batches) * self.tcfg.micro_batch_size * self.st.dp
            if self.tcfg.iterations_to_skip and (self.iteration + 1) in self.tcfg.iterations_to_skip:
                # a batch known to be bad: it is consumed (the data order of the other steps stays what it was) and
                # nothing is trained on it
                self.log(f"[skip] iteration {self.iteration + 1} is listed in iterations_to_skip: batch dropped")
                self.stager.prefetch()
                self.scheduler.step()
                self.iteration += 1
                return self.loss_accum.zero_().clone().reshape(())
            if self.st.cp > 1:
                micro_batches = [self._cp_shard(mb) for mb in micro_batches]
        if self.st.pp > 1 and self.tcfg.pp_warmup and not getattr(self, "_pp_warmed", False):
            from ..parallel.pipeline import pipeline_warmup

            pipeline_warmup(self, micro_batches[0])
            self._pp_warmed = True
        for buf in self.buffers:
            buf.zero_grad()
        if self.fsdp:
            self.optimizer.zero_grad()
        if self.mcfg.num_experts:
            # the load-balancing loss of every micro-batch is weighted like the language-model loss
            from ..models.moe import AuxLossScaler

            AuxLossScaler.scale = 1.0 / float(self.num_microbatches)
        timers("forward-backward", 1).start()
        if self.st.pp > 1:
            from ..parallel.pipeline import run_pipeline_schedule

            timeline = None
            it = self.iteration + 1
            t0_, t1_ = self.tcfg.zero_bubble_pipeline_timers_start_iter, self.tcfg.zero_bubble_pipeline_timers_end_iter
            measuring = t1_ > t0_ and t0_ <= it < t1_
            if (self.tcfg.dump_pp_data and self.st.dp_rank == 0 and self.st.tp_rank == 0) or measuring:
                from ..parallel.pipeline import PipelineTimeline

                timeline = PipelineTimeline()
            loss = run_pipeline_schedule(self, micro_batches, timeline)
            if measuring:
                self._pp_measured = getattr(self, "_pp_measured", []) + timeline.events
                if it == t1_ - 1:
                    from ..parallel.pipeline import replan_from_measurements

                    self.pp_replan_report = replan_from_measurements(self, self._pp_measured, len(micro_batches),
                                                                     self.log if (not dist.is_initialized() or dist.get_rank() == 0) else None)
                    self._pp_measured = []
            if timeline is not None and self.tcfg.dump_pp_data and self.st.dp_rank == 0 and self.st.tp_rank == 0:
                d = self.tcfg.pp_dump_dir or os.path.join(self.tcfg.save or ".", "pp_data")
                timeline.dump(os.path.join(d, f"pp_rank{self.st.pp_rank}_iter{self.iteration + 1}.json"), self.st.pp_rank,
                              self.iteration + 1, {"schedule": self.tcfg.pipeline_schedule, "pp": self.st.pp})
        else:
            loss = self.forward_backward_no_pipelining(micro_batches)
        timers("forward-backward", 1).stop()
        self.stager.prefetch()  # stage the next step's batch while the optimizer runs
        if not self.fsdp:
            with timers("all-grads-sync", 1):
                self._pre_sync_sp_norm_grads()
                self.finalize_grads()
        timers("optimizer", 1).start()
        lr = self.scheduler.get_lr(self.iteration + 1)
        if getattr(self, "lora", None) is not None:  # adapter-only training: base weights stay frozen
            self.optimizer.compute_grad_norm()
            self.lora.optimizer_step(lr)
        else:
            group_lr = None
            if getattr(self, "_lr_groups", None):
                group_lr = {1: self._decoupled_scheduler.get_lr(self.iteration + 1)} if 1 in self._lr_groups else {}
                if 2 in self._lr_groups:
                    group_lr[2] = (group_lr.get(1, lr) if self.tcfg.decoupled_lr is not None else lr) * self.tcfg.head_lr_mult
            if group_lr and not self.fsdp:
                self.optimizer.step(lr=lr, weight_decay=self.scheduler.get_wd(self.iteration + 1), group_lr=group_lr)
            else:
                self.optimizer.step(lr=lr, weight_decay=self.scheduler.get_wd(self.iteration + 1))
        _gemm_ops.roll_fp8_scales()      # delayed scaling: this step's maxima become history (no-op for other recipes)
        if self._emb_primary or self._emb_replica:
            for buf in self.buffers:
                buf.finish_param_sync()        # the updated embedding must be complete before it is re-sent
            self._sync_embedding_replica()
        timers("optimizer", 1).stop()
        if self.mcfg.moe_router_enable_expert_bias:
            st = self.st
            groups = [st.dp_cp_group if st.cp > 1 else st.dp_group]
            if self.mcfg.sequence_parallel and st.tp > 1:
                groups.append(st.tp_group)
            for chunk in self.model_chunks:
                for mod in chunk.modules():
                    if hasattr(mod, "update_expert_bias"):
                        mod.update_expert_bias(groups)
        self.scheduler.step()
        self.iteration += 1
        self._steps_since_timer_log = getattr(self, "_steps_since_timer_log", 0) + 1
        return loss

    def reduced_loss(self, loss: torch.Tensor) -> float:
        """Average over data-parallel ranks and fetch to the host (synchronises)."""
        l = loss.detach().clone()
        if self.st.cp > 1:  # every context-parallel rank holds its slice's share (already scaled by cp)
            dist.all_reduce(l, group=self.st.dp_cp_group)
            l /= self.st.dp * self.st.cp
        elif self.st.dp > 1:
            dist.all_reduce(l, group=self.st.dp_group)
            l /= self.st.dp
        if self.st.pp > 1:
            dist.broadcast(l, src=self.st.pp_ranks[self.loss_pp_rank], group=self.st.pp_group)
        return float(l.item())

    # ------------------------------------------------------------------ loop
    def train(self, num_iters: Optional[int] = None, on_step: Optional[Callable] = None) -> list[float]:
        """Runs the step loop.  With ``inprocess_restart`` a failure that every rank sees at the same step (non-finite
        reduced loss, a persistent fault reported by the rerun state machine) does not end the process: the trainer
        reloads the newest checkpoint under ``save`` and continues, up to ``inprocess_max_restarts`` times (the role
        of the reference's in-process restart wrapper, primus/backends/megatron/megatron_pretrain_trainer.py:195-204).
        Failures that only one rank can see are re-raised: they need the job-level restart."""
        tc = self.tcfg
        if tc.skip_train:
            if tc.eval_iters:
                self.evaluate(tc.eval_iters)
            return []
        if not tc.inprocess_restart:
            return self._train_loop(num_iters, on_step)
        from . import checkpoint, fault

        target = self.iteration + (num_iters if num_iters is not None else tc.train_iters - self.iteration)
        losses: list[float] = []
        restarts = 0
        while True:
            try:
                self._train_loop(target - self.iteration, on_step, losses)
                return losses
            except (FloatingPointError, fault.PersistentFault) as e:
                while losses and not math.isfinite(losses[-1]):
                    losses.pop()             # the value that tripped the guard
                latest = checkpoint.latest_iteration(tc.save) if tc.save else None
                if restarts >= tc.inprocess_max_restarts or latest is None:
                    raise
                restarts += 1
                self.log(f"[inprocess_restart] {type(e).__name__}: {e}; restart {restarts}/{tc.inprocess_max_restarts} "
                         f"from iteration {latest}")
                self.load_checkpoint(tc.save)
                self.restarts = restarts

    def _trace_reports(self, profiler, writer, out_dir) -> None:
        """After the profiled window: kernel-level reports of this rank's traces (``generate_tracelens_report``, or
        implied by ``mlflow_upload_tracelens_report``) and artifact hand-over (``mlflow_upload_traces``)."""
        tc = self.tcfg
        want_report = tc.generate_tracelens_report or tc.mlflow_upload_tracelens_report
        if not (profiler.enabled and (want_report or tc.mlflow_upload_traces)):
            return
        try:
            from ..tools import trace_report as TR

            mine = [p for p in TR.find_traces(profiler.out_dir) if TR.rank_of(p) == self.st.rank]
            files = []
            if want_report and mine and (tc.mlflow_tracelens_ranks is None or self.st.rank in tc.mlflow_tracelens_ranks):
                fmt = tc.mlflow_tracelens_output_format if tc.mlflow_tracelens_output_format in ("md", "csv", "tsv", "jsonl") \
                    else "md"
                files = TR.write_report(mine, os.path.join(profiler.out_dir, "trace_report"), fmt)
                self.log(f"[profiler] trace report: {files[0] if files else 'no GPU events in the trace'}")
            upload = (files if tc.mlflow_upload_tracelens_report else []) + (mine if tc.mlflow_upload_traces else [])
            if upload:
                writer.log_artifacts(upload, out_dir, log=self.log)
        except Exception as e:  # noqa: BLE001  (a report must never take the training run down)
            self.log(f"[profiler] trace report failed: {type(e).__name__}: {e}")

    def _train_loop(self, num_iters: Optional[int] = None, on_step: Optional[Callable] = None,
                    losses: Optional[list] = None) -> list[float]:
        tc = self.tcfg
        n = num_iters if num_iters is not None else tc.train_iters - self.iteration
        losses = [] if losses is None else losses
        if tc.manual_gc and not self._gc_disabled:
            gc.disable()  # the reference disables Python GC around trainer.train()
            self._gc_disabled = True
        from . import fault

        start_wall = time.time()
        guard = fault.LossGuard(tc.check_for_nan_in_loss_and_grad, tc.check_for_spiky_loss, 10.0, tc.check_for_large_grads)
        exit_flag = fault.GracefulExit() if tc.exit_signal_handler else None
        straggler = fault.StragglerDetector() if tc.log_straggler else None
        from . import observability as obs

        st = self.st
        out_dir = tc.tensorboard_dir or (os.path.join(tc.save, "tensorboard") if tc.save else None)
        profiler = obs.StepProfiler(tc.profile, st.rank, tc.profile_step_start, tc.profile_step_end, tc.profile_ranks,
                                    os.path.join(out_dir, "profiler") if out_dir else None, tc.exp_name,
                                    not tc.disable_profiler_activity_cpu, record_shapes=tc.torch_profiler_record_shapes,
                                    with_stack=tc.torch_profiler_with_stack, use_gzip=tc.torch_profiler_use_gzip,
                                    record_memory_history=tc.record_memory_history,
                                    memory_snapshot_path=tc.memory_snapshot_path, log=self.log)
        writer = obs.MetricsWriter(st.rank, st.rank == st.world_size - 1 or st.world_size == 1, out_dir,
                                   not tc.disable_tensorboard, tc.wandb_project, tc.mlflow_experiment_name,
                                   tc.mlflow_run_name or tc.exp_name, log=self.log,
                                   wandb_options=dict(name=tc.wandb_exp_name, entity=tc.wandb_entity, dir=tc.wandb_save_dir))
        ml = self._mlperf_logger()
        last_ml_step = self.iteration
        try:
            for _ in range(n):
                t0 = time.perf_counter()
                if ml is not None:
                    ml.run_start()
                with obs.nvtx_range(f"iteration {self.iteration + 1}", tc.nvtx_ranges):
                    loss = self.train_step()
                profiler.step()
                if self.iteration % tc.log_interval == 0 or on_step is not None:
                    lv = self.reduced_loss(loss)  # synchronises
                    self._check_device_status()
                    dt = time.perf_counter() - t0
                    losses.append(lv)
                    self._log_step(lv, dt)
                    writer.write(self.iteration, self.last_metrics)
                    problem = guard.check(lv, float(self.optimizer.grad_norm.item()))
                    if problem and not math.isfinite(lv):
                        raise FloatingPointError(f"iteration {self.iteration}: {problem}")
                    if problem:
                        self.log(f"[guard] iteration {self.iteration}: {problem}")
                    if straggler is not None:
                        straggler.record(dt)
                        if self.iteration % max(tc.log_interval * 10, 10) == 0:
                            rep = straggler.report()
                            if rep.get("stragglers"):
                                self.log(f"[straggler] slow ranks {rep['stragglers']} (median {rep['median_s']:.3f} s)")
                    if on_step is not None:
                        on_step(self, lv)
                    if ml is not None:
                        ml.on_step(self.iteration, lv, self.last_metrics.get("lr", tc.lr), self.iteration - last_ml_step)
                        last_ml_step = self.iteration
                if tc.manual_gc and tc.manual_gc_interval and self.iteration % tc.manual_gc_interval == 0:
                    gc.collect()
                n_hash = tc.check_weight_hash_across_dp_replicas_interval
                if n_hash and self.iteration % n_hash == 0:
                    self.check_replicas_agree()
                if tc.eval_interval and tc.eval_iters and self.iteration % tc.eval_interval == 0:
                    if ml is not None:
                        ml.clock.step(self.iteration - last_ml_step)
                        last_ml_step = self.iteration
                        ml.eval_begin(self.iteration)
                    val = self.evaluate(tc.eval_iters)
                    if ml is not None and ml.eval_end(self.iteration, val):      # every rank sees the same reduced loss
                        self.log(f"[mlperf] validation loss {val:.4f} reached the target {ml.target} at iteration "
                                 f"{self.iteration}: run complete")
                        break
                if tc.save and tc.save_interval and self.iteration % tc.save_interval == 0:
                    self.save_checkpoint()
                elif tc.non_persistent_save_interval and self.iteration % tc.non_persistent_save_interval == 0:
                    self.save_non_persistent_checkpoint()
                if exit_flag is not None and exit_flag.requested:
                    self.log(f"signal {exit_flag.signum} received: checkpointing at iteration {self.iteration} and leaving")
                    if tc.save:
                        self.save_checkpoint()
                    break
                if tc.exit_interval and self.iteration % tc.exit_interval == 0:
                    break
                if tc.exit_duration_in_mins and (time.time() - start_wall) / 60.0 > tc.exit_duration_in_mins:
                    break
            if any(getattr(buf, "copy_engine_gather", False) for buf in self.buffers):
                # peers pull this rank's parameter shards: do not return (and possibly exit) while they are being read
                self.finish_param_sync()
                torch.cuda.current_stream().synchronize()
        finally:
            from . import checkpoint as _ckpt

            _ckpt.finalize_async_save()
            if ml is not None and (self.iteration >= tc.train_iters or ml.converged):
                ml.run_stop(ml.converged, self.iteration)
                ml.close()
            profiler.close()
            self._trace_reports(profiler, writer, out_dir)
            writer.close()
            if exit_flag is not None:
                exit_flag.restore()
            if self._gc_disabled:
                gc.enable()
                self._gc_disabled = False
        return losses

    @torch.no_grad()
    def check_replicas_agree(self) -> None:
        """``check_weight_hash_across_dp_replicas_interval``: the parameters every data-parallel replica holds must be the
        same bits.  Every rank sums its parameters in fp64 (per buffer); the minimum and the maximum of the sums over the
        data-parallel group must coincide.  Expert parameters are compared over their own, smaller replica group."""
        st = self.st
        for buf in self.buffers:
            group, size = buf.dp_group, buf.dp_size
            if size <= 1:
                continue
            self.finish_param_sync()
            v = buf.param_data.double()
            sig = torch.stack([v.sum(), (v * v).sum()])
            lo, hi = sig.clone(), sig.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
            if not torch.equal(lo, hi):
                raise RuntimeError(f"iteration {self.iteration}: the data-parallel replicas of a parameter buffer differ "
                                   f"(checksums {lo.tolist()} .. {hi.tolist()}, rank {st.rank})")

    def _mlperf_logger(self):
        """The run's MLPerf logger (``mlperf_mode``), created once; only the logging rank writes."""
        tc, st = self.tcfg, self.st
        if not tc.mlperf_mode:
            return None
        if getattr(self, "_mlperf", None) is None:
            from .mlperf_logging import MLPerfLogger

            self._mlperf = MLPerfLogger(tc.mlperf_benchmark, tc.global_batch_size, tc.mlperf_target_eval_loss,
                                        tc.mlperf_submission_org, tc.mlperf_submission_platform,
                                        enabled=st.rank == st.world_size - 1 or st.world_size == 1,
                                        sink=self.log, path=tc.mlperf_log_path)
            self._mlperf.log_init(tc.seed)
            self._mlperf.log_hyperparams(tc, self.num_microbatches, tc.train_iters * tc.global_batch_size,
                                         (tc.eval_iters or 0) * tc.global_batch_size)
        return self._mlperf

    # ------------------------------------------------------------------ evaluation
    def _eval_stager(self):
        """Validation data: a separate stream of the same dataset class (mock data: a different seed; indexed data:
        the ``valid_data_path`` file when given, else the tail of the training file)."""
        if getattr(self, "_eval_stager_obj", None) is None:
            tc, st = self.tcfg, self.st
            if tc.mock_data or not tc.data_path:
                ds = MockGPTDataset(self.mcfg.vocab_size, tc.seq_length, tc.data_seed + 1000003)
            else:
                from .data import IndexedTokenDataset

                if tc.valid_data_path or not tc.split:
                    ds = _open_corpus(tc.valid_data_path or tc.data_path, tc.seq_length, tc.data_seed + 1000003, tc)
                else:       # the validation share of the same sample order as training: disjoint from what is trained on
                    ds = split_view(_open_corpus(tc.data_path, tc.seq_length, tc.data_seed, tc), tc.split, 1)
            sampler = MicroBatchSampler(tc.global_batch_size, tc.micro_batch_size, st.dp, st.dp_rank)
            self._eval_stager_obj = BatchStager(ds, sampler, self.device)
        return self._eval_stager_obj

    @torch.no_grad()
    def evaluate(self, iters: int) -> float:
        """Mean validation loss over ``iters`` global batches (forward only; under pipeline parallelism the forward
        nodes of the training schedule).  Logs the ``validation loss at iteration`` line of the reference's evaluator
        (primus/backends/megatron/training/evaluator.py:23-208)."""
        stager = self._eval_stager()
        total = torch.zeros(1, dtype=torch.float32, device=self.device)
        for m in self.model_chunks:
            m.eval()                      # no dropout in validation
        try:
            total = self._evaluate_batches(stager, iters, total)
        finally:
            for m in self.model_chunks:
                m.train()
        val = self.reduced_loss(total / max(iters, 1))
        self._check_device_status()
        ppl = math.exp(min(val, 20.0))
        self.last_metrics.update(validation_loss=val, validation_ppl=ppl)
        if self.st.rank == self.st.world_size - 1 or self.st.world_size == 1:
            self.log(f" validation loss at iteration {self.iteration} | lm loss value: {val:.6E} | lm loss PPL: {ppl:.6E} |")
        return val

    def _evaluate_batches(self, stager, iters: int, total: torch.Tensor) -> torch.Tensor:
        for _ in range(iters):
            mbs = stager.next_step()
            if self.st.cp > 1:
                mbs = [self._cp_shard(mb) for mb in mbs]
            if self.st.pp > 1:
                from ..parallel.pipeline import run_pipeline_schedule

                total += run_pipeline_schedule(self, mbs, forward_only=True).detach().float()
                continue
            for mb in mbs:
                w = self._loss_weights(mb)
                pos = mb.get("position_ids") if (getattr(self, "use_position_ids", False) or self.st.cp > 1) else None
                total += self.model(mb["tokens"], mb["labels"], loss_weights=w, position_ids=pos,
                                    cu_seqlens=mb.get("host_cu_seqlens")).detach().float()
        return total

    def _log_step(self, loss: float, dt: float):
        tc, st = self.tcfg, self.st
        tokens = tc.seq_length * getattr(self, "current_global_batch", tc.global_batch_size)
        tps_gpu = tokens / dt / max(st.world_size, 1)
        avg = self.meter.update(tps_gpu)
        tflops = tokens * self.flops_per_token / dt / max(st.world_size, 1) / 1e12
        gn = float(self.optimizer.grad_norm.item())
        mem = torch.cuda.max_memory_allocated(self.device) / 2**30 if self.is_cuda else 0.0
        self.last_metrics = dict(iteration=self.iteration, loss=loss, ms=dt * 1e3, tokens_per_s_gpu=tps_gpu,
                                 tokens_per_s_gpu_avg=avg, tflops_gpu=tflops, grad_norm=gn, mem_gib=mem,
                                 lr=self.scheduler.get_lr(self.iteration))
        aux = [m_.last_aux_loss for mc_ in self.model_chunks for m_ in mc_.modules()
               if getattr(m_, "last_aux_loss", None) is not None]
        extra_text = ""
        if tc.log_params_norm:
            sq = torch.zeros((), dtype=torch.float64, device=self.device)
            for m in self.model_chunks:
                for p in m.parameters():
                    sq += p.detach().double().pow(2).sum()
            if dist.is_initialized() and st.world_size > 1:      # every parameter shard once: model-parallel ranks add up
                for g in (st.tp_group, st.pp_group):
                    if g is not None:
                        dist.all_reduce(sq, group=g)
            self.last_metrics["params_norm"] = float(sq.sqrt())
            extra_text += f" params norm: {self.last_metrics['params_norm']:.3f} |"
        if tc.log_num_zeros_in_grad:
            z = sum(int((buf.grad_data == 0).sum()) for buf in self.buffers)
            self.last_metrics["num_zeros_in_grad"] = z
            extra_text += f" num zeros: {z} |"
        moe_text = ""
        if aux:   # per-layer load-balancing losses of the last micro-batch, averaged over this rank's MoE layers
            v = float(torch.stack([a.detach().float().reshape(()) for a in aux]).mean().item())
            self.last_metrics["load_balancing_loss"] = v
            moe_text = f" load balancing loss: {v:.6E} |"
        if st.rank == st.world_size - 1 or st.world_size == 1:
            self.log(
                f" iteration {self.iteration:8d}/{tc.train_iters:8d} | elapsed time per iteration (ms): {dt * 1e3:.1f} | " +
                (f"throughput per GPU (TFLOP/s/GPU): {tflops:.1f} | tokens/s/GPU: {tps_gpu:.1f} (avg {avg:.1f}) | "
                 if tc.log_throughput else "") +
                f"learning rate: {self.last_metrics['lr']:.6E} | global batch size: {getattr(self, 'current_global_batch', tc.global_batch_size):5d} | "
                f"lm loss: {loss:.6E} |{moe_text} grad norm: {gn:.3f} |{extra_text} max mem (GiB): {mem:.2f} |")
        if tc.timing_log_level > 0:
            text = self.timers.log(normalizer=max(getattr(self, "_steps_since_timer_log", 1), 1))
            self._steps_since_timer_log = 0
            if text and (st.rank == st.world_size - 1 or st.world_size == 1):
                self.log(text)
            if tc.log_timers_to_tensorboard:
                self.last_metrics.update({f"timers/{k}": v for k, v in self.timers.last_max_ms.items()})

    def _check_device_status(self):
        """Reads the status word that kernels with bounded waits (mbarrier / flag / barrier) and the fused
        expert-parallel capacity check write to.  Called where the loop synchronises anyway (after the loss has been
        fetched, before a checkpoint is written, after an evaluation).  A recorded error means this step's results
        cannot be trusted, so it is raised as a :class:`fault.PersistentFault`: the in-process restart (or the job-level
        one) goes back to the newest checkpoint instead of training on."""
        if not self.is_cuda:
            return
        from ..ops import _lib
        from . import fault

        try:
            _lib.check_status(self.device)
        except _lib.NativeLibraryError as e:
            raise fault.PersistentFault(f"iteration {self.iteration}: {e}") from e

    # ------------------------------------------------------------------ checkpoint
    def save_checkpoint(self, path: Optional[str] = None):
        from . import checkpoint

        self._check_device_status()   # never persist the state of a step whose kernels reported an error
        root = path or self.tcfg.save
        d = checkpoint.save_checkpoint(self, root)
        keep = self.tcfg.save_retain_interval
        if keep and not self.tcfg.async_save and (not dist.is_initialized() or dist.get_rank() == 0):
            import re
            import shutil

            for name in os.listdir(root):       # older checkpoints off the retention grid go; the newest always stays
                m = re.fullmatch(r"iter_(\d{7})", name)
                if m and int(m.group(1)) != self.iteration and int(m.group(1)) % int(keep):
                    shutil.rmtree(os.path.join(root, name), ignore_errors=True)
        return d

    def non_persistent_root(self) -> Optional[str]:
        tc = self.tcfg
        kind = (tc.non_persistent_ckpt_type or "").lower()
        if not kind:
            return None
        if kind == "global":
            return tc.non_persistent_global_ckpt_dir or (os.path.join(tc.save, "non_persistent") if tc.save else None)
        if kind == "local":
            return tc.non_persistent_local_ckpt_dir or os.path.join("/tmp", "primus_b200_non_persistent", tc.exp_name)
        if kind == "in_memory":
            return os.path.join("/dev/shm", "primus_b200_non_persistent", tc.exp_name)
        raise ValueError(f"non_persistent_ckpt_type {kind!r}: global | local | in_memory")

    def save_non_persistent_checkpoint(self) -> Optional[str]:
        """Write a throw-away checkpoint and drop the older ones of its kind."""
        import shutil

        from . import checkpoint

        root = self.non_persistent_root()
        if root is None:
            return None
        self._check_device_status()
        d = checkpoint.save_checkpoint(self, root)
        checkpoint.finalize_async_save()
        if dist.is_initialized():
            dist.barrier()
        if not dist.is_initialized() or dist.get_rank() == 0:
            keep = os.path.basename(d)
            for name in os.listdir(root):
                if name.startswith("iter_") and name != keep:
                    shutil.rmtree(os.path.join(root, name), ignore_errors=True)
        return d

    def load_checkpoint(self, path: Optional[str] = None) -> int:
        from . import checkpoint

        path = path or self.tcfg.load
        np_root = self.non_persistent_root()
        if np_root and os.path.isdir(np_root):
            newest_np = checkpoint.latest_iteration(np_root)
            newest = checkpoint.latest_iteration(path) if path and os.path.isdir(path) else None
            if newest_np is not None and (newest is None or newest_np > newest):
                self.log(f"[checkpoint] resuming from the non-persistent checkpoint of iteration {newest_np} in {np_root}")
                return checkpoint.load_checkpoint(self, np_root)
        it = checkpoint.load_checkpoint(self, path) if path and os.path.isdir(path) else 0
        tc = self.tcfg
        if it == 0 and path and checkpoint.read_tracker(path) is None:
            if tc.pretrained_checkpoint:
                self.log(f"[checkpoint] nothing under {path}: starting from the weights in {tc.pretrained_checkpoint}")
                checkpoint.load_checkpoint(self, tc.pretrained_checkpoint, finetune=True)
            elif tc.exit_on_missing_checkpoint:
                raise SystemExit(f"no checkpoint under {path} and exit_on_missing_checkpoint is set")
        return it
