"""TrainingSession: everything one rank needs to run optimizer steps from a RunSpec.

This is the public programmatic entry point (`turbo_dllm_b200.train` builds one and loops it;
`bench.py` drives it directly): model, objective runtime, data runtime, packed row layout,
attention transport, sharded optimizer and LR schedule. `step()` performs zero-grad → data →
corruption → forward → fused linear-CE loss → backward → gradient sync → clip → AdamW, and
returns the step's loss numerator/denominator as device tensors (no host sync inside).

It plays the role of the set-up half of the reference trainer
(dllm_parallel/training/block_diffusion_trainer.py:501-1265) plus one iteration of its step loop
(:1265-1545).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..config.run_spec import RunSpec
from ..data.runtimes import DataBatch, HostStagedRandomRuntime, RandomTokenDataRuntime
from ..models.config import ModelConfig, model_config_from_run_spec
from ..models.dense import LocalAttention, compact_supervised_rows
from ..objectives.runtime import CorruptedBatch, build_objective_runtime
from ..optim.flat_adamw import FlatAdamW
from ..optim.schedule import RunSpecLRScheduler
from ..parallel.layout import (PackedLayout, build_packed_layout, clean_positions_for_rank,
                               runtime_clean_layout)

_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


@dataclass
class StepResult:
    loss_sum: torch.Tensor        # Σ weighted CE over this rank's supervised rows (device scalar)
    denominator: float            # global loss denominator of the step
    supervised_rows: torch.Tensor
    input_tokens: int             # tokens of this rank's micro-batches (clean copy not counted)
    h2d_bytes: int


class TrainingSession:
    def __init__(self, spec: RunSpec, *, device: str | torch.device | None = None, runtime=None,
                 host_staged_data: bool = False):
        self.spec = spec
        self.runtime = runtime  # parallel runtime (None = single rank)
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        if device is None:
            device = f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        if self.device.type == "cuda":
            if self.device.index is None:
                self.device = torch.device("cuda", torch.cuda.current_device())
            torch.cuda.set_device(self.device)
        self.dtype = _DTYPES[spec.model.dtype]
        if self.device.type == "cpu" and self.dtype != torch.float32:
            raise ValueError("CPU runs use model.dtype=fp32 (the reference path is the fp32 oracle)")
        self.cfg: ModelConfig = model_config_from_run_spec(spec)
        seed = spec.launch.seed
        self.task = None
        from ..profiling.system_trace import PhaseTimer

        self.sharded = None
        self.trace = None                       # the trainer hands its SystemTrace over
        self.phase_timer = PhaseTimer(self.device)
        if spec.objective.name == "dflash_distillation":
            self._init_dflash(seed, runtime, host_staged_data)
            return
        ep = runtime.expert_parallel_size if runtime is not None else 1
        # the family's executor builds the model: no family names are spelled out here
        from ..models.contracts import BuildContext
        from ..models.registry import executor_for_family, family_of_config

        self.executor = executor_for_family(family_of_config(self.cfg, spec))
        problems = self.executor.validate_run_spec(spec)
        if problems:
            raise ValueError("run spec does not fit the model family:\n  - " + "\n  - ".join(problems))
        self.model = self.executor.build_model(BuildContext(
            spec=spec, cfg=self.cfg, device=self.device, dtype=self.dtype, runtime=runtime, seed=seed,
            activation_offload=self._want_activation_offload()))
        self.memory_report("model built")
        from ..models.hf_loader import load_hf_weights, pretrained_directory

        self.pretrained = None if spec.model.random_init else pretrained_directory(spec.model.id)
        if self.pretrained is not None:
            # model.id names a local checkpoint: start from its weights (every rank reads its own shard)
            load_hf_weights(self.model, self.pretrained)
        self.lora = None
        self.sharded = None      # parameter sharding (optimizer.backend: fsdp)
        if spec.adapter.type == "lora":
            from ..adapters.lora import apply_lora

            tp_ctx = getattr(self.model, "tp", None)
            self.lora = apply_lora(self.model, rank=spec.adapter.rank, alpha=spec.adapter.alpha,
                                   dropout=spec.adapter.dropout, targets=spec.adapter.targets or ("attention", "mlp"),
                                   seed=seed, tp=tp_ctx)
        keep = os.environ.get("TDLLM_KEEP_ATTENTION")
        _, off_attn, keep_attn, resident = self._memory_plan()
        self.model.store.keep_attention = (keep == "1") if keep is not None else keep_attn
        self.model.store.offload_attention = off_attn and self.device.type == "cuda"
        self.model.store.attention_resident_from = self.cfg.num_layers - resident
        if self.model.store.offload_attention and self.model.store.stream is None:
            self.model.store.stream = torch.cuda.Stream(device=self.device)
        dp_rank = runtime.sample_parallel_rank if runtime is not None else self.rank
        self.dp_size = runtime.data_parallel_size * ep if runtime is not None else self.world
        self.objective = build_objective_runtime(spec, mask_token_id=self.cfg.mask_token_id,
                                                 seed=seed + 7919 * (dp_rank + 1), device=self.device,
                                                 vocab_size=self.cfg.vocab_size)
        if hasattr(self.objective, "pack_response_suffix") and (
                self.cfg.is_hybrid or (runtime is not None and runtime.context_parallel_size > 1)):
            # context parallelism plans its clean shards and exchanges for whole sequences (and the hybrid family
            # scans whole sequences): the response stays in place and the supervision mask selects the scored rows.
            # Tensor parallelism divides heads, not rows, so it packs like a single rank; block parallelism alone
            # divides the decoder blocks of the packed response among its ranks.
            self.objective.pack_response_suffix = False
        elif hasattr(self.objective, "pack_response_suffix") and runtime is not None and runtime.block_parallel_size > 1:
            # every block-parallel rank needs a decoder block: short responses are padded up to that many
            self.objective.minimum_decoder_blocks = max(self.objective.minimum_decoder_blocks, runtime.block_parallel_size)
        # diffusiongemma_native_sft: the clean stream is causal and carries a next-token loss of its own
        # (dllm_parallel/core/models/backbones/nemotron/model.py:1089-1096, :1966-2030)
        self.encoder_loss_weight = (float(spec.objective.encoder_loss_weight)
                                    if self.objective.name == "diffusiongemma_native_sft" else 0.0)
        self.last_encoder_loss = None
        self.dp_rank = dp_rank
        self.data = self.executor.build_data_runtime(spec, self.cfg, self.device, dp_rank, self.dp_size,
                                                     host_staged=host_staged_data)
        if self.cfg.is_hybrid and runtime is not None:
            runtime.share_clean_replicas = False    # linear-attention layers trade row shards inside a CP chunk
        self.layout = self._build_layout()
        self.attend = self._build_attention()
        self._first_layout, self._first_attend = self.layout, self.attend
        if self.cfg.is_hybrid:
            from ..models.hybrid import BlockRows

            self.attend.block_rows = BlockRows(self.layout, spec.model.seq_len,
                                               head_parallel=self._build_head_parallel_plan())
        o = spec.optimizer
        okw = dict(lr=o.lr, betas=(o.adam_beta1, o.adam_beta2), eps=o.adam_eps, weight_decay=o.weight_decay)
        self.expert_optimizer = None
        if self.cfg.is_moe:
            dense_group = runtime.group("dense_optimizer") if runtime is not None else (
                dist.group.WORLD if self.world > 1 else None)
            expert_group = runtime.optimizer_group if runtime is not None else dense_group
            if self.lora is not None:     # only the adapters train: replicated pairs and per-expert pairs
                lora_tp = runtime.tensor_group if (runtime is not None and runtime.tensor_parallel_size > 1) else None
                self.optimizer = FlatAdamW(self.lora.flat, group=dense_group, tp_group=lora_tp, **okw)
                if self.lora.flat_experts is not None:
                    self.expert_optimizer = FlatAdamW(self.lora.flat_experts, group=expert_group, **okw)
            else:
                moe_tp = runtime.tensor_group if (runtime is not None and runtime.tensor_parallel_size > 1) else None
                if o.backend in ("fsdp", "fsdp2") and dense_group is not None and dist.get_world_size(dense_group) > 1:
                    # parameter sharding of the replicated (non-expert) part over all ranks that hold a copy of it;
                    # the experts are already divided by expert parallelism and keep their sharded optimizer
                    from ..parallel.fsdp import ShardedAdamW, ShardedParameters

                    if moe_tp is not None:
                        raise ValueError("optimizer.backend=fsdp for the mixture-of-experts decoder is built without "
                                         "tensor parallelism")
                    peer = (self.device.type == "cuda" and spec.kernel.impl not in ("cpu_reference", "nccl_baseline"))
                    if peer:
                        from ..parallel.symm import peer_access_available

                        peer = peer_access_available(dense_group)
                    self.sharded = ShardedParameters(self.model.flat, dense_group, self.device, use_peer_kernels=peer,
                                                     num_layers=self.cfg.num_layers)
                    self.model.attach_parameter_sharding(self.sharded)
                    self.optimizer = ShardedAdamW(self.sharded, **okw)
                else:
                    self.optimizer = FlatAdamW(self.model.flat, group=dense_group, tp_group=moe_tp, **okw)
                # (router and experts are replicated over the tensor-parallel ranks: counted once in the norm)
                self.expert_optimizer = FlatAdamW(self.model.flat_experts, group=expert_group, **okw)
            self.ep_group = runtime.group("expert") if ep > 1 else None
        else:
            group = runtime.optimizer_group if runtime is not None else (dist.group.WORLD if self.world > 1 else None)
            tp_group = runtime.tensor_group if (runtime is not None and runtime.tensor_parallel_size > 1) else None
            if o.backend in ("fsdp", "fsdp2") and group is not None and dist.get_world_size(group) > 1:
                from ..parallel.fsdp import ShardedAdamW, ShardedParameters

                if self.lora is not None:
                    raise ValueError("optimizer.backend=fsdp shards the base model's parameters; adapter runs use the "
                                     "sharded-optimizer backends")
                peer = (self.device.type == "cuda" and spec.kernel.impl not in ("cpu_reference", "nccl_baseline"))
                if peer:
                    from ..parallel.symm import peer_access_available

                    peer = peer_access_available(group)
                self.sharded = ShardedParameters(self.model.flat, group, self.device, use_peer_kernels=peer,
                                                 num_layers=self.cfg.num_layers)
                self.model.attach_parameter_sharding(self.sharded)
                self.optimizer = ShardedAdamW(self.sharded, tp_group=tp_group, **okw)
            else:
                self.optimizer = FlatAdamW(self.lora.flat if self.lora is not None else self.model.flat, group=group,
                                           tp_group=tp_group,
                                           fused_sync=None if tp_group is not None else self._build_fused_sync(group),
                                           **okw)
        if (spec.data.optimizer_step_unit == "trajectory" and self.dp_size > 1
                and (self.sharded is not None or getattr(self, "ep_group", None) is not None)):
            # data-parallel ranks take different trajectories, so their optimizer steps have different numbers of
            # micro-batches; parameter sharding and expert parallelism run collectives among those ranks inside every
            # forward and backward pass, which would no longer pair up
            raise ValueError("data.optimizer_step_unit=trajectory with more than one data-parallel rank needs replicated "
                             "parameters and no expert parallelism (use the sharded-optimizer backends)")
        self.scheduler = RunSpecLRScheduler.from_run_spec(spec)
        self.steps_done = 0
        self.memory_report("session built")

    def close(self) -> None:
        """Returns symmetric (peer-visible) buffers to the driver. They are allocated outside the
        caching allocator, so dropping the session alone does not free them. Collective: every rank of
        the optimizer group closes at the same point, after the last step has finished."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        sync = getattr(getattr(self, "optimizer", None), "fused_sync", None)
        if sync is not None:
            if dist.is_initialized():
                dist.barrier(group=sync.group)   # no peer may still be reading this rank's buffers
            flat = sync.flat
            data, grad = flat.data.clone(), torch.zeros_like(flat.grad)
            flat.data, flat.grad = data, grad
            for name, (o, n, shape, decay) in flat.offsets.items():
                p = flat.params[name]
                p.data = data[o:o + n].view(shape)
                p.main_grad = grad[o:o + n].view(shape)
            sync.close()
            self.optimizer.fused_sync = None
        if getattr(self, "sharded", None) is not None:
            self.sharded.close()
            self.sharded = None
        ee = getattr(getattr(self, "model", None), "expert_exchange", None)
        if ee and ee.get("exchange") is not None:
            ee["exchange"].close()
            ee["exchange"] = None
        exchange = getattr(getattr(self, "attend", None), "exchange", None)
        if exchange is not None and hasattr(exchange, "close"):
            exchange.close()
            self.attend.exchange = None

    def flats(self):
        if getattr(self, "lora", None) is not None:
            return [self.lora.flat] + ([self.lora.flat_experts] if self.lora.flat_experts is not None else [])
        out = [self.model.flat]
        if getattr(self.model, "flat_experts", None) is not None:
            out.append(self.model.flat_experts)
        return out

    # ---------------------------------------------------------------- set-up
    def _init_dflash(self, seed, runtime, host_staged_data):
        from .dflash_task import DFlashTask

        spec = self.spec
        dp_rank = runtime.data_parallel_rank if runtime is not None else self.rank
        self.dp_size = runtime.data_parallel_size if runtime is not None else self.world
        exchange = None
        if runtime is not None and runtime.local_parallel_size > 1:
            from ..parallel.dflash_context import DFlashContextParallel

            exchange = DFlashContextParallel(runtime.group("local_parallel"),
                                             context_sharded=runtime.context_parallel_size > 1,
                                             anchors_sharded=runtime.block_parallel_size > 1,
                                             mode=spec.kernel.dflash_context_exchange)
        self.task = DFlashTask(spec, self.cfg, dtype=self.dtype, device=self.device, seed=seed, dp_rank=dp_rank,
                               exchange=exchange, replicas=self.dp_size if runtime is not None else None)
        self.model, self.objective = self.task.model, self.task.objective
        tcfg = self.task.target.cfg
        if self.task.feature_store is not None:
            from ..data.dflash_features import FeatureStoreDataRuntime

            rows = None
            if exchange is not None and exchange.context_sharded:
                rows = lambda b, l: exchange.context_rows(b, l, "cpu")     # read this rank's context shard only
            self.data = FeatureStoreDataRuntime(self.task.feature_store, batch_size=spec.training.batch_size,
                                                device=self.device, dp_rank=dp_rank, dp_size=self.dp_size,
                                                context_rows=rows)
        else:
            data_kw = dict(batch_size=spec.training.batch_size, seq_len=spec.model.seq_len,
                           vocab_size=tcfg.vocab_size, mask_token_id=tcfg.mask_token_id,
                           seed=seed + 104729 * (dp_rank + 1), vocab_sample_size=spec.data.vocab_sample_size)
            self.data = (HostStagedRandomRuntime(device=self.device, **data_kw) if host_staged_data
                         else RandomTokenDataRuntime(device=self.device, **data_kw))
        self.layout, self.attend = None, None
        self.expert_optimizer = None
        group = runtime.optimizer_group if runtime is not None else (dist.group.WORLD if self.world > 1 else None)
        o = spec.optimizer
        self.optimizer = FlatAdamW(self.model.flat, lr=o.lr, betas=(o.adam_beta1, o.adam_beta2), eps=o.adam_eps,
                                   weight_decay=o.weight_decay, group=group, fused_sync=self._build_fused_sync(group))
        self.scheduler = RunSpecLRScheduler.from_run_spec(spec)
        self.steps_done = 0

    def _memory_plan(self) -> tuple[bool, bool, bool, int]:
        """(offload layer inputs, offload attention out/lse, keep attention out/lse at all, number of
        last layers whose attention outputs stay on the device although the others are offloaded).

        Keeping the attention output of every layer saves the forward kernel in the recomputation.
        Everything stays in HBM when it fits next to parameters, gradients, optimizer shard and one
        layer's working set; otherwise the attention outputs go to pinned host memory first (all but as
        many of the last layers as still fit), and the layer inputs follow only if that is still not
        enough. The copies hide behind the GEMMs as long as the host link keeps up, so less is better."""
        env = os.environ.get("TDLLM_ACTIVATION_OFFLOAD")
        if env is not None:
            return env == "1", env == "1", True, 0
        if self.device.type != "cuda" or not self.spec.training.activation_checkpointing:
            return False, False, self.device.type == "cuda", 0
        cfg, s = self.cfg, self.spec
        rows = 3 * s.model.seq_len * s.training.batch_size  # upper bound: two noisy views + clean
        per_layer = rows * cfg.hidden_size * 2
        ckpt = per_layer * cfg.num_layers
        work = rows * 2 * (6 * cfg.hidden_size + 2 * cfg.qkv_dim + 5 * max(cfg.intermediate_size, 1))
        if s.optimizer.backend in ("fsdp", "fsdp2") and self.world > 1:
            # shards of parameters, fp32 gradients and AdamW state; two layers and the embeddings at full size
            static = cfg.num_params() * 18 / self.world + 4 * 2 * cfg.layer_params() + 8 * cfg.vocab_size * cfg.hidden_size
        elif cfg.is_moe:
            # experts are divided over the expert-parallel ranks (weights, gradients and AdamW state of the local
            # experts stay on their rank); everything else is replicated with a sharded optimizer state
            rt = self.runtime
            ep = rt.expert_parallel_size if rt is not None else 1
            expert = cfg.num_layers * cfg.num_experts * 3 * cfg.hidden_size * cfg.moe_intermediate_size
            dense = cfg.num_params() - expert
            static = dense * (2 + 2 + 12 / max(self.world, 1)) + expert / max(ep, 1) * (2 + 2 + 12)
            k = max(cfg.num_experts_per_token, 1)
            # dispatched rows (three exchange slabs at twice the mean load) and the experts' activations
            work += rows * k * 2 * (3 * 2 * cfg.hidden_size + 5 * cfg.moe_intermediate_size)
        else:
            static = cfg.num_params() * (2 + 2 + 12 / max(self.world, 1))
        budget = 0.85 * torch.cuda.get_device_properties(self.device).total_memory
        if static + 2 * ckpt + work < budget:
            return False, False, True, 0
        if static + ckpt + work < budget:
            resident = int((budget - static - ckpt - work) // (per_layer * 1.02))
            return False, True, True, max(0, min(resident, cfg.num_layers))
        # both streams go to the host. Keeping some attention outputs resident was measured slower here:
        # with 156 of 178 GiB allocated the caching allocator runs out of reusable blocks mid-step
        # (growable segments were slower still), so the whole budget is left to the working set.
        return True, True, True, 0

    def _want_activation_offload(self) -> bool:
        return self._memory_plan()[0]

    def _select_layout(self, seq_len: int, response: tuple[int, int, int] | None = None) -> None:
        """Row layout and attention for micro-batches whose sequences are shorter than `model.seq_len` (indexed
        datasets hand out same-length batches of any block-aligned length), or whose noisy rows cover only a
        response suffix (`response` = (response start, valid length, decoder rows per sequence)). Layouts are built
        once per shape."""
        key = seq_len if response is None else (seq_len, *response)
        if key == getattr(self, "_layout_len", self.spec.model.seq_len):
            return
        cache = self.__dict__.setdefault("_layouts", {self.spec.model.seq_len: (self._first_layout, self._first_attend)})
        if key not in cache and response is not None:
            from ..parallel.layout import build_response_layout

            if len(cache) > 64:       # response starts vary from batch to batch: keep the table bounded
                for k in [k for k in cache if isinstance(k, tuple)][:32]:
                    del cache[k]
            s, rt = self.spec, self.runtime
            owned = None
            if rt is not None and rt.block_parallel_size > 1:
                # block parallelism alone: the decoder blocks of the response are scheduled over the ranks like the
                # blocks of a whole sequence (every rank keeps all clean rows)
                from ..parallel.schedule import build_block_schedule

                sched = build_block_schedule(response[2] // s.objective.block_size, rt.block_parallel_size)
                owned = sched.blocks_by_worker[rt.block_parallel_rank]
            lay = build_response_layout(
                seq_len=seq_len, block_size=s.objective.block_size, batch=s.training.batch_size,
                response_start=response[0], valid_length=response[1], decoder_length=response[2],
                window=self.cfg.sliding_window if self.cfg.has_sliding_layers else None, device=self.device,
                clean_causal=getattr(self, "encoder_loss_weight", 0.0) > 0.0, owned_blocks=owned)
            cache[key] = (lay, LocalAttention(getattr(self.model, "lcfg", self.cfg), lay.mask,
                                              store=self.model.store, window_mask=lay.window_mask))
        if key not in cache:
            rt = self.runtime
            if rt is not None and (rt.context_parallel_size > 1 or rt.block_parallel_size > 1):
                raise ValueError("variable sequence lengths are built for data-parallel runs; context / block "
                                 "parallelism plans its row layout for model.seq_len")
            if seq_len % self.spec.objective.block_size or seq_len > self.spec.model.seq_len:
                raise ValueError(f"a batch of length {seq_len} does not fit block size "
                                 f"{self.spec.objective.block_size} / model.seq_len {self.spec.model.seq_len}")
            lay = self._build_layout(seq_len)
            cache[seq_len] = (lay, LocalAttention(getattr(self.model, "lcfg", self.cfg), lay.mask,
                                                  store=self.model.store, window_mask=lay.window_mask))
        self.layout, self.attend = cache[key]
        self._layout_len = key

    def _build_layout(self, seq_len: int | None = None) -> PackedLayout:
        s, rt = self.spec, self.runtime
        owned, clean = None, None
        if rt is not None and rt.block_parallel_size > 1:
            owned = rt.owned_blocks
        if rt is not None and rt.context_parallel_size > 1:
            lay = runtime_clean_layout(s.kernel.cp_bp_clean_kv_layout, rt.block_parallel_size)
            clean = clean_positions_for_rank(s.model.seq_len, rt.context_parallel_size, rt.context_parallel_rank,
                                             lay, s.objective.block_size, self.device)
            if not rt.owns_clean_shard:     # another rank computes this shard's clean stream; its K/V are pulled
                clean = clean[:0]
        elif rt is not None and rt.block_parallel_size > 1 and s.topology.replicate_clean_prefix:
            last = max(owned)
            # the clean tokens in front of the rank's last block; linear-attention layers scan whole sequences
            # (their chunk states are indexed by position), so the hybrid family keeps every clean row, and so does a
            # run whose clean stream carries a next-token loss (every position is then scored by exactly one rank)
            whole = self.cfg.is_hybrid or getattr(self, "encoder_loss_weight", 0.0) > 0.0
            stop = s.model.seq_len if whole else last * s.objective.block_size
            clean = torch.arange(0, stop, device=self.device)
        offsets = None
        if rt is not None and rt.splits_block_tokens and not self.cfg.is_hybrid:
            from ..parallel.layout import pure_context_offsets

            offsets = pure_context_offsets(s.objective.block_size, rt.context_parallel_size, rt.context_parallel_rank)
        return build_packed_layout(seq_len=seq_len or s.model.seq_len, block_size=s.objective.block_size,
                                   batch=s.training.batch_size, views=self.objective.views,
                                   owned_blocks=owned, clean_pos=clean, device=self.device, noisy_offsets=offsets,
                                   window=self.cfg.sliding_window if self.cfg.has_sliding_layers else None,
                                   clean_causal=getattr(self, "encoder_loss_weight", 0.0) > 0.0)

    def _build_head_parallel_plan(self):
        """Row bookkeeping of the head <-> sequence exchange that linear-attention layers use when the
        clean rows are sharded over a context-parallel group (None otherwise)."""
        rt, s = self.runtime, self.spec
        if rt is None or rt.context_parallel_size <= 1:
            return None
        from ..models.hybrid import HeadParallelPlan

        bs, batch = s.objective.block_size, s.training.batch_size
        lay = runtime_clean_layout(s.kernel.cp_bp_clean_kv_layout, rt.block_parallel_size)
        nblocks = s.model.seq_len // bs
        noisy, clean = [], []
        for phys in rt.groups.ranks["context_block_parallel"]:
            a = rt.plan.rank_assignments[phys]
            owned = sorted(a.owned_blocks) if rt.block_parallel_size > 1 else list(range(nblocks))
            starts = torch.tensor(owned, device=self.device) * bs
            reps = batch * self.objective.views
            seq = torch.arange(batch, device=self.device).repeat_interleave(self.objective.views * len(owned))
            noisy.append((seq, starts.repeat(reps)))
            clean.append(clean_positions_for_rank(s.model.seq_len, rt.context_parallel_size, a.context_parallel_rank,
                                                  lay, bs, self.device))
        return HeadParallelPlan(group=rt.context_group, index=dist.get_rank(rt.context_group), noisy_blocks=noisy,
                                clean_positions=clean, batch=batch, seq_len=s.model.seq_len, block_size=bs,
                                device=self.device)

    def _build_attention(self):
        rt = self.runtime
        if rt is not None and rt.context_parallel_size > 1:
            from ..parallel.context_attention import ContextParallelAttention

            return ContextParallelAttention(getattr(self.model, "lcfg", self.cfg), self.layout, rt, self.spec,
                                            store=getattr(self.model, "store", None))
        return LocalAttention(getattr(self.model, "lcfg", self.cfg), self.layout.mask, store=self.model.store,
                              window_mask=self.layout.window_mask)

    def _build_fused_sync(self, group):
        if group is None or self.device.type != "cuda" or self.spec.kernel.impl in ("cpu_reference", "nccl_baseline"):
            return None
        if self.spec.optimizer.backend not in ("auto", "zero_fused"):
            return None
        try:
            from ..parallel.fused_zero import FusedZeroSync

            # the buffer the optimizer owns: the adapters when LoRA freezes the base model
            lora = getattr(self, "lora", None)
            return FusedZeroSync.create(lora.flat if lora is not None else self.model.flat, group)
        except Exception as e:  # no peer access, IPC refused, ...: keep the NCCL path, say why
            if self.spec.optimizer.backend == "zero_fused":
                raise
            if self.rank == 0:
                print(f"[turbo_dllm_b200] fused ZeRO sync unavailable ({e}); using NCCL collectives", flush=True)
            return None

    # ------------------------------------------------------------------ rows
    def assemble_rows(self, cb: CorruptedBatch):
        """Gathers this rank's packed rows from a corrupted batch.
        Returns (tokens [rows], labels [rows], weights [rows] or None)."""
        lay = self.layout
        bs = lay.block_size
        # response-suffix packing indexes the decoder tensors by the row's offset from the response start
        at = lay.noisy_pos if lay.noisy_offset is None else lay.noisy_offset
        noisy = cb.noisy_input_ids[lay.noisy_seq, lay.noisy_view, at]
        clean = cb.clean_input_ids[lay.clean_seq, lay.clean_pos]
        tokens = torch.cat([noisy, clean])
        nlab = cb.labels[lay.noisy_seq, lay.noisy_view, at]
        labels = torch.cat([nlab, torch.full_like(clean, -100)])
        w = cb.loss_weights[lay.noisy_seq, lay.noisy_view, at // bs]
        weights = torch.cat([w, torch.zeros(clean.shape[0], device=w.device)])
        return tokens, labels, weights

    def memory_report(self, tag: str) -> None:
        """With TDLLM_MEMORY_REPORT=1, every rank writes one line of device-memory figures to stderr."""
        if self.device.type != "cuda" or os.environ.get("TDLLM_MEMORY_REPORT") != "1":
            return
        import sys

        free, total = torch.cuda.mem_get_info(self.device)
        gib = 2.0 ** 30
        print(f"[memory rank {self.rank}] {tag}: torch allocated {torch.cuda.memory_allocated(self.device) / gib:.2f} "
              f"peak {torch.cuda.max_memory_allocated(self.device) / gib:.2f} reserved "
              f"{torch.cuda.memory_reserved(self.device) / gib:.2f} GiB; device in use {(total - free) / gib:.2f} "
              f"of {total / gib:.2f} GiB", file=sys.stderr, flush=True)

    # ------------------------------------------------------------------ step
    def forward_backward(self, batch: DataBatch, denominator: float):
        extra = {}
        if batch.valid_mask is not None:
            if self.objective.name != "diffusiongemma_native_sft":
                raise ValueError("padded batches (valid_mask) are built for diffusiongemma_native_sft")
            extra["valid_mask"] = batch.valid_mask
        cb = self.objective.corrupt(batch.input_ids, supervision_mask=batch.supervision_mask,
                                    supervision_count=batch.supervision_count, **extra)
        valid_len = int(batch.input_ids.shape[1])
        if not self.cfg.is_hybrid:
            response = None
            if cb.response_start is not None:       # decoder rows cover the response only
                response = (cb.response_start, cb.valid_length, int(cb.noisy_input_ids.shape[2]))
                valid_len = cb.valid_length
            self._select_layout(int(batch.input_ids.shape[1]), response)
        tokens, labels, weights = self.assemble_rows(cb)
        n_noisy = self.layout.n_noisy
        if self.encoder_loss_weight > 0.0:
            # clean row (s, p) predicts the clean token at p + 1; the term has its own denominator (pairs of
            # consecutive tokens over the whole step), folded into the row weights so that one division by
            # the decoder's denominator normalises both terms
            lay, x0 = self.layout, cb.clean_input_ids
            nxt = (lay.clean_pos + 1).clamp_max(x0.shape[1] - 1)
            enc_labels = torch.where(lay.clean_pos + 1 < valid_len, x0[lay.clean_seq, nxt],
                                     torch.full_like(nxt, -100))      # padding is neither input nor target
            rt = self.runtime
            if rt is not None and rt.block_parallel_size > 1 and rt.context_parallel_size == 1:
                # block parallelism alone: every rank holds the whole clean sequence; each scores the clean positions
                # of its own blocks, so the term is counted once over the group
                own = torch.zeros(x0.shape[1] // lay.block_size + 1, dtype=torch.bool, device=lay.clean_pos.device)
                own[torch.as_tensor(sorted(rt.owned_blocks), device=own.device)] = True
                enc_labels = torch.where(own[lay.clean_pos // lay.block_size], enc_labels, torch.full_like(enc_labels, -100))
            labels = torch.cat([labels[:n_noisy], enc_labels.to(labels.dtype)])
            enc_w = self.encoder_loss_weight * float(denominator) / self._encoder_denominator
            weights = torch.cat([weights[:n_noisy], torch.full_like(weights[n_noisy:], enc_w)])
        with self._phase("forward"):
            soft, soft_rows = self._self_conditioning_inputs(tokens, cb)
            hidden = self.model(tokens, self.layout.positions, self.attend, soft, soft_rows)
        self.memory_report("after forward")
        with self._phase("loss"):
            h, l, w, kept = compact_supervised_rows(hidden, labels, weights)
            loss_sum, per_row = self.model.loss(h, l, w, self.objective.exclude_mask_token)
            if self.encoder_loss_weight > 0.0 and per_row is not None:
                clean_rows = kept >= n_noisy
                self.last_encoder_loss = (per_row.detach()[clean_rows].sum() / self._encoder_denominator)
        self.memory_report("after loss")
        with self._phase("backward"):
            (loss_sum / denominator).backward()
            if self.sharded is not None:
                # per micro-batch (the gradient buffers restart each time), once the gradients are in their buffers
                self.sharded.end_micro_batch(before_reduce=self._sync_tensor_parallel_partial_gradients)
        self.memory_report("after backward")
        return loss_sum.detach(), l.shape[0], cb

    def _self_conditioning_inputs(self, tokens: torch.Tensor, cb):
        """Self-conditioning (diffusiongemma_native_sft): for the samples the objective marked, a detached
        first pass predicts every noisy row and the expected embedding under that prediction
        (`ops.soft_embedding`) is added to the row's input embedding in the real pass."""
        chosen = getattr(cb, "self_conditioning_mask", None)
        if chosen is None or getattr(self, "lora", None) is not None:
            return None, None
        from ..ops.soft_embedding import streaming_soft_embedding

        lay = self.layout
        rows = chosen.to(self.device)[lay.noisy_seq].nonzero(as_tuple=True)[0]   # noisy rows come first in the packing
        need = rows.numel() > 0
        run = need
        ep_group = getattr(self, "ep_group", None)
        if ep_group is not None:
            # expert-parallel ranks hold different samples, and the model's forward exchanges tokens among them: if
            # any of them has a marked sample, all of them run the first pass (the others discard its result)
            flag = torch.tensor([int(need)], dtype=torch.int32, device=self.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=ep_group)
            run = bool(int(flag))
        if not run:
            return None, None
        with torch.no_grad():
            hidden0 = self.model(tokens, lay.positions, self.attend)
            if not need:
                return None, None
            o = self.spec.objective
            tp = getattr(self.model, "tp", None)
            soft = streaming_soft_embedding(hidden0.index_select(0, rows), self.model.lm_head,
                                            row_chunk_size=o.self_conditioning_row_chunk_size,
                                            vocab_chunk_size=o.self_conditioning_vocab_chunk_size,
                                            tp_group=tp.group if tp is not None and tp.size > 1 else None)
        return soft, rows

    def global_denominator(self, batches: list[DataBatch]) -> float:
        """Loss denominator of the whole optimizer step over all data-parallel ranks."""
        b, l = batches[0].input_ids.shape
        per = (l - 1) if self.objective.name == "fast_dllm_v2" else l
        # pure context parallelism (no block parallelism) keeps every noisy block on every rank of the context
        # group: their loss terms are computed that many times and the summed gradients must be divided by it
        rt = self.runtime
        copies = (rt.context_parallel_size if rt is not None and rt.context_parallel_size > 1
                  and rt.block_parallel_size == 1 and not (rt.splits_block_tokens and not self.cfg.is_hybrid) else 1)
        if all(x.supervision_mask is None for x in batches):
            return float(b * per * len(batches) * self.dp_size * copies)
        cnt = torch.zeros(1, dtype=torch.float64, device=self.device)
        for x in batches:
            m = x.supervision_mask
            cnt += (m[:, 1:] if self.objective.name == "fast_dllm_v2" else m).sum()
        if self.world > 1:
            dist.all_reduce(cnt)
            bpcp = (self.runtime.local_parallel_size * self.runtime.tensor_parallel_size) if self.runtime else 1
            cnt /= bpcp
        return float(cnt) * copies

    def _sync_tensor_parallel_partial_gradients(self) -> None:
        tp = getattr(self.model, "tp", None)
        if tp is not None and tp.size > 1:
            from ..parallel.tensor_parallel import sync_partial_gradients

            sync_partial_gradients(self.model.flat.params.values(), tp)
            if getattr(self, "lora", None) is not None:
                sync_partial_gradients(self.lora.flat.params.values(), tp)
                if self.lora.flat_experts is not None:
                    sync_partial_gradients(self.lora.flat_experts.params.values(), tp)

    def _phase(self, name: str):
        return self.phase_timer.phase(name, self.trace)

    def step(self) -> StepResult:
        spec = self.spec
        with self._phase("zero_grad"):
            for f in self.flats():
                f.zero_grad()
            if self.sharded is not None:
                self.sharded.zero_grad()
        with self._phase("data"):
            batches = self.data.next_optimizer_step_batches(spec.training.gradient_accumulation_steps)
        total = torch.zeros((), dtype=torch.float32, device=self.device)
        rows = 0
        if self.task is not None:
            # per-micro-batch normalisation by the weighted supervised count of that micro-batch;
            # gradients are averaged over micro-batches and data-parallel ranks
            scale = float(len(batches) * self.dp_size)
            denom = 0.0
            self.task.set_optimizer_step(self.steps_done, max(int(spec.training.steps or 1), 1))
            for b in batches:
                with self._phase("forward"):     # drafter tasks run forward, loss and backward as one call
                    ls, n, d = self.task.forward_backward(b)
                total += ls.float() / d.float() / scale
                rows += n
            denom = 1.0
            self._grad_div = scale
        else:
            turn_mean = (spec.data.trajectory_loss_reduction == "turn_mean"
                         and all(b.turn_weight is not None for b in batches))
            denom = 1.0 if turn_mean else self.global_denominator(batches)
            if self.encoder_loss_weight > 0.0:
                b0, l0 = batches[0].input_ids.shape
                pairs = sum(int((x.valid_mask.sum(1) - 1).clamp_min(0).sum()) if x.valid_mask is not None
                            else b0 * (l0 - 1) for x in batches)
                self._encoder_denominator = float(max(pairs * self.dp_size, 1))
            wsum = sum(b.turn_weight for b in batches) if turn_mean else 0.0
            shifted = self.objective.name == "fast_dllm_v2"
            for b in batches:
                if turn_mean:
                    # mean over the trajectory's turns (terminal turn weighted) of each turn's token-mean loss,
                    # averaged over the data-parallel ranks' trajectories
                    # (dllm_parallel/core/data.py:739, block_diffusion_trainer.py:385-415)
                    cnt = b.supervision_count_shifted if shifted else b.supervision_count
                    d = float(max(cnt, 1)) * wsum / b.turn_weight * self.dp_size
                    ls, n, _ = self.forward_backward(b, d)
                    total += ls.float() / d
                else:
                    ls, n, _ = self.forward_backward(b, denom)
                    total += ls.float()
                rows += n
        with self._phase("gradient_sync"):
            if self.sharded is None:       # sharded parameters reduce their gradients layer by layer in the backward
                for f in self.flats():
                    f.collect_grads()
                self._sync_tensor_parallel_partial_gradients()     # once, on the sums over the micro-batches
            elif self.expert_optimizer is not None:
                self.model.flat_experts.collect_grads()            # the experts are not part of the sharded buffer
            if getattr(self, "_grad_div", 1.0) != 1.0:
                self.model.flat.grad.div_(self._grad_div)
        if spec.debug.grad_finite:      # debug.grad_finite: stop at the first non-finite gradient, naming the buffer
            for i, f in enumerate(self.flats()):
                if not bool(torch.isfinite(f.grad).all()):
                    bad = [n for n, p in f.params.items() if not bool(torch.isfinite(p.main_grad).all())]
                    raise FloatingPointError(f"non-finite gradient at step {self.steps_done + 1} in buffer {i}: "
                                             f"{', '.join(bad[:8])}")
        lr, wd = self.scheduler.step()
        clip = spec.optimizer.gradient_clip_norm
        if spec.training.skip_optimizer_step:
            pass
        elif self.expert_optimizer is None:
            # reduce-scatter, global-norm clip, AdamW and parameter all-gather are one fused sequence
            with self._phase("optimizer"):
                self.optimizer.step(lr=lr, weight_decay=wd, max_grad_norm=clip)
        else:
            # one global norm over replicated and expert-sharded parameters
            with self._phase("gradient_sync"):
                dense_sq = self.optimizer.reduce_gradients()
                expert_sq = self.expert_optimizer.reduce_gradients()
                if self.ep_group is not None:
                    dist.all_reduce(expert_sq, group=self.ep_group)
                total_sq = dense_sq + expert_sq
            with self._phase("optimizer"):
                self.optimizer.apply_update(total_sq, lr=lr, weight_decay=wd, max_grad_norm=clip)
                self.expert_optimizer.apply_update(total_sq, lr=lr, weight_decay=wd, max_grad_norm=clip)
        if spec.debug.optimizer_finite and not spec.training.skip_optimizer_step:
            for i, f in enumerate(self.flats()):      # debug.optimizer_finite: parameters after the update
                if not bool(torch.isfinite(f.data).all()):
                    bad = [n for n, p in f.params.items() if not bool(torch.isfinite(p).all())]
                    raise FloatingPointError(f"non-finite parameters after the optimizer step {self.steps_done + 1} in "
                                             f"buffer {i}: {', '.join(bad[:8])}")
        self.steps_done += 1
        return StepResult(total, denom, torch.tensor(rows), sum(int(b.input_ids.numel()) for b in batches),
                          sum(b.h2d_bytes for b in batches))

    # ------------------------------------------------------------- checkpoint
    def state_dict(self) -> dict:
        extra = {}
        if self.expert_optimizer is not None:
            extra = {"expert_model": self.model.flat_experts.data, "expert_optimizer": self.expert_optimizer.state_dict()}
        if getattr(self, "lora", None) is not None:
            # the adapters are what training changes; every rank holds the whole (replicated) adapter buffer
            extra["adapter"] = self.lora.flat.data
            if self.lora.flat_experts is not None:       # this expert-parallel rank's per-expert pairs
                extra["adapter_experts"] = self.lora.flat_experts.data
        model_state = self.sharded.param_shard if self.sharded is not None else self.model.flat.data
        return {**extra, "model": model_state, "optimizer": self.optimizer.state_dict(),
                "scheduler": self.scheduler.state_dict(), "objective": self.objective.state_dict(),
                "data": self.data.state_dict(), "steps_done": self.steps_done}

    def load_state_dict(self, state: dict) -> None:
        (self.sharded.param_shard if self.sharded is not None else self.model.flat.data).copy_(state["model"])
        if getattr(self, "lora", None) is not None and "adapter" in state:
            self.lora.flat.data.copy_(state["adapter"])
            if self.lora.flat_experts is not None and "adapter_experts" in state:
                self.lora.flat_experts.data.copy_(state["adapter_experts"])
        self.optimizer.load_state_dict(state["optimizer"])
        # the optimizer restored this rank's shard of its buffer from the fp32 master; the other shards come
        # from their owners (a no-op on one rank)
        self.optimizer._all_gather_params()
        if self.expert_optimizer is not None and "expert_model" in state:
            self.model.flat_experts.data.copy_(state["expert_model"])
            self.expert_optimizer.load_state_dict(state["expert_optimizer"])
        self.scheduler.load_state_dict(state["scheduler"])
        self.objective.load_state_dict(state["objective"])
        self.data.load_state_dict(state["data"])
        self.steps_done = int(state["steps_done"])
