"""The training loop (`dllm-train`, `turbo_dllm_b200.train`).

One canonical loop: initialise distributed state (NCCL with a device id, plus a gloo group for
Python objects), build the parallel runtime and a `TrainingSession`, resume from a checkpoint
when asked, then run optimizer steps. Rank 0 prints one JSON line per event (`run_start`, `step`,
`checkpoint`, `summary`, `fatal_exception`), sorted keys, same field names as the reference's
events so log tooling carries over. Step timing excludes `profiler.warmup_steps`; the summary
reports the max over ranks of the mean timed step, tokens/s and MFU.

Counterpart of `run_block_diffusion_training` (dllm_parallel/training/block_diffusion_trainer.py:501-1978;
step loop :1265-1734, loss readback :157-233, summary :1807-1935, failure path :1938-1978).
"""
from __future__ import annotations

import json
import os
import sys
import time
import traceback
from typing import Sequence

import torch
import torch.distributed as dist

from ..config.run_spec import RunSpec, RunSpecError, build_run_spec_arg_parser, run_spec_from_args
from ..profiling.perf import (hardware_peak_tflops, model_attention_pairs, model_flops_utilization_pct,
                              transformer_step_flops)
from . import checkpointing as ckpt_policy
from .fault_tolerance import install_fault_handlers, write_fatal_marker
from .session import TrainingSession
from ..profiling.system_trace import SystemTrace
from .metrics import WandBRunLogger
from .token_accounting import TokenCounters, collect_run_context


def emit(event: dict) -> None:
    print(json.dumps(event, sort_keys=True, default=str), flush=True)


def init_distributed(device_type: str):
    """Returns (rank, world, local_rank, gloo_group)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    gloo = None
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if device_type == "cuda":
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            gloo = dist.new_group(backend="gloo")
        else:
            dist.init_process_group("gloo")
            gloo = dist.group.WORLD
    return rank, world, local_rank, gloo


class AsyncLossReadback:
    """Accumulates (loss numerator, supervised rows) on the device; one small all-reduce and one
    non-blocking copy to pinned memory per step, read when the step event is written."""

    def __init__(self, device, world: int):
        self.device, self.world = device, world
        self.buf = torch.zeros(2, dtype=torch.float64, device=device)
        self.host = torch.zeros(2, dtype=torch.float64, pin_memory=(device.type == "cuda"))
        self.event = torch.cuda.Event() if device.type == "cuda" else None

    def enqueue(self, loss_sum: torch.Tensor, rows: int, replicas: int = 1) -> None:
        """`replicas`: ranks that hold the SAME loss terms (tensor-parallel ranks all return the full loss of
        their shared rows): their copies are divided out of the world sum."""
        self.buf[0] = loss_sum.double()
        self.buf[1] = float(rows)
        if replicas > 1:
            self.buf /= float(replicas)
        if self.world > 1:
            from ..profiling.operator_trace import communication_scope

            with communication_scope("world", "loss", "all_reduce", self.buf.numel() * 8):
                dist.all_reduce(self.buf)
        self.host.copy_(self.buf, non_blocking=True)
        if self.event is not None:
            self.event.record()

    def resolve(self) -> tuple[float, float]:
        if self.event is not None:
            self.event.synchronize()
        return float(self.host[0]), float(self.host[1])


def run_training(spec: RunSpec) -> dict:
    """Runs the spec to completion on this rank. Returns the summary dict (rank 0) or {}."""
    use_cuda = torch.cuda.is_available() and spec.model.dtype != "fp32" or \
        (torch.cuda.is_available() and os.environ.get("TDLLM_FORCE_CUDA") == "1")
    device_type = "cuda" if use_cuda else "cpu"
    rank, world, local_rank, gloo = init_distributed(device_type)
    device = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")
    install_fault_handlers()
    spec.validate(world_size=world)
    run_dir = os.environ.get("DLLM_RUN_DIR")
    session = None
    runtime = None
    try:
        if world > 1:
            from ..parallel.runtime import build_parallel_runtime

            runtime = build_parallel_runtime(spec, device=device, rank=rank, world_size=world)
            runtime.warm_collectives()
        session = TrainingSession(spec, device=device, runtime=runtime,
                                  host_staged_data=(spec.data.input_mode == "random" and use_cuda
                                                    and os.environ.get("TDLLM_HOST_STAGED", "0") == "1"))
        start_step = 0
        load_dir, tag = ckpt_policy.resolve_load_checkpoint(spec)
        if load_dir is not None:
            from ..checkpoint import load_training_checkpoint

            meta = load_training_checkpoint(load_dir, tag, session, rank=rank, world_size=world, runtime=runtime)
            start_step = int(meta["step"])
        if spec.objective.skip_rng_steps:
            session.objective.skip(spec.objective.skip_rng_steps, (spec.training.batch_size, spec.model.seq_len))
        if rank == 0:
            emit({"event": "run_start", "world_size": world, "device": str(device), "model_id": spec.model.id,
                  "parameters": session.cfg.num_params(), "objective": spec.objective.name,
                  "layout": runtime.plan.layout if runtime else "dp", "resume_step": start_step,
                  "config": spec.to_dict()})
        readback = AsyncLossReadback(device, world)
        wb = WandBRunLogger(spec, rank)
        counters = TokenCounters()
        timed_counters = TokenCounters()
        trace = SystemTrace.from_run_spec(spec, rank, barrier=(dist.barrier if world > 1 else None))
        run_ctx = collect_run_context(world)
        timed_ms: list[float] = []
        t_train0 = time.monotonic()
        session.trace = trace
        session.phase_timer.configure(spec.profiler.phase_timing, spec.profiler.phase_timing_sync)
        control = ckpt_policy.StepControl(spec, spec.training.steps, rank=rank, world=world, group=gloo, device=device)
        tp_replicas = runtime.tensor_parallel_size if runtime is not None else 1
        dp = session.dp_size
        tokens_per_step = spec.global_batch(dp) * spec.model.seq_len
        total_steps = spec.training.steps
        last_loss = float("nan")
        for step in range(start_step + 1, total_steps + 1):
            if use_cuda:
                torch.cuda.reset_peak_memory_stats(device)
            trace.begin_step(step)
            traced = trace.active          # a step under the profiler pays for the tracing: it is not timed
            t0 = time.perf_counter()
            res = session.step()
            readback.enqueue(res.loss_sum, int(res.supervised_rows), tp_replicas)
            if use_cuda:
                torch.cuda.synchronize(device)
            ms = (time.perf_counter() - t0) * 1e3
            trace.end_step(step)
            if use_cuda:
                from ..kernels import native

                native.raise_on_device_error()   # bounded device waits report here instead of hanging
            loss_sum, rows = readback.resolve()
            last_loss = loss_sum / res.denominator
            if last_loss != last_loss or abs(last_loss) == float("inf"):
                raise FloatingPointError(f"non-finite loss at step {step}: {last_loss}")
            timed = step - start_step > spec.profiler.warmup_steps and not traced
            if timed:
                timed_ms.append(ms)
            # drafter distillation normalises per micro-batch (denominator 1): its supervised count is the rows
            supervised = rows if session.task is not None else float(res.denominator)
            counters.add(input_tokens=tokens_per_step, supervised_tokens=supervised, active_tokens=rows)
            if timed:      # throughput counts the tokens of the steps whose time it divides by
                timed_counters.add(input_tokens=tokens_per_step, supervised_tokens=supervised, active_tokens=rows)
            if rank == 0:
                ev = ({"event": "step", "step": step, "completed_steps": step, "target_total_steps": total_steps,
                      "timed": timed, "loss": last_loss, "lr": session.scheduler.lr_at(session.scheduler.step_count),
                      "grad_norm": session.optimizer.grad_norm(), "gradient_clip_norm": spec.optimizer.gradient_clip_norm,
                      "ms": ms, "active_tokens": rows, "valid_tokens": res.denominator, "input_tokens": tokens_per_step,
                      "perf": {"input_tokens_per_second": tokens_per_step / (ms / 1e3),
                               "input_tokens_per_second_per_gpu": tokens_per_step / (ms / 1e3) / world},
                      "optimizer_step": not spec.training.skip_optimizer_step,
                      "gradient_accumulation_steps": spec.training.gradient_accumulation_steps,
                      "optimizer_backend": ("fsdp_sharded" if getattr(session, "sharded", None) is not None else
                                            "zero_fused" if session.optimizer.fused_sync else "flat_adamw"),
                      "peak_mib": (torch.cuda.max_memory_allocated(device) / 2 ** 20) if use_cuda else None})
                if spec.profiler.phase_timing:
                    ev["phase_ms"] = session.phase_timer.take()
                emit(ev)
                wb.log_event(ev)
            elif spec.profiler.phase_timing:
                session.phase_timer.take()
            # rank 0's clock decides for everybody (a rank acting on its own clock would save or stop alone)
            verdict = control.decide(step)
            if verdict.save:
                from ..checkpoint import save_training_checkpoint

                tagname = save_training_checkpoint(spec.checkpointing.save_checkpoint_dir, session, step=step,
                                                   rank=rank, world_size=world, runtime=runtime, spec=spec,
                                                   control_group=gloo, tag=verdict.tag)
                if rank == 0:
                    emit({"event": "checkpoint", "step": step, "tag": tagname,
                          "dir": spec.checkpointing.save_checkpoint_dir})
            if verdict.stop:
                if rank == 0:
                    emit({"event": "duration_limit", "step": step, "elapsed_seconds": control.elapsed()})
                break
        mean_ms = sum(timed_ms) / len(timed_ms) if timed_ms else float("nan")
        # every rank's own figures, gathered as Python objects over the host-side group: the summary shows which rank
        # is slow or holds the most memory (dllm_parallel/training/block_diffusion_trainer.py:1771-1806)
        mine = {"rank": rank, "avg_ms": mean_ms, "min_ms": min(timed_ms) if timed_ms else None,
                "max_ms": max(timed_ms) if timed_ms else None, "measured_steps": len(timed_ms),
                "peak_mib": (torch.cuda.max_memory_allocated(device) / 2 ** 20) if use_cuda else None}
        rank_metrics = [mine]
        if world > 1:
            rank_metrics = [None] * world
            dist.all_gather_object(rank_metrics, mine, group=gloo)
            t = torch.tensor([mean_ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            mean_ms = float(t)
        eval_metrics = {}
        if spec.evaluation.batches > 0:
            from .evaluation import evaluate_masked_token_accuracy

            eval_metrics = evaluate_masked_token_accuracy(session, spec.evaluation.batches, spec.evaluation.seed)
        summary = {}
        if rank == 0:
            views = getattr(session.objective, "views", 1)
            gb = spec.global_batch(dp)
            if session.task is not None:       # drafter distillation: drafter + frozen target + frozen head
                from ..profiling.perf import dflash_step_flops

                task = session.task
                fl = dflash_step_flops(
                    session.cfg, task.target.cfg, seq_len=spec.model.seq_len,
                    block_size=task.objective.block_size, anchors=task.objective.max_anchors,
                    num_target_layers=len(spec.model.target_layer_ids), batch=gb,
                    online_target=spec.data.target_features == "online", loss=spec.objective.dflash_loss,
                    draft_vocab_size=task.draft_vocab.size if task.draft_vocab is not None else None)
            else:
                fl = transformer_step_flops(
                    session.cfg, rows=(views + 1) * spec.model.seq_len * gb,
                    pairs=model_attention_pairs(session.cfg, spec.model.seq_len, spec.objective.block_size, views) * gb,
                    vocab_rows=gb * spec.model.seq_len)
            mfu = None
            if use_cuda and mean_ms == mean_ms:
                try:
                    peak = hardware_peak_tflops(torch.cuda.get_device_name(device))
                    mfu = model_flops_utilization_pct(fl.total, mean_ms / 1e3, world, peak)
                except ValueError:
                    mfu = None
            summary = {"event": "summary", "model_id": spec.model.id, "seq_len": spec.model.seq_len,
                       "batch_size": spec.training.batch_size, "steps": total_steps, "final_loss": last_loss,
                       "step_time_ms": mean_ms, "measured_steps": len(timed_ms),
                       "input_tokens_per_second": tokens_per_step / (mean_ms / 1e3) if mean_ms == mean_ms else None,
                       "model_tflop_per_step": fl.total / 1e12, "mfu_pct": mfu, "world_size": world,
                       "parallel_layout": runtime.plan.layout if runtime else "dp",
                       "training_elapsed_seconds": time.monotonic() - t_train0, "run_context": run_ctx.to_dict(),
                       "system_trace": trace.exported, "rank_metrics": rank_metrics, **eval_metrics,
                       **timed_counters.throughput(sum(timed_ms) / 1e3, world)}
            emit(summary)
            wb.log_event(summary)
            wb.log_summary(summary)
        wb.finish()
        from ..checkpoint import wait_for_async_saves

        wait_for_async_saves()
        session.close()
        return summary
    except Exception as e:
        info = {"event": "fatal_exception", "rank": rank, "error": f"{type(e).__name__}: {e}",
                "traceback": traceback.format_exc()[-4000:]}
        emit(info)
        if run_dir:
            write_fatal_marker(run_dir, rank, info)
        raise
    finally:
        if runtime is not None:
            runtime.destroy()
        if dist.is_initialized() and world > 1:
            dist.destroy_process_group()


def train(argv_or_spec: Sequence[str] | RunSpec | None = None) -> dict:
    """Public entry: a RunSpec, or dllm-train style arguments (`--config train.yaml --flag value`)."""
    if isinstance(argv_or_spec, RunSpec):
        return run_training(argv_or_spec)
    return main(argv_or_spec)


def main(argv: Sequence[str] | None = None):
    ap = build_run_spec_arg_parser("dllm-train")
    args = ap.parse_args(list(sys.argv[1:] if argv is None else argv))
    if args.print_supported_configs:
        from ..models.registry import describe_supported_configs

        print(json.dumps(describe_supported_configs(), indent=1))
        return {}
    try:
        spec = run_spec_from_args(args)
        spec.validate()
    except RunSpecError as e:
        print(f"error: {e}", file=sys.stderr)
        raise SystemExit(2)
    if args.print_config:
        print(spec.to_yaml())
        return {}
    if args.validate_only:
        print(json.dumps({"valid": True, "model_id": spec.model.id, "objective": spec.objective.name}))
        return {}
    return run_training(spec)


if __name__ == "__main__":
    main()
