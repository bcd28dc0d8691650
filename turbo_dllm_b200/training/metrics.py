"""Rank-0 experiment logging to Weights & Biases (optional dependency) with sanitised ids/tags.

Counterpart of dllm_parallel/training/metrics.py:35-393. When `wandb` is not installed or
`logging.wandb_mode=disabled`, the logger is a no-op that still accepts every call.
"""
from __future__ import annotations

import os
import re
import time
from typing import Any, Mapping

FAILED_STATES = ("failed", "crashed", "killed")
DEFAULT_POLL_TIMEOUT_S = 900
DEFAULT_POLL_INTERVAL_S = 30

_ID_RE = re.compile(r"[^A-Za-z0-9_.-]+")


def sanitize_wandb_id(value: str, max_len: int = 64) -> str:
    out = _ID_RE.sub("-", value.strip()).strip("-.")
    return out[:max_len] or "run"


def sanitize_wandb_tags(tags) -> list[str]:
    seen, out = set(), []
    for t in tags or ():
        t = _ID_RE.sub("-", str(t).strip())[:64].strip("-")
        if t and t not in seen:
            seen.add(t)
            out.append(t)
    return out


def flatten_event(event: dict, prefix: str = "") -> dict:
    flat = {}
    for k, v in event.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict):
            flat.update(flatten_event(v, key + "/"))
        elif isinstance(v, (int, float)) and not isinstance(v, bool):
            flat[key] = v
    return flat


def resolve_run_id(configured_id: str | None, run_name: str | None, env: Mapping[str, str] | None = None) -> str | None:
    """The id a (possibly requeued) job logs under: WANDB_RUN_ID wins, then the configured id, then the run name,
    so that a restarted job continues its own run instead of opening a new one."""
    env = os.environ if env is None else env
    if env.get("WANDB_RUN_ID"):
        return sanitize_wandb_id(env["WANDB_RUN_ID"])
    if configured_id:
        return sanitize_wandb_id(configured_id)
    return sanitize_wandb_id(run_name) if run_name else None


def resolve_resume(env: Mapping[str, str] | None = None) -> str:
    """W&B resume mode: WANDB_RESUME, else `allow` (safe under preemption)."""
    env = os.environ if env is None else env
    return env.get("WANDB_RESUME") or "allow"


def _tag(value: object) -> str:
    text = str(value).strip()
    return re.sub(r"\s+", "_", text) if text else "unset"


def config_tags(config: Mapping[str, Any] | None) -> list[str]:
    """Stable tags from the run's own fields: model size fields, block size, learning rate, and the parallel layout
    when any model-parallel axis is used."""
    config = config or {}
    tags: list[str] = []
    model, objective = config.get("model"), config.get("objective")
    optimizer, topo = config.get("optimizer"), config.get("topology")
    if isinstance(model, Mapping):
        for key in ("seq_len", "hidden_size", "num_layers"):
            if model.get(key) is not None:
                tags.append(f"{key}:{_tag(model[key])}")
    if isinstance(objective, Mapping):
        if objective.get("name") is not None:
            tags.append(f"objective:{_tag(objective['name'])}")
        if objective.get("block_size") is not None:
            tags.append(f"block_size:{_tag(objective['block_size'])}")
    if isinstance(optimizer, Mapping) and optimizer.get("lr") is not None:
        tags.append(f"lr:{_tag(optimizer['lr'])}")
    if isinstance(topo, Mapping):
        cp, bp, tp, ep = (int(topo.get(k, 1) or 1) for k in ("context_parallel_size", "block_parallel_size",
                                                            "tensor_parallel_size", "expert_parallel_size"))
        if max(cp, bp, tp, ep) > 1:
            tags += ["parallel:topology", f"active_blocks:{'dual_end' if bp > 1 else 'all_blocks'}",
                     f"kv_backend:{'ring' if cp > 1 else 'replicated'}", f"cp:{cp}", f"bp:{bp}", f"tp:{tp}", f"ep:{ep}"]
    return list(dict.fromkeys(t[:64] for t in tags))


def default_run_name(config: Mapping[str, Any] | None) -> str:
    config = config or {}
    model = config.get("model") if isinstance(config.get("model"), Mapping) else {}
    topo = config.get("topology") if isinstance(config.get("topology"), Mapping) else {}
    cp, bp, tp, ep = (int(topo.get(k, 1) or 1) for k in ("context_parallel_size", "block_parallel_size",
                                                        "tensor_parallel_size", "expert_parallel_size"))
    return sanitize_wandb_id(f"{model.get('id', 'dllm')}-{model.get('seq_len', 'seq')}-cp{cp}-bp{bp}-tp{tp}-ep{ep}")


def poll_runs(*, entity: str, project: str, run_ids: list[str], min_step: int = 0,
              timeout_s: float = DEFAULT_POLL_TIMEOUT_S, poll_interval_s: float = DEFAULT_POLL_INTERVAL_S,
              api=None, sleep=time.sleep, clock=time.time) -> dict[str, dict]:
    """Polls W&B until every run id has reached `min_step` without being in a failed state, or the time runs out.
    Returns the last seen state per run: state, step, url, loss and the throughput / MFU summary fields. Without
    the wandb package every run is reported `unmonitored`."""
    if api is None:
        try:
            import wandb
        except ModuleNotFoundError:
            return {r: {"state": "unmonitored", "error": "wandb is not installed"} for r in run_ids}
        api = wandb.Api()
    deadline = clock() + timeout_s
    states: dict[str, dict] = {r: {"state": "pending"} for r in run_ids}
    while True:
        healthy = 0
        for r in run_ids:
            try:
                run = api.run(f"{entity}/{project}/{r}")
                summary = dict(run.summary)
                step = int(summary.get("step/step", summary.get("summary/steps", summary.get("step", summary.get("_step", -1)))))
                state = getattr(run, "state", None)
                states[r] = {"state": state, "step": step, "url": getattr(run, "url", None),
                             "loss": summary.get("step/loss", summary.get("loss")),
                             "input_tokens_per_second": summary.get("summary/input_tokens_per_second",
                                                                    summary.get("step/perf/input_tokens_per_second")),
                             "mfu_pct": summary.get("summary/mfu_pct")}
                if step >= min_step and state not in FAILED_STATES:
                    healthy += 1
            except Exception as e:     # the API raises its own error types for runs that do not exist yet
                states[r] = {"state": "pending", "error": type(e).__name__}
        if healthy == len(run_ids) or clock() >= deadline:
            return states
        sleep(poll_interval_s)


class WandBRunLogger:
    def __init__(self, spec, rank: int, config: dict | None = None, module=None):
        lg = spec.logging
        self.enabled = bool(lg.wandb) and rank == 0 and lg.wandb_mode != "disabled"
        self.run = None
        if not self.enabled:
            return
        try:
            wandb = module if module is not None else __import__("wandb")
        except ImportError:
            self.enabled = False
            return
        cfg = config or spec.to_dict()
        name = lg.wandb_name or default_run_name(cfg)
        self.run = wandb.init(project=lg.wandb_project, entity=lg.wandb_entity, name=name,
                              group=lg.wandb_group, id=resolve_run_id(lg.wandb_id, lg.wandb_name),
                              mode=lg.wandb_mode, dir=lg.wandb_dir,
                              tags=sanitize_wandb_tags(lg.wandb_tags) + config_tags(cfg),
                              config=cfg, resume=resolve_resume())

    def log_event(self, event: dict) -> None:
        if self.run is None:
            return
        step = event.get("step")
        payload = flatten_event({k: v for k, v in event.items() if k not in ("event", "config")},
                                prefix=f"{event.get('event', 'event')}/")
        self.run.log(payload, step=step)

    def log_summary(self, summary: dict) -> None:
        """The run's final figures go to the W&B summary (what `poll_runs` and dashboards read), not the history."""
        if self.run is None:
            return
        flat = flatten_event({k: v for k, v in summary.items() if k not in ("event", "run_context")}, prefix="summary/")
        try:
            self.run.summary.update(flat)
        except AttributeError:
            self.run.log(flat)

    def finish(self, exit_code: int = 0) -> None:
        if self.run is not None:
            self.run.finish(exit_code=exit_code)
            self.run = None
