"""Rank-0 experiment logging to Weights & Biases (optional dependency) with sanitised ids/tags.

Counterpart of dllm_parallel/training/metrics.py:35-393. When `wandb` is not installed or
`logging.wandb_mode=disabled`, the logger is a no-op that still accepts every call.
"""
from __future__ import annotations

import re

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
        self.run = wandb.init(project=lg.wandb_project, entity=lg.wandb_entity, name=lg.wandb_name,
                              group=lg.wandb_group, id=sanitize_wandb_id(lg.wandb_id) if lg.wandb_id else None,
                              mode=lg.wandb_mode, dir=lg.wandb_dir, tags=sanitize_wandb_tags(lg.wandb_tags),
                              config=config or spec.to_dict(), resume="allow")

    def log_event(self, event: dict) -> None:
        if self.run is None:
            return
        step = event.get("step")
        payload = flatten_event({k: v for k, v in event.items() if k not in ("event", "config")},
                                prefix=f"{event.get('event', 'event')}/")
        self.run.log(payload, step=step)

    def finish(self, exit_code: int = 0) -> None:
        if self.run is not None:
            self.run.finish(exit_code=exit_code)
            self.run = None
