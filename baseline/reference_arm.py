"""`bench.py --impl reference`: runs the UNMODIFIED reference package installed under
baseline/_ref through its own public API (`dllm_parallel.train(["--config", recipe])`, the same
call `dllm-train` makes) on the benchmark's model shape, and reports the same JSON line.

Nothing of this repository's models, kernels or engine is on that path: this file only writes
a Hugging Face model directory with random-init weights of the named shape (the reference loads
models with `from_pretrained`), a recipe YAML, and parses the reference trainer's `summary`
event. If the reference cannot run on this machine the line is
`{"impl": "reference", "unavailable": "<why>"}`.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

SHAPES = {
    "synthetic:qwen3-8b": dict(hidden_size=4096, num_hidden_layers=36, num_attention_heads=32,
                               num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                               vocab_size=151936, tie_word_embeddings=False),
    "synthetic:qwen3-1.7b": dict(hidden_size=2048, num_hidden_layers=28, num_attention_heads=16,
                                 num_key_value_heads=8, head_dim=128, intermediate_size=6144,
                                 vocab_size=151936, tie_word_embeddings=True),
    "synthetic:tiny-hd128": dict(hidden_size=512, num_hidden_layers=2, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=128, intermediate_size=1024,
                                 vocab_size=2048, tie_word_embeddings=False),
}

_MAKE_MODEL = r"""
import sys, json, torch
from transformers import Qwen3Config, Qwen3ForCausalLM
shape = json.loads(sys.argv[1]); out = sys.argv[2]
cfg = Qwen3Config(rope_theta=1e6, rms_norm_eps=1e-6, max_position_embeddings=262144, **shape)
torch.manual_seed(0)
dev = "cuda" if torch.cuda.is_available() else "cpu"
with torch.device(dev):
    model = Qwen3ForCausalLM(cfg).to(torch.bfloat16)
model.save_pretrained(out, safe_serialization=True)
print("saved", out)
"""

_RUN_REF = r"""
import sys
sys.path.insert(0, sys.argv[1])
import dllm_parallel
dllm_parallel.train(["--config", sys.argv[2]])
"""


def _recipe(model_dir, shape, seq_len, block_size, batch, steps, warmup, mask_id):
    return {
        "launch": {"recipe_kind": "smoke"},
        "model": {"id": model_dir, "family": "causal_lm", "seq_len": seq_len, "mask_token_id": mask_id,
                  "dtype": "bf16"},
        "objective": {"name": "fast_dllm_v2", "block_size": block_size, "noise_schedule_epsilon": 0.1,
                      "noise_schedule": "linear_mask", "loss_weighting": "unit"},
        "data": {"input_mode": "random"},
        "training": {"batch_size": batch, "steps": steps + warmup, "activation_checkpointing": True},
        "profiler": {"warmup_steps": warmup},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1, "tensor_parallel_size": 1,
                     "sequence_parallel": False},
        "kernel": {"runtime_jit": True},
        "optimizer": {"backend": "torch_adamw", "lr": 1e-5, "gradient_clip_norm": 1.0},
    }


def _first_error(text: str) -> str:
    lines = [l.strip() for l in text.splitlines() if l.strip()]
    for l in reversed(lines):
        if any(k in l for k in ("Error", "error:", "Exception", "requires", "not supported", "unavailable")):
            return l[:300]
    return (lines[-1] if lines else "no output")[:300]


def _run_reference(recipe: dict, timeout: float, single_process: bool = False):
    """Runs the reference trainer on `recipe` in a child process. `single_process`: drop the launcher's
    rendezvous variables so that the child is a one-GPU run on this rank's device (used by the probe)."""
    import yaml

    with tempfile.NamedTemporaryFile("w", suffix=".yaml", delete=False) as f:
        yaml.safe_dump(recipe, f)
        path = f.name
    env = dict(os.environ)
    env["PYTHONPATH"] = REF + os.pathsep + env.get("PYTHONPATH", "")
    env.setdefault("DLLM_RUN_DIR", tempfile.mkdtemp(prefix="dllm_ref_run_"))
    if single_process:
        local = env.get("LOCAL_RANK", "0")
        for k in list(env):
            if k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "GROUP_RANK", "GROUP_WORLD_SIZE",
                     "MASTER_ADDR", "MASTER_PORT", "ROLE_RANK", "ROLE_WORLD_SIZE", "ROLE_NAME") or \
                    k.startswith("TORCHELASTIC_"):
                del env[k]
        env["CUDA_VISIBLE_DEVICES"] = local
    try:
        proc = subprocess.run([sys.executable, "-c", _RUN_REF, REF, path], capture_output=True, text=True,
                              timeout=timeout, env=env)
    except subprocess.TimeoutExpired:
        return None, f"reference trainer did not finish within {int(timeout)} s"
    summary = None
    for line in proc.stdout.splitlines():
        line = line.strip()
        if line.startswith("{") and '"event"' in line:
            try:
                ev = json.loads(line)
            except ValueError:
                continue
            if ev.get("event") == "summary":
                summary = ev
    if proc.returncode != 0 or summary is None:
        return None, _first_error(proc.stderr + "\n" + proc.stdout)
    return summary, None


def _find_step_ms(summary: dict):
    def walk(d):
        if isinstance(d, dict):
            if "step_time_ms" in d:
                return float(d["step_time_ms"])
            for v in d.values():
                r = walk(v)
                if r is not None:
                    return r
        return None

    return walk(summary)


def run(args) -> dict:
    base = {"impl": "reference"}
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not os.path.isdir(os.path.join(REF, "dllm_parallel")):
        return {**base, "unavailable": "baseline/_ref is empty: install the reference package there with pip --no-index --no-deps --target baseline/_ref <reference source tree>"}
    shape = SHAPES.get(args.model)
    if shape is None:
        return {**base, "unavailable": f"no Hugging Face shape for {args.model}"}
    if args.layers is not None:
        shape = {**shape, "num_hidden_layers": args.layers}
    try:
        import torch

        if not torch.cuda.is_available():
            return {**base, "unavailable": "no CUDA device (the reference trainer is CUDA-only)"}
    except Exception as e:  # pragma: no cover
        return {**base, "unavailable": f"torch import failed: {e}"}

    work = tempfile.mkdtemp(prefix="dllm_ref_model_")
    # 1) cheap probe: a one-layer model at seq 1024 shows whether the reference runs here at all
    probe_dir = os.path.join(work, "probe")
    probe_shape = {**SHAPES["synthetic:tiny-hd128"], "num_hidden_layers": 1}
    p = subprocess.run([sys.executable, "-c", _MAKE_MODEL, json.dumps(probe_shape), probe_dir],
                       capture_output=True, text=True)
    if p.returncode != 0:
        return {**base, "unavailable": "cannot build a Hugging Face Qwen3 model dir: " + _first_error(p.stderr)}
    _, err = _run_reference(_recipe(probe_dir, probe_shape, 1024, args.block_size, 1, 1, 0,
                                    probe_shape["vocab_size"] - 1), timeout=600, single_process=True)
    if err is not None:
        return {**base, "unavailable": "reference trainer refuses to run on this machine: " + err}
    # 2) the real measurement
    model_dir = os.path.join(work, "model")
    if int(os.environ.get("LOCAL_RANK", "0")) == 0:
        p = subprocess.run([sys.executable, "-c", _MAKE_MODEL, json.dumps(shape), model_dir],
                           capture_output=True, text=True)
        open(os.path.join(work, "done" if p.returncode == 0 else "failed"), "w").write(p.stderr[-2000:])
    t0 = time.time()
    while not (os.path.exists(os.path.join(work, "done")) or os.path.exists(os.path.join(work, "failed"))):
        if time.time() - t0 > 1800:
            return {**base, "unavailable": "timed out writing random-init weights"}
        time.sleep(1)
    if os.path.exists(os.path.join(work, "failed")):
        return {**base, "unavailable": "cannot write random-init weights: " + _first_error(open(os.path.join(work, "failed")).read())}
    summary, err = _run_reference(_recipe(model_dir, shape, args.seq_len, args.block_size, args.batch_per_gpu,
                                          args.steps, args.warmup, shape["vocab_size"] - 1), timeout=3 * 3600)
    if err is not None:
        return {**base, "unavailable": "reference trainer failed on the benchmark config: " + err}
    ms = _find_step_ms(summary)
    if ms is None:
        return {**base, "unavailable": "reference summary event carries no step_time_ms"}
    if rank != 0:
        return {**base, "rank": rank}
    tokens = args.batch_per_gpu * args.seq_len * world
    return {**base, "metric": "train tokens/sec (box, max over ranks) + MFU, Qwen3-8B shape 32k-128k ctx, 1/2/4/8 GPU",
            "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
            "config": {"model": args.model, "global_batch": args.batch_per_gpu * world, "seq_len": args.seq_len,
                       "parallelism": f"dp{world}", "optimizer_backend": summary.get("optimizer_backend")}}
