"""`dllm init DIR`: writes a starter project (prepare.yaml, train.yaml, README.md, .gitignore)
without overwriting anything; a failure removes the files created so far
(cf. dllm_parallel/cli/init.py:21-264)."""
from __future__ import annotations

import argparse
import os
import sys

PREPARE_YAML = """format: dllm.data.prepare.v1
source:
  type: jsonl            # jsonl | text | parquet | huggingface | pretokenized
  path: data/raw.jsonl   # relative to this file; a directory or a glob works too
records:
  type: text             # text | messages | prompt_completion | pretokenized
  text_field: text
tokenizer:
  model: byte            # or a local Hugging Face tokenizer directory
  add_eos: true
supervision:
  policy: full           # full | assistant_only | completion_only | provided
packing:
  maximum_length: 4096
  overflow: split        # reject | split | truncate_left | truncate_right
output:
  path: data/prepared
  format: auto           # packed stream for full supervision, indexed samples otherwise
"""

TRAIN_YAML = """launch:
  recipe_kind: smoke
model:
  id: synthetic:tiny-hd128       # a built-in shape preset; see `dllm-train --print-supported-configs`
  seq_len: 4096
  dtype: bf16
objective:
  name: fast_dllm_v2
  block_size: 32
  noise_schedule_epsilon: 0.1
data:
  input_mode: dataset
  dataset_path: data/prepared
training:
  batch_size: 1
  steps: 100
  activation_checkpointing: true
topology:
  context_parallel_size: 1
  block_parallel_size: 1
optimizer:
  lr: 1.0e-5
  gradient_clip_norm: 1.0
checkpointing:
  save_checkpoint_dir: checkpoints
  save_checkpoint_interval: 50
  keep_last_n: 2
  auto_resume: true
"""

README = """# {name}

1. put JSON-lines records with a `text` field in `data/raw.jsonl`
2. `dllm data prepare --config prepare.yaml`
3. `dllm doctor --config train.yaml`
4. `dllm launch --config train.yaml --nproc-per-node 1`
"""

GITIGNORE = "data/prepared/\ncheckpoints/\nruns/\n"


def initialize_project(directory: str) -> list[str]:
    os.makedirs(directory, exist_ok=True)
    files = {"prepare.yaml": PREPARE_YAML, "train.yaml": TRAIN_YAML,
             "README.md": README.format(name=os.path.basename(os.path.abspath(directory))), ".gitignore": GITIGNORE}
    existing = [n for n in files if os.path.exists(os.path.join(directory, n))]
    if existing:
        raise FileExistsError(f"refusing to overwrite {', '.join(existing)} in {directory}")
    created = []
    try:
        for name, text in files.items():
            path = os.path.join(directory, name)
            fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o644)
            with os.fdopen(fd, "w") as f:
                f.write(text)
            created.append(path)
    except Exception:
        for p in created:
            try:
                os.unlink(p)
            except OSError:
                pass
        raise
    return created


def run_init(argv) -> int:
    ap = argparse.ArgumentParser(prog="dllm init")
    ap.add_argument("directory", nargs="?", default=".")
    a = ap.parse_args(argv)
    try:
        for p in initialize_project(a.directory):
            print(p)
        return 0
    except FileExistsError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
