"""`dllm dflash …`: prepare-features, build-draft-vocab, export, validate-export, validate-vllm, serve-sglang, serve-vllm,
verify-sglang, verify-vllm (cf. dllm_parallel/cli/dflash.py:13-110)."""
from __future__ import annotations

import argparse
import json
import shlex
import sys


def run_dflash(argv) -> int:
    from ..config.run_spec import RunSpecError, load_run_spec
    from ..models import export as ex
    from ..serving import dflash_servers as srv

    ap = argparse.ArgumentParser(prog="dllm dflash")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("prepare-features", help="run the frozen target over a dataset and store hidden states")
    p.add_argument("--config", required=True)
    p.add_argument("--output", required=True)
    p.add_argument("--batches", type=int, default=8)
    p.add_argument("--resume", action="store_true", help="keep records that are already written and verified")
    p = sub.add_parser("build-draft-vocab", help="t2d / d2t maps of the most frequent tokens of a prepared dataset")
    p.add_argument("--dataset", required=True, help="prepared artifact directory (tokens.i32)")
    p.add_argument("--size", type=int, required=True, help="draft vocabulary size")
    p.add_argument("--verifier-vocab-size", type=int, required=True)
    p.add_argument("--keep-ids", type=int, nargs="*", default=[], help="ids kept whatever their frequency (eos, ...)")
    p.add_argument("--output", required=True)
    p = sub.add_parser("export")
    p.add_argument("--config", required=True)
    p.add_argument("--checkpoint", required=True)
    p.add_argument("--output", required=True)
    p.add_argument("--format", choices=("native", "speculators"), default="native",
                   help="speculators: module-style tensor names with the verifier's embedding and head (DFlash drafter)")
    p = sub.add_parser("validate-export")
    p.add_argument("path")
    p.add_argument("--block-size", type=int, default=None, help="the block size the export must carry")
    p = sub.add_parser("validate-vllm", help="check an exported drafter against what the vLLM loader reads")
    p.add_argument("path")
    p.add_argument("--block-size", type=int, default=None)
    for name in ("serve-sglang", "serve-vllm"):
        p = sub.add_parser(name, help="print (default) or start the server command for an exported drafter")
        p.add_argument("--target-model", required=True)
        p.add_argument("--draft", required=True)
        p.add_argument("--port", type=int, default=None)
        p.add_argument("--host", default="127.0.0.1")
        p.add_argument("--tp", type=int, default=1)
        p.add_argument("--block-size", type=int, default=16, help="the drafter's training block size")
        p.add_argument("--num-speculative-tokens", type=int, default=None,
                       help="deprecated: derived from --block-size (block_size - 1)")
        p.add_argument("--memory-fraction", type=float, default=None)
        p.add_argument("--max-model-len", type=int, default=None)
        p.add_argument("--launch", action="store_true", help="start the server and wait until it answers")
        p.add_argument("--ready-timeout", type=float, default=1800.0)
        p.add_argument("--log", default=None)
        p.add_argument("--skip-export-check", action="store_true")
    for name in ("verify-sglang", "verify-vllm"):
        p = sub.add_parser(name, help="gate a running server on one deterministic completion")
        p.add_argument("--base-url", required=True)
        p.add_argument("--model", required=True)
        p.add_argument("--min-acceptance-length", type=float, default=1.5)
        p.add_argument("--prompt", default=None)
        p.add_argument("--expected-text", default=None, help="the target model's own greedy continuation of the prompt")
        p.add_argument("--block-size", type=int, default=16)
        p.add_argument("--tokenizer", default=None, help="tokenizer directory (default: whitespace tokens)")
    a = ap.parse_args(argv)
    try:
        if a.cmd == "prepare-features":
            from ..data.dflash_features import capture_features

            # under torchrun every rank captures its share of the records and rank 0 writes the manifest
            import os

            rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
            barrier = None
            if world > 1:
                import torch
                import torch.distributed as dist

                if not dist.is_initialized():
                    dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
                barrier = dist.barrier
            man = capture_features(load_run_spec(a.config).validate(), a.output, a.batches, rank=rank, world=world,
                                   barrier=barrier, resume=a.resume)
            if rank == 0:
                print(json.dumps(man))
            return 0
        if a.cmd == "build-draft-vocab":
            import os

            import numpy as np
            import torch

            from ..models.dflash import DraftVocabulary

            toks = np.memmap(os.path.join(a.dataset, "tokens.i32"), dtype="<i4", mode="r")
            counts = np.bincount(toks, minlength=a.verifier_vocab_size)
            if counts.size > a.verifier_vocab_size:
                raise ValueError(f"the dataset holds token id {counts.size - 1}, outside a vocabulary of {a.verifier_vocab_size}")
            if not 0 < a.size <= a.verifier_vocab_size:
                raise ValueError("--size must be in (0, verifier vocabulary size]")
            counts = counts.astype(np.int64)
            counts[list(a.keep_ids)] = np.iinfo(np.int64).max
            order = np.argsort(-counts, kind="stable")[: a.size]      # ties: the lower id first
            dv = DraftVocabulary.from_ids(torch.from_numpy(order.copy()), a.verifier_vocab_size)
            dv.save(a.output)
            covered = float(np.minimum(counts[order], toks.size).sum() / max(toks.size, 1)) if not a.keep_ids else None
            print(json.dumps({"output": a.output, "draft_vocab_size": dv.size, "token_coverage": covered}))
            return 0
        if a.cmd == "export":
            from ..checkpoint import load_model_weights, load_training_checkpoint, read_metadata
            from ..training.session import TrainingSession

            import torch

            from ..models import hf_loader

            spec = load_run_spec(a.config).validate()
            if not torch.cuda.is_available() and spec.model.dtype != "fp32":
                # no GPU here: the drafter is rebuilt in fp32 and its tensors are written in the run's dtype
                hf_loader.EXPORT_DTYPE = {"bf16": torch.bfloat16, "fp16": torch.float16}[spec.model.dtype]
                spec = spec.with_overrides({"model": {"dtype": "fp32"}})
            if int(read_metadata(a.checkpoint)["world_size"]) > 1:
                # a drafter trained on several ranks: the weights are replicated, one process reads rank 0's file
                spec = spec.with_overrides({"topology": {"context_parallel_size": 1, "block_parallel_size": 1}})
                s = TrainingSession(spec)
                load_model_weights(a.checkpoint, "latest", s)
            else:
                s = TrainingSession(spec)
                load_training_checkpoint(a.checkpoint, "latest", s, rank=0, world_size=1, restore_rng=False)
            try:
                if a.format == "speculators":
                    man = ex.export_speculators_checkpoint(s.model, s.task.target, spec, a.output)
                else:
                    man = ex.export_dflash_drafter(s.model, spec, a.output)
            finally:
                hf_loader.EXPORT_DTYPE = None
            print(json.dumps({"files": sorted(man["files"])}))
            return 0
        if a.cmd == "validate-export":
            import os

            # a DFlash2 export carries config.json with its architecture; check its tensor inventory too
            is_v2 = os.path.exists(os.path.join(a.path, "config.json"))
            problems = ex.validate_dflash2_export(a.path) if is_v2 else ex.validate_dflash_export(a.path)
            if a.block_size is not None and is_v2 and not problems:
                try:
                    srv.validate_export_for_server(a.path, "sglang", a.block_size)
                except ValueError as e:
                    problems = [str(e)]
            print(json.dumps({"ok": not problems, "problems": problems}))
            return 0 if not problems else 1
        if a.cmd == "validate-vllm":
            problems = ex.validate_dflash2_export(a.path)
            if problems:
                print(json.dumps({"ok": False, "problems": problems}))
                return 1
            print(json.dumps({"ok": True, **srv.validate_export_for_server(a.path, "vllm", a.block_size)}))
            return 0
        if a.cmd in ("serve-sglang", "serve-vllm"):
            backend = "sglang" if a.cmd == "serve-sglang" else "vllm"
            block = a.block_size if a.num_speculative_tokens is None else a.num_speculative_tokens + 1
            cfg = srv.ServerConfig.from_mapping({
                "backend": backend, "target_model": a.target_model, "draft_export": a.draft, "block_size": block,
                "host": a.host, "port": a.port, "tensor_parallel_size": a.tp, "memory_fraction": a.memory_fraction,
                "max_model_len": a.max_model_len})
            cmd = cfg.command()
            if not a.launch:
                print(" ".join(shlex.quote(c) for c in cmd))
                return 0
            srv.require_server_version(backend)
            if not a.skip_export_check:
                print(json.dumps(srv.validate_export_for_server(a.draft, backend, block)))
            server = srv.ServerProcess(cmd, cfg.url, log_path=a.log).start()
            try:
                models = server.wait_ready(a.ready_timeout)
                print(json.dumps({"event": "ready", "url": cfg.url, "pid": server.proc.pid,
                                  "models": [m.get("id") for m in models.get("data", [])]}), flush=True)
                return server.proc.wait()
            except KeyboardInterrupt:
                return 130
            finally:
                server.stop()
        if a.prompt is not None and a.expected_text is not None:
            encode = str.split
            if a.tokenizer:
                from transformers import AutoTokenizer

                tok = AutoTokenizer.from_pretrained(a.tokenizer)
                encode = lambda t: tok.encode(t, add_special_tokens=False)
            res = srv.verify_server(server_url=a.base_url, model=a.model, prompt=a.prompt,
                                    expected_text=a.expected_text, encode=encode, block_size=a.block_size)
            print(json.dumps(res))
            return 0 if res["passed"] else 1
        res = srv.verify_acceptance(a.base_url, a.model, ["The capital of France is", "def fib(n):"],
                                    a.min_acceptance_length)
        print(json.dumps(res))
        return 0 if res["ok"] else 1
    except (RunSpecError, FileNotFoundError, ValueError, OSError, RuntimeError, TimeoutError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
