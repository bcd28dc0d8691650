import gzip
import json

import pytest
import torch


def test_release_gates_pass_on_this_tree():
    from turbo_dllm_b200.profiling.release_gates import run_gates

    res = run_gates()
    assert all(r.ok for r in res), [(r.name, r.detail) for r in res if not r.ok]


def test_communication_labels_roundtrip_and_trace_summary(tmp_path):
    from turbo_dllm_b200.profiling.operator_trace import communication_label, parse_communication_label
    from turbo_dllm_b200.profiling.trace_analysis import analyze_kineto_trace, classify_kernel

    lab = communication_label("context_parallel", "forward", "all_gather", 1024, 8192)
    assert parse_communication_label(lab) == {"domain": "context_parallel", "phase": "forward",
                                              "collective": "all_gather", "input_bytes": 1024, "logical_bytes": 8192}
    assert classify_kernel("tdllm::gemm_bf16_kernel(...)") == "dense_gemm"
    assert classify_kernel("attn_dkv::attn_bwd_dkv_kernel") == "attention_bwd"
    assert classify_kernel("ncclDevKernel_AllGather_RING_LL") == "nccl"
    events = [{"ph": "X", "cat": "kernel", "name": "tdllm::gemm_bf16_kernel", "ts": 0, "dur": 100},
              {"ph": "X", "cat": "kernel", "name": "ncclDevKernel_AllGather", "ts": 50, "dur": 100},
              {"ph": "X", "cat": "user_annotation", "name": lab, "ts": 50, "dur": 100}]
    p = tmp_path / "rank_0.trace.json.gz"
    with gzip.open(p, "wt") as f:
        json.dump({"traceEvents": events}, f)
    s = analyze_kineto_trace(str(p))
    assert s["exposed_communication_us"] == 50.0
    assert s["communication_labels"]["context_parallel/forward/all_gather"]["logical_bytes"] == 8192


def test_scopes_are_inert_outside_a_trace_window():
    import contextlib

    from turbo_dllm_b200.profiling.operator_trace import communication_scope, operator_scope

    assert isinstance(operator_scope("x"), contextlib.nullcontext)
    assert isinstance(communication_scope("a", "b", "c"), contextlib.nullcontext)


def test_wandb_sanitising_and_fake_module():
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.training.metrics import WandBRunLogger, sanitize_wandb_id, sanitize_wandb_tags

    assert sanitize_wandb_id(" my run/№1 ") == "my-run-1"
    assert sanitize_wandb_tags(["a b", "a b", "", "x"]) == ["a-b", "x"]

    class Run:
        def __init__(self):
            self.logged, self.finished = [], False

        def log(self, payload, step=None):
            self.logged.append((step, payload))

        def finish(self, exit_code=0):
            self.finished = True

    class Fake:
        def __init__(self):
            self.kw, self.run = None, Run()

        def init(self, **kw):
            self.kw = kw
            return self.run

    spec = RunSpec.from_mapping({"logging": {"wandb": True, "wandb_mode": "offline", "wandb_tags": ["t 1"],
                                             "wandb_id": "id!"}})
    fake = Fake()
    lg = WandBRunLogger(spec, 0, module=fake)
    lg.log_event({"event": "step", "step": 3, "loss": 1.5, "perf": {"tps": 10.0}, "note": "x"})
    lg.finish()
    assert fake.kw["tags"][0] == "t-1" and "seq_len:1024" in fake.kw["tags"] and fake.kw["id"] == "id"
    assert fake.kw["resume"] == "allow" and fake.kw["name"].startswith("nvidia-Nemotron-Labs-Diffusion-3B-1024-cp")
    assert fake.run.logged == [(3, {"step/step": 3, "step/loss": 1.5, "step/perf/tps": 10.0})] and fake.run.finished
    assert WandBRunLogger(spec, 1, module=fake).run is None


def test_bundle_catalog_selection_and_hash_check(tmp_path):
    from turbo_dllm_b200.kernels import bundle_manifest as bm

    wheel = tmp_path / "turbo_dllm_b200-0.1.0-cp312-linux_x86_64.whl"
    wheel.write_bytes(b"not really a wheel")
    env = {"python": "cp312", "cuda": "128", "arch": "sm100"}
    cat = {"format": bm.CATALOG_FORMAT, "bundles": [{"key": bm.bundle_key(env), "assets": [
        {"name": wheel.name, "url": str(wheel), "sha256": bm._sha256(str(wheel))}]}]}
    path = tmp_path / "catalog.json"
    path.write_text(json.dumps(cat))
    b = bm.select_bundle(bm.load_catalog(str(path)), env)
    out = bm.fetch_asset(b["assets"][0], str(tmp_path / "dl") if (tmp_path / "dl").mkdir() is None else "")
    assert out.endswith(".whl")
    b["assets"][0]["sha256"] = "0" * 64
    with pytest.raises(bm.BundleError, match="sha256"):
        bm.fetch_asset(b["assets"][0], str(tmp_path / "dl"))
    with pytest.raises(bm.BundleError, match="no bundle"):
        bm.select_bundle(cat, {"python": "cp39", "cuda": "118", "arch": "sm80"})


def test_hf_export_and_reload_roundtrip(tmp_path):
    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.dense import BlockDiffusionTransformer
    from turbo_dllm_b200.models.hf_loader import export_hf_checkpoint, load_hf_config, load_hf_weights

    cfg = PRESETS["synthetic:tiny-qwen3"]
    a = BlockDiffusionTransformer(cfg, dtype=torch.float32, seed=5)
    export_hf_checkpoint(a, str(tmp_path / "hf"))
    cfg2 = load_hf_config(str(tmp_path / "hf"))
    assert cfg2.hidden_size == cfg.hidden_size and cfg2.num_key_value_heads == cfg.num_key_value_heads and cfg2.qk_norm
    b = BlockDiffusionTransformer(cfg2, dtype=torch.float32, seed=99)
    load_hf_weights(b, str(tmp_path / "hf"))
    assert torch.equal(a.flat.data, b.flat.data)


def test_serving_command_builders_and_acceptance_parsing():
    from turbo_dllm_b200.serving import dflash_servers as srv

    cmd = srv.build_vllm_command(target_model="T", draft_export="D", num_speculative_tokens=7)
    assert cmd[:3] == ["vllm", "serve", "T"] and json.loads(cmd[4])["num_speculative_tokens"] == 7
    assert "--speculative-draft-model-path" in srv.build_sglang_command(target_model="T", draft_export="D")
    assert srv.parse_acceptance_length("vllm:spec_decode_mean_acceptance_length 2.75\n") == 2.75
    txt = "spec_decode_num_accepted_tokens_total 30\nspec_decode_num_drafts_total 20\n"
    assert srv.parse_acceptance_length(txt) == 2.5
    res = srv.verify_acceptance("http://x", "m", ["p"], 2.0, post=lambda u, p: {}, fetch_metrics=lambda: txt)
    assert res["ok"] and res["acceptance_length"] == 2.5


def test_fault_marker_and_doctor(tmp_path):
    from turbo_dllm_b200.diagnostics import inspect_training_runtime
    from turbo_dllm_b200.training.fault_tolerance import fatal_marker_path, write_fatal_marker

    p = write_fatal_marker(str(tmp_path), 3, {"event": "fatal_exception", "error": "boom"})
    assert p == fatal_marker_path(str(tmp_path), 3) and p.endswith("fatal_rank_00003.json")
    assert json.load(open(p))["error"] == "boom"
    rep = inspect_training_runtime(portable_only=True)
    assert rep.ready and any(c.name == "torch" for c in rep.checks)


def test_launch_command_and_environment(tmp_path):
    import argparse

    from turbo_dllm_b200.cli.launch import (add_launch_arguments, build_launch_command, build_launch_environment,
                                            parse_nnodes, require_idle_assigned_gpus)
    from turbo_dllm_b200.config.run_spec import RunSpecError

    ap = argparse.ArgumentParser()
    add_launch_arguments(ap)
    a = ap.parse_args(["--config", "t.yaml", "--nproc-per-node", "8", "--max-restarts", "2"])
    cmd = build_launch_command(a, "t.yaml", ["--steps", "5"])
    assert "torch.distributed.run" in cmd and "--nproc-per-node=8" in cmd and "--max-restarts=2" in cmd
    assert cmd[-4:] == ["--config", "t.yaml", "--steps", "5"]
    a1 = ap.parse_args(["--config", "t.yaml"])
    assert build_launch_command(a1, "t.yaml", [])[1:3] == ["-m", "turbo_dllm_b200.training"]
    with pytest.raises(RunSpecError, match="rdzv"):
        build_launch_command(ap.parse_args(["--config", "t.yaml", "--nnodes", "1:2"]), "t.yaml", [])
    assert parse_nnodes("2:4") == (2, 4)
    env = build_launch_environment(ap.parse_args(["--config", "t", "--run-dir", str(tmp_path)]), base_env={})
    assert env["DLLM_RUN_DIR"] == str(tmp_path) and env["PYTORCH_CUDA_ALLOC_CONF"] == "expandable_segments:True"

    class R:
        returncode, stdout, stderr = 0, "GPU-1, 123, 400 MiB\n", ""

    with pytest.raises(RunSpecError, match="not idle"):
        require_idle_assigned_gpus(1, command_runner=lambda cmd: R())


def test_execution_facade_and_launch_wrappers():
    import os

    from turbo_dllm_b200.training.execution import Execution, execution_for

    assert execution_for(None, 4, 2).data_parallel_rank == 2
    assert execution_for(None, 4, 2).active_block_mode == "all_blocks"
    assert Execution(block_parallel_size=4).active_block_mode == "dual_end"
    here = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "turbo_dllm_b200", "cli")
    for name in ("torchrun.sh", "slurm.sh"):
        text = open(os.path.join(here, name)).read()
        assert "turbo_dllm_b200.cli.main launch" in text and os.access(os.path.join(here, name), os.X_OK)


def test_family_executors_and_registration():
    """Every family has an executor with capabilities, the session goes through it, and a new family plugs in by
    registering one (no edit of the session)."""
    import torch

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.models import contracts as c
    from turbo_dllm_b200.models.registry import (FAMILY_OBJECTIVES, executor_for_family, register_executor,
                                                 supported_families)
    from turbo_dllm_b200.training.session import TrainingSession

    for fam in supported_families():
        ex = executor_for_family(fam)
        assert isinstance(ex, c.BackboneExecutor) and ex.family.name == fam
        assert ex.family.objectives == FAMILY_OBJECTIVES[fam]
    assert executor_for_family("causal_lm").capabilities.parameter_sharding
    assert executor_for_family("qwen3_8").capabilities.tensor_parallel
    assert executor_for_family("qwen3_8").capabilities.sequence_parallel
    assert executor_for_family("diffusion_gemma").capabilities.tensor_parallel
    assert executor_for_family("qwen3_8").capabilities.parameter_sharding
    assert not executor_for_family("dflash").capabilities.tensor_parallel
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "num_layers": 1},
        "objective": {"name": "standard_block_diffusion", "block_size": 16},
        "training": {"batch_size": 1, "steps": 1},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1}}).validate()
    hybrid = executor_for_family("qwen3_8")
    assert not hybrid.validate_run_spec(spec.with_overrides(
        {"topology": {"tensor_parallel_size": 2}, "objective": {"name": "fast_dllm_v2"}}))
    assert not hybrid.validate_run_spec(spec.with_overrides(
        {"topology": {"tensor_parallel_size": 2, "sequence_parallel": True, "context_parallel_size": 2,
                      "block_parallel_size": 2}, "objective": {"name": "fast_dllm_v2"}}))
    assert not executor_for_family("diffusion_gemma").validate_run_spec(spec.with_overrides(
        {"topology": {"tensor_parallel_size": 2, "sequence_parallel": True}}))
    assert not hybrid.validate_run_spec(spec.with_overrides({"optimizer": {"backend": "fsdp"}, "objective": {"name": "fast_dllm_v2"},
                                                             "topology": {"tensor_parallel_size": 2}}))
    problems = executor_for_family("dflash").validate_run_spec(spec.with_overrides(
        {"topology": {"tensor_parallel_size": 2}, "objective": {"name": "dflash_distillation"}}))
    assert any("tensor-parallel" in p for p in problems)

    built = []

    class Custom(c.DenseExecutor):
        def build_model(self, ctx):
            built.append(ctx.cfg.hidden_size)
            return super().build_model(ctx)

    old = executor_for_family("causal_lm")
    try:
        register_executor("causal_lm", Custom(old.family))
        s = TrainingSession(spec, device="cpu")
        assert built == [s.cfg.hidden_size] and isinstance(s.executor, Custom)
        assert torch.isfinite(s.step().loss_sum)
        assert s.executor.parallel_work_units(spec) == 4
        assert s.executor.parameter_shard_units(s.model)[-1] == "norm_weights"
    finally:
        register_executor("causal_lm", old)


def test_portable_artifact_check_and_release_manifest(tmp_path):
    import importlib.util
    import json
    import zipfile
    from pathlib import Path

    from turbo_dllm_b200.profiling.portable_artifacts import REQUIRED_SUFFIXES, check_artifact

    def wheel(path, extra=()):
        with zipfile.ZipFile(path, "w") as z:
            for s in REQUIRED_SUFFIXES:
                z.writestr(s, "# ok\n")
            for name, data in extra:
                z.writestr(name, data)

    good = tmp_path / "turbo_dllm_b200-0.1-py3-none-any.whl"
    wheel(good)
    assert check_artifact(str(good), "portable").ok
    bad = tmp_path / "bad.whl"
    wheel(bad, [("turbo_dllm_b200/_C/libtdllm_kernels.so", b"\x7fELF"), ("turbo_dllm_b200/x.py", "p = '/root/secret'\n")])
    rep = check_artifact(str(bad), "portable")
    assert not rep.ok and any("native binary" in p for p in rep.problems) and any("forbidden" in p for p in rep.problems)
    gpu = tmp_path / "gpu.whl"
    wheel(gpu, [("turbo_dllm_b200/_C/libtdllm_kernels.so", b"\x7fELF"), ("turbo_dllm_b200/_C/native_kernels.json", "{}")])
    assert check_artifact(str(gpu), "gpu").ok
    assert not check_artifact(str(good), "gpu").ok              # the GPU wheel must carry the kernel library

    spec = importlib.util.spec_from_file_location("release", Path(__file__).resolve().parent.parent / "packaging" / "release.py")
    rel = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rel)
    dist = tmp_path / "dist"
    dist.mkdir()
    wheel(dist / "turbo_dllm_b200-0.1-cp312-linux_x86_64.whl",
          [("turbo_dllm_b200/_C/libtdllm_kernels.so", b"\x7fELF"), ("turbo_dllm_b200/_C/native_kernels.json", "{}")])
    man = rel.build_manifest(str(dist))
    assert man["bundle"] == "gpu-sm100a-cu129-cp312" and len(man["files"]) == 1
    (dist / "release_manifest.json").write_text(json.dumps(man))
    assert rel.verify(str(dist / "release_manifest.json")) == []
    with open(dist / man["files"][0]["name"], "ab") as f:
        f.write(b"tampered")
    assert any("SHA-256" in p for p in rel.verify(str(dist / "release_manifest.json")))
    assert {c["name"] for c in rel.sbom()["components"]} >= {"torch", "numpy"}


def test_wandb_run_identity_tags_and_polling():
    from turbo_dllm_b200.training import metrics as m

    assert m.resolve_run_id("cfg id", "name", env={"WANDB_RUN_ID": "env/id"}) == "env-id"
    assert m.resolve_run_id("cfg id", "name", env={}) == "cfg-id"
    assert m.resolve_run_id(None, "my name", env={}) == "my-name" and m.resolve_run_id(None, None, env={}) is None
    assert m.resolve_resume({}) == "allow" and m.resolve_resume({"WANDB_RESUME": "must"}) == "must"
    cfg = {"model": {"id": "org/Model", "seq_len": 4096, "num_layers": 2}, "objective": {"name": "fast_dllm_v2", "block_size": 32},
           "optimizer": {"lr": 1e-4}, "topology": {"context_parallel_size": 2, "block_parallel_size": 4}}
    tags = m.config_tags(cfg)
    assert {"seq_len:4096", "block_size:32", "cp:2", "bp:4", "tp:1", "active_blocks:dual_end", "kv_backend:ring",
            "parallel:topology"} <= set(tags)
    assert "parallel:topology" not in m.config_tags({"topology": {"context_parallel_size": 1}})
    assert m.default_run_name(cfg) == "org-Model-4096-cp2-bp4-tp1-ep1"

    class Run:
        def __init__(self, state, step):
            self.state, self.summary, self.url = state, {"step/step": step, "step/loss": 2.5}, "http://w/run"

    class Api:
        def __init__(self):
            self.calls = 0

        def run(self, path):
            self.calls += 1
            if path.endswith("/late") and self.calls < 4:
                raise KeyError(path)              # not created yet
            if path.endswith("/dead"):
                return Run("crashed", 50)
            return Run("running", 10 if self.calls < 6 else 120)

    now = [0.0]
    ok = m.poll_runs(entity="e", project="p", run_ids=["a", "late"], min_step=100, timeout_s=100, poll_interval_s=1,
                     api=Api(), sleep=lambda s: now.__setitem__(0, now[0] + s), clock=lambda: now[0])
    assert all(v["state"] == "running" and v["step"] >= 100 for v in ok.values()) and ok["a"]["loss"] == 2.5
    now[0] = 0.0
    bad = m.poll_runs(entity="e", project="p", run_ids=["dead"], min_step=10, timeout_s=3, poll_interval_s=1,
                      api=Api(), sleep=lambda s: now.__setitem__(0, now[0] + s), clock=lambda: now[0])
    assert bad["dead"]["state"] == "crashed" and now[0] >= 3


def test_bundle_manifest_schema_host_check_catalog_and_install(tmp_path):
    from turbo_dllm_b200.kernels import bundle_manifest as bm

    wheel = tmp_path / "turbo_dllm_b200-0.1.0-cp312-cp312-linux_x86_64.whl"
    wheel.write_bytes(b"wheel bytes")
    kw = dict(package_version="0.1.0", source_revision="abc1234", python_abi="cp312", platform="linux_x86_64",
              cuda="12.9", architectures=["10.0a"])
    man = bm.create_bundle_manifest([str(wheel)], base_url="https://example.org/r/v0.1.0", **kw)
    assert man["artifacts"][0]["url"].endswith("/" + wheel.name) and man["artifacts"][0]["size"] == 11
    host = bm.BundleEnvironment("0.1.0", "cp312", "linux_x86_64", "12.9", "10.0")
    assert bm.validate_bundle_manifest(man, host)[0]["name"] == wheel.name
    for field, value, msg in (("python_abi", "cp311", "Python ABI"), ("cuda", "12.8", "CUDA"),
                              ("package_version", "0.2.0", "package version")):
        with pytest.raises(bm.BundleError, match=msg):
            bm.validate_bundle_manifest({**man, field: value}, host)
    with pytest.raises(bm.BundleError, match="compute capability"):
        bm.validate_bundle_manifest(man, bm.BundleEnvironment("0.1.0", "cp312", "linux_x86_64", "12.9", "9.0"))
    bad = lambda **ch: {**man, "artifacts": [{**man["artifacts"][0], **ch}]}
    for change, msg in (({"url": "http://example.org/" + wheel.name}, "HTTPS"),
                        ({"url": "https://example.org/other.whl"}, "does not match"),
                        ({"sha256": "xyz"}, "SHA-256"), ({"size": 0}, "size"), ({"name": "../x.whl"}, "invalid wheel name")):
        with pytest.raises(bm.BundleError, match=msg):
            bm.validate_bundle_schema(bad(**change))
    with pytest.raises(bm.BundleError, match="duplicate"):
        bm.validate_bundle_schema({**man, "artifacts": man["artifacts"] * 2})
    with pytest.raises(bm.BundleError, match="git revision"):
        bm.validate_bundle_schema({**man, "source_revision": "not a rev"})
    # a release catalog over a local mirror: resolve for the host, verify hash and size, hand the wheel to pip
    local = bm.create_bundle_manifest([str(wheel)], base_url="file://" + str(tmp_path), allow_local=True, **kw)
    mpath = tmp_path / "bundle.json"
    mpath.write_text(json.dumps(local))
    cat = bm.create_bundle_catalog("v0.1.0", [local], [str(mpath)])
    assert bm.resolve_bundle(cat, host)["artifacts"][0]["sha256"] == local["artifacts"][0]["sha256"]
    with pytest.raises(bm.BundleError, match="has no bundle"):
        bm.resolve_bundle(cat, bm.BundleEnvironment("0.1.0", "cp310", "linux_x86_64", "12.9", "10.0"))
    calls = []
    rc = bm.install_bundle_manifest(local, host, pip_runner=lambda cmd: calls.append(cmd) or 0, allow_local=True)
    assert rc == 0 and calls[0][-1].endswith(wheel.name) and "--no-deps" in calls[0]
    wheel.write_bytes(b"tampered!!!")
    with pytest.raises(bm.BundleError, match="sha256"):
        bm.install_bundle_manifest(local, host, pip_runner=lambda cmd: 0, allow_local=True)
    assert bm.main(["validate", str(mpath), "--schema-only"]) == 2      # file:// URLs are refused outside a mirror install


def test_checked_kernel_build_is_a_separate_library(monkeypatch):
    """DLLM_KERNEL_CHECKS=1 selects the library built with -DTDLLM_KERNEL_CHECKS (index checks that record
    ERR_BAD_INDEX and skip the access); the regular library and its manifest are untouched by that build."""
    from turbo_dllm_b200.kernels import build as kb
    from turbo_dllm_b200.kernels import native

    monkeypatch.delenv("DLLM_KERNEL_CHECKS", raising=False)
    monkeypatch.delenv("TDLLM_KERNEL_CHECKS", raising=False)
    assert native.library_path().name == kb.LIB_NAME and not kb.checks_requested()
    monkeypatch.setenv("DLLM_KERNEL_CHECKS", "1")
    assert native.library_path().name == kb.CHECKED_LIB_NAME and kb.checks_requested()
    assert kb.CHECK_FLAGS == ["-DTDLLM_KERNEL_CHECKS=1"]
    src = (kb.CSRC / "common.cuh").read_text()
    assert "#ifdef TDLLM_KERNEL_CHECKS" in src and "ERR_BAD_INDEX" in src
    users = [p.name for p in kb.all_source_files() if "TD_CHECKED(" in p.read_text() and p.name != "common.cuh"]
    assert {"peer_pull.cuh", "comm.cu", "moe_dispatch.cu"} <= set(users)


def test_trace_tables_per_rank_view_and_comparison(tmp_path, capsys):
    from turbo_dllm_b200.profiling import trace_analysis as ta
    from turbo_dllm_b200.profiling.operator_trace import communication_label

    lab = communication_label("tensor", "forward", "allgather_gemm", 4_000_000, 8_000_000)

    def write(rank, gemm_us, nccl_us):
        ev = [{"ph": "X", "cat": "user_annotation", "name": "dllm.step.3", "ts": 0, "dur": 1000},
              {"ph": "X", "cat": "user_annotation", "name": "dllm.phase.forward", "ts": 0, "dur": 400},
              {"ph": "X", "cat": "kernel", "name": "tdllm::gemm_bf16_kernel<1,false>(...)", "ts": 10, "dur": gemm_us},
              {"ph": "X", "cat": "kernel", "name": "ncclDevKernel_AllReduce_Sum", "ts": 10 + gemm_us, "dur": nccl_us},
              {"ph": "X", "cat": "user_annotation", "name": lab, "ts": 10, "dur": 100}]
        p = tmp_path / f"rank_{rank}.trace.json.gz"
        with gzip.open(p, "wt") as f:
            json.dump({"traceEvents": ev}, f)
        return str(p)

    a, b = write(0, 500, 100), write(1, 700, 50)
    table = ta.format_table(ta.analyze_kineto_trace(a))
    assert "| tensor/forward/allgather_gemm | 1 | 0.10 | 4.0 | 8.0 | 80.0 |" in table      # 8 MB in 100 us
    assert "| forward | 1 | 0.4 | 40.0 % |" in table
    per = ta.analyze_directory(str(tmp_path))
    assert per["slowest_rank_by_compute"] == 1 and per["ranks"][0]["exposed_communication_ms"] == pytest.approx(0.1)
    assert per["compute_spread_pct"] == pytest.approx(40.0)
    diff = ta.compare_summaries(ta.analyze_kineto_trace(a), ta.analyze_kineto_trace(b))
    assert "| `gemm_bf16_kernel` | 0.5 | 0.7 | +0.2 |" in diff and "| traced span | 1.0 | 1.0 | +0.0 |" in diff
    assert ta.main([str(tmp_path)]) == 0 and "slowest rank by compute time: 1" in capsys.readouterr().out
    assert ta.main([a, "--compare", b]) == 0 and "AllReduce" in capsys.readouterr().out


def test_partial_rotary_is_a_permutation_of_head_dimensions(tmp_path):
    """A checkpoint that rotates pairs (j, j + R/2) of its first R head dimensions gives the same attention scores
    here, where the kernels rotate pairs (i, i + D/2) with frequency 0 on the pass-through pairs, once its q/k head
    dimensions are permuted at load time; export restores the checkpoint's order."""
    from dataclasses import replace

    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.dense import BlockDiffusionTransformer
    from turbo_dllm_b200.models.hf_loader import export_hf_checkpoint, load_hf_config, load_hf_weights
    from turbo_dllm_b200.ops.rope import partial_rotary_permutation, qk_norm_rope_reference, rope_inv_freq

    D, R, theta = 64, 16, 1.0e4
    perm = partial_rotary_permutation(D, R)
    assert sorted(perm.tolist()) == list(range(D)) and perm[:8].tolist() == list(range(8))
    assert perm[32:40].tolist() == list(range(8, 16))
    freq = rope_inv_freq(D, theta, rotary_dim=R)
    assert (freq[8:] == 0).all() and torch.allclose(freq[:8], 1.0 / theta ** (torch.arange(0, R, 2) / R))
    torch.manual_seed(0)
    q, k = torch.randn(5, D), torch.randn(7, D)
    pq, pk = torch.arange(5), torch.arange(7) + 3

    def hf_rotate(x, pos):            # the checkpoint's convention
        ang = pos[:, None].float() * (1.0 / theta ** (torch.arange(0, R, 2) / R))[None, :]
        cos, sin = torch.cat([ang.cos()] * 2, -1), torch.cat([ang.sin()] * 2, -1)
        rot, rest = x[:, :R], x[:, R:]
        half = torch.cat([-rot[:, R // 2:], rot[:, : R // 2]], -1)
        return torch.cat([rot * cos + half * sin, rest], -1)

    want = hf_rotate(q, pq) @ hf_rotate(k, pk).t()
    mine_q = qk_norm_rope_reference(q[:, perm], pq, freq, None, None, 1, 0, D, 1e-6)[:, :D]
    mine_k = qk_norm_rope_reference(k[:, perm], pk, freq, None, None, 1, 0, D, 1e-6)[:, :D]
    assert torch.allclose(mine_q @ mine_k.t(), want, rtol=1e-4, atol=1e-4)
    # loader: export keeps the checkpoint's order, import permutes; a round trip is the identity
    cfg = replace(PRESETS["synthetic:tiny-qwen3"], partial_rotary_factor=0.25, num_layers=1)
    a = BlockDiffusionTransformer(cfg, dtype=torch.float32, seed=5)
    assert (a.inv_freq[cfg.rotary_dim // 2:] == 0).all()
    export_hf_checkpoint(a, str(tmp_path / "hf"))
    cfg2 = load_hf_config(str(tmp_path / "hf"))
    assert cfg2.partial_rotary_factor == 0.25
    b = BlockDiffusionTransformer(cfg2, dtype=torch.float32, seed=99)
    load_hf_weights(b, str(tmp_path / "hf"))
    assert torch.equal(a.flat.data, b.flat.data)
    from safetensors import safe_open

    with safe_open(str(tmp_path / "hf" / "model.safetensors"), "pt") as f:
        on_disk = f.get_tensor("model.layers.0.self_attn.q_norm.weight")
    assert torch.equal(on_disk[perm], a.layers[0].q_norm.detach())


def test_training_starts_from_a_local_pretrained_checkpoint(tmp_path):
    """`model.id` naming a local checkpoint directory gives the architecture AND the starting weights; model.random_init
    keeps the architecture only; a mixture-of-experts checkpoint round-trips through the same loader."""
    import dataclasses

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.dense import BlockDiffusionTransformer
    from turbo_dllm_b200.models.hf_loader import export_hf_checkpoint
    from turbo_dllm_b200.training.session import TrainingSession

    cfg = dataclasses.replace(PRESETS["synthetic:tiny-qwen3"], num_layers=2)
    a = BlockDiffusionTransformer(cfg, dtype=torch.float32, seed=5, init_std=0.05)
    hf = str(tmp_path / "hf")
    export_hf_checkpoint(a, hf)
    base = {"model": {"id": hf, "seq_len": 64, "dtype": "fp32"},
            "objective": {"name": "standard_block_diffusion", "block_size": 16},
            "training": {"batch_size": 1, "steps": 1}, "topology": {"context_parallel_size": 1, "block_parallel_size": 1}}
    s = TrainingSession(RunSpec.from_mapping(base).validate(), device="cpu")
    assert s.pretrained == hf and s.cfg.num_layers == 2 and s.cfg.hidden_size == cfg.hidden_size
    assert torch.equal(s.model.flat.data, a.flat.data)
    s.step()
    assert not torch.equal(s.model.flat.data, a.flat.data)
    r = TrainingSession(RunSpec.from_mapping({**base, "model": {**base["model"], "random_init": True, "max_layers": 1}}).validate(),
                        device="cpu")
    assert r.pretrained is None and r.cfg.num_layers == 1 and not torch.equal(r.model.flat.data[:100], a.flat.data[:100])
    with pytest.raises(ValueError, match="local checkpoint"):
        TrainingSession(RunSpec.from_mapping({**base, "model": {**base["model"], "id": str(tmp_path / "nowhere")}}).validate(),
                        device="cpu")
    # mixture of experts with the dense branch: export -> a session that starts from it
    from turbo_dllm_b200.models.export import export_moe_checkpoint

    moe = {**base, "model": {"id": "synthetic:tiny-moe", "seq_len": 64, "dtype": "fp32", "num_layers": 2,
                             "moe_shared_intermediate_size": 64}}
    m1 = TrainingSession(RunSpec.from_mapping(moe).validate(), device="cpu")
    m1.step()
    out = str(tmp_path / "moe")
    export_moe_checkpoint(m1.model, out)
    m2 = TrainingSession(RunSpec.from_mapping({**moe, "model": {"id": out, "seq_len": 64, "dtype": "fp32"}}).validate(), device="cpu")
    assert m2.cfg.is_moe and m2.cfg.moe_shared_intermediate_size == 64
    assert torch.equal(m2.model.flat.data, m1.model.flat.data) and torch.equal(m2.model.flat_experts.data, m1.model.flat_experts.data)


def _tp_checkpoint_round_trip(rank, world, hf_dense, hf_hybrid, out_dir):
    import torch.distributed as dist

    from turbo_dllm_b200.models.dense import BlockDiffusionTransformer
    from turbo_dllm_b200.models.hf_loader import export_hf_checkpoint, load_hf_config, load_hf_weights
    from turbo_dllm_b200.models.hybrid import HybridBlockDiffusionTransformer
    from turbo_dllm_b200.parallel.tensor_parallel import TPContext

    torch.set_num_threads(2)
    tp = TPContext(dist.group.WORLD)
    same = {}
    for kind, cls, src in (("dense", BlockDiffusionTransformer, hf_dense), ("hybrid", HybridBlockDiffusionTransformer, hf_hybrid)):
        cfg = load_hf_config(src)
        # the model this rank would have built from the single-rank weights: same seed -> shards of the same tensors
        model = cls(cfg, dtype=torch.float32, seed=99, tp=tp)
        load_hf_weights(model, src)
        export_hf_checkpoint(model, f"{out_dir}/{kind}")
        same[kind] = float(model.flat.data.double().sum())
    return same


def test_tensor_parallel_ranks_load_their_shards_and_export_the_whole(tmp_path):
    """Two tensor-parallel ranks read their slices of a checkpoint (dense and hybrid family); gathering them back
    writes a file identical, tensor by tensor, to the one they were read from."""
    import dataclasses

    from safetensors import safe_open

    from tests._harness import run_ranks
    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.dense import BlockDiffusionTransformer
    from turbo_dllm_b200.models.hf_loader import export_hf_checkpoint
    from turbo_dllm_b200.models.hybrid import HybridBlockDiffusionTransformer

    dense = BlockDiffusionTransformer(dataclasses.replace(PRESETS["synthetic:tiny-qwen3"], num_layers=2), dtype=torch.float32,
                                      seed=5, init_std=0.05)
    hybrid = HybridBlockDiffusionTransformer(PRESETS["synthetic:tiny-qwen3_8"], dtype=torch.float32, seed=7, init_std=0.05)
    with torch.no_grad():
        for m in (dense, hybrid):
            for p in m.flat.params.values():
                if not p.decay:
                    p.add_(torch.randn_like(p) * 0.1)       # norms, biases, decay rates: distinctive values
    export_hf_checkpoint(dense, str(tmp_path / "dense"))
    export_hf_checkpoint(hybrid, str(tmp_path / "hybrid"))
    run_ranks(_tp_checkpoint_round_trip, 2, args=(str(tmp_path / "dense"), str(tmp_path / "hybrid"), str(tmp_path / "out")),
              deadline_s=240)
    for kind in ("dense", "hybrid"):
        with safe_open(str(tmp_path / kind / "model.safetensors"), framework="pt") as a, \
                safe_open(str(tmp_path / "out" / kind / "model.safetensors"), framework="pt") as b:
            assert set(a.keys()) == set(b.keys())
            for k in a.keys():
                assert torch.equal(a.get_tensor(k), b.get_tensor(k)), (kind, k)


def test_model_inspector(tmp_path, capsys):
    from turbo_dllm_b200.benchmarks.inspect_models import main, summarize
    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.dense import BlockDiffusionTransformer
    from turbo_dllm_b200.models.hf_loader import export_hf_checkpoint

    s = summarize("synthetic:qwen3-8b")
    assert s["family"] == "causal_lm" and 8.1e9 < s["parameters"] < 8.3e9 and s["attention_path"].startswith("fused")
    assert 0.3 < s["attention_share_of_flops"] < 0.5
    export_hf_checkpoint(BlockDiffusionTransformer(PRESETS["synthetic:tiny-qwen3"], dtype=torch.float32), str(tmp_path / "hf"))
    assert main([str(tmp_path / "hf"), "--json", "--seq-len", "256", "--block-size", "16"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["source"] == "checkpoint directory" and rep["hidden_size"] == PRESETS["synthetic:tiny-qwen3"].hidden_size
    assert main(["nowhere"]) == 2


def test_flop_models_count_exactly_what_the_masks_allow():
    """The pair counters equal the number of visible entries of the dense masks (full prefix and sliding window), and
    the drafter-distillation model adds up its parts."""
    import dataclasses

    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.ops.attention import block_diffusion_layout
    from turbo_dllm_b200.profiling.perf import (block_diffusion_pairs, dflash_step_flops, model_attention_pairs,
                                                transformer_step_flops)

    L, bs = 96, 16
    pos = torch.arange(L)
    for views in (1, 2):
        npos = pos.repeat(views)
        ngrp = (pos // bs).repeat(views) + torch.arange(views).repeat_interleave(L) * (L // bs)
        for window in (None, 40, 16):
            lay = block_diffusion_layout(npos, ngrp, pos, bs, window=window)
            assert int(lay.dense_mask().sum()) == block_diffusion_pairs(L, bs, views, window), (views, window)
    cfg = dataclasses.replace(PRESETS["synthetic:tiny-qwen3"], num_layers=4, sliding_window=40, sliding_window_pattern=2)
    want = (2 * block_diffusion_pairs(L, bs, 1, 40) + 2 * block_diffusion_pairs(L, bs, 1)) / 4
    assert model_attention_pairs(cfg, L, bs) == want
    full = dataclasses.replace(cfg, sliding_window=None)
    a = transformer_step_flops(cfg, rows=2 * L, pairs=model_attention_pairs(cfg, L, bs), vocab_rows=L)
    b = transformer_step_flops(full, rows=2 * L, pairs=model_attention_pairs(full, L, bs), vocab_rows=L)
    assert a.attention < b.attention and a.dense == b.dense
    draft, target = PRESETS["synthetic:dflash-draft-5l"], PRESETS["synthetic:qwen3-8b"]
    kw = dict(seq_len=4096, block_size=16, anchors=128, num_target_layers=5)
    online = dflash_step_flops(draft, target, **kw)
    offline = dflash_step_flops(draft, target, online_target=False, **kw)
    ce = dflash_step_flops(draft, target, loss="paper_ce", **kw)
    small = dflash_step_flops(draft, target, draft_vocab_size=32000, **kw)
    # the frozen 36-layer target forward dominates an online step; it is 2 FLOPs per weight and row
    per_row = target.hidden_size * target.qkv_dim + target.q_dim * target.hidden_size + 3 * target.hidden_size * target.intermediate_size
    assert online.dense - offline.dense == pytest.approx(2.0 * 4096 * per_row * 36)
    assert online.head - ce.head == pytest.approx(2.0 * 128 * 16 * target.hidden_size * target.vocab_size)
    assert small.head < online.head and dflash_step_flops(draft, target, batch=3, **kw).total == pytest.approx(3 * online.total)


def test_a_bf16_run_is_exported_on_a_machine_without_a_gpu(tmp_path):
    """The export entry rebuilds the model in fp32 where there is no GPU and writes the run's dtype."""
    from safetensors import safe_open

    from turbo_dllm_b200.checkpoint import save_training_checkpoint
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.models import hf_loader
    from turbo_dllm_b200.models.export import export_training_checkpoint
    from turbo_dllm_b200.training.session import TrainingSession

    if torch.cuda.is_available():
        pytest.skip("this path is for machines without a GPU")
    base = {"model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "num_layers": 1},
            "objective": {"name": "standard_block_diffusion", "block_size": 16},
            "training": {"batch_size": 1, "steps": 1}, "topology": {"context_parallel_size": 1, "block_parallel_size": 1}}
    s = TrainingSession(RunSpec.from_mapping(base).validate(), device="cpu")
    s.step()
    save_training_checkpoint(str(tmp_path / "ck"), s, step=1, rank=0, world_size=1)
    bf16 = RunSpec.from_mapping({**base, "model": {**base["model"], "dtype": "bf16"}}).validate()
    export_training_checkpoint(bf16, str(tmp_path / "ck"), str(tmp_path / "hf"))
    assert hf_loader.EXPORT_DTYPE is None
    with safe_open(str(tmp_path / "hf" / "model.safetensors"), framework="pt") as f:
        w = f.get_tensor("model.layers.0.self_attn.o_proj.weight")
    assert w.dtype == torch.bfloat16 and torch.equal(w, s.model.flat.params["layers.0.w_o"].to(torch.bfloat16))
