"""Combinations of parallel axes, model families and objectives on gloo ranks: two optimizer steps of every combination
must reproduce the single-process losses and gradient norm (same seed, same data). The single-axis cases live in the
families' own test files; this file covers what only shows up when axes meet (a layout one family cannot take, a collective
that only some ranks enter, a gradient counted twice)."""
import pytest
import torch

from tests._harness import run_ranks


def _run(rank, world, mapping, steps=2):
    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping(mapping).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device="cpu", runtime=rt)
    tp = spec.topology.tensor_parallel_size
    losses = []
    for _ in range(steps):
        r = s.step()
        t = r.loss_sum.double().clone()
        if world > 1:
            dist.all_reduce(t)
        losses.append(float(t) / float(r.denominator) / tp)
    return losses, float(s.optimizer.grad_norm())


def _spec(model=None, objective=None, topology=None, **sections):
    m = {"model": {"id": "synthetic:tiny-qwen3", "seq_len": 128, "dtype": "fp32", "num_layers": 2, **(model or {})},
         "objective": {"name": "standard_block_diffusion", "block_size": 16, "sampling_epsilon_min": 0.1, **(objective or {})},
         "training": {"batch_size": 2, "steps": 2},
         "topology": {"context_parallel_size": 1, "block_parallel_size": 1, **(topology or {})},
         "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}
    for k, v in sections.items():
        m[k] = {**m.get(k, {}), **v}
    return m


LORA = {"adapter": {"type": "lora", "rank": 4, "alpha": 8.0, "targets": ["attention", "mlp"]}}
HYBRID = {"id": "synthetic:tiny-qwen3_8", "family": "qwen3_8", "num_layers": 4, "linear_num_key_heads": 4,
          "linear_num_value_heads": 8}
MOE = {"id": "synthetic:tiny-moe", "family": "diffusion_gemma", "num_layers": 2}
V2 = {"name": "fast_dllm_v2"}
SFT = {"name": "diffusiongemma_native_sft", "noise_schedule": "loglinear", "loss_weighting": "unit",
       "self_conditioning_probability": 0.5}
CSBP2 = {"context_parallel_size": 2, "block_parallel_size": 2}
BP2 = {"block_parallel_size": 2, "replicate_clean_prefix": True}
WINDOW = {"sliding_window": 48, "sliding_window_pattern": 2}

CASES = {
    # name: (ranks, what differs from the single-process reference, the reference)
    "dense lora x csbp2": (2, dict(topology=CSBP2, **LORA), dict(**LORA)),
    "hybrid lora x csbp2": (2, dict(model=HYBRID, objective=V2, topology=CSBP2, **LORA), dict(model=HYBRID, objective=V2, **LORA)),
    "hybrid lora x tp2 + sp": (2, dict(model=HYBRID, objective=V2, topology={"tensor_parallel_size": 2, "sequence_parallel": True}, **LORA),
                               dict(model=HYBRID, objective=V2, **LORA)),
    "sliding window x tp2": (2, dict(model=WINDOW, topology={"tensor_parallel_size": 2}), dict(model=WINDOW)),
    "pure cp2 x tp2": (4, dict(topology={"context_parallel_size": 2, "tensor_parallel_size": 2}), dict()),
    "pure bp2 x tp2 + sp": (4, dict(topology={**BP2, "tensor_parallel_size": 2, "sequence_parallel": True}), dict()),
    "fast-dllm v2 x tp2 x csbp2": (4, dict(objective=V2, topology={**CSBP2, "tensor_parallel_size": 2}), dict(objective=V2)),
    "mlp-scope checkpointing x csbp2": (2, dict(topology=CSBP2, training={"activation_checkpointing_scope": "mlp"}), dict()),
    "native sft (dense) x tp2 + sp": (2, dict(model={"family": "diffusion_gemma"}, objective=SFT,
                                              topology={"tensor_parallel_size": 2, "sequence_parallel": True}),
                                      dict(model={"family": "diffusion_gemma"}, objective=SFT)),
    "native sft (dense) x pure bp2": (2, dict(model={"family": "diffusion_gemma"}, objective=SFT, topology=BP2),
                                      dict(model={"family": "diffusion_gemma"}, objective=SFT)),
    "gradient accumulation x csbp2": (2, dict(topology=CSBP2, training={"gradient_accumulation_steps": 2}),
                                      dict(training={"gradient_accumulation_steps": 2})),
    "hybrid x tp2 x bp2": (4, dict(model=HYBRID, objective=V2, topology={**BP2, "tensor_parallel_size": 2}),
                           dict(model=HYBRID, objective=V2)),
    "hybrid x tp2 + sp x pure cp2": (4, dict(model=HYBRID, objective=V2, topology={"context_parallel_size": 2, "tensor_parallel_size": 2,
                                                                                   "sequence_parallel": True}),
                                     dict(model=HYBRID, objective=V2)),
    "moe x pure bp2": (2, dict(model=MOE, objective={"block_size": 32}, topology=BP2), dict(model=MOE, objective={"block_size": 32})),
    "moe expert adapters x csbp2": (2, dict(model=MOE, objective={"block_size": 32}, topology=CSBP2,
                                            adapter={"type": "lora", "rank": 4, "alpha": 8.0, "targets": ["attention", "experts"]}),
                                    dict(model=MOE, objective={"block_size": 32},
                                         adapter={"type": "lora", "rank": 4, "alpha": 8.0, "targets": ["attention", "experts"]})),
    "moe adapters incl. experts x tp2 + sp": (2, dict(model={**MOE, "moe_shared_intermediate_size": 64}, objective={"block_size": 32},
                                                   topology={"tensor_parallel_size": 2, "sequence_parallel": True},
                                                   adapter={"type": "lora", "rank": 4, "alpha": 8.0, "targets": ["attention", "mlp", "experts"]}),
                                              dict(model={**MOE, "moe_shared_intermediate_size": 64}, objective={"block_size": 32},
                                                   adapter={"type": "lora", "rank": 4, "alpha": 8.0, "targets": ["attention", "mlp", "experts"]})),
    "clean-replica sharing cp2 bp4": (4, dict(topology={"context_parallel_size": 2, "block_parallel_size": 4}), dict()),
    "streaming transport x contiguous shards": (2, dict(topology=CSBP2, kernel={"cp_bp_clean_kv_transport": "streaming",
                                                                                 "cp_bp_clean_kv_layout": "contiguous"}), dict()),
}


def _run_many(rank, world, cases):
    """Several combinations in one group of spawned ranks (starting the ranks costs more than the steps)."""
    import torch.distributed as dist

    out = {}
    for name, mapping in cases:
        out[name] = _run(rank, world, mapping)
        dist.barrier()
    return out


@pytest.mark.distributed
@pytest.mark.parametrize("world", [2, 4])
def test_combinations_match_single_process(world):
    """Every combination of `CASES` that runs on `world` ranks (TDLLM_MATRIX_CASE=<name> runs one of them alone)."""
    import os

    only = os.environ.get("TDLLM_MATRIX_CASE")
    names = [n for n in sorted(CASES) if CASES[n][0] == world and (only is None or n == only)]
    if not names:
        pytest.skip("no combination selected for this number of ranks")
    refs = {n: _run(0, 1, _spec(**CASES[n][2])) for n in names}
    got = run_ranks(_run_many, world, args=([(n, _spec(**CASES[n][1])) for n in names],), deadline_s=900)[0]
    wrong = []
    for n in names:
        losses, norm = got[n]
        if losses != pytest.approx(refs[n][0], rel=3e-4, abs=3e-4) or norm != pytest.approx(refs[n][1], rel=4e-3):
            wrong.append(f"{n}: {losses} / {norm} against {refs[n][0]} / {refs[n][1]}")
    assert not wrong, "\n".join(wrong)


@pytest.mark.distributed
def test_hybrid_parameter_sharding_equals_the_sharded_optimizer():
    """Hybrid family with `optimizer.backend: fsdp` under context-sharded block parallelism (2 ranks)."""
    kw = dict(model=HYBRID, objective=V2, topology=CSBP2)
    a = run_ranks(_run, 2, args=(_spec(optimizer={"backend": "torch_adamw"}, **kw), 3), deadline_s=400)[0]
    b = run_ranks(_run, 2, args=(_spec(optimizer={"backend": "fsdp"}, **kw), 3), deadline_s=400)[0]
    assert b[0] == pytest.approx(a[0], rel=3e-4, abs=3e-4) and b[1] == pytest.approx(a[1], rel=1e-3)
    # with tensor parallelism some non-decayed vectors are shards too: the gradient norm splits at the buffer's own boundary
    kw = dict(model=HYBRID, objective=V2, topology={"tensor_parallel_size": 2, "sequence_parallel": True})
    a = run_ranks(_run, 4, args=(_spec(optimizer={"backend": "torch_adamw"}, **kw), 3), deadline_s=400)[0]
    b = run_ranks(_run, 4, args=(_spec(optimizer={"backend": "fsdp"}, **kw), 3), deadline_s=400)[0]
    assert b[0] == pytest.approx(a[0], rel=3e-4, abs=3e-4) and b[1] == pytest.approx(a[1], rel=2e-4)


@pytest.mark.distributed
def test_parameter_sharding_equals_the_sharded_optimizer_on_a_three_axis_topology():
    """Data parallelism 2 x tensor parallelism 2 with sequence parallelism x context-sharded block parallelism 2
    (8 ranks): parameter sharding and the sharded optimizer give the same step."""
    topo = {**CSBP2, "tensor_parallel_size": 2, "sequence_parallel": True}
    a = run_ranks(_run, 8, args=(_spec(topology=topo, optimizer={"backend": "torch_adamw"}),), deadline_s=600)[0]
    b = run_ranks(_run, 8, args=(_spec(topology=topo, optimizer={"backend": "fsdp"}),), deadline_s=600)[0]
    assert b[0] == pytest.approx(a[0], rel=3e-4, abs=3e-4) and b[1] == pytest.approx(a[1], rel=4e-3)
