"""End-to-end parity of the sm_100a path with the fp32 PyTorch reference path on one tiny model."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _spec(dtype, objective="fast_dllm_v2", model="synthetic:tiny-hd128"):
    from turbo_dllm_b200.config.run_spec import RunSpec

    extra, family = {}, {}
    if objective == "diffusiongemma_native_sft":   # causal clean stream + encoder next-token term (weight 1)
        extra = {"loss_weighting": "unit", "self_conditioning_probability": 0.0}
        family = {"family": "diffusion_gemma"}     # the family this objective belongs to (dense FFN variant)
    return RunSpec.from_mapping({
        "model": {"id": model, "seq_len": 256, "dtype": dtype, **family},
        "objective": {"name": objective, "block_size": 32, "noise_schedule_epsilon": 0.1, **extra},
        "training": {"batch_size": 2, "steps": 2, "activation_checkpointing": True},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate()


@pytest.mark.parametrize("objective,model", [("fast_dllm_v2", "synthetic:tiny-hd128"),
                                             ("standard_block_diffusion", "synthetic:tiny-hd128"),
                                             ("fast_dllm_v2", "synthetic:tiny-qwen3_8-hd128"),
                                             ("diffusiongemma_native_sft", "synthetic:tiny-hd128")])
def test_loss_and_grads_match_cpu_reference(objective, model):
    """The last case is the hybrid family: Gated DeltaNet layers (projections on the tcgen05 GEMM,
    recurrence as batched products) and a gated softmax-attention layer."""
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.training.session import TrainingSession

    gpu = TrainingSession(_spec("bf16", objective, model), device="cuda")
    cpu = TrainingSession(_spec("fp32", objective, model), device="cpu")
    cpu.model.flat.data.copy_(gpu.model.flat.data.float().cpu())
    batch = gpu.data.next_batch()
    cb = gpu.objective.corrupt(batch.input_ids)
    denom = float(cb.loss_denominator)

    def run(sess, cb_):
        sess.model.flat.zero_grad()
        tok, lab, w = sess.assemble_rows(cb_)
        hid = sess.model(tok, sess.layout.positions, sess.attend)
        from turbo_dllm_b200.models.dense import compact_supervised_rows

        h, l, ww, _ = compact_supervised_rows(hid, lab, w)
        loss, _ = sess.model.loss(h, l, ww, sess.objective.exclude_mask_token)
        (loss / denom).backward()
        sess.model.flat.collect_grads()
        return float(loss) / denom, sess.model.flat.grad.float().cpu()

    import dataclasses

    cb_cpu = dataclasses.replace(cb, **{f.name: (getattr(cb, f.name).cpu() if torch.is_tensor(getattr(cb, f.name))
                                                  else getattr(cb, f.name)) for f in dataclasses.fields(cb)})
    lg, gg = run(gpu, cb)
    torch.cuda.synchronize()
    native.raise_on_device_error()
    lc, gc = run(cpu, cb_cpu)
    assert abs(lg - lc) < 2e-2 * max(1.0, abs(lc)), (lg, lc)
    cos = torch.nn.functional.cosine_similarity(gg, gc, dim=0).item()
    assert cos > 0.99, cos
    rel = (gg - gc).norm().item() / gc.norm().item()
    assert rel < 0.1, rel


def test_training_steps_run_and_update_parameters():
    from turbo_dllm_b200.training.session import TrainingSession

    s = TrainingSession(_spec("bf16"), device="cuda", host_staged_data=True)
    before = s.model.flat.data.clone()
    losses = [float(s.step().loss_sum) for _ in range(3)]
    assert all(l == l and l > 0 for l in losses)
    assert not torch.equal(before, s.model.flat.data)
    assert s.optimizer.grad_norm() > 0


def _moe_spec(dtype, extra_model=None, adapter=None):
    from turbo_dllm_b200.config.run_spec import RunSpec

    m = {"model": {"id": "synthetic:tiny-moe-hd128", "seq_len": 256, "dtype": dtype, "family": "diffusion_gemma",
                   **(extra_model or {})},
         "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
         "training": {"batch_size": 2, "steps": 2, "activation_checkpointing": True},
         "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
         "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}
    if adapter:
        m["adapter"] = adapter
    return RunSpec.from_mapping(m).validate()


def test_moe_with_shared_dense_branch_matches_cpu_loss_and_replays_routes():
    """One GPU, routed experts (grouped GEMMs) plus the dense feed-forward beside them, under activation
    checkpointing: the first loss equals the fp32 CPU path, the recomputation uses the recorded routes."""
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.training.session import TrainingSession

    extra = {"moe_shared_intermediate_size": 256}
    g = TrainingSession(_moe_spec("bf16", extra), device="cuda")
    c = TrainingSession(_moe_spec("fp32", extra), device="cpu")
    c.model.flat.data.copy_(g.model.flat.data.float().cpu())
    c.model.flat_experts.data.copy_(g.model.flat_experts.data.float().cpu())
    rg, rc = g.step(), c.step()
    torch.cuda.synchronize()
    native.raise_on_device_error()
    lg, lc = float(rg.loss_sum) / rg.denominator, float(rc.loss_sum) / rc.denominator
    assert lg == pytest.approx(lc, rel=3e-2)
    assert not any(isinstance(k, tuple) and k[1] == "moe_route" for k in g.model.store.kept)
    assert float(g.step().loss_sum) > 0


@pytest.mark.parametrize("moe", [False, True])
def test_lora_adapters_train_on_the_gpu(moe):
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.training.session import TrainingSession

    if moe:
        spec = _moe_spec("bf16", adapter={"type": "lora", "rank": 8, "alpha": 16.0, "targets": ["attention", "experts"]})
    else:
        spec = RunSpec.from_mapping({
            "model": {"id": "synthetic:tiny-hd128", "seq_len": 256, "dtype": "bf16"},
            "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
            "adapter": {"type": "lora", "rank": 8, "alpha": 16.0, "targets": ["attention", "mlp"]},
            "training": {"batch_size": 2, "steps": 2}, "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
            "optimizer": {"lr": 1e-2, "gradient_clip_norm": 1.0}}).validate()
    s = TrainingSession(spec, device="cuda")
    base = s.model.flat.data.clone()
    before = [f.data.clone() for f in s.flats()]
    losses = [float(r.loss_sum) / r.denominator for r in (s.step() for _ in range(3))]
    torch.cuda.synchronize()
    native.raise_on_device_error()
    assert all(l == l and l > 0 for l in losses)
    assert torch.equal(s.model.flat.data, base)
    assert all(not torch.equal(f.data, b) for f, b in zip(s.flats(), before))
