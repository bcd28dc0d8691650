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
