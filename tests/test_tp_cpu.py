"""Tensor parallelism over gloo ranks reproduces the single-process model (fp32, CPU)."""
import copy

import pytest
import torch

from tests._harness import assert_params_close, run_ranks

MAPPING = {
    "model": {"id": "synthetic:tiny-qwen3", "seq_len": 128, "dtype": "fp32", "num_layers": 2},
    "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
    "training": {"batch_size": 2, "steps": 3},
    "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
    "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0},
}


def _run(rank, world, tp, steps, sp=False):
    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    m = copy.deepcopy(MAPPING)
    m["topology"]["tensor_parallel_size"] = tp
    m["topology"]["sequence_parallel"] = bool(sp)
    spec = RunSpec.from_mapping(m).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device="cpu", runtime=rt)
    losses, norms = [], []
    for _ in range(steps):
        r = s.step()
        losses.append(float(r.loss_sum) / r.denominator)
        norms.append(s.optimizer.grad_norm())
    names = {n: p.detach().clone() for n, p in s.model.flat.params.items()}
    return (losses, norms, names["final_norm"], names["layers.1.w_down"], names["layers.0.w_qkv"],
            names["layers.0.q_norm"], names["layers.1.input_norm"])


@pytest.mark.distributed
def test_tp2_matches_single_process():
    ref = _run(0, 1, 1, 3)
    outs = run_ranks(_run, 2, args=(2, 3), deadline_s=240)
    for r, (losses, norms, fnorm, w_down, w_qkv, q_norm, in_norm) in enumerate(outs):
        assert losses == pytest.approx(ref[0], rel=2e-4, abs=2e-4)
        assert norms == pytest.approx(ref[1], rel=2e-3)
        assert_params_close(fnorm, ref[2], rtol=1e-3, atol=2e-5)
        full = ref[3]
        n = full.shape[1] // 2
        assert_params_close(w_down, full[:, r * n:(r + 1) * n], rtol=1e-3, atol=1e-4)
        # replicated weights whose gradient a rank sees only partly (its heads) stay equal to the single-rank run
        assert_params_close(q_norm, ref[5], rtol=1e-3, atol=2e-5)


@pytest.mark.distributed
def test_tp2_with_sequence_parallel_rows_matches_single_process():
    """Residual stream sharded by rows inside the tensor-parallel pair: gather → column GEMM, row GEMM →
    reduce-scatter, layer-norm gradients summed over the pair."""
    ref = _run(0, 1, 1, 3)
    outs = run_ranks(_run, 2, args=(2, 3, True), deadline_s=240)
    for r, (losses, norms, fnorm, w_down, w_qkv, q_norm, in_norm) in enumerate(outs):
        assert losses == pytest.approx(ref[0], rel=2e-4, abs=2e-4)
        assert norms == pytest.approx(ref[1], rel=2e-3)
        assert_params_close(fnorm, ref[2], rtol=1e-3, atol=2e-5)
        assert_params_close(q_norm, ref[5], rtol=1e-3, atol=2e-5)
        assert_params_close(in_norm, ref[6], rtol=1e-3, atol=2e-5)
        full = ref[3]
        n = full.shape[1] // 2
        assert_params_close(w_down, full[:, r * n:(r + 1) * n], rtol=1e-3, atol=1e-4)


def _run_lora(rank, world, tp, steps, sp=False):
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    m = copy.deepcopy(MAPPING)
    m["topology"]["tensor_parallel_size"] = tp
    m["topology"]["sequence_parallel"] = bool(sp)
    m["adapter"] = {"type": "lora", "rank": 4, "alpha": 8.0, "targets": ["attention", "mlp"]}
    m["optimizer"]["lr"] = 1e-2
    spec = RunSpec.from_mapping(m).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device="cpu", runtime=rt)
    losses, norms = [], []
    for _ in range(steps):
        r = s.step()
        losses.append(float(r.loss_sum) / r.denominator)
        norms.append(s.optimizer.grad_norm())
    p = {n: t.detach().clone() for n, t in s.lora.flat.params.items()}
    return (losses, norms, p["layers.0.w_qkv.lora_A"], p["layers.1.w_down.lora_B"], p["layers.1.w_down.lora_A"],
            p["layers.0.w_gate_up.lora_B"])


@pytest.mark.distributed
@pytest.mark.parametrize("sp", [False, True])
def test_lora_under_tensor_parallelism_matches_single_process(sp):
    """Adapters with the projections' local shapes: column-parallel B and row-parallel A are shards, the other
    halves are replicated and stay equal on both ranks (under sequence parallelism through the partial-gradient
    sum); losses, gradient norms and adapter weights follow the single-process LoRA run."""
    ref = _run_lora(0, 1, 1, 3)
    assert ref[0][-1] < ref[0][0]                      # the adapters do train
    outs = run_ranks(_run_lora, 2, args=(2, 3, sp), deadline_s=240)
    for r, (losses, norms, qkv_a, down_b, down_a, gu_b) in enumerate(outs):
        assert losses == pytest.approx(ref[0], rel=3e-4, abs=3e-4)
        assert norms == pytest.approx(ref[1], rel=3e-3)
        assert_params_close(qkv_a, ref[2], rtol=2e-3, atol=2e-5)       # replicated A
        assert_params_close(down_b, ref[3], rtol=2e-3, atol=2e-5)      # replicated B
        full = ref[4]
        n = full.shape[1] // 2
        assert_params_close(down_a, full[:, r * n:(r + 1) * n], rtol=2e-3, atol=2e-5)
        full = ref[5]
        n = full.shape[0] // 2
        assert_params_close(gu_b, full[r * n:(r + 1) * n], rtol=2e-3, atol=2e-5)


def _run_hybrid(rank, world, tp, steps, sp=False):
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3_8", "seq_len": 64, "dtype": "fp32"},
        "objective": {"name": "fast_dllm_v2", "block_size": 16, "noise_schedule_epsilon": 0.1},
        "training": {"batch_size": 2, "steps": steps},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1, "tensor_parallel_size": tp,
                     "sequence_parallel": sp},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device="cpu", runtime=rt)
    assert bool(getattr(s.model.tp, "sequence_parallel", False)) == (sp and tp > 1)
    losses, norms = [], []
    for _ in range(steps):
        r = s.step()
        losses.append(float(r.loss_sum) / r.denominator)
        norms.append(s.optimizer.grad_norm())
    p = {n: t.detach().clone() for n, t in s.model.flat.params.items()}
    return (losses, norms, p["layers.0.w_in"], p["layers.0.A_log"], p["layers.0.gdn_norm"], p["layers.3.w_attn_gate"],
            p["layers.0.w_out"], p["layers.3.q_norm"], p["layers.0.input_norm"], p["layers.3.post_norm"])


@pytest.mark.distributed
@pytest.mark.parametrize("sp", [False, True])
def test_hybrid_family_under_tensor_parallelism_matches_single_process(sp):
    """Gated DeltaNet layers with half of the key / value heads per rank (fused input projection by head segments,
    per-head decay vectors, output projection by value-head columns) and the gated softmax-attention layer with half
    of its heads: losses, gradient norms and weights follow the single-process run."""
    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.hybrid import fused_projection_rows

    ref = _run_hybrid(0, 1, 1, 3)
    outs = run_ranks(_run_hybrid, 2, args=(2, 3, sp), deadline_s=300)
    cfg = PRESETS["synthetic:tiny-qwen3_8"]
    for r, (losses, norms, w_in, a_log, gdn_norm, gate, w_out, q_norm, in_norm, post_norm) in enumerate(outs):
        # with sequence parallelism the layer norms see this rank's rows only: their partial gradients are summed
        assert_params_close(in_norm, ref[8], rtol=2e-3, atol=2e-5)
        assert_params_close(post_norm, ref[9], rtol=2e-3, atol=2e-5)
        assert losses == pytest.approx(ref[0], rel=3e-4, abs=3e-4)
        assert norms == pytest.approx(ref[1], rel=3e-3)
        rows, _ = fused_projection_rows(cfg, r, 2)
        got = torch.from_numpy(w_in)
        assert torch.allclose(got[: rows.numel()], ref[2][rows], rtol=2e-3, atol=2e-5)
        hv = cfg.linear_num_value_heads // 2
        assert_params_close(a_log, ref[3][r * hv:(r + 1) * hv], rtol=2e-3, atol=2e-5)
        assert_params_close(gdn_norm, ref[4], rtol=2e-3, atol=2e-5)        # replicated, partial grads summed
        n = ref[5].shape[0] // 2
        assert_params_close(gate, ref[5][r * n:(r + 1) * n], rtol=2e-3, atol=2e-5)
        n = ref[6].shape[1] // 2
        assert_params_close(w_out, ref[6][:, r * n:(r + 1) * n], rtol=2e-3, atol=2e-5)
        assert_params_close(q_norm, ref[7], rtol=2e-3, atol=2e-5)


def _run_eval(rank, world, tp, sp, data_path, steps=12):
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.evaluation import evaluate_masked_token_accuracy
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 128, "dtype": "fp32", "num_layers": 2},
        "objective": {"name": "standard_block_diffusion", "block_size": 16, "sampling_epsilon_min": 0.1},
        "data": {"input_mode": "dataset", "dataset_path": data_path},
        "training": {"batch_size": 2, "steps": steps},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1, "tensor_parallel_size": tp, "sequence_parallel": sp},
        "optimizer": {"lr": 3e-3}}).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device="cpu", runtime=rt)
    for _ in range(steps):
        s.step()
    return evaluate_masked_token_accuracy(s, 2, 7)


@pytest.mark.distributed
def test_evaluation_under_tensor_parallelism_counts_once_and_finds_the_argmax(tmp_path):
    """Masked-token accuracy with the vocabulary split over two ranks (the largest logit over the ranks, ties to the
    smallest id) and the counts of the identical tensor-parallel copies taken once: the figures of the single process.
    The data repeats seven token ids of the upper vocabulary half, so a few steps make some predictions right."""
    import numpy as np

    path = str(tmp_path / "cycle.i32")
    (np.arange(16384) % 7 + 600).astype("<i4").tofile(path)
    ref = _run_eval(0, 1, 1, False, path)
    assert ref["eval_masked_token_accuracy"] > 0.02
    for out in run_ranks(_run_eval, 2, args=(2, True, path), deadline_s=300):
        assert out["eval_masked_tokens"] == ref["eval_masked_tokens"]
        assert out["eval_masked_token_accuracy"] == pytest.approx(ref["eval_masked_token_accuracy"], abs=0.01)
        assert out["eval_loss"] == pytest.approx(ref["eval_loss"], rel=1e-3)
