"""Expert-parallel MoE on gloo ranks: dispatch/combine against the dense expert oracle, and a
training run whose replicated parameters stay identical across ranks."""
import pytest
import torch

from tests._harness import run_ranks


def _bank(rank, world):
    import torch.distributed as dist

    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.moe import MoEBlockDiffusionTransformer, reference_experts, route_topk

    torch.set_num_threads(2)
    cfg = PRESETS["synthetic:tiny-moe"]
    m = MoEBlockDiffusionTransformer(cfg, ep_group=dist.group.WORLD, dtype=torch.float32, device="cpu", seed=3)
    bank = m.layers[0].experts
    torch.manual_seed(100 + rank)
    x = torch.randn(37 + 5 * rank, cfg.hidden_size, requires_grad=True)
    y = bank(x)
    y.sum().backward()
    # oracle with every rank's experts gathered
    gu = [torch.empty_like(bank.w_gu) for _ in range(world)]
    dn = [torch.empty_like(bank.w_down) for _ in range(world)]
    dist.all_gather(gu, bank.w_gu.detach().contiguous())
    dist.all_gather(dn, bank.w_down.detach().contiguous())
    xr = x.detach().clone().requires_grad_()
    w, idx = route_topk(xr @ bank.router.t(), cfg.num_experts_per_token)
    ref = reference_experts(xr, torch.cat(gu), torch.cat(dn), w, idx)
    ref.sum().backward()
    return float((y - ref).abs().max()), float((x.grad - xr.grad).abs().max())


@pytest.mark.distributed
def test_expert_parallel_bank_matches_dense_oracle():
    for fwd_err, bwd_err in run_ranks(_bank, 2, deadline_s=120):
        assert fwd_err < 1e-5 and bwd_err < 1e-4


def _train(rank, world):
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-moe", "seq_len": 128, "dtype": "fp32", "family": "diffusion_gemma"},
        "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
        "training": {"batch_size": 1, "steps": 2},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1, "expert_parallel_size": 2},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world)
    s = TrainingSession(spec, device="cpu", runtime=rt)
    assert s.dp_size == 2 and s.model.flat_experts.params["layers.0.experts_down"].shape[0] == 4
    losses = [float(s.step().loss_sum) for _ in range(2)]
    return losses, s.model.flat.data.clone(), s.model.flat_experts.data.clone(), s.optimizer.grad_norm()


@pytest.mark.distributed
def test_expert_parallel_training_keeps_dense_parameters_in_sync():
    a, b = run_ranks(_train, 2, deadline_s=240)
    assert (a[1] == b[1]).all()            # replicated parameters
    assert not (a[2] == b[2]).all()        # different experts per rank
    assert a[3] == pytest.approx(b[3], rel=1e-6)   # one global gradient norm
    assert all(l == l and l > 0 for l in a[0] + b[0])


def test_shared_dense_branch_and_replayed_routes():
    """A layer with a dense feed-forward beside its experts equals experts + dense branch computed by hand, and a
    checkpointed layer's recomputation takes the experts its first pass chose."""
    from dataclasses import replace

    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.dense import LocalAttention
    from turbo_dllm_b200.models.moe import MoEBlockDiffusionTransformer
    from turbo_dllm_b200.parallel.layout import build_packed_layout

    cfg = replace(PRESETS["synthetic:tiny-moe"], moe_shared_intermediate_size=96)
    m = MoEBlockDiffusionTransformer(cfg, dtype=torch.float32, seed=5, init_std=0.05, activation_checkpointing=True)
    layer = m.layers[0]
    assert layer.w_gate_up.shape == (192, cfg.hidden_size) and layer.w_down.shape == (cfg.hidden_size, 96)
    lay = build_packed_layout(seq_len=64, block_size=16, batch=1)
    attend = LocalAttention(cfg, lay.mask)
    h = torch.randn(lay.rows, cfg.hidden_size) * 0.3
    with torch.no_grad():
        out = layer(h, lay.positions, m.inv_freq, attend)
        w_gu, w_dn = layer.w_gate_up, layer.w_down
        layer.w_gate_up = layer.w_down = None
        base = layer(h, lay.positions, m.inv_freq, attend)
        layer.w_gate_up, layer.w_down = w_gu, w_dn
        from turbo_dllm_b200.ops.norm import rmsnorm
        from turbo_dllm_b200.ops.gemm import linear_residual
        from turbo_dllm_b200.ops.rope import qk_norm_rope
        from turbo_dllm_b200.ops.gemm import linear

        y, _ = rmsnorm(h, layer.input_norm, cfg.rms_norm_eps)
        qkv = qk_norm_rope(linear(y, layer.w_qkv), lay.positions, m.inv_freq, layer.q_norm, layer.k_norm,
                           cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        h1 = linear_residual(attend(qkv, 0), layer.w_o, h)
        y2, _ = rmsnorm(h1, layer.post_norm, cfg.rms_norm_eps)
        gu = y2 @ w_gu.t()
        dense = (torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]) @ w_dn.t()
    assert torch.allclose(out, base + dense, rtol=1e-4, atol=1e-5)
    # whole model under checkpointing: the replay finds the recorded routes and uses them
    tokens = torch.randint(0, cfg.vocab_size, (lay.rows,), generator=torch.Generator().manual_seed(1))
    seen = []
    bank = m.layers[1].experts
    orig = bank._route

    def spy(logits, k):
        had = bank.store.replaying and bank.store.has((1, "moe_route"))
        w, idx = orig(logits, k)
        seen.append((bool(bank.store.recording), bool(had), idx.clone()))
        return w, idx

    bank._route = spy
    m(tokens, lay.positions, attend).square().sum().backward()
    assert [s[:2] for s in seen] == [(True, False), (False, True)] and torch.equal(seen[0][2], seen[1][2])
    assert not any(isinstance(k, tuple) and k[1] == "moe_route" for k in m.store.kept)
    assert m.flat.params["layers.0.w_gate_up"].main_grad.abs().sum() > 0


def _ep_checkpoint(rank, world, src, out):
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.models.export import export_moe_checkpoint
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": src, "seq_len": 128, "dtype": "fp32", "family": "diffusion_gemma"},
        "objective": {"name": "standard_block_diffusion", "block_size": 32},
        "training": {"batch_size": 1, "steps": 1},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1, "expert_parallel_size": 2}}).validate(world_size=world)
    s = TrainingSession(spec, device="cpu", runtime=build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world))
    bank = s.model.layers[1].experts
    export_moe_checkpoint(s.model, out)
    return bank.ep_rank, bank.e_local, bank.w_down.detach().clone()


@pytest.mark.distributed
def test_expert_parallel_ranks_load_their_experts_and_export_all(tmp_path):
    """From one checkpoint, each expert-parallel rank loads its own experts; exporting from the two ranks writes the
    file back tensor for tensor."""
    from safetensors import safe_open

    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.export import export_moe_checkpoint
    from turbo_dllm_b200.models.moe import MoEBlockDiffusionTransformer

    full = MoEBlockDiffusionTransformer(PRESETS["synthetic:tiny-moe"], dtype=torch.float32, device="cpu", seed=4, init_std=0.05)
    src, out = str(tmp_path / "src"), str(tmp_path / "out")
    export_moe_checkpoint(full, src)
    res = run_ranks(_ep_checkpoint, 2, args=(src, out), deadline_s=240)
    for ep_rank, e_local, w_down in res:
        want = full.layers[1].experts.w_down[ep_rank * e_local:(ep_rank + 1) * e_local]
        assert e_local == 4 and torch.equal(torch.as_tensor(w_down), want)
    with safe_open(src + "/model.safetensors", framework="pt") as a, safe_open(out + "/model.safetensors", framework="pt") as b:
        assert set(a.keys()) == set(b.keys())
        for k in a.keys():
            assert torch.equal(a.get_tensor(k), b.get_tensor(k)), k


def _moe_parallel(rank, world, tp, cp, bp, sp, ep=1, steps=2):
    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-moe", "seq_len": 128, "dtype": "fp32", "family": "diffusion_gemma", "num_layers": 2,
                  "moe_shared_intermediate_size": 64},
        "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
        "training": {"batch_size": 2, "steps": steps},
        "topology": {"context_parallel_size": cp, "block_parallel_size": bp, "tensor_parallel_size": tp,
                     "sequence_parallel": sp, "expert_parallel_size": ep},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device="cpu", runtime=rt)
    losses = []
    for _ in range(steps):
        r = s.step()
        t = r.loss_sum.double().clone()
        if world > 1:
            dist.all_reduce(t)
        losses.append(float(t) / r.denominator / tp)
    p = s.model.flat.params
    return (losses, s.optimizer.grad_norm(), p["layers.0.router"].detach().clone(), p["layers.1.experts_down"].detach().clone(),
            p["layers.0.post_norm"].detach().clone(), p["layers.1.w_down"].detach().clone())


@pytest.mark.distributed
@pytest.mark.parametrize("world,tp,cp,bp,sp", [(2, 2, 1, 1, False), (2, 2, 1, 1, True), (4, 2, 2, 2, True)])
def test_moe_decoder_under_tensor_and_sequence_parallelism(world, tp, cp, bp, sp):
    """Attention and the dense branch sharded over the tensor-parallel ranks, router and experts replicated; with
    sequence parallelism every rank routes its own rows and the partial gradients of router, experts and norms are
    summed. Alone and together with context-sharded block parallelism the step equals the single-process one."""
    from tests._harness import assert_params_close

    ref = _moe_parallel(0, 1, 1, 1, 1, False)
    for r, out in enumerate(run_ranks(_moe_parallel, world, args=(tp, cp, bp, sp), deadline_s=600)):
        assert out[0] == pytest.approx(ref[0], rel=2e-4, abs=2e-4)
        assert out[1] == pytest.approx(ref[1], rel=3e-3)
        for i in (2, 3, 4):                                # router, experts, layer norm: replicated
            assert_params_close(out[i], ref[i], rtol=2e-3, atol=2e-5)
        n = ref[5].shape[1] // tp                           # dense branch: row-parallel columns of this rank
        # (ranks are laid out with the tensor-parallel coordinate fastest)
        assert_params_close(out[5], ref[5][:, (r % tp) * n:(r % tp + 1) * n], rtol=2e-3, atol=2e-5)


@pytest.mark.distributed
def test_moe_tensor_parallelism_composes_with_expert_parallelism():
    """Tensor x expert parallelism (4 ranks) against expert parallelism alone (2 ranks): same data-parallel width and
    the same experts per expert-parallel coordinate, so losses, norm and weights must agree."""
    from tests._harness import assert_params_close

    a = run_ranks(_moe_parallel, 2, args=(1, 1, 1, False, 2), deadline_s=600)
    b = run_ranks(_moe_parallel, 4, args=(2, 1, 1, True, 2), deadline_s=600)
    assert b[0][0] == pytest.approx(a[0][0], rel=2e-4, abs=2e-4) and b[0][1] == pytest.approx(a[0][1], rel=3e-3)
    for rb in b:
        assert_params_close(rb[2], torch.as_tensor(a[0][2]), rtol=2e-3, atol=2e-5)          # router: replicated everywhere
        # this rank's experts equal those of exactly one expert-parallel coordinate of the 2-rank run
        close = [float((torch.as_tensor(rb[3]) - torch.as_tensor(ra[3])).abs().max()) < 1e-4 for ra in a]
        assert sum(close) == 1


def _native_sft(rank, world, cp, bp, ep, steps=3):
    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-moe", "seq_len": 128, "dtype": "fp32", "family": "diffusion_gemma", "num_layers": 2},
        "objective": {"name": "diffusiongemma_native_sft", "block_size": 32, "noise_schedule": "loglinear",
                      "loss_weighting": "unit", "self_conditioning_probability": 0.5, "sampling_epsilon_min": 0.1},
        "training": {"batch_size": 1, "steps": steps},
        "topology": {"context_parallel_size": cp, "block_parallel_size": bp, "expert_parallel_size": ep},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    s = TrainingSession(spec, device="cpu", runtime=build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world))
    losses = []
    for _ in range(steps):
        r = s.step()
        t = r.loss_sum.double().clone()
        dist.all_reduce(t)
        losses.append(float(t) / r.denominator)
    return losses, s.optimizer.grad_norm()


@pytest.mark.distributed
def test_self_conditioning_pass_is_collective_over_expert_parallel_ranks():
    """Expert-parallel ranks hold different samples; with one sample per rank and probability 0.5 they often disagree on
    whether a sample is self-conditioned. The first pass exchanges tokens among them, so all of them run it when any
    needs it (a rank deciding alone left the others waiting in the exchange). EP 2 alone and EP 2 x CSBP 2 agree."""
    a = run_ranks(_native_sft, 2, args=(1, 1, 2), deadline_s=300)
    b = run_ranks(_native_sft, 4, args=(2, 2, 2), deadline_s=600)
    assert b[0][0] == pytest.approx(a[0][0], rel=2e-4, abs=2e-4) and b[0][1] == pytest.approx(a[0][1], rel=3e-3)
