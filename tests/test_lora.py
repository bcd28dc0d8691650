"""LoRA adapters on the dense decoder: only the adapters train, and merging them into the weights
reproduces the adapted model (dllm_parallel/core/adapters/lora.py:26-130, :591-627)."""
import torch

from turbo_dllm_b200.adapters.lora import apply_lora, merge_lora
from turbo_dllm_b200.models.config import PRESETS
from turbo_dllm_b200.models.dense import BlockDiffusionTransformer, LocalAttention
from turbo_dllm_b200.parallel.layout import build_packed_layout


def _run(model, tokens, layout):
    return model(tokens, layout.positions, LocalAttention(model.cfg, layout.mask, store=model.store))


def test_dense_lora_trains_adapters_only_and_merges():
    cfg = PRESETS["synthetic:tiny-qwen3"]
    model = BlockDiffusionTransformer(cfg, dtype=torch.float32, activation_checkpointing=True, seed=2, init_std=0.05)
    st = apply_lora(model, rank=4, alpha=8.0, targets=("attention", "mlp"), seed=3)
    assert st.flat.numel < model.flat.numel // 4
    with torch.no_grad():
        for n, p in st.flat.params.items():
            if n.endswith("lora_B"):
                p.normal_(0, 0.05)
    layout = build_packed_layout(seq_len=64, block_size=16, batch=1, views=1)
    tokens = torch.randint(0, cfg.vocab_size, (layout.rows,), generator=torch.Generator().manual_seed(4))
    st.flat.zero_grad()
    _run(model, tokens, layout).square().sum().backward()
    st.flat.collect_grads()
    assert st.flat.grad.abs().sum() > 0
    assert all(p.grad is None and not p.requires_grad for p in model.flat.params.values())
    with torch.no_grad():
        adapted = _run(model, tokens, layout)
        merge_lora(model)
        for layer in model.layers:
            layer.lora = None
        model.lora = None
        merged = _run(model, tokens, layout)
    assert torch.allclose(adapted, merged, atol=2e-4, rtol=1e-3)


def test_unknown_role_is_rejected():
    import pytest

    cfg = PRESETS["synthetic:tiny-qwen3"]
    model = BlockDiffusionTransformer(cfg, dtype=torch.float32, seed=2)
    with pytest.raises(ValueError):
        apply_lora(model, rank=4, targets=("router",))
    with pytest.raises(ValueError):
        apply_lora(model, rank=0)


def test_expert_adapters_train_and_merge():
    """Mixture-of-experts decoder: replicated pairs on the attention projections, per-expert pairs on the stacked
    gate/up and down weights; the frozen experts get no gradient, merging reproduces the adapted model."""
    from turbo_dllm_b200.models.moe import MoEBlockDiffusionTransformer

    cfg = PRESETS["synthetic:tiny-moe"]
    model = MoEBlockDiffusionTransformer(cfg, dtype=torch.float32, seed=2, init_std=0.05)
    st = apply_lora(model, rank=4, alpha=8.0, targets=("attention", "experts"), seed=3)
    assert st.flat_experts is not None and all(b.lora is st for b in (l.experts for l in model.layers))
    with torch.no_grad():
        for flat in (st.flat, st.flat_experts):
            for n, p in flat.params.items():
                if n.endswith("lora_B"):
                    p.normal_(0, 0.05)
    layout = build_packed_layout(seq_len=64, block_size=16, batch=1, views=1)
    tokens = torch.randint(0, cfg.vocab_size, (layout.rows,), generator=torch.Generator().manual_seed(4))
    for f in (st.flat, st.flat_experts, model.flat_experts):
        f.zero_grad()
    model.flat_experts.grad.zero_()
    _run(model, tokens, layout).square().sum().backward()
    st.flat.collect_grads()
    st.flat_experts.collect_grads()
    assert st.flat.grad.abs().sum() > 0 and st.flat_experts.grad.abs().sum() > 0
    assert model.flat_experts.grad.abs().sum() == 0           # the experts themselves are frozen
    with torch.no_grad():
        adapted = _run(model, tokens, layout)
        merge_lora(model)
        for layer in model.layers:
            layer.lora = None
            layer.experts.lora = None
        model.lora = None
        merged = _run(model, tokens, layout)
    assert torch.allclose(adapted, merged, atol=3e-4, rtol=1e-3)


def test_moe_session_trains_only_the_adapters():
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.training.session import TrainingSession

    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-moe", "seq_len": 64, "dtype": "fp32", "family": "diffusion_gemma"},
        "objective": {"name": "standard_block_diffusion", "block_size": 16, "sampling_epsilon_min": 0.1},
        "adapter": {"type": "lora", "rank": 4, "alpha": 8.0, "targets": ["attention", "experts"]},
        "training": {"batch_size": 2, "steps": 3},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
        "optimizer": {"lr": 1e-2, "gradient_clip_norm": 1.0}}).validate()
    s = TrainingSession(spec, device="cpu")
    base = s.model.flat.data.clone(), s.model.flat_experts.data.clone()
    a0 = s.lora.flat_experts.data.clone()
    losses = [float(r.loss_sum) / r.denominator for r in (s.step() for _ in range(4))]
    assert losses[-1] < losses[0]
    assert torch.equal(s.model.flat.data, base[0]) and torch.equal(s.model.flat_experts.data, base[1])
    assert not torch.equal(s.lora.flat_experts.data, a0)
    state = s.state_dict()
    assert "adapter" in state and "adapter_experts" in state


def test_moe_export_merges_adapters_by_a_checked_plan(tmp_path):
    """Export of a mixture-of-experts model with adapters: the plan lists linear and grouped merges with their
    shapes (and refuses a pair that does not fit), the written expert weights are the merged ones, the dense
    branch beside the experts is exported too."""
    from dataclasses import replace

    import pytest
    from safetensors import safe_open

    from turbo_dllm_b200.adapters.lora import lora_merge_plan
    from turbo_dllm_b200.models.export import export_moe_checkpoint
    from turbo_dllm_b200.models.hf_loader import interleave_gate_up
    from turbo_dllm_b200.models.moe import MoEBlockDiffusionTransformer

    cfg = replace(PRESETS["synthetic:tiny-moe"], moe_shared_intermediate_size=64, num_layers=1)
    model = MoEBlockDiffusionTransformer(cfg, dtype=torch.float32, seed=2, init_std=0.05)
    st = apply_lora(model, rank=4, alpha=8.0, targets=("attention", "experts"), seed=3)
    with torch.no_grad():
        for flat in (st.flat, st.flat_experts):
            for n, p in flat.params.items():
                if n.endswith("lora_B"):
                    p.normal_(0, 0.05)
    plan = lora_merge_plan(model)
    kinds = {e["target"]: e["kind"] for e in plan}
    assert kinds["layers.0.experts_gate_up"] == "grouped" and kinds["layers.0.w_qkv"] == "linear"
    bank = model.layers[0].experts
    a, b = st.expert_pair(0, "experts_down")
    want_down = bank.w_down.detach() + torch.bmm(b.float(), a.float()) * st.scale
    a, b = st.expert_pair(0, "experts_gate_up")
    want_gu = bank.w_gu.detach() + torch.bmm(b.float(), a.float()) * st.scale
    export_moe_checkpoint(model, str(tmp_path / "out"))
    assert model.lora is None
    with safe_open(str(tmp_path / "out" / "model.safetensors"), "pt") as f:
        names = set(f.keys())
        down3 = f.get_tensor("model.layers.0.mlp.experts.3.down_proj.weight")
        g3 = f.get_tensor("model.layers.0.mlp.experts.3.gate_proj.weight")
        u3 = f.get_tensor("model.layers.0.mlp.experts.3.up_proj.weight")
    assert torch.allclose(down3, want_down[3], atol=1e-6)
    assert torch.allclose(interleave_gate_up(g3, u3), want_gu[3], atol=1e-6)
    assert "model.layers.0.mlp.shared_expert.down_proj.weight" in names
    # a pair that does not fit its target is refused before anything is merged
    model2 = MoEBlockDiffusionTransformer(cfg, dtype=torch.float32, seed=2, init_std=0.05)
    st2 = apply_lora(model2, rank=4, targets=("attention", "experts"), seed=3)
    good = st2.flat.params["layers.0.w_o.lora_B"]
    st2.flat.params["layers.0.w_o.lora_B"] = torch.nn.Parameter(good.detach()[:-1].clone())
    with pytest.raises(ValueError, match="does not fit"):
        lora_merge_plan(model2)


def test_token_mask_limits_the_adapters_to_selected_rows():
    """Inside `lora_token_mask` the adapters change only the selected rows and take gradients only from them, also when
    a checkpointed layer is recomputed in the backward pass; `False` switches the adapters off."""
    from turbo_dllm_b200.adapters.lora import current_lora_token_mask, lora_token_mask

    cfg = PRESETS["synthetic:tiny-qwen3"]
    model = BlockDiffusionTransformer(cfg, dtype=torch.float32, activation_checkpointing=True, seed=2, init_std=0.05)
    base = BlockDiffusionTransformer(cfg, dtype=torch.float32, activation_checkpointing=True, seed=2, init_std=0.05)
    st = apply_lora(model, rank=4, alpha=8.0, targets=("mlp",), seed=3)
    with torch.no_grad():
        for n, p in st.flat.params.items():
            if n.endswith("lora_B"):
                p.normal_(0, 0.05)
    # one layer, so rows do not mix after the adapted feed-forward
    model.layers = model.layers[:1]
    base.layers = base.layers[:1]
    layout = build_packed_layout(seq_len=64, block_size=16, batch=1, views=1)
    tokens = torch.randint(0, cfg.vocab_size, (layout.rows,), generator=torch.Generator().manual_seed(4))
    mask = torch.zeros(layout.rows, dtype=torch.bool)
    mask[::3] = True
    with torch.no_grad():
        plain = _run(base, tokens, layout)
        everywhere = _run(model, tokens, layout)
        with lora_token_mask(mask):
            assert current_lora_token_mask() is mask
            some = _run(model, tokens, layout)
        with lora_token_mask(False):
            off = _run(model, tokens, layout)
    assert current_lora_token_mask() is None
    assert torch.allclose(off, plain, atol=1e-6) and not torch.allclose(everywhere, plain, atol=1e-4)
    assert torch.allclose(some[~mask], plain[~mask], atol=1e-6) and torch.allclose(some[mask], everywhere[mask], atol=1e-6)
    # gradients: only the selected rows reach the adapters (the replay in the checkpointed backward sees the mask)
    def adapter_grad(m, weight_rows):
        st.flat.zero_grad()
        with lora_token_mask(m):
            (_run(model, tokens, layout) * weight_rows[:, None]).sum().backward()
        st.flat.collect_grads()
        return st.flat.grad.clone()

    ones = torch.ones(layout.rows)
    g_masked = adapter_grad(mask, ones)
    g_selected_rows_only = adapter_grad(None, mask.float())
    assert g_masked.abs().sum() > 0
    # the loss on unselected rows still reaches layer-0 adapters through attention in deeper layers; with one layer it
    # cannot, so both gradients agree
    assert torch.allclose(g_masked, g_selected_rows_only, atol=1e-5, rtol=1e-4)
