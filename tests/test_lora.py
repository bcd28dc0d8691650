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
