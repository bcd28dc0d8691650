"""Hybrid (Gated DeltaNet + gated softmax attention) block-diffusion model on CPU.

The packed model is compared with a plain per-sequence oracle: for a noisy block b the oracle runs
the sequence `[clean tokens of blocks < b ; noisy tokens of block b]` token by token (recurrence) and
with a dense block-causal softmax (attention layers). Modelled on the reference's
tests/unit/models/ Qwen3.8 DeltaNet tests (packed model against a reference recurrence)."""
import math

import pytest
import torch
import torch.nn.functional as F

from turbo_dllm_b200.models.config import PRESETS
from turbo_dllm_b200.models.dense import LocalAttention
from turbo_dllm_b200.models.hybrid import BlockRows, HybridBlockDiffusionTransformer, _HeadShard
from turbo_dllm_b200.ops.gated_delta import (causal_conv_reference, expand_key_heads, gated_delta_reference,
                                              gated_rmsnorm, gdn_gate, l2_normalize)
from turbo_dllm_b200.ops.rope import qk_norm_rope
from turbo_dllm_b200.parallel.layout import build_packed_layout

CFG = PRESETS["synthetic:tiny-qwen3_8"]


def _rms(x, w, eps):
    x = x.float()
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()


def _mlp(layer, h, eps):
    y = _rms(h, layer.post_norm, eps)
    gu = y @ layer.w_gate_up.float().t()
    return h + (F.silu(gu[:, 0::2]) * gu[:, 1::2]) @ layer.w_down.float().t()


def oracle_forward(model, tokens, positions, block_size):
    """One sequence [T] -> final-norm hidden states [T, H], no packing, no chunking."""
    c = model.cfg
    h = model.embed.float()[tokens]
    blk = positions // block_size
    visible = blk[None, :] <= blk[:, None]
    for layer, kind in zip(model.layers, model.layer_kinds):
        y = _rms(h, layer.input_norm, c.rms_norm_eps)
        if kind == "linear_attention":
            p = (y @ layer.w_in.float().t())[None]
            qkv, z, b, a = layer._split(p, _HeadShard(layer))
            conv = causal_conv_reference(qkv, layer.conv_w, layer.conv_b)
            kd = c.linear_key_dim
            T = tokens.shape[0]
            q = l2_normalize(conv[..., :kd].reshape(1, T, c.linear_num_key_heads, -1))
            k = l2_normalize(conv[..., kd:2 * kd].reshape(1, T, c.linear_num_key_heads, -1))
            v = conv[..., 2 * kd:].reshape(1, T, c.linear_num_value_heads, -1)
            q, k = expand_key_heads(q, c.linear_num_value_heads), expand_key_heads(k, c.linear_num_value_heads)
            o, _, _ = gated_delta_reference(q, k, v, gdn_gate(a, layer.A_log, layer.dt_bias), torch.sigmoid(b))
            o = gated_rmsnorm(o, z.reshape(1, T, c.linear_num_value_heads, -1), layer.gdn_norm, c.rms_norm_eps)
            h = h + o.reshape(T, -1) @ layer.w_out.float().t()
        else:
            qkv = qk_norm_rope(y @ layer.w_qkv.float().t(), positions.to(torch.int32), model.inv_freq, layer.q_norm,
                               layer.k_norm, c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.rms_norm_eps)
            T, D = tokens.shape[0], c.head_dim
            q = qkv[:, :c.q_dim].reshape(T, c.num_attention_heads, D)
            k = qkv[:, c.q_dim:c.q_dim + c.kv_dim].reshape(T, c.num_key_value_heads, D)
            v = qkv[:, c.q_dim + c.kv_dim:].reshape(T, c.num_key_value_heads, D)
            rep = c.num_attention_heads // c.num_key_value_heads
            k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
            s = torch.einsum("qhd,khd->hqk", q.float(), k.float()) / math.sqrt(D)
            s = s.masked_fill(~visible[None], float("-inf"))
            a = torch.einsum("hqk,khd->qhd", s.softmax(-1), v.float()).reshape(T, -1)
            a = a * torch.sigmoid(y @ layer.w_attn_gate.float().t())
            h = h + a @ layer.w_o.float().t()
        h = _mlp(layer, h, c.rms_norm_eps)
    return _rms(h, model.final_norm, c.rms_norm_eps)


def _packed(model, clean, noisy, layout):
    """clean [B, S], noisy [B, views, S] -> packed hidden states."""
    tokens = torch.cat([noisy[layout.noisy_seq, layout.noisy_view, layout.noisy_pos],
                        clean[layout.clean_seq, layout.clean_pos]])
    attend = LocalAttention(model.cfg, layout.mask, store=model.store)
    attend.block_rows = BlockRows(layout, clean.shape[1])
    return model(tokens, layout.positions, attend)


@pytest.mark.parametrize("views", [1, 2])
def test_packed_model_matches_per_sequence_oracle(views):
    torch.manual_seed(0)
    S, bs, B = 32, 8, 2
    model = HybridBlockDiffusionTransformer(CFG, dtype=torch.float32, activation_checkpointing=False, seed=3,
                                            init_std=0.08, branch_group=3)
    assert model.layer_kinds == ("linear_attention",) * 3 + ("full_attention",)
    clean = torch.randint(0, CFG.vocab_size - 1, (B, S))
    noisy = torch.where(torch.rand(B, views, S) < 0.5, torch.full((B, views, S), CFG.mask_token_id), clean[:, None])
    layout = build_packed_layout(seq_len=S, block_size=bs, batch=B, views=views)
    with torch.no_grad():
        got = _packed(model, clean, noisy, layout)
        pos = torch.arange(S)
        # clean rows: the plain block-causal run over the clean sequence
        for b in range(B):
            want = oracle_forward(model, clean[b], pos, bs)
            rows = layout.n_noisy + b * S + pos
            assert torch.allclose(got[rows], want, atol=2e-4, rtol=2e-3)
        # noisy blocks: clean prefix + the block's own noisy tokens
        for (b, v, blk) in [(0, 0, 0), (1, views - 1, 2), (0, views - 1, 3)]:
            lo, hi = blk * bs, (blk + 1) * bs
            seq = torch.cat([clean[b, :lo], noisy[b, v, lo:hi]])
            want = oracle_forward(model, seq, pos[:hi], bs)[lo:]
            sel = ((layout.noisy_seq == b) & (layout.noisy_view == v) & (layout.noisy_pos >= lo)
                   & (layout.noisy_pos < hi)).nonzero(as_tuple=True)[0]
            assert sel.numel() == bs
            assert torch.allclose(got[sel], want, atol=2e-4, rtol=2e-3)


def test_checkpointed_layers_give_the_same_gradients():
    S, bs, B = 32, 8, 1
    clean = torch.randint(0, CFG.vocab_size - 1, (B, S), generator=torch.Generator().manual_seed(1))
    noisy = clean[:, None].clone()
    noisy[:, :, ::3] = CFG.mask_token_id
    layout = build_packed_layout(seq_len=S, block_size=bs, batch=B, views=1)
    grads = []
    for ckpt in (False, True):
        model = HybridBlockDiffusionTransformer(CFG, dtype=torch.float32, activation_checkpointing=ckpt, seed=5,
                                                init_std=0.05)
        model.flat.zero_grad()
        out = _packed(model, clean, noisy, layout)
        out[: layout.n_noisy].float().square().sum().backward()
        model.flat.collect_grads()
        grads.append(model.flat.grad.clone())
    assert grads[0].abs().sum() > 0
    assert torch.allclose(grads[0], grads[1], atol=1e-5, rtol=1e-4)
    # the noisy rows' loss reaches the recurrence parameters of the first (linear-attention) layer
    for leaf in ("A_log", "dt_bias", "conv_w", "w_in"):
        assert model.flat.params[f"layers.0.{leaf}"].main_grad.abs().sum() > 0


def test_block_rows_rejects_sharded_clean_rows():
    layout = build_packed_layout(seq_len=32, block_size=8, batch=1, views=1, clean_pos=torch.arange(0, 16))
    with pytest.raises(ValueError):
        BlockRows(layout, 32)


def test_training_session_steps_on_the_hybrid_family():
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.training.session import TrainingSession

    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3_8", "family": "qwen3_8", "seq_len": 64, "dtype": "fp32"},
        "objective": {"name": "fast_dllm_v2", "block_size": 16},
        "training": {"batch_size": 2, "steps": 3, "activation_checkpointing": True},
        "optimizer": {"lr": 3e-3},
        "data": {"input_mode": "random", "vocab_sample_size": 8},
    }).validate()
    session = TrainingSession(spec, device="cpu")
    losses = []
    for _ in range(4):
        r = session.step()
        losses.append(float(r.loss_sum) / r.denominator)
    assert all(math.isfinite(x) for x in losses)
    assert losses[-1] < losses[0]


# ------------------------------------------------------------------ context sharding (gloo ranks)
def _exchange_worker(rank, world):
    import torch.distributed as dist

    from turbo_dllm_b200.parallel.head_sequence import head_to_sequence_parallel, sequence_to_head_parallel

    counts = [3, 5]                      # rows held by rank 0 and rank 1
    F = 4                                # features per head shard
    g = torch.Generator().manual_seed(10)
    full = [torch.randn(c, world * F, generator=g) for c in counts]      # every rank's rows, all heads
    mine = full[rank].clone().requires_grad_(True)
    parts = [mine[:, r * F:(r + 1) * F] for r in range(world)]
    got = sequence_to_head_parallel(parts, counts, dist.group.WORLD)
    want = torch.cat([f[:, rank * F:(rank + 1) * F] for f in full])
    ok_fwd = torch.allclose(got, want)
    back = head_to_sequence_parallel(got * 2.0, counts, rank, dist.group.WORLD)
    ok_back = torch.allclose(back, 2.0 * full[rank])
    w = torch.arange(back.numel(), dtype=torch.float32).view_as(back)
    (back * w).sum().backward()
    ok_grad = torch.allclose(mine.grad, 2.0 * w)
    return [bool(ok_fwd), bool(ok_back), bool(ok_grad)]


@pytest.mark.distributed
def test_head_sequence_exchange_round_trip_and_gradient():
    from tests._harness import assert_params_close, run_ranks

    for flags in run_ranks(_exchange_worker, 2, deadline_s=120):
        assert all(flags), flags


def _hybrid_run(rank, world, cp, bp, steps):
    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3_8", "family": "qwen3_8", "seq_len": 128, "dtype": "fp32"},
        "objective": {"name": "fast_dllm_v2", "block_size": 16, "sampling_epsilon_min": 0.1},
        "training": {"batch_size": 2, "steps": steps, "activation_checkpointing": True},
        "topology": {"context_parallel_size": cp, "block_parallel_size": bp, "replicate_clean_prefix": cp == 1 and bp > 1},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device="cpu", runtime=rt)
    losses = []
    for _ in range(steps):
        r = s.step()
        t = r.loss_sum.double().clone()
        if world > 1:
            dist.all_reduce(t)
        losses.append(float(t) / r.denominator)
    return losses, s.model.flat.data.clone()


@pytest.mark.distributed
@pytest.mark.parametrize("cp,bp", [(2, 2), (1, 2)])
def test_hybrid_context_sharded_run_matches_single_process(cp, bp):
    """Two gloo ranks. CSBP degree 2 (clean rows and blocks sharded): the linear-attention layers trade row shards
    for head shards and back. Block parallelism alone: every rank keeps the whole clean sequence (the layers' chunk
    states are indexed by position) and its own noisy blocks. Losses and parameters follow the single-process run."""
    from tests._harness import assert_params_close, run_ranks

    ref_losses, ref_params = _hybrid_run(0, 1, 1, 1, 2)
    outs = run_ranks(_hybrid_run, 2, args=(cp, bp, 2), deadline_s=300)
    for losses, params in outs:
        assert losses == pytest.approx(ref_losses, rel=2e-4, abs=2e-4)
        assert_params_close(params, ref_params)


def test_lora_on_the_hybrid_family_trains_adapters_only_and_merges():
    from turbo_dllm_b200.adapters.lora import apply_lora, merge_lora

    S, bs, B = 32, 8, 1
    model = HybridBlockDiffusionTransformer(CFG, dtype=torch.float32, activation_checkpointing=True, seed=9,
                                            init_std=0.05)
    st = apply_lora(model, rank=4, alpha=8.0, targets=("attention", "mlp"), seed=1)
    names = set(n.split(".", 2)[2].rsplit(".", 1)[0] for n in st.flat.params)
    assert {"w_in", "w_out", "w_qkv", "w_o", "w_attn_gate", "w_gate_up", "w_down"} <= names
    with torch.no_grad():       # non-zero B so that the adapters change the output
        for n, p in st.flat.params.items():
            if n.endswith("lora_B"):
                p.normal_(0, 0.05)
    clean = torch.randint(0, CFG.vocab_size - 1, (B, S), generator=torch.Generator().manual_seed(2))
    noisy = clean[:, None].clone()
    noisy[:, :, ::2] = CFG.mask_token_id
    layout = build_packed_layout(seq_len=S, block_size=bs, batch=B, views=1)
    st.flat.zero_grad()
    out = _packed(model, clean, noisy, layout)
    out.square().sum().backward()
    st.flat.collect_grads()
    assert st.flat.grad.abs().sum() > 0
    assert all(p.grad is None and not p.requires_grad for p in model.flat.params.values())
    with torch.no_grad():
        with_adapters = _packed(model, clean, noisy, layout)
        merge_lora(model)
        for layer in model.layers:
            layer.lora = None
        model.lora = None
        merged = _packed(model, clean, noisy, layout)
    assert torch.allclose(with_adapters, merged, atol=2e-4, rtol=1e-3)


def test_hybrid_hugging_face_round_trip(tmp_path):
    from turbo_dllm_b200.models.hf_loader import export_hf_checkpoint, load_hf_config, load_hf_weights

    a = HybridBlockDiffusionTransformer(CFG, dtype=torch.float32, seed=11, init_std=0.05)
    with torch.no_grad():
        for n, p in a.flat.params.items():          # make every tensor distinctive, norms and biases included
            if not p.decay:
                p.add_(torch.randn_like(p) * 0.1)
    path = export_hf_checkpoint(a, str(tmp_path / "hf"))
    cfg = load_hf_config(path)
    assert cfg.is_hybrid and cfg.linear_num_value_heads == CFG.linear_num_value_heads
    assert [cfg.layer_kind(i) for i in range(cfg.num_layers)] == list(a.layer_kinds)
    from safetensors import safe_open

    with safe_open(path + "/model.safetensors", framework="pt") as f:
        keys = set(f.keys())
        q = f.get_tensor("model.layers.3.self_attn.q_proj.weight")
    assert "model.layers.0.linear_attn.in_proj_qkv.weight" in keys and "model.layers.0.linear_attn.A_log" in keys
    assert q.shape == (2 * CFG.q_dim, CFG.hidden_size)
    # per head: query rows then gate rows
    D = CFG.head_dim
    assert torch.equal(q[:D], a.layers[3].w_qkv[:D]) and torch.equal(q[D:2 * D], a.layers[3].w_attn_gate[:D])
    import dataclasses

    b = HybridBlockDiffusionTransformer(dataclasses.replace(cfg, mask_token_id=CFG.mask_token_id),
                                        dtype=torch.float32, seed=99, init_std=0.02)
    load_hf_weights(b, path)
    for n, p in a.flat.params.items():
        assert torch.equal(p, b.flat.params[n]), n


def test_head_shards_partition_the_projection_and_plan_checks_coverage():
    from turbo_dllm_b200.models.hybrid import HeadParallelPlan

    model = HybridBlockDiffusionTransformer(CFG, dtype=torch.float32, seed=1)
    layer = model.layers[0]
    shards = [_HeadShard(layer, r, 2) for r in range(2)]
    cols = torch.cat([s.columns for s in shards])
    real = CFG.linear_conv_channels + CFG.linear_value_dim + 2 * CFG.linear_num_value_heads
    assert cols.numel() == real and torch.equal(cols.sort().values, torch.arange(real))
    assert shards[0].hk == CFG.linear_num_key_heads // 2 and shards[1].A_log.shape[0] == CFG.linear_num_value_heads // 2
    with pytest.raises(ValueError):
        _HeadShard(layer, 0, 4)          # two key heads cannot be split four ways
    blocks = (torch.zeros(2, dtype=torch.long), torch.tensor([0, 8]))
    ok = HeadParallelPlan(group=None, index=0, noisy_blocks=[blocks, blocks],
                          clean_positions=[torch.arange(0, 8), torch.arange(8, 16)], batch=1, seq_len=16,
                          block_size=8, device="cpu")
    assert ok.total_rows == 2 * (16 + 8) and ok.row_counts == [24, 24]
    # gathered row of (sequence 0, position p): rank 0 holds positions 0..7 after its 16 noisy rows
    assert ok.clean_rows.tolist() == list(range(16, 24)) + list(range(40, 48))
    with pytest.raises(ValueError):      # position 8..15 missing, 0..7 twice
        HeadParallelPlan(group=None, index=0, noisy_blocks=[blocks, blocks],
                         clean_positions=[torch.arange(0, 8), torch.arange(0, 8)], batch=1, seq_len=16,
                         block_size=8, device="cpu")


def _hybrid_tp_cp_run(rank, world, tp, cp, bp, sp, steps=2):
    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3_8", "family": "qwen3_8", "seq_len": 128, "dtype": "fp32",
                  "linear_num_key_heads": 4, "linear_num_value_heads": 8},
        "objective": {"name": "fast_dllm_v2", "block_size": 16, "sampling_epsilon_min": 0.1},
        "training": {"batch_size": 2, "steps": steps, "activation_checkpointing": True},
        "topology": {"context_parallel_size": cp, "block_parallel_size": bp, "tensor_parallel_size": tp,
                     "sequence_parallel": sp},
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
    return (losses, s.optimizer.grad_norm(), p["layers.0.gdn_norm"].detach().clone(), p["layers.1.post_norm"].detach().clone(),
            p["layers.3.q_norm"].detach().clone())


@pytest.mark.distributed
def test_hybrid_tensor_sequence_and_context_parallelism_together():
    """The shape of the family's large recipes in miniature: tensor parallelism 2 with sequence parallelism, times
    context-sharded block parallelism 2 (4 gloo ranks). Linear-attention layers own 1/2 of the heads per tensor-parallel
    rank and trade row shards for a further 1/2 of those heads inside the context group."""
    from tests._harness import assert_params_close, run_ranks

    ref = _hybrid_tp_cp_run(0, 1, 1, 1, 1, False)
    outs = run_ranks(_hybrid_tp_cp_run, 4, args=(2, 2, 2, True), deadline_s=600)
    for losses, norm, gdn_norm, post_norm, q_norm in outs:
        assert losses == pytest.approx(ref[0], rel=2e-4, abs=2e-4)
        assert norm == pytest.approx(ref[1], rel=3e-3)
        for got, want in ((gdn_norm, ref[2]), (post_norm, ref[3]), (q_norm, ref[4])):      # replicated, partial gradients summed
            assert_params_close(got, want, rtol=2e-3, atol=2e-5)
