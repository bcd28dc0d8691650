import pytest
import torch

from turbo_dllm_b200.objectives.dflash import DFlashObjectiveRuntime, document_starts, reference_dflash_loss
from turbo_dllm_b200.objectives.runtime import FastDLLMv2Runtime, StandardBlockDiffusionRuntime

KW = dict(block_size=8, mask_token_id=99, max_seq_len=64, seed=11)


def test_standard_corruption_rules_and_determinism():
    rt = StandardBlockDiffusionRuntime(sampling_epsilon_min=0.1, **KW)
    x0 = torch.randint(0, 90, (3, 64))
    cb = rt.corrupt(x0)
    assert cb.noisy_input_ids.shape == (3, 1, 64) and cb.loss_weights.shape == (3, 1, 8)
    m = cb.noisy_input_ids[:, 0] == 99
    assert torch.equal(cb.labels[:, 0][m], x0[m]) and (cb.labels[:, 0][~m] == -100).all()
    assert torch.equal(cb.noisy_input_ids[:, 0][~m], x0[~m])
    assert torch.allclose(cb.loss_weights[:, 0], 1.0 / cb.diffusion_times)
    assert (cb.diffusion_times >= 0.1).all() and (cb.diffusion_times <= 1.0).all()
    assert cb.valid_tokens == 192 and int(cb.active_tokens) == int(m.sum())
    # antithetic strata: sorted times are evenly spaced by 1/N of the sampling range
    ts = ((cb.diffusion_times.flatten() - 0.1) / 0.9).sort().values
    assert torch.allclose(ts[1:] - ts[:-1], torch.full((23,), 1 / 24), atol=1e-5)
    rt2 = StandardBlockDiffusionRuntime(sampling_epsilon_min=0.1, **KW)
    assert torch.equal(rt2.corrupt(x0).noisy_input_ids, cb.noisy_input_ids)
    assert not torch.equal(rt2.corrupt(x0).noisy_input_ids, cb.noisy_input_ids)


def test_state_dict_roundtrip_resumes_the_stream():
    a = StandardBlockDiffusionRuntime(**KW)
    x0 = torch.randint(0, 90, (2, 64))
    a.corrupt(x0)
    st = a.state_dict()
    want = a.corrupt(x0).noisy_input_ids
    b = StandardBlockDiffusionRuntime(**KW)
    b.load_state_dict(st)
    assert torch.equal(b.corrupt(x0).noisy_input_ids, want)
    with pytest.raises(ValueError):
        FastDLLMv2Runtime(**KW).load_state_dict(st)


def test_fast_dllm_v2_complementary_views_and_shifted_labels():
    rt = FastDLLMv2Runtime(noise_schedule_epsilon=0.1, **KW)
    x0 = torch.randint(0, 90, (2, 64))
    cb = rt.corrupt(x0)
    a, b = cb.noisy_input_ids[:, 0] == 99, cb.noisy_input_ids[:, 1] == 99
    assert (a ^ b).all()                                   # every position masked in exactly one view
    assert cb.valid_tokens == 2 * 63 and cb.loss_denominator == 126.0
    assert (cb.labels[:, :, -1] == -100).all()
    for v, m in enumerate((a, b)):
        lab = cb.labels[:, v, :-1]
        assert torch.equal(lab[m[:, 1:]], x0[:, 1:][m[:, 1:]]) and (lab[~m[:, 1:]] == -100).all()
    assert int(cb.active_tokens) == 126                   # the two views together supervise every position once
    assert (cb.loss_weights == 1).all() and rt.exclude_mask_token is False


def test_supervision_mask_limits_masking():
    rt = StandardBlockDiffusionRuntime(**KW)
    x0 = torch.randint(0, 90, (2, 64))
    sup = torch.zeros(2, 64, dtype=torch.bool)
    sup[:, 32:] = True
    cb = rt.corrupt(x0, supervision_mask=sup)
    assert (cb.noisy_input_ids[:, 0, :32] != 99).all() and cb.valid_tokens == 64
    with pytest.raises(ValueError):
        rt.corrupt(x0[:, :60])


def test_dflash_anchor_blocks_and_document_boundaries():
    rt = DFlashObjectiveRuntime(block_size=4, max_anchors=6, mask_token_id=99, seed=3, decay_gamma=2.0)
    x = torch.randint(0, 90, (2, 40))
    docs = torch.zeros(2, 40, dtype=torch.long)
    docs[:, 20:] = 1
    assert document_starts(docs)[0, 25] == 20
    b = rt.prepare(x, document_ids=docs)
    assert b.draft_input_ids.shape == (2, 24) and b.supervised_mask.shape == (2, 24)
    d = b.draft_input_ids.view(2, 6, 4)
    assert torch.equal(d[:, :, 0], x.gather(1, b.anchor_positions)) and (d[:, :, 1:] == 99).all()
    sup = b.supervised_mask.view(2, 6, 4)
    assert not sup[:, :, 0].any()
    # no supervision across a document boundary or past the end
    tgt_doc = document_starts(docs).gather(1, b.target_token_positions.view(2, -1)).view(2, 6, 4)
    anchor_doc = document_starts(docs).gather(1, b.anchor_positions)[:, :, None]
    assert (tgt_doc[sup] == anchor_doc.expand_as(tgt_doc)[sup]).all()
    assert torch.equal(b.context_stops[b.anchor_valid].long(), b.anchor_positions[b.anchor_valid])
    assert (b.anchor_positions[:, 1:] >= b.anchor_positions[:, :-1])[b.anchor_valid[:, 1:]].all()
    w = b.position_weights.view(2, 6, 4)[0, 0]
    assert w[1] == 1.0 and w[3] < w[2] < w[1]
    s, t = torch.randn(24, 50), torch.randn(24, 50)
    loss, per = reference_dflash_loss(s, t, sup.view(2, -1)[0], b.position_weights[0])
    assert loss >= 0 and per.shape == (24,)


def test_diffusiongemma_native_replaces_tokens_and_scores_every_position():
    from turbo_dllm_b200.objectives.runtime import LABEL_IGNORE_INDEX, DiffusionGemmaNativeRuntime

    # the masked full-length form (the response stays in place); the packed form is covered by
    # tests/test_native_sft_packing.py
    rt = DiffusionGemmaNativeRuntime(vocab_size=500, self_conditioning_probability=0.5, block_size=16,
                                     mask_token_id=499, max_seq_len=128, seed=11, pack_response_suffix=False)
    x0 = torch.randint(0, 400, (6, 128))
    sup = torch.zeros_like(x0, dtype=torch.bool)
    sup[:, 32:] = True
    cb = rt.corrupt(x0, supervision_mask=sup)
    noisy, labels = cb.noisy_input_ids[:, 0], cb.labels[:, 0]
    assert cb.views == 1 and (cb.loss_weights == 1).all()
    # labels: the clean token on every scored position, nothing elsewhere
    assert (labels[:, 32:] == x0[:, 32:]).all() and (labels[:, :32] == LABEL_IGNORE_INDEX).all()
    # corruption only inside the scored region, by replacement (never the mask id by construction of this data)
    assert (noisy[:, :32] == x0[:, :32]).all()
    changed = (noisy != x0)
    assert changed.any() and int(changed.sum()) <= int(cb.replaced_tokens)
    assert cb.loss_denominator == float(sup.sum()) and int(cb.active_tokens) == int(sup.sum())
    assert cb.self_conditioning_mask.shape == (6,) and cb.self_conditioning_mask.dtype == torch.bool
    # deterministic and resumable through the batch counter alone
    rt2 = DiffusionGemmaNativeRuntime(vocab_size=500, self_conditioning_probability=0.5, block_size=16,
                                      mask_token_id=499, max_seq_len=128, seed=11, pack_response_suffix=False)
    cb2 = rt2.corrupt(x0, supervision_mask=sup)
    assert (cb2.noisy_input_ids == cb.noisy_input_ids).all()
    rt2.load_state_dict(rt.state_dict())
    a, b = rt.corrupt(x0), rt2.corrupt(x0)
    assert (a.noisy_input_ids == b.noisy_input_ids).all() and (a.self_conditioning_mask == b.self_conditioning_mask).all()


def test_streaming_soft_embedding_matches_dense_softmax():
    from turbo_dllm_b200.ops.soft_embedding import streaming_soft_embedding

    torch.manual_seed(0)
    h, w = torch.randn(37, 48), torch.randn(301, 48) * 0.3
    ref = torch.softmax(h @ w.t(), 1) @ w
    out = streaming_soft_embedding(h, w, row_chunk_size=10, vocab_chunk_size=64)
    assert torch.allclose(out, ref, atol=1e-5) and not out.requires_grad
    cap = 5.0
    ref2 = torch.softmax(cap * torch.tanh(h @ w.t() / cap), 1) @ w * 2
    out2 = streaming_soft_embedding(h.view(1, 37, 48), w, row_chunk_size=100, vocab_chunk_size=1000,
                                    logit_softcap=cap, embedding_scale=2.0)
    assert out2.shape == (1, 37, 48) and torch.allclose(out2[0], ref2, atol=1e-5)


def test_native_sft_session_step_with_self_conditioning():
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.training.session import TrainingSession

    def run(p):
        spec = RunSpec.from_mapping({
            "model": {"id": "synthetic:tiny-moe", "seq_len": 128, "dtype": "fp32"},
            "objective": {"name": "diffusiongemma_native_sft", "block_size": 16, "loss_weighting": "unit",
                          "self_conditioning_probability": p, "self_conditioning_row_chunk_size": 64,
                          "self_conditioning_vocab_chunk_size": 100},
            "training": {"batch_size": 2, "steps": 1, "skip_optimizer_step": True},
            "optimizer": {"lr": 1e-3}}).validate()
        s = TrainingSession(spec, device="cpu")
        r = s.step()
        return float(r.loss_sum) / r.denominator, s.model.flat.grad.clone()

    l0, g0 = run(0.0)
    l1, g1 = run(1.0)
    assert l0 == l0 and l1 == l1 and l0 > 0 and l1 > 0
    assert abs(l0 - l1) > 1e-6, "feeding the first pass back must change the prediction"
    assert g1.abs().sum() > 0 and not torch.allclose(g0, g1)


def test_clean_causal_layout_hides_later_tokens_of_the_block():
    import torch

    from turbo_dllm_b200.parallel.layout import build_packed_layout

    a = build_packed_layout(seq_len=16, block_size=4, batch=2, views=1)
    b = build_packed_layout(seq_len=16, block_size=4, batch=2, views=1, clean_causal=True)
    n = a.n_noisy
    assert torch.equal(a.mask.q_hi[:n], b.mask.q_hi[:n])                # noisy rows unchanged
    stride = 1 << 24
    assert torch.equal(b.mask.q_hi[n:].long(), a.clean_seq * stride + a.clean_pos + 1)
    assert torch.equal(a.mask.q_hi[n:].long(), a.clean_seq * stride + (a.clean_pos // 4 + 1) * 4)
    assert b.clean_causal and not a.clean_causal


def test_native_sft_encoder_next_token_term():
    """With objective.encoder_loss_weight > 0 the clean stream is causal and adds Σ CE(h[p] -> x[p+1]) / pairs;
    the clean hidden state at p must then not depend on the token at p + 1."""
    import torch

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.training.session import TrainingSession

    def session(weight):
        spec = RunSpec.from_mapping({
            "model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "family": "diffusion_gemma",
                      "num_layers": 2},
            "objective": {"name": "diffusiongemma_native_sft", "block_size": 16, "loss_weighting": "unit",
                          "self_conditioning_probability": 0.0, "encoder_loss_weight": weight},
            "training": {"batch_size": 2, "steps": 1, "skip_optimizer_step": True},
            "optimizer": {"lr": 1e-3}}).validate()
        return TrainingSession(spec, device="cpu")

    s0, s1 = session(0.0), session(1.0)
    assert not s0.layout.clean_causal and s1.layout.clean_causal
    r0, r1 = s0.step(), s1.step()
    l0, l1 = float(r0.loss_sum) / r0.denominator, float(r1.loss_sum) / r1.denominator
    enc = float(s1.last_encoder_loss)
    assert s0.last_encoder_loss is None and enc > 0
    assert l1 > l0 and abs(enc - 6.9) < 1.0          # ~ln(1024) at initialisation
    # causality of the clean stream: change the last token of a block, earlier clean rows keep their states
    lay = s1.layout
    tokens = torch.randint(0, 1000, (lay.rows,), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        h_a = s1.model(tokens, lay.positions, s1.attend)
        t2 = tokens.clone()
        row = lay.n_noisy + 15                         # sequence 0, position 15 (end of block 0)
        t2[row] = (t2[row] + 1) % 1000
        h_b = s1.model(t2, lay.positions, s1.attend)
    assert torch.allclose(h_a[lay.n_noisy:row], h_b[lay.n_noisy:row], atol=1e-6)
    assert not torch.allclose(h_a[row], h_b[row], atol=1e-4)
