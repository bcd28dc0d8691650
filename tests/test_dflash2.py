"""DFlash2 drafter: block-local dynamic convolution, D-PACE weights, cross-entropy with top-k
candidates through the frozen head, candidate selector, and a training step (CPU, fp32)."""
import math

import pytest
import torch

from turbo_dllm_b200.ops.dflash2 import (dpace_weight, frozen_linear_ce_topk, grouped_dynamic_conv,
                                          selector_schedule_factor, transform_logits)


def test_grouped_dynamic_conv_against_a_direct_loop():
    torch.manual_seed(0)
    bs, H, taps, groups, nb = 4, 6, 3, 2, 3
    x = torch.randn(nb * bs, H)
    dyn = torch.randn(nb * bs, taps, groups) * 0.3
    base = torch.randn(taps, H)
    got = grouped_dynamic_conv(x, dyn, base, bs)
    want = torch.zeros_like(x)
    for r in range(nb * bs):
        t = r % bs
        for i in range(taps):
            if t - i < 0:
                continue        # nothing in front of the block start
            for c in range(H):
                want[r, c] += (base[i, c] + dyn[r, i, c // (H // groups)]) * x[r - i, c]
    assert torch.allclose(got, want, atol=1e-5)
    ident = torch.zeros(taps, H)
    ident[0] = 1.0
    assert torch.allclose(grouped_dynamic_conv(x, torch.zeros_like(dyn), ident, bs), x)
    with pytest.raises(ValueError):
        grouped_dynamic_conv(x[:-1], dyn[:-1], base, bs)


def test_dpace_weights():
    p = torch.tensor([[0.9, 0.5, 0.2, 0.7]])
    m = torch.tensor([[1.0, 1.0, 0.0, 1.0]])
    a = 0.5
    smooth = [(1 - a) * 0.9 + a, (1 - a) * 0.5 + a, 1.0, (1 - a) * 0.7 + a]
    prefix = [smooth[0], smooth[0] * smooth[1], smooth[0] * smooth[1], smooth[0] * smooth[1] * smooth[3]]
    suffix = [prefix[0] + prefix[1] + prefix[3], prefix[1] + prefix[3], prefix[3], prefix[3]]
    assert torch.allclose(dpace_weight(p, m, alpha=a, kind="dpace-cumulative-confidence-only"), torch.tensor([prefix]))
    assert torch.allclose(dpace_weight(p, m, alpha=a, kind="dpace"), torch.tensor([suffix]))
    cont = [s / q for s, q in zip(suffix, prefix)]
    assert torch.allclose(dpace_weight(p, m, alpha=a, kind="dpace-continuation-value-only"), torch.tensor([cont]))
    with pytest.raises(ValueError):
        dpace_weight(p, m, alpha=a, kind="other")


def test_selector_schedule():
    f = lambda s: selector_schedule_factor(s, 100, 0.1, 0.2)
    assert f(0) == 0.0 and f(9) == 0.0
    assert f(10) == pytest.approx(1 / 20) and f(19) == pytest.approx(0.5) and f(29) == 1.0 and f(99) == 1.0
    assert selector_schedule_factor(0, 100, 0.0, 0.0) == 1.0


@pytest.mark.parametrize("softcap,mult", [(None, 1.0), (5.0, 0.5)])
def test_frozen_linear_ce_topk_matches_dense_logits(softcap, mult):
    torch.manual_seed(1)
    n, H, V, k = 37, 16, 203, 4
    h = torch.randn(n, H, requires_grad=True)
    w = torch.randn(V, H)
    labels = torch.randint(0, V, (n,))
    wts = torch.rand(n)
    ce_sum, ce, prob, topz, ids = frozen_linear_ce_topk(h, w, labels, top_k=k, vocab_block_size=64,
                                                        output_multiplier=mult, logit_softcap=softcap,
                                                        loss_weights=wts)
    hr = h.detach().clone().requires_grad_(True)
    z = transform_logits(hr @ w.t(), mult, softcap)
    ce_ref = torch.nn.functional.cross_entropy(z, labels, reduction="none")
    assert torch.allclose(ce, ce_ref.detach(), atol=1e-4)
    assert torch.allclose(prob, torch.exp(-ce_ref.detach()), atol=1e-5)
    zr, ir = z.topk(k, dim=-1)
    assert torch.equal(ids, ir)
    assert torch.allclose(topz, zr.detach(), atol=1e-4)
    assert not ce.requires_grad and not prob.requires_grad and topz.requires_grad
    g = torch.randn(n, k)
    (ce_sum + (topz * g).sum()).backward()
    ((ce_ref * wts).sum() + (zr * g).sum()).backward()
    assert torch.allclose(h.grad, hr.grad, atol=1e-4, rtol=1e-3)


def _models():
    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.dflash import DFlashDraftModel
    from turbo_dllm_b200.models.dflash2 import DFlash2DraftModel

    cfg = PRESETS["synthetic:tiny-qwen3"]
    kw = dict(target_hidden=32, num_target_layers=2, dtype=torch.float32, seed=3, init_std=0.05)
    v1 = DFlashDraftModel(cfg, **kw)
    v2 = DFlash2DraftModel(cfg, block_size=8, conv_kernel_size=3, conv_group_size=64, selector_rank=6,
                           selector_top_k=4, verifier_vocab_size=cfg.vocab_size, **kw)
    return cfg, v1, v2


def _draft_inputs(cfg, bs=8, blocks=3, ctx=24):
    from turbo_dllm_b200.ops.attention import MaskLayout

    g = torch.Generator().manual_seed(4)
    nd = bs * blocks
    emb = torch.randn(nd, cfg.hidden_size, generator=g)
    feats = torch.randn(ctx, 64, generator=g)
    starts = torch.tensor([4, 10, 20])
    pos_d = (starts[:, None] + torch.arange(bs)[None]).reshape(-1)
    pos_c = torch.arange(ctx)
    i32 = torch.int32
    q_lo = torch.zeros(nd, dtype=i32)
    q_hi = starts.repeat_interleave(bs).to(i32)
    q_grp = -(torch.arange(blocks).repeat_interleave(bs) + 1).to(i32)
    mask = MaskLayout(q_lo, q_hi, q_grp, torch.cat([q_grp, pos_c.to(i32)]))
    return emb, feats, pos_d, pos_c, mask


def test_fresh_dflash2_equals_dflash_and_convolutions_train():
    cfg, v1, v2 = _models()
    with torch.no_grad():
        for name, p in v1.flat.params.items():
            v2.flat.params[name].copy_(p)
    emb, feats, pos_d, pos_c, mask = _draft_inputs(cfg)
    with torch.no_grad():
        a, b = v1(emb, feats, pos_d, pos_c, mask), v2(emb, feats, pos_d, pos_c, mask)
    assert torch.allclose(a, b, atol=1e-5)
    v2.flat.zero_grad()
    out = v2(emb, feats, pos_d, pos_c, mask)
    out.square().sum().backward()
    v2.flat.collect_grads()
    for leaf in ("attn_conv_base", "attn_conv_proj", "mlp_conv_base", "mlp_conv_proj"):
        assert v2.flat.params[f"layers.0.{leaf}"].main_grad.abs().sum() > 0, leaf
    # a non-zero correction changes the output, and only inside blocks: perturb the first block's input
    with torch.no_grad():
        v2.flat.params["layers.0.attn_conv_base"][0, 1] = 0.5
        c = v2(emb, feats, pos_d, pos_c, mask)
    assert not torch.allclose(b, c, atol=1e-4)


def test_candidate_selector_lattice_and_greedy_path():
    cfg, _, v2 = _models()
    sel = v2.candidate_selector
    with torch.no_grad():
        sel.successor.normal_(0, 0.5)
    b, L, k = 2, 5, sel.top_k
    g = torch.Generator().manual_seed(6)
    cand = torch.stack([torch.randperm(cfg.vocab_size, generator=g)[:k] for _ in range(b * L)]).view(b, L, k)
    unary = torch.randn(b, L, k, generator=g)
    hid = torch.randn(b, L, cfg.hidden_size, generator=g)
    anchor = torch.randint(0, cfg.vocab_size, (b,), generator=g)
    lat = sel.build_lattice(candidate_ids=cand, unary_logits=unary, hidden_states=hid, anchor_token_ids=anchor)
    assert lat.shape == (b, L, k, k)
    # row p of the lattice at position t = scores after predecessor candidate p of position t-1
    t, p = 3, 2
    s = sel.score_candidates(candidate_ids=cand[:, t], unary_logits=unary[:, t], hidden_states=hid[:, t],
                             predecessor_ids=cand[:, t - 1, p])
    assert torch.allclose(lat[:, t, p], s, atol=1e-5)
    s0 = sel.score_candidates(candidate_ids=cand[:, 0], unary_logits=unary[:, 0], hidden_states=hid[:, 0],
                              predecessor_ids=anchor)
    assert torch.allclose(lat[:, 0, 0], s0, atol=1e-5)
    path = sel.greedy_path(candidate_ids=cand, unary_logits=unary, hidden_states=hid, anchor_token_ids=anchor)
    assert path.shape == (b, L)
    assert torch.equal(path[:, 0], cand[:, 0].gather(1, s0.argmax(-1, keepdim=True))[:, 0])
    assert all(int(path[i, j]) in cand[i, j].tolist() for i in range(b) for j in range(L))


@pytest.mark.parametrize("loss,lk", [("dpace", None), ("dflash", "lambda"), ("dpace-continuation-value-only", "tv")])
def test_dflash2_training_step(loss, lk):
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.training.session import TrainingSession

    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 128, "dtype": "fp32", "family": "dflash",
                  "verifier_id": "synthetic:tiny-qwen3", "target_layer_ids": [0, 2], "max_layers": 2,
                  "dflash2_conv_kernel_size": 3, "dflash2_conv_group_size": 64, "dflash2_selector_rank": 8,
                  "dflash2_selector_top_k": 4},
        "objective": {"name": "dflash_distillation", "block_size": 8, "max_anchors": 6, "decay_gamma": 4.0,
                      "dflash_loss": loss, "lk_loss_type": lk, "selector_loss_alpha": 0.5,
                      "dflash_vocab_block_size": 300},
        "data": {"target_features": "online"}, "training": {"batch_size": 2, "steps": 4},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
        "optimizer": {"lr": 2e-3, "gradient_clip_norm": 1.0}}).validate()
    s = TrainingSession(spec, device="cpu")
    from turbo_dllm_b200.models.dflash2 import DFlash2DraftModel

    assert isinstance(s.model, DFlash2DraftModel)
    before = s.model.flat.data.clone()
    losses = []
    for _ in range(3):
        r = s.step()
        losses.append(float(r.loss_sum))
    assert all(math.isfinite(x) and x > 0 for x in losses)
    moved = lambda n: (s.model.flat.params[n] - before[s.model.flat.offsets[n][0]:][: s.model.flat.params[n].numel()]
                       .view_as(s.model.flat.params[n])).abs().sum() > 0
    assert moved("selector_proj") and moved("layers.0.attn_conv_proj") and moved("layers.0.w_q")
    m = s.task.last_objective_metrics
    assert 0.0 <= float(m["selector_coverage"]) <= 1.0 and 0.0 < float(m["target_probability"]) < 1.0


def test_dpace_loss_needs_the_dflash2_drafter():
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.training.session import TrainingSession

    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "family": "dflash",
                  "verifier_id": "synthetic:tiny-qwen3", "target_layer_ids": [0]},
        "objective": {"name": "dflash_distillation", "block_size": 8, "dflash_loss": "dpace"},
        "data": {"target_features": "online"}, "training": {"batch_size": 1, "steps": 1},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1}}).validate()
    with pytest.raises(ValueError):
        TrainingSession(spec, device="cpu")


def test_dflash2_export_round_trip(tmp_path):
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.models.export import (export_dflash_drafter, normalize_dflash2_config,
                                               validate_dflash2_export)

    cfg, _, v2 = _models()
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "family": "dflash", "verifier_id": "synthetic:tiny-qwen3",
                  "target_layer_ids": [0, 2]},
        "objective": {"name": "dflash_distillation", "block_size": 8}})
    out = str(tmp_path / "export")
    export_dflash_drafter(v2, spec, out)
    assert validate_dflash2_export(out, expected_block_size=8) == []
    import json
    import os

    conf = json.load(open(os.path.join(out, "config.json")))
    assert conf["architectures"] == ["DFlash2DraftModel"] and conf["dflash_config"]["selector_top_k"] == 4
    from safetensors import safe_open

    with safe_open(os.path.join(out, "model.safetensors"), framework="pt") as f:
        assert tuple(f.get_slice("layers.0.attn_conv_proj").get_shape()) == (2 * 3 * (cfg.hidden_size // 64),
                                                                             cfg.hidden_size)
        assert "embed" not in f.keys() and "lm_head" not in f.keys()
    assert any("block_size" in p for p in validate_dflash2_export(out, expected_block_size=16))
    # the command-line checks: the shared export check with a block size, and the vLLM loader's contract
    from turbo_dllm_b200.cli.dflash import run_dflash

    assert run_dflash(["validate-export", out, "--block-size", "8"]) == 0
    assert run_dflash(["validate-vllm", out, "--block-size", "8"]) == (0 if conf.get("model_type") == "qwen3" else 2)
    assert run_dflash(["validate-vllm", out, "--block-size", "16"]) == 2
    bad = dict(conf, architectures=["DFlashDraftModel"])
    with pytest.raises(ValueError):
        normalize_dflash2_config(bad)
    # a tampered tensor file is caught by the manifest hashes
    with open(os.path.join(out, "model.safetensors"), "ab") as f:
        f.write(b"x")
    assert validate_dflash2_export(out) != []


def _dflash2_dp(rank, world):
    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "family": "dflash",
                  "verifier_id": "synthetic:tiny-qwen3", "target_layer_ids": [0, 2], "max_layers": 2,
                  "dflash2_conv_kernel_size": 2, "dflash2_conv_group_size": 64, "dflash2_selector_rank": 4,
                  "dflash2_selector_top_k": 2},
        "objective": {"name": "dflash_distillation", "block_size": 8, "max_anchors": 4, "dflash_loss": "dpace",
                      "lk_loss_type": "lambda", "dflash_vocab_block_size": 512},
        "data": {"target_features": "online"}, "training": {"batch_size": 1, "steps": 2},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    s = TrainingSession(spec, device="cpu")
    batch = s.data.next_batch()
    s.model.flat.zero_grad()
    _, _, denom = s.task.forward_backward(batch)
    local = torch.tensor(float(denom))
    both = [torch.zeros(()) for _ in range(world)]
    dist.all_gather(both, local)
    for _ in range(2):
        s.step()
    return [float(x) for x in both], s.model.flat.data.clone()


@pytest.mark.distributed
def test_dflash2_denominator_is_shared_by_the_data_parallel_ranks():
    from tests._harness import run_ranks

    outs = run_ranks(_dflash2_dp, 2, deadline_s=240)
    (d0, p0), (d1, p1) = outs
    assert d0[0] == pytest.approx(d0[1]) and d0 == pytest.approx(d1)      # same global count on both ranks
    assert (p0 == p1).all()                                                # replicas stay in sync


def test_topk_scan_and_gather_dot_in_small_chunks():
    """Row and vocabulary chunking must not change the candidates, their order or the gradients."""
    from turbo_dllm_b200.ops.dflash2 import _GatherDot, _topk_candidates

    torch.manual_seed(8)
    h, w = torch.randn(21, 12), torch.randn(97, 12)
    ids = _topk_candidates(h, w, 5, 10, 1.0, None, row_chunk=4)
    want = (h @ w.t()).topk(5, dim=-1).indices
    assert torch.equal(ids, want)
    capped = _topk_candidates(h, w, 3, 97, 2.0, 30.0, row_chunk=100)   # a cap far from saturation: no ties
    assert torch.equal(capped, transform_logits(h @ w.t(), 2.0, 30.0).topk(3, dim=-1).indices)
    a = h.clone().requires_grad_(True)
    b = h.clone().requires_grad_(True)
    g = torch.randn(21, 5)
    (_GatherDot.apply(a, w, ids, 4) * g).sum().backward()
    (torch.einsum("nh,nkh->nk", b, w[ids]) * g).sum().backward()
    assert torch.allclose(a.grad, b.grad, atol=1e-5)
