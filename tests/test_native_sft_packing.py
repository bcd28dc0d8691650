"""diffusiongemma_native_sft with response-suffix packing: decoder rows cover the supervised response only, blocks are
counted from the response start, padding is neither scored nor an encoder target."""
import pytest
import torch

from turbo_dllm_b200.config.run_spec import RunSpec
from turbo_dllm_b200.data.runtimes import DataBatch
from turbo_dllm_b200.training.session import TrainingSession


def _spec(pack=True, min_blocks=1):
    return RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 128, "dtype": "fp32", "family": "diffusion_gemma",
                  "num_layers": 2},
        "objective": {"name": "diffusiongemma_native_sft", "block_size": 16, "loss_weighting": "unit",
                      "self_conditioning_probability": 0.0, "pack_response_suffix": pack,
                      "minimum_decoder_blocks": min_blocks},
        "training": {"batch_size": 2, "steps": 2, "activation_checkpointing": True},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
        "optimizer": {"lr": 1e-3}}).validate()


def test_suffix_detection_and_decoder_shapes():
    s = TrainingSession(_spec(min_blocks=5), device="cpu")
    ob = s.objective
    ids = torch.randint(0, 1000, (2, 128))
    sm = torch.zeros(2, 128, dtype=torch.bool)
    sm[:, 40:100] = True
    vm = torch.zeros(2, 128, dtype=torch.bool)
    vm[:, :100] = True
    assert ob.response_suffix(sm, vm) == (40, 100)
    assert ob.response_suffix(None) is None
    gap = sm.clone()
    gap[:, 60] = False                         # not one contiguous suffix: the masked full-length form applies
    assert ob.response_suffix(gap, vm) is None
    other = sm.clone()
    other[1, 40:50] = False                    # rows with different response starts
    assert ob.response_suffix(other, vm) is None
    with pytest.raises(ValueError, match="cannot score padding"):
        ob.response_suffix(torch.ones(2, 128, dtype=torch.bool), vm)
    with pytest.raises(ValueError, match="contiguous non-empty prefix"):
        ob.response_suffix(sm, ~vm)
    cb = ob.corrupt(ids, supervision_mask=sm, supervision_count=120, valid_mask=vm)
    # 60 response tokens -> 4 blocks of 16, raised to the minimum of 5; rows past the response are padding
    assert cb.response_start == 40 and cb.valid_length == 100 and cb.noisy_input_ids.shape == (2, 1, 80)
    assert int((cb.labels != -100).sum()) == 120 and cb.valid_tokens == 120 and cb.diffusion_times.shape == (2, 5)
    assert torch.equal(cb.labels[:, 0, :60], ids[:, 40:100]) and bool((cb.labels[:, 0, 60:] == -100).all())
    with pytest.raises(ValueError, match="supervision_count"):
        ob.corrupt(ids, supervision_mask=sm, supervision_count=7, valid_mask=vm)


def test_decoder_rows_see_what_the_full_layout_shows_them():
    """With the response starting on a block boundary the packed decoder rows are the full layout's noisy rows of
    the same positions: same keys, same hidden states."""
    from turbo_dllm_b200.models.dense import LocalAttention
    from turbo_dllm_b200.parallel.layout import build_packed_layout, build_response_layout

    s = TrainingSession(_spec(), device="cpu")
    full = build_packed_layout(seq_len=128, block_size=16, batch=2, clean_causal=True)
    pack = build_response_layout(seq_len=128, block_size=16, batch=2, response_start=32, valid_length=128,
                                 decoder_length=96, clean_causal=True)
    assert pack.n_noisy == 2 * 96 and pack.n_clean == 2 * 128
    torch.manual_seed(0)
    clean = torch.randint(0, 1000, (2, 128))
    noisy = torch.randint(0, 1000, (2, 128))
    tok_full = torch.cat([noisy[full.noisy_seq, full.noisy_pos], clean[full.clean_seq, full.clean_pos]])
    tok_pack = torch.cat([noisy[:, 32:][pack.noisy_seq, pack.noisy_offset], clean[pack.clean_seq, pack.clean_pos]])
    with torch.no_grad():
        h_full = s.model(tok_full, full.positions, LocalAttention(s.cfg, full.mask))
        h_pack = s.model(tok_pack, pack.positions, LocalAttention(s.cfg, pack.mask))
    rows = (full.noisy_pos >= 32).nonzero(as_tuple=True)[0]
    assert torch.allclose(h_pack[: pack.n_noisy], h_full[rows], rtol=1e-4, atol=1e-5)
    assert torch.allclose(h_pack[pack.n_noisy:], h_full[full.n_noisy:], rtol=1e-4, atol=1e-5)
    # off a block boundary the blocks follow the response start: block 0 of a response starting at 40 sees clean
    # positions < 40 and itself
    odd = build_response_layout(seq_len=128, block_size=16, batch=1, response_start=40, valid_length=100,
                                decoder_length=64)
    dense = odd.mask.dense_mask()
    first = dense[0]
    clean_keys = first[odd.n_noisy:]
    assert bool(clean_keys[:40].all()) and not bool(clean_keys[40:].any())
    assert bool(first[:16].all()) and not bool(first[16: odd.n_noisy].any())
    last_block_row = dense[48]                  # block 3: offsets 48..63, positions 88..99 then padding
    assert bool(last_block_row[odd.n_noisy:][:88].all()) and not bool(last_block_row[odd.n_noisy:][88:].any())


def test_training_steps_with_packed_and_padded_batches():
    class Fixed:
        def __init__(self, b):
            self.b = b

        def next_optimizer_step_batches(self, n):
            return [self.b] * n

        def state_dict(self):
            return {}

    torch.manual_seed(1)
    ids = torch.randint(0, 1000, (2, 128))
    sm = torch.zeros(2, 128, dtype=torch.bool)
    sm[:, 40:100] = True
    vm = torch.zeros(2, 128, dtype=torch.bool)
    vm[:, :100] = True
    out = {}
    for pack in (True, False):
        s = TrainingSession(_spec(pack), device="cpu")
        s.data = Fixed(DataBatch(ids, supervision_mask=sm, supervision_count=120, valid_mask=vm if pack else None))
        r1 = s.step()
        r2 = s.step()
        out[pack] = (float(r1.loss_sum) / r1.denominator, float(r2.loss_sum) / r2.denominator, s.layout.n_noisy)
        assert r1.denominator == 120 and out[pack][1] < out[pack][0] + 1.0 and out[pack][0] == out[pack][0]
    assert out[True][2] == 2 * 64 and out[False][2] == 2 * 128        # a third of the noisy rows are gone
    # both forms score the same 120 tokens; their losses are of the same size (different noise draws)
    assert abs(out[True][0] - out[False][0]) < 0.5 * out[False][0]


def _packed_sft_run(rank, world, tp, sp, path, steps=3, bp=1):
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 128, "dtype": "fp32", "num_layers": 2, "family": "diffusion_gemma"},
        "objective": {"name": "diffusiongemma_native_sft", "block_size": 16, "noise_schedule": "loglinear",
                      "loss_weighting": "unit", "self_conditioning_probability": 0.5, "sampling_epsilon_min": 0.1,
                      "minimum_decoder_blocks": 2},
        "data": {"input_mode": "dataset", "dataset_path": path},
        "training": {"batch_size": 2, "steps": steps},
        "topology": {"context_parallel_size": 1, "block_parallel_size": bp, "replicate_clean_prefix": bp > 1,
                     "tensor_parallel_size": tp, "sequence_parallel": sp},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device="cpu", runtime=rt)
    assert s.objective.pack_response_suffix
    out = []
    for _ in range(steps):
        r = s.step()
        out.append(float(r.loss_sum) / float(r.denominator))
    return out, float(s.optimizer.grad_norm()), int(s.layout.n_noisy)


def test_response_packing_under_tensor_and_sequence_parallelism(tmp_path):
    """Tensor parallelism divides heads, not rows: the decoder rows still cover the response only, and the step equals
    the single-process packed step."""
    import numpy as np

    from tests._harness import run_ranks
    from turbo_dllm_b200.data.artifacts import write_indexed_artifact

    rng = np.random.default_rng(0)
    samples = []
    for i in range(32):
        mask = np.zeros(128, np.uint8)
        mask[[32, 64][i % 2]:] = 1
        samples.append({"tokens": rng.integers(0, 1000, 128).astype(np.int32), "loss_mask": mask, "sample_id": i})
    write_indexed_artifact(tmp_path / "idx", samples, metadata={"tokenizer": {"vocab_size": 1024}})
    ref = _packed_sft_run(0, 1, 1, False, str(tmp_path / "idx"))
    assert ref[2] < 2 * 128                                  # fewer decoder rows than whole sequences would need
    for out in run_ranks(_packed_sft_run, 2, args=(2, True, str(tmp_path / "idx")), deadline_s=300):
        assert out[0] == pytest.approx(ref[0], rel=3e-4) and out[1] == pytest.approx(ref[1], rel=4e-3) and out[2] == ref[2]
    # block parallelism alone: the response's decoder blocks are divided over the ranks (their losses add up to the whole)
    import torch.distributed  # noqa: F401

    outs = run_ranks(_packed_sft_run, 2, args=(1, False, str(tmp_path / "idx"), 3, 2), deadline_s=300)
    assert sum(o[2] for o in outs) == ref[2] and all(0 < o[2] < ref[2] for o in outs)
    total = [sum(o[0][i] for o in outs) for i in range(3)]
    assert total == pytest.approx(ref[0], rel=3e-4) and outs[0][1] == pytest.approx(ref[1], rel=4e-3)
