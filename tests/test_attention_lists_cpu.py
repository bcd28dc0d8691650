"""Host-side structures of the attention kernels and of activation checkpointing, checked on CPU."""
import pytest
import torch


@pytest.mark.parametrize("chunk", [0, 1, 4, 5, 32, 1000])
@pytest.mark.parametrize("views", [1, 2])
def test_backward_work_items_cover_every_visible_tile_pair_once(chunk, views):
    from turbo_dllm_b200.ops.attention import single_sequence_layout

    lay = single_sequence_layout(1536, 32, "cpu", views)
    L = lay.tile_lists()
    W = lay.backward_work(chunk)
    nkt, nqt = L["nkt"], L["nqt"]
    visible, full = lay._cache["visible"]
    seen = torch.zeros(nqt, nkt, dtype=torch.int32)
    order = W["w_order"][: W["n_work"]].tolist()
    assert len(set(order)) == len(order)
    for w in order:
        kt, c = w % nkt, w // nkt
        ents = W["w_idx"][W["w_ptr"][w]:W["w_ptr"][w + 1]].tolist()
        assert ents, "empty work items must not be scheduled"
        for e in ents:
            qt = e >> 1
            assert qt // W["chunk_tiles"] == c
            assert bool(e & 1) == (not bool(full[qt, kt])), "mask flag must mark the tiles that are not fully visible"
            seen[qt, kt] += 1
    assert (seen == visible.int()).all()
    chunks = [w // nkt for w in order]
    assert chunks == sorted(chunks), "the grid must run chunk by chunk"
    # heaviest first inside a chunk
    sizes = [int(W["w_ptr"][w + 1] - W["w_ptr"][w]) for w in order]
    for c in set(chunks):
        s = [sz for sz, cc in zip(sizes, chunks) if cc == c]
        assert s == sorted(s, reverse=True)


def _grads(checkpoint: bool):
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.training.session import TrainingSession

    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 128, "dtype": "fp32"},
        "objective": {"name": "fast_dllm_v2", "block_size": 16},
        "training": {"batch_size": 2, "steps": 1, "activation_checkpointing": checkpoint, "skip_optimizer_step": True},
        "optimizer": {"lr": 1e-3}}).validate()
    s = TrainingSession(spec, device="cpu")
    r = s.step()
    return float(r.loss_sum) / r.denominator, s.model.flat.grad.clone()


def test_replay_without_the_layer_output_gives_the_same_gradients():
    """The checkpoint replay skips the layer's last product (its value is never read); gradients must
    equal those of the run that keeps every activation."""
    la, ga = _grads(False)
    lb, gb = _grads(True)
    assert la == pytest.approx(lb, rel=1e-6)
    assert torch.allclose(ga, gb, rtol=1e-5, atol=1e-7)


def test_skip_flag_only_applies_inside_the_replay():
    from turbo_dllm_b200.ops import gemm as G

    assert G._Replay.skip_last_output is False
    with G.skip_last_output():
        assert G._Replay.skip_last_output is True
    assert G._Replay.skip_last_output is False


def test_grouped_row_layout_tables():
    from turbo_dllm_b200.ops.grouped import PAD, build_grouped_rows

    counts = torch.tensor([300, 0, 17, 512, 1])
    rows = int(counts.sum())
    g = build_grouped_rows(counts, rows)
    assert g.capacity % PAD == 0 and g.capacity >= rows
    begin = g.row_begin.tolist()
    assert all(b % PAD == 0 for b in begin) and begin == sorted(begin)
    # every sorted row lands inside its expert's padded segment, in order, without collisions
    dest = g.dest.tolist()
    assert len(set(dest)) == rows
    off = 0
    for e, n in enumerate(counts.tolist()):
        assert dest[off:off + n] == list(range(begin[e], begin[e] + n))
        off += n
    # tile -> expert table agrees with the segments (tiles of empty experts do not exist)
    for t, e in enumerate(g.mt_group.tolist()):
        row = t * 128
        owners = [k for k in range(len(begin)) if begin[k] <= row < begin[k] + (int(counts[k]) + PAD - 1) // PAD * PAD]
        assert not owners or owners[0] == e
    assert g.row_blocks_end.tolist() == [(b + (int(n) + 63) // 64 * 64) // 64 for b, n in zip(begin, counts.tolist())]


def test_wide_attention_chunks_cover_every_query_tile_and_every_visible_key():
    """The product-and-softmax form of attention (head widths other than 128) walks chunks of whole query tiles and,
    per chunk, the key tiles some row of the chunk can see: together the chunks cover all query rows once, and no
    visible key is left out of its chunk."""
    import torch

    from turbo_dllm_b200.ops import wide_attention as wa
    from turbo_dllm_b200.ops.attention import single_sequence_layout

    layout = single_sequence_layout(640, 32, "cpu", 2)              # 1920 rows: 15 query tiles
    dense = layout.dense_mask()
    old = wa.SCORE_BYTES
    try:
        for budget in (1 << 30, 4 * 128 * 4 * 128 * 6):           # one chunk; a budget that forces several chunks
            wa.SCORE_BYTES = budget
            layout._cache.pop(("wide_chunks", 4), None)
            chunks = wa._chunks(layout, 4)
            covered = torch.zeros(dense.shape[0], dtype=torch.bool)
            for r0, rows, krows, valid in chunks:
                assert r0 % 128 == 0 and rows % 128 == 0 and krows.numel() % 128 == 0
                live = slice(r0, min(r0 + rows, dense.shape[0]))
                assert not covered[live].any()
                covered[live] = True
                seen = torch.zeros(dense.shape[1], dtype=torch.bool)
                seen[krows[valid]] = True
                assert not (dense[live].any(0) & ~seen).any()      # every key some row of the chunk sees is present
            assert covered.all()
            if budget < (1 << 30):
                assert len(chunks) > 1
                # block-causal structure: the first chunk needs far fewer key tiles than there are
                assert chunks[0][2].numel() < dense.shape[1]
    finally:
        wa.SCORE_BYTES = old
