"""DFlash distillation from an offline feature store: `dllm dflash prepare-features` output is what the trainer
reads, and training from it equals training with the target run online on the same tokens."""
import pytest
import torch

from turbo_dllm_b200.config.run_spec import RunSpec
from turbo_dllm_b200.data.dflash_features import FeatureStore, capture_features
from turbo_dllm_b200.training.session import TrainingSession


def _spec(features, path=None):
    data = {"target_features": features}
    if path:
        data["target_feature_path"] = str(path)
    return RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "family": "dflash",
                  "verifier_id": "synthetic:tiny-qwen3", "target_layer_ids": [0, 2], "max_layers": 2},
        "objective": {"name": "dflash_distillation", "block_size": 8, "max_anchors": 4},
        "data": data, "training": {"batch_size": 2, "steps": 3},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
        "optimizer": {"lr": 1e-3}}).validate()


def test_training_from_the_feature_store_equals_the_online_target(tmp_path):
    store = tmp_path / "features"
    man = capture_features(_spec("online"), str(store), batches=3)
    assert man["format"] == "dllm.dflash_features.v1" and len(man["shards"]) == 3
    online = TrainingSession(_spec("online"), device="cpu")
    offline = TrainingSession(_spec("offline", store), device="cpu")
    assert len(offline.task.target.model.layers) == 0           # only the verifier's embedding and head are built
    a = [float(online.step().loss_sum) for _ in range(3)]
    b = [float(offline.step().loss_sum) for _ in range(3)]
    assert b == pytest.approx(a, rel=1e-5)
    assert torch.allclose(online.model.flat.data, offline.model.flat.data, rtol=1e-4, atol=1e-6)
    st = offline.data.state_dict()
    nxt = offline.data.next_batch().input_ids
    offline.data.load_state_dict(st)
    assert torch.equal(offline.data.next_batch().input_ids, nxt)


def test_a_store_captured_for_other_layers_is_refused(tmp_path):
    store = tmp_path / "features"
    capture_features(_spec("online"), str(store), batches=1)
    bad = _spec("offline", store).with_overrides({"model": {"target_layer_ids": [1, 3]}})
    with pytest.raises(ValueError, match="captured for target layers"):
        TrainingSession(bad, device="cpu")
    FeatureStore(str(store), verify=True)
    (store / "shard_00000.pt").write_bytes(b"damaged")
    with pytest.raises(ValueError, match="sha256"):
        FeatureStore(str(store), verify=True)


def _capture(rank, world, out, batches, resume=False):
    import torch.distributed as dist

    torch.set_num_threads(2)
    man = capture_features(_spec("online"), out, batches, rank=rank, world=world, barrier=dist.barrier, resume=resume)
    return man.get("shards", []) if man else []


def test_capture_over_two_ranks_and_resume(tmp_path):
    """Two ranks write alternating records and rank 0 merges the manifest in record order; an interrupted capture
    (a record deleted, another damaged) is completed by --resume without rewriting the verified records."""
    import os

    from tests._harness import run_ranks

    out = str(tmp_path / "features")
    outs = run_ranks(_capture, 2, args=(out, 5), deadline_s=240)
    names = [sh["name"] for sh in outs[0]]
    assert names == [f"shard_{i:05d}.pt" for i in range(5)] and outs[1] == []
    store = FeatureStore(out, verify=True)
    assert store.manifest["captured_by_ranks"] == 2 and not [f for f in os.listdir(out) if f.startswith("manifest.rank")]
    # single-process capture of the same spec writes the same record 0 (rank 0 of one data-parallel rank)
    solo = str(tmp_path / "solo")
    man = capture_features(_spec("online"), solo, 1)
    assert man["shards"][0]["sha256"] == store.manifest["shards"][0]["sha256"]
    # resume: one record missing, one damaged -> both are rewritten, the rest kept
    man2 = capture_features(_spec("online"), str(tmp_path / "r"), 3)
    kept = os.path.getmtime(os.path.join(tmp_path / "r", "shard_00000.pt"))
    os.unlink(os.path.join(tmp_path / "r", "shard_00001.pt"))
    open(os.path.join(tmp_path / "r", "shard_00002.pt"), "wb").write(b"damaged")
    import json as _json

    _json.dump([{**sh, "index": i} for i, sh in enumerate(man2["shards"])],
               open(os.path.join(tmp_path / "r", "manifest.rank000.json"), "w"))
    man3 = capture_features(_spec("online"), str(tmp_path / "r"), 3, resume=True)
    assert [s["sha256"] for s in man3["shards"]] == [s["sha256"] for s in man2["shards"]]
    assert os.path.getmtime(os.path.join(tmp_path / "r", "shard_00000.pt")) == kept
    FeatureStore(str(tmp_path / "r"), verify=True)


def test_reduced_draft_vocabulary(tmp_path, capsys):
    """A drafter over a subset of the verifier's vocabulary: the maps are validated, the KL loss uses the head rows of
    the subset (equal to the dense formula), hard-label CE skips tokens outside it, and the export carries the maps."""
    import json

    import numpy as np

    from turbo_dllm_b200.cli.dflash import run_dflash
    from turbo_dllm_b200.models.dflash import DraftVocabulary
    from turbo_dllm_b200.models.export import export_dflash_drafter

    V = 1024
    ds = tmp_path / "ds"
    ds.mkdir()
    rng = np.random.default_rng(0)
    np.concatenate([rng.integers(0, 64, 5000), rng.integers(0, V, 500)]).astype("<i4").tofile(ds / "tokens.i32")
    path = str(tmp_path / "draft_vocab.safetensors")
    assert run_dflash(["build-draft-vocab", "--dataset", str(ds), "--size", "128", "--verifier-vocab-size", str(V),
                       "--output", path]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["draft_vocab_size"] == 128 and rep["token_coverage"] > 0.9
    dv = DraftVocabulary.load(path, V)
    assert dv.size == 128 and set(range(64)) <= set(dv.selected.tolist())
    assert torch.equal(dv.selected, torch.arange(128) + dv.d2t)
    ids = torch.tensor([int(dv.selected[5]), int((~dv.t2d).nonzero()[0])])
    assert dv.to_draft_ids(ids).tolist() == [5, -1]
    with pytest.raises(ValueError, match="d2t"):
        DraftVocabulary(dv.t2d, dv.d2t + 1, V)
    with pytest.raises(ValueError, match="verifier"):
        DraftVocabulary.load(path, V + 1)

    def spec(loss, vocab):
        s = _spec("online")
        return s.with_overrides({"model": {"draft_vocab_path": vocab}, "objective": {"dflash_loss": loss}}).validate()

    # KL over the subset == the dense formula on the selected head rows
    full = TrainingSession(spec("speculators_kl", None), device="cpu")
    sub = TrainingSession(spec("speculators_kl", path), device="cpu")
    assert sub.task.head.shape[0] == 128 and torch.equal(sub.task.head, full.task.target.lm_head[dv.selected])
    l_full, l_sub = float(full.step().loss_sum), float(sub.step().loss_sum)
    assert l_sub > 0 and l_sub != pytest.approx(l_full, rel=1e-3)
    # hard labels: a vocabulary that holds every id gives the full-vocabulary loss; the subset supervises fewer tokens
    everything = str(tmp_path / "all.safetensors")
    DraftVocabulary.from_ids(torch.arange(V), V).save(everything)
    ce_full = float(TrainingSession(spec("paper_ce", None), device="cpu").step().loss_sum)
    ce_all = float(TrainingSession(spec("paper_ce", everything), device="cpu").step().loss_sum)
    ce_sub = float(TrainingSession(spec("paper_ce", path), device="cpu").step().loss_sum)
    assert ce_all == pytest.approx(ce_full, rel=1e-5) and 0 <= ce_sub < ce_full
    out = str(tmp_path / "export")
    export_dflash_drafter(sub.model, sub.spec, out)
    from safetensors import safe_open

    with safe_open(out + "/model.safetensors", framework="pt") as f:
        assert torch.equal(f.get_tensor("t2d"), dv.t2d) and torch.equal(f.get_tensor("d2t"), dv.d2t)
    assert json.load(open(out + "/dflash_config.json"))["draft_vocab_size"] == 128
    with pytest.raises(Exception, match="draft_vocab_path"):
        _spec("online").with_overrides({"model": {"draft_vocab_path": path, "dflash2_selector_rank": 4}}).validate()


def test_sliding_window_drafter_and_context_compaction(monkeypatch, tmp_path):
    """Sliding-window drafter layers see the last window - 1 context tokens before the anchor; when every layer has the
    window, dropping the context rows no window reaches changes neither the loss nor the update."""
    import json

    from turbo_dllm_b200.models.dflash import dflash_mask_layout, window_context_rows
    from turbo_dllm_b200.objectives.dflash import DFlashObjectiveRuntime

    obj = DFlashObjectiveRuntime(block_size=8, max_anchors=3, mask_token_id=1023, seed=3, device="cpu")
    ids = torch.randint(0, 1000, (2, 64), generator=torch.Generator().manual_seed(0))
    ob = obj.prepare(ids, None)
    lay = dflash_mask_layout(ob, 64, 8, window=5)
    stop, start = ob.context_stops.long(), ob.document_starts.long()
    seq = torch.arange(2)[:, None] * (1 << 24)
    assert torch.equal(lay.q_hi.view(2, 3, 8)[:, :, 0].long(), seq + stop)
    assert torch.equal(lay.q_lo.view(2, 3, 8)[:, :, 0].long(), seq + torch.maximum(start, stop - 4))
    keep = window_context_rows(ob, 64, 5, min_rows=0)
    want = torch.zeros(2, 64, dtype=torch.bool)
    for b in range(2):
        for a in range(3):
            want[b, int(max(start[b, a], stop[b, a] - 4)):int(stop[b, a])] = True
    assert torch.equal(keep, want.reshape(-1).nonzero(as_tuple=True)[0])
    assert window_context_rows(ob, 64, 5, min_rows=40).numel() == 40

    def spec(**model):
        return _spec("online").with_overrides({"model": {"seq_len": 256, **model}}).validate()

    def run(s, compact):
        monkeypatch.setenv("TDLLM_DFLASH_COMPACT_CONTEXT", "1" if compact else "0")
        t = TrainingSession(s, device="cpu")
        loss = float(t.step().loss_sum)
        return loss, t.model.flat.data.clone(), t.task.last_context_rows

    full = run(spec(), True)
    all_windowed = spec(sliding_window=6)
    a, b = run(all_windowed, True), run(all_windowed, False)
    assert a[2] == 128 and b[2] is None        # 2 x 256 context rows, the windows reach at most 4 x 5 per sequence
    assert a[0] == pytest.approx(b[0], rel=1e-6) and torch.allclose(a[1], b[1], atol=1e-6)
    assert a[0] != pytest.approx(full[0], rel=1e-4)
    mixed = run(spec(sliding_window=6, sliding_window_pattern=2), True)      # every second layer attends to everything
    assert mixed[2] is None and mixed[0] != pytest.approx(a[0], rel=1e-4) and mixed[0] != pytest.approx(full[0], rel=1e-4)
    from turbo_dllm_b200.models.export import export_dflash_drafter

    t = TrainingSession(spec(sliding_window=6, sliding_window_pattern=2), device="cpu")
    export_dflash_drafter(t.model, t.spec, str(tmp_path / "e"))
    conf = json.load(open(tmp_path / "e" / "dflash_config.json"))
    assert conf["sliding_window"] == 6 and conf["sliding_window_non_causal"] is True
    assert conf["layer_types"] == ["sliding_attention", "full_attention"]


def test_speculators_checkpoint_round_trip(tmp_path):
    """The deployable layout (module-style names, verifier embedding and head, speculators_config) reloads into a fresh
    drafter tensor for tensor; with a draft vocabulary the head holds the subset's rows."""
    import json

    from safetensors import safe_open

    from turbo_dllm_b200.models.dflash import DraftVocabulary
    from turbo_dllm_b200.models.export import export_speculators_checkpoint, load_speculators_checkpoint

    vocab = str(tmp_path / "dv.safetensors")
    DraftVocabulary.from_ids(torch.arange(0, 1024, 4), 1024).save(vocab)
    s = TrainingSession(_spec("online").with_overrides({"model": {"draft_vocab_path": vocab}}).validate(), device="cpu")
    s.step()
    out = str(tmp_path / "spec")
    man = export_speculators_checkpoint(s.model, s.task.target, s.spec, out)
    assert man["kind"] == "dflash_speculators"
    conf = json.load(open(out + "/config.json"))
    assert conf["speculators_config"]["proposal_methods"][0]["speculative_tokens"] == 7       # block 8, anchor = bonus token
    assert conf["speculators_config"]["verifier"]["name_or_path"] == "synthetic:tiny-qwen3"
    assert conf["draft_vocab_size"] == 256 and conf["vocab_size"] == 1024 and conf["aux_hidden_state_layer_ids"] == [0, 2]
    cfg = s.model.cfg
    with safe_open(out + "/model.safetensors", framework="pt") as f:
        keys = set(f.keys())
        assert {"fc.weight", "hidden_norm.weight", "norm.weight", "embed_tokens.weight", "lm_head.weight", "t2d", "d2t",
                "layers.0.self_attn.k_proj.weight", "layers.1.mlp.up_proj.weight"} <= keys
        assert tuple(f.get_tensor("lm_head.weight").shape) == (256, cfg.hidden_size)
        assert torch.equal(f.get_tensor("lm_head.weight"), s.task.target.lm_head[::4])
        assert tuple(f.get_tensor("layers.0.self_attn.v_proj.weight").shape) == (cfg.kv_dim, cfg.hidden_size)
        gate = f.get_tensor("layers.0.mlp.gate_proj.weight")
    assert torch.equal(gate, s.model.flat.params["layers.0.w_gate_up"][0::2])
    fresh = TrainingSession(_spec("online"), device="cpu")
    assert not torch.equal(fresh.model.flat.data, s.model.flat.data)
    load_speculators_checkpoint(fresh.model, out)
    assert torch.equal(fresh.model.flat.data, s.model.flat.data)
    # model.id naming the exported directory: the architecture comes from its config, the weights from its tensors
    cont = TrainingSession(_spec("online").with_overrides({"model": {"id": out, "max_layers": None}}).validate(), device="cpu")
    assert torch.equal(cont.model.flat.data, s.model.flat.data)
    # a drafter of another width is refused tensor by tensor
    other = TrainingSession(_spec("online").with_overrides({"model": {"intermediate_size": 128}}).validate(), device="cpu")
    with pytest.raises(ValueError, match="checkpoint shape"):
        load_speculators_checkpoint(other.model, out)


def test_export_command_from_a_training_checkpoint(tmp_path, capsys):
    import json

    import yaml

    from turbo_dllm_b200.checkpoint import save_training_checkpoint
    from turbo_dllm_b200.cli.dflash import run_dflash

    spec = _spec("online")
    s = TrainingSession(spec, device="cpu")
    s.step()
    save_training_checkpoint(str(tmp_path / "ck"), s, step=1, rank=0, world_size=1)
    (tmp_path / "draft.yaml").write_text(yaml.safe_dump(spec.to_dict()))
    for fmt, must_have in (("native", "dflash_config.json"), ("speculators", "config.json")):
        out = str(tmp_path / fmt)
        assert run_dflash(["export", "--config", str(tmp_path / "draft.yaml"), "--checkpoint", str(tmp_path / "ck"),
                           "--output", out, "--format", fmt]) == 0
        files = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["files"]
        assert must_have in files and "model.safetensors" in files
    from safetensors import safe_open

    with safe_open(str(tmp_path / "native" / "model.safetensors"), framework="pt") as f:
        assert torch.equal(f.get_tensor("fc"), s.model.flat.params["fc"])
    assert run_dflash(["validate-export", str(tmp_path / "native")]) == 0
