import json

import numpy as np
import pytest
import torch

from turbo_dllm_b200.data.artifact_runtimes import (BlendedPackedTokenDataRuntime, IndexedSupervisedTokenDataRuntime,
                                                     PackedTokenDataRuntime)
from turbo_dllm_b200.data.artifacts import (ArtifactError, dataset_fingerprint, load_manifest, validate_artifact,
                                            validate_artifact_for_run)
from turbo_dllm_b200.data.prepare import PreparationError, PreparationSpec, prepare_dataset


def _jsonl(path, rows):
    path.write_text("\n".join(json.dumps(r) for r in rows) + "\n")


def _packed(tmp_path, name="packed", n=40, seqlen=64):
    src = tmp_path / f"{name}.jsonl"
    _jsonl(src, [{"text": f"document {i} " + "x" * (i % 17 + 30)} for i in range(n)])
    spec = PreparationSpec.from_mapping({"source": {"kind": "jsonl", "path": str(src)},
                                         "packing": {"mode": "packed", "sequence_length": seqlen},
                                         "output": {"path": str(tmp_path / name)}})
    return prepare_dataset(spec), tmp_path / name


def test_packed_prepare_validate_and_fingerprint_is_reproducible(tmp_path):
    m1, root = _packed(tmp_path, "a")
    m2, root2 = _packed(tmp_path, "b")
    assert m1["format"] == "dllm_parallel.packed_tokens" and m1["version"] == 1
    assert set(m1["files"]["tokens.i32"]) == {"dtype", "elements", "bytes", "sha256"}
    assert m1["files"]["tokens.i32"]["sha256"] == m2["files"]["tokens.i32"]["sha256"]
    validate_artifact(root)
    toks = np.fromfile(root / "tokens.i32", dtype="<i4")
    assert toks.size == m1["token_count"] and toks.max() <= 257
    fp = dataset_fingerprint(format_name=m1["format"], version=1, metadata=m1["metadata"], files=m1["files"],
                             sample_count=m1["sample_count"], token_count=m1["token_count"])
    assert fp == m1["metadata"]["dataset_fingerprint"]
    assert validate_artifact_for_run(root, vocab_size=1024, mask_token_id=1023, block_size=32)["compatible"]
    with pytest.raises(ArtifactError, match="model vocabulary"):
        validate_artifact_for_run(root, vocab_size=100, mask_token_id=None, block_size=32)


def test_corruption_is_detected(tmp_path):
    _, root = _packed(tmp_path)
    data = bytearray((root / "tokens.i32").read_bytes())
    data[10] ^= 0xFF
    (root / "tokens.i32").write_bytes(bytes(data))
    with pytest.raises(ArtifactError, match="sha256 mismatch"):
        validate_artifact(root)
    (root / "tokens.i32").write_bytes(bytes(data[:-4]))
    with pytest.raises(ArtifactError, match="size"):
        validate_artifact(root)
    man = json.loads((root / "manifest.json").read_text())
    man["token_count"] += 1
    (root / "manifest.json").write_text(json.dumps(man))
    with pytest.raises(ArtifactError):
        validate_artifact(root, check_hashes=False)


def test_indexed_prepare_with_assistant_only_supervision(tmp_path):
    src = tmp_path / "chat.jsonl"
    _jsonl(src, [{"messages": [{"role": "user", "content": "hi there " * (i + 1)},
                               {"role": "assistant", "content": "answer " * (i + 2)}]} for i in range(12)])
    out = tmp_path / "idx"
    spec = PreparationSpec.from_mapping({
        "source": {"kind": "jsonl", "path": str(src)}, "records": {"type": "messages"},
        "supervision": {"mode": "assistant_only"},
        "packing": {"mode": "indexed", "sequence_length": 256, "overflow": "truncate_right", "alignment": 32},
        "output": {"path": str(out)}})
    m = prepare_dataset(spec)
    assert m["format"] == "dllm_parallel.indexed_supervised_tokens"
    assert m["files"]["index.i64"]["columns"] == ["token_offset", "sequence_length", "supervision_start", "sample_id"]
    validate_artifact(out)
    idx = np.fromfile(out / "index.i64", dtype="<i8").reshape(-1, 4)
    assert (idx[:, 1] % 32 == 0).all()
    mask = np.fromfile(out / "loss_mask.u8", dtype=np.uint8)
    assert 0 < mask.sum() < mask.size
    rt = IndexedSupervisedTokenDataRuntime(out, batch_size=2, block_size=32, max_seq_len=256, seed=1)
    b = rt.next_batch()
    assert b.input_ids.shape[0] == 2 and b.supervision_mask.shape == b.input_ids.shape
    assert b.supervision_count == int(b.supervision_mask.sum())


def test_spec_validation_and_overwrite_protection(tmp_path):
    with pytest.raises(PreparationError, match="unknown section"):
        PreparationSpec.from_mapping({"sauce": {}})
    with pytest.raises(PreparationError, match="unknown field"):
        PreparationSpec.from_mapping({"source": {"pth": "x"}, "output": {"path": "y"}})
    with pytest.raises(PreparationError, match="assistant_only"):
        PreparationSpec.from_mapping({"source": {"path": "x"}, "supervision": {"mode": "assistant_only"},
                                      "output": {"path": "y"}})
    _, root = _packed(tmp_path)
    spec = PreparationSpec.from_mapping({"source": {"kind": "jsonl", "path": str(tmp_path / "packed.jsonl")},
                                         "output": {"path": str(root)}})
    with pytest.raises(PreparationError, match="exists"):
        prepare_dataset(spec)


def test_packed_runtime_shards_resumes_and_blends(tmp_path):
    _, root = _packed(tmp_path, n=200)
    a = PackedTokenDataRuntime(root, batch_size=2, seq_len=64, dp_rank=0, dp_size=2, seed=3)
    b = PackedTokenDataRuntime(root, batch_size=2, seq_len=64, dp_rank=1, dp_size=2, seed=3)
    ia, ib = a.next_batch().sample_ids, b.next_batch().sample_ids
    assert not set(ia.tolist()) & set(ib.tolist())
    a.next_batch()
    state = a.state_dict()
    want = a.next_batch().input_ids
    c = PackedTokenDataRuntime(root, batch_size=2, seq_len=64, dp_rank=0, dp_size=2, seed=3)
    c.load_state_dict(state)
    assert torch.equal(c.next_batch().input_ids, want)
    _, root2 = _packed(tmp_path, "other", n=150)
    blend = BlendedPackedTokenDataRuntime([(3.0, PackedTokenDataRuntime(root, batch_size=1, seq_len=64)),
                                           (1.0, PackedTokenDataRuntime(root2, batch_size=1, seq_len=64))], seed=5)
    seq1 = [blend.next_batch().input_ids.clone() for _ in range(4)]
    st = blend.state_dict()
    nxt = blend.next_batch().input_ids
    blend2 = BlendedPackedTokenDataRuntime([(3.0, PackedTokenDataRuntime(root, batch_size=1, seq_len=64)),
                                            (1.0, PackedTokenDataRuntime(root2, batch_size=1, seq_len=64))], seed=5)
    blend2.load_state_dict(st)
    assert torch.equal(blend2.next_batch().input_ids, nxt)


def test_cli_data_and_init(tmp_path, capsys):
    from turbo_dllm_b200.cli.main import run

    proj = tmp_path / "proj"
    assert run(["init", str(proj)]) == 0
    assert (proj / "train.yaml").exists() and (proj / "prepare.yaml").exists()
    assert run(["init", str(proj)]) == 2
    _, root = _packed(tmp_path)
    assert run(["data", "validate", str(root)]) == 0
    assert run(["data", "stats", str(root)]) == 0
    assert run(["data", "validate", str(tmp_path / "missing")]) == 2


def _trajectory_artifact(root, lengths_by_group, vocab=900, seed=0):
    from turbo_dllm_b200.data.artifacts import write_indexed_artifact

    rng = np.random.default_rng(seed)
    samples, sid = [], 0
    for gid, lens in lengths_by_group.items():
        for L in lens:
            mask = np.zeros(L, dtype=np.uint8)
            mask[L // 2:] = 1
            samples.append({"tokens": rng.integers(0, vocab, L), "loss_mask": mask, "sample_id": sid, "group": gid})
            sid += 1
    write_indexed_artifact(root, samples, metadata={"block_size": 32, "tokenizer": {"vocab_size": vocab}},
                           with_groups=True)


def test_trajectory_step_units_and_turn_mean_reduction(tmp_path):
    """One optimizer step = one trajectory (its turns as micro-batches, last turn weighted); `turn_mean` averages
    the turns' token-mean losses instead of pooling tokens (dllm_parallel/core/data.py:966-1010, :739)."""
    from turbo_dllm_b200.config.run_spec import RunSpec, RunSpecError
    from turbo_dllm_b200.training.session import TrainingSession

    root = tmp_path / "traj"
    _trajectory_artifact(root, {7: [64, 128, 64], 3: [128], 9: [64, 64]})
    rt = IndexedSupervisedTokenDataRuntime(root, batch_size=1, block_size=32, max_seq_len=128, shuffle=False,
                                           optimizer_step_unit="trajectory", terminal_turn_weight=3.0)
    steps = [rt.next_optimizer_step_batches(1) for _ in range(3)]
    assert [len(s) for s in steps] == [1, 3, 2]                       # groups 3, 7, 9 in id order
    assert [b.turn_weight for b in steps[1]] == [1.0, 1.0, 3.0]
    assert [b.input_ids.shape[1] for b in steps[1]] == [64, 128, 64]
    state = rt.state_dict()
    first_again = rt.next_optimizer_step_batches(1)                   # wraps into the next epoch
    rt2 = IndexedSupervisedTokenDataRuntime(root, batch_size=1, block_size=32, max_seq_len=128, shuffle=False,
                                            optimizer_step_unit="trajectory", terminal_turn_weight=3.0)
    rt2.load_state_dict(state)
    assert torch.equal(rt2.next_optimizer_step_batches(1)[0].input_ids, first_again[0].input_ids)
    with pytest.raises(ArtifactError, match="hand out whole optimizer steps"):
        rt.next_batch()
    # a trajectory with a turn that does not fit is refused, never shortened
    bad = tmp_path / "bad"
    _trajectory_artifact(bad, {1: [64, 96 + 1]})
    with pytest.raises(ArtifactError, match="ineligible"):
        IndexedSupervisedTokenDataRuntime(bad, batch_size=1, block_size=32, max_seq_len=128,
                                          optimizer_step_unit="trajectory")

    def spec(reduction):
        return RunSpec.from_mapping({
            "model": {"id": "synthetic:tiny-qwen3", "seq_len": 128, "dtype": "fp32", "num_layers": 1},
            "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
            "data": {"input_mode": "dataset", "dataset_path": str(root), "shuffle": False,
                     "optimizer_step_unit": "trajectory", "trajectory_loss_reduction": reduction,
                     "trajectory_terminal_turn_weight": 3.0},
            "training": {"batch_size": 1, "steps": 3},
            "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
            "optimizer": {"lr": 1e-3}}).validate()

    a, b = TrainingSession(spec("token_mean"), device="cpu"), TrainingSession(spec("turn_mean"), device="cpu")
    ra = [a.step() for _ in range(3)]
    rb = [b.step() for _ in range(3)]
    la = [float(r.loss_sum) / r.denominator for r in ra]
    lb = [float(r.loss_sum) / r.denominator for r in rb]
    assert all(x == x and x > 0 for x in la + lb)
    assert la[0] == pytest.approx(lb[0], rel=1e-5)        # a single-turn trajectory: both reductions agree
    assert abs(la[1] - lb[1]) > 1e-6                      # three turns of different lengths and weights: they differ
    assert not torch.equal(a.model.flat.data, b.model.flat.data)
    with pytest.raises(RunSpecError, match="turn_mean"):
        RunSpec.from_mapping({"data": {"trajectory_loss_reduction": "turn_mean"},
                              "model": {"id": "synthetic:tiny-qwen3", "dtype": "fp32"}}).validate()
