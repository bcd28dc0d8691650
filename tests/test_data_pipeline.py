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


def test_preparation_front_end_schema_sources_and_policies(tmp_path):
    """The documented schema end to end: relative paths against the file, gzip + glob sources, nested fields, string
    ids, assistant-only supervision through the template's own mask, automatic artifact format."""
    import gzip

    import yaml

    from turbo_dllm_b200.data.prepare import load_preparation_spec, redact_secrets

    (tmp_path / "raw").mkdir()
    rows = [{"id": f"conv-{i}", "meta": {"thread": f"t{i // 2}"},
             "dialog": {"turns": [{"speaker": "user", "body": "question " * (i + 3)},
                                  {"speaker": "assistant", "body": "reply " * (i + 4), "tool_calls": []}]}}
            for i in range(10)]
    with gzip.open(tmp_path / "raw" / "a-000.jsonl.gz", "wt") as f:
        f.write("\n".join(json.dumps(r) for r in rows[:5]) + "\n\n")
    _jsonl(tmp_path / "raw" / "a-001.jsonl", rows[5:])
    (tmp_path / "prepare.yaml").write_text(yaml.safe_dump({
        "format": "dllm.data.prepare.v1",
        "source": {"type": "jsonl", "path": "raw/a-*.jsonl*", "loader_kwargs": {"hf_token": "s3cret", "n": 1}},
        "records": {"type": "messages", "messages_field": "dialog.turns", "role_field": "speaker", "content_field": "body",
                    "sample_id_field": "id", "group_id_field": "meta.thread"},
        "tokenizer": {"model": "byte", "add_eos": True},
        "supervision": {"policy": "assistant_only"},
        "packing": {"maximum_length": 512, "alignment": 16, "alignment_policy": "truncate_left", "minimum_length": 16},
        "output": {"path": "prepared", "format": "auto"}}))
    spec = load_preparation_spec(tmp_path / "prepare.yaml")
    assert spec.artifact_format == "indexed" and spec.output["path"] == str(tmp_path / "prepared")
    m = prepare_dataset(spec)
    assert m["format"] == "dllm_parallel.indexed_supervised_tokens" and m["sample_count"] == 10
    assert "groups.i64" in m["files"] and m["metadata"]["supervision_shape"] == "assistant_only"
    assert m["metadata"]["preparation"]["source"]["loader_kwargs"] == {"hf_token": "<redacted>", "n": 1}
    assert m["metadata"]["source"]["loader_kwargs"]["hf_token"] == "<redacted>"
    assert [f["name"] for f in m["metadata"]["source"]["files"]] == ["a-000.jsonl.gz", "a-001.jsonl"]
    validate_artifact(tmp_path / "prepared")
    idx = np.fromfile(tmp_path / "prepared" / "index.i64", dtype="<i8").reshape(-1, 4)
    assert (idx[:, 1] % 16 == 0).all() and len(set(idx[:, 3].tolist())) == 10 and (idx[:, 3] > 0).all()
    groups = np.fromfile(tmp_path / "prepared" / "groups.i64", dtype="<i8")
    assert groups[0] == groups[1] and groups[1] != groups[2]          # the same thread -> the same hashed group id
    toks = np.fromfile(tmp_path / "prepared" / "tokens.i32", dtype="<i4")
    mask = np.fromfile(tmp_path / "prepared" / "loss_mask.u8", dtype=np.uint8)
    # left truncation keeps the end of each sample: the explicit EOS is the last token and is supervised
    ends = idx[:, 0] + idx[:, 1] - 1
    assert (toks[ends] == 257).all() and mask[ends].all()
    assert not mask[toks == 260].any()                                  # user role markers are never supervised
    assert redact_secrets({"a": [{"api_key": 1, "b": 2}]}) == {"a": [{"api_key": "<redacted>", "b": 2}]}
    # conflicting spellings of one setting are refused
    with pytest.raises(PreparationError, match="two names"):
        PreparationSpec.from_mapping({"source": {"type": "jsonl", "kind": "text", "path": "x"}, "output": {"path": "y"}})
    with pytest.raises(PreparationError, match="output.format=packed"):
        PreparationSpec.from_mapping({"source": {"path": "x"}, "records": {"type": "messages"},
                                      "supervision": {"policy": "assistant_only"}, "output": {"path": "y", "format": "packed"}})
    with pytest.raises(PreparationError, match="split"):
        PreparationSpec.from_mapping({"source": {"path": "x"}, "records": {"type": "messages"},
                                      "supervision": {"policy": "assistant_only"},
                                      "packing": {"maximum_length": 64, "overflow": "split"}, "output": {"path": "y"}})


def test_pretokenized_sources_prompt_completion_and_separators(tmp_path):
    from turbo_dllm_b200.data import prepare as prep

    # raw int32 stream (one record) + a 2-D .npy (one record per row), split into chunks, separators between documents only
    np.arange(100, dtype="<i4").tofile(tmp_path / "a.i32")
    np.save(tmp_path / "b.npy", np.arange(200, 260, dtype=np.int64).reshape(2, 30))
    m = prepare_dataset(PreparationSpec.from_mapping({
        "source": {"type": "pretokenized", "paths": [str(tmp_path / "a.i32"), str(tmp_path / "b.npy")]},
        "records": {"type": "pretokenized"},
        "packing": {"maximum_length": 64, "overflow": "split", "separator_token_id": 999},
        "output": {"path": str(tmp_path / "tok")}}))
    toks = np.fromfile(tmp_path / "tok" / "tokens.i32", dtype="<i4")
    assert toks.tolist() == list(range(100)) + [999] + list(range(200, 230)) + [999] + list(range(230, 260))
    assert m["stats"]["split_records"] == 1 and m["stats"]["separator_tokens"] == 2 and m["sample_count"] == 3
    # provided supervision: loss_mask wins, labels != -100 is the fallback; named masks for the other policies
    _jsonl(tmp_path / "p.jsonl", [
        {"input_ids": list(range(8)), "loss_mask": [0, 0, 0, 0, 1, 1, 1, 1], "labels": [1] * 8},
        {"input_ids": list(range(8)), "labels": [-100, -100, 5, 5, 5, 5, 5, 5], "assistant_masks": [0] * 7 + [1]}])
    for policy, want in (("provided", [4, 6]), ("assistant_only", None)):
        out = tmp_path / f"prov_{policy}"
        spec = PreparationSpec.from_mapping({
            "source": {"type": "pretokenized", "path": str(tmp_path / "p.jsonl")}, "records": {"type": "pretokenized"},
            "supervision": {"policy": policy}, "packing": {"maximum_length": 8}, "output": {"path": str(out)}})
        if want is None:
            with pytest.raises(PreparationError, match="assistant_masks"):
                prepare_dataset(spec)           # the first record has no assistant mask: nothing is guessed
            continue
        prepare_dataset(spec)
        mask = np.fromfile(out / "loss_mask.u8", dtype=np.uint8).reshape(2, 8)
        assert mask.sum(1).tolist() == want
    # prompt / completion given as message lists: the rendered prompt must be a prefix; only the completion is supervised
    _jsonl(tmp_path / "pc.jsonl", [{"prompt": [{"role": "user", "content": "explain"}],
                                    "completion": [{"role": "assistant", "content": "because"}]},
                                   {"prompt": "2+2=", "completion": "4"}])
    with pytest.raises(PreparationError, match="both be strings or both"):
        _jsonl(tmp_path / "bad.jsonl", [{"prompt": "x", "completion": [{"role": "assistant", "content": "y"}]}])
        prepare_dataset(PreparationSpec.from_mapping({
            "source": {"path": str(tmp_path / "bad.jsonl")}, "records": {"type": "prompt_completion"},
            "supervision": {"policy": "completion_only"}, "output": {"path": str(tmp_path / "bad")}}))
    prepare_dataset(PreparationSpec.from_mapping({
        "source": {"path": str(tmp_path / "pc.jsonl")}, "records": {"type": "prompt_completion"},
        "supervision": {"policy": "completion_only"}, "output": {"path": str(tmp_path / "pc")}}))
    idx = np.fromfile(tmp_path / "pc" / "index.i64", dtype="<i8").reshape(-1, 4)
    mask = np.fromfile(tmp_path / "pc" / "loss_mask.u8", dtype=np.uint8)
    toks = np.fromfile(tmp_path / "pc" / "tokens.i32", dtype="<i4")
    first = slice(idx[0, 0], idx[0, 0] + idx[0, 1])
    # user marker + "explain" + end-of-turn + assistant marker are the prompt; "because" + end-of-turn the completion
    assert mask[first].tolist() == [0] * (1 + 7 + 1 + 1) + [1] * (7 + 1) and toks[first][9] == prep.ByteTokenizer.ROLE["assistant"]
    second = slice(idx[1, 0], idx[1, 0] + idx[1, 1])
    assert mask[second].tolist() == [0, 0, 0, 0, 1]
    # alignment policies of supervised samples
    rec = prep.TokenizedRecord(np.arange(10, dtype=np.int32), np.ones(10, np.uint8), 0)
    assert prep.align_record(rec, 4, "truncate_right", 0).tokens.tolist() == list(range(8))
    assert prep.align_record(rec, 4, "truncate_left", 0).tokens.tolist() == list(range(2, 10))
    padded = prep.align_record(rec, 4, "pad", 7)
    assert padded.tokens.tolist() == list(range(10)) + [7, 7] and padded.loss_mask[-2:].tolist() == [0, 0]
    assert prep.align_record(prep.TokenizedRecord(np.arange(3, dtype=np.int32), np.ones(3, np.uint8), 0), 4, "truncate_right", 0) is None
    with pytest.raises(PreparationError, match="alignment_policy=reject"):
        prep.align_record(rec, 4, "reject", 0)
    # text in line mode
    (tmp_path / "lines.txt").write_text("first line\n\nsecond line\n")
    m = prepare_dataset(PreparationSpec.from_mapping({"source": {"type": "text", "path": str(tmp_path / "lines.txt"), "text_mode": "line"},
                                                      "output": {"path": str(tmp_path / "lines")}}))
    assert m["sample_count"] == 2 and m["token_count"] == len("first line") + len("second line")


def test_registered_sources_formatters_and_cli_overrides(tmp_path, capsys):
    import yaml

    from turbo_dllm_b200.cli.main import run
    from turbo_dllm_b200.data import prepare as prep

    prep.register_source("unit_counter", lambda src: ({"n": i} for i in range(int(src["limit"] or 4))), replace=True)
    prep.register_formatter("unit_number_words", lambda rec, r: prep.FormattedRecord(text=f"number {rec['n']}", sample_id=rec["n"]),
                            replace=True)
    with pytest.raises(ValueError, match="already registered"):
        prep.register_source("unit_counter", lambda src: iter(()))
    with pytest.raises(PreparationError, match="source.type"):
        PreparationSpec.from_mapping({"source": {"type": "nowhere", "path": "x"}, "output": {"path": "y"}})
    cfg = tmp_path / "prepare.yaml"
    cfg.write_text(yaml.safe_dump({"source": {"type": "unit_counter", "id": "counter"}, "records": {"type": "unit_number_words"},
                                   "output": {"path": "out_a"}}))
    assert run(["data", "prepare", "--config", str(cfg)]) == 0
    first = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert first["samples"] == 4 and (tmp_path / "out_a" / "manifest.json").exists()
    assert run(["data", "prepare", "--config", str(cfg)]) == 2                       # exists, no overwrite
    capsys.readouterr()
    assert run(["data", "prepare", "--config", str(cfg), "--overwrite"]) == 0
    capsys.readouterr()
    assert run(["data", "prepare", "--config", str(cfg), "--output", str(tmp_path / "out_b")]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["dataset_fingerprint"] == first["dataset_fingerprint"]
    # compatibility of the artifact with a training run
    train = tmp_path / "train.yaml"
    train.write_text(yaml.safe_dump({"model": {"id": "synthetic:tiny-qwen3", "seq_len": 64},
                                     "objective": {"name": "standard_block_diffusion", "block_size": 16}}))
    assert run(["data", "validate", str(tmp_path / "out_b"), "--config", str(train)]) == 2   # 36 tokens < one 64-token sequence
    assert "fewer than one sequence" in capsys.readouterr().err
    train.write_text(yaml.safe_dump({"model": {"id": "synthetic:tiny-qwen3", "seq_len": 32},
                                     "objective": {"name": "standard_block_diffusion", "block_size": 16},
                                     "topology": {"context_parallel_size": 1, "block_parallel_size": 1}}))
    assert run(["data", "validate", str(tmp_path / "out_b"), "--config", str(train)]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["run"]["compatible"]


def _tiny_hf_tokenizer(path, template):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    vocab = {"<unk>": 0, "<eos>": 1, "<|user|>": 2, "<|assistant|>": 3, "<|end|>": 4}
    for i, w in enumerate("hello how are you fine thanks explain because".split()):
        vocab[w] = 5 + i
    t = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    t.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok = PreTrainedTokenizerFast(tokenizer_object=t, unk_token="<unk>", eos_token="<eos>")
    if template:
        tok.chat_template = template
    tok.save_pretrained(str(path))


def test_chat_template_supervision_with_a_hugging_face_tokenizer(tmp_path):
    """Assistant-only supervision comes from the template's generation markers; a template without them is refused
    rather than guessed; message-shaped prompt / completion pairs split at the rendered prompt."""
    marked = ("{% for m in messages %}{% if m['role']=='assistant' %}<|assistant|> {% generation %}{{ m['content'] }} <|end|> "
              "{% endgeneration %}{% else %}<|user|> {{ m['content'] }} <|end|> {% endif %}{% endfor %}"
              "{% if add_generation_prompt %}<|assistant|> {% endif %}")
    plain = marked.replace("{% generation %}", "").replace("{% endgeneration %}", "")
    _tiny_hf_tokenizer(tmp_path / "tok_marked", marked)
    _tiny_hf_tokenizer(tmp_path / "tok_plain", plain)
    _tiny_hf_tokenizer(tmp_path / "tok_none", None)
    _jsonl(tmp_path / "chat.jsonl", [{"messages": [{"role": "user", "content": "hello how are you"},
                                                   {"role": "assistant", "content": "fine thanks"}]}])

    def spec(tok, out, **over):
        return PreparationSpec.from_mapping({
            "source": {"type": "jsonl", "path": str(tmp_path / "chat.jsonl")}, "records": {"type": "messages"},
            "tokenizer": {"model": str(tmp_path / tok), "add_eos": True, **over.get("tokenizer", {})},
            "supervision": {"policy": over.get("policy", "assistant_only")}, "output": {"path": str(tmp_path / out)}})

    m = prepare_dataset(spec("tok_marked", "a"))
    toks = np.fromfile(tmp_path / "a" / "tokens.i32", dtype="<i4").tolist()
    mask = np.fromfile(tmp_path / "a" / "loss_mask.u8", dtype=np.uint8).tolist()
    assert toks == [2, 5, 6, 7, 8, 4, 3, 9, 10, 4, 1] and mask == [0] * 7 + [1, 1, 1, 1]
    assert m["metadata"]["tokenizer"]["vocab_size"] == 13
    with pytest.raises(PreparationError, match="never guessed"):
        prepare_dataset(spec("tok_plain", "b"))
    with pytest.raises(PreparationError, match="no chat template"):
        prepare_dataset(spec("tok_none", "c"))
    # the template given in the spec replaces the tokenizer's own
    prepare_dataset(spec("tok_none", "d", tokenizer={"chat_template": marked}))
    assert np.fromfile(tmp_path / "d" / "loss_mask.u8", dtype=np.uint8).tolist() == mask
    # prompt / completion as message lists
    _jsonl(tmp_path / "pc.jsonl", [{"prompt": [{"role": "user", "content": "explain"}],
                                    "completion": [{"role": "assistant", "content": "because"}]}])
    prepare_dataset(PreparationSpec.from_mapping({
        "source": {"type": "jsonl", "path": str(tmp_path / "pc.jsonl")}, "records": {"type": "prompt_completion"},
        "tokenizer": {"model": str(tmp_path / "tok_plain")}, "supervision": {"policy": "completion_only"},
        "output": {"path": str(tmp_path / "e")}}))
    assert np.fromfile(tmp_path / "e" / "tokens.i32", dtype="<i4").tolist() == [2, 11, 4, 3, 12, 4]
    assert np.fromfile(tmp_path / "e" / "loss_mask.u8", dtype=np.uint8).tolist() == [0, 0, 0, 0, 1, 1]


def test_flat_token_files_text_files_and_text_mode(tmp_path):
    """`data.dataset_path` may name a flat token file or a text file instead of a prepared artifact, and
    `data.input_mode: text` trains on a built-in paragraph; all are sharded by rank and resumable."""
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.training.session import TrainingSession

    stream = (np.arange(4096) % 1000).astype("<i4")
    stream.tofile(tmp_path / "flat.i32")
    stream.astype("<i8").tofile(tmp_path / "flat.bin")
    torch.save({"input_ids": torch.from_numpy(stream.astype(np.int64))}, tmp_path / "flat.pt")
    runs = {}
    for name in ("flat.i32", "flat.bin", "flat.pt"):
        rt = PackedTokenDataRuntime.from_token_file(tmp_path / name, batch_size=2, seq_len=64, seed=1, vocab_size=1024)
        runs[name] = rt.next_batch().input_ids
        assert rt.fingerprint.startswith("file:")
    assert torch.equal(runs["flat.i32"], runs["flat.bin"]) and torch.equal(runs["flat.i32"], runs["flat.pt"])
    with pytest.raises(ArtifactError, match="outside the model vocabulary"):
        PackedTokenDataRuntime.from_token_file(tmp_path / "flat.i32", batch_size=2, seq_len=64, vocab_size=500)
    a = PackedTokenDataRuntime.from_token_file(tmp_path / "flat.i32", batch_size=2, seq_len=64, dp_rank=0, dp_size=2, seed=1)
    b = PackedTokenDataRuntime.from_token_file(tmp_path / "flat.i32", batch_size=2, seq_len=64, dp_rank=1, dp_size=2, seed=1)
    assert not set(a.next_batch().sample_ids.tolist()) & set(b.next_batch().sample_ids.tolist())
    state = a.state_dict()
    want = a.next_batch().input_ids
    c = PackedTokenDataRuntime.from_token_file(tmp_path / "flat.i32", batch_size=2, seq_len=64, dp_rank=0, dp_size=2, seed=1)
    c.load_state_dict(state)
    assert torch.equal(c.next_batch().input_ids, want)
    np.zeros(4096, dtype="<i4").tofile(tmp_path / "other.i32")
    with pytest.raises(ArtifactError, match="different dataset"):
        PackedTokenDataRuntime.from_token_file(tmp_path / "other.i32", batch_size=2, seq_len=64, dp_size=2).load_state_dict(state)

    base = {"model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "num_layers": 1},
            "objective": {"name": "standard_block_diffusion", "block_size": 16}, "training": {"batch_size": 2, "steps": 1},
            "topology": {"context_parallel_size": 1, "block_parallel_size": 1}}
    (tmp_path / "corpus.txt").write_text("some plain text for a quick run. " * 40)
    for data in ({"input_mode": "dataset", "dataset_path": str(tmp_path / "flat.i32")},
                 {"input_mode": "dataset", "dataset_path": str(tmp_path / "corpus.txt")},
                 {"input_mode": "text"}):
        s = TrainingSession(RunSpec.from_mapping({**base, "data": data}).validate(), device="cpu")
        r = s.step()
        assert torch.isfinite(r.loss_sum) and isinstance(s.data, PackedTokenDataRuntime)
    assert int(s.data.tokens.max()) < 256                    # the byte stand-in tokenised the built-in paragraph


def test_blend_manifest_file(tmp_path):
    """A JSON blend manifest mixes prepared artifacts and flat token files by weight; member paths are relative to it."""
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.data.artifact_runtimes import build_artifact_runtime

    _packed(tmp_path, "prepared", n=200)
    (np.full(8192, 7)).astype("<i4").tofile(tmp_path / "sevens.i32")
    (tmp_path / "blend.json").write_text(json.dumps({"datasets": [{"path": "prepared", "weight": 1.0},
                                                                  {"path": "sevens.i32", "weight": 3.0}]}))
    spec = RunSpec.from_mapping({"model": {"id": "synthetic:tiny-qwen3", "seq_len": 64},
                                 "objective": {"name": "standard_block_diffusion", "block_size": 16},
                                 "training": {"batch_size": 1}, "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
                                 "data": {"input_mode": "dataset", "dataset_path": str(tmp_path / "blend.json"), "blend_seed": 5}}).validate()
    rt = build_artifact_runtime(spec, device="cpu", dp_rank=0, dp_size=1)
    assert isinstance(rt, BlendedPackedTokenDataRuntime)
    sevens = sum(bool((rt.next_batch().input_ids == 7).all()) for _ in range(40))
    assert 20 <= sevens <= 38                                   # weight 3 : 1
    (tmp_path / "bad.json").write_text(json.dumps({"datasets": []}))
    with pytest.raises(ArtifactError, match="blend manifest"):
        build_artifact_runtime(spec.with_overrides({"data": {"dataset_path": str(tmp_path / "bad.json")}}), device="cpu", dp_rank=0, dp_size=1)


def test_batches_share_the_response_start_for_native_sft(tmp_path):
    from turbo_dllm_b200.data.artifacts import write_indexed_artifact

    rng = np.random.default_rng(0)
    samples = []
    for i in range(64):
        start = [16, 32][i % 2]
        mask = np.zeros(64, np.uint8)
        mask[start:] = 1
        samples.append({"tokens": rng.integers(0, 500, 64).astype(np.int32), "loss_mask": mask, "sample_id": i})
    write_indexed_artifact(tmp_path / "idx", samples, metadata={"tokenizer": {"vocab_size": 512}})
    grouped = IndexedSupervisedTokenDataRuntime(tmp_path / "idx", batch_size=4, block_size=16, max_seq_len=64, seed=1,
                                                group_by_supervision_start=True)
    plain = IndexedSupervisedTokenDataRuntime(tmp_path / "idx", batch_size=4, block_size=16, max_seq_len=64, seed=1)
    mixed = 0
    for _ in range(8):
        starts = grouped.next_batch().supervision_mask.int().argmax(1)
        assert len(set(starts.tolist())) == 1
        mixed += len(set(plain.next_batch().supervision_mask.int().argmax(1).tolist())) > 1
    assert mixed > 0
