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
