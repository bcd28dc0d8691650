"""`python -m turbo_dllm_b200.training --config train.yaml`: the dllm-train worker entry point.
Wrapped in torch elastic's error recorder so torchrun collects a per-rank error file
(cf. dllm_parallel/training/entrypoint.py:14-60)."""
from torch.distributed.elastic.multiprocessing.errors import record

from .trainer import main

if __name__ == "__main__":
    record(main)()
