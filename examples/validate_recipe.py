"""Validates a packaged recipe (or a train.yaml path) for a world size and prints the resolved topology.

    python examples/validate_recipe.py csbp8-qwen3-1p7b-128k 8
"""
import sys

from turbo_dllm_b200.config.run_spec import RunSpec, load_run_spec
from turbo_dllm_b200.recipes import recipe_text


def main(argv):
    name, world = argv[0], int(argv[1]) if len(argv) > 1 else 1
    if name.endswith((".yaml", ".yml")):
        spec = load_run_spec(name)
    else:
        import yaml

        spec = RunSpec.from_mapping(yaml.safe_load(recipe_text(name)))
    spec = spec.validate(world_size=world)
    t = spec.topology
    local = max(t.context_parallel_size, t.block_parallel_size)
    dp = max(world // (local * t.tensor_parallel_size * t.expert_parallel_size), 1)
    print(f"{name}: ok for {world} ranks; DP {dp} CP {t.context_parallel_size} BP {t.block_parallel_size} "
          f"TP {t.tensor_parallel_size} EP {t.expert_parallel_size}; global batch {spec.global_batch(dp)}")


if __name__ == "__main__":
    main(sys.argv[1:] or ["cpu-single"])
