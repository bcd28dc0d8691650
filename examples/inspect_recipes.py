"""Lists the packaged recipes (works from an installed wheel: no source checkout needed)."""
from turbo_dllm_b200.recipes import list_recipes

for r in list_recipes():
    print(f"{r['name']:32s} {r['kind']:8s} {r['description']}")
