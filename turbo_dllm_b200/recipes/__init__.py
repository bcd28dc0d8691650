"""Packaged recipe catalog (`dllm recipe list|show|copy`, `dllm launch --recipe NAME`).

`manifest.yaml` (format `dllm.recipe_catalog.v1`) lists smoke, example and production recipes;
each is a plain RunSpec YAML. Counterpart of dllm_parallel/recipes/__init__.py:13-77.
"""
from __future__ import annotations

import os
from pathlib import Path

import yaml

ROOT = Path(__file__).resolve().parent
CATALOG_FORMAT = "dllm.recipe_catalog.v1"


def _manifest() -> dict:
    data = yaml.safe_load((ROOT / "manifest.yaml").read_text())
    if data.get("format") != CATALOG_FORMAT:
        raise ValueError(f"unexpected recipe catalog format {data.get('format')!r}")
    return data


def list_recipes(kind: str | None = None) -> list[dict]:
    return [r for r in _manifest()["recipes"] if kind is None or r["kind"] == kind]


def recipe_path(name: str) -> Path:
    for r in _manifest()["recipes"]:
        if r["name"] == name:
            return ROOT / r["path"]
    raise KeyError(f"unknown recipe {name!r}; known: {', '.join(r['name'] for r in _manifest()['recipes'])}")


def recipe_text(name: str) -> str:
    return recipe_path(name).read_text()


def copy_recipe(name: str, destination: str) -> str:
    """Exclusive create: never overwrites an existing file."""
    text = recipe_text(name)
    fd = os.open(destination, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o644)
    with os.fdopen(fd, "w") as f:
        f.write(text)
    return destination
