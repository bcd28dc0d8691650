"""Documentation consistency: what the docs, the README and the packaged recipes name must exist
(cf. the reference's release tier, tests/release/: docs consistency and repository boundary checks)."""
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
DOCS = sorted((ROOT / "docs").rglob("*.md")) + [ROOT / "README.md"]


def _schema():
    from turbo_dllm_b200.config import schema

    return {name: {f.name for f in rows} for name, rows in schema.SECTIONS.items()}


def test_run_spec_fields_named_in_the_docs_exist():
    """Every `section.field` in back-ticks whose section is a run-spec section names a real field (wildcards such as
    `optimizer.zero_*` must match at least one)."""
    secs = _schema()
    pat = re.compile(r"`(" + "|".join(secs) + r")\.([a-z0-9_*]+)(?::[^`]*)?`")
    missing = []
    for doc in DOCS:
        for sec, field in pat.findall(doc.read_text()):
            if "*" in field:
                rx = re.compile("^" + field.replace("*", ".*") + "$")
                if not any(rx.match(f) for f in secs[sec]):
                    missing.append(f"{doc.relative_to(ROOT)}: {sec}.{field}")
            elif field not in secs[sec]:
                missing.append(f"{doc.relative_to(ROOT)}: {sec}.{field}")
    # attribute-style mentions that are not run-spec fields (methods, file suffixes, ...)
    allowed = {"model.safetensors", "model.flat", "model.id directory"}
    missing = [m for m in missing if m.split(": ")[1] not in allowed]
    assert not missing, "\n".join(missing)


def test_files_and_modules_named_in_the_docs_exist():
    """Package paths in back-ticks (`parallel/fsdp.py`, `models/hf_loader.py::name`, `csrc/*.cu`, tests, recipes) exist,
    and a `file.py::symbol` names something defined in that file."""
    pkg = ROOT / "turbo_dllm_b200"
    pat = re.compile(r"`((?:[a-zA-Z0-9_]+/)+[a-zA-Z0-9_.*]+\.(?:py|cu|cuh|h|yaml|sh|md|json))(?:::([A-Za-z0-9_.]+))?`")
    problems = []
    for doc in DOCS + [ROOT / "DESIGN.md"]:
        for path, symbol in pat.findall(doc.read_text()):
            if path.startswith(("dllm_parallel/", "data/", "export/", "ckpts/", "features/", "gpurun_out/", "dist/", "raw/",
                                "shards/", "corpus/")):
                continue                     # reference citations and example user paths
            cands = [ROOT / path, pkg / path]
            if "*" in path:
                hit = any(list(c.parent.glob(c.name)) for c in cands if c.parent.exists())
                if not hit:
                    problems.append(f"{doc.name}: {path} matches nothing")
                continue
            found = next((c for c in cands if c.exists()), None)
            if found is None:
                problems.append(f"{doc.name}: {path} does not exist")
            elif symbol and found.suffix == ".py":
                name = symbol.split(".")[0]
                text = found.read_text()
                if not re.search(rf"^\s*(def|class)\s+{re.escape(name)}\b|^{re.escape(name)}\s*[:=]", text, re.M):
                    problems.append(f"{doc.name}: {path} defines no {name}")
    assert not problems, "\n".join(sorted(set(problems)))


def test_cli_commands_named_in_the_docs_exist():
    """`dllm <command> <sub-command>` in the docs are commands the dispatcher knows."""
    from turbo_dllm_b200.cli import main as cli

    top = {"bundle", "config", "data", "doctor", "dflash", "init", "launch", "recipe", "train", "checkpoint"}
    subs = {"data": {"prepare", "inspect", "validate", "stats"},
            "dflash": {"prepare-features", "build-draft-vocab", "export", "validate-export", "validate-vllm", "serve-sglang",
                       "serve-vllm", "verify-sglang", "verify-vllm"}}
    bad = []
    for doc in DOCS:
        for cmd, sub in re.findall(r"`?dllm ([a-z]+)(?: ([a-z][a-z-]+))?", doc.read_text()):
            if cmd not in top:
                bad.append(f"{doc.name}: dllm {cmd}")
            elif cmd in subs and sub and sub not in subs[cmd] and not sub.startswith("-"):
                bad.append(f"{doc.name}: dllm {cmd} {sub}")
    assert not bad, "\n".join(sorted(set(bad)))
    assert callable(cli.run)


def test_every_packaged_recipe_validates_and_is_listed():
    import yaml

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.recipes import list_recipes, recipe_text

    names = [r["name"] if isinstance(r, dict) else r for r in list_recipes()]
    assert len(names) >= 15
    for name in names:
        RunSpec.from_mapping(yaml.safe_load(recipe_text(name))).validate()
    on_disk = {p.stem for p in (ROOT / "turbo_dllm_b200" / "recipes").rglob("*.yaml") if p.name != "manifest.yaml"}
    assert on_disk == {n.split("/")[-1] for n in names}


def test_shell_scripts_parse_and_are_executable():
    """Every shipped shell script passes `bash -n` and carries the executable bit."""
    import os
    import subprocess

    scripts = sorted(ROOT.glob("packaging/**/*.sh")) + sorted((ROOT / "turbo_dllm_b200" / "cli").glob("*.sh"))
    assert len(scripts) >= 10
    for sh in scripts:
        assert subprocess.run(["bash", "-n", str(sh)], capture_output=True).returncode == 0, sh
        assert os.access(sh, os.X_OK), f"{sh} is not executable"
