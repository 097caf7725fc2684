"""The documentation names only things that exist, and documents every configuration field."""
import dataclasses
import os
import re

import forgeminds_b200 as fm

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = [os.path.join(ROOT, "docs", "documentation.md"), os.path.join(ROOT, "README.md"),
        os.path.join(ROOT, "docs", "performance.md"), os.path.join(ROOT, "docs", "offload.md")]


def _text(path):
    with open(path, encoding="utf-8") as f:
        return f.read()


def _resolve(dotted: str):
    import importlib
    obj, path = fm, fm.__name__
    for part in dotted.split(".")[1:]:
        path = f"{path}.{part}"
        try:
            obj = getattr(obj, part)
        except AttributeError:
            try:
                obj = importlib.import_module(path)          # a submodule that nothing imported yet
            except ImportError:
                raise AttributeError(dotted) from None
    return obj


def test_every_fm_name_in_the_docs_resolves():
    names = set()
    for path in DOCS:
        if os.path.exists(path):
            names |= set(re.findall(r"\bfm(?:\.[A-Za-z_][A-Za-z0-9_]*)+", _text(path)))
    assert len(names) > 30
    missing = []
    for name in sorted(names):
        try:
            _resolve(name)
        except AttributeError:
            missing.append(name)
    assert not missing, missing


def test_every_config_field_is_documented():
    text = _text(DOCS[0])
    for cls in (fm.ParallelConfig, fm.QuantConfig, fm.OffloadConfig, fm.TrainConfig, fm.GPTConfig):
        for f in dataclasses.fields(cls):
            assert f"| `{f.name}` |" in text, f"{cls.__name__}.{f.name} is not in docs/documentation.md"


def test_documented_cli_tools_exist():
    from forgeminds_b200.cli import __main__ as cli
    for path in DOCS:
        for tool in re.findall(r"(?:python|torchrun[^`\n]*) -m forgeminds_b200\.cli (\w+)", _text(path)):
            assert tool in cli.TOOLS, (path, tool)


def test_profiles_and_guides_name_existing_files():
    """Paths written as `dir/file.ext` in the guides and profile summaries exist in the tree."""
    docs = DOCS + [os.path.join(ROOT, "profiles", f) for f in sorted(os.listdir(os.path.join(ROOT, "profiles")))]
    missing = []
    for path in docs:
        for ref in re.findall(r"`((?:forgeminds_b200|tests|profiles|docs|examples)/[A-Za-z0-9_./-]+\.(?:py|md|cu|cuh|cpp|h))`", _text(path)):
            if not os.path.exists(os.path.join(ROOT, ref)):
                missing.append((os.path.basename(path), ref))
    assert not missing, missing


def test_kernel_names_in_the_kernel_guide_exist_in_the_sources():
    """docs/kernels.md describes the device code kernel by kernel: every ``*_kernel`` it names is in csrc/."""
    import pathlib
    import re
    root = pathlib.Path(__file__).resolve().parent.parent
    text = (root / "docs" / "kernels.md").read_text()
    named = set(re.findall(r"`([a-z0-9_]+_kernel)\b", text))
    assert len(named) >= 15, named
    sources = "\n".join(p.read_text() for p in (root / "forgeminds_b200" / "csrc").glob("*.cu"))
    missing = sorted(n for n in named if n not in sources)
    assert not missing, missing
