"""Every ``# runnable`` block of docs/guide.md is executed: the guide shows calls that exist and behave as it says."""
import pathlib
import re

import pytest

GUIDE = pathlib.Path(__file__).resolve().parent.parent / "docs" / "guide.md"
BLOCKS = [b for b in re.findall(r"```python\n(.*?)```", GUIDE.read_text(), flags=re.S) if b.lstrip().startswith("# runnable")]


def test_the_guide_has_runnable_blocks():
    assert len(BLOCKS) >= 7


@pytest.mark.parametrize("index", range(len(BLOCKS)))
def test_guide_block_runs(index):
    exec(compile(BLOCKS[index], f"guide.md block {index}", "exec"), {"__name__": "__guide__"})
