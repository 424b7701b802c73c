"""The import lines of every Python example in README.md and docs/*.md resolve, and the README quick start runs."""
import glob
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FILES = [os.path.join(ROOT, "README.md")] + sorted(glob.glob(os.path.join(ROOT, "docs", "*.md")))


def python_blocks(path):
    text = open(path).read()
    return re.findall(r"```python\n(.*?)```", text, flags=re.S)


@pytest.mark.parametrize("path", FILES, ids=[os.path.basename(f) for f in FILES])
def test_import_lines_of_examples_resolve(path):
    lines = []
    for block in python_blocks(path):
        for line in block.splitlines():
            s = line.strip()
            if s.startswith(("from flodl_b200", "import flodl_b200")):
                lines.append(s.split("#")[0].strip())
    for s in lines:
        exec(s, {})                                   # raises ImportError / AttributeError on a stale name


def test_readme_quick_start_runs():
    blocks = python_blocks(os.path.join(ROOT, "README.md"))
    quick = [b for b in blocks if "FlowBuilder.from_" in b and "opt.step()" in b]
    assert quick, "quick-start block not found"
    env = {}
    exec(quick[0].replace("range(200)", "range(20)"), env)
    assert float(env["loss"].t.detach()) == float(env["loss"].t.detach())      # finite, and the names of the example exist


# ---- tutorials: every Python block is executed, in order, in one namespace per file ------------------------------------
TUTORIALS = sorted(f for f in glob.glob(os.path.join(ROOT, "docs", "tutorials", "*.md")) if os.path.basename(f) != "README.md")
SKIP_MARK = "# (not run by the docs test"


@pytest.mark.parametrize("path", TUTORIALS, ids=[os.path.basename(f) for f in TUTORIALS])
def test_tutorial_code_runs(path, tmp_path, monkeypatch):
    """Blocks whose first line starts with `# (not run by the docs test` (they need GPUs, several processes or the
    network) only have their import lines checked."""
    monkeypatch.chdir(tmp_path)
    env = {"__name__": "__tutorial__"}
    ran = 0
    for block in python_blocks(path):
        if block.lstrip().startswith(SKIP_MARK):
            for line in block.splitlines():
                s = line.strip()
                if s.startswith(("from flodl_b200", "import flodl_b200")):
                    exec(s.split("#")[0].strip(), {})
            continue
        exec(compile(block, f"{os.path.basename(path)}:block{ran}", "exec"), env)
        ran += 1
    assert ran > 0, "a tutorial without a runnable block"


def test_tutorial_index_lists_every_file():
    index = open(os.path.join(ROOT, "docs", "tutorials", "README.md")).read() if TUTORIALS else ""
    for path in TUTORIALS:
        name = os.path.basename(path)
        assert name in index, f"{name} is not linked from docs/tutorials/README.md"
