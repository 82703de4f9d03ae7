"""The usage example of README.md runs as written on a B200."""
import os
import re

import pytest

pytestmark = pytest.mark.gpu


def test_readme_example_runs():
    text = open(os.path.join(os.path.dirname(__file__), "..", "README.md")).read()
    blocks = re.findall(r"```python\n(.*?)```", text, flags=re.S)
    assert blocks, "README.md has no python example"
    scope = {}
    exec(compile(blocks[0], "README.md", "exec"), scope)       # sys.path is set up by tests/conftest.py
    import torch
    for name in ("y", "z", "g", "up", "s", "v3", "a", "fused"):
        assert name in scope and scope[name].device.type == "vulkan" and torch.isfinite(scope[name].detach().cpu()).all(), name
    assert scope["x"].grad is not None and scope["fused"].is_contiguous(memory_format=torch.channels_last)
