"""Every launch script under examples/ must be valid shell and carry a flag set that the argument parser, the config
builder and the validators accept for the world size the script asks for."""
import glob
import os
import re
import shlex
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = sorted(glob.glob(os.path.join(ROOT, "examples", "**", "*.sh"), recursive=True))


def _train_args(text: str):
    """The arguments after ``-m loongforge_b200.train`` with shell variables replaced by plain values."""
    m = re.search(r"-m loongforge_b200\.train\s*\\?\n(.*)", text, re.S)
    if not m:
        return None
    body = m.group(1).replace("\\\n", " ")
    body = body.split("\n")[0] if "\n" in body.strip() and not body.strip().startswith("--") else body
    body = re.sub(r'"\$\{DATA_ARGS\[@\]\}"', "--mock-data", body)
    defaults = dict(re.findall(r"^([A-Z_]+)=\$\{\1:-([^}$]*)\}", text, re.M))  # VAR=${VAR:-default} lines
    defaults["GPUS"] = "8"
    body = re.sub(r'"?\$\{?([A-Z_]+)(:-[^}]*)?\}?"?', lambda m: defaults.get(m.group(1)) or "/tmp/x", body)
    return [a for a in shlex.split(body.strip().splitlines()[0] if "\n" in body else body) if a]


@pytest.mark.parametrize("path", SCRIPTS, ids=[os.path.relpath(p, ROOT) for p in SCRIPTS])
def test_example_script(path, monkeypatch):
    assert subprocess.run(["bash", "-n", path]).returncode == 0
    args = _train_args(open(path).read())
    if args is None:
        return  # tools / other entry points
    from loongforge_b200.config.arguments import parse_args
    from loongforge_b200.config.build import build_configs

    monkeypatch.setenv("WORLD_SIZE", "8")
    a, ov = parse_args(args)
    cfg, tc, dims, _ = build_configs(a, ov)
    assert tc.train_iters > 0 and 8 % (dims.tp * dims.pp * dims.cp) == 0
