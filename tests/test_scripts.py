"""Launch scripts: every ``--flag`` they pass exists in the command-line parser of the program they start, the
programs exist, and the scripts are valid shell."""
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = sorted(f for f in os.listdir(os.path.join(ROOT, "scripts")) if f.endswith(".sh"))
LAUNCHER_FLAGS = {"--nnodes", "--nproc-per-node", "--master-addr", "--master-port", "--max-restarts",     # torchrun
                  "--gres", "--ntasks-per-node", "--cpus-per-task"}                                    # srun


_HELP = {}


def _help_text(target):
    if target in _HELP:
        return _HELP[target]
    cmd = [sys.executable] + (["-m", target] if not target.endswith(".py") else [os.path.join(ROOT, target)]) + ["--help"]
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    _HELP[target] = out.stdout
    return out.stdout


@pytest.mark.parametrize("name", SCRIPTS)
def test_script_flags_exist_in_the_program_it_starts(name):
    path = os.path.join(ROOT, "scripts", name)
    assert subprocess.run(["bash", "-n", path]).returncode == 0
    text = "\n".join(l for l in open(path).read().splitlines() if not l.lstrip().startswith("#"))
    targets = set(re.findall(r"-m (easyllm_b200[\w.]+)", text)) | set(re.findall(r"\$ROOT/(tools/\w+\.py)", text))
    assert targets, f"{name} starts no program of this repository"
    flags = set(re.findall(r"(?<![\w-])(--[a-zA-Z][\w-]*)", text)) - LAUNCHER_FLAGS
    for target in targets:
        help_text = _help_text(target)
        known = set(re.findall(r"(--[a-zA-Z][\w-]*)", help_text))
        missing = {f for f in flags if f not in known and f.replace("_", "-") not in known and f.replace("-", "_") not in known}
        assert not missing, f"{name} passes {sorted(missing)} which {target} does not accept"
