"""The command line's usage errors, exit codes and the commands that need no GPU."""
import json
import os
import subprocess
import sys

from conftest import ROOT, TINY_A

import contextlib
import io
from types import SimpleNamespace

TGE = [sys.executable, os.path.join(ROOT, "bin", "tge")]


def _run(*args):
    """Runs the command line in this process (the entry script only forwards to cli.main)."""
    from aegean_tge_b200.cli import main
    out, err = io.StringIO(), io.StringIO()
    with contextlib.redirect_stdout(out), contextlib.redirect_stderr(err):
        code = main(list(args))
    return SimpleNamespace(returncode=code, stdout=out.getvalue(), stderr=err.getvalue())


def test_entry_script_runs_as_a_program():
    out = subprocess.run(TGE + ["version"], capture_output=True, text=True)
    assert out.returncode == 0 and "aegean-tge b200" in out.stdout
    assert subprocess.run(TGE + ["generate"], capture_output=True, text=True).returncode == 2


def test_version_and_help():
    out = _run("version")
    assert out.returncode == 0 and "aegean-tge b200" in out.stdout
    assert _run().returncode == 0 and "generate" in _run("--help").stdout


def test_usage_errors_exit_with_2():
    assert _run("generate").returncode == 2                                   # neither --model nor --random-config
    assert _run("nonsense").returncode == 2
    out = _run("generate", "--model", "x", "--prompt", "hello")
    assert out.returncode == 2 and "tokenizer" in out.stderr
    assert _run("generate", "--model", "x", "--n", "0").returncode == 2
    assert _run("generate", "--model", "x", "--top-p", "1.5", "--tokens", "1 2").returncode == 2
    assert _run("bench", "sideways").returncode == 2
    assert _run("fidelity", "--model", "x", "--tokens", "1").returncode == 2
    assert _run("bench", "continuous", "--model", "x", "--requests", "0").returncode == 2
    assert _run("bench", "continuous", "--model", "x", "--prompt-tokens", "9", "--prompt-max", "3").returncode == 2
    assert _run("replay", "--model", "x").returncode == 2


def test_make_random_and_plan(tmp_path):
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY_A))
    out = _run("make-random", "--config", str(config), "--out", str(tmp_path / "m"), "--seed", "3")
    assert out.returncode == 0, out.stderr
    assert (tmp_path / "m" / "model.safetensors").exists() and (tmp_path / "m" / "config.json").exists()
    out = _run("plan", "--model", str(tmp_path / "m"), "--context", "256", "--sessions", "2")
    assert out.returncode == 0, out.stderr
    assert "kv       : 256 bytes per token" in out.stdout           # 2 layers x 2 (k, v) x 32 x 2 bytes
    assert "ceiling" in out.stdout


def test_load_failures_exit_with_1(tmp_path):
    out = _run("plan", "--model", str(tmp_path))
    assert out.returncode == 1 and "config.json" in out.stderr
    out = _run("make-random", "--config", str(tmp_path / "missing.json"), "--out", str(tmp_path / "m"))
    assert out.returncode == 1


def test_info_json_needs_no_gpu():
    out = _run("info", "--json")
    assert out.returncode == 0
    facts = json.loads(out.stdout)
    assert facts["kernel_target"] == "sm_100a" and facts["page_size"] == 64
