"""``python -m rosellm_b200.cli_generate`` as a child process on the GPU: the ids it prints
against the plain implementation's greedy continuation."""
import ast
import os
import subprocess
import sys

import pytest

import plain_gpt2 as P
from tiny import write_tiny

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROMPT = [5, 17, 3, 250, 9, 44, 101]
NEW = 8


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return write_tiny("A_sharp", str(tmp_path_factory.mktemp("cli")))


def run_cli(*argv) -> str:
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run([sys.executable, "-m", "rosellm_b200.cli_generate", *argv], capture_output=True, text=True,
                         timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-3000:]
    return res.stdout


def printed_ids(stdout: str, stream: bool) -> list[int]:
    if stream:
        line = next(l for l in stdout.splitlines() if l.startswith("[rosellm_b200] streaming output: "))
        return [int(t) for t in line.split(": ", 1)[1].split()]
    line = next(l for l in stdout.splitlines() if l.startswith("[rosellm_b200] output: "))
    return list(ast.literal_eval(line.split(": ", 1)[1]))


@pytest.mark.parametrize("stream", [False, True], ids=["whole", "stream"])
@pytest.mark.parametrize("precision", [["--no-amp"], ["--dtype", "fp32"], []], ids=["no-amp", "fp32", "bf16"])
def test_the_command_line_prints_the_plain_greedy_ids(folder, tmp_path, precision, stream):
    cfg, t = P.load_folder(folder)
    ids_file = tmp_path / "prompt.txt"
    ids_file.write_text(" ".join(map(str, PROMPT)) + "\n")
    how = ["--prompt-ids", ",".join(map(str, PROMPT))] if stream else ["--prompt-ids-file", str(ids_file)]
    out = run_cli("--model", folder, *how, "--max-new-tokens", str(NEW), "--no-stop-on-eos", "--num-pages", "12",
                  "--max-num-batched-tokens", "64", "--max-num-seqs", "2", *precision, *(["--stream"] if stream else []))
    assert f"[rosellm_b200] use_amp: {not precision}" in out
    got = printed_ids(out, stream)
    assert len(got) == NEW
    if precision:  # 32-bit: the very tokens of the plain implementation
        assert got == P.greedy(cfg, t, PROMPT, NEW)
    else:          # bfloat16: each token the plain arg-max given the tokens before it, or within rounding of it
        from test_generate_gpu import check_greedy

        check_greedy(folder, PROMPT, got, "bfloat16")
