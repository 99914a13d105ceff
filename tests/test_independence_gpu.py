"""The product path needs no other engine and no compiler of kernels: generation runs with those packages
made un-importable (tests/qil/test_independence.py:6-22 of the reference does the same for its engine)."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests import harness
from tests.tiny_configs import TINY_B

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

BLOCKED = ("triton", "transformers", "vllm", "nano_vllm", "flash_attn", "flashinfer", "cutlass", "tilelang", "xformers")

RUNNER = """
import builtins, json, sys

BLOCKED = {blocked!r}
original = builtins.__import__

def restricted(name, *args, **kwargs):
    if name.split(".")[0] in BLOCKED:
        raise ImportError("import of " + name + " is blocked in this test")
    return original(name, *args, **kwargs)

builtins.__import__ = restricted
for name in BLOCKED:
    try:
        __import__(name)
    except ImportError:
        continue
    raise SystemExit(name + " could still be imported")
from qwen_inference_lab_b200.__main__ import main
code = main({argv!r})
loaded = sorted(name for name in sys.modules if name.split(".")[0] in BLOCKED)
print("LOADED", json.dumps(loaded))
sys.exit(code)
"""


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_with_other_engines_and_kernel_compilers_blocked(tmp_path, dtype):
    folder = tmp_path / "model"
    weights = harness.write_folder(TINY_B, 1, folder)
    prompt = harness.random_tokens(TINY_B, 40, 3)
    output = tmp_path / "result.json"
    argv = ["--model", str(folder), "--token-ids", json.dumps(prompt), "--dtype", dtype, "--max-new-tokens", "6",
            "--pages", "16", "--page-size", "8", "--chunk-size", "16", "--ignore-eos", "--output", str(output)]
    done = subprocess.run([sys.executable, "-c", RUNNER.format(blocked=BLOCKED, argv=argv)], capture_output=True,
                          text=True, cwd=str(ROOT))
    assert done.returncode == 0, done.stderr[-2000:]
    assert done.stdout.strip().splitlines()[-1] == "LOADED []"
    result = json.loads(output.read_text())
    assert result["state"] == "completed" and len(result["token_ids"]) == 6
    harness.check_greedy(prompt, result["token_ids"], weights, TINY_B,
                         dict(float32=torch.float32, bfloat16=torch.bfloat16)[dtype])

