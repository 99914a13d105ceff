"""bin/trace_run as a user runs it: a subprocess fed one JSON step a line, logits read back from files."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import harness
from tests.tiny_configs import TINY_B, TINY_C

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def replay(folder, out, dtype, max_tokens, schedule, vocab, extra=(), split=None):
    """Feed ``schedule`` to the program; {(id, position): logits row}.  With ``split`` a pair of such dicts: the rows
    of the steps before that index and of the steps from it on (an id may live twice)."""
    process = subprocess.Popen([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                                "--out", str(out), "--max-tokens", str(max_tokens), *extra],
                               stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    rows, position = {}, {}
    before = None
    for number, (entries, ended) in enumerate(schedule):
        if split is not None and number == split:
            before, rows = rows, {}
        step = dict(step=number, entries=[dict(id=rid, tokens=tokens, want=want) for rid, tokens, want in entries],
                    end=ended)
        process.stdin.write(json.dumps(step) + "\n")
        process.stdin.flush()
        assert process.stdout.readline().strip() == f"done {number}"
        wanted = [(rid, position.get(rid, 0) + w) for rid, tokens, want in entries for w in want]
        path = out / f"{number}.f32"
        if wanted:
            data = np.fromfile(path, dtype="<f4").reshape(len(wanted), vocab)
            for key, row in zip(wanted, data):
                rows[key] = torch.from_numpy(row.copy())
        else:
            assert not path.exists()
        for rid, tokens, _ in entries:
            position[rid] = position.get(rid, 0) + len(tokens)
        for rid in ended:
            position.pop(rid, None)
    process.stdin.close()
    assert process.wait(timeout=60) == 0
    return rows if split is None else (before, rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_mixed_requests_with_reused_pages(tmp_path, dtype):
    cfg = TINY_B
    weights = harness.write_folder(cfg, 1, tmp_path / "model")
    requests = {f"r{i}": harness.random_tokens(cfg, n, 30 + i) for i, n in enumerate((100, 9, 64, 31, 150, 70, 45, 120, 18))}
    schedule = harness.mixed_schedule(requests)
    # only some places are wanted in some steps: every third position, and always a request's last
    thinned = []
    seen = {}
    for entries, ended in schedule:
        new_entries = []
        for rid, tokens, want in entries:
            base = seen.get(rid, 0)
            keep = [w for w in want if (base + w) % 3 == 0 or base + w == len(requests[rid]) - 1]
            new_entries.append((rid, tokens, keep))
            seen[rid] = base + len(tokens)
        thinned.append((new_entries, ended))
    # --max-tokens as its help defines it: the most that live requests hold at any time, each rounded up to 64
    page_size = 16
    max_tokens = harness.peak_pages(thinned, page_size, round_to=64) * page_size
    handovers, peak_held = harness.simulate_pages(thinned, max_tokens // page_size, page_size)
    assert handovers > 10 and peak_held > 0.75 * max_tokens // page_size, "this trace should make the program reuse pages"
    rows = replay(tmp_path / "model", tmp_path / "out", dtype, max_tokens, thinned, cfg["vocab_size"])
    torch_dtype = dict(float32=torch.float32, bfloat16=torch.bfloat16)[dtype]
    expected_all = harness.plain_rows(requests, weights, cfg, torch.float32)
    expected = {k: v for k, v in expected_all.items() if k in rows}
    assert len(rows) > 120 and all((rid, len(t) - 1) in rows for rid, t in requests.items())
    yardstick = None
    if torch_dtype == torch.bfloat16:
        full = harness.plain_rows(requests, weights, cfg, torch.bfloat16)
        yardstick = {k: full[k] for k in rows}
    harness.assert_rows_close(rows, expected, torch_dtype, f"trace_run {dtype}", yardstick)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_an_ended_id_comes_back_in_another_row(tmp_path, dtype):
    """``"end": ["a"]`` and then ``"id": "a"`` again while "b" is live: the second "a" sits in another block-table
    row, and its single-token steps must run with that row."""
    cfg = TINY_C
    weights = harness.write_folder(cfg, 2, tmp_path / "model")
    first, second, other = (harness.random_tokens(cfg, n, 40 + i) for i, n in enumerate((12, 20, 40)))
    schedule = [([("a", first[:8], [7]), ("b", other[:5], [4])], [])]
    schedule += [([("a", [first[i]], [0]), ("b", [other[i - 3]], [0])], ["a"] if i == 11 else []) for i in range(8, 12)]
    split = len(schedule)
    schedule += [([("b", other[9:20], [10]), ("a", second[:6], [5])], [])]
    schedule += [([("a", [second[i]], [0]), ("b", [other[i + 14]], [0])], []) for i in range(6, 20)]
    schedule += [([("b", other[34:], [5])], ["a", "b"])]
    torch_dtype = dict(float32=torch.float32, bfloat16=torch.bfloat16)[dtype]
    names = {"a1": first, "a2": second, "b": other}
    plain_all = harness.plain_rows(names, weights, cfg, torch.float32)
    plain_low = harness.plain_rows(names, weights, cfg, torch_dtype) if dtype == "bfloat16" else None
    rows = replay(tmp_path / "model", tmp_path / "out", dtype, 192, schedule, cfg["vocab_size"], split=split)
    for life, part in (("a1", rows[0]), ("a2", rows[1])):
        rename = lambda key: (life, key[1]) if key[0] == "a" else key
        expected = {key: plain_all[rename(key)] for key in part}
        yardstick = {key: plain_low[rename(key)] for key in part} if plain_low else None
        harness.assert_rows_close(part, expected, torch_dtype, f"trace_run re-admitted id ({life}) {dtype}", yardstick)
    assert len(rows[0]) == 10 and len(rows[1]) == 31


def test_trace_run_small_pages_and_empty_steps(tmp_path):
    cfg = TINY_C
    weights = harness.write_folder(cfg, 2, tmp_path / "model", storage=torch.float32)   # a folder stored in 32 bits
    tokens = harness.random_tokens(cfg, 67, 1)
    schedule = [([("a", tokens[:2], [])], []), ([("a", tokens[2:40], [37])], []), ([], []),
                ([("a", tokens[40:41], [0]), ("b", tokens[:5], [4])], ["b"]), ([("a", tokens[41:], [0, 25])], ["a"])]
    rows = replay(tmp_path / "model", tmp_path / "out", "float32", 128, schedule, cfg["vocab_size"],
                  extra=("--page-size", "4"))
    expected_all = harness.plain_rows({"a": tokens, "b": tokens[:5]}, weights, cfg)
    assert set(rows) == {("a", 39), ("a", 40), ("b", 4), ("a", 41), ("a", 66)}
    harness.assert_rows_close(rows, {k: expected_all[k] for k in rows}, torch.float32, "trace_run small pages")
