"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits files read
back and compared with the plain implementation.  The same requests are replayed
whole, with the last 32 tokens one by one, and in batches of unequal lengths that
follow one another on a cache too small for two of them."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import plain_llama, tiny_configs
from tests.test_engine_gpu import REL_TOL, prompts

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def replay(model_dir, dtype, out_dir, max_tokens, steps):
    """Runs trace_run on ``steps`` (list of dicts); checks the ``done`` protocol."""
    proc = subprocess.Popen([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype",
                             dtype, "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for st in steps:
        proc.stdin.write(json.dumps(st) + "\n")
        proc.stdin.flush()
        line = proc.stdout.readline().strip()
        assert line == f"done {st['step']}", line
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0


def read_logits(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(Path(out_dir) / f"{step}.f32", dtype="<f4").reshape(-1, vocab).copy())


def check(got, ref, dtype):
    tol = REL_TOL[torch.float32 if dtype == "float32" else torch.bfloat16]
    err = (got - ref).abs().max().item()
    assert err <= tol * ref.abs().max().item(), err


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16"),
                                        ("E", "bfloat16")])
def test_trace_replay_modes(tmp_path, name, dtype):
    folder = tiny_configs.make_folder(tmp_path, name, seed=31)
    raw, w = tiny_configs.read_folder(folder)
    vocab = raw["vocab_size"]
    reqs = prompts(vocab, [40, 33, 75, 50, 36], seed=2)
    refs = [plain_llama.forward(w, raw, r) for r in reqs]

    # 1. each request alone and whole
    steps = [{"step": i, "entries": [{"id": f"r{i}", "tokens": r, "want": list(range(len(r)))}], "end": [f"r{i}"]}
             for i, r in enumerate(reqs)]
    out = tmp_path / "whole"
    replay(folder, dtype, out, 128, steps)
    for i, ref in enumerate(refs):
        check(read_logits(out, i, vocab), ref, dtype)

    # 2. the last 32 tokens one by one
    steps, n = [], 0
    where = []
    for i, r in enumerate(reqs):
        head = len(r) - 32
        first = n
        steps.append({"step": n, "entries": [{"id": f"r{i}", "tokens": r[:head], "want": list(range(head))}], "end": []})
        n += 1
        for j, t in enumerate(r[head:]):
            steps.append({"step": n, "entries": [{"id": f"r{i}", "tokens": [t], "want": [0]}],
                          "end": [f"r{i}"] if j == 31 else []})
            n += 1
        where.append((first, n))
    out = tmp_path / "cut"
    replay(folder, dtype, out, 128, steps)
    for (a, b), ref in zip(where, refs):
        check(torch.cat([read_logits(out, s, vocab) for s in range(a, b)]), ref, dtype)

    # 3. batches of unequal lengths, one after another; a step without wants writes no file
    steps, n = [], 0
    pieces = {i: [] for i in range(len(reqs))}
    for batch in ([0, 1, 2], [3, 4]):
        decode = {i: 4 + 3 * k for k, i in enumerate(batch)}
        heads = {i: len(reqs[i]) - decode[i] for i in batch}
        steps.append({"step": n, "entries": [{"id": f"r{i}", "tokens": reqs[i][:heads[i]], "want": list(range(heads[i]))}
                                            for i in batch], "end": []})
        for i in batch:
            pieces[i].append((n, heads[i]))
        n += 1
        k = 0
        live = list(batch)
        while live:
            ent = [{"id": f"r{i}", "tokens": [reqs[i][heads[i] + k]], "want": [0]} for i in live]
            done = [i for i in live if k + 1 == decode[i]]
            steps.append({"step": n, "entries": ent, "end": [f"r{i}" for i in done]})
            for i in live:
                pieces[i].append((n, 1))
            n += 1
            k += 1
            live = [i for i in live if i not in done]
    steps.append({"step": n, "entries": [{"id": "x", "tokens": reqs[0][:3], "want": []}], "end": ["x"]})
    out = tmp_path / "batches"
    # the three requests of the first batch hold 64 + 64 + 128 tokens
    replay(folder, dtype, out, 256, steps)
    assert not (out / f"{n}.f32").exists()
    files = {}
    for i, ref in enumerate(refs):
        rows = []
        for step, cnt in pieces[i]:
            if step not in files:
                files[step] = [read_logits(out, step, vocab), 0]
            t, o = files[step]
            rows.append(t[o:o + cnt])
            files[step][1] = o + cnt
        check(torch.cat(rows), ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_goes_beyond_the_configurations_trained_length(tmp_path, dtype):
    """A request longer than ``max_position_embeddings`` (128 in configuration A): nothing in the
    replay depends on that length, and the plain implementation has no such limit either."""
    folder = tiny_configs.make_folder(tmp_path, "A", seed=5)
    raw, w = tiny_configs.read_folder(folder)
    vocab = raw["vocab_size"]
    assert raw["max_position_embeddings"] == 128
    (req,) = prompts(vocab, [200], seed=9)
    ref = plain_llama.forward(w, raw, req)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": req[:170], "want": list(range(170))}], "end": []}]
    steps += [{"step": 1 + j, "entries": [{"id": "a", "tokens": [t], "want": [0]}], "end": ["a"] if j == 29 else []}
              for j, t in enumerate(req[170:])]
    out = tmp_path / "long"
    replay(folder, dtype, out, 256, steps)
    check(torch.cat([read_logits(out, s, vocab) for s in range(31)]), ref, dtype)
