"""``bin/trace_run`` as a user runs it: a child process fed step by step on standard input
(needs a GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama4 as plain
import traces
from conftest import ROOT, TINY
from test_engine_gpu import MARGIN, TOL

pytestmark = pytest.mark.gpu


def run_trace(model_dir, dtype, steps, out_dir, extra=()):
    cmd = [os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out", str(out_dir),
           "--max-tokens", str(traces.max_tokens(steps)), *extra]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            assert line.strip() == f"done {st['step']}", f"expected 'done {st['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    got, at = {}, {}
    vocab = None
    for st in steps:
        wanted = sum(len(e["want"]) for e in st["entries"])
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
        else:
            data = np.fromfile(path, dtype="<f4")
            assert data.size % wanted == 0
            vocab = data.size // wanted
            rows = torch.from_numpy(data.reshape(wanted, vocab).copy())
        r = 0
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            for wpos in e["want"]:
                got[(e["id"], base + wpos)] = rows[r]
                r += 1
            at[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            at.pop(rid, None)
    return got, vocab


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_trace_through_the_program(model_dirs, tmp_path, dtype):
    name = "A"
    cfg, w = plain.load_folder(model_dirs[name])
    reqs = {f"r{i}": traces.random_tokens(cfg["vocab_size"], n, seed=31 * i + n) for i, n in enumerate([5, 17, 40, 70, 66, 90])}
    steps = traces.mixed(reqs, max_live=4)
    # ask for only some places in some steps, and none in others
    for st in steps:
        for e in st["entries"]:
            if st["step"] % 3 == 1:
                e["want"] = []
            elif st["step"] % 3 == 2:
                e["want"] = [len(e["tokens"]) - 1]
    got, vocab = run_trace(model_dirs[name], dtype, steps, tmp_path, extra=("--trace-routers",) if dtype == "bfloat16" else ())
    assert vocab == cfg["vocab_size"]
    forced = {}
    if dtype == "bfloat16":
        # the program's own expert choices, step by step, for the plain implementation to follow (a near-tie may
        # fall the other way in bfloat16; anything further off fails)
        for st in steps:
            with open(os.path.join(tmp_path, f"{st['step']}.experts.json")) as fh:
                picks = json.load(fh)
            row = 0
            for e in st["entries"]:
                per_layer = forced.setdefault(e["id"], [[] for _ in picks])
                for layer, p in enumerate(picks):
                    per_layer[layer].extend(p[row:row + len(e["tokens"])])
                row += len(e["tokens"])
    ref = {}
    for rid, toks in reqs.items():
        margins = []
        ref[rid] = plain.forward(cfg, w, toks, forced=forced.get(rid), margins=margins)
        assert all(max(layer, default=0.0) < MARGIN for layer in margins), rid
    err, where = traces.worst_error(got, ref)
    print(f"trace_run {dtype}: worst relative error {err:.3e} at {where}")
    assert err < TOL[dtype], (err, where)


def test_whole_equals_decoded_tail_in_the_program(model_dirs, tmp_path):
    name = "B"
    cfg, w = plain.load_folder(model_dirs[name])
    reqs = {"a": traces.random_tokens(cfg["vocab_size"], 100, seed=5)}
    got_whole, _ = run_trace(model_dirs[name], "float32", traces.whole(reqs), tmp_path / "w")
    got_tail, _ = run_trace(model_dirs[name], "float32", traces.tail_decode(reqs), tmp_path / "t", extra=("--page-size", "16"))
    ref = {"a": plain.forward(cfg, w, reqs["a"])}
    assert traces.worst_error(got_whole, ref)[0] < TOL["float32"]
    assert traces.worst_error(got_tail, ref)[0] < TOL["float32"]
    for key in got_whole:
        assert torch.allclose(got_whole[key], got_tail[key], rtol=0, atol=1e-6 * float(got_whole[key].abs().max()))


def test_bad_input_fails_loudly(model_dirs, tmp_path):
    cmd = [os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs["A"], "--dtype", "float32", "--out",
           str(tmp_path), "--max-tokens", "64"]
    bad = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [999999], "want": [0]}], "end": []}) + "\n"
    proc = subprocess.run(cmd, input=bad, capture_output=True, text=True, timeout=300)
    assert proc.returncode != 0 and "vocabulary" in proc.stderr
    too_many = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1] * 200, "want": []}], "end": []}) + "\n"
    proc = subprocess.run(cmd, input=too_many, capture_output=True, text=True, timeout=300)
    assert proc.returncode != 0 and "page" in proc.stderr
