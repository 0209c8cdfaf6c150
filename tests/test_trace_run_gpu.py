"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits read
back from <out>/<step>.f32."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import TINY, TOL, first_wrong, make_folder, plain_logits, random_ids, trace_mixed, trace_tail_decoded

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _run(folder, dtype, steps, out, max_tokens, env=None):
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(max_tokens)],
        input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True, timeout=600,
        env=None if env is None else {**os.environ, **env})
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    return proc


def _collect(steps, out, vocab):
    got, pos = {}, {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        f = Path(out) / f"{s['step']}.f32"
        if n_want == 0:
            assert not f.exists()
            for e in s["entries"]:
                pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
            continue
        arr = np.fromfile(f, dtype="<f4").reshape(n_want, vocab)
        row = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got.setdefault(e["id"], {})[base + w] = arr[row]
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
    return got


@pytest.mark.parametrize("dtype,name", [("float32", "A"), ("bfloat16", "B")])
def test_trace_run_mixed_and_sparse_wants(tmp_path, dtype, name):
    stored = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    folder = make_folder(tmp_path, name, stored=stored)
    vocab = TINY[name][0]["vocab_size"]
    reqs = {f"q{i}": random_ids(40 + i, n, vocab) for i, n in enumerate([70, 45, 130, 64, 20, 99])}
    steps = trace_mixed(reqs, capacity_tokens=384, max_live=4, seed=9)
    # ask for only some places: every third wanted place is dropped, some steps want nothing
    for k, s in enumerate(steps):
        for e in s["entries"]:
            e["want"] = [] if k % 5 == 4 else [w for w in e["want"] if (w + k) % 3]
    out = tmp_path / "out"
    _run(folder, dtype, steps, out, max_tokens=384)
    got = _collect(steps, out, vocab)
    for rid, ids in reqs.items():
        want = plain_logits(folder, ids)
        rows = sorted(got[rid])
        bad = first_wrong(np.stack([got[rid][p] for p in rows]), want[rows], TOL[dtype])
        assert bad is None, f"{rid}: first wrong wanted place {rows[bad[0]]} (rel err {bad[1]:.3g})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_without_programmatic_dependent_launch(tmp_path, dtype):
    """The kernels read what they can before their dependency wait (metadata, weights, cache and state
    of earlier steps) so that a step's kernels overlap; with GIBBS_B200_PDL=0 every kernel starts
    after the one in front has ended.  Both ways must give the plain implementation's logits: a
    difference between them would be a read that was moved in front of the wait by mistake."""
    stored = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    folder = make_folder(tmp_path, "C", stored=stored)
    vocab = TINY["C"][0]["vocab_size"]
    reqs = {f"q{i}": random_ids(60 + i, n, vocab) for i, n in enumerate([90, 33, 150, 64])}
    steps = trace_mixed(reqs, capacity_tokens=320, max_live=4, seed=4)
    want = {rid: plain_logits(folder, ids) for rid, ids in reqs.items()}
    results = {}
    for mode, env in (("serial", {"GIBBS_B200_PDL": "0"}), ("overlapped", {"GIBBS_B200_PDL": "1"})):
        out = tmp_path / f"out_{mode}"
        _run(folder, dtype, steps, out, max_tokens=320, env=env)
        got = results[mode] = _collect(steps, out, vocab)
        for rid in reqs:
            rows = sorted(got[rid])
            bad = first_wrong(np.stack([got[rid][p] for p in rows]), want[rid][rows], TOL[dtype])
            assert bad is None, f"{mode}, {rid}: first wrong place {rows[bad[0]]} (rel err {bad[1]:.3g})"
    # the same kernels add in the same order either way: the two runs agree to the bit
    for rid in reqs:
        for p in sorted(results["serial"][rid]):
            assert np.array_equal(results["serial"][rid][p], results["overlapped"][rid][p]), (rid, p)


def test_trace_run_fresh_env(tmp_path):
    """Runs with an empty HOME and no inherited python path."""
    folder = make_folder(tmp_path, "A")
    vocab = TINY["A"][0]["vocab_size"]
    reqs = {"only": random_ids(7, 50, vocab)}
    steps = trace_tail_decoded(reqs, tail=8)
    home = tmp_path / "home"
    home.mkdir()
    env = {k: v for k, v in os.environ.items() if k not in ("PYTHONPATH",)}
    env["HOME"] = str(home)
    proc = subprocess.run(
        [str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "o"),
         "--max-tokens", "64"],
        input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True, timeout=600, env=env,
        cwd=str(tmp_path))
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = _collect(steps, tmp_path / "o", vocab)
    want = plain_logits(folder, reqs["only"])
    assert first_wrong(np.stack([got["only"][p] for p in sorted(got["only"])]), want, TOL["float32"]) is None


def test_trace_run_potivik_with_and_without_dependent_launch(tmp_path):
    """The Potivik design through the same runner: a model folder on disk (bfloat16 weights), float32
    compute, mixed steps with sparse wants in a pool that makes pages and slots go round; the runs with
    and without programmatic dependent launch agree with the plain implementation and with each other
    to the bit."""
    import plain_potivik
    from potivik_helpers import CFG_A, make_weights, rel_rows, write_model
    W = make_weights(CFG_A, 21)
    folder = write_model(tmp_path / "potivik_a", CFG_A, W)
    vocab = CFG_A["vocab"]
    reqs = {f"q{i}": random_ids(80 + i, n, vocab) for i, n in enumerate([70, 45, 130, 1, 64, 20])}
    steps = trace_mixed(reqs, capacity_tokens=320, max_live=4, seed=5)
    for k, s in enumerate(steps):
        for e in s["entries"]:
            e["want"] = [] if k % 5 == 4 else [w for w in e["want"] if (w + k) % 3]
    want = {rid: plain_potivik.forward(CFG_A, W, ids).numpy() for rid, ids in reqs.items()}
    results = {}
    for mode, env in (("serial", {"GIBBS_B200_PDL": "0"}), ("overlapped", {"GIBBS_B200_PDL": "1"})):
        out = tmp_path / f"out_{mode}"
        _run(folder, "float32", steps, out, max_tokens=320, env=env)
        got = results[mode] = _collect(steps, out, vocab)
        for rid in reqs:
            rows = sorted(got.get(rid, {}))
            if rows:
                e = rel_rows(np.stack([got[rid][p] for p in rows]), want[rid][rows])
                assert e.max() <= 2e-4, f"{mode}, {rid}: place {rows[int(e.argmax())]} differs by {e.max():.3g}"
    for rid in results["serial"]:
        for p in results["serial"][rid]:
            assert np.array_equal(results["serial"][rid][p], results["overlapped"][rid][p]), (rid, p)


def test_trace_run_petelix_with_and_without_dependent_launch(tmp_path):
    """The Petelix design through the same runner: a model folder on disk (bfloat16 weights), float32
    compute, mixed steps with sparse wants in a pool that makes pages go round (two groups of pages:
    one windowed, one that keeps everything); the runs with and without programmatic dependent launch
    agree with the plain implementation and with each other to the bit."""
    import plain_petelix
    from petelix_helpers import CFG_A, make_weights
    from potivik_helpers import rel_rows, write_model
    W = make_weights(CFG_A, 31)
    folder = write_model(tmp_path / "petelix_a", CFG_A, W)
    vocab = CFG_A["vocab"]
    reqs = {f"q{i}": random_ids(60 + i, n, vocab) for i, n in enumerate([70, 45, 130, 1, 64, 20])}
    steps = trace_mixed(reqs, capacity_tokens=320, max_live=4, seed=6)
    for k, s in enumerate(steps):
        for e in s["entries"]:
            e["want"] = [] if k % 5 == 4 else [w for w in e["want"] if (w + k) % 3]
    want = {rid: plain_petelix.forward(CFG_A, W, ids).numpy() for rid, ids in reqs.items()}
    results = {}
    for mode, env in (("serial", {"GIBBS_B200_PDL": "0"}), ("overlapped", {"GIBBS_B200_PDL": "1"})):
        out = tmp_path / f"out_{mode}"
        _run(folder, "float32", steps, out, max_tokens=320, env=env)
        got = results[mode] = _collect(steps, out, vocab)
        for rid in reqs:
            rows = sorted(got.get(rid, {}))
            if rows:
                e = rel_rows(np.stack([got[rid][p] for p in rows]), want[rid][rows])
                assert e.max() <= 2e-4, f"{mode}, {rid}: place {rows[int(e.argmax())]} differs by {e.max():.3g}"
    for rid in results["serial"]:
        for p in results["serial"][rid]:
            assert np.array_equal(results["serial"][rid][p], results["overlapped"][rid][p]), (rid, p)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_sisadra_from_a_folder_without_rank_keys(tmp_path, dtype):
    """The Sisadra design through the same runner: a model folder on disk whose config.json does not name the
    ranks of the low-rank projections (the checkpoint's shapes give them), mixed steps with sparse wants in a
    pool that makes pages and the four state slots go round (two groups of pages kept by blocks, one that
    keeps everything)."""
    import copy
    import plain_sisadra
    from potivik_helpers import rel_rows, write_model
    from sisadra_helpers import CFG_A, make_weights
    W = make_weights(CFG_A, 31)
    cfg = copy.deepcopy(CFG_A)
    for layer in cfg["layers"]:
        layer["mixer"].pop("decay_rank", None), layer["mixer"].pop("gate_rank", None)
    folder = write_model(tmp_path / "sisadra_a", cfg, W)
    vocab = cfg["vocab"]
    reqs = {f"q{i}": random_ids(60 + i, n, vocab) for i, n in enumerate([70, 45, 130, 1, 64, 20, 33])}
    steps = trace_mixed(reqs, capacity_tokens=320, max_live=4, seed=6)
    for k, s in enumerate(steps):
        for e in s["entries"]:
            e["want"] = [] if k % 5 == 4 else [w for w in e["want"] if (w + k) % 3]
    want = {rid: plain_sisadra.forward(CFG_A, W, ids).numpy() for rid, ids in reqs.items()}
    out = tmp_path / "out"
    _run(folder, dtype, steps, out, max_tokens=320)
    got = _collect(steps, out, vocab)
    for rid in reqs:
        rows = sorted(got.get(rid, {}))
        if rows:
            e = rel_rows(np.stack([got[rid][p] for p in rows]), want[rid][rows])
            assert e.max() <= (2e-4 if dtype == "float32" else 4e-2), f"{rid}: place {rows[int(e.argmax())]} differs by {e.max():.3g}"


def test_trace_run_selivik(tmp_path):
    """The Selivik design through the same runner: a model folder on disk (bfloat16 weights), both compute
    dtypes, mixed steps with sparse wants in a pool that makes pages go round (windows with kept first
    positions among them)."""
    import plain_selivik
    from potivik_helpers import rel_rows, write_model
    from selivik_helpers import CFG_D, make_weights
    W = make_weights(CFG_D, 23)
    folder = write_model(tmp_path / "selivik_d", CFG_D, W)
    vocab = CFG_D["vocab"]
    reqs = {f"q{i}": random_ids(90 + i, n, vocab) for i, n in enumerate([70, 45, 130, 1, 64, 20])}
    steps = trace_mixed(reqs, capacity_tokens=320, max_live=4, seed=6)
    for k, s in enumerate(steps):
        for e in s["entries"]:
            e["want"] = [] if k % 5 == 4 else [w for w in e["want"] if (w + k) % 3]
    want = {rid: plain_selivik.forward(CFG_D, W, ids).numpy() for rid, ids in reqs.items()}
    for dtype, tol in (("float32", 2e-4), ("bfloat16", 4e-2)):
        out = tmp_path / f"out_{dtype}"
        _run(folder, dtype, steps, out, max_tokens=320)
        got = _collect(steps, out, vocab)
        errs = []
        for rid in reqs:
            rows = sorted(got.get(rid, {}))
            if rows:
                errs.append(rel_rows(np.stack([got[rid][p] for p in rows]), want[rid][rows]))
        errs = np.concatenate(errs)
        if dtype == "float32":
            assert errs.max() <= tol, f"a place differs by {errs.max():.3g}"
        else:                        # (a router's choice at a near tie may flip under bfloat16 rounding)
            assert np.median(errs) <= tol and (errs <= tol).mean() >= 0.9
