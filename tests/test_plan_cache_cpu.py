"""The plan and weight cache on disk: a graph that was compiled before is neither imported nor lowered again, and a set
of weights that was written before is not written again -- by the same process or by another one.  (The reference names
its artefact after a hash of the module text, src/Compiler/Compiler.cpp:305-309, but rebuilds it and re-dumps every
weight on each compile.)  Plans run on the CPU interpreter here; the GPU side of the cache (the uploaded weight pool) is
covered in tests/test_models_gpu.py."""
import copy
import os
import subprocess
import sys

import pytest
import torch

from helpers import InterpreterCompiler, compile_with
from llcompiler_b200.importer import Importer
from oracle.models import build_model

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _files(root):
    return {os.path.join(d, f): os.stat(os.path.join(d, f)).st_mtime_ns for d, _, fs in os.walk(root) for f in fs}


def test_second_compile_imports_nothing_and_writes_nothing(tmp_path, monkeypatch):
    monkeypatch.setenv("LLC_CACHE_DIR", str(tmp_path))
    model = build_model("mlp")
    x = torch.randn(8, 784, generator=torch.Generator().manual_seed(2))
    first = InterpreterCompiler()
    with torch.no_grad():
        want = compile_with(first, copy.deepcopy(model))(x)
    assert first.cache_hits == 0
    before = _files(tmp_path)
    assert any(p.endswith("plan.llcplan") for p in before) and any(p.endswith(".npy") for p in before)

    def no_import(*a, **k):
        raise AssertionError("the importer ran although the graph is in the cache")
    monkeypatch.setattr(Importer, "importer", no_import)
    monkeypatch.setattr(InterpreterCompiler, "_compile_text", no_import)
    second = InterpreterCompiler()
    with torch.no_grad():
        got = compile_with(second, copy.deepcopy(model))(x)
    assert second.cache_hits == 1 and torch.equal(got, want)
    assert _files(tmp_path) == before                      # nothing new, nothing rewritten


def test_other_weights_get_a_directory_of_their_own(tmp_path, monkeypatch):
    monkeypatch.setenv("LLC_CACHE_DIR", str(tmp_path))
    model = build_model("mlp")
    x = torch.randn(4, 784)
    a = InterpreterCompiler()
    with torch.no_grad():
        ya = compile_with(a, copy.deepcopy(model))(x)
    other = copy.deepcopy(model)
    with torch.no_grad():
        other.fc2.bias.add_(1.0)
    b = InterpreterCompiler()
    with torch.no_grad():
        yb = compile_with(b, other)(x)
    assert b.cache_hits == 1                               # same graph ...
    assert a.compiled[0].weight_dir != b.compiled[0].weight_dir   # ... other values
    assert torch.allclose(yb, ya + 1.0, atol=1e-5)


def test_cache_is_shared_between_processes_and_can_be_switched_off(tmp_path, monkeypatch):
    script = (
        "import sys, copy, torch\n"
        f"sys.path.insert(0, {ROOT!r}); sys.path.insert(0, {os.path.join(ROOT, 'tests')!r})\n"
        "from helpers import InterpreterCompiler, compile_with\n"
        "from oracle.models import build_model\n"
        "c = InterpreterCompiler()\n"
        "with torch.no_grad():\n"
        "    y = compile_with(c, build_model('mlp'))(torch.ones(2, 784))\n"
        "print('hits', c.cache_hits, float(y.sum()))\n")
    env = dict(os.environ, LLC_CACHE_DIR=str(tmp_path))
    outs = [subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=300) for _ in range(2)]
    assert all(o.returncode == 0 for o in outs), outs[-1].stderr[-2000:]
    assert "hits 0" in outs[0].stdout and "hits 1" in outs[1].stdout
    assert outs[0].stdout.split()[-1] == outs[1].stdout.split()[-1]
    off = subprocess.run([sys.executable, "-c", script], env=dict(env, LLC_CACHE_DIR="off"), capture_output=True, text=True, timeout=300)
    assert off.returncode == 0 and "hits 0" in off.stdout


def _publish_worker(args):
    entry, n_files, size = args
    import numpy as np
    from llcompiler_b200.compiler.compiler import publish_weight_set

    def write_set(directory):
        for i in range(n_files):
            np.save(os.path.join(directory, f"w{i}.npy"), np.full(size, i, dtype=np.float32))

    d = publish_weight_set(entry, "v_test", write_set)
    # whatever directory came back must be complete the moment it is returned: every file whole and right
    for i in range(n_files):
        a = np.load(os.path.join(d, f"w{i}.npy"))
        if a.shape != (size,) or not (a == i).all():
            return False
    return os.path.exists(os.path.join(d, ".complete"))


def test_weight_set_is_published_once_by_racing_processes(tmp_path):
    """The ranks of a multi-GPU job compile the same graph at the same time: none of them may read a weight file that
    another one is still writing."""
    import multiprocessing as mp
    entry = str(tmp_path / "g_race")
    os.makedirs(entry)
    with mp.get_context("spawn").Pool(6) as pool:
        ok = pool.map(_publish_worker, [(entry, 12, 200_000)] * 6)
    assert all(ok)
    left = sorted(os.listdir(entry))
    assert left == ["v_test"], left                      # the losers of the race removed their copies


def test_weight_set_beside_an_unfinished_directory(tmp_path):
    from llcompiler_b200.compiler.compiler import publish_weight_set
    entry = str(tmp_path / "g_old")
    os.makedirs(os.path.join(entry, "v_x"))              # a directory without its marker: a writer that died
    open(os.path.join(entry, "v_x", "stale.npy"), "w").close()
    d = publish_weight_set(entry, "v_x", lambda directory: open(os.path.join(directory, "w.npy"), "w").close())
    assert d != os.path.join(entry, "v_x") and os.path.exists(os.path.join(d, "w.npy")) and os.path.exists(os.path.join(d, ".complete"))
