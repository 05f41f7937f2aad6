"""bench.py's host-side contract that needs no GPU: one JSON line on stdout whatever libraries print
there, and search parameters given on the command line filled up with the defaults."""
import json
import os
import subprocess
import sys
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_stdout_carries_only_the_json_line():
    code = (
        "import os, sys; sys.path.insert(0, %r); import bench\n"
        "bench.claim_stdout()\n"
        "print('a library banner')\n"
        "os.system('echo a child process')\n"
        "bench.emit({'metric': 'm', 'value': 1.5})\n" % ROOT)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, check=True)
    lines = out.stdout.splitlines()
    assert len(lines) == 1
    assert json.loads(lines[0]) == {"metric": "m", "value": 1.5}
    assert "a library banner" in out.stderr and "a child process" in out.stderr


def test_given_search_fills_defaults():
    sys.path.insert(0, ROOT)
    import bench
    sp = bench.given_search(types.SimpleNamespace(search='{"read": 4, "starts": 16}'))
    assert sp["read"] == 4 and sp["starts"] == 16
    assert {"waves", "rerank", "wave_rerank"} <= set(sp)


def test_workloads_name_generators_that_exist():
    sys.path.insert(0, ROOT)
    import bench
    from octex_b200 import synth
    for name, w in bench.WORKLOADS.items():
        assert callable(getattr(synth, w["gen"])), name
        assert w["build"]["copies"] >= 1 and w["nq"] >= 1
