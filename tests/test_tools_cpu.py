"""The black-box clients against a live server (scripted mock engine) on a local port."""
import asyncio
import json
import socket
import sys
import threading
import time

import pytest
from aiohttp import web

from ferrite_b200.server.app import AppState, make_app
from ferrite_b200.server.engine_api import MockEngine
from ferrite_b200.server.profiles import GenDefaults
from ferrite_b200.server.template import ChatTemplate
from ferrite_b200.server.tokenizer import load_tokenizer


def _serve(capture_dir=None):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    tok = load_tokenizer(None, 4096)
    app = make_app(lambda: AppState(MockEngine(tok, "mock-model", max_batch=8, max_len=4096), tok, ChatTemplate.from_dir(None),
                                    GenDefaults.from_dir(None, "default"), "mock-model", 8, capture_dir=capture_dir))
    loop = asyncio.new_event_loop()
    started = threading.Event()

    def run():
        asyncio.set_event_loop(loop)
        runner = web.AppRunner(app)
        loop.run_until_complete(runner.setup())
        loop.run_until_complete(web.TCPSite(runner, "127.0.0.1", port).start())
        started.set()
        loop.run_forever()
    threading.Thread(target=run, daemon=True).start()
    assert started.wait(20)
    return f"http://127.0.0.1:{port}", loop


def test_conformance_suite_passes_on_the_mock_server(capsys):
    from ferrite_b200.tools.conformance import main
    url, loop = _serve()
    try:
        rc = main(["--base-url", url, "--mock", "--tier", "all"])
    finally:
        loop.call_soon_threadsafe(loop.stop)
    out = capsys.readouterr().out
    assert rc == 0, out
    assert "FAIL" not in out


def test_conformance_profile_and_replay_of_captured_requests(capsys, tmp_path):
    """A server that captures its requests; the suite then checks the model profile and sends the captured requests
    again (greedy ones twice, same text)."""
    from ferrite_b200.tools.conformance import main
    from ferrite_b200.tools.httpc import Client
    cap = tmp_path / "cap"
    url, loop = _serve(capture_dir=str(cap))
    try:
        c = Client(url)
        for body in ({"messages": [{"role": "user", "content": "say hello twice"}], "max_tokens": 12, "temperature": 0},
                     {"messages": [{"role": "user", "content": "[[say:alpha beta]]"}], "max_tokens": 8}):
            assert c.post("/v1/chat/completions", dict(body, model="mock-model"))[0] == 200
        assert len(list(cap.glob("*.request.json"))) == 2
        rc = main(["--base-url", url, "--mock", "--only", "replay", "--profile", "mock", "--replay", str(cap)])
        out = capsys.readouterr().out
        assert rc == 0 and "PASS replay" in out and "FAIL" not in out, out
        rc = main(["--base-url", url, "--mock", "--only", "profile", "--profile", "mock"])
        out = capsys.readouterr().out
        assert rc == 0 and "PASS profile" in out, out
        bad = tmp_path / "p.json"
        bad.write_text(json.dumps({"model": "other-model", "context": 16, "skip": ["health"]}))
        rc = main(["--base-url", url, "--only", "profile", "--profile", str(bad)])
        out = capsys.readouterr().out
        assert rc == 1 and "FAIL profile" in out, out
    finally:
        loop.call_soon_threadsafe(loop.stop)


def test_quickbench_reports_streams(capsys):
    from ferrite_b200.tools.quickbench import main
    url, loop = _serve()
    try:
        rc = main(["--base-url", url, "--streams", "3", "--prompt-tokens", "16", "--max-tokens", "24"])
    finally:
        loop.call_soon_threadsafe(loop.stop)
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and line["ok"] == 3 and line["total_tokens"] > 0


def test_workload_clients_on_the_mock_server(capsys, tmp_path):
    """edit / lanes (with the gate) / mixed / agents against the scripted mock: each prints one JSON line and succeeds."""
    from ferrite_b200.tools.workloads import main
    url, loop = _serve()
    try:
        lines = {}
        for argv in (["edit", "--streams", "2", "--max-tokens", "32", "--max-source-chars", "600", "--out", str(tmp_path / "e")],
                     ["lanes", "--lanes", "1,3,64", "--prefix-tokens", "120", "--max-tokens", "24", "--runs", "1", "--gate"],
                     ["mixed", "--decoders", "2", "--prompts", "2", "--prompt-tokens", "200", "--max-tokens", "40", "--lead-s", "0.05"],
                     ["agents", "--agents", "2", "--turns", "3", "--prefix-tokens", "80", "--max-tokens", "32"]):
            rc = main(argv[:1] + ["--base-url", url] + argv[1:])
            line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
            assert rc == 0, line
            lines[line["workload"]] = line
    finally:
        loop.call_soon_threadsafe(loop.stop)
    assert lines["edit"]["streams"] == 2 and (tmp_path / "e-1.txt").exists()
    pts = {p["lanes"]: p for p in lines["lanes"]["points"]}
    assert pts[3]["gate_lanes_differing_from_alone"] == [] and pts[3]["cached_tokens"] > 0 and "skipped" in pts[64]
    assert lines["mixed"]["chunk_gap_ms"]["median"] is not None and len(lines["mixed"]["prompt_ttft_s"]) == 2
    assert lines["agents"]["cached_share_after_first_turn"] > 0.5


def test_mode_gate_and_turns_on_the_mock_server(capsys, tmp_path):
    """modes: hashes saved by one run compare equal on the next and a changed reference is reported with the first
    differing characters; turns: the growing conversation is served from the cache after its first turn."""
    from ferrite_b200.tools.workloads import main
    url, loop = _serve()
    ref = str(tmp_path / "ref.json")
    try:
        assert main(["modes", "--base-url", url, "--save", ref, "--max-tokens", "24", "--long-tokens", "150", "--max-source-chars", "500"]) == 0
        first = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert first["cases"] == 7 and first["saved"] == ref
        assert main(["modes", "--base-url", url, "--compare", ref, "--max-tokens", "24", "--long-tokens", "150", "--max-source-chars", "500"]) == 0
        assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["different"] == {}
        data = json.load(open(ref))
        data["hashes"]["code"] = "0" * 16
        data["texts"]["code"] = "X" + data["texts"]["code"][1:]
        json.dump(data, open(ref, "w"))
        assert main(["modes", "--base-url", url, "--compare", ref, "--max-tokens", "24", "--long-tokens", "150", "--max-source-chars", "500"]) == 1
        diff = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["different"]
        assert list(diff) == ["code"] and diff["code"]["at"] == 0
        assert main(["turns", "--base-url", url, "--turns", "3", "--prefix-tokens", "200", "--tool-tokens", "50", "--max-tokens", "16"]) == 0
        t = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert len(t["turns"]) == 3 and t["turns"][2]["cached_tokens"] > 0 and t["turns"][2]["prompt_tokens"] > t["turns"][0]["prompt_tokens"]
    finally:
        loop.call_soon_threadsafe(loop.stop)


def test_release_gate_on_the_mock_server(capsys):
    from ferrite_b200.tools.release_gate import main
    url, loop = _serve()
    try:
        rc = main(["--base-url", url, "--mock", "--lanes", "1,2", "--prefix-tokens", "100", "--streams", "2"])
        out = capsys.readouterr().out
        assert rc == 0 and "release gate: PASS" in out, out
        rc = main(["--base-url", url, "--mock", "--lanes", "1", "--prefix-tokens", "50", "--streams", "2", "--min-tok-s", "1e9"])
        out = capsys.readouterr().out
        assert rc == 1 and "FAIL serving rate" in out, out
    finally:
        loop.call_soon_threadsafe(loop.stop)


def test_launch_commands_and_step_summary():
    from ferrite_b200.tools.launch import command
    from ferrite_b200.tools.sched_steps import summarise
    one = command(1, ["--preset", "tiny"])
    assert one[1:3] == ["-m", "ferrite_b200.server"]
    tp = command(8, ["--preset", "27b"], master_port=29500)
    assert "--nproc-per-node=8" in tp and tp[tp.index("--master-addr") + 1] == "127.0.0.1" and tp[-2:] == ["--preset", "27b"]
    s = summarise(["step 1: dec 0 rows, prompt 64 rows, 3.10 ms", "step 2: dec 2 rows, prompt 64 rows, 3.50 ms",
                   "noise", "step 3: dec 2 rows, prompt 0 rows, 1.00 ms"])
    assert s["prompt"]["steps"] == 1 and s["mixed"]["rows"] == 66 and s["decode"]["ms_per_step"] == 1.0


def test_launcher_presets_and_gpu_locks(tmp_path, capsys, monkeypatch):
    """Presets expand to server arguments + environment (the caller's arguments come last, so they win); a GPU's lock
    file is exclusive, names its holder, and is released for the next launcher."""
    import subprocess
    import sys

    from ferrite_b200.tools import launch
    assert launch.main(["--preset", "27b-spec", "--port", "8123", "--dry-run", "--", "--slots", "2"]) == 0
    line = capsys.readouterr().out.strip()
    assert "FE_SPEC=16" in line and "--drafter block" in line and line.endswith("--slots 2 --port 8123")
    assert launch.main(["--preset", "27b-tp8", "--dry-run"]) == 0
    assert "--nproc-per-node=8" in capsys.readouterr().out
    assert launch.main(["--gpus", "2", "--gpu-ids", "4,5", "--dry-run"]) == 0
    assert "CUDA_VISIBLE_DEVICES=4,5" in capsys.readouterr().out
    assert launch.main(["--preset", "nope", "--dry-run"]) == 2 and launch.main(["--gpus", "2", "--gpu-ids", "1", "--dry-run"]) == 2
    capsys.readouterr()
    base = str(tmp_path / "gpu.lock")
    fds = launch.take_gpu_locks([1, 0], base=base, note="server A")
    # flock is per open file description: a second process (here: a child) must be refused and told who holds the GPU
    code = ("import sys; from ferrite_b200.tools import launch\n"
            "try:\n    launch.take_gpu_locks([2, 1], base=sys.argv[1])\n"
            "except launch.LockBusy as e:\n    print(e); sys.exit(4)\n")
    r = subprocess.run([sys.executable, "-c", code, base], capture_output=True, text=True)
    assert r.returncode == 4 and "GPU 1 is in use" in r.stdout and "server A" in r.stdout and f"pid {__import__('os').getpid()}" in r.stdout
    launch.release_locks(fds)
    r = subprocess.run([sys.executable, "-c", code, base], capture_output=True, text=True)
    assert r.returncode == 0
    assert launch.port_of(["--x", "--port", "81"]) == 81 and launch.port_of(["--port=82"]) == 82 and launch.port_of([]) == 0


def test_sched_budget_replays_a_verify_trace():
    """A speculative run with FE_SCHED_PROF=2-style tracing: the tool reads the verify steps and reports what smaller
    draft budgets would have accepted; the summary tool still reads the longer lines."""
    import contextlib
    import io

    import torch

    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.sampler import Sampling
    from ferrite_b200.engine.scheduler import SchedOptions, Scheduler, generate
    from ferrite_b200.tools import sched_budget as SB
    from ferrite_b200.tools.sched_steps import summarise
    cfg = tiny_hybrid()
    eng = Engine(cfg, None, EngineConfig(n_slots=2, max_ctx=256), device="cpu")
    base = torch.randint(1, cfg.vocab, (30,), generator=torch.Generator().manual_seed(0)).tolist()
    p = base + base + base[:10]                                   # the copier has something to propose
    err = io.StringIO()
    with contextlib.redirect_stderr(err):
        generate(Scheduler(eng, SchedOptions(spec=8, prof=2, arrival_ms=0)), [p, p[5:]], Sampling(max_tokens=24))
    lines = err.getvalue().splitlines()
    steps = SB.parse(lines)
    assert steps and all(len(s[2]) == len(s[3]) == len(s[4]) for s in steps)
    rep = SB.budgets(steps, [(2, 8.9), (9, 9.4)], 1.5)
    for slot in rep.values():
        accs = [c["accepted"] for c in slot["budgets"].values()]
        assert accs == sorted(accs) and accs[-1] <= slot["mean_accepted"] + 1e-9 and "tok_s" in slot["budgets"][1]
    assert summarise(lines)["decode"]["steps"] >= len(steps)
    assert SB.interp([(2, 1.0), (4, 3.0)], 3) == 2.0 and SB.interp([(2, 1.0), (4, 3.0)], 9) == 3.0


def test_control_tool_and_environment_check(tmp_path, monkeypatch, capsys):
    """ctl: start a mock server in the background (own session, log + pid files), refuse a second start, report status,
    stop it. check_env: the report names the toolchain and asks for GPUs only when told to."""
    from ferrite_b200.tools import check_env, ctl
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    monkeypatch.setenv("FERRITE_LOG_DIR", str(tmp_path))
    monkeypatch.setenv("FERRITE_START_TIMEOUT", "120")
    assert ctl.main(["start", "--preset", "mock", "--port", str(port)]) == 0
    try:
        assert "serving on" in capsys.readouterr().out
        assert ctl.main(["start", "--preset", "mock", "--port", str(port)]) == 1         # one server a port
        assert ctl.main(["status", "--port", str(port)]) == 0
        st = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert st["running"] and st["health"]["engine"] == "mock"
        assert (tmp_path / f"server-{port}.log").exists() and (tmp_path / f"server-{port}.pid").exists()
    finally:
        assert ctl.main(["stop", "--port", str(port)]) == 0
    assert ctl.main(["status", "--port", str(port)]) == 1
    capsys.readouterr()
    rep = check_env.check(build=True)
    assert rep["torch"] and rep["nvcc_sm_100a"] is True and rep["extension_loads"] and not rep["errors"]
    assert check_env.check(gpus=2)["errors"]                      # no GPU on the test machine: asking for two is an error


@pytest.mark.parametrize("drafter", ["none", "block"])
def test_tp_gate_with_two_cpu_ranks(capsys, drafter):
    """The tensor-parallel server gate end to end on two gloo ranks: start, concurrent lanes equal to solo runs, repeat,
    ranks alive, stop; with a block drafter, mirrored on both ranks, speculation must have run too."""
    from ferrite_b200.tools.tp_gate import main
    rc = main(["--gpus", "2", "--lanes", "1,2", "--prefix-tokens", "60", "--start-timeout", "180", "--",
               "--preset", "tiny", "--device", "cpu", "--slots", "2", "--max-model-len", "2048", "--drafter", drafter])
    out = capsys.readouterr().out
    assert rc == 0 and out.count("PASS") == (6 if drafter == "none" else 7) and "tp gate: PASS" in out, out


def test_check_model_reports_missing_tensors_and_changed_files(tmp_path, capsys):
    import torch
    from ferrite_b200.config import tiny_hybrid
    from ferrite_b200.formats.loader import save_native
    from ferrite_b200.models.weights import init_weights
    from ferrite_b200.tools import check_model
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0, dtype=torch.bfloat16)
    good = tmp_path / "good"
    good.mkdir()
    save_native(w, str(good / "model.safetensors"), cfg)
    assert check_model.main([str(good), "--preset", "tiny", "--manifest"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["missing"] == [] and rep["storage"]["bfloat16"]["tensors"] > 10 and rep["params"] == cfg.param_count()
    (tmp_path / "m.json").write_text(json.dumps(rep))
    assert check_model.main([str(good), "--preset", "tiny", "--verify", str(tmp_path / "m.json")]) == 0
    capsys.readouterr()
    bad = tmp_path / "bad"
    bad.mkdir()
    w2 = {k: v for k, v in w.items() if k != "l1.down"}
    w2["l0.down"] = w2["l0.down"][:, :-8].contiguous()
    save_native(w2, str(bad / "model.safetensors"), cfg)
    assert check_model.main([str(bad), "--preset", "tiny", "--verify", str(tmp_path / "m.json")]) == 1
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["missing"] == ["l1.down"] and "l0.down" in rep["shape_mismatches"]
    assert any("differs from the manifest" in p for p in rep["problems"])


def test_sweep_runs_points(capsys):
    from ferrite_b200.tools.sweep import main
    url, loop = _serve()
    try:
        rc = main(["--base-url", url, "--streams", "1,2", "--prompt-tokens", "8", "--max-tokens", "8"])
    finally:
        loop.call_soon_threadsafe(loop.stop)
    out = capsys.readouterr().out
    assert rc == 0 and "agg tok/s" in out


def test_chart_writes_an_svg_from_json_lines(tmp_path):
    """The chart tool reads sweep / bench JSON lines (nested keys too) and writes a self-contained SVG."""
    import json
    import xml.etree.ElementTree as ET

    from ferrite_b200.tools import chart
    a, b = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    a.write_text("noise\n" + "\n".join(json.dumps({"streams": n, "aggregate_tok_s": 100.0 * n ** 0.8, "e2e": {"value": n}})
                                         for n in (1, 2, 4, 8)))
    b.write_text("\n".join(json.dumps({"streams": n, "aggregate_tok_s": 60.0 * n}) for n in (1, 2, 4)))
    assert chart.read_points(str(a), "streams", "e2e.value") == [(1.0, 1.0), (2.0, 2.0), (4.0, 4.0), (8.0, 8.0)]
    out = tmp_path / "c.svg"
    assert chart.main([str(a), str(b), "--title", "decode", "-o", str(out)]) == 0
    root = ET.fromstring(out.read_text())
    tags = [e.tag.split("}")[-1] for e in root.iter()]
    assert tags.count("polyline") == 2 and tags.count("circle") == 7


def test_package_builds_an_archive_and_refuses_machine_traces(tmp_path):
    """The release packer on a small stand-in tree: archive + checksum + BUILD-INFO with per-file hashes; a private
    network address in a packed text file stops the release and names the line."""
    import hashlib
    import tarfile

    from ferrite_b200.tools import package as P
    root = tmp_path / "repo"
    (root / "ferrite_b200" / "csrc").mkdir(parents=True)
    (root / "ferrite_b200" / "__pycache__").mkdir()
    (root / "profiles").mkdir()
    (root / "tests").mkdir()
    (root / "ferrite_b200" / "__init__.py").write_text('__version__ = "9.9.9"\n')
    (root / "ferrite_b200" / "_C.so").write_bytes(b"\x7fELF stand-in")
    (root / "ferrite_b200" / "csrc" / "k.cu").write_text("__global__ void k() {}\n")
    (root / "ferrite_b200" / "__pycache__" / "x.pyc").write_bytes(b"junk")
    (root / "bench.py").write_text("print('bench')\n")
    (root / "README.md").write_text("connect to 127.0.0.1:8000\n")
    path, info = P.package(str(root), str(tmp_path / "dist"), build=False, allow=[r"127\.0\.0\.1"])
    name = "ferrite-b200-9.9.9-sm100a"
    assert path.endswith(name + ".tar.gz")
    with tarfile.open(path) as tar:
        names = sorted(tar.getnames())
        build = json.loads(tar.extractfile(f"{name}/BUILD-INFO").read())
    assert f"{name}/ferrite_b200/_C.so" in names and f"{name}/ferrite_b200/csrc/k.cu" in names and f"{name}/bench.py" in names
    assert not any("__pycache__" in n for n in names)
    assert build["files"]["bench.py"] == hashlib.sha256(b"print('bench')\n").hexdigest()
    digest, fname = open(path + ".sha256").read().split()
    assert fname == name + ".tar.gz" and digest == hashlib.sha256(open(path, "rb").read()).hexdigest()
    (root / "README.md").write_text("line one\nour box is 192.168.7.20, ask there\n")
    with pytest.raises(SystemExit) as e:
        P.package(str(root), str(tmp_path / "dist2"), build=False, allow=[r"127\.0\.0\.1"])
    assert "README.md:2" in str(e.value) and "192.168.7.20" in str(e.value)
    assert not (tmp_path / "dist2").exists()
