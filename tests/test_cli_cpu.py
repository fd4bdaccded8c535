"""The engine's command line on the CPU engine: generate, logits, sched-test, park-test."""
import json

import torch

from ferrite_b200 import cli
from ferrite_b200.config import PRESETS, EngineConfig
from ferrite_b200.engine.engine import Engine


def _run(capsys, *argv):
    rc = cli.main(list(argv) + ["--device", "cpu"])
    return rc, json.loads(capsys.readouterr().out.strip().splitlines()[-1])


def test_generate_matches_engine_generate(capsys):
    rc, out = _run(capsys, "generate", "--ids", "5,9,33,70,12", "--max-tokens", "6")
    assert rc == 0 and out["prompt_tokens"] == 5 and out["new_tokens"] == 6
    eng = Engine(PRESETS["tiny"](), None, EngineConfig(n_slots=1, max_ctx=256), device="cpu")
    assert out["ids"] == eng.generate([5, 9, 33, 70, 12], 6)


def test_logits_dump_is_chunk_invariant(capsys, tmp_path):
    ids = tmp_path / "ids.txt"
    ids.write_text(",".join(str(3 + 7 * i) for i in range(19)))
    outs = []
    for chunk in (4, 32):
        path = tmp_path / f"l{chunk}.pt"
        rc, out = _run(capsys, "logits", "--ids-file", str(ids), "--out", str(path), "--chunk", str(chunk))
        assert rc == 0 and out["positions"] == 19 and out["finite"]
        outs.append(torch.load(path)["logits"])
    assert outs[0].shape == (19, PRESETS["tiny"]().vocab)
    assert torch.allclose(outs[0], outs[1], atol=2e-4, rtol=1e-4)


def test_sched_test_and_park_test_pass(capsys):
    for argv in (["sched-test"], ["sched-test", "--spec", "4", "--slots", "2"], ["park-test"]):
        rc, out = _run(capsys, *argv)
        assert rc == 0 and out["ok"], out


def test_logits_are_schedule_invariant_and_layer_dump(capsys, tmp_path, monkeypatch):
    rc, out = _run(capsys, "logits-test", "--tokens", "90", "--chunk", "32")
    assert rc == 0 and out["ok"] and set(out["max_abs_diff"]) == {"stagger", "split", "mix"}
    ids = tmp_path / "ids.txt"
    ids.write_text(",".join(str(3 + 5 * i) for i in range(40)))
    a, b = tmp_path / "a.pt", tmp_path / "b.pt"
    assert _run(capsys, "logits", "--ids-file", str(ids), "--out", str(a), "--chunk", "16")[0] == 0
    assert _run(capsys, "logits", "--ids-file", str(ids), "--out", str(b), "--chunk", "16", "--schedule", "mix")[0] == 0
    assert torch.allclose(torch.load(a)["logits"], torch.load(b)["logits"], atol=1e-4)
    # FE_LOG_DUMP: one hash line per layer and step; the same input gives the same lines
    monkeypatch.setenv("FE_LOG_DUMP", "1")
    runs = []
    for _ in range(2):
        cli.main(["generate", "--ids", "5,6,7", "--max-tokens", "1", "--device", "cpu"])
        runs.append([ln for ln in capsys.readouterr().err.splitlines() if ln.startswith("layer ")])
    n_layers = PRESETS["tiny"]().n_layers
    assert len(runs[0]) == 2 * n_layers and runs[0] == runs[1] and "sha1" in runs[0][0]


def test_stored_reference_kl_workflow(capsys, tmp_path):
    """logits dump -> top-k reference -> score: an engine scored against its own reference gives 0, one with a 4-bit KV
    cache a small positive KL, other token ids are refused."""
    from ferrite_b200.utils import kl_score
    ids = tmp_path / "ids.txt"
    ids.write_text(",".join(str(3 + 11 * i % 4000) for i in range(80)))
    ref_l, same_l, ref_t = tmp_path / "ref.pt", tmp_path / "same.pt", tmp_path / "topk.pt"
    assert _run(capsys, "logits", "--ids-file", str(ids), "--out", str(ref_l), "--chunk", "40")[0] == 0
    assert _run(capsys, "logits", "--ids-file", str(ids), "--out", str(same_l), "--chunk", "16")[0] == 0
    assert kl_score.main(["make-ref", "--logits", str(ref_l), "--topk", "32", "--out", str(ref_t)]) == 0
    made = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert made["positions"] == 80 and made["topk"] == 32
    assert kl_score.main(["score", "--ref", str(ref_t), "--logits", str(same_l), "--skip", "10"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert abs(out["kl_mean"]) < 1e-5 and out["sequences"][0]["positions"] == 70 and out["sequences"][0]["top1_agreement"] == 1.0
    full = torch.load(ref_l)["logits"]
    noisy = tmp_path / "noisy.pt"
    torch.save({"ids": torch.load(ref_l)["ids"], "logits": full + 0.3 * torch.randn(full.shape, generator=torch.Generator().manual_seed(1))}, noisy)
    assert kl_score.main(["score", "--ref", str(ref_t), "--logits", str(noisy)]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    exact = torch.nn.functional.kl_div(torch.log_softmax(torch.load(noisy)["logits"], -1), torch.log_softmax(full, -1),
                                       log_target=True, reduction="batchmean").item()
    assert 0 < out["kl_mean"] <= exact + 1e-6                     # the bucketed form is a lower bound of the full KL
    other = tmp_path / "other.pt"
    torch.save({"ids": [1] * 80, "logits": full}, other)
    assert kl_score.main(["score", "--ref", str(ref_t), "--logits", str(other)]) == 2


def _ids(n, seed=3):
    g = torch.Generator().manual_seed(seed)
    return ",".join(str(int(t)) for t in torch.randint(1, PRESETS["tiny"]().vocab, (n,), generator=g))


def test_selftest_tree_test_and_snaptest_pass(capsys):
    rc = cli.main(["selftest", "--device", "cpu"])
    lines = capsys.readouterr().out.strip().splitlines()
    rep = json.loads(lines[-2])
    assert rc == 0 and json.loads(lines[-1]) == "selftest: all OK"
    assert rep["checks"]["oracle_ok"] and rep["checks"]["oracle_max_abs_err"] < 1e-3 and rep["checks"]["repeat_bit_equal"]
    rc, out = _run(capsys, "tree-test", "--ids", _ids(40), "--max-tokens", "40", "--nodes", "7")
    assert rc == 0 and out["same_text"] and out["tree_rounds"] > 0 and out["rounds"] < 40, out
    rc, out = _run(capsys, "df-snaptest", "--tokens", "200")
    assert rc == 0 and out["ok"] and not out["rebuilt_in_between"], out
    rc, out = _run(capsys, "df-snaptest", "--tokens", "400", "--window", "64")
    assert rc == 0 and out["ok"] and out["rebuilt_in_between"], out


def test_decoy_tree_is_a_well_formed_tree():
    g = torch.Generator().manual_seed(0)
    truth = list(range(100, 120))
    seen_sibling_first = False
    for _ in range(200):
        toks, pars = cli.decoy_tree(truth, 7, 1000, g)
        assert len(toks) == len(pars) <= 7
        assert all(0 <= p <= i for i, p in enumerate(pars))          # a parent is the root or an earlier row
        # the true chain is in the tree as far as it goes: follow it from the root
        node, depth = 0, 0
        while True:
            kids = [i + 1 for i, p in enumerate(pars) if p == node]
            nxt = next((k for k in kids if toks[k - 1] == truth[depth]), None)
            if nxt is None:
                break
            seen_sibling_first |= kids[0] != nxt
            node, depth = nxt, depth + 1
        assert (depth > 0) == (len(toks) > 0)
    assert seen_sibling_first


def test_bench_reports_every_length_and_the_streams(capsys):
    rc, out = _run(capsys, "bench", "--lens", "40,90", "--dec", "4", "--slots", "2")
    assert rc == 0 and [x["len"] for x in out["lens"]] == [40, 90]
    assert all(x["prefill_tok_s"] > 0 and x["decode_tok_s"] > 0 for x in out["lens"])
    assert out["streams"]["slots"] == 2 and out["streams"]["tok_s_total"] > 0


def test_lockstep_tensor_parallel_generate_equals_one_rank(capsys):
    """The same command on two gloo ranks under torch.distributed.run: rank 0 prints the text of one rank."""
    import subprocess
    import sys
    ids = _ids(12, seed=8)
    rc, want = _run(capsys, "generate", "--ids", ids, "--max-tokens", "10")
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), "-m", "ferrite_b200.cli", "generate", "--device", "cpu",
                        "--ids", ids, "--max-tokens", "10"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-800:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1                                            # rank 0 only
    assert json.loads(lines[0])["ids"] == want["ids"]
