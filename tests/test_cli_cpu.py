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
