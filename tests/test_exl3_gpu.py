"""EXL3 kernels against the host float64 statement (`formats/exl3.py`): tile decode, rotations, decode-row GEMV and the
prompt path through the decoded W_hat."""
import numpy as np
import pytest
import torch

from ferrite_b200.formats.exl3 import Exl3Tensor

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops(ext):
    from ferrite_b200.ops.cuda_ops import CudaOps
    return CudaOps(DEV)


@pytest.mark.parametrize("bits", [2, 3, 4, 6, 8])
def test_decode_matches_host(ops, bits):
    from ferrite_b200.ops.exl3_linear import Exl3Linear
    t = Exl3Tensor.random(256, 384, bits, seed=bits)
    lin = Exl3Linear(t, DEV)
    want = torch.from_numpy(t.w_hat().astype(np.float32)).t()              # [n, k]
    w_hat_t = torch.empty(384, 256, dtype=torch.bfloat16, device=DEV)
    ops.C.exl3_decode(w_hat_t, lin.trellis, bits)
    got = w_hat_t.float().cpu()
    assert torch.equal(got, want.to(torch.bfloat16).float())


@pytest.mark.parametrize("bits", [3, 4])
@pytest.mark.parametrize("M", [1, 5, 8, 40, 200])
def test_linear_matches_host(ops, bits, M):
    from ferrite_b200.ops.exl3_linear import Exl3Linear
    k, n = 1024, 768
    t = Exl3Tensor.random(k, n, bits, seed=10 + bits)
    lin = Exl3Linear(t, DEV)
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, k, generator=g).to(torch.bfloat16)
    res = torch.randn(M, n, generator=g).to(torch.bfloat16)
    want = t.linear(x.float()).float() + res.float()
    got = lin.forward(ops, x.to(DEV), res.to(DEV)).float().cpu()
    scale = max(1.0, want.abs().max().item())
    assert (got - want).abs().max().item() < (2e-2 if M <= 8 else 4e-2) * scale


def test_engine_runs_from_packed_exl3(ops):
    """`weight_dtype="exl3"`: the big projections are synthetic EXL3 tensors kept packed on the device; the engine's
    logits match the fp32 oracle run on the same tensors dequantised, for decode rows (trellis GEMV) and for a prompt
    chunk (W_hat decoded per use onto the tensor-core GEMM)."""
    import dataclasses
    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.ops.qweight import Exl3Weight, StackWeight
    cfg = dataclasses.replace(tiny_hybrid(), hidden=256, inter=768)
    eng = Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=256, weight_dtype="exl3"), device=DEV, seed=3)
    kinds = {type(v).__name__ for k, v in eng.ex.w.items() if k.endswith(("in_proj", "out_proj", "gate_up", "down"))}
    assert kinds <= {"Exl3Weight", "StackWeight"} and "Exl3Weight" in kinds, kinds
    # the oracle multiplies by the dequantised tensors
    from ferrite_b200.formats.exl3 import Exl3Tensor as _T   # noqa: F401
    dense = {}
    for k, v in eng.ex.w.items():
        if isinstance(v, (Exl3Weight, StackWeight)):
            dense[k] = v.dequantize().cpu()
        else:
            dense[k] = v.float().cpu()
    ref = Engine(cfg, dense, EngineConfig(n_slots=1, max_ctx=256), device="cpu")
    toks = torch.randint(0, cfg.vocab, (72,), generator=torch.Generator().manual_seed(9)).tolist()
    want, _, _ = ref.forward([Segment(0, 0, toks, "all")])
    got, _, _ = eng.forward([Segment(0, 0, toks[:64], "all")], greedy=False)
    rows = [got.float().cpu().clone()]
    for i in range(64, 72):
        lg, _, _ = eng.forward([Segment(0, i, [toks[i]], "last")], greedy=False)
        rows.append(lg.float().cpu().clone())
    got = torch.cat(rows)
    kl = torch.nn.functional.kl_div(torch.log_softmax(got, -1), torch.log_softmax(want, -1), log_target=True,
                                    reduction="batchmean").item()
    assert kl < 2e-2, kl
