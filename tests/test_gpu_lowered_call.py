"""From the reference's IR to the kernels: `quantforge-opt --convert-linalg-to-quantforge --lower-qf-to-runtime`
turns a quantised linalg.matmul into a call of the runtime's C entry point, and quantforge_b200.lowered executes that
call (weight repacked from the matmul's [K, N] orientation). The result must be what the ORIGINAL linalg.matmul with
the reference's unpack / dequant semantics computes, evaluated by the CPU oracle."""
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import qf_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("func,M,K,N,act_i8,scale,zp", [("gemv", 1, 4096, 4096, False, 0.5, 8),
                                                       ("int8_lhs", 2, 256, 512, True, 1.0, 0)])
def test_lowered_matmul_runs_on_the_runtime(func, M, K, N, act_i8, scale, zp):
    from quantforge_b200 import build, lowered
    opt = build.build_opt()
    src = os.path.join(ROOT, "tests", "mlir", "gemv.mlir")
    text = subprocess.run([opt, "--convert-linalg-to-quantforge", "--lower-qf-to-runtime", src], check=True,
                          capture_output=True, text=True).stdout
    assert 'qf.runtime_symbol = "qf_w4a16_linear"' in text
    rng = np.random.default_rng(K + N)
    dev = torch.device("cuda:0")
    # the B operand of the matmul: [K, N] bytes; only the low nibble is a code (upper bits are masked by qf.unpack)
    w_kn = rng.integers(-128, 128, size=(K, N), dtype=np.int8)
    if act_i8:
        act = rng.integers(-8, 8, size=(M, K), dtype=np.int8)
        x_f = act.astype(np.float32)
        act_t = torch.from_numpy(act).to(dev)
    else:
        x_f = O.round_to(rng.normal(size=(M, K)).astype(np.float32) * 0.05, "f16")
        act_t = torch.from_numpy(x_f).to(torch.float16).to(dev)
    y = lowered.run_lowered(text, func, {"act": act_t, "weight": torch.from_numpy(w_kn).to(dev)})
    torch.cuda.synchronize()
    # the original op: Y = X . dequant(unpack(W)) with W[K, N], rank-0 scale and zero point, all in f16
    codes_nk = np.ascontiguousarray((w_kn.view(np.uint8) & 0x0F).astype(np.int8).T)
    w = O.dequant(codes_nk, np.full((1, N), scale, dtype=np.float32), zp, K, "f16")
    want = (x_f.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)
    assert tuple(y.shape) == (M, N) and y.dtype == torch.float16
    assert O.rel_err(y.float().cpu().numpy(), want) < 1e-2
