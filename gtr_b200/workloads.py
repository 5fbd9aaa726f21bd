"""Seeded synthetic workloads: the shapes and value distributions of the benchmark configurations.

These stand in for the reference's datasets and checkpoints (none of which is reproduced): the operator
benchmark, the parity tests and the smoke test all draw their inputs here, so that a number and the test that
vouches for it are about the same data.  Inputs are generated in fp32 on the CPU in the order q, k, v, g and cast
afterwards, so that a CPU reference and the GPU see identical values.

Gate distributions follow the reference's own operator test (engine/gtr/backbone/csrc/test_gla.py:58-71):
``g = logsigmoid(mean + std * randn) / normalizer`` per (token, head, key channel).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

CONFIGS = {
    # name: batch, heads, tokens, patch grid, std of q/k/v, gate = (kind, mean, std, normalizer), key channels
    "c1": dict(B=1, H=6, T=1600, grid=(40, 40), std=1.0 / 8, gate=("ls", 0.0, 1.0, 16.0), K=64),
    "c2": dict(B=8, H=6, T=1600, grid=(40, 40), std=1.0 / 8, gate=("ls", 0.0, 1.0, 16.0), K=64),
    "c3": dict(B=4, H=12, T=6400, grid=(80, 80), std=1.0 / 8, gate=("ls", 0.0, 1.0, 16.0), K=64),
    "c5": dict(B=2, H=8, T=8192, grid=(64, 128), std=3.0, gate=("ls", 4.0, 2.0, 1.0), K=64),
    # the throughput point with the key heads of the released GTR models (and of the reference's own kernel)
    "k32": dict(B=4, H=12, T=6400, grid=(80, 80), std=1.0 / 8, gate=("ls", 0.0, 1.0, 16.0), K=32),
}


def make_inputs(B, T, H, K=64, V=64, std=1.0 / 8, gate=("ls", 0.0, 1.0, 16.0), seed=0, dtype=torch.float16):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=gen) * std
    k = torch.randn(B, T, H, K, generator=gen) * std
    v = torch.randn(B, T, H, V, generator=gen) * std
    kind, mean, gstd, norm = gate
    assert kind == "ls"
    g = F.logsigmoid(torch.randn(B, T, H, K, generator=gen) * gstd + mean) / norm
    return tuple(x.to(dtype) for x in (q, k, v, g))


def config_inputs(name: str, seed: int = 0, dtype=torch.float16, B=None):
    c = CONFIGS[name]
    return make_inputs(B or c["B"], c["T"], c["H"], K=c["K"], std=c["std"], gate=c["gate"], seed=seed, dtype=dtype)


def algorithmic_bytes_per_token_head(K: int = 64, V: int = 64, gated: bool = False) -> int:
    """fp16 bytes that must cross HBM per (token, head): q, k, g read (3 K), v read and o written (2 V), plus the
    output gate (V) when the fused RMSNorm * w * silu(gate) epilogue is used.  Workspace traffic and re-reads do not
    count."""
    return 2 * (3 * K + 2 * V + (V if gated else 0))
