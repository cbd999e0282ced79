"""Seeded synthetic inputs of the five benchmark configurations.

No dataset is involved: the reference measures this path on random tensors
(``tests/causal_product/test_causal_product_gpu.py:88-117``) and so does this package.
Everything is drawn on the CPU from ``torch.Generator().manual_seed(1000*config + trial)``
in fp32 (CPU and GPU random streams differ) and then moved/cast, so the oracle and the
kernels consume identical values.

config 1: N2  H4  L1024   D=M=64   fp32   Q,K = elu(x)+1, x~N(0,1); V,G ~ N(0,1)
config 2: N8  H8  L4096   D=M=64   fp32   same recipe
config 3: 16-layer causal-linear encoder, 8 heads x 64, FFN 2048, X~U[0,1) (16, 8192, 512)
config 4: N1  H16 L262144 D=M=128  bf16 I/O, recipe of config 1 then rounded to bf16
config 5: N4  H12 L16384  D=256 (Favor, 256 features of a 64-dim query), M=64, fp32;
          pre-map q,k,v ~ N(0, sigma^2) with sigma^2 = 1/sqrt(64)
"""
import math

import torch

SHAPES = {
    1: dict(N=2, H=4, L=1024, D=64, M=64, dtype=torch.float32),
    2: dict(N=8, H=8, L=4096, D=64, M=64, dtype=torch.float32),
    4: dict(N=1, H=16, L=262144, D=128, M=128, dtype=torch.bfloat16),
    5: dict(N=4, H=12, L=16384, D=256, M=64, dtype=torch.float32),
}

ENCODER = dict(n_layers=16, n_heads=8, query_dimensions=64, value_dimensions=64,
               feed_forward_dimensions=2048, attention_type="causal-linear", dropout=0.0)
ENCODER_INPUT = dict(N=16, L=8192, d_model=512)


def generator(config, trial=0):
    return torch.Generator().manual_seed(1000 * config + trial)


def _elu1(x):
    return torch.nn.functional.elu(x) + 1


def elu_inputs(N, H, L, D, M, gen, dtype=torch.float32):
    """Q, K = elu(x)+1 with x~N(0,1); V, G ~ N(0,1); all (N, H, L, dim) on the CPU."""
    Q = _elu1(torch.randn(N, H, L, D, generator=gen))
    K = _elu1(torch.randn(N, H, L, D, generator=gen))
    V = torch.randn(N, H, L, M, generator=gen)
    G = torch.randn(N, H, L, M, generator=gen)
    return tuple(t.to(dtype) for t in (Q, K, V, G))


def favor_omega(query_dims, n_dims, gen):
    """omega (query_dims x n_dims/2) with the block-orthogonal, chi-norm construction of
    the reference's ``orthogonal_random_matrix_`` (fourier_features.py:19-41), drawn from
    ``gen`` on the CPU."""
    cols = n_dims // 2
    w = torch.zeros(query_dims, cols)
    for start in range(0, cols, query_dims):
        end = min(start + query_dims, cols)
        block = torch.randn(query_dims, query_dims, generator=gen)
        norms = block.pow(2).sum(dim=1).sqrt()
        Qm, _ = torch.linalg.qr(block)
        w[:, start:end] = Qm[:, :end - start] * norms[None, :end - start]
    return w


def favor_map(x, omega):
    """Favor features with the default temperature 1/sqrt(E) (fourier_features.py:218-243)."""
    E = x.shape[-1]
    n_dims = 2 * omega.shape[1]
    x = x * math.sqrt(1.0 / math.sqrt(E))
    off = 0.5 * (x * x).sum(-1, keepdim=True) + 0.5 * math.log(n_dims)
    u = x @ omega
    return torch.cat([torch.exp(u - off), torch.exp(-u - off)], dim=-1)


def favor_inputs(N, H, L, E, n_dims, M, gen):
    sigma = math.sqrt(1.0 / math.sqrt(E))
    q = torch.randn(N, H, L, E, generator=gen) * sigma
    k = torch.randn(N, H, L, E, generator=gen) * sigma
    V = torch.randn(N, H, L, M, generator=gen) * sigma
    G = torch.randn(N, H, L, M, generator=gen)
    omega = favor_omega(E, n_dims, gen)
    return favor_map(q, omega), favor_map(k, omega), V, G


def make_inputs(config, trial=0, scale_L=None, scale_N=None, scale_H=None):
    """(Q, K, V, G) CPU tensors of ``config`` (1, 2, 4 or 5); the optional arguments
    replace L, N or H to get a reduced case with the same recipe."""
    s = dict(SHAPES[config])
    if scale_L:
        s["L"] = scale_L
    if scale_N:
        s["N"] = scale_N
    if scale_H:
        s["H"] = scale_H
    gen = generator(config, trial)
    if config == 5:
        return favor_inputs(s["N"], s["H"], s["L"], 64, s["D"], s["M"], gen)
    return elu_inputs(s["N"], s["H"], s["L"], s["D"], s["M"], gen, s["dtype"])


# algorithmic work per token-head (each tensor touched once; multiply-add = 2 flop)
WIDE_GOLDEN_SHAPES = ((128, 128), (256, 64), (64, 192))     # (D, M) of tests/golden/product_wide.npz
WIDE_GOLDEN_ROWS = slice(3, None, 8)                        # the rows that fixture keeps


def wide_golden_inputs(D, M, L=200):
    """Inputs behind ``tests/golden/product_wide.npz`` for one (D, M): one (batch, head) pair of
    ``L`` positions from numpy's legacy generator (stable across versions), so that the fixture
    holds the reference's outputs only.  Returns Q, K (1, 1, L, D) and V, grad_out (1, 1, L, M)."""
    import numpy as np
    r = np.random.RandomState(1000 * D + M)
    Q, K = (torch.from_numpy(r.rand(1, 1, L, D).astype(np.float32) * 0.5) for _ in range(2))
    V, G = (torch.from_numpy(r.randn(1, 1, L, M).astype(np.float32)) for _ in range(2))
    return Q, K, V, G


def algorithmic_bytes(D, M, elem_bytes):
    return (6 * D + 5 * M) * elem_bytes


def algorithmic_flops(D, M):
    return 14 * D * M
