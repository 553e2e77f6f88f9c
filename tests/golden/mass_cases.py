"""Seeded inputs of the group-mass golden cases, shared by ``make_golden.py`` (which runs the reference's
kernel on them) and by the tests (which run the oracle and the CUDA kernel on them)."""

import math

import torch


def mass_inputs(case):
    """Seeded q, k (B,H,L,D) and the exact fp64 log-sum-exp of the scaled logits, rounded to fp32; shared
    by this generator and the tests (only the kernel OUTPUT is stored in the fixture)."""
    B, H, Lq, Lk, D, dtype, seed, clustered = (case[n] for n in ("B", "H", "Lq", "Lk", "D", "dtype", "seed", "clustered"))
    g = torch.Generator().manual_seed(seed)
    if clustered:
        cent = torch.randn(H, 8, D, generator=g)
        q = cent[:, torch.randint(0, 8, (Lq,), generator=g)] + 0.3 * torch.randn(H, Lq, D, generator=g)
        k = cent[:, torch.randint(0, 8, (Lk,), generator=g)] + 0.3 * torch.randn(H, Lk, D, generator=g)
        q, k = q.unsqueeze(0), k.unsqueeze(0)
    else:
        q, k = torch.randn(B, H, Lq, D, generator=g), torch.randn(B, H, Lk, D, generator=g)
    # "bf16_as_f32": bf16 values carried in fp32 tensors (the interpreter cannot execute bf16 on the CPU;
    # products of bf16 values are exact in fp32, so this is the bf16 kernel up to its output rounding)
    if dtype == "bf16_as_f32":
        q, k = q.to(torch.bfloat16).float(), k.to(torch.bfloat16).float()
    elif dtype == "f16":
        q, k = q.half(), k.half()
    scale = 1.0 / math.sqrt(D)
    lse = torch.logsumexp(q.double() @ k.double().transpose(-1, -2) * scale, dim=-1).float()
    return q, k, lse, scale


MASS_CASES = [
    dict(B=1, H=2, Lq=300, Lk=300, D=64, dtype="f16", seed=21, clustered=False),
    dict(B=1, H=2, Lq=384, Lk=520, D=128, dtype="f16", seed=22, clustered=True),
    dict(B=2, H=1, Lq=200, Lk=333, D=128, dtype="bf16_as_f32", seed=23, clustered=False),
    dict(B=1, H=2, Lq=640, Lk=640, D=128, dtype="bf16_as_f32", seed=24, clustered=True),
]
