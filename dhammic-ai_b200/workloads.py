"""Seeded synthetic workloads for the SSD chunked scan.

The five benchmark configurations are described by shape and value
distribution only (no dataset is involved); the same generator feeds the
parity tests, the benchmark and the CPU baseline so that every arm sees
identical numbers.

Draw order (fp32, CPU, ``torch.Generator().manual_seed(1000 + config_idx)``):
x ~ N(0,1); dt = clamp(softplus(0.5*N(0,1) + b0), 1e-3, 1e-1) with
b0 = log(expm1(0.02)); A_head = -exp(U(ln 1, ln 16)) per head;
B, C ~ N(0,1)/sqrt(d_state) per group; D ~ N(0,1) per head; dy ~ N(0,1);
the Mamba-3 variant additionally draws raw_angles = U(-pi,pi)*sigmoid(N(0,1))
per (batch, pos, head, d_state/2) and lam = sigmoid(N(0,1)) per
(batch, pos, head).  For bf16 workloads x, B, C, dy (and raw_angles) are
rounded to bf16; dt, A_head, D and lam stay fp32.

The log-decay convention follows the reference caller
(src/mamba_base_engine.py:128-130, 170-173): the scan receives
``x * dt`` and ``dt * A_head``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch


@dataclass(frozen=True)
class SSDConfig:
    name: str
    batch: int          # per GPU for the weak-scaling configs
    seqlen: int         # per GPU for the sequence-parallel config
    nheads: int
    headdim: int
    d_state: int
    ngroups: int
    chunk: int
    dtype: str          # "fp32" | "bf16"
    mamba3: bool = False
    seq_parallel: bool = False
    index: int = 0

    @property
    def tokens(self) -> int:
        return self.batch * self.seqlen

    def bytes_per_token(self) -> int:
        """Algorithmic HBM bytes per token, forward + backward.

        Each operand and result is touched once per pass at its storage
        width; intermediates (states, decay masks, C.B^T) count zero.
        fwd reads x,B,C,dt and writes y; bwd reads x,dy,B,C,dt and writes
        dx,dB,dC,ddt.
        """
        w = 2 if self.dtype == "bf16" else 4
        ex = self.nheads * self.headdim
        eb = self.ngroups * self.d_state
        edt = self.nheads
        total = 5 * w * ex + 6 * w * eb + 12 * edt
        if self.mamba3:
            total += 3 * w * self.nheads * self.d_state // 2 + 12 * self.nheads
        return total

    def flops_per_token(self) -> int:
        """Algorithmic tensor FLOPs per token, forward + backward.

        2*M*N*K of each dense contraction on full chunk x chunk tiles,
        C.B^T counted once per group (per head for the Mamba-3 variant,
        whose rotation is per head); backward recomputes C.B^T once.
        """
        l, h, p, n = self.chunk, self.nheads, self.headdim, self.d_state
        gcb = h if self.mamba3 else self.ngroups
        fwd = 2 * l * gcb * n + h * (2 * l * p + 4 * n * p)
        bwd = 6 * l * gcb * n + h * (4 * l * p + 8 * n * p)
        return fwd + bwd


CONFIGS = {
    0: SSDConfig("cfg0_cpu_fp32_b2_T512_h8_p64_n64_g1_l64", 2, 512, 8, 64, 64, 1, 64, "fp32", index=0),
    1: SSDConfig("cfg1_130M_bf16_b8_T2048_h24_p64_n128_g1_l64", 8, 2048, 24, 64, 128, 1, 64, "bf16", index=1),
    2: SSDConfig("cfg2_1p3B_bf16_b16_T4096_h64_p64_n128_g8_l128", 16, 4096, 64, 64, 128, 8, 128, "bf16", index=2),
    3: SSDConfig("cfg3_mamba3_bf16_b16_T4096_h64_p64_n128_g8_l128", 16, 4096, 64, 64, 128, 8, 128, "bf16",
                 mamba3=True, index=3),
    4: SSDConfig("cfg4_seqpar_bf16_b1_T131072_h64_p64_n128_g8_l128", 1, 131072, 64, 64, 128, 8, 128, "bf16",
                 seq_parallel=True, index=4),
}

DT_BIAS0 = math.log(math.expm1(0.02))


def shrink(cfg: SSDConfig, batch: int | None = None, seqlen: int | None = None) -> SSDConfig:
    """Same per-token shape with a smaller batch / sequence (for oracle-sized parity cases)."""
    return replace(cfg, batch=batch or cfg.batch, seqlen=seqlen or cfg.seqlen)


def make_inputs(cfg: SSDConfig, seed: int | None = None, device: str | torch.device = "cpu",
                rank: int = 0) -> dict[str, torch.Tensor]:
    """Draw one workload.  Returned tensors are in storage dtype on ``device``.

    Keys: x (b,T,h,p), dt (b,T,h) fp32, A_head (h,) fp32, B, C (b,T,g,n),
    D (h,) fp32, dy (b,T,h,p) and, for the Mamba-3 variant, raw_angles
    (b,T,h,n/2) and lam (b,T,h) fp32.
    """
    if seed is None:
        seed = 1000 + cfg.index
    g = torch.Generator().manual_seed(seed + 7919 * rank)
    b, T, h, p, n, ng = cfg.batch, cfg.seqlen, cfg.nheads, cfg.headdim, cfg.d_state, cfg.ngroups
    store = torch.bfloat16 if cfg.dtype == "bf16" else torch.float32

    def randn(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float32)

    def rand(*shape):
        return torch.rand(*shape, generator=g, dtype=torch.float32)

    x = randn(b, T, h, p)
    dt = torch.nn.functional.softplus(0.5 * randn(b, T, h) + DT_BIAS0).clamp_(1e-3, 1e-1)
    A_head = -torch.exp(rand(h) * math.log(16.0))
    B = randn(b, T, ng, n) / math.sqrt(n)
    C = randn(b, T, ng, n) / math.sqrt(n)
    D = randn(h)
    dy = randn(b, T, h, p)
    out = {
        "x": x.to(store), "dt": dt, "A_head": A_head, "B": B.to(store), "C": C.to(store),
        "D": D, "dy": dy.to(store),
    }
    if cfg.mamba3:
        ang = (rand(b, T, h, n // 2) * 2 - 1) * math.pi * torch.sigmoid(randn(b, T, h, n // 2))
        out["raw_angles"] = ang.to(store)
        out["lam"] = torch.sigmoid(randn(b, T, h))
    return {k: v.to(device) for k, v in out.items()}


def make_reference_test_inputs(b: int, seqlen: int, n_heads: int, d_head: int, d_state: int,
                               dtype: torch.dtype = torch.float32, seed: int = 0) -> tuple[torch.Tensor, ...]:
    """Inputs with the value ranges the reference's own scan tests use
    (tests/kernels/test_ssd_scan.py:31-39): x, B, C ~ 0.5*N(0,1), A = -0.1*U(0,1).
    Drawn on CPU so that the oracle and the GPU path see identical numbers."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(b, seqlen, n_heads, d_head, generator=g) * 0.5
    A = -torch.rand(b, seqlen, n_heads, generator=g) * 0.1
    B = torch.randn(b, seqlen, n_heads, d_state, generator=g) * 0.5
    C = torch.randn(b, seqlen, n_heads, d_state, generator=g) * 0.5
    return tuple(t.to(dtype) for t in (x, A, B, C))


def kernel_algorithmic_bytes(cfg: SSDConfig) -> dict[str, int]:
    """Algorithmic HBM bytes ONE launch of each kernel moves for this workload: the operator inputs it
    must read and the operator outputs it must write, each once at storage width.  Intermediates
    (chunk states, cumulative decays, partial sums) count zero, so a kernel that re-reads or spills
    shows up as a lower achieved bandwidth.  The backward of the tensor-core path is two kernels that both
    need dy and C (the reverse walk for the state gradients, the tile kernel for everything else): each is
    charged what it must read itself, so those two add up to `ex + eb` more than the backward's share of
    ``bytes_per_token``; whole-step figures always use ``bytes_per_token``."""
    w = 2 if cfg.dtype == "bf16" else 4
    ex = cfg.nheads * cfg.headdim * w
    eb = cfg.ngroups * cfg.d_state * w
    edt = cfg.nheads * 4
    tok = cfg.tokens
    per_token = {
        "chunk_cumsum": edt,
        "chunk_state": ex + eb + edt,
        "chunk_scan": 2 * ex + 2 * eb + edt,
        "chunk_dstate": ex + eb,
        "bwd_row": 2 * ex + 3 * eb,
        "bwd_col": 3 * ex + 3 * eb + edt,
        "decay_grad": 2 * edt,
        "tc_fwd_walk": 2 * ex + 2 * eb + edt,
        "tc_bwd_state": ex + eb,
        "tc_summary": ex + eb,
        "tc_bwd_walk": 3 * ex + 4 * eb + 2 * edt,
    }
    return {k: v * tok for k, v in per_token.items()}
