"""CPU tests of the oracle itself: against outputs of the reference stored as golden fixtures
(tests/golden/ref_*.npz, written by oracle/pin_against_reference.py from the imported reference),
against the reference's own stored golden vectors (tests/golden/ces_*.npz, headdim-1 form) and
against the step-by-step recurrence."""
import glob

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import GOLDEN, load_golden, rel_err

REF_CASES = sorted(p.split("/")[-1] for p in glob.glob(str(GOLDEN / "ref_*.npz")))
CES_CASES = sorted(p.split("/")[-1] for p in glob.glob(str(GOLDEN / "ces_*.npz")))


def _t(a):
    return torch.from_numpy(np.asarray(a))


def test_fixtures_present():
    assert len(REF_CASES) == 4 and len(CES_CASES) == 3


@pytest.mark.parametrize("name", REF_CASES)
def test_oracle_reproduces_reference_outputs(oracle, name):
    g = load_golden(name)
    chunk = int(g["chunk"])
    leaves = [_t(g[k]).clone().requires_grad_(True) for k in ("x", "A", "B", "C")]
    init = _t(g["init"]).clone().requires_grad_(True) if g["init"].size else None
    Y, fs, cache = oracle.fused_ssd_scan_oracle(*leaves, chunk, init)
    assert rel_err(Y, _t(g["Y"])) < 1e-6
    assert rel_err(fs, _t(g["final_state"])) < 1e-6
    assert rel_err(cache["A_cumsum"], _t(g["A_cumsum"])) < 1e-6
    outs, gouts = [Y], [_t(g["dY"])]
    if g["dfinal"].size:
        outs.append(fs)
        gouts.append(_t(g["dfinal"]))
    ins = leaves + ([init] if init is not None else [])
    grads = torch.autograd.grad(outs, ins, gouts)
    for k, gr in zip(("dx", "dA", "dB", "dC", "dinit"), grads):
        assert rel_err(gr, _t(g[k])) < 1e-5, k
    # cached second call: decay gradient is dropped, as in the reference
    l2 = [_t(g[k]).clone().requires_grad_(True) for k in ("x2", "A", "B2", "C")]
    Y2, _, _ = oracle.fused_ssd_scan_oracle(*l2, chunk, None, cache)
    assert rel_err(Y2, _t(g["Y_cached"])) < 1e-6
    g2 = torch.autograd.grad([Y2], l2, [_t(g["dY"])], allow_unused=True)
    assert g2[1] is None and float(np.abs(g["dA_cached"]).max()) == 0.0
    assert rel_err(g2[0], _t(g["dx_cached"])) < 1e-5


@pytest.mark.parametrize("name", CES_CASES)
def test_oracle_reproduces_stored_golden_vectors(oracle, name):
    """The reference's stored vectors are the headdim-1 Mamba-2 form: X = x*softplus(dt+bias), a = dt*A."""
    g = load_golden(name)
    x, A, B, C, D = (_t(g[k]) for k in ("x", "A", "B", "C", "D"))
    dt = F.softplus(_t(g["dt"]) + _t(g["dt_bias"]))
    expected = _t(g["expected_y"])
    Y, _, _ = oracle.ssd_chunked((x * dt).unsqueeze(-1), dt * A, B, C, 64)
    assert rel_err(Y[..., 0] + D * x, expected) < 1e-5
    Ys, _ = oracle.ssd_recurrence((x * dt).unsqueeze(-1), dt * A, B, C)
    assert rel_err(Ys[..., 0] + D.double() * x.double(), expected) < 1e-5
    Ym, _ = oracle.mamba2_operator(x.unsqueeze(-1), dt, A, B, C, D, 32)
    assert rel_err(Ym[..., 0], expected) < 1e-5


def test_chunked_equals_recurrence_and_sequence_split(oracle, pkg):
    cfg = pkg.shrink(pkg.CONFIGS[0], batch=1, seqlen=256)
    inp = pkg.make_inputs(cfg)
    h = cfg.nheads
    X = inp["x"] * inp["dt"].unsqueeze(-1)
    a = inp["dt"] * inp["A_head"]
    Bh, Ch = oracle.expand_groups(inp["B"], h), oracle.expand_groups(inp["C"], h)
    Y, fs, _ = oracle.ssd_chunked(X, a, Bh, Ch, cfg.chunk)
    Ys, Hs = oracle.ssd_recurrence(X, a, Bh, Ch)
    assert rel_err(Y, Ys) < 1e-5 and rel_err(fs, Hs) < 1e-5
    # halves chained through initial_states / final_state reproduce the full run
    Y1, f1, _ = oracle.ssd_chunked(X[:, :128], a[:, :128], Bh[:, :128], Ch[:, :128], cfg.chunk)
    Y2, f2, _ = oracle.ssd_chunked(X[:, 128:], a[:, 128:], Bh[:, 128:], Ch[:, 128:], cfg.chunk, f1.unsqueeze(1))
    assert rel_err(torch.cat([Y1, Y2], 1), Y) < 1e-5 and rel_err(f2, fs) < 1e-5


def test_oracle_rejects_ragged_sequence(oracle):
    x = torch.zeros(1, 100, 2, 4)
    with pytest.raises(AssertionError, match="not divisible"):
        oracle.ssd_chunked(x, torch.zeros(1, 100, 2), torch.zeros(1, 100, 2, 4), torch.zeros(1, 100, 2, 4), 64)


def test_workload_distributions(pkg):
    cfg = pkg.shrink(pkg.CONFIGS[2], batch=1, seqlen=256)
    inp = pkg.make_inputs(cfg)
    assert inp["x"].dtype == torch.bfloat16 and inp["dt"].dtype == torch.float32
    assert inp["B"].shape == (1, 256, 8, 128) and inp["x"].shape == (1, 256, 64, 64)
    assert 0.999e-3 <= float(inp["dt"].min()) and float(inp["dt"].max()) <= 1.001e-1
    assert -16.0 <= float(inp["A_head"].min()) and float(inp["A_head"].max()) <= -1.0
    again = pkg.make_inputs(cfg)
    assert all(torch.equal(inp[k], again[k]) for k in inp)
    assert pkg.CONFIGS[2].bytes_per_token() == 54016 and pkg.CONFIGS[1].bytes_per_token() == 17184
    assert pkg.CONFIGS[2].flops_per_token() == 10485760 and pkg.CONFIGS[1].flops_per_token() == 3014656
    assert pkg.CONFIGS[3].bytes_per_token() == 79360 and pkg.CONFIGS[3].flops_per_token() == 17825792


def test_mamba3_two_call_equals_two_term_recurrence(oracle, pkg):
    """The trapezoidal two-call composition equals H_t = e^{a_t} H_{t-1} + g_t x_t B_t + b_t x_{t-1} B_{t-1}."""
    from dataclasses import replace
    cfg = replace(pkg.shrink(pkg.CONFIGS[3], batch=1, seqlen=64), nheads=4, ngroups=2, d_state=16, headdim=8,
                  chunk=32, dtype="fp32")
    inp = {k: v.double() for k, v in pkg.make_inputs(cfg).items()}
    y = oracle.mamba3_operator(inp["x"], inp["dt"], inp["A_head"], inp["B"], inp["C"], inp["D"], inp["raw_angles"],
                               inp["lam"], cfg.chunk)
    h = cfg.nheads
    dA = inp["dt"] * inp["A_head"]
    gam, bet = inp["lam"] * inp["dt"], (1 - inp["lam"]) * inp["dt"] * torch.exp(dA)
    cum = -torch.cumsum(inp["raw_angles"], 1)
    Br = oracle.apply_rope(oracle.expand_groups(inp["B"], h), cum)
    Cr = oracle.apply_rope(oracle.expand_groups(inp["C"], h), cum)
    H = torch.zeros(1, h, cfg.headdim, cfg.d_state, dtype=torch.float64)
    ys = []
    for t in range(cfg.seqlen):
        H = torch.exp(dA[:, t])[..., None, None] * H + gam[:, t, :, None, None] * inp["x"][:, t, :, :, None] * Br[:, t, :, None, :]
        if t > 0:
            H = H + bet[:, t, :, None, None] * inp["x"][:, t - 1, :, :, None] * Br[:, t - 1, :, None, :]
        ys.append(torch.einsum("bhpn,bhn->bhp", H, Cr[:, t]) + inp["D"][None, :, None] * inp["x"][:, t])
    assert rel_err(y, torch.stack(ys, 1)) < 1e-6


def test_oracle_reproduces_reference_mamba3_composition(oracle):
    """The block's two-call composition built from the reference's own pieces (its tests' eager rotation and
    coefficients, its scan with the second call on the first call's cache), stored by
    oracle/pin_against_reference.py.  d dt is not compared: the reference's cached call drops its decay gradient."""
    g = load_golden("m3_reference_block.npz")
    t = {k: torch.as_tensor(v) for k, v in g.items() if k != "chunk"}
    names = ("x", "dt", "A_head", "B", "C", "D", "raw_angles", "lam")
    lv = {k: t[k].clone().requires_grad_(True) for k in names}
    y = oracle.mamba3_operator(*[lv[k] for k in names], int(g["chunk"]))
    gr = dict(zip(names, torch.autograd.grad([y], list(lv.values()), [t["dY"]])))
    assert rel_err(y, t["Y"]) < 1e-6
    for k, ref in (("x", "dx"), ("lam", "dlam"), ("B", "dB"), ("C", "dC"), ("raw_angles", "d_raw_angles")):
        assert rel_err(gr[k], t[ref]) < 1e-5, k
