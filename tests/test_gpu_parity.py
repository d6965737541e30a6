"""GPU parity tests: the CUDA path, called through the C ABI by the operator, against the CPU oracle
and the golden fixtures.  Metric: max|a-b| / max|b| per output tensor; bars: 1e-4 for fp32,
2e-2 for bf16 inputs with fp32 accumulation (the oracle then runs in fp32 on the bf16-rounded inputs,
as the reference's own bf16 test does, tests/kernels/test_ssd_scan.py:74-96)."""
import glob
from dataclasses import replace

import numpy as np
import pytest
import torch

from conftest import GOLDEN, TOL_BF16, TOL_FP32, load_golden, rel_err

pytestmark = pytest.mark.gpu

DEV = "cuda"
REF_CASES = sorted(p.split("/")[-1] for p in glob.glob(str(GOLDEN / "ref_*.npz")))


def _t(a, dtype=None):
    t = torch.from_numpy(np.asarray(a))
    return t if dtype is None else t.to(dtype)


def run_operator(pkg, x, A, B, C, chunk, init=None, dY=None, dfinal=None, cache=None):
    """fused_ssd_scan forward + backward on the GPU; returns CPU tensors."""
    leaves = [t.detach().to(DEV).requires_grad_(True) for t in (x, A, B, C)]
    il = init.detach().to(DEV).requires_grad_(True) if init is not None else None
    Y, fs, ch = pkg.fused_ssd_scan(*leaves, chunk, il, cache)
    res = {"Y": Y.detach().cpu(), "final": fs.detach().cpu(), "cache": ch}
    if dY is not None:
        outs, gouts = [Y], [dY.to(DEV).to(Y.dtype)]
        if dfinal is not None:
            outs.append(fs)
            gouts.append(dfinal.to(DEV).to(fs.dtype))
        ins = leaves + ([il] if il is not None else [])
        grads = torch.autograd.grad(outs, ins, gouts, allow_unused=True)
        for k, g in zip(("dx", "dA", "dB", "dC", "dinit"), grads):
            res[k] = None if g is None else g.detach().cpu()
    torch.cuda.synchronize()
    return res


@pytest.mark.parametrize("name", REF_CASES)
def test_fp32_against_reference_fixtures(pkg, cabi, name):
    g = load_golden(name)
    chunk = int(g["chunk"])
    init = _t(g["init"]) if g["init"].size else None
    dfinal = _t(g["dfinal"]) if g["dfinal"].size else None
    r = run_operator(pkg, _t(g["x"]), _t(g["A"]), _t(g["B"]), _t(g["C"]), chunk, init, _t(g["dY"]), dfinal)
    assert rel_err(r["Y"], _t(g["Y"])) < TOL_FP32
    assert rel_err(r["final"], _t(g["final_state"])) < TOL_FP32
    assert rel_err(r["cache"]["A_cumsum"], _t(g["A_cumsum"])) < TOL_FP32
    for k in ("dx", "dA", "dB", "dC"):
        assert rel_err(r[k], _t(g[k])) < TOL_FP32, k
    if init is not None:
        assert rel_err(r["dinit"], _t(g["dinit"])) < TOL_FP32
    # cached second call (the caller's beta path): same A and C, shifted x and B; no decay gradient
    r2 = run_operator(pkg, _t(g["x2"]), _t(g["A"]), _t(g["B2"]), _t(g["C"]), chunk, None, _t(g["dY"]), None,
                      cache=r["cache"])
    assert rel_err(r2["Y"], _t(g["Y_cached"])) < TOL_FP32
    assert r2["dA"] is None
    for k in ("dx", "dB", "dC"):
        assert rel_err(r2[k], _t(g[k + "_cached"])) < TOL_FP32, k


@pytest.mark.parametrize("shape", [(2, 512, 4, 32, 8), (2, 256, 4, 16, 8), (1, 1024, 4, 16, 8), (2, 512, 8, 32, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reference_test_shapes(pkg, cabi, oracle, shape, dtype):
    """Shapes, value ranges and chunk size of the reference's own scan tests
    (tests/kernels/test_ssd_scan.py:31-52), forward and gradients."""
    b, T, h, p, n = shape
    x, A, B, C = pkg.make_reference_test_inputs(b, T, h, p, n, dtype, seed=0)
    gen = torch.Generator().manual_seed(5)
    dY = torch.randn(b, T, h, p, generator=gen).to(dtype)
    r = run_operator(pkg, x, A, B, C, 128, None, dY)
    lv = [t.float().requires_grad_(True) for t in (x, A, B, C)]
    Yo, fo, co = oracle.ssd_chunked(*lv, 128)
    go = torch.autograd.grad([Yo], lv, [dY.float()])
    tol = TOL_FP32 if dtype == torch.float32 else TOL_BF16
    assert r["Y"].dtype == dtype and r["final"].dtype == dtype
    assert rel_err(r["Y"], Yo) < tol and rel_err(r["final"], fo) < tol
    for k, g in zip(("dx", "dA", "dB", "dC"), go):
        assert rel_err(r[k], g) < tol, k
    # cache contract: keys and shapes (tests/kernels/test_ssd_scan.py:99-110), values as the reference builds them
    c = T // 128
    cache = r["cache"]
    assert set(cache.keys()) == {"L", "decay_chunk", "A_cumsum"}
    assert cache["A_cumsum"].shape == (b, h, c, 128)
    assert cache["L"].shape == (b, h, c, 128, 128) and cache["decay_chunk"].shape == (b, h, c + 1, c + 1)
    assert rel_err(cache["L"], co["L"]) < tol and rel_err(cache["decay_chunk"], co["decay_chunk"]) < tol


def mamba2_gpu(pkg, inp, chunk, init=None, dfinal=None):
    leaves = {k: inp[k].detach().to(DEV).requires_grad_(True) for k in ("x", "dt", "A_head", "B", "C", "D")}
    il = init.detach().to(DEV).requires_grad_(True) if init is not None else None
    y, fs = pkg.ssd_mamba2(leaves["x"], leaves["dt"], leaves["A_head"], leaves["B"], leaves["C"], leaves["D"], chunk, il)
    outs, gouts = [y], [inp["dy"].to(DEV)]
    if dfinal is not None:
        outs.append(fs)
        gouts.append(dfinal.to(DEV))
    ins = list(leaves.values()) + ([il] if il is not None else [])
    grads = torch.autograd.grad(outs, ins, gouts)
    res = {"y": y.detach().cpu(), "final_state": fs.detach().cpu()}
    for k, g in zip(list(leaves.keys()) + (["init"] if il is not None else []), grads):
        res["d" + k] = g.detach().cpu()
    torch.cuda.synchronize()
    return res


def check_mamba2(pkg, oracle, cfg, tol, init=False, dfinal=False, seed=None):
    inp = pkg.make_inputs(cfg, seed=seed)
    g = torch.Generator().manual_seed(77)
    i0 = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g) * 0.2 if init else None
    df = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g) if dfinal else None
    got = mamba2_gpu(pkg, inp, cfg.chunk, i0, df)
    want = oracle.mamba2_fwd_bwd(inp, cfg.chunk, torch.float32, None if i0 is None else i0.unsqueeze(1), df)
    errs = {k: rel_err(got[k], want[k].reshape(got[k].shape)) for k in got}
    bad = {k: v for k, v in errs.items() if not v < tol}
    assert not bad, (cfg.name, errs)
    return errs


def test_config0_fp32_full_size(pkg, cabi, oracle):
    check_mamba2(pkg, oracle, pkg.CONFIGS[0], TOL_FP32)


def test_config0_fp32_with_states(pkg, cabi, oracle):
    check_mamba2(pkg, oracle, pkg.CONFIGS[0], TOL_FP32, init=True, dfinal=True)


@pytest.mark.parametrize("path", ["simt", "tc"])
@pytest.mark.parametrize("idx,batch,seqlen", [(1, 2, 512), (2, 1, 512), (2, 2, 256)])
def test_bf16_config_shapes_reduced(pkg, cabi, oracle, idx, batch, seqlen, path):
    """Per-token shapes of the bf16 benchmark configurations at oracle-sized batch / sequence."""
    pkg.set_kernel_path(path)
    try:
        check_mamba2(pkg, oracle, pkg.shrink(pkg.CONFIGS[idx], batch, seqlen), TOL_BF16, init=(batch == 2),
                     dfinal=(batch == 2))
    finally:
        pkg.set_kernel_path("auto")


@pytest.mark.parametrize("heads,groups,batch", [(16, 2, 4), (6, 2, 4), (4, 4, 2)])
def test_tensor_core_path_with_several_items_per_cta(pkg, cabi, oracle, heads, groups, batch):
    """The backward tile kernel is persistent: with more (tile, group, batch) items than the GPU has SMs some CTAs
    process two items in a row.  8, 3 and 1 heads per group: the buffer indices and mbarrier phases carried from
    one item to the next start even, odd, and alternate every item."""
    seqlen = 128 * 20
    cfg = replace(pkg.shrink(pkg.CONFIGS[2], batch, seqlen), nheads=heads, ngroups=groups)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert (seqlen // 128) * groups * batch > sms
    assert pkg.resolved_path_name(cfg) == "tc"
    check_mamba2(pkg, oracle, cfg, TOL_BF16, init=True, dfinal=True, seed=21)


@pytest.mark.parametrize("batch,seqlen,heads,groups", [(1, 128, 3, 1), (2, 256, 3, 1), (1, 128, 1, 1), (3, 384, 5, 5),
                                                       (1, 512, 6, 2), (2, 128, 9, 3), (5, 256, 7, 1), (1, 1024, 10, 2)])
@pytest.mark.parametrize("states", [False, True])
def test_tensor_core_path_edge_shapes(pkg, cabi, oracle, batch, seqlen, heads, groups, states):
    """Shapes at the edges of the tensor-core kernels' bookkeeping: one tile per sequence, one head, an odd number of
    heads per group (the double-buffered x / dy tiles and the mbarrier phases of the backward tile kernel then start an
    item on either parity, and the reverse walk runs one head per CTA), fewer work items than SMs."""
    cfg = replace(pkg.shrink(pkg.CONFIGS[2], batch, seqlen), nheads=heads, ngroups=groups)
    assert pkg.resolved_path_name(cfg) == "tc"
    check_mamba2(pkg, oracle, cfg, TOL_BF16, init=states, dfinal=states, seed=33)


@pytest.mark.parametrize("h,p,n,g,l,T", [(3, 24, 12, 1, 32, 96), (4, 80, 40, 2, 48, 96), (6, 16, 72, 3, 100, 200),
                                         (2, 128, 130, 1, 64, 64), (2, 8, 8, 2, 16, 16)])
def test_ragged_shapes_fp32(pkg, cabi, oracle, h, p, n, g, l, T):
    """Sizes that are not multiples of the 64-wide tiles, odd head/group counts, a single chunk."""
    cfg = replace(pkg.CONFIGS[0], batch=2, seqlen=T, nheads=h, headdim=p, d_state=n, ngroups=g, chunk=l)
    check_mamba2(pkg, oracle, cfg, TOL_FP32, init=True, dfinal=True, seed=4242)


def test_sequence_split_through_states(pkg, cabi, oracle):
    """Two halves chained through final_state -> initial_states reproduce the full run (fwd and grads)."""
    cfg = pkg.shrink(pkg.CONFIGS[0], batch=1, seqlen=256)
    inp = pkg.make_inputs(cfg)
    full = mamba2_gpu(pkg, inp, cfg.chunk)
    lo = {k: (v[:, :128] if v.dim() >= 3 else v) for k, v in inp.items()}
    hi = {k: (v[:, 128:] if v.dim() >= 3 else v) for k, v in inp.items()}
    first = mamba2_gpu(pkg, lo, cfg.chunk)
    second = mamba2_gpu(pkg, hi, cfg.chunk, init=first["final_state"])
    assert rel_err(torch.cat([first["y"], second["y"]], 1), full["y"]) < TOL_FP32
    assert rel_err(second["final_state"], full["final_state"]) < TOL_FP32
    # backward: the second half's d_init is the first half's dfinal
    first_b = mamba2_gpu(pkg, lo, cfg.chunk, dfinal=second["dinit"])
    assert rel_err(torch.cat([first_b["dx"], second["dx"]], 1), full["dx"]) < TOL_FP32
    assert rel_err(torch.cat([first_b["ddt"], second["ddt"]], 1), full["ddt"]) < TOL_FP32
    assert rel_err(first_b["dA_head"] + second["dA_head"], full["dA_head"]) < TOL_FP32


def test_error_behaviour_on_gpu(pkg, cabi):
    x = torch.zeros(1, 100, 2, 8, device=DEV)
    A = torch.zeros(1, 100, 2, device=DEV)
    B = torch.zeros(1, 100, 2, 4, device=DEV)
    with pytest.raises(AssertionError, match="not divisible"):
        pkg.fused_ssd_scan(x, A, B, B, 64)
    with pytest.raises(RuntimeError, match="same dtype"):
        pkg.fused_ssd_scan(x[:, :64], A[:, :64], B[:, :64].bfloat16(), B[:, :64], 64)


def test_noncontiguous_inputs_and_determinism(pkg, cabi):
    """The caller passes products and padded views (src/mamba_base_engine.py:170-181); results are
    bitwise reproducible run to run."""
    x, A, B, C = pkg.make_reference_test_inputs(2, 256, 4, 16, 8, torch.float32, seed=3)
    xv = torch.cat([x, x], -1).to(DEV)[..., :16]
    Bv = B.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)
    assert not xv.is_contiguous() and not Bv.is_contiguous()
    outs = []
    for _ in range(2):
        xl = xv.detach().requires_grad_(True)
        Al = A.to(DEV).requires_grad_(True)
        Y, fs, _ = pkg.fused_ssd_scan(xl, Al, Bv, C.to(DEV), 128)
        gx, gA = torch.autograd.grad([Y], [xl, Al], [torch.ones_like(Y)])
        outs.append((Y, fs, gx, gA))
    Yc, fc, _ = pkg.fused_ssd_scan(x.to(DEV), A.to(DEV), B.to(DEV), C.to(DEV), 128)
    assert torch.equal(outs[0][0], Yc) and torch.equal(outs[0][1], fc)
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("chunk", [64, 128, 256])
@pytest.mark.parametrize("a_dtype", [torch.bfloat16, torch.float32])
def test_tensor_core_path_operator_form(pkg, cabi, oracle, chunk, a_dtype):
    """fused_ssd_scan on the tcgen05 kernels (one head per group, as the reference caller uses it):
    forward, all gradients, initial/final state, and the cached second call."""
    b, T, h, p, n = 2, 512, 3, 64, 128
    x, A, B, C = pkg.make_reference_test_inputs(b, T, h, p, n, torch.bfloat16, seed=11)
    A = (A.float() * 3.0).to(a_dtype)
    gen = torch.Generator().manual_seed(12)
    dY = torch.randn(b, T, h, p, generator=gen).bfloat16()
    init = (torch.randn(b, 1, h, p, n, generator=gen) * 0.3).bfloat16()
    dfinal = torch.randn(b, h, p, n, generator=gen).bfloat16()
    pkg.set_kernel_path("tc")
    try:
        r = run_operator(pkg, x, A, B, C, chunk, init, dY, dfinal)
        x2 = torch.nn.functional.pad(x[:, :-1], (0, 0, 0, 0, 1, 0))
        B2 = torch.nn.functional.pad(B[:, :-1], (0, 0, 0, 0, 1, 0))
        r2 = run_operator(pkg, x2, A, B2, C, chunk, None, dY, None, cache=r["cache"])
    finally:
        pkg.set_kernel_path("auto")
    lv = [t.float().requires_grad_(True) for t in (x, A, B, C)]
    il = init.float().requires_grad_(True)
    Yo, fo, co = oracle.ssd_chunked(*lv, chunk, il)
    go = torch.autograd.grad([Yo, fo], lv + [il], [dY.float(), dfinal.float()])
    errs = {"Y": rel_err(r["Y"], Yo), "final": rel_err(r["final"], fo)}
    for k, g in zip(("dx", "dA", "dB", "dC", "dinit"), go):
        errs[k] = rel_err(r[k], g)
    l2 = [t.float().requires_grad_(True) for t in (x2, A, B2, C)]
    Y2, _, _ = oracle.fused_ssd_scan_oracle(*l2, chunk, None, co)
    g2 = torch.autograd.grad([Y2], [l2[0], l2[2], l2[3]], [dY.float()])
    errs["Y_cached"] = rel_err(r2["Y"], Y2)
    for k, g in zip(("dx", "dB", "dC"), g2):
        errs[k + "_cached"] = rel_err(r2[k], g)
    assert r2["dA"] is None
    bad = {k: v for k, v in errs.items() if not v < TOL_BF16}
    assert not bad, errs


def test_tensor_core_path_is_deterministic_and_selected(pkg, cabi):
    cfg = pkg.shrink(pkg.CONFIGS[2], 2, 512)
    assert pkg.resolved_path_name(cfg) == "tc"
    assert pkg.resolved_path_name(pkg.CONFIGS[0]) == "simt"
    inp = pkg.make_inputs(cfg)
    a = mamba2_gpu(pkg, inp, cfg.chunk)
    b = mamba2_gpu(pkg, inp, cfg.chunk)
    for k in a:
        assert torch.equal(a[k], b[k]), k


def test_saved_states_equal_recomputed_states(pkg, cabi):
    """The backward gives the same gradients whether the forward kept its per-tile states or the
    backward recomputes them (the reference's input-only checkpointing)."""
    cfg = pkg.shrink(pkg.CONFIGS[2], 2, 512)
    inp = pkg.make_inputs(cfg)
    g = torch.Generator().manual_seed(9)
    init = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g) * 0.2
    kept = mamba2_gpu(pkg, inp, cfg.chunk, init)
    pkg.set_save_states(False)
    try:
        redone = mamba2_gpu(pkg, inp, cfg.chunk, init)
    finally:
        pkg.set_save_states(True)
    for k in kept:
        assert torch.equal(kept[k], redone[k]), k


def test_mamba3_variant_takes_fp32_angles_with_bf16_tensors(pkg, cabi, oracle):
    """Angles given in fp32 (the reference's fp32 dt * theta product) are summed at that precision although x, B and C
    are bf16; their gradient comes back in fp32."""
    cfg = pkg.shrink(pkg.CONFIGS[3], 1, 512)
    inp = pkg.make_inputs(cfg)
    g = torch.Generator().manual_seed(3)
    inp["raw_angles"] = (torch.rand(inp["raw_angles"].shape, generator=g) * 2 - 1) * 0.37   # not bf16-representable
    names = ("x", "dt", "A_head", "B", "C", "D", "raw_angles", "lam")
    lv = {k: inp[k].to(DEV).requires_grad_(True) for k in names}
    y = pkg.ssd_mamba3(*[lv[k] for k in names], cfg.chunk)
    grads = torch.autograd.grad([y], list(lv.values()), [inp["dy"].to(DEV)])
    torch.cuda.synchronize()
    assert grads[6].dtype == torch.float32
    ol = {k: inp[k].float().requires_grad_(True) for k in names}
    yo = oracle.mamba3_operator(*[ol[k] for k in names], cfg.chunk)
    go = torch.autograd.grad([yo], list(ol.values()), [inp["dy"].float()])
    errs = {"y": rel_err(y, yo)}
    for k, a, b in zip(names, grads, go):
        errs["d" + k] = rel_err(a, b)
    bad = {k: v for k, v in errs.items() if not v < TOL_BF16}
    assert not bad, errs


@pytest.mark.parametrize("dtype,tol", [("fp32", TOL_FP32), ("bf16", TOL_BF16)])
def test_mamba3_variant(pkg, cabi, oracle, dtype, tol):
    """Rotary state angles + trapezoidal two-term form (config 3 per-token shape, reduced batch / sequence)
    against the oracle's two-call composition under plain autograd, all gradients including d raw_angles, d lam."""
    cfg = replace(pkg.shrink(pkg.CONFIGS[3], 1, 256), dtype=dtype)
    inp = pkg.make_inputs(cfg)
    names = ("x", "dt", "A_head", "B", "C", "D", "raw_angles", "lam")
    lv = {k: inp[k].to(DEV).requires_grad_(True) for k in names}
    y = pkg.ssd_mamba3(*[lv[k] for k in names], cfg.chunk)
    grads = torch.autograd.grad([y], list(lv.values()), [inp["dy"].to(DEV)])
    torch.cuda.synchronize()
    ol = {k: inp[k].float().requires_grad_(True) for k in names}
    yo = oracle.mamba3_operator(*[ol[k] for k in names], cfg.chunk)
    go = torch.autograd.grad([yo], list(ol.values()), [inp["dy"].float()])
    errs = {"y": rel_err(y, yo)}
    for k, a, b in zip(names, grads, go):
        errs["d" + k] = rel_err(a, b)
    bad = {k: v for k, v in errs.items() if not v < tol}
    assert not bad, errs


def test_mamba3_against_reference_fixture(pkg, cabi):
    """The one-scan Mamba-3 form on the GPU against outputs of the reference's own two-call composition
    (tests/golden/m3_reference_block.npz: reference rotation convention, coefficients and scan), fp32."""
    g = load_golden("m3_reference_block.npz")
    t = {k: torch.as_tensor(v) for k, v in g.items() if k != "chunk"}
    names = ("x", "dt", "A_head", "B", "C", "D", "raw_angles", "lam")
    lv = {k: t[k].to(DEV).requires_grad_(True) for k in names}
    y = pkg.ssd_mamba3(*[lv[k] for k in names], int(g["chunk"]))
    gr = dict(zip(names, torch.autograd.grad([y], list(lv.values()), [t["dY"].to(DEV)])))
    torch.cuda.synchronize()
    errs = {"Y": rel_err(y, t["Y"])}
    for k, ref in (("x", "dx"), ("lam", "dlam"), ("B", "dB"), ("C", "dC"), ("raw_angles", "d_raw_angles")):
        errs[ref] = rel_err(gr[k], t[ref])
    bad = {k: v for k, v in errs.items() if not v < TOL_FP32}
    assert not bad, errs


def test_host_pipeline_matches_direct_call(pkg, cabi):
    """The host-buffer entry (micro-batches over three streams) returns what one call on device tensors returns."""
    cfg = pkg.shrink(pkg.CONFIGS[2], 4, 256)
    inp = pkg.make_inputs(cfg)
    pinned = {k: v.pin_memory() for k, v in inp.items()}
    out = pkg.HostPipeline.alloc_outputs(pinned)
    pipe = pkg.HostPipeline("cuda", micro_batches=2)
    for _ in range(2):  # twice: slot reuse across calls
        pipe.run(pinned, out, cfg.chunk)
    got = {k: v.clone() for k, v in out.items()}  # read by the CPU right after run() returned: no device synchronise
    want = mamba2_gpu(pkg, inp, cfg.chunk)
    for k in ("y", "dx", "ddt", "dB", "dC"):
        assert torch.equal(got[k], want[k]), k
    assert rel_err(got["dA_head"], want["dA_head"]) < 1e-5 and rel_err(got["dD"], want["dD"]) < 1e-5
    # the stream-ordered form: nothing may be read before the returned event has completed
    ev = pipe.run(pinned, out, cfg.chunk, wait=False)
    ev.synchronize()
    assert torch.equal(out["y"], want["y"])


@pytest.mark.parametrize("idx,batch,seqlen,slice_len", [(2, 1, 1024, 256), (2, 2, 512, 128), (0, 2, 512, 128)])
def test_sequence_streamer_is_exact_across_slices(pkg, cabi, idx, batch, seqlen, slice_len):
    """The sequence-sliced host runner (state carried from slice to slice, its gradient carried back) returns what
    one call over the whole sequence returns, within the rounding of one pass."""
    cfg = pkg.shrink(pkg.CONFIGS[idx], batch, seqlen)
    inp = pkg.make_inputs(cfg)
    pinned = {k: v.pin_memory() for k, v in inp.items()}
    out = pkg.HostPipeline.alloc_outputs(pinned)
    runner = pkg.SequenceStreamer("cuda", slice_len=slice_len)
    for _ in range(2):  # twice: slot reuse across calls
        runner.run(pinned, out, cfg.chunk)
    got = {k: v.clone() for k, v in out.items()}  # CPU read right after run() returned
    want = mamba2_gpu(pkg, inp, cfg.chunk)
    tol = TOL_BF16 if cfg.dtype == "bf16" else TOL_FP32
    errs = {k: rel_err(got[k], want[k]) for k in ("y", "dx", "ddt", "dB", "dC", "dA_head", "dD")}
    bad = {k: v for k, v in errs.items() if not v < tol}
    assert not bad, errs


@pytest.mark.parametrize("idx,batch,seqlen,tol", [(2, 2, 512, TOL_BF16), (1, 2, 256, TOL_BF16), (0, 2, 256, TOL_FP32)])
def test_scan_with_gated_norm_output_stage(pkg, cabi, oracle, idx, batch, seqlen, tol):
    """ssd_mamba2_gated = scan + the block's output stage norm(y) * silu(z) (src/mamba_base_engine.py:189-191): on the
    tensor-core path the norm takes its row statistic from the partial sums the forward walk leaves behind (config 2
    and 1 shapes); on the fp32 path it computes it itself.  Against the oracle scan followed by the eager norm."""
    cfg = pkg.shrink(pkg.CONFIGS[idx], batch, seqlen)
    inp = pkg.make_inputs(cfg)
    b, T, h, p = inp["x"].shape
    g = torch.Generator().manual_seed(123)
    z = torch.randn(b, T, h * p, generator=g).to(inp["x"].dtype)
    w = 1.0 + 0.1 * torch.randn(h * p, generator=g)
    dout = torch.randn(b, T, h, p, generator=g).to(inp["x"].dtype)
    names = ("x", "dt", "A_head", "B", "C", "D")
    lv = {k: inp[k].to(DEV).requires_grad_(True) for k in names}
    zl, wl = z.to(DEV).requires_grad_(True), w.to(DEV).requires_grad_(True)
    out, fs = pkg.ssd_mamba2_gated(lv["x"], lv["dt"], lv["A_head"], lv["B"], lv["C"], lv["D"], zl, wl, 1e-6, cfg.chunk)
    grads = torch.autograd.grad([out], list(lv.values()) + [zl, wl], [dout.to(DEV)])
    torch.cuda.synchronize()
    ol = {k: inp[k].float().requires_grad_(True) for k in names}
    zo, wo = z.float().requires_grad_(True), w.clone().requires_grad_(True)
    yo, fo = oracle.mamba2_operator(ol["x"], ol["dt"], ol["A_head"], ol["B"], ol["C"], ol["D"], cfg.chunk)
    yf = yo.reshape(b, T, h * p)
    oo = (yf * torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + 1e-6) * wo * torch.nn.functional.silu(zo)).reshape(b, T, h, p)
    go = torch.autograd.grad([oo], list(ol.values()) + [zo, wo], [dout.float()])
    errs = {"out": rel_err(out, oo), "final": rel_err(fs, fo)}
    for k, a, c in zip(list(names) + ["z", "w"], grads, go):
        errs["d" + k] = rel_err(a, c)
    bad = {k: v for k, v in errs.items() if not v < tol}
    assert not bad, errs
    # and equal to the two-call composition of this package (same kernels apart from where the statistic comes from)
    y2, _ = pkg.ssd_mamba2(lv["x"], lv["dt"], lv["A_head"], lv["B"], lv["C"], lv["D"], cfg.chunk)
    o2 = pkg.fused_gate_norm(y2.reshape(b, T, h * p), zl, wl, 1e-6).reshape(b, T, h, p)
    assert rel_err(out, o2) < (1e-2 if cfg.dtype == "bf16" else 1e-5)


def test_scaled_operator_form_matches_mamba2_form(pkg, cabi):
    """The scan's third calling form (log-decay a, input weight dt and skip coefficient all per position; what the
    one-scan Mamba-3 composition uses) against the Mamba-2 form with a = dt * A_head and skip = D on the same data:
    same y, dx, dB, dC, and  ddt = d weight + da * A_head,  dA_head = sum da * dt,  dD = sum dskip."""
    import importlib
    S = importlib.import_module("dhammic-ai_b200.ssd_scan")
    cfg = pkg.shrink(pkg.CONFIGS[2], 2, 512)
    inp = {k: v.to(DEV) for k, v in pkg.make_inputs(cfg).items()}
    want = mamba2_gpu(pkg, {k: v.cpu() for k, v in inp.items()}, cfg.chunk)
    b, T, h, p = inp["x"].shape
    a = (inp["dt"] * inp["A_head"]).contiguous()
    skip = inp["D"].expand(b, T, h).contiguous()
    y, final, cum, shape, states = S._run_fwd(inp["x"], a, inp["dt"], None, None, inp["B"], inp["C"], cfg.chunk, None, None,
                                             want_states=True, skip=skip)
    dx, da, dw, dskip, dB, dC = S._run_bwd_scaled(shape, inp["x"], a, inp["dt"], skip, inp["B"], inp["C"], cum, inp["dy"], states)
    torch.cuda.synchronize()
    got = {"y": y, "final_state": final, "dx": dx, "dB": dB, "dC": dC,
           "ddt": dw + da * inp["A_head"], "dA_head": (da * inp["dt"]).sum((0, 1)), "dD": dskip.sum((0, 1))}
    errs = {k: rel_err(got[k], want[k]) for k in got}
    bad = {k: v for k, v in errs.items() if not v < 1e-3}   # same kernels, same roundings up to the order of the sums
    assert not bad, errs


def test_unused_outputs_are_not_materialised(pkg, cabi):
    """The operators ask autograd not to build zero gradients for outputs the loss does not use: with only y used the
    backward runs without a final-state gradient (no seed for the reverse walk), with only the final state used it
    builds the zero dY itself.  Both must equal the calls with explicit zeros."""
    cfg = pkg.shrink(pkg.CONFIGS[2], 2, 512)
    inp = {k: v.to(DEV) for k, v in pkg.make_inputs(cfg).items()}
    names = ("x", "dt", "A_head", "B", "C", "D")

    def grads(use_y, use_final, explicit):
        lv = {k: inp[k].clone().requires_grad_(True) for k in names}
        y, fs = pkg.ssd_mamba2(*[lv[k] for k in names], cfg.chunk)
        gfs = torch.ones_like(fs) * 0.5
        if explicit:
            outs, gs = [y, fs], [inp["dy"] if use_y else torch.zeros_like(y), gfs if use_final else torch.zeros_like(fs)]
        else:
            outs, gs = ([y] if use_y else []) + ([fs] if use_final else []), ([inp["dy"]] if use_y else []) + ([gfs] if use_final else [])
        return torch.autograd.grad(outs, list(lv.values()), gs)

    for use_y, use_final in ((True, False), (False, True)):
        a, b = grads(use_y, use_final, False), grads(use_y, use_final, True)
        for name, u, v in zip(names, a, b):
            assert torch.equal(u, v), (use_y, use_final, name)
