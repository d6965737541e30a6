"""The forward entry point that brings its own scratch memory (ssd_b200_fwd_static_scratch).

It exists for hosts that have no way to allocate device memory themselves and therefore cannot pass the
workspace the normal forward wants: here the library uses a fixed 64 MiB array inside its own device
code instead.  The test drives both entry points through the C ABI with ctypes and requires the new one
to reproduce the normal one, twice in a row with different inputs (the array is shared between calls and
keeps the previous call's contents, so the second call must not see anything stale).  The file name
sorts last so that it is collected after every other test."""
import ctypes as C

import pytest
import torch

from conftest import TOL_BF16, TOL_FP32, rel_err


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _forward(cabi, pkg, entry, cfg, inp, use_workspace):
    lib = cabi.load()
    dev = torch.device("cuda", 0)
    x, dt, Ah, B, Cm, D = (inp[k].to(dev).contiguous() for k in ("x", "dt", "A_head", "B", "C", "D"))
    b, T, h, p = x.shape
    n = B.shape[3]
    shape = cabi.Shape(cabi.ABI_VERSION, cabi.BF16 if x.dtype == torch.bfloat16 else cabi.F32, cabi.F32,
                       cabi.PATH_AUTO, b, T, h, p, n, B.shape[2], cfg.chunk)
    y = torch.empty_like(x)
    final = torch.empty(b, h, p, n, dtype=torch.float32, device=dev)
    cum = torch.empty(b, h, T // cfg.chunk, cfg.chunk, dtype=torch.float32, device=dev)
    ws = None
    if use_workspace:
        ws = torch.empty(lib.ssd_b200_workspace_bytes(C.byref(shape), cabi.PASS_FWD), dtype=torch.uint8, device=dev)
    args = cabi.FwdArgs(shape, _ptr(x), None, _ptr(dt), _ptr(Ah), _ptr(D), _ptr(B), _ptr(Cm), None, _ptr(y),
                        _ptr(final), _ptr(cum), 0, 0, _ptr(ws), 0 if ws is None else ws.numel(), None)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    cabi.check(getattr(lib, entry)(C.byref(args), stream))
    # bounded-wait status of the call: a NULL workspace asks about the library's own array
    cabi.check(lib.ssd_b200_device_status(C.byref(shape), _ptr(ws), stream))
    torch.cuda.synchronize(dev)
    return y.float().cpu(), final.cpu(), cum.cpu()


@pytest.mark.gpu
@pytest.mark.parametrize("idx,batch,seqlen,tol", [(0, 2, 512, TOL_FP32), (2, 2, 512, TOL_BF16)])
def test_static_scratch_forward_matches_workspace_forward(pkg, cabi, idx, batch, seqlen, tol):
    cfg = pkg.shrink(pkg.CONFIGS[idx], batch, seqlen)
    for seed in (31, 32):  # two calls in a row on the shared array, different data each time
        inp = pkg.make_inputs(cfg, seed=seed)
        want = _forward(cabi, pkg, "ssd_b200_fwd", cfg, inp, use_workspace=True)
        got = _forward(cabi, pkg, "ssd_b200_fwd_static_scratch", cfg, inp, use_workspace=False)
        for name, a, b in zip(("y", "final_state", "a_cumsum"), got, want):
            assert rel_err(a, b) < tol, (cfg.name, seed, name)


def test_static_scratch_refuses_shapes_beyond_its_array(cabi):
    """Host-side check, needs no GPU: the full 1.3B-layer batch needs ~33.6 MB and fits, a 4x longer one does not."""
    lib = cabi.load()
    limit = lib.ssd_b200_static_scratch_bytes()
    assert limit == 64 << 20
    big = cabi.Shape(cabi.ABI_VERSION, cabi.BF16, cabi.F32, cabi.PATH_AUTO, 16, 4 * 4096, 64, 64, 128, 8, 128)
    assert lib.ssd_b200_workspace_bytes(C.byref(big), cabi.PASS_FWD) > limit
    args = cabi.FwdArgs(shape=big)
    assert lib.ssd_b200_fwd_static_scratch(C.byref(args), None) == cabi.EWORKSPACE
    msg = cabi.last_error()
    assert "built-in array" in msg and str(limit) in msg
