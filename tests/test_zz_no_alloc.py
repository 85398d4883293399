"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Collected last (file name) so that it also runs after every other GPU test has used the library.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else None)


def _inputs(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)   # noqa: E731
    h, dy, dres = mk(rows, cols), mk(rows, cols), mk(rows, cols)
    w = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).to(torch.bfloat16)
    rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-5)
    return dy, h, w, rstd, dres


def _call_static(L, dy, h, w, rstd, dres, accumulate=False, dw=None):
    from easyllm_b200.ops import cuda as cu
    rows, cols = h.shape
    dh = torch.empty_like(h)
    dw = dw if dw is not None else torch.empty(cols, dtype=torch.float32, device="cuda")
    fn = L.ell_rmsnorm_bwd_static
    fn.restype = ctypes.c_int
    rc = fn(_ptr(dy), _ptr(h), _ptr(w), _ptr(rstd), _ptr(dres), _ptr(dh), _ptr(dw), ctypes.c_int(rows),
            ctypes.c_int(cols), ctypes.c_int(1 if accumulate else 0), cu._stream())
    return rc, dh, dw


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (777, 1024), (3000, 8192)])
def test_static_scratch_matches_regular_entry(rows, cols):
    from easyllm_b200.ops import cuda as cu
    L = cu.lib()
    L.ell_static_strerror.restype = ctypes.c_char_p
    # two calls in a row with different data: the second must not see the first one's partials
    for seed, with_res in ((1, True), (2, False)):
        dy, h, w, rstd, dres = _inputs(rows, cols, seed)
        dres = dres if with_res else None
        rc, dh, dw = _call_static(L, dy, h, w, rstd, dres)
        assert rc == 0, L.ell_static_strerror(rc).decode()
        dh_ref, dw_ref = cu.rmsnorm_bwd(dy, h, w, rstd, dres)
        torch.cuda.synchronize()
        torch.testing.assert_close(dh.float(), dh_ref.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(dw, dw_ref, rtol=2e-3, atol=2e-2 * (rows ** 0.5) / 8)
        # and against plain fp32 math
        xh = h.float() * rstd[:, None]
        gg = dy.float() * w.float()
        ref = rstd[:, None] * (gg - xh * (gg * xh).mean(-1, keepdim=True))
        if dres is not None:
            ref = ref + dres.float()
        torch.testing.assert_close(dh.float(), ref, rtol=3e-2, atol=3e-2)
        torch.testing.assert_close(dw, (dy.float() * xh).sum(0), rtol=2e-3, atol=2e-2 * (rows ** 0.5) / 8)


def test_static_scratch_accumulates_and_rejects_oversize():
    from easyllm_b200.ops import cuda as cu
    L = cu.lib()
    L.ell_static_strerror.restype = ctypes.c_char_p
    dy, h, w, rstd, _ = _inputs(512, 2048, 5)
    base = torch.full((2048,), 3.0, device="cuda")
    rc, _, dw = _call_static(L, dy, h, w, rstd, None, accumulate=True, dw=base.clone())
    assert rc == 0
    _, dw_ref = cu.rmsnorm_bwd(dy, h, w, rstd, None)
    torch.testing.assert_close(dw, dw_ref + 3.0, rtol=2e-3, atol=5e-2)
    # beyond the fixed scratch: refused before anything is launched
    big = torch.empty(8, 8192 + 8, device="cuda", dtype=torch.bfloat16)
    rc, _, _ = _call_static(L, big, big, big[0], torch.empty(8, device="cuda"), None)
    assert rc == -2 and b"exceeds" in L.ell_static_strerror(rc)
    odd = torch.empty(8, 100, device="cuda", dtype=torch.bfloat16)
    rc, _, _ = _call_static(L, odd, odd, odd[0], torch.empty(8, device="cuda"), None)
    assert rc == -1
