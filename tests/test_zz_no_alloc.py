"""GroupNorm entry point with a built-in workspace: called through the exported C symbol, compared with the regular op.

Named so that it is collected after every other test file: the entry point has to work in a process where the library
has already done a lot of other work, and also when it is the first thing the process runs."""
import ctypes

import pytest
import torch

from mojodiffusion_b200.ops import native

pytestmark = pytest.mark.gpu

MAX_GROUPS = 8192
ERR_TOO_SMALL = -20


def _lib():
    native.load(True)
    lib = ctypes.CDLL(str(native.lib_path()))
    fn = lib.mdb_group_norm_static_ws
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    return fn


def _call(fn, x, w, b, groups, eps, act, check_free=True):
    y = torch.empty_like(x)                       # the caller owns inputs and outputs; the call allocates nothing
    N, H, W, C = x.shape
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = fn(x.data_ptr(), y.data_ptr(), w.data_ptr() if w is not None else None, b.data_ptr() if b is not None else None,
            N, H * W, C, groups, eps, act, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    # the driver's count of free device memory is the same before and after: nothing was allocated (or freed) by the call,
    # neither through a CUDA allocation call nor through a library pool
    if check_free:
        assert torch.cuda.mem_get_info()[0] == free_before, "the static-workspace entry point changed the amount of free device memory"
    return rc, y


def test_static_workspace_group_norm_matches_regular_op_twice():
    fn = _lib()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    G, eps = 32, 1e-6
    w = torch.randn(256, device=dev).bfloat16()
    b = torch.randn(256, device=dev).bfloat16()
    # One unchecked call first: the driver loads a kernel's code into device memory the first time the kernel is launched
    # (lazy module loading), which is not an allocation made by the entry point but would show up in the free-memory count.
    _call(fn, torch.zeros(1, 4, 4, 64, device=dev, dtype=torch.bfloat16), w[:64], b[:64], G, eps, 2, check_free=False)
    _call(fn, torch.zeros(1, 4, 4, 64, device=dev, dtype=torch.bfloat16), None, None, G, eps, 0, check_free=False)
    # two calls in a row with different shapes and data: the second must not see anything the first left behind
    for (N, H, W, C), act, ww, bb in (((3, 24, 40, 256), 2, w, b), ((2, 16, 16, 128), 0, None, None)):
        x = (torch.randn(N, H, W, C, device=dev) * 2 + 0.5).bfloat16()
        rc, y = _call(fn, x, ww[:C] if ww is not None else None, bb[:C] if bb is not None else None, G, eps, act)
        assert rc == 0
        ref = torch.ops.mdb200.group_norm_nhwc(x, ww[:C] if ww is not None else None, bb[:C] if bb is not None else None,
                                               G, eps, act)
        torch.cuda.synchronize()
        # the regular op may split a sample over many blocks (another summation order): equal to within one bf16 step
        assert (y.float() - ref.float()).abs().max() <= 2.0 ** -7 * ref.float().abs().max()
        # and against plain fp32 PyTorch
        xf = x.float().permute(0, 3, 1, 2)
        pt = torch.nn.functional.group_norm(xf, G, ww[:C].float() if ww is not None else None,
                                            bb[:C].float() if bb is not None else None, eps)
        pt = torch.nn.functional.silu(pt) if act == 2 else pt          # 2 is this library's code for SiLU
        assert (y.float() - pt.permute(0, 2, 3, 1)).abs().max() < 0.06


def test_static_workspace_rejects_oversize_and_bad_args():
    fn = _lib()
    dev = torch.device("cuda", 0)
    x = torch.zeros(1, 2, 2, 64, device=dev, dtype=torch.bfloat16)
    y = torch.empty_like(x)
    st = torch.cuda.current_stream().cuda_stream
    # N * G one past the limit: refused before anything is launched (pointers are never touched)
    assert fn(x.data_ptr(), y.data_ptr(), None, None, MAX_GROUPS // 32 + 1, 4, 64, 32, 1e-6, 0, st) == ERR_TOO_SMALL
    assert fn(x.data_ptr(), y.data_ptr(), None, None, 1, 4, 60, 32, 1e-6, 0, st) == -1
    torch.cuda.synchronize()
    rc, out = _call(fn, x + 1, None, None, 32, 1e-6, 0)          # still usable afterwards
    torch.cuda.synchronize()
    assert rc == 0 and torch.isfinite(out.float()).all()
