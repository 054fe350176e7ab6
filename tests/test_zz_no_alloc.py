"""The arg-max entry point that brings its own scratch memory (csrc/cuda/argmax_noalloc.h), called through its
exported C symbol and compared with the entry point that takes caller-provided scratch.  Collected last on purpose:
it has to pass alone and after every other GPU test has used the device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

F16, BF16, F32 = 0, 1, 2
MAX_ROWS = 4096


@pytest.fixture(scope="module")
def clib():
    from onnxruntime_b200.ops import _kernels as K
    lib = ctypes.CDLL(K.lib_path())
    lib.ortb200_argmax_noalloc.restype = ctypes.c_int
    lib.ortb200_argmax_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
    lib.ortb200_argmax_noalloc_prepare.restype = ctypes.c_int
    lib.ortb200_argmax_noalloc_strerror.restype = ctypes.c_char_p
    lib.ortb200_argmax_noalloc_strerror.argtypes = [ctypes.c_int]
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    assert lib.ortb200_argmax_noalloc_prepare() == 0  # set-up step: looks the scratch address up for this device
    return lib


def call(lib, x, out):
    rows, n = x.numel() // x.shape[-1], x.shape[-1]
    code = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}[x.dtype]
    return lib.ortb200_argmax_noalloc(x.data_ptr(), out.data_ptr(), rows, n, code, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("rows,n,dtype", [(8, 128256, torch.bfloat16), (1, 32000, torch.float16), (300, 1000, torch.float32),
                                          (MAX_ROWS, 257, torch.bfloat16), (3, 5, torch.float32)])
def test_matches_existing_entry_point_twice_in_a_row(clib, rows, n, dtype):
    from onnxruntime_b200.ops import _kernels as K
    g = torch.Generator(device="cuda").manual_seed(rows * 7919 + n)
    out = torch.full((rows,), -1, dtype=torch.int64, device="cuda")
    for attempt in range(2):  # the second call finds the scratch as the first one left it
        x = torch.randn(rows, n, device="cuda", generator=g).to(dtype)
        out.fill_(-1)
        assert call(clib, x, out) == 0
        want = K.argmax(x)
        torch.cuda.synchronize()
        assert torch.equal(out, want), (attempt, (out != want).nonzero()[:4])
        assert torch.equal(out, x.float().argmax(-1))


def test_ties_and_nan_follow_the_same_rules(clib):
    from onnxruntime_b200.ops import _kernels as K
    x = torch.zeros(4, 9000, device="cuda")
    x[0, 17] = x[0, 8000] = 3.0          # first maximum wins
    x[1, :] = float("nan")               # all-NaN row gives 0
    x[2, 5] = float("nan"); x[2, 4500] = 1.0
    x[3, :] = -5.0; x[3, 8999] = -4.0
    out = torch.empty(4, dtype=torch.int64, device="cuda")
    assert call(clib, x, out) == 0
    torch.cuda.synchronize()
    assert out.tolist() == [17, 0, 4500, 8999]
    assert torch.equal(out, K.argmax(x))


def test_sizes_beyond_the_built_in_scratch_are_refused(clib):
    x = torch.zeros(MAX_ROWS + 1, 8, device="cuda")
    out = torch.full((MAX_ROWS + 1,), -7, dtype=torch.int64, device="cuda")
    rc = call(clib, x, out)
    assert rc == -20
    msg = clib.ortb200_argmax_noalloc_strerror(rc).decode()
    assert "4096" in msg and "ortb200_argmax()" in msg
    torch.cuda.synchronize()
    assert bool((out == -7).all())  # nothing was launched
    assert clib.ortb200_argmax_noalloc(None, out.data_ptr(), 1, 8, F32, None) == -1
    assert clib.ortb200_argmax_noalloc(x.data_ptr(), out.data_ptr(), 1, 8, 9, None) == -4


def test_allocates_nothing(clib):
    x = torch.randn(16, 50000, device="cuda").bfloat16()
    out = torch.empty(16, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    torch_before = torch.cuda.memory_allocated()
    for _ in range(3):
        assert call(clib, x, out) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == torch_before
    assert free_after == free_before
