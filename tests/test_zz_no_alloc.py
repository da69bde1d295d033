"""The allocation-free backward fold, called through its exported C symbol the way a host without an allocator would
call it, against the ordinary path (transpose into a caller's buffer, then the backward tile kernel).

Collected last on purpose: a failure here, under ``-x``, comes after every other test has run."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKSPACE_BYTES = 2 * 1024 * 1024


def _symbol(ext):
    library = ctypes.CDLL(ext.__file__)
    function = library.sc_fold_gradient_no_alloc
    function.restype = ctypes.c_int
    function.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
                         ctypes.POINTER(ctypes.c_uint32), ctypes.c_uint32, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p,
                         ctypes.c_char_p, ctypes.c_size_t]
    return function


def _call(function, cube, candidates, gradient, ends, scale, status):
    rows_q, hidden = gradient.shape
    rows_c = candidates.shape[0]
    ladder = (ctypes.c_uint32 * len(ends))(*ends)
    message = ctypes.create_string_buffer(256)
    code = function(cube.data_ptr(), candidates.data_ptr(), gradient.data_ptr(), rows_q, rows_c, hidden, ladder, len(ends),
                    scale, status.data_ptr(), torch.cuda.current_stream().cuda_stream, message, len(message))
    return code, message.value.decode()


def test_two_calls_in_a_row_match_the_ordinary_path(ext):
    function = _symbol(ext)
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    generator = torch.Generator(device="cuda").manual_seed(11)
    # Two different problems back to back, the second smaller than the first: whatever the first call left in the
    # shared workspace must not leak into the second result.
    for rows_q, rows_c, hidden, ends in ((256, 512, 768, [48, 96, 192, 384, 768]), (128, 128, 256, [64, 128, 256])):
        cube = (torch.randn(len(ends), rows_q, rows_c, device="cuda", generator=generator) * 0.1).to(torch.bfloat16)
        candidates = torch.randn(rows_c, hidden, device="cuda", generator=generator).to(torch.bfloat16)
        start = torch.randn(rows_q, hidden, device="cuda", generator=generator)
        expected, measured = start.clone(), start.clone()
        transposed = torch.empty(hidden, rows_c, dtype=torch.bfloat16, device="cuda")
        ext.transpose(candidates.data_ptr(), transposed.data_ptr(), rows_c, hidden, stream)
        ext.backward(cube.data_ptr(), transposed.data_ptr(), expected.data_ptr(), status.data_ptr(), rows_q, rows_c, hidden, ends, 1,
                     0.25, 2_000_000_000, stream)
        code, message = _call(function, cube, candidates, measured, ends, 0.25, status)
        torch.cuda.synchronize()
        assert code == 0, message
        assert status.tolist()[0] == 0
        # same kernels, same order of operations: the tolerance of the other backward tests holds with room to spare
        reference = start + 0.25 * torch.cat([cube[b].float() @ candidates.float()[:, (0 if b == 0 else ends[b - 1]):ends[b]]
                                              for b in range(len(ends))], dim=1)
        assert torch.equal(measured, expected)
        assert (measured - reference).norm() / reference.norm() < 1e-5


def test_sizes_beyond_the_workspace_and_bad_shapes_are_refused(ext):
    function = _symbol(ext)
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    rows_c, hidden = 2048, 1024  # 4 MiB of transposed candidates: twice the built-in workspace
    assert rows_c * hidden * 2 > WORKSPACE_BYTES
    cube = torch.zeros(1, 128, rows_c, dtype=torch.bfloat16, device="cuda")
    candidates = torch.zeros(rows_c, hidden, dtype=torch.bfloat16, device="cuda")
    gradient = torch.zeros(128, hidden, device="cuda")
    code, message = _call(function, cube, candidates, gradient, [hidden], 1.0, status)
    assert code == 1 and "exceeds the built-in workspace" in message
    small = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    code, message = _call(function, cube, small, torch.zeros(100, 64, device="cuda"), [64], 1.0, status)
    assert code == 2 and "multiple of 128" in message
    # ladders that do not ascend, or whose ends are not multiples of 16, are refused before anything is launched
    candidates = torch.zeros(64, 256, dtype=torch.bfloat16, device="cuda")
    cube = torch.zeros(3, 128, 64, dtype=torch.bfloat16, device="cuda")
    gradient_small = torch.zeros(128, 256, device="cuda")
    for ends in ([128, 64, 256], [64, 64, 256], [24, 128, 256]):
        code, message = _call(function, cube, candidates, gradient_small, ends, 1.0, status)
        assert code == 2 and "ascend" in message, (ends, code, message)
    torch.cuda.synchronize()
    assert int(gradient.abs().sum()) == 0 and int(gradient_small.abs().sum()) == 0  # a refused call touches nothing
