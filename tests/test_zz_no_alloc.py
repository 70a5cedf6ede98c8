"""tb_attention_split_static: attention for callers that cannot allocate device memory.

Some users of this library run where cudaMalloc is off limits: a loop whose memory was fixed at
start-up, a host program that owns all device memory itself.  For them the library exports one C
entry point whose scratch (the partial results of the key slices) is a fixed 8 MiB array inside
the library.  This test calls it through its exported C symbol, twice in a row with different
inputs (the array keeps the first call's contents), and checks each result against the ordinary
entry point, which takes its scratch from the caller.  It also checks that a problem too large for
the array is refused.  The file is named to be collected last, and passes alone in a fresh
process as well as after the other tests.
"""
import ctypes
import math

import pytest
import torch

from kernel_inputs import attention_case

pytestmark = pytest.mark.gpu


def _static_entry():
    from transformer_b200.csrc import lib
    fn = lib.library().tb_attention_split_static
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P] * 9 + [I] * 8 + [F, I, P]
    fn.restype = I
    return fn


def _both(case, dtype, splits):
    from transformer_b200.csrc import lib
    c = case
    nt, nh, dh = c["nt"], c["nh"], c["dh"]
    scale = 1.0 / math.sqrt(dh)
    out_ref = torch.zeros(nt, nh * dh, dtype=dtype, device="cuda")
    partial = torch.empty(nt * nh * splits * (dh + 2), dtype=torch.float32, device="cuda")
    lib.call("tb_attention_" + lib.suffix(dtype), c["q"].data_ptr(), out_ref.data_ptr(), c["kc"].data_ptr(),
             c["vc"].data_ptr(), c["tile_seq"].data_ptr(), c["tile_t0"].data_ptr(), c["tile_nq"].data_ptr(),
             c["tok_pos"].data_ptr(), c["table"].data_ptr(), partial.data_ptr(), c["tiles"], nt, c["max_pages"],
             nh * dh, nh, c["nkvh"], dh, splits, scale)
    out = torch.zeros_like(out_ref)
    stream = torch.cuda.current_stream().cuda_stream
    rc = _static_entry()(c["q"].data_ptr(), out.data_ptr(), c["kc"].data_ptr(), c["vc"].data_ptr(),
                         c["tile_seq"].data_ptr(), c["tile_t0"].data_ptr(), c["tile_nq"].data_ptr(),
                         c["tok_pos"].data_ptr(), c["table"].data_ptr(), c["tiles"], nt, c["max_pages"], nh * dh,
                         nh, c["nkvh"], dh, splits, scale, 1 if dtype == torch.bfloat16 else 0, stream)
    assert rc == 0, f"tb_attention_split_static returned {rc}"
    torch.cuda.synchronize()
    return out, out_ref


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_matches_on_two_calls_in_a_row(dtype):
    from transformer_b200.csrc import lib
    tq = lib.attention_tile_tokens(4, 2)
    # first call: long contexts, 5 key slices; second: other sizes and 3 slices, stale scratch below it
    first = attention_case([1, 1, 1], [200, 37, 130], 4, 2, 32, dtype, tq, seed=1)
    second = attention_case([1, 6], [90, 10], 4, 2, 32, dtype, tq, seed=2)
    for case, splits in ((first, 5), (second, 3)):
        out, out_ref = _both(case, dtype, splits)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert float((out.float() - out_ref.float()).abs().max()) <= 1e-6, "differs from the ordinary entry point"
        want = case["ref"].reshape(case["nt"], -1).float().cuda()
        assert float((out.float() - want).abs().max()) <= tol


def test_static_scratch_refuses_what_does_not_fit():
    tq = 8
    case = attention_case([1], [10], 4, 2, 32, torch.float32, tq, seed=3)
    c = case
    out = torch.zeros(1, 4 * 32, dtype=torch.float32, device="cuda")
    # claim a huge problem: nt * nh * splits * (dh + 2) floats far beyond 8 MiB; nothing may launch
    rc = _static_entry()(c["q"].data_ptr(), out.data_ptr(), c["kc"].data_ptr(), c["vc"].data_ptr(),
                         c["tile_seq"].data_ptr(), c["tile_t0"].data_ptr(), c["tile_nq"].data_ptr(),
                         c["tok_pos"].data_ptr(), c["table"].data_ptr(), c["tiles"], 100000, c["max_pages"],
                         4 * 32, 4, 2, 32, 8, 0.1, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0
