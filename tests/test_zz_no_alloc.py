"""``sharpi_sample_rows_no_alloc``: the sampler for hosts that may not allocate device memory
(a serving loop with a fixed memory partition, a plug-in inside another program's budget; see
``csrc/sampling_no_alloc.h``).  Its work area is an array inside the library, so the test calls it the
way such a host would, through the exported C symbol with raw pointers, and checks that it picks
exactly the tokens the allocating entry point picks, twice in a row, because the second call starts
from whatever the first left in the shared work area.  Needs a GPU.  The file name makes pytest
collect it last."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_FLOATS = 4 << 20


def exported_symbol():
    from sharpinference_b200.kernels import build
    lib = ctypes.CDLL(build.build_library("sampling"))
    fn = lib.sharpi_sample_rows_no_alloc
    P, I = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [P, I, I, P, P, P, P, P, P, P]
    fn.restype = I
    return fn


def inputs(rows, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(rows, vocab, generator=g) * 2.0).to(DEV)
    temperature = torch.tensor([0.8, 0.0, 1.3, 0.7, 1.0][:rows] + [0.9] * max(0, rows - 5), device=DEV)
    top_k = torch.tensor([0, 0, 40, 40, 7][:rows] + [0] * max(0, rows - 5), dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.95, 1.0][:rows] + [1.0] * max(0, rows - 5), device=DEV)
    min_p = torch.tensor([0.0, 0.0, 0.0, 0.05, 0.02][:rows] + [0.0] * max(0, rows - 5), device=DEV)
    uniform = torch.rand(rows, generator=g).clamp(1e-6, 1 - 1e-6).to(DEV)
    return logits, temperature, top_k, top_p, min_p, uniform


def call(fn, logits, temperature, top_k, top_p, min_p, uniform, out):
    return fn(logits.data_ptr(), logits.shape[0], logits.shape[1], temperature.data_ptr(), top_k.data_ptr(),
              top_p.data_ptr(), min_p.data_ptr(), uniform.data_ptr(), out.data_ptr(),
              torch.cuda.current_stream().cuda_stream)


def test_same_tokens_as_the_allocating_entry_point_twice_in_a_row():
    from sharpinference_b200.kernels import ops
    fn = exported_symbol()
    for seed, (rows, vocab) in enumerate([(5, 1000), (3, 202048), (5, 777)]):     # the last call reuses a dirtier area
        args = inputs(rows, vocab, seed)
        want = ops.sample_rows(*args)
        out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        assert call(fn, *args, out) == 0
        torch.cuda.synchronize()
        assert out.tolist() == want.tolist()


def test_a_request_beyond_the_work_area_is_refused_and_writes_nothing():
    fn = exported_symbol()
    rows, vocab = 33, 131072                       # 33 * 131072 floats: just above the 4 Mi float limit
    assert rows * vocab > MAX_FLOATS
    logits = torch.zeros(rows, vocab, device=DEV)
    ones = torch.ones(rows, device=DEV)
    out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
    status = call(fn, logits, ones, torch.zeros(rows, dtype=torch.int32, device=DEV), ones, torch.zeros(rows, device=DEV),
                  ones * 0.5, out)
    torch.cuda.synchronize()
    assert status == 4 and out.tolist() == [-7] * rows
    # exactly at the limit is accepted
    rows = 32
    out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
    status = call(fn, logits[:rows], ones[:rows], torch.zeros(rows, dtype=torch.int32, device=DEV), ones[:rows],
                  torch.zeros(rows, device=DEV), ones[:rows] * 0.5, out)
    torch.cuda.synchronize()
    assert status == 0 and all(0 <= t < vocab for t in out.tolist())
