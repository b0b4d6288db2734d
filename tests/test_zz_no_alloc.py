"""The sampling entry point that allocates nothing, called the way a program
without any tensor library would call it: through its exported C symbol.

Who needs it: a caller that cannot give the sampler a scratch buffer because it
cannot get one - a C host that links the library alone, a server that handed
all device memory to its own pools at start-up, a loop that may not touch the
CUDA allocator once it runs.  The library keeps the scratch in a fixed device
array of its own instead (64 KiB, at most 256 rows per call).

The test calls it twice in a row (the array keeps the first call's values; the
second call must not be disturbed by them) and compares each result with the
ordinary entry point, which gets its scratch from the caller.  It runs last so
that a failure here cannot hide another test's."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

P, I = ctypes.c_void_p, ctypes.c_int


def library():
    from alofa_b200.csrc.build import load_library

    lib = load_library("alofa_sampling", ["kernels/sampling.cu"])
    lib.alofa_sample_noalloc.restype = I
    lib.alofa_sample_noalloc.argtypes = [P, P, P, P, I, I, I, P]
    lib.alofa_sample_noalloc_max_rows.restype = I
    lib.alofa_sample.restype = I
    lib.alofa_sample.argtypes = [P, P, P, P, I, I, P, I, P]
    return lib


def test_no_alloc_sampling_matches_the_ordinary_entry_point_twice():
    lib = library()
    rng = np.random.default_rng(0)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.alofa_sample_noalloc_max_rows() == 256
    for call, (rows, vocab) in enumerate([(37, 5003), (8, 151936)]):
        logits = torch.from_numpy(rng.normal(0, 3, size=(rows, vocab)).astype(np.float32)).cuda()
        temps = rng.choice([0.0, 0.0, 0.7, 1.3], size=rows).astype(np.float32)
        if call == 1:
            logits[0, [11, 90000]] = 50.0  # a tie at the top goes to the lower index
            temps[0] = 0.0
        temperature = torch.from_numpy(temps).cuda()
        uniform = torch.from_numpy(rng.random(rows).astype(np.float32)).cuda()
        want = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        scratch = torch.empty(2 * rows * 32, dtype=torch.float32, device="cuda")
        assert lib.alofa_sample(want.data_ptr(), logits.data_ptr(), temperature.data_ptr(), uniform.data_ptr(), rows, vocab, scratch.data_ptr(), 1, stream) == 0
        got = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        if call == 0:  # the first call on a device may load the library's image and looks the array up
            assert lib.alofa_sample_noalloc(got.data_ptr(), logits.data_ptr(), temperature.data_ptr(), uniform.data_ptr(), rows, vocab, 1, stream) == 0
            torch.cuda.synchronize()
            got.fill_(-1)
        # free device memory as the driver counts it (not only what the tensor library's own pool
        # holds): a cudaMalloc inside the entry point would lower it
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.alofa_sample_noalloc(got.data_ptr(), logits.data_ptr(), temperature.data_ptr(), uniform.data_ptr(), rows, vocab, 1, stream)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.mem_get_info()[0] == free_before
        assert got.cpu().tolist() == want.cpu().tolist(), f"call {call}"
        greedy = [int(np.argmax(r)) for r in logits.cpu().numpy()]
        for r in range(rows):
            if temps[r] == 0.0:
                assert int(got[r]) == greedy[r]
        if call == 1:
            assert int(got[0]) == 11


def test_no_alloc_sampling_refuses_a_draw_without_its_uniform_number():
    """A row with a positive temperature needs a uniform number: without the
    array the call is refused (1) and nothing is written; with any_hot = 0 the
    caller promises that no row draws, and every row gets its largest logit."""
    lib = library()
    rows, vocab = 5, 301
    stream = torch.cuda.current_stream().cuda_stream
    logits = torch.from_numpy(np.random.default_rng(3).normal(0, 2, size=(rows, vocab)).astype(np.float32)).cuda()
    temperature = torch.tensor([0.0, 0.9, 0.0, 1.1, 0.5], device="cuda")
    tokens = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    assert lib.alofa_sample_noalloc(tokens.data_ptr(), logits.data_ptr(), temperature.data_ptr(), None, rows, vocab, 1, stream) == 1
    torch.cuda.synchronize()
    assert tokens.cpu().tolist() == [-7] * rows
    assert lib.alofa_sample_noalloc(tokens.data_ptr(), logits.data_ptr(), temperature.data_ptr(), None, rows, vocab, 0, stream) == 0
    torch.cuda.synchronize()
    assert tokens.cpu().tolist() == logits.argmax(dim=1).cpu().tolist()


def test_no_alloc_sampling_refuses_too_many_rows():
    lib = library()
    rows, vocab = 257, 16
    logits = torch.zeros(rows, vocab, device="cuda")
    tokens = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    rc = lib.alofa_sample_noalloc(tokens.data_ptr(), logits.data_ptr(), None, None, rows, vocab, 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 3 and int(tokens[0]) == -7  # refused, nothing launched
    assert lib.alofa_sample_noalloc(tokens.data_ptr(), logits.data_ptr(), None, None, 256, vocab, 0, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert tokens[:256].cpu().tolist() == [0] * 256
