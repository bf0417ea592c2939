"""The allocation-free decode attention entry point, called through its exported C symbol.

Some hosts of the kernel library cannot allocate device memory when they call it (they
run where cudaMalloc is forbidden or would stall the device, or they own a fixed arena).
``lgml_decode_attention_noalloc`` serves them: same inputs and output as
``lgml_decode_attention``, with the scratch for the key ranges' partial results taken
from an array built into the library.  This test calls the symbol with ctypes, twice in
a row with different problems (the array keeps the first call's contents), and compares
with the regular entry point, which gets its scratch from the caller.  It is collected
last so that a run that stops at the first failure has run everything else before.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 4 << 20   # LGML_NOALLOC_SCRATCH_FLOATS


def problem(seed, n_seqs, H, Hkv, D, lens, n_pages=96, width=12):
    g = torch.Generator().manual_seed(seed)
    dev = "cuda:0"
    k = torch.randn(n_pages, Hkv, 64, D, generator=g).to(dev, torch.bfloat16)
    v = torch.randn(n_pages, Hkv, 64, D, generator=g).to(dev, torch.bfloat16)
    q = (torch.randn(n_seqs, H * D, generator=g) * 2).to(dev, torch.bfloat16)
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n_seqs, width), -1, dtype=torch.int32)
    for s, n in enumerate(lens):
        for b in range(-(-n // 64)):
            table[s, b] = perm.pop()
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=dev)
    seq_of = torch.arange(n_seqs, dtype=torch.int32, device=dev)
    return q, positions, seq_of, table.to(dev), k, v


def call_noalloc(lib, q, positions, seq_of, table, k, v, H, n_splits, scale, window, status):
    fn = lib.lgml_decode_attention_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int,
                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
    out = torch.empty_like(q)
    n_pages, hkv, page, d = k.shape
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = fn(q.data_ptr(), q.stride(0), positions.data_ptr(), seq_of.data_ptr(), table.data_ptr(), table.shape[1], k.data_ptr(),
            v.data_ptr(), n_pages, page, out.data_ptr(), out.stride(0), n_splits, q.shape[0], H, hkv, d, scale, window, 1,
            status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    call_noalloc.took = free_before - torch.cuda.mem_get_info()[0]      # device memory the call itself took
    err = lib.lgml_attention_decode_noalloc_last_error
    err.restype = ctypes.c_char_p
    return rc, out, err().decode()


def test_noalloc_entry_point_matches_the_regular_one_twice_in_a_row():
    from lgml_b200 import csrc, ops

    lib = csrc.load("attention_decode_noalloc")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    cases = [
        dict(seed=1, n_seqs=5, H=8, Hkv=2, D=64, lens=[700, 64, 1, 333, 129], n_splits=11, window=0),
        dict(seed=2, n_seqs=3, H=6, Hkv=6, D=48, lens=[200, 450, 65], n_splits=3, window=100),
    ]
    for i, c in enumerate(cases):
        q, positions, seq_of, table, k, v = problem(c["seed"], c["n_seqs"], c["H"], c["Hkv"], c["D"], c["lens"])
        scale = c["D"] ** -0.5
        want = torch.empty_like(q)
        ops.decode_attention(q, positions, seq_of, table, k, v, want, c["H"], scale, c["window"], status, c["n_splits"])
        rc, got, msg = call_noalloc(lib, q, positions, seq_of, table, k, v, c["H"], c["n_splits"], scale, c["window"], status)
        torch.cuda.synchronize()
        if i > 0:
            # the property in its name: once the first call on the device has run (it may load the
            # kernels' code), a call takes no device memory: the free memory the driver reports just
            # before and just after the call is the same
            assert call_noalloc.took == 0
        assert rc == 0, msg
        assert int(status.item()) == 0
        assert torch.isfinite(got.float()).all()
        # same kernels, same order of sums: the tolerance of the bfloat16 tests is far more than needed
        assert torch.allclose(got.float(), want.float(), atol=1.5e-2, rtol=1.5e-2)
        assert torch.equal(got, want)


def test_noalloc_entry_point_at_the_edges_of_its_array():
    """The largest problem the array holds (4 floats under its size), one key range (no scratch
    at all), and no tokens."""
    from lgml_b200 import csrc, ops

    lib = csrc.load("attention_decode_noalloc")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    H, D, n_seqs, n_splits = 41, 64, 31, 50
    assert SCRATCH_FLOATS - 66 < n_seqs * H * n_splits * (D + 2) <= SCRATCH_FLOATS
    lens = [64 * (1 + s % 7) + s for s in range(n_seqs)]
    q, positions, seq_of, table, k, v = problem(4, n_seqs, H, H, D, lens, n_pages=200, width=8)
    want = torch.empty_like(q)
    ops.decode_attention(q, positions, seq_of, table, k, v, want, H, D ** -0.5, 0, status, n_splits)
    rc, got, msg = call_noalloc(lib, q, positions, seq_of, table, k, v, H, n_splits, D ** -0.5, 0, status)
    torch.cuda.synchronize()
    assert rc == 0, msg
    assert int(status.item()) == 0 and torch.equal(got, want)
    # one key range: the kernel writes the output itself and the array is not touched
    ops.decode_attention(q, positions, seq_of, table, k, v, want, H, D ** -0.5, 0, status, 1)
    rc, got, msg = call_noalloc(lib, q, positions, seq_of, table, k, v, H, 1, D ** -0.5, 0, status)
    torch.cuda.synchronize()
    assert rc == 0, msg
    assert torch.equal(got, want)
    # no tokens: nothing to do, no error
    rc, _, msg = call_noalloc(lib, q[:0], positions[:0], seq_of[:0], table, k, v, H, 4, D ** -0.5, 0, status)
    assert rc == 0, msg


def test_noalloc_entry_point_refuses_what_its_array_cannot_hold():
    from lgml_b200 import csrc

    lib = csrc.load("attention_decode_noalloc")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    H, Hkv, D, n_seqs, n_splits = 32, 8, 128, 64, 20
    assert n_seqs * H * n_splits * (D + 2) > SCRATCH_FLOATS
    q, positions, seq_of, table, k, v = problem(3, n_seqs, H, Hkv, D, [100] * n_seqs, n_pages=160, width=4)
    rc, _, msg = call_noalloc(lib, q, positions, seq_of, table, k, v, H, n_splits, D ** -0.5, 0, status)
    assert rc != 0 and "floats of scratch" in msg and "holds" in msg
