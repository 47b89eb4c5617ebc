"""The attention entry point that allocates nothing, called through its exported C symbol.

Some callers of this library may not allocate device memory while they run (all of it was
given to their own arena at start-up, or their host process forbids it).  For them
`braid_attn_mma_noalloc` keeps the scratch of the sliced-context attention in a fixed array
inside the library.  This test calls it twice in a row on different inputs, so the second
call finds the first call's leftovers in the shared array, and checks each result against
the ordinary entry point, which gets a scratch buffer from the caller.

The file is named to be collected last: a run that stops at the first failure has then
already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def make_case(seed, hd, nqh, nkh, lens, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    pages = sum(-(-(l + 1) // 64) for l in lens) + 1
    cache = torch.randn(pages, 2, nkh, 64, hd, device=dev, generator=g).bfloat16()
    cols = max(-(-(l + 1) // 64) for l in lens)
    table = torch.full((len(lens), cols), -1, dtype=torch.int32)
    k = 0
    for i, l in enumerate(lens):
        for c in range(-(-(l + 1) // 64)):
            table[i, c] = k
            k += 1
    rows = len(lens)
    qkv = torch.randn(rows, (nqh + 2 * nkh) * hd, device=dev, generator=g).bfloat16()
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    return dict(cache=cache, table=table.to(dev), qkv=qkv, q_start=t(list(range(rows))), q_len=t([1] * rows),
                kv_before=t(lens), token_seq=t(list(range(rows))), rows=rows)


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from braidinfer_b200.csrc.api import get_kernels
    K = get_kernels(verbose=False)
    dev = torch.device("cuda:0")
    hd, nqh, nkh = 128, 32, 8
    lib = K.attn_mma_library(hd)
    fn = lib.braid_attn_mma_noalloc                      # the exported C symbol
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_int] * 13 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    lib.braid_attn_noalloc_capacity_floats.restype = ctypes.c_longlong
    cap = lib.braid_attn_noalloc_capacity_floats()
    assert cap == 2 * 1024 * 1024
    stream = torch.cuda.current_stream().cuda_stream
    flag = torch.zeros(1, dtype=torch.int32, device=dev)         # the caller's own int for the page guard

    def call(c, out, window, splits):
        return fn(c["qkv"].data_ptr(), out.data_ptr(), c["cache"].data_ptr(), c["table"].data_ptr(),
                  c["q_start"].data_ptr(), c["q_len"].data_ptr(), c["kv_before"].data_ptr(), c["token_seq"].data_ptr(),
                  c["qkv"].stride(0), out.stride(0), c["rows"], c["rows"], 1, nqh, nkh, hd, c["table"].shape[1],
                  c["cache"].shape[0], window, splits, 1, 1 / math.sqrt(hd), flag.data_ptr(), stream)

    # sliced contexts twice in a row (the second call finds the first one's leftovers), then a
    # window, then a single slice, which uses no scratch at all
    for seed, lens, splits, window in [(1, [2047, 100, 0, 63, 700], 8, 0), (2, [300, 1500, 64], 5, 0),
                                       (4, [900, 2000, 130, 5], 6, 500), (5, [400, 77, 1000], 1, 0),
                                       (6, [400, 77, 1000], 1, 128)]:
        c = make_case(seed, hd, nqh, nkh, lens, dev)
        want = torch.zeros(c["rows"], nqh * hd, device=dev, dtype=torch.bfloat16)
        K.attn_mma(c["qkv"], want, c["cache"], c["table"], c["q_start"], c["q_len"], c["kv_before"], c["token_seq"],
                   c["rows"], 1, nqh, nkh, hd, window or None, 1 / math.sqrt(hd), n_splits=splits, few_tokens=True)
        got = torch.full_like(want, 9.0)
        rc = call(c, got, window, splits)
        assert rc == 0, lib.braid_last_error().decode()
        torch.cuda.synchronize()
        # the same kernels over the same slices in the same order of sums: bit for bit
        assert torch.equal(got, want), (seed, (got.float() - want.float()).abs().max().item())
        assert flag.item() == 0
    K.check_device_errors()
    # a step beyond the array's size is refused with a clear message, not truncated
    c = make_case(3, hd, nqh, nkh, [10] * 64, dev)
    out = torch.empty(64, nqh * hd, device=dev, dtype=torch.bfloat16)
    rc = call(c, out, 0, 64)
    assert rc != 0 and b"holds" in lib.braid_last_error()
