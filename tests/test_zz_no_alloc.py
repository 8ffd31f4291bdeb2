"""The attention entry point that allocates nothing, called through its exported C symbol.

Some users of the library cannot allocate device memory while they run (code hosted inside
another program's memory pool, loops that must not enter the allocator).  For them the library
keeps the scratch of the split-key attention in a fixed array of its own.  This test calls that
entry point the way such a user would, through the C symbol with raw pointers, twice in a row on
different inputs, and compares each result with the ordinary entry point's and with the plain
float64 attention; it also checks the property the entry point is named for: the device memory
in use is the same after the calls as before them.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu


def _case(seed, lengths, n_q, n_kv, d, page_size):
    g = torch.Generator().manual_seed(seed)
    pages_needed = [(n + page_size - 1) // page_size for n in lengths]
    total = sum(pages_needed) + 2
    order = torch.randperm(total, generator=g).tolist()
    width = max(pages_needed)
    tables, cursor = [], 0
    for need in pages_needed:
        tables.append(order[cursor:cursor + need] + [0] * (width - need))
        cursor += need
    rand = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16).cuda()
    n = len(lengths)
    as_int = lambda values: torch.tensor(values, dtype=torch.int32).cuda()
    return dict(q=rand(n, n_q, d), k_pool=rand(total, n_kv, page_size, d), v_pool=rand(total, n_kv, page_size, d),
                tables=as_int(tables), request_of_token=as_int(list(range(n))), positions=as_int([x - 1 for x in lengths]),
                query_start=as_int(list(range(n + 1))), context_lens=as_int(lengths), max_ctx=max(lengths))


def _device_bytes_in_use() -> int:
    free, total = torch.cuda.mem_get_info()      # cudaMemGetInfo: everything the process and others hold on the device
    return total - free


@pytest.mark.parametrize("n_q,n_kv,d,splits", [(16, 8, 128, 6), (40, 2, 64, 5)])
def test_static_scratch_entry_point_matches_the_ordinary_one(n_q, n_kv, d, splits):
    """(16, 8, 128): the one-warp kernel of decode steps; (40, 2, 64): twenty query heads per key/value head
    are more than one warp's sixteen rows, so the four-warp kernel runs with its keys split."""
    import miniserve_b200  # noqa: F401
    from miniserve_b200 import kernels

    lib = kernels.library()
    entry = lib.ms_paged_attention_decode_static
    entry.restype = ctypes.c_int
    page_size = 16
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    cases = [_case(seed, lengths, n_q, n_kv, d, page_size) for seed, lengths in ((1, [700, 33, 1, 1500]), (2, [64, 2047, 900]))]
    references = []
    for c in cases:
        ordinary = torch.empty_like(c["q"])
        kernels.paged_attention(c["q"], c["k_pool"], c["v_pool"], c["tables"], c["request_of_token"], c["positions"],
                                c["query_start"], c["context_lens"], 1, c["max_ctx"], d ** -0.5, None, ordinary)
        plain = torch.empty(c["q"].shape, dtype=torch.float64)
        plain_ops.paged_attention(c["q"].cpu(), c["k_pool"].cpu(), c["v_pool"].cpu(), c["tables"].cpu(),
                                  c["request_of_token"].cpu(), c["positions"].cpu(), c["query_start"].cpu(),
                                  c["context_lens"].cpu(), 1, c["max_ctx"], d ** -0.5, None, plain)
        references.append((ordinary, plain.cuda()))
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(c, out):
        n = c["q"].shape[0]
        code = entry(ptr(c["q"]), ptr(c["k_pool"]), ptr(c["v_pool"]), ptr(c["tables"]), ctypes.c_int(c["tables"].shape[1]),
                     ptr(c["query_start"]), ptr(c["context_lens"]), ctypes.c_int(page_size), ctypes.c_int(n_q),
                     ctypes.c_int(n_kv), ctypes.c_int(d), ctypes.c_float(d ** -0.5), ctypes.c_int(0), ptr(out),
                     ctypes.c_int(splits), ctypes.c_int(n), ctypes.c_int(n), stream)
        assert code == 0, lib.ms_last_error().decode()

    # The first call on a device sets the entry point up (it looks up where the device keeps the array, and the
    # driver may load the kernels' code then); a caller makes it once at start-up, as here.
    call(cases[0], torch.zeros_like(cases[0]["q"]))
    outs = [torch.zeros_like(c["q"]) for c in cases]
    torch.cuda.synchronize()
    held_by_torch, in_use = torch.cuda.memory_allocated(), _device_bytes_in_use()
    for c, out in zip(cases, outs):                    # two calls in a row: each finds the array as the call before left it
        call(c, out)
    torch.cuda.synchronize()
    # nothing was allocated: neither through the framework's allocator nor behind its back
    assert torch.cuda.memory_allocated() == held_by_torch
    assert _device_bytes_in_use() == in_use
    for out, (ordinary, plain) in zip(outs, references):
        assert torch.allclose(out.float(), ordinary.float(), atol=2e-2, rtol=2e-2), float((out.float() - ordinary.float()).abs().max())
        assert torch.allclose(out.double(), plain, atol=2e-2, rtol=2e-2), float((out.double() - plain).abs().max())


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    import miniserve_b200  # noqa: F401
    from miniserve_b200 import kernels

    lib = kernels.library()
    entry = lib.ms_paged_attention_decode_static
    entry.restype = ctypes.c_int
    n_kv, d, page_size = 8, 128, 16
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    # beyond the built-in scratch: refused with a message, nothing launched
    c = _case(3, [10] * 4, 16, n_kv, d, page_size)
    out = torch.zeros_like(c["q"])
    code = entry(ptr(c["q"]), ptr(c["k_pool"]), ptr(c["v_pool"]), ptr(c["tables"]), ctypes.c_int(c["tables"].shape[1]),
                 ptr(c["query_start"]), ptr(c["context_lens"]), ctypes.c_int(page_size), ctypes.c_int(4096),
                 ctypes.c_int(n_kv), ctypes.c_int(d), ctypes.c_float(1.0), ctypes.c_int(0), ptr(out), ctypes.c_int(64),
                 ctypes.c_int(4), ctypes.c_int(4), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert code != 0 and "exceed the built-in scratch" in lib.ms_last_error().decode()
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0
