"""The allocation-free decode-attention entry point, called through its C symbol.

Some programs that embed this library may not allocate device memory once they are
running: they gave the whole GPU to a pool of their own, or they sit in a loop that
cannot afford the device-wide synchronisation inside cudaMalloc and cudaFree.  For them
``ek_attention_decode_bf16_noalloc`` keeps the scratch of the key-split path in a fixed
array inside the library (see csrc/attention_decode_noalloc.h).  This test loads the
library with ctypes, calls that symbol directly - twice in a row, with different inputs
and sizes, since the array is shared and keeps the previous call's contents - and checks
the result against the ordinary entry point, which takes caller-provided scratch.  It
also checks that a request larger than the array is refused without touching the output.
The file is named so that pytest collects it last.
"""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
SCRATCH_FLOATS = 2 * 1024 * 1024          # EK_NOALLOC_SCRATCH_FLOATS
TOO_LARGE = -3                            # EK_NOALLOC_TOO_LARGE
TOL = 2e-2                                # the bfloat16 bound of tests/test_kernels_gpu.py


def load_symbol():
    from enginekernel_b200.ops import build
    lib = ctypes.CDLL(build.ensure_built("attention_decode_bf16"))
    fn = lib.ek_attention_decode_bf16_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p]
    return fn


def make_case(seed, n_slots, length, nq, nkv, d):
    """A paged cache with shuffled pages and one query token per sequence at its end."""
    g = torch.Generator().manual_seed(seed)
    per = -(-length // 64)
    n_pages = n_slots * per + 2
    table = torch.randperm(n_pages, generator=g)[: n_slots * per].view(n_slots, per).to(torch.int32).to(DEV)
    k = (torch.randn(n_pages, nkv, 64, d, generator=g)).to(torch.bfloat16).to(DEV)
    v = (torch.randn(n_pages, nkv, 64, d, generator=g)).to(torch.bfloat16).to(DEV)
    q = torch.randn(n_slots, nq * d, generator=g).to(torch.bfloat16).to(DEV)
    positions = torch.tensor([length - 1 - 3 * s for s in range(n_slots)], dtype=torch.int32, device=DEV)
    slots = torch.arange(n_slots, dtype=torch.int32, device=DEV)
    return dict(q=q, k=k, v=v, table=table, positions=positions, slots=slots, nq=nq, nkv=nkv, d=d,
                n=n_slots, scale=1.0 / math.sqrt(d))


def call_noalloc(fn, c, out, splits, per_split):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(out.data_ptr(), c["q"].data_ptr(), c["q"].stride(0), c["positions"].data_ptr(),
              c["slots"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), c["table"].data_ptr(),
              c["table"].stride(0), c["n"], c["nq"], c["nkv"], c["d"], c["scale"], 0, splits,
              per_split, stream)


def call_ordinary(c, out, splits, per_split):
    from enginekernel_b200.ops import kernels
    acc = torch.empty(c["n"] * c["nq"] * splits * c["d"], device=DEV)
    ml = torch.empty(c["n"] * c["nq"] * splits * 2, device=DEV)
    kernels.attention_decode_bf16(out, c["q"], c["n"], c["positions"], c["slots"], c["k"], c["v"],
                                  c["table"], c["nq"], c["nkv"], c["d"], c["scale"], None, splits,
                                  per_split, acc, ml)


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    fn = load_symbol()
    # the second call is smaller and uses other data: leftovers of the first would show
    cases = [(make_case(1, 6, 700, 32, 8, 128), 6, 128), (make_case(2, 3, 300, 12, 3, 64), 4, 80)]
    for c, splits, per_split in cases:
        got = torch.full((c["n"], c["nq"] * c["d"]), 3.0, dtype=torch.bfloat16, device=DEV)
        want = torch.full_like(got, -3.0)
        before = torch.cuda.memory_allocated()
        status = call_noalloc(fn, c, got, splits, per_split)
        assert status == 0
        assert torch.cuda.memory_allocated() == before           # torch's allocator was not used
        call_ordinary(c, want, splits, per_split)
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item() / want.float().abs().max().item()
        assert err <= TOL, err
        assert torch.equal(got, want)                            # same kernels, same order of sums


def test_no_alloc_entry_point_refuses_what_its_array_cannot_hold():
    fn = load_symbol()
    c = make_case(3, 4, 128, 32, 8, 128)
    splits = SCRATCH_FLOATS // (c["n"] * c["nq"] * (c["d"] + 2)) + 1
    out = torch.full((c["n"], c["nq"] * c["d"]), 5.0, dtype=torch.bfloat16, device=DEV)
    assert call_noalloc(fn, c, out, splits, 16) == TOO_LARGE
    torch.cuda.synchronize()
    assert (out == 5.0).all()                                    # nothing was launched
    # one split needs no scratch at all and is always accepted
    assert call_noalloc(fn, c, out, 1, 0) == 0
    want = torch.empty_like(out)
    call_ordinary(c, want, 1, 0)
    torch.cuda.synchronize()
    assert torch.equal(out, want)
