"""The entry point that allocates nothing (csrc/no_alloc.h), called through its exported C
symbol the way a program without a device allocator of its own would call it.

Some callers of this library may not allocate while they run: a server that gave all device
memory to a pool at start-up, a loop that must not risk the synchronisation or the failure of
a cudaMalloc in the middle of a request, code running inside another framework's stream.  For
them the split decode attention comes in a variant whose scratch is an array inside the
library.  This test gives both variants the same inputs (the usual one gets scratch tensors
from torch) and expects the same output within the tolerance the other kernel tests use, on
two calls in a row: the second call finds the array as the first left it.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def _lib():
    from nimbus_infer_rs_b200.csrc import build
    lib = ctypes.CDLL(str(build.build()))
    lib.nb_last_error.restype = ctypes.c_char_p
    lib.nb_attention_decode_static_capacity.restype = ctypes.c_longlong
    return lib


def _inputs(dtype, n_rows, H, Hk, hd, seed):
    """Queries, a paged cache with shuffled pages, and per-row slots and positions."""
    g = torch.Generator().manual_seed(seed)
    lens = [int(x) for x in torch.randint(1, 600, (n_rows,), generator=g)]
    lens[0], lens[-1] = 1, 599
    pages_per_seq = [-(-l // PAGE) for l in lens]
    n_pages = sum(pages_per_seq) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_pages = max(pages_per_seq)
    table = torch.zeros(n_rows, max_pages, dtype=torch.int32)
    it = iter(perm)
    for s, n in enumerate(pages_per_seq):
        for p in range(n):
            table[s, p] = next(it)
    k = torch.randn(n_pages, Hk, PAGE, hd, generator=g).to(dtype).to(DEV)
    v = torch.randn(n_pages, Hk, PAGE, hd, generator=g).to(dtype).to(DEV)
    q = torch.randn(n_rows, H * hd, generator=g).to(dtype).to(DEV)
    slot = torch.arange(n_rows, dtype=torch.int32)
    slot[1] = -1                                      # a padding row
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32)
    return q, k, v, table.to(DEV), slot.to(DEV), pos.to(DEV), max_pages


def _code(dtype):
    return 0 if dtype == torch.float32 else 1


@pytest.mark.parametrize("dtype, H, Hk, hd, n_splits", [(torch.bfloat16, 12, 12, 64, 4),
                                                        (torch.float32, 6, 2, 32, 7),
                                                        (torch.bfloat16, 8, 1, 128, 1)])
def test_static_scratch_variant_matches_the_usual_entry_point(dtype, H, Hk, hd, n_splits):
    lib = _lib()
    n_rows = 9
    q, k, v, table, slot, pos, max_pages = _inputs(dtype, n_rows, H, Hk, hd, seed=H + hd)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    scale = 1.0 / math.sqrt(hd)
    common = lambda out: (  # noqa: E731
        c_void_p(q.data_ptr()), c_int(_code(dtype)), c_int(q.shape[1]), c_int(0),
        c_void_p(slot.data_ptr()), c_void_p(pos.data_ptr()), c_void_p(k.data_ptr()),
        c_void_p(v.data_ptr()), c_void_p(table.data_ptr()), c_int(max_pages), c_int(PAGE),
        c_int(H), c_int(Hk), c_int(hd), c_void_p(out.data_ptr()), c_int(_code(dtype)),
        c_int(H * hd), c_float(scale), c_int(0), c_int(n_rows), c_int(n_splits))

    # the usual entry point, scratch from the caller
    acc = torch.empty(n_rows * H * n_splits * hd, dtype=torch.float32, device=DEV)
    ml = torch.empty(n_rows * H * n_splits * 2, dtype=torch.float32, device=DEV)
    counters = torch.zeros(n_rows * Hk, dtype=torch.int32, device=DEV)
    want = torch.full((n_rows, H * hd), 3.0, dtype=dtype, device=DEV)
    rc = lib.nb_attention_decode(*common(want), c_void_p(acc.data_ptr()), c_void_p(ml.data_ptr()),
                                 c_void_p(counters.data_ptr()), c_int(0), c_int(0), c_int(0), stream)
    assert rc == 0, lib.nb_last_error()
    torch.cuda.synchronize()
    assert torch.isfinite(want.float()).all() and (want[1] == 0).all()

    # a plain float64 restatement of the operation, so that this file stands on its own
    page_of = table.cpu()
    for r in (0, 2, n_rows - 1):
        n_keys = int(pos[r]) + 1
        ks = torch.cat([k[int(page_of[r, p])] for p in range(-(-n_keys // PAGE))], dim=1)[:, :n_keys]
        vs = torch.cat([v[int(page_of[r, p])] for p in range(-(-n_keys // PAGE))], dim=1)[:, :n_keys]
        for h in (0, H - 1):
            qh = q[r, h * hd:(h + 1) * hd].double()
            sc = (ks[h // (H // Hk)].double() @ qh) * scale
            ref = torch.softmax(sc, 0) @ vs[h // (H // Hk)].double()
            err = (want[r, h * hd:(h + 1) * hd].double() - ref).abs().max()
            assert err <= (2e-5 if dtype == torch.float32 else 1.5e-2) * max(1.0, float(ref.abs().max()))

    # the variant that allocates nothing, twice in a row on the same built-in array; between
    # the two calls another call with other sizes and another number of splits leaves partial
    # sums and non-zero bytes where the second call's counters and sums go
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    for call in range(2):
        got = torch.full((n_rows, H * hd), -5.0, dtype=dtype, device=DEV)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]           # the driver's count, not torch's
        before = torch.cuda.memory_allocated()
        rc = lib.nb_attention_decode_static(*common(got), stream)
        assert rc == 0, lib.nb_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] >= free_before   # no device memory was taken
        err = (got.double() - want.double()).abs().max()
        assert err <= tol * max(1.0, float(want.double().abs().max())), (call, float(err))
        if call == 0:
            other = torch.empty(3, H * hd, dtype=dtype, device=DEV)
            args = list(common(other))
            args[19], args[20] = c_int(3), c_int(n_splits + 2)        # rows, splits
            rc = lib.nb_attention_decode_static(*args, stream)
            assert rc == 0, lib.nb_last_error()
            torch.cuda.synchronize()
            assert (other.double() - want[:3].double()).abs().max() <= \
                tol * max(1.0, float(want.double().abs().max()))


def test_sizes_beyond_the_built_in_array_are_refused():
    lib = _lib()
    cap = lib.nb_attention_decode_static_capacity()
    assert cap == 4 * 1024 * 1024
    dtype, H, Hk, hd = torch.bfloat16, 12, 12, 64
    n_rows = 64
    q, k, v, table, slot, pos, max_pages = _inputs(dtype, n_rows, H, Hk, hd, seed=1)
    out = torch.zeros(n_rows, H * hd, dtype=dtype, device=DEV)
    n_splits = 32                       # 64 x 12 x 32 x 66 floats = 6.5 MB > 4 MiB
    rc = lib.nb_attention_decode_static(
        c_void_p(q.data_ptr()), c_int(1), c_int(q.shape[1]), c_int(0), c_void_p(slot.data_ptr()),
        c_void_p(pos.data_ptr()), c_void_p(k.data_ptr()), c_void_p(v.data_ptr()),
        c_void_p(table.data_ptr()), c_int(max_pages), c_int(PAGE), c_int(H), c_int(Hk), c_int(hd),
        c_void_p(out.data_ptr()), c_int(1), c_int(H * hd), c_float(0.125), c_int(0), c_int(n_rows),
        c_int(n_splits), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0
    msg = lib.nb_last_error().decode()
    assert "bytes of scratch" in msg and "4194304" in msg
    assert (out == 0).all()
